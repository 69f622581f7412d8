// Layout operations that the reference's compiler inserts on either side of a SegOp:
// batched transposition of 4-byte elements.  Replaces the map_transpose_4b kernels of the
// reference's runtime (rts/opencl/transpose.cl:3-275: the tiled kernel and its low-width,
// low-height, small and large variants; rts/c/gpu.h:144-168).
//
// One kernel.  A CTA of 256 threads moves 64 x 64 tiles through shared memory: rows of the
// input are read as 16-byte vectors (a warp covers two rows of 256 bytes), the tile is held
// with a pitch of 65 words, and rows of the output are written as 16-byte vectors again, so
// both sides of HBM see full 128-byte lines.  Tiles are dealt to a persistent grid in the
// order of the OUTPUT rows, so that concurrently running CTAs write neighbouring lines.
// Shapes whose rows are not a multiple of 4 elements, or whose bases are not 16-byte
// aligned, take element-wise guarded accesses on the side concerned; ragged edge tiles are
// guarded in the same way.  Narrow or short matrices need no variants of their own here: a
// tile that is mostly outside the matrix costs little, and the grid is sized by tiles.
#include "common.cuh"
#include "kernels.h"

namespace fb {

constexpr int TR_TILE = 64, TR_PITCH = TR_TILE + 1, TR_THREADS = 256;

__global__ void __launch_bounds__(TR_THREADS)
transpose_b32_kernel(const uint32_t *__restrict__ in, uint32_t *__restrict__ out, int64_t nb, int64_t rows, int64_t cols,
                     int64_t tiles_r, int64_t tiles_c) {
  __shared__ uint32_t s_t[TR_TILE * TR_PITCH];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;           // 16 vectors across, 16 rows down
  const bool in_vec = ((cols & 3) == 0) && ((((uintptr_t)in) & 15) == 0);
  const bool out_vec = ((rows & 3) == 0) && ((((uintptr_t)out) & 15) == 0);
  const int64_t per_batch = tiles_r * tiles_c, total = per_batch * nb;
  for (int64_t t = blockIdx.x; t < total; t += gridDim.x) {
    const int64_t b = t / per_batch, rem = t - b * per_batch;
    const int64_t tc = rem / tiles_r, tr = rem - tc * tiles_r;     // consecutive tiles share output rows
    const int64_t r0 = tr * TR_TILE, c0 = tc * TR_TILE;
    const uint32_t *src = in + b * rows * cols;
    uint32_t *dst = out + b * rows * cols;
    const bool inner = (r0 + TR_TILE <= rows) && (c0 + TR_TILE <= cols);
    // ---- input tile [r0 .. r0+64) x [c0 .. c0+64) into shared memory, row by row
#pragma unroll
    for (int k = 0; k < 4; k++) {
      const int r = ty + 16 * k;
      if (inner && in_vec) {
        const int4 v = ld_stream_v4(src + (r0 + r) * cols + c0 + 4 * tx);
        uint32_t *p = s_t + r * TR_PITCH + 4 * tx;
        p[0] = v.x; p[1] = v.y; p[2] = v.z; p[3] = v.w;
      } else if (r0 + r < rows) {
#pragma unroll
        for (int j = 0; j < 4; j++) {
          const int64_t c = c0 + 4 * tx + j;
          if (c < cols) s_t[r * TR_PITCH + 4 * tx + j] = src[(r0 + r) * cols + c];
        }
      }
    }
    __syncthreads();
    // ---- output tile [c0 .. c0+64) x [r0 .. r0+64): output row = input column
#pragma unroll
    for (int k = 0; k < 4; k++) {
      const int c = ty + 16 * k;                    // input column = output row
      if (inner && out_vec) {
        int4 v;
        v.x = s_t[(4 * tx + 0) * TR_PITCH + c]; v.y = s_t[(4 * tx + 1) * TR_PITCH + c];
        v.z = s_t[(4 * tx + 2) * TR_PITCH + c]; v.w = s_t[(4 * tx + 3) * TR_PITCH + c];
        st_stream_v4(dst + (c0 + c) * rows + r0 + 4 * tx, v);
      } else if (c0 + c < cols) {
#pragma unroll
        for (int j = 0; j < 4; j++) {
          const int64_t r = r0 + 4 * tx + j;
          if (r < rows) dst[(c0 + c) * rows + r] = s_t[(4 * tx + j) * TR_PITCH + c];
        }
      }
    }
    __syncthreads();
  }
}

cudaError_t launch_transpose_b32(const void *in, void *out, int64_t nb, int64_t rows, int64_t cols, int num_sms,
                                 cudaStream_t stream) {
  if (nb <= 0 || rows <= 0 || cols <= 0) return cudaSuccess;
  const int64_t tiles_r = (rows + TR_TILE - 1) / TR_TILE, tiles_c = (cols + TR_TILE - 1) / TR_TILE;
  const int64_t total = tiles_r * tiles_c * nb;
  const int64_t resident = (int64_t)num_sms * 8;    // 8 CTAs of 256 threads and 16.6 KB of shared memory per SM
  const int grid = (int)(total < resident ? total : resident);
  transpose_b32_kernel<<<grid, TR_THREADS, 0, stream>>>(reinterpret_cast<const uint32_t *>(in),
                                                       reinterpret_cast<uint32_t *>(out), nb, rows, cols, tiles_r, tiles_c);
  return cudaGetLastError();
}

}  // namespace fb
