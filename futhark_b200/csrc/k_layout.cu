// Layout operations that the reference's compiler inserts on either side of a SegOp:
// batched transposition of 1-, 2-, 4- and 8-byte elements, strided (LMAD) copies (second half
// of the file), and the replicate / iota fills.  Replaces the map_transpose_{1,2,4,8}b kernels
// of the reference's runtime (rts/opencl/transpose.cl:3-277: the tiled kernel and its
// low-width, low-height, small and large variants; rts/c/gpu.h:144-168, 333-461) and the fill
// kernels its compiler generates (src/Futhark/CodeGen/ImpGen/GPU/Base.hs:1274-1436).
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

// ---- the other element widths ------------------------------------------------------------------
// The same 64 x 64 tile through shared memory for 1-, 2- and 8-byte elements: a row of the tile
// is read by 64 consecutive threads, a row of the output written by 64 consecutive threads, the
// tile pitch is 65 elements.  (The 4-byte kernel above additionally moves 16-byte vectors.)
template <typename T>
__global__ void __launch_bounds__(TR_THREADS)
transpose_any_kernel(const T *__restrict__ in, T *__restrict__ out, int64_t nb, int64_t rows, int64_t cols,
                     int64_t tiles_r, int64_t tiles_c) {
  __shared__ T s_t[TR_TILE * TR_PITCH];
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;      // 64 across, 4 down
  const int64_t per_batch = tiles_r * tiles_c, total = per_batch * nb;
  for (int64_t t = blockIdx.x; t < total; t += gridDim.x) {
    const int64_t b = t / per_batch, rem = t - b * per_batch;
    const int64_t tc = rem / tiles_r, tr = rem - tc * tiles_r;
    const int64_t r0 = tr * TR_TILE, c0 = tc * TR_TILE;
    const T *src = in + b * rows * cols;
    T *dst = out + b * rows * cols;
#pragma unroll
    for (int k = 0; k < 16; k++) {
      const int r = ty + 4 * k;
      if (r0 + r < rows && c0 + tx < cols) s_t[r * TR_PITCH + tx] = src[(r0 + r) * cols + c0 + tx];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 16; k++) {
      const int c = ty + 4 * k;                     // input column = output row
      if (c0 + c < cols && r0 + tx < rows) dst[(c0 + c) * rows + r0 + tx] = s_t[tx * TR_PITCH + c];
    }
    __syncthreads();
  }
}

cudaError_t launch_transpose(int elem_size, const void *in, void *out, int64_t nb, int64_t rows, int64_t cols, int num_sms,
                             cudaStream_t stream) {
  if (nb <= 0 || rows <= 0 || cols <= 0) return cudaSuccess;
  if (elem_size == 4) return launch_transpose_b32(in, out, nb, rows, cols, num_sms, stream);
  const int64_t tiles_r = (rows + TR_TILE - 1) / TR_TILE, tiles_c = (cols + TR_TILE - 1) / TR_TILE;
  const int64_t total = tiles_r * tiles_c * nb;
  const int64_t resident = (int64_t)num_sms * (elem_size == 8 ? 4 : 8);
  const int grid = (int)(total < resident ? total : resident);
  if (elem_size == 1)
    transpose_any_kernel<uint8_t><<<grid, TR_THREADS, 0, stream>>>(reinterpret_cast<const uint8_t *>(in), reinterpret_cast<uint8_t *>(out), nb, rows, cols, tiles_r, tiles_c);
  else if (elem_size == 2)
    transpose_any_kernel<uint16_t><<<grid, TR_THREADS, 0, stream>>>(reinterpret_cast<const uint16_t *>(in), reinterpret_cast<uint16_t *>(out), nb, rows, cols, tiles_r, tiles_c);
  else if (elem_size == 8)
    transpose_any_kernel<uint64_t><<<grid, TR_THREADS, 0, stream>>>(reinterpret_cast<const uint64_t *>(in), reinterpret_cast<uint64_t *>(out), nb, rows, cols, tiles_r, tiles_c);
  else
    return cudaErrorInvalidValue;
  return cudaGetLastError();
}

// ---- replicate and iota (ImpGen/GPU/Base.hs:1342-1436: sReplicate, sIota) ---------------------------
template <typename T>
__global__ void __launch_bounds__(256) replicate_kernel(T *__restrict__ dst, int64_t n, T v) {
  const int64_t stride = (int64_t)gridDim.x * 256;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += stride) dst[i] = v;
}
// dst[i] = start + i * step in the integer type T (wrapping, as the reference's iota over a sized type)
template <typename T>
__global__ void __launch_bounds__(256) iota_kernel(T *__restrict__ dst, int64_t n, int64_t start, int64_t step) {
  const int64_t stride = (int64_t)gridDim.x * 256;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += stride)
    dst[i] = (T)((uint64_t)start + (uint64_t)i * (uint64_t)step);
}
static int fill_grid(int64_t n, int num_sms) {
  const int64_t want = (n + 255) / 256, cap = (int64_t)num_sms * 8;
  return (int)(want < 1 ? 1 : (want < cap ? want : cap));
}
cudaError_t launch_replicate(int elem_size, void *dst, int64_t n, uint64_t value_bits, int num_sms, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  const int grid = fill_grid(n, num_sms);
  switch (elem_size) {
    case 1: replicate_kernel<uint8_t><<<grid, 256, 0, stream>>>(reinterpret_cast<uint8_t *>(dst), n, (uint8_t)value_bits); break;
    case 2: replicate_kernel<uint16_t><<<grid, 256, 0, stream>>>(reinterpret_cast<uint16_t *>(dst), n, (uint16_t)value_bits); break;
    case 4: replicate_kernel<uint32_t><<<grid, 256, 0, stream>>>(reinterpret_cast<uint32_t *>(dst), n, (uint32_t)value_bits); break;
    case 8: replicate_kernel<uint64_t><<<grid, 256, 0, stream>>>(reinterpret_cast<uint64_t *>(dst), n, value_bits); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}
cudaError_t launch_iota(int elem_size, void *dst, int64_t n, int64_t start, int64_t step, int num_sms, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  const int grid = fill_grid(n, num_sms);
  switch (elem_size) {
    case 1: iota_kernel<uint8_t><<<grid, 256, 0, stream>>>(reinterpret_cast<uint8_t *>(dst), n, start, step); break;
    case 2: iota_kernel<uint16_t><<<grid, 256, 0, stream>>>(reinterpret_cast<uint16_t *>(dst), n, start, step); break;
    case 4: iota_kernel<uint32_t><<<grid, 256, 0, stream>>>(reinterpret_cast<uint32_t *>(dst), n, start, step); break;
    case 8: iota_kernel<uint64_t><<<grid, 256, 0, stream>>>(reinterpret_cast<uint64_t *>(dst), n, start, step); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

// ---- strided (LMAD) copies -------------------------------------------------------------------
// dst[dst_offset + sum_i idx_i * dst_strides_i] = src[src_offset + sum_i idx_i * src_strides_i]
// for every index below `shape`; offsets and strides count elements.  Stands where the
// reference's lmad_copy_gpu2gpu_{1,2,4,8}b stands (rts/c/gpu.h:540-586 with the classification
// of rts/c/copy.h:60-190): a copy that is a batched transposition goes to the transposition
// kernel above, one where both sides are the same dense layout becomes one device-to-device
// copy, anything else takes the general kernel (the role of rts/opencl/copy.cl:3-83).
//
// The classification works on a normal form of the copy: dimensions of extent 1 are dropped,
// the rest are ordered by falling destination stride (so the fastest-varying index of the
// general kernel walks the destination's smallest stride: coalesced writes), and neighbours
// that are dense with respect to each other on BOTH sides are merged.  In that form a flat
// copy has rank <= 1 with unit strides, and a batched transposition has the strides
// (n*m, m, 1) against (n*m, 1, n), with or without the leading dimension.

struct LmadArgs {
  int r;
  int64_t shape[LMAD_MAX_RANK], dst[LMAD_MAX_RANK], src[LMAD_MAX_RANK];
  int64_t total;
};

// IDX: the type the linear index is taken apart in (32-bit division where the copy has fewer
// than 2^31 elements).
template <typename T, typename IDX>
__global__ void __launch_bounds__(256)
lmad_copy_kernel(T *__restrict__ dst, const T *__restrict__ src, const LmadArgs a) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < a.total; i += stride) {
    IDX rem = (IDX)i;
    int64_t d = 0, s = 0;
#pragma unroll 1
    for (int k = a.r - 1; k > 0; k--) {
      const IDX ext = (IDX)a.shape[k], q = rem / ext, idx = rem - q * ext;
      d += (int64_t)idx * a.dst[k];
      s += (int64_t)idx * a.src[k];
      rem = q;
    }
    d += (int64_t)rem * a.dst[0];
    s += (int64_t)rem * a.src[0];
    dst[d] = src[s];
  }
}

template <typename T>
static void launch_general(void *d, const void *s, const LmadArgs &a, int grid, cudaStream_t stream) {
  if (a.total < (int64_t)1 << 31)
    lmad_copy_kernel<T, uint32_t><<<grid, 256, 0, stream>>>(reinterpret_cast<T *>(d), reinterpret_cast<const T *>(s), a);
  else
    lmad_copy_kernel<T, uint64_t><<<grid, 256, 0, stream>>>(reinterpret_cast<T *>(d), reinterpret_cast<const T *>(s), a);
}

int lmad_normalise(int r, const int64_t *dst_strides, const int64_t *src_strides, const int64_t *shape,
                   int64_t *n_shape, int64_t *n_dst, int64_t *n_src) {
  int n = 0;
  for (int i = 0; i < r; i++) {
    if (shape[i] == 1) continue;
    // insertion by falling destination stride (ties: the longer dimension first); stable otherwise
    int p = n;
    while (p > 0 && (n_dst[p - 1] < dst_strides[i] || (n_dst[p - 1] == dst_strides[i] && n_shape[p - 1] < shape[i]))) {
      n_shape[p] = n_shape[p - 1]; n_dst[p] = n_dst[p - 1]; n_src[p] = n_src[p - 1];
      p--;
    }
    n_shape[p] = shape[i]; n_dst[p] = dst_strides[i]; n_src[p] = src_strides[i];
    n++;
  }
  // merge dimension k+1 into k where k strides over exactly the extent of k+1 on both sides
  int m = 0;
  for (int k = 0; k < n; k++) {
    if (m > 0 && n_dst[m - 1] == n_dst[k] * n_shape[k] && n_src[m - 1] == n_src[k] * n_shape[k]) {
      n_shape[m - 1] *= n_shape[k]; n_dst[m - 1] = n_dst[k]; n_src[m - 1] = n_src[k];
    } else {
      n_shape[m] = n_shape[k]; n_dst[m] = n_dst[k]; n_src[m] = n_src[k];
      m++;
    }
  }
  return m;
}

int lmad_classify(int r, const int64_t *shape, const int64_t *dst, const int64_t *src, int64_t *nb, int64_t *rows,
                  int64_t *cols) {
  if (r == 0 || (r == 1 && dst[0] == 1 && src[0] == 1)) return LMAD_FLAT;
  if (r == 2 || r == 3) {
    const int o = r - 2;
    const int64_t A = shape[o], B = shape[o + 1];
    const bool batch_ok = (r == 2) || (dst[0] == A * B && src[0] == A * B);
    // destination row-major [A][B], source holds the same matrix as [B][A]
    if (batch_ok && dst[o] == B && dst[o + 1] == 1 && src[o] == 1 && src[o + 1] == A) {
      *nb = r == 3 ? shape[0] : 1; *rows = B; *cols = A;
      return LMAD_TRANSPOSE;
    }
  }
  return LMAD_GENERAL;
}

cudaError_t launch_lmad_copy(int elem_size, int r, void *dst, int64_t dst_offset, const int64_t *dst_strides,
                             const void *src, int64_t src_offset, const int64_t *src_strides, const int64_t *shape,
                             int num_sms, cudaStream_t stream, int *kind_out) {
  if (kind_out) *kind_out = LMAD_NOTHING;
  if (r < 0 || r > LMAD_MAX_RANK) return cudaErrorInvalidValue;
  if (elem_size != 1 && elem_size != 2 && elem_size != 4 && elem_size != 8) return cudaErrorInvalidValue;
  int64_t total = 1;
  for (int i = 0; i < r; i++) {
    if (shape[i] < 0) return cudaErrorInvalidValue;
    total *= shape[i];
  }
  if (total == 0) return cudaSuccess;
  LmadArgs a;
  a.r = lmad_normalise(r, dst_strides, src_strides, shape, a.shape, a.dst, a.src);
  a.total = total;
  char *d = reinterpret_cast<char *>(dst) + dst_offset * elem_size;
  const char *s = reinterpret_cast<const char *>(src) + src_offset * elem_size;
  // (named d/s: the char pointers already include the offsets)
  int64_t nb = 0, rows = 0, cols = 0;
  int kind = lmad_classify(a.r, a.shape, a.dst, a.src, &nb, &rows, &cols);
  if (kind_out) *kind_out = kind;
  if (kind == LMAD_FLAT) return cudaMemcpyAsync(d, s, (size_t)total * elem_size, cudaMemcpyDeviceToDevice, stream);
  if (kind == LMAD_TRANSPOSE) return launch_transpose(elem_size, s, d, nb, rows, cols, num_sms, stream);
  if (a.r == 0) { a.r = 1; a.shape[0] = 1; a.dst[0] = 0; a.src[0] = 0; }
  // Widen the element while the innermost dimension is contiguous on both sides and everything
  // else (extent, the other strides, both addresses) stays a multiple of the doubled size: rows
  // then move as 16-byte words instead of single elements.
  int es = elem_size;
  while (es < 16 && a.dst[a.r - 1] == 1 && a.src[a.r - 1] == 1 && (a.shape[a.r - 1] & 1) == 0 &&
         ((reinterpret_cast<uintptr_t>(d) | reinterpret_cast<uintptr_t>(s)) & (uintptr_t)(2 * es - 1)) == 0) {
    bool ok = true;
    for (int k = 0; k + 1 < a.r; k++) ok = ok && (a.dst[k] & 1) == 0 && (a.src[k] & 1) == 0;
    if (!ok) break;
    for (int k = 0; k + 1 < a.r; k++) { a.dst[k] /= 2; a.src[k] /= 2; }
    a.shape[a.r - 1] /= 2;
    a.total /= 2;
    es *= 2;
  }
  total = a.total;
  const int64_t want = (total + 255) / 256, cap = (int64_t)num_sms * 8;
  const int grid = (int)(want < cap ? want : cap);
  switch (es) {
    case 1: launch_general<uint8_t>(d, s, a, grid, stream); break;
    case 2: launch_general<uint16_t>(d, s, a, grid, stream); break;
    case 4: launch_general<uint32_t>(d, s, a, grid, stream); break;
    case 8: launch_general<uint64_t>(d, s, a, grid, stream); break;
    default: launch_general<uint4>(d, s, a, grid, stream); break;
  }
  return cudaGetLastError();
}

}  // namespace fb
