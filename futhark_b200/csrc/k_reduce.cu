// Reductions: reduce (+) over i32, row sums of a regular [rows][cols] f32 array, and
// the irregular segmented sum over f32 with segments given by offsets.  They replace
// the generated segred_nonseg / segred_small / segred_large kernels of the reference
// (src/Futhark/CodeGen/ImpGen/GPU/SegRed.hs:327-636) and the scan-then-gather form
// the reference uses for irregular segments
// (src/Futhark/Pass/Flatten/Builtins.hs:582-602).
//
// All three are one pass over HBM with 128-bit streaming loads where alignment
// allows, several independent loads in flight per thread, and warp shuffles instead
// of shared-memory trees.
#include "common.cuh"
#include "kernels.h"

namespace fb {

constexpr int RED_THREADS = 256;
constexpr int RED_MAX_BLOCKS = 4096;

// a ticket word, then room for one partial per CTA; the fused-redomap template (redomap.cuh) shares
// the area and keeps up to 16 bytes per CTA
size_t reduce_scratch_bytes() { return 256 + RED_MAX_BLOCKS * 16; }

// ---- reduce (+) 0 over i32 ----------------------------------------------------------
// Stage one: grid-stride over 16-byte vectors, four loads in flight per thread.
// Stage two: the CTA that draws the last ticket folds the per-CTA partials
// (same election as reductionStageTwo, SegRed.hs:923-1047, without the extra barrier
// rounds).  Integer addition wraps, so any order gives the reference's bits.
__global__ void __launch_bounds__(RED_THREADS)
reduce_i32_kernel(const int32_t *__restrict__ in, int64_t n, int32_t *__restrict__ d_out,
                  uint32_t *ticket, uint32_t *partials) {
  __shared__ uint32_t s_warp[RED_THREADS / 32];
  __shared__ uint32_t s_last;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t gtid = (int64_t)blockIdx.x * RED_THREADS + tid;
  const int64_t gthreads = (int64_t)gridDim.x * RED_THREADS;

  // peel to a 16-byte boundary
  const uintptr_t addr = (uintptr_t)in;
  int64_t head = (int64_t)(((16 - (addr & 15)) & 15) >> 2);
  if (head > n) head = n;
  const int4 *vec = reinterpret_cast<const int4 *>(in + head);
  const int64_t nvec = (n - head) >> 2;
  const int64_t tail_start = head + (nvec << 2);

  uint32_t a0 = 0, a1 = 0, a2 = 0, a3 = 0;
  int64_t i = gtid;
  for (; i + 3 * gthreads < nvec; i += 4 * gthreads) {
    int4 v0 = ld_stream_v4(vec + i);
    int4 v1 = ld_stream_v4(vec + i + gthreads);
    int4 v2 = ld_stream_v4(vec + i + 2 * gthreads);
    int4 v3 = ld_stream_v4(vec + i + 3 * gthreads);
    a0 += (uint32_t)v0.x + (uint32_t)v0.y + (uint32_t)v0.z + (uint32_t)v0.w;
    a1 += (uint32_t)v1.x + (uint32_t)v1.y + (uint32_t)v1.z + (uint32_t)v1.w;
    a2 += (uint32_t)v2.x + (uint32_t)v2.y + (uint32_t)v2.z + (uint32_t)v2.w;
    a3 += (uint32_t)v3.x + (uint32_t)v3.y + (uint32_t)v3.z + (uint32_t)v3.w;
  }
  for (; i < nvec; i += gthreads) {
    int4 v0 = ld_stream_v4(vec + i);
    a0 += (uint32_t)v0.x + (uint32_t)v0.y + (uint32_t)v0.z + (uint32_t)v0.w;
  }
  uint32_t acc = a0 + a1 + a2 + a3;
  if (gtid < head) acc += (uint32_t)in[gtid];
  if (tail_start + gtid < n) acc += (uint32_t)in[tail_start + gtid];   // fewer than 4 elements

  acc = warp_sum(acc);
  if (lane == 0) s_warp[warp] = acc;
  __syncthreads();
  if (warp == 0) {
    uint32_t b = (lane < RED_THREADS / 32) ? s_warp[lane] : 0u;
    b = warp_sum(b);
    if (lane == 0) {
      partials[blockIdx.x] = b;
      __threadfence();
      uint32_t t = atomicAdd(ticket, 1u);
      s_last = (t == gridDim.x - 1) ? 1u : 0u;
    }
  }
  __syncthreads();
  if (s_last) {
    __threadfence();
    uint32_t s = 0;
    for (int j = tid; j < (int)gridDim.x; j += RED_THREADS)
      s += *reinterpret_cast<volatile uint32_t *>(&partials[j]);
    s = warp_sum(s);
    __syncthreads();
    if (lane == 0) s_warp[warp] = s;
    __syncthreads();
    if (warp == 0) {
      uint32_t b = (lane < RED_THREADS / 32) ? s_warp[lane] : 0u;
      b = warp_sum(b);
      if (lane == 0) { *d_out = (int32_t)b; *ticket = 0u; }
    }
  }
}

cudaError_t launch_reduce_i32(const int32_t *in, int64_t n, int32_t *d_out, void *scratch, int num_sms,
                              cudaStream_t stream) {
  if (n <= 0) return cudaMemsetAsync(d_out, 0, sizeof(int32_t), stream);   // the neutral element
  uint32_t *ticket = reinterpret_cast<uint32_t *>(scratch);
  uint32_t *partials = reinterpret_cast<uint32_t *>(reinterpret_cast<char *>(scratch) + 256);
  int64_t want = (n / 4 + RED_THREADS - 1) / RED_THREADS;
  int blocks = num_sms * 8;
  if (blocks > RED_MAX_BLOCKS) blocks = RED_MAX_BLOCKS;
  if (want < blocks) blocks = want < 1 ? 1 : (int)want;
  reduce_i32_kernel<<<blocks, RED_THREADS, 0, stream>>>(in, n, d_out, ticket, partials);
  return cudaGetLastError();
}

// ---- map (reduce (+) 0) over the rows of [rows][cols] f32 -------------------------------
// One warp per row (persistent, grid-stride over rows): lane l adds the 16-byte
// vectors l, l+32, ... of the row into four running sums, then a shuffle tree.
template <bool VEC>
__global__ void __launch_bounds__(RED_THREADS)
rowsum_warp_kernel(const float *__restrict__ in, int64_t rows, int64_t cols, float *__restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t warp_global = ((int64_t)blockIdx.x * RED_THREADS + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * RED_THREADS) >> 5;
  for (int64_t r = warp_global; r < rows; r += nwarps) {
    const float *row = in + r * cols;
    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
    if (VEC) {
      const int4 *v = reinterpret_cast<const int4 *>(row);
      const int64_t nv = cols >> 2;
      int64_t i = lane;
#pragma unroll 1
      for (; i + 96 < nv; i += 128) {
        int4 q0 = ld_stream_v4(v + i), q1 = ld_stream_v4(v + i + 32);
        int4 q2 = ld_stream_v4(v + i + 64), q3 = ld_stream_v4(v + i + 96);
        s0 += __int_as_float(q0.x); s1 += __int_as_float(q0.y); s2 += __int_as_float(q0.z); s3 += __int_as_float(q0.w);
        s0 += __int_as_float(q1.x); s1 += __int_as_float(q1.y); s2 += __int_as_float(q1.z); s3 += __int_as_float(q1.w);
        s0 += __int_as_float(q2.x); s1 += __int_as_float(q2.y); s2 += __int_as_float(q2.z); s3 += __int_as_float(q2.w);
        s0 += __int_as_float(q3.x); s1 += __int_as_float(q3.y); s2 += __int_as_float(q3.z); s3 += __int_as_float(q3.w);
      }
      for (; i < nv; i += 32) {
        int4 q0 = ld_stream_v4(v + i);
        s0 += __int_as_float(q0.x); s1 += __int_as_float(q0.y); s2 += __int_as_float(q0.z); s3 += __int_as_float(q0.w);
      }
    } else {
      for (int64_t i = lane; i < cols; i += 32) s0 += row[i];
    }
    float s = warp_sum_down((s0 + s1) + (s2 + s3));
    if (lane == 0) out[r] = s;
  }
}

// One CTA per row, for rows too long for a single warp to stream efficiently.
__global__ void __launch_bounds__(RED_THREADS)
rowsum_block_kernel(const float *__restrict__ in, int64_t rows, int64_t cols, float *__restrict__ out) {
  __shared__ float s_warp[RED_THREADS / 32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const float *row = in + r * cols;
    float s0 = 0.f, s1 = 0.f;
    int64_t i = tid;
    for (; i + RED_THREADS < cols; i += 2 * RED_THREADS) { s0 += row[i]; s1 += row[i + RED_THREADS]; }
    if (i < cols) s0 += row[i];
    float s = warp_sum_down(s0 + s1);
    __syncthreads();
    if (lane == 0) s_warp[warp] = s;
    __syncthreads();
    if (warp == 0) {
      float b = (lane < RED_THREADS / 32) ? s_warp[lane] : 0.f;
      b = warp_sum_down(b);
      if (lane == 0) out[r] = b;
    }
  }
}

// One thread per row, for very short rows.
__global__ void __launch_bounds__(RED_THREADS)
rowsum_thread_kernel(const float *__restrict__ in, int64_t rows, int64_t cols, float *__restrict__ out) {
  const int64_t gthreads = (int64_t)gridDim.x * RED_THREADS;
  for (int64_t r = (int64_t)blockIdx.x * RED_THREADS + threadIdx.x; r < rows; r += gthreads) {
    const float *row = in + r * cols;
    float s = 0.f;
    for (int64_t i = 0; i < cols; i++) s += row[i];
    out[r] = s;
  }
}

cudaError_t launch_rowsum_f32(const float *in, int64_t rows, int64_t cols, float *out, int num_sms,
                              cudaStream_t stream) {
  if (rows <= 0) return cudaSuccess;
  if (cols <= 0) return cudaMemsetAsync(out, 0, (size_t)rows * sizeof(float), stream);
  if (cols < 16) {
    int64_t want = (rows + RED_THREADS - 1) / RED_THREADS;
    int blocks = (int)(want < (int64_t)num_sms * 8 ? want : (int64_t)num_sms * 8);
    rowsum_thread_kernel<<<blocks, RED_THREADS, 0, stream>>>(in, rows, cols, out);
  } else if (cols <= 16384) {
    int64_t want = (rows * 32 + RED_THREADS - 1) / RED_THREADS;
    int blocks = (int)(want < (int64_t)num_sms * 8 ? want : (int64_t)num_sms * 8);
    const bool vec = (cols % 4 == 0) && ((((uintptr_t)in) & 15) == 0);
    if (vec) rowsum_warp_kernel<true><<<blocks, RED_THREADS, 0, stream>>>(in, rows, cols, out);
    else rowsum_warp_kernel<false><<<blocks, RED_THREADS, 0, stream>>>(in, rows, cols, out);
  } else {
    int blocks = (int)(rows < (int64_t)num_sms * 8 ? rows : (int64_t)num_sms * 8);
    rowsum_block_kernel<<<blocks, RED_THREADS, 0, stream>>>(in, rows, cols, out);
  }
  return cudaGetLastError();
}

// ---- irregular segmented sum: out[s] = sum xs[offsets[s] .. offsets[s+1]) ------------------
// One warp per segment, persistent over the segments, two segments at a time: the chain
// offsets -> data -> shuffle tree -> store is latency-bound per segment, so a warp issues
// the loads of two segments (8 + 8 per lane, predicated on the segment length) before it
// reduces either, and the offsets of its next pair are already in flight.  Segment starts
// are arbitrary, so loads are 4-byte, contiguous across the warp.  Offsets are clamped to
// [0,n], so a malformed offsets array cannot cause an out-of-range read.
constexpr int SEG_U = 8;   // loads per lane and segment issued up front (covers 256 elements)

__device__ __forceinline__ void clamp_range(int64_t &lo, int64_t &hi, int64_t n) {
  lo = lo < 0 ? 0 : (lo > n ? n : lo);
  hi = hi < lo ? lo : (hi > n ? n : hi);
}

__global__ void __launch_bounds__(RED_THREADS)
segreduce_f32_kernel(const int64_t *__restrict__ offsets, int64_t nseg, const float *__restrict__ xs, int64_t n,
                     float *__restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t warp_global = ((int64_t)blockIdx.x * RED_THREADS + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * RED_THREADS) >> 5;
  int64_t sA = warp_global, sB = warp_global + nwarps;
  int64_t loA = 0, hiA = 0, loB = 0, hiB = 0;
  if (sA < nseg) { loA = offsets[sA]; hiA = offsets[sA + 1]; }
  if (sB < nseg) { loB = offsets[sB]; hiB = offsets[sB + 1]; }
  while (sA < nseg) {
    const int64_t nA = sA + 2 * nwarps, nB = sB + 2 * nwarps;
    int64_t nloA = 0, nhiA = 0, nloB = 0, nhiB = 0;
    if (nA < nseg) { nloA = offsets[nA]; nhiA = offsets[nA + 1]; }
    if (nB < nseg) { nloB = offsets[nB]; nhiB = offsets[nB + 1]; }
    clamp_range(loA, hiA, n);
    clamp_range(loB, hiB, n);
    float a[SEG_U], b[SEG_U];
#pragma unroll
    for (int u = 0; u < SEG_U; u++) {
      const int64_t ia = loA + lane + 32 * u, ib = loB + lane + 32 * u;
      a[u] = (ia < hiA) ? __int_as_float(ld_stream_b32(xs + ia)) : 0.f;
      b[u] = (ib < hiB) ? __int_as_float(ld_stream_b32(xs + ib)) : 0.f;
    }
    float tA = ((a[0] + a[1]) + (a[2] + a[3])) + ((a[4] + a[5]) + (a[6] + a[7]));
    float tB = ((b[0] + b[1]) + (b[2] + b[3])) + ((b[4] + b[5]) + (b[6] + b[7]));
    // the rest of segments longer than 256 elements
    for (int64_t i = loA + lane + 32 * SEG_U; i < hiA; i += 128) {
      const float q0 = __int_as_float(ld_stream_b32(xs + i));
      const float q1 = (i + 32 < hiA) ? __int_as_float(ld_stream_b32(xs + i + 32)) : 0.f;
      const float q2 = (i + 64 < hiA) ? __int_as_float(ld_stream_b32(xs + i + 64)) : 0.f;
      const float q3 = (i + 96 < hiA) ? __int_as_float(ld_stream_b32(xs + i + 96)) : 0.f;
      tA += (q0 + q1) + (q2 + q3);
    }
    for (int64_t i = loB + lane + 32 * SEG_U; i < hiB; i += 128) {
      const float q0 = __int_as_float(ld_stream_b32(xs + i));
      const float q1 = (i + 32 < hiB) ? __int_as_float(ld_stream_b32(xs + i + 32)) : 0.f;
      const float q2 = (i + 64 < hiB) ? __int_as_float(ld_stream_b32(xs + i + 64)) : 0.f;
      const float q3 = (i + 96 < hiB) ? __int_as_float(ld_stream_b32(xs + i + 96)) : 0.f;
      tB += (q0 + q1) + (q2 + q3);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      tA += __shfl_down_sync(kFull, tA, o);
      tB += __shfl_down_sync(kFull, tB, o);
    }
    if (lane == 0) {
      out[sA] = tA;
      if (sB < nseg) out[sB] = tB;
    }
    sA = nA; sB = nB; loA = nloA; hiA = nhiA; loB = nloB; hiB = nhiB;
  }
}

cudaError_t launch_segreduce_f32(const int64_t *offsets, int64_t nseg, const float *xs, int64_t n, float *out,
                                 int num_sms, cudaStream_t stream) {
  if (nseg <= 0) return cudaSuccess;
  int64_t want = (nseg * 16 + RED_THREADS - 1) / RED_THREADS;     // a warp takes two segments at a time
  if (want < 1) want = 1;
  // persistent warps: exactly what is resident at once, so that no CTA waits for a second wave
  static int occ_dev[64];
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  if (occ_dev[dev] == 0) {
    int occ = 0;
    cudaError_t err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, segreduce_f32_kernel, RED_THREADS, 0);
    if (err != cudaSuccess) return err;
    occ_dev[dev] = occ < 1 ? 1 : occ;
  }
  const int64_t resident = (int64_t)num_sms * occ_dev[dev];
  int blocks = (int)(want < resident ? want : resident);
  segreduce_f32_kernel<<<blocks, RED_THREADS, 0, stream>>>(offsets, nseg, xs, n, out);
  return cudaGetLastError();
}

}  // namespace fb
