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
// the area and keeps up to 16 bytes per CTA; the segmented sum needs a little more (see below)
size_t segreduce_scratch_bytes();
size_t reduce_scratch_bytes() {
  const size_t a = 256 + RED_MAX_BLOCKS * 16, b = segreduce_scratch_bytes();
  return a > b ? a : b;
}

// ---- reduce (+) 0 over i32 ----------------------------------------------------------
// Stage one: the warps stride over 2 KiB chunks of 16-byte vectors, four loads in flight per thread.
// Stage two (reductionStageTwo, SegRed.hs:923-1047, elects the last block with a counter and lets it
// fold the partials): here one 64-bit atomic addition per CTA does both.  The upper half of the word
// accumulates the partial sums (integer addition wraps, so any order gives the reference's bits, and
// what overflows the word is dropped), the lower half counts the CTAs and cannot carry into the sum;
// the CTA whose addition returns the count gridDim.x - 1 has the sum of all the others in the same
// answer, adds its own, writes the result and clears the word for the next launch.
// Six CTAs per SM, all resident at once (40 registers).  Measured at 2^26 elements: 8 per SM (32 registers,
// spills) 46.4 us, 6 per SM 45.3 us, 5 per SM 45.2 us, 4 per SM 45.6 us.
constexpr int RED_I32_CTAS_PER_SM = 6;
__global__ void __launch_bounds__(RED_THREADS, RED_I32_CTAS_PER_SM)
reduce_i32_kernel(const int32_t *__restrict__ in, int64_t n, int32_t *__restrict__ d_out, unsigned long long *sum_and_count) {
  __shared__ uint32_t s_warp[RED_THREADS / 32];
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
  // a warp takes 2 KiB at a time: four 16-byte loads per lane, 512 bytes apart, all in flight
  const int64_t nw = gthreads >> 5;
  int64_t base = (gtid >> 5) * 128 + lane;
  for (; base + 96 < nvec; base += nw * 128) {
    int4 v0 = ld_stream_v4(vec + base);
    int4 v1 = ld_stream_v4(vec + base + 32);
    int4 v2 = ld_stream_v4(vec + base + 64);
    int4 v3 = ld_stream_v4(vec + base + 96);
    a0 += (uint32_t)v0.x + (uint32_t)v0.y + (uint32_t)v0.z + (uint32_t)v0.w;
    a1 += (uint32_t)v1.x + (uint32_t)v1.y + (uint32_t)v1.z + (uint32_t)v1.w;
    a2 += (uint32_t)v2.x + (uint32_t)v2.y + (uint32_t)v2.z + (uint32_t)v2.w;
    a3 += (uint32_t)v3.x + (uint32_t)v3.y + (uint32_t)v3.z + (uint32_t)v3.w;
  }
#pragma unroll
  for (int k = 0; k < 4; k++)              // the last, partly filled chunk (every later one lies beyond the end)
    if (base + 32 * k < nvec) {
      int4 v0 = ld_stream_v4(vec + base + 32 * k);
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
      const unsigned long long old = atomicAdd(sum_and_count, ((unsigned long long)b << 32) | 1ull);
      if ((uint32_t)old == gridDim.x - 1) {
        *d_out = (int32_t)((uint32_t)(old >> 32) + b);
        *sum_and_count = 0ull;
      }
    }
  }
}

cudaError_t launch_reduce_i32(const int32_t *in, int64_t n, int32_t *d_out, void *scratch, int num_sms,
                              cudaStream_t stream, int block_cap) {
  if (n <= 0) return cudaMemsetAsync(d_out, 0, sizeof(int32_t), stream);   // the neutral element
  // the word lives in the head of the scratch area, beside the ticket of the other reductions; like the
  // ticket it is zero between launches
  unsigned long long *sum_and_count = reinterpret_cast<unsigned long long *>(reinterpret_cast<char *>(scratch) + 64);
  int64_t want = (n / 4 + RED_THREADS - 1) / RED_THREADS;
  int blocks = num_sms * RED_I32_CTAS_PER_SM;
  if (blocks > RED_MAX_BLOCKS) blocks = RED_MAX_BLOCKS;
  if (want < blocks) blocks = want < 1 ? 1 : (int)want;
  if (block_cap > 0 && block_cap < blocks) blocks = block_cap;       // reduce_i32.segred_num_tblocks
  reduce_i32_kernel<<<blocks, RED_THREADS, 0, stream>>>(in, n, d_out, sum_and_count);
  return cudaGetLastError();
}

// ---- a segmented redomap with a map-out result ---------------------------------------------------------
// map (\xs -> (reduce (+) 0 (map i64.f32 xs), map (\x -> f64.f32 (-x)) xs)) xss (tests/segredomap/ex1-comm.fut:11-15):
// the body's results that are not reduced are written by the thread that computes them while it reads
// (SegRed.hs:138-143, "write map-out result(s)").  One warp per row; i64.f32 is fptosi_f32_i64
// (rts/c/scalar.h:975-981): 0 for NaN and infinities.
__global__ void __launch_bounds__(RED_THREADS)
rowsum_mapout_kernel(const float *__restrict__ in, int64_t rows, int64_t cols, int64_t *__restrict__ sums, double *__restrict__ neg) {
  const int lane = threadIdx.x & 31;
  const int64_t warp_global = ((int64_t)blockIdx.x * RED_THREADS + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * RED_THREADS) >> 5;
  for (int64_t r = warp_global; r < rows; r += nwarps) {
    const float *row = in + r * cols;
    double *nrow = neg + r * cols;
    unsigned long long acc = 0ull;
    for (int64_t i = lane; i < cols; i += 32) {
      const float x = row[i];
      const bool odd = (x != x) || (fabsf(x) == INFINITY);
      acc += odd ? 0ull : (unsigned long long)(long long)x;
      nrow[i] = (double)(-x);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_down_sync(kFull, acc, o);
    if (lane == 0) sums[r] = (int64_t)acc;
  }
}
cudaError_t launch_rowsum_mapout(const float *in, int64_t rows, int64_t cols, int64_t *sums, double *neg, int num_sms, cudaStream_t stream) {
  if (rows <= 0) return cudaSuccess;
  int64_t want = (rows * 32 + RED_THREADS - 1) / RED_THREADS;
  const int64_t cap = (int64_t)num_sms * 8;
  rowsum_mapout_kernel<<<(int)(want < cap ? want : cap), RED_THREADS, 0, stream>>>(in, rows, cols, sums, neg);
  return cudaGetLastError();
}

// ---- reduce (map2 (+)) (replicate cols 0) over the rows of [rows][cols] i32 -------------------------
// A reduction whose operator works on whole rows (tests/soacs/reduce4.fut, reduce5.fut) is interchanged
// with the inner map (src/Futhark/Transform/ISRWIM.hs, irwim): every column is reduced on its own.  A thread
// owns a column over a band of rows, so a warp reads 128 consecutive bytes of every row; the bands of a
// column meet in one atomic addition each (integer addition wraps: any order gives the same bits).
__global__ void __launch_bounds__(RED_THREADS)
colsum_i32_kernel(const int32_t *__restrict__ in, int64_t rows, int64_t cols, int64_t band, int32_t *__restrict__ out) {
  const int64_t c = (int64_t)blockIdx.x * RED_THREADS + threadIdx.x;
  if (c >= cols) return;
  const int64_t r0 = (int64_t)blockIdx.y * band, r1 = r0 + band < rows ? r0 + band : rows;
  uint32_t a0 = 0, a1 = 0, a2 = 0, a3 = 0;
  int64_t r = r0;
  for (; r + 3 < r1; r += 4) {
    a0 += (uint32_t)in[r * cols + c];
    a1 += (uint32_t)in[(r + 1) * cols + c];
    a2 += (uint32_t)in[(r + 2) * cols + c];
    a3 += (uint32_t)in[(r + 3) * cols + c];
  }
  for (; r < r1; r++) a0 += (uint32_t)in[r * cols + c];
  atomicAdd(reinterpret_cast<uint32_t *>(out) + c, a0 + a1 + a2 + a3);
}
cudaError_t launch_colsum_i32(const int32_t *in, int64_t rows, int64_t cols, int32_t *out, int num_sms, cudaStream_t stream) {
  if (cols <= 0) return cudaSuccess;
  cudaError_t err = cudaMemsetAsync(out, 0, (size_t)cols * sizeof(int32_t), stream);     // the neutral element
  if (err != cudaSuccess || rows <= 0) return err;
  const int64_t col_blocks = (cols + RED_THREADS - 1) / RED_THREADS;
  int64_t bands = ((int64_t)num_sms * 8 + col_blocks - 1) / col_blocks;                   // enough CTAs to fill the GPU
  if (bands > (rows + 7) / 8) bands = (rows + 7) / 8;                                     // at least 8 rows per band
  if (bands > 65535) bands = 65535;
  if (bands < 1) bands = 1;
  const int64_t band = (rows + bands - 1) / bands;
  if (col_blocks > 2147483647) return cudaErrorInvalidValue;
  colsum_i32_kernel<<<dim3((unsigned)col_blocks, (unsigned)((rows + band - 1) / band)), RED_THREADS, 0, stream>>>(in, rows, cols, band, out);
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
                              cudaStream_t stream, int64_t suff_outer_par, int block_cap) {
  if (rows <= 0) return cudaSuccess;
  if (cols <= 0) return cudaMemsetAsync(out, 0, (size_t)rows * sizeof(float), stream);
  if (cols < 16) {
    int64_t want = (rows + RED_THREADS - 1) / RED_THREADS;
    int blocks = (int)(want < (int64_t)num_sms * 8 ? want : (int64_t)num_sms * 8);
    rowsum_thread_kernel<<<blocks, RED_THREADS, 0, stream>>>(in, rows, cols, out);
  } else if (cols <= 16384 || rows >= suff_outer_par) {
    int64_t want = (rows * 32 + RED_THREADS - 1) / RED_THREADS;
    int blocks = (int)(want < (int64_t)num_sms * 8 ? want : (int64_t)num_sms * 8);
    if (block_cap > 0 && block_cap < blocks) blocks = block_cap;       // rowsum_f32.segred_num_tblocks
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
// The values are streamed through shared memory in tiles of 7168 elements, each CTA owning a
// contiguous run of tiles, the next tile's bulk async copy (TMA) in flight while the current
// one is summed.  Segment boundaries come from the offsets alone (the flags of the entry point
// are not consulted: what is summed is exactly [offsets[s], offsets[s+1])).
//
// A CTA has nine warps.  In the eight worker warps a thread owns a chunk of 28 consecutive
// elements of the tile; with segments of a few hundred elements nine chunks in ten contain no
// boundary, so the work is split by who has something to do:
//
//   * The ninth warp (the walker) only walks the offsets, one tile ahead of the workers and
//     without touching the values.  A CTA finds its first offset by a 288-ary search, then
//     the walker moves a cursor forward, 32 offsets per round, loaded a tile ahead of their
//     use.  For every boundary in the tile one lane notes the boundary's chunk, the elements
//     of that chunk that lie in front of it (back to the chunk's start or to the previous
//     boundary, whichever is nearer) and, for the chunk's last boundary, where it lies.
//   * A worker adds up its chunk: 27 additions and no tests, or, if the chunk has a
//     boundary, the elements behind the last one (they open the next segment).
//   * Then one segmented scan with the lifted operator (f1|f2, f2 ? v2 : v1+v2) of
//     Pass/Flatten/Builtins.hs:374-393 runs over the 256 chunk values (a chunk with a
//     boundary counts as flagged): shuffles inside the warps, the 8 warp totals through
//     shared memory.  It is the scan-then-pick of genSegRed (Pass/Flatten/Builtins.hs:582-602)
//     at one value per 28 elements.
//   * Finally worker b finishes boundary b: it sums the elements in front of the boundary
//     inside the boundary's chunk out of the tile buffer; that, plus the scan value of the
//     chunk before (with the carry of the earlier tiles), is the segment's total, stored at
//     the segment's index = cursor + b - 1.
//   * A tile with equal offsets (empty segments) or more than 256 boundaries takes a general
//     route: the boundaries become one bit per element, every thread folds its 28 elements
//     under them, the scanned tile goes back into the buffer and one thread per offset picks
//     its value (0 for an empty segment).
//   * What crosses a tile edge is carried in registers; what crosses the edge between two
//     CTAs' runs goes through one record per CTA (sum in front of its first segment end, sum
//     behind its last, index of the first ending segment), and the CTA that finishes last
//     joins the records in order.  No atomics on floats: the result is deterministic.
constexpr int SR_V = 7, SR_ITEMS = SR_V * 4, SR_TILE = RED_THREADS * SR_ITEMS;   // 7168 elements, 28 KiB (SR_V odd: conflict-free 16-byte reads; SR_ITEMS <= 31)
constexpr int SR_WARPS = RED_THREADS / 32;
constexpr int SR_MAX_CTAS = 2048;
constexpr int SR_THREADS = RED_THREADS + 32;                       // 8 warps on the chunks, one on the offsets
// Two tile buffers and three CTAs per SM.  Measured at 2^27 elements, elements per thread x buffers x CTAs per SM:
// 28 x 2 x 3 99.1 us; 20 x 2 x 4 103.5 us; 24 x 2 x 4 103.9 us (two-way bank conflicts); 20 x 3 x 3 110.9 us;
// 20 x 4 x 2 121.7 us.
constexpr int SR_NBUF = 2, SR_CTAS_PER_SM = 3;
constexpr int SR_BIG = 1 << 29;

struct SegRedRecord {       // 16 bytes, one per CTA, in the reduce scratch behind the ticket
  float head;               // sum of the CTA's elements in front of its first segment end
  float tail;               // sum behind its last segment end (of everything if it has none)
  int32_t any_end;
  int32_t pad;
};

__device__ __forceinline__ void seg_combine(float lv, uint32_t lf, float rv, uint32_t rf, float &ov, uint32_t &of) {
  ov = rf ? rv : lv + rv;
  of = lf | rf;
}

// Inclusive scan of the SR_WARPS warp totals in shared memory, done by every warp for itself:
// lane w < SR_WARPS ends up with the fold of warps 0..w.
__device__ __forceinline__ void scan_warp_totals(const float *s_wv, const uint32_t *s_wf, int lane, float &wv, uint32_t &wf) {
  wv = lane < SR_WARPS ? s_wv[lane] : 0.f;
  wf = lane < SR_WARPS ? s_wf[lane] : 0u;
#pragma unroll
  for (int o = 1; o < SR_WARPS; o <<= 1) {
    const float lv = __shfl_up_sync(kFull, wv, o);
    const uint32_t lf = __shfl_up_sync(kFull, wf, o);
    if (lane >= o) seg_combine(lv, lf, wv, wf, wv, wf);
  }
}

// s[0] + ... + s[N-1] as a tree: the largest power of two below N on the left, the rest on the right
template <int N>
__device__ __forceinline__ float tree_sum(const float *s) {
  if constexpr (N == 1) return s[0];
  else {
    constexpr int H = (N > 4) ? 4 : (N > 2) ? 2 : 1;
    static_assert(N <= 8, "tree_sum: at most 8 terms");
    return tree_sum<H>(s) + tree_sum<N - H>(s + H);
  }
}

__device__ __forceinline__ void workers_barrier() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

__global__ void __launch_bounds__(SR_THREADS, SR_CTAS_PER_SM)
segreduce_tiled_kernel(const int64_t *__restrict__ offsets, int64_t nseg, const float *xs_al, int shift, int64_t n,
                       float *__restrict__ out, uint32_t num_tiles, uint32_t tiles_per_cta, uint32_t *ticket,
                       SegRedRecord *records, int64_t *head_seg, int *failure) {
  constexpr int NBUF = SR_NBUF;
  extern __shared__ __align__(128) unsigned char sr_smem[];
  float *s_buf = reinterpret_cast<float *>(sr_smem);                   // NBUF tile buffers
  __shared__ __align__(8) uint64_t s_bar[NBUF];
  __shared__ uint32_t s_rl[2][RED_THREADS];     // chunk with a boundary: 1 + the element behind which its last boundary lies (cleared by its thread once read)
  __shared__ float s_scan_v[RED_THREADS];       // warp-local inclusive scan of the chunk values
  __shared__ uint32_t s_scan_f[RED_THREADS];
  __shared__ uint32_t s_pe[2][RED_THREADS];     // boundary b of the tile: chunk | last element in front << 8 | first element of the sum in front << 13 | segment began inside the chunk << 18
  __shared__ int s_ctl[2][2];                   // boundaries in the tile, general route wanted
  __shared__ int64_t s_cur[2][2];               // cursor in front of the tile and behind it
  __shared__ uint32_t s_mask[RED_THREADS];      // general route: one bit per element
  __shared__ float s_wv[SR_WARPS];
  __shared__ uint32_t s_wf[SR_WARPS];
  __shared__ uint32_t s_last;
  __shared__ volatile uint32_t s_fail;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bool walker = (warp == SR_WARPS);                              // the ninth warp walks the offsets, one tile ahead of the others
  const uint32_t t0 = blockIdx.x * tiles_per_cta;
  const uint32_t t1 = (t0 + tiles_per_cta < num_tiles) ? t0 + tiles_per_cta : num_tiles;
  const int64_t nv = n + shift;                                        // elements of the shifted (16-byte aligned) array
  const int64_t noff = nseg + 1;
  // offset j as a position in the shifted array, clamped into it
  auto off_at = [&](int64_t j) -> int64_t {
    if (j >= noff) return INT64_MAX;
    int64_t o = offsets[j];
    o = o < 0 ? 0 : (o > n ? n : o);
    return o + shift;
  };
  auto arm = [&](int b, uint32_t t) {                                  // thread 0
    const int64_t tb = (int64_t)t * SR_TILE;
    int64_t cnt = nv - tb;
    if (cnt > SR_TILE) cnt = SR_TILE;
    const uint32_t bytes = (uint32_t)(((cnt + 3) >> 2) << 4);          // whole 16-byte pieces; the last may reach past nv inside its piece
    mbar_expect_tx(&s_bar[b], bytes);
    bulk_g2s(s_buf + b * SR_TILE, xs_al + tb, bytes, &s_bar[b]);
  };
  // Waits for the copy of the CTA's tile number `rel`; every thread waits for every tile once, in order.
  auto landed = [&](uint32_t rel) {
    if (!mbar_wait_bounded(&s_bar[rel % NBUF], (rel / NBUF) & 1u)) {
      atomicCAS(failure, FAIL_NONE, FAIL_BULK_COPY_TIMEOUT);
      s_fail = 1;
    }
  };
  uint32_t armed_to = t0;                                              // thread 0: tiles below this have had their copy started
  if (tid == 0) {
    for (int b = 0; b < NBUF; b++) mbar_init(&s_bar[b], 1);
    fence_mbar_init();
    s_fail = 0;
    records[blockIdx.x].head = 0.f;
    head_seg[blockIdx.x] = -1;                                         // until a thread meets the run's first segment end
    for (int b = 0; b < NBUF - 1; b++)
      if (t0 + b < t1) { arm(b, t0 + b); armed_to = t0 + b + 1; }
  }
  if (tid < RED_THREADS) { s_rl[0][tid] = 0u; s_rl[1][tid] = 0u; s_mask[tid] = 0u; }
  __syncthreads();

  // ---- cursor: first offset behind the start of this CTA's run
  const int64_t run_lo = (int64_t)t0 * SR_TILE;
  int64_t cur0;
  {
    int64_t lo = 0, hi = noff;                                         // offsets below lo are <= run_lo, offsets from hi on are > run_lo
    while (lo < hi) {
      const int64_t span = hi - lo, step = (span + SR_THREADS - 1) / SR_THREADS;
      const int64_t idx = lo + (int64_t)tid * step + (step - 1);
      const bool le = (idx < hi) && (off_at(idx) <= run_lo);
      const int64_t c = __syncthreads_count(le);
      const int64_t nlo = lo + c * step;
      const int64_t nhi = (c < SR_THREADS && nlo + step - 1 < hi) ? nlo + step - 1 : hi;
      lo = nlo < hi ? nlo : hi;
      hi = nhi;
      if (step == 1) break;
    }
    cur0 = lo;                                                         // the offset that is the CTA's first segment end, if it has one
  }
  // offsets equal to position 0 (CTA 0 only, array not shifted): all but the last start an empty segment
  if (t0 == 0)
    for (int64_t j = 1 + tid; j < cur0; j += SR_THREADS) out[j - 1] = 0.f;

  // ---- the walker: the boundaries of one tile into the shared-memory set `par` (positions only: it never touches the values)
  int64_t cur = cur0;                                                  // walker: the cursor
  int64_t w_off = INT64_MAX, w_nxt = INT64_MAX;                        // walker: the window of the next round, and the offsets one further
  if (walker) { w_off = off_at(cur + lane); w_nxt = off_at(cur + lane + 1); }
  auto walk = [&](uint32_t t, int par) {
    const int64_t tb = (int64_t)t * SR_TILE;
    int total = 0, p_prev = 0;
    bool general = false;
    if (lane == 0) s_cur[par][0] = cur;
    while (true) {
      const bool in = (w_off <= tb + SR_TILE);
      const int c = __popc(__ballot_sync(kFull, in));
      if (c == 0) break;
      const int p = in ? (int)(w_off - tb) : SR_BIG;                   // boundary in front of element p, 1 <= p <= TILE
      const int pn = (w_nxt <= tb + SR_TILE) ? (int)(w_nxt - tb) : SR_BIG;
      int pp = __shfl_up_sync(kFull, p, 1);
      if (lane == 0) pp = p_prev;
      const bool bad = in && (p <= pp || p < 1);                       // equal offsets (or offsets out of order): not for this route
      if (__any_sync(kFull, bad) || total + c > RED_THREADS) general = true;
      if (in && !general) {
        const int e = p - 1, ke = e / SR_ITEMS, base = ke * SR_ITEMS, r = e - base;
        const bool inner = (pp - 1 >= base);                           // the segment that ends here began in this chunk
        const int start = inner ? pp - base : 0;
        if (pn - 1 >= base + SR_ITEMS) s_rl[par][ke] = (uint32_t)(r + 1);      // the chunk's last boundary
        s_pe[par][total + lane] = (uint32_t)ke | ((uint32_t)r << 8) | ((uint32_t)start << 13) | (inner ? (1u << 18) : 0u);
      }
      p_prev = __shfl_sync(kFull, p, c - 1);
      total += c;
      cur += c;
      w_off = off_at(cur + lane);
      w_nxt = off_at(cur + lane + 1);
      if (c < 32) break;
    }
    if (lane == 0) { s_ctl[par][0] = total; s_ctl[par][1] = general ? 1 : 0; s_cur[par][1] = cur; }
  };
  if (walker && t0 < t1) walk(t0, 0);

  float carry_v = 0.f;
  uint32_t carry_f = 0u;
  int64_t cur_end = cur0;                                              // workers: the cursor behind the last tile they finished
  for (uint32_t t = t0; t < t1; t++) {
    const int par = (int)((t - t0) & 1u);
    __syncthreads();                                                   // tile t's boundaries are in set `par`; tile t-1 is finished
    if (s_fail) break;
    // the buffer of tile t-1 is free
    if (tid == 0 && t + NBUF - 1 < t1) { arm((int)((t - t0 + NBUF - 1) % NBUF), t + NBUF - 1); armed_to = t + NBUF; }
    if (walker) {
      if (t + 1 < t1) walk(t + 1, par ^ 1);
      continue;
    }
    landed(t - t0);
    const int64_t tb = (int64_t)t * SR_TILE;
    float *tile = s_buf + ((t - t0) % NBUF) * SR_TILE;
    const int nbound = s_ctl[par][0];
    const bool general = s_ctl[par][1] != 0;
    const int64_t cur_tile = s_cur[par][0];
    cur_end = s_cur[par][1];

    if (!general) {
      // ---- the thread's chunk: its plain sum, or what lies behind its last boundary; then the segmented scan of these values
      float x[SR_ITEMS];
      {
        const float4 *s4 = reinterpret_cast<const float4 *>(tile) + tid * SR_V;
#pragma unroll
        for (int j = 0; j < SR_V; j++) {
          const float4 q = s4[j];
          x[4 * j + 0] = q.x; x[4 * j + 1] = q.y; x[4 * j + 2] = q.z; x[4 * j + 3] = q.w;
        }
      }
      const uint32_t rl = s_rl[par][tid];
      uint32_t ifl = rl ? 1u : 0u;
      float iv;
      if (rl == 0u) {
        float q4[SR_V];
#pragma unroll
        for (int j = 0; j < SR_V; j++) q4[j] = (x[4 * j] + x[4 * j + 1]) + (x[4 * j + 2] + x[4 * j + 3]);
        iv = tree_sum<SR_V>(q4);
      } else {
        s_rl[par][tid] = 0u;
        iv = 0.f;
#pragma unroll
        for (int q = 1; q < SR_ITEMS; q++) iv += ((uint32_t)q >= rl) ? x[q] : 0.f;
      }
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float lv = __shfl_up_sync(kFull, iv, o);
        const uint32_t lf = __shfl_up_sync(kFull, ifl, o);
        if (lane >= o) seg_combine(lv, lf, iv, ifl, iv, ifl);
      }
      s_scan_v[tid] = iv; s_scan_f[tid] = ifl;
      if (lane == 31) { s_wv[warp] = iv; s_wf[warp] = ifl; }
      workers_barrier();                                               // scan known
      float wv;
      uint32_t wf;
      scan_warp_totals(s_wv, s_wf, lane, wv, wf);
      // ---- thread b finishes boundary b
      uint32_t pe = 0u;
      if (tid < nbound) pe = s_pe[par][tid];
      const int ke = (int)(pe & 255u);
      const int wsrc = ke > 0 ? ((ke - 1) >> 5) : 0;                   // warp of the chunk in front
      const float bwv = __shfl_sync(kFull, wv, wsrc > 0 ? wsrc - 1 : 0);
      const uint32_t bwf = __shfl_sync(kFull, wf, wsrc > 0 ? wsrc - 1 : 0);
      if (tid < nbound) {
        // the sum in front of the boundary inside its chunk, straight out of the tile
        const int r = (int)((pe >> 8) & 31u), start = (int)((pe >> 13) & 31u);
        float L = 0.f;
        {
          const float4 *c4 = reinterpret_cast<const float4 *>(tile + ke * SR_ITEMS);
#pragma unroll
          for (int k = 0; k < SR_V; k++) {
            const float4 q4 = c4[k];
            L += (4 * k + 0 >= start && 4 * k + 0 <= r) ? q4.x : 0.f;
            L += (4 * k + 1 >= start && 4 * k + 1 <= r) ? q4.y : 0.f;
            L += (4 * k + 2 >= start && 4 * k + 2 <= r) ? q4.z : 0.f;
            L += (4 * k + 3 >= start && 4 * k + 3 <= r) ? q4.w : 0.f;
          }
        }
        float v = L;
        if (!(pe & (1u << 18))) {
          float pv = carry_v;
          uint32_t pf = carry_f;
          if (ke > 0) {
            if (wsrc > 0) seg_combine(pv, pf, bwv, bwf, pv, pf);
            seg_combine(pv, pf, s_scan_v[ke - 1], s_scan_f[ke - 1], pv, pf);
          }
          v = pv + L;
        }
        const int64_t j = cur_tile + tid;                              // this boundary is offset j: it closes segment j - 1
        if (j == cur0) { records[blockIdx.x].head = v; head_seg[blockIdx.x] = j - 1; }
        else out[j - 1] = v;
      }
      seg_combine(carry_v, carry_f, __shfl_sync(kFull, wv, SR_WARPS - 1), __shfl_sync(kFull, wf, SR_WARPS - 1), carry_v, carry_f);
      continue;
    }

    // ---- general route: one bit per element "a segment ends behind this element"
    s_rl[par][tid] = 0u;                                               // what the walker may have left before it gave up
    for (int64_t j = cur_tile + tid; j < cur_end; j += RED_THREADS) {
      const int64_t p = off_at(j) - tb;
      if (p >= 1 && p <= SR_TILE) atomicOr(&s_mask[(uint32_t)(p - 1) / SR_ITEMS], 1u << ((uint32_t)(p - 1) % SR_ITEMS));
    }
    workers_barrier();
    const uint32_t ends = s_mask[tid];
    const uint32_t before = tid > 0 ? (s_mask[tid - 1] >> (SR_ITEMS - 1)) & 1u : 0u;
    const uint32_t last_bit = (s_mask[RED_THREADS - 1] >> (SR_ITEMS - 1)) & 1u;
    const uint32_t starts = ((ends << 1) | before) & ((1u << SR_ITEMS) - 1u);
    float x[SR_ITEMS];
    {
      const float4 *s4 = reinterpret_cast<const float4 *>(tile) + tid * SR_V;
#pragma unroll
      for (int j = 0; j < SR_V; j++) {
        const float4 q = s4[j];
        x[4 * j + 0] = q.x; x[4 * j + 1] = q.y; x[4 * j + 2] = q.z; x[4 * j + 3] = q.w;
      }
    }
    float acc = 0.f;
#pragma unroll
    for (int q = 0; q < SR_ITEMS; q++) {
      acc = ((starts >> q) & 1u) ? x[q] : acc + x[q];
      x[q] = acc;
    }
    float iv = acc;
    uint32_t ifl = starts ? 1u : 0u;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float lv = __shfl_up_sync(kFull, iv, o);
      const uint32_t lf = __shfl_up_sync(kFull, ifl, o);
      if (lane >= o) seg_combine(lv, lf, iv, ifl, iv, ifl);
    }
    float xv = __shfl_up_sync(kFull, iv, 1);
    uint32_t xf = __shfl_up_sync(kFull, ifl, 1);
    if (lane == 0) { xv = 0.f; xf = 0u; }
    if (lane == 31) { s_wv[warp] = iv; s_wf[warp] = ifl; }
    workers_barrier();
    s_mask[tid] = 0u;
    float wv;
    uint32_t wf;
    scan_warp_totals(s_wv, s_wf, lane, wv, wf);
    float lv = carry_v;
    uint32_t lf = carry_f;
    if (warp > 0) seg_combine(lv, lf, __shfl_sync(kFull, wv, warp - 1), __shfl_sync(kFull, wf, warp - 1), lv, lf);
    seg_combine(lv, lf, xv, xf, lv, lf);                               // what precedes this thread, the carry included
    const int first = starts ? (__ffs(starts) - 1) : SR_ITEMS;
#pragma unroll
    for (int q = 0; q < SR_ITEMS; q++)
      if (q < first) x[q] = lv + x[q];
    {
      float4 *s4 = reinterpret_cast<float4 *>(tile) + tid * SR_V;
#pragma unroll
      for (int j = 0; j < SR_V; j++) s4[j] = make_float4(x[4 * j + 0], x[4 * j + 1], x[4 * j + 2], x[4 * j + 3]);
    }
    fence_proxy_async_smem();                                          // a later bulk copy refills this buffer
    workers_barrier();
    for (int64_t j = cur_tile + tid; j < cur_end; j += RED_THREADS) {
      const int64_t o = off_at(j), p = o - tb;
      if (p < 1 || p > SR_TILE || j < 1) continue;                     // offset 0 ends nothing
      const bool empty = off_at(j - 1) == o;
      const float v = empty ? 0.f : tile[p - 1];
      if (j == cur0) { records[blockIdx.x].head = v; head_seg[blockIdx.x] = j - 1; }
      else out[j - 1] = v;
    }
    seg_combine(carry_v, carry_f, __shfl_sync(kFull, wv, SR_WARPS - 1), __shfl_sync(kFull, wf, SR_WARPS - 1), carry_v, carry_f);
    if (last_bit) { carry_v = 0.f; carry_f = 1u; }                     // a boundary behind the tile's last element
  }
  // ---- this CTA's record, then the last CTA to finish joins the records in order
  __syncthreads();
  if (tid == 0) {
    records[blockIdx.x].tail = carry_v;
    records[blockIdx.x].any_end = (cur_end > cur0) ? 1 : 0;
    __threadfence();
    const uint32_t tk = atomicAdd(ticket, 1u);
    s_last = (tk == gridDim.x - 1) ? 1u : 0u;
    // after a failure copies may still be in flight: they must land before the CTA's shared memory goes
    if (s_fail)
      for (uint32_t t = t0; t < armed_to; t++) (void)mbar_wait_bounded(&s_bar[(t - t0) % NBUF], ((t - t0) / NBUF) & 1u, 1u << 16);
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // Exclusive segmented scan over the records (flag = the CTA has a segment end, value = tail):
  // the sum that is open in front of CTA c.  Each of 256 threads takes a contiguous group of records.
  const int C = (int)gridDim.x;
  const int per = (C + RED_THREADS - 1) / RED_THREADS;
  const int c_lo = tid * per < C ? tid * per : C, c_hi = (c_lo + per < C) ? c_lo + per : C;
  const volatile SegRedRecord *rec = records;
  float gv = 0.f;
  uint32_t gf = 0u;
  for (int c = c_lo; c < c_hi; c++) seg_combine(gv, gf, rec[c].tail, (uint32_t)rec[c].any_end, gv, gf);
  float iv = gv;
  uint32_t ifl = gf;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float lv = __shfl_up_sync(kFull, iv, o);
    const uint32_t lf = __shfl_up_sync(kFull, ifl, o);
    if (lane >= o) seg_combine(lv, lf, iv, ifl, iv, ifl);
  }
  float xv = __shfl_up_sync(kFull, iv, 1);
  uint32_t xf = __shfl_up_sync(kFull, ifl, 1);
  if (lane == 0) { xv = 0.f; xf = 0u; }
  if (lane == 31 && warp < SR_WARPS) { s_wv[warp] = iv; s_wf[warp] = ifl; }
  __syncthreads();
  float wv;
  uint32_t wf;
  scan_warp_totals(s_wv, s_wf, lane, wv, wf);
  float run_v = 0.f;
  uint32_t run_f = 0u;
  if (warp > 0) { run_v = __shfl_sync(kFull, wv, warp - 1); run_f = __shfl_sync(kFull, wf, warp - 1); }
  seg_combine(run_v, run_f, xv, xf, run_v, run_f);
  const volatile int64_t *hs = head_seg;
  for (int c = c_lo; c < c_hi; c++) {
    if (rec[c].any_end) {
      const int64_t sg = hs[c];
      if (sg >= 0) out[sg] = run_v + rec[c].head;
    }
    seg_combine(run_v, run_f, rec[c].tail, (uint32_t)rec[c].any_end, run_v, run_f);
  }
  if (tid == 0) *ticket = 0u;
}

// Scratch layout: [0,4) ticket | 256: records (16 B x SR_MAX_CTAS) | one i64 per CTA (index of the segment its first end closes).
size_t segreduce_scratch_bytes() { return 256 + (size_t)SR_MAX_CTAS * 16 + 8 * (size_t)SR_MAX_CTAS; }

cudaError_t launch_segreduce_f32(const int64_t *offsets, int64_t nseg, const float *xs, int64_t n, float *out,
                                 void *scratch, int *failure, int num_sms, cudaStream_t stream) {
  if (nseg <= 0) return cudaSuccess;
  if (n <= 0) return cudaMemsetAsync(out, 0, (size_t)nseg * sizeof(float), stream);     // every segment is empty
  // the array seen from the 16-byte boundary at or below its first element
  const int shift = (int)((reinterpret_cast<uintptr_t>(xs) & 15u) >> 2);
  const float *xs_al = xs - shift;
  const int64_t nv = n + shift;
  const uint32_t num_tiles = (uint32_t)((nv + SR_TILE - 1) / SR_TILE);
  uint32_t *ticket = reinterpret_cast<uint32_t *>(scratch);
  SegRedRecord *records = reinterpret_cast<SegRedRecord *>(reinterpret_cast<char *>(scratch) + 256);
  int64_t *head_seg = reinterpret_cast<int64_t *>(reinterpret_cast<char *>(scratch) + 256 + (size_t)SR_MAX_CTAS * 16);
  constexpr size_t smem = (size_t)SR_NBUF * SR_TILE * sizeof(float);
  // static + dynamic shared memory exceed 48 KiB: the dynamic part has to be opted into (per device)
  static bool opted[64];
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  if (!opted[dev]) {
    cudaError_t err = cudaFuncSetAttribute(segreduce_tiled_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return err;
    opted[dev] = true;
  }
  uint32_t ctas = (uint32_t)(num_sms * SR_CTAS_PER_SM);
  if (ctas > (uint32_t)SR_MAX_CTAS) ctas = SR_MAX_CTAS;
  if (ctas > num_tiles) ctas = num_tiles;
  const uint32_t per = (num_tiles + ctas - 1) / ctas;
  const uint32_t grid = (num_tiles + per - 1) / per;
  segreduce_tiled_kernel<<<grid, SR_THREADS, smem, stream>>>(offsets, nseg, xs_al, shift, n, out, num_tiles, per, ticket, records,
                                                           head_seg, failure);
  return cudaGetLastError();
}

}  // namespace fb
