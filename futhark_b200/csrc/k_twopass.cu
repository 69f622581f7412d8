// Two-pass scan for operators the single-pass kernel cannot carry: its tile status word holds
// a 32-bit value, so an operator on 8-byte values or on tuples needs another route, as the
// reference's does when its single-pass kernel does not apply
// (src/Futhark/CodeGen/ImpGen/GPU/SegScan.hs:51-90 picks; SegScan/TwoPass.hs:146-316 scan
// stage one, :318-488 the scan of the per-block carries, :490-610 stage three, driver :621-682).
//
// Three launches over a grid of G CTAs, each owning one contiguous chunk of the input:
//   1. every CTA folds its chunk, tile by tile in order, into one aggregate;
//   2. one CTA scans the G aggregates (exclusive): the carry into each chunk;
//   3. every CTA scans its chunk, tile by tile, starting from its carry, and writes.
// The operator may be non-commutative: operands are always combined left to right.  A tile is
// 256 threads x 8 consecutive elements; a thread scans its elements, the warp scans the thread
// totals with shuffles (a value of any size is shuffled 32 bits at a time), the 8 warp totals go
// through shared memory.  The input is read twice and the output written once: 3 x 8 bytes per
// element for an 8-byte type against the 2 x 8 of a single pass, the price the reference's
// two-pass route pays as well.
//
// A specification supplies the value type T, identity(), combine(l, r), load(in0, in1, i) and
// store(out, i, v); the two below are the i64 prefix sum and the composition of affine maps
// x -> a * x + b, whose scan solves a first-order linear recurrence.
#include <string.h>

#include "common.cuh"
#include "kernels.h"

namespace fb {

constexpr int TP_THREADS = 256, TP_ITEMS = 8, TP_TILE = TP_THREADS * TP_ITEMS, TP_WARPS = TP_THREADS / 32;
constexpr int TP_MAX_CTAS = 1024;

struct TpAddI64 {
  using T = long long;
  static __device__ __forceinline__ T identity() { return 0; }
  static __device__ __forceinline__ T combine(T l, T r) { return (T)((unsigned long long)l + (unsigned long long)r); }   // wraps, as add64 does
  static __device__ __forceinline__ T load(const void *in0, const void *, int64_t i) { return reinterpret_cast<const T *>(in0)[i]; }
  static __device__ __forceinline__ void store(void *out, int64_t i, T v) { reinterpret_cast<T *>(out)[i] = v; }
};
// (a1, b1) then (a2, b2): x -> a2 * (a1 * x + b1) + b2.  No fused multiply-add, as in the
// reference's C (compiled without contraction).
struct TpAffineF32 {
  using T = float2;
  static __device__ __forceinline__ T identity() { return make_float2(1.f, 0.f); }
  static __device__ __forceinline__ T combine(T l, T r) {
    return make_float2(__fmul_rn(l.x, r.x), __fadd_rn(__fmul_rn(l.y, r.x), r.y));
  }
  static __device__ __forceinline__ T load(const void *in0, const void *in1, int64_t i) {
    return make_float2(reinterpret_cast<const float *>(in0)[i], reinterpret_cast<const float *>(in1)[i]);
  }
  static __device__ __forceinline__ void store(void *out, int64_t i, T v) { reinterpret_cast<float *>(out)[i] = v.y; }   // map (.1)
};

template <typename T>
__device__ __forceinline__ T shfl_up_any(T v, int delta) {
  static_assert(sizeof(T) % 4 == 0, "shuffled 32 bits at a time");
  uint32_t w[sizeof(T) / 4];
  memcpy(w, &v, sizeof(T));
#pragma unroll
  for (int k = 0; k < (int)(sizeof(T) / 4); k++) w[k] = __shfl_up_sync(kFull, w[k], delta);
  memcpy(&v, w, sizeof(T));
  return v;
}
template <typename T>
__device__ __forceinline__ T shfl_any(T v, int src) {
  uint32_t w[sizeof(T) / 4];
  memcpy(w, &v, sizeof(T));
#pragma unroll
  for (int k = 0; k < (int)(sizeof(T) / 4); k++) w[k] = __shfl_sync(kFull, w[k], src);
  memcpy(&v, w, sizeof(T));
  return v;
}

// The thread totals of one tile, in order: returns what precedes this thread inside the tile
// (exclusive), and in `tile_total` the fold of the whole tile.  `s_w` holds TP_WARPS values.
template <typename S>
__device__ __forceinline__ typename S::T block_exclusive(typename S::T total, typename S::T *s_w, typename S::T &tile_total) {
  using T = typename S::T;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  T inc = total;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const T l = shfl_up_any(inc, o);
    if (lane >= o) inc = S::combine(l, inc);
  }
  T exc = shfl_up_any(inc, 1);
  if (lane == 0) exc = S::identity();
  __syncthreads();                              // the previous tile's readers are done with s_w
  if (lane == 31) s_w[warp] = inc;
  __syncthreads();
  T w = lane < TP_WARPS ? s_w[lane] : S::identity();
#pragma unroll
  for (int o = 1; o < TP_WARPS; o <<= 1) {
    const T l = shfl_up_any(w, o);
    if (lane >= o) w = S::combine(l, w);
  }
  tile_total = shfl_any(w, TP_WARPS - 1);
  const T before = shfl_any(w, warp > 0 ? warp - 1 : 0);       // fold of the warps in front
  if (warp > 0) exc = S::combine(before, exc);
  return exc;
}

// stage 1 (WRITE = false, result to agg[blockIdx.x]) and stage 3 (WRITE = true, seeded with carry[blockIdx.x])
template <typename S, bool WRITE>
__global__ void __launch_bounds__(TP_THREADS)
twopass_chunk_kernel(const void *in0, const void *in1, void *out, int64_t n, int64_t chunk, typename S::T *agg, const typename S::T *carry) {
  using T = typename S::T;
  __shared__ T s_w[TP_WARPS];
  const int64_t lo = (int64_t)blockIdx.x * chunk, hi = lo + chunk < n ? lo + chunk : n;
  T running = WRITE ? carry[blockIdx.x] : S::identity();
  for (int64_t tb = lo; tb < hi; tb += TP_TILE) {
    const int64_t first = tb + (int64_t)threadIdx.x * TP_ITEMS;
    T x[TP_ITEMS];
#pragma unroll
    for (int q = 0; q < TP_ITEMS; q++) x[q] = (first + q < hi) ? S::load(in0, in1, first + q) : S::identity();
#pragma unroll
    for (int q = 1; q < TP_ITEMS; q++) x[q] = S::combine(x[q - 1], x[q]);
    T tile_total;
    const T exc = block_exclusive<S>(x[TP_ITEMS - 1], s_w, tile_total);
    if (WRITE) {
      const T pre = S::combine(running, exc);
#pragma unroll
      for (int q = 0; q < TP_ITEMS; q++)
        if (first + q < hi) S::store(out, first + q, S::combine(pre, x[q]));
    }
    running = S::combine(running, tile_total);
  }
  if (!WRITE && threadIdx.x == 0) agg[blockIdx.x] = running;
}

// stage 2: exclusive scan of the G <= 1024 aggregates by one CTA (4 per thread)
template <typename S>
__global__ void __launch_bounds__(TP_THREADS)
twopass_carries_kernel(const typename S::T *agg, typename S::T *carry, int G) {
  using T = typename S::T;
  __shared__ T s_w[TP_WARPS];
  constexpr int PER = TP_MAX_CTAS / TP_THREADS;
  T x[PER];
#pragma unroll
  for (int q = 0; q < PER; q++) { const int i = threadIdx.x * PER + q; x[q] = i < G ? agg[i] : S::identity(); }
#pragma unroll
  for (int q = 1; q < PER; q++) x[q] = S::combine(x[q - 1], x[q]);
  T total;
  const T exc = block_exclusive<S>(x[PER - 1], s_w, total);
#pragma unroll
  for (int q = 0; q < PER; q++) {
    const int i = threadIdx.x * PER + q;
    if (i < G) carry[i] = q == 0 ? exc : S::combine(exc, x[q - 1]);
  }
}

size_t twopass_scratch_bytes() { return 256 + 2 * (size_t)TP_MAX_CTAS * 8; }

template <typename S>
static cudaError_t launch_twopass(const void *in0, const void *in1, void *out, int64_t n, void *scratch, int num_sms, cudaStream_t stream) {
  using T = typename S::T;
  static_assert(sizeof(T) <= 8, "the scratch area holds 8 bytes per CTA and stage");
  if (n <= 0) return cudaSuccess;
  const int64_t tiles = (n + TP_TILE - 1) / TP_TILE;
  int64_t G = (int64_t)num_sms * 4;
  if (G > TP_MAX_CTAS) G = TP_MAX_CTAS;
  if (G > tiles) G = tiles;
  const int64_t chunk = ((tiles + G - 1) / G) * TP_TILE;        // whole tiles per CTA
  G = (n + chunk - 1) / chunk;
  T *agg = reinterpret_cast<T *>(reinterpret_cast<char *>(scratch) + 256);
  T *carry = agg + TP_MAX_CTAS;
  twopass_chunk_kernel<S, false><<<(int)G, TP_THREADS, 0, stream>>>(in0, in1, nullptr, n, chunk, agg, nullptr);
  twopass_carries_kernel<S><<<1, TP_THREADS, 0, stream>>>(agg, carry, (int)G);
  twopass_chunk_kernel<S, true><<<(int)G, TP_THREADS, 0, stream>>>(in0, in1, out, n, chunk, nullptr, carry);
  return cudaGetLastError();
}

cudaError_t launch_scan_i64(const int64_t *in, int64_t *out, int64_t n, void *scratch, int num_sms, cudaStream_t stream) {
  return launch_twopass<TpAddI64>(in, nullptr, out, n, scratch, num_sms, stream);
}
cudaError_t launch_linrec_f32(const float *as, const float *bs, float *out, int64_t n, void *scratch, int num_sms, cudaStream_t stream) {
  return launch_twopass<TpAffineF32>(as, bs, out, n, scratch, num_sms, stream);
}

}  // namespace fb
