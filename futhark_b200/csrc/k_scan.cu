// Single-pass decoupled look-back kernels: inclusive scan (+) over i32, flagged
// segmented inclusive scan (+) over f32, and filter / partition compaction of u32
// keys.  They replace the generated `segscan` kernel of the reference
// (src/Futhark/CodeGen/ImpGen/GPU/SegScan/SinglePass.hs:327-879) and, for
// compaction, the scan + scatter that prelude/soacs.fut:241-286 expands into.
//
// Shape shared by the three kernels (one CTA per tile of 256 x 20 elements):
//   1. thread 0 draws a tile number from a ticket counter, so tile i starts only
//      after every tile < i has started -- the property that makes waiting on
//      predecessors safe (the reference draws its `dyn_id` the same way, :444-461);
//   2. the tile is brought into shared memory with ONE bulk async copy (TMA) per
//      array and awaited on an mbarrier; a thread then owns 20 CONSECUTIVE elements
//      = 5 x 16 bytes, a stride of 5 sixteen-byte units, which is odd, so the
//      128-bit shared-memory reads are bank-conflict free without padding;
//   3. per-thread sequential scan, warp-shuffle scan of thread totals, 8 warp totals
//      through shared memory;
//   4. warp 0 publishes the tile aggregate and looks back over its predecessors,
//      32 status words at a time; every wait is bounded and polls the failure word;
//   5. results go back to shared memory and leave with one bulk async store (scan),
//      or are compacted in shared memory and written as contiguous runs (compaction).
// A tile that is ragged (the last one) or whose global addresses are not 16-byte
// aligned uses plain guarded loads and stores instead of the bulk copies.
#include <stdio.h>

#include <mutex>

#include "../../include/futhark_b200.h"
#include "common.cuh"
#include "kernels.h"

namespace fb {

constexpr int SCAN_THREADS = 256;
constexpr int SCAN_ITEMS = 20;
constexpr int SCAN_TILE = SCAN_THREADS * SCAN_ITEMS;  // 5120 elements
constexpr int SCAN_WARPS = SCAN_THREADS / 32;
constexpr uint32_t LOOKBACK_MAX_ROUNDS = 1u << 21;

// ---- operators on (value bits, flag) pairs -----------------------------------------
struct OpAddU32 {  // wrapping integer add; the flag is unused (always 0)
  static __device__ __forceinline__ void combine(uint32_t lv, uint32_t lf, uint32_t rv, uint32_t rf,
                                                 uint32_t &ov, uint32_t &of) {
    ov = lv + rv; of = 0; (void)lf; (void)rf;
  }
  static constexpr bool kHasFlag = false;
};
struct OpSegAddF32 {  // (f1,v1) (+) (f2,v2) = (f1|f2, f2 ? v2 : v1+v2) on f32 bit patterns
  static __device__ __forceinline__ void combine(uint32_t lv, uint32_t lf, uint32_t rv, uint32_t rf,
                                                 uint32_t &ov, uint32_t &of) {
    float s = __uint_as_float(lv) + __uint_as_float(rv);
    ov = rf ? rv : __float_as_uint(s);
    of = lf | rf;
  }
  static constexpr bool kHasFlag = true;
};

// ---- ticket ---------------------------------------------------------------------
// Returns this CTA's tile number; the CTA that draws the last ticket rewinds the
// counter for the next launch.
__device__ __forceinline__ uint32_t draw_tile(uint32_t *ticket, uint32_t num_tiles, uint32_t *s_slot) {
  if (threadIdx.x == 0) {
    uint32_t t = atomicAdd(ticket, 1u);
    if (t == num_tiles - 1) atomicExch(ticket, 0u);
    *s_slot = t;
  }
  __syncthreads();
  return *s_slot;
}

// ---- look-back (warp 0 only, all 32 lanes) ---------------------------------------
// Publishes this tile's aggregate (or, when the tile's own prefix does not depend on
// its predecessors, its inclusive prefix), then combines predecessors from the
// nearest one backwards until one with a known inclusive prefix (or, for the
// segmented operator, one containing a segment start) is met.  Returns the exclusive
// prefix of the tile in (ev, ef) -- valid in every lane -- or false after a timeout.
template <typename Op>
__device__ __forceinline__ bool tile_lookback(uint64_t *status, uint32_t tile, uint32_t epoch,
                                              uint32_t agg_v, uint32_t agg_f,
                                              uint32_t carry_v, int *failure,
                                              uint32_t &ev, uint32_t &ef) {
  const int lane = threadIdx.x & 31;
  if (tile == 0) {
    ev = carry_v; ef = 0;
    uint32_t iv, iflag;
    Op::combine(ev, ef, agg_v, agg_f, iv, iflag);
    if (lane == 0) st_status(&status[0], pack_status(iv, epoch, iflag, ST_PREFIX));
    return true;
  }
  // A tile containing a segment start has an inclusive prefix equal to its aggregate.
  const bool self_contained = Op::kHasFlag && agg_f;
  if (lane == 0)
    st_status(&status[tile], pack_status(agg_v, epoch, agg_f, self_contained ? ST_PREFIX : ST_AGG));

  uint32_t acc_v = 0, acc_f = 0;        // identity of both operators
  bool have_acc = false;
  int64_t j = (int64_t)tile - 1;        // nearest predecessor handled by lane 0
  uint32_t rounds = 0;
  while (true) {
    const int64_t idx = j - lane;
    uint64_t w = 0;
    uint32_t st;
    // poll until every lane of the window has something
    while (true) {
      if (idx >= 0) { w = ld_status(&status[idx]); st = status_state(w, epoch); }
      else { st = ST_PREFIX; }
      if (__all_sync(kFull, st != ST_NONE)) break;
      rounds++;
      if ((rounds & 63u) == 0) {
        int f = (lane == 0) ? ld_failure(failure) : 0;
        f = __shfl_sync(kFull, f, 0);
        if (f != FAIL_NONE) return false;
        if (rounds >= LOOKBACK_MAX_ROUNDS) {
          if (lane == 0) atomicCAS(failure, FAIL_NONE, FAIL_LOOKBACK_TIMEOUT);
          return false;
        }
      }
      if (rounds > 16) __nanosleep(rounds > 1024 ? 256 : 32);
    }
    uint32_t v, f;
    if (idx >= 0) { v = status_value(w); f = Op::kHasFlag ? status_flag(w) : 0u; }
    else { v = (idx == -1) ? carry_v : 0u; f = 0u; }   // virtual tile -1 carries the seed
    const bool stop = (st == ST_PREFIX) || (Op::kHasFlag && f);
    const unsigned stop_mask = __ballot_sync(kFull, stop);
    const int p = stop_mask ? (__ffs(stop_mask) - 1) : 32;   // nearest stopping lane
    if (lane > p) { v = 0; f = 0; }
    // ordered fold: lane l holds array position j-l, so the LEFT operand comes from
    // the higher lane.
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      uint32_t ov = __shfl_down_sync(kFull, v, o);
      uint32_t of = __shfl_down_sync(kFull, f, o);
      if (lane + o < 32) Op::combine(ov, of, v, f, v, f);
    }
    v = __shfl_sync(kFull, v, 0);
    f = __shfl_sync(kFull, f, 0);
    if (have_acc) Op::combine(v, f, acc_v, acc_f, acc_v, acc_f);
    else { acc_v = v; acc_f = f; have_acc = true; }
    if (p < 32) break;
    j -= 32;
  }
  ev = acc_v; ef = acc_f;
  if (!self_contained && lane == 0) {
    uint32_t iv, iflag;
    Op::combine(ev, ef, agg_v, agg_f, iv, iflag);
    st_status(&status[tile], pack_status(iv, epoch, iflag, ST_PREFIX));
  }
  return true;
}

__device__ __forceinline__ bool aligned16(const void *p) { return (((uintptr_t)p) & 15u) == 0; }

// ---- inclusive scan (+) over i32 -------------------------------------------------------
__global__ void __launch_bounds__(SCAN_THREADS)
scan_i32_kernel(const int32_t *__restrict__ in, int32_t *__restrict__ out, int64_t n, uint32_t num_tiles,
                uint32_t *ticket, uint64_t *status, uint32_t epoch, int *failure, uint32_t carry_in,
                const uint32_t *__restrict__ carry_vals, int carry_n) {
  __shared__ __align__(128) uint32_t s_tile[SCAN_TILE];
  __shared__ __align__(8) uint64_t s_bar;
  __shared__ uint32_t s_warp[SCAN_WARPS];
  __shared__ uint32_t s_slot, s_prefix, s_ok;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (ld_failure(failure) != FAIL_NONE) return;

  if (tid == 0) { mbar_init(&s_bar, 1); fence_mbar_init(); }
  const uint32_t tile = draw_tile(ticket, num_tiles, &s_slot);   // contains __syncthreads
  const int64_t base = (int64_t)tile * SCAN_TILE;
  const int count = (int)((n - base) < SCAN_TILE ? (n - base) : SCAN_TILE);
  const bool bulk = (count == SCAN_TILE) && aligned16(in + base) && aligned16(out + base);

  if (bulk) {
    if (tid == 0) {
      mbar_expect_tx(&s_bar, SCAN_TILE * 4);
      bulk_g2s(s_tile, in + base, SCAN_TILE * 4, &s_bar);
    }
    if (!mbar_wait_bounded(&s_bar, 0)) {
      atomicCAS(failure, FAIL_NONE, FAIL_BULK_COPY_TIMEOUT);
      return;   // every thread of the CTA sees the same outcome of the same barrier phase
    }
  } else {
    for (int i = tid; i < SCAN_TILE; i += SCAN_THREADS)
      s_tile[i] = (i < count) ? (uint32_t)in[base + i] : 0u;
    __syncthreads();
  }

  uint32_t x[SCAN_ITEMS];
  {
    const int4 *src = reinterpret_cast<const int4 *>(s_tile) + tid * (SCAN_ITEMS / 4);
#pragma unroll
    for (int j = 0; j < SCAN_ITEMS / 4; j++) {
      int4 v = src[j];
      x[4 * j + 0] = v.x; x[4 * j + 1] = v.y; x[4 * j + 2] = v.z; x[4 * j + 3] = v.w;
    }
  }
  uint32_t sum = 0;
#pragma unroll
  for (int k = 0; k < SCAN_ITEMS; k++) { sum += x[k]; x[k] = sum; }   // x = in-thread inclusive scan

  const uint32_t incl = warp_incl_scan_add(sum, lane);
  if (lane == 31) s_warp[warp] = incl;
  __syncthreads();
  uint32_t warp_excl = 0, tile_agg = 0;
#pragma unroll
  for (int w = 0; w < SCAN_WARPS; w++) {
    uint32_t t = s_warp[w];
    if (w < warp) warp_excl += t;
    tile_agg += t;
  }
  const uint32_t thread_excl = warp_excl + incl - sum;

  if (warp == 0) {
    uint32_t ev, ef;
    // carry of a sharded scan: the totals of the shards before this one, summed here
    if (carry_vals != nullptr && tile < 32u)
      for (int q = 0; q < carry_n; q++) carry_in += carry_vals[q];
    bool ok = tile_lookback<OpAddU32>(status, tile, epoch, tile_agg, 0u, carry_in, failure, ev, ef);
    if (lane == 0) { s_prefix = ev; s_ok = ok ? 1u : 0u; }
  }
  __syncthreads();
  if (!s_ok) return;
  const uint32_t start = s_prefix + thread_excl;

  {
    int4 *dst = reinterpret_cast<int4 *>(s_tile) + tid * (SCAN_ITEMS / 4);
#pragma unroll
    for (int j = 0; j < SCAN_ITEMS / 4; j++) {
      int4 v;
      v.x = start + x[4 * j + 0]; v.y = start + x[4 * j + 1];
      v.z = start + x[4 * j + 2]; v.w = start + x[4 * j + 3];
      dst[j] = v;
    }
  }
  if (bulk) {
    fence_proxy_async_smem();
    __syncthreads();
    if (tid == 0) {
      bulk_s2g(out + base, s_tile, SCAN_TILE * 4);
      bulk_commit();
      bulk_wait_read0();
    }
  } else {
    __syncthreads();
    for (int i = tid; i < count; i += SCAN_THREADS) out[base + i] = (int32_t)s_tile[i];
  }
}

// ---- flagged segmented inclusive scan (+) over f32 -----------------------------------------
__global__ void __launch_bounds__(SCAN_THREADS)
segscan_f32_kernel(const uint8_t *__restrict__ flags, const float *__restrict__ in, float *__restrict__ out,
                   int64_t n, uint32_t num_tiles, uint32_t *ticket, uint64_t *status, uint32_t epoch,
                   int *failure, float carry_in) {
  __shared__ __align__(128) float s_tile[SCAN_TILE];
  __shared__ __align__(128) uint32_t s_flag[SCAN_TILE / 4];
  __shared__ __align__(8) uint64_t s_bar;
  __shared__ uint32_t s_wv[SCAN_WARPS], s_wf[SCAN_WARPS];
  __shared__ uint32_t s_slot, s_pv, s_pf, s_ok;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (ld_failure(failure) != FAIL_NONE) return;

  if (tid == 0) { mbar_init(&s_bar, 1); fence_mbar_init(); }
  const uint32_t tile = draw_tile(ticket, num_tiles, &s_slot);
  const int64_t base = (int64_t)tile * SCAN_TILE;
  const int count = (int)((n - base) < SCAN_TILE ? (n - base) : SCAN_TILE);
  const bool bulk = (count == SCAN_TILE) && aligned16(in + base) && aligned16(out + base) &&
                    aligned16(flags + base);

  if (bulk) {
    if (tid == 0) {
      mbar_expect_tx(&s_bar, SCAN_TILE * 4 + SCAN_TILE);
      bulk_g2s(s_tile, in + base, SCAN_TILE * 4, &s_bar);
      bulk_g2s(s_flag, flags + base, SCAN_TILE, &s_bar);
    }
    if (!mbar_wait_bounded(&s_bar, 0)) {
      atomicCAS(failure, FAIL_NONE, FAIL_BULK_COPY_TIMEOUT);
      return;
    }
  } else {
    uint8_t *sf = reinterpret_cast<uint8_t *>(s_flag);
    for (int i = tid; i < SCAN_TILE; i += SCAN_THREADS) {
      s_tile[i] = (i < count) ? in[base + i] : 0.0f;
      sf[i] = (i < count) ? flags[base + i] : (uint8_t)0;
    }
    __syncthreads();
  }

  float x[SCAN_ITEMS];
  uint32_t fw[SCAN_ITEMS / 4];
  {
    const float4 *src = reinterpret_cast<const float4 *>(s_tile) + tid * (SCAN_ITEMS / 4);
#pragma unroll
    for (int j = 0; j < SCAN_ITEMS / 4; j++) {
      float4 v = src[j];
      x[4 * j + 0] = v.x; x[4 * j + 1] = v.y; x[4 * j + 2] = v.z; x[4 * j + 3] = v.w;
      fw[j] = s_flag[tid * (SCAN_ITEMS / 4) + j];
    }
  }
  // in-thread lifted scan: x[k] becomes the inclusive value relative to the thread
  // start; fbits marks, per element, whether a segment start lies at or before it.
  uint32_t fbits = 0;       // bit k: element k is a segment start
  float acc = 0.0f;
  uint32_t seen = 0;
#pragma unroll
  for (int k = 0; k < SCAN_ITEMS; k++) {
    const uint32_t fl = (fw[k >> 2] >> (8 * (k & 3))) & 0xffu;
    if (fl) { acc = x[k]; seen = 1; fbits |= (1u << k); }
    else acc = acc + x[k];
    x[k] = acc;
  }
  // warp inclusive scan of (acc, seen) pairs
  uint32_t pv = __float_as_uint(acc), pf = seen;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    uint32_t lv = __shfl_up_sync(kFull, pv, o);
    uint32_t lf = __shfl_up_sync(kFull, pf, o);
    if (lane >= o) OpSegAddF32::combine(lv, lf, pv, pf, pv, pf);
  }
  if (lane == 31) { s_wv[warp] = pv; s_wf[warp] = pf; }
  // exclusive within the warp
  uint32_t xv = __shfl_up_sync(kFull, pv, 1), xf = __shfl_up_sync(kFull, pf, 1);
  if (lane == 0) { xv = 0; xf = 0; }
  __syncthreads();
  uint32_t wv = 0, wf = 0, tv = 0, tf = 0;     // exclusive prefix of this warp; tile aggregate
#pragma unroll
  for (int w = 0; w < SCAN_WARPS; w++) {
    if (w == warp) { wv = tv; wf = tf; }
    OpSegAddF32::combine(tv, tf, s_wv[w], s_wf[w], tv, tf);
  }
  uint32_t thv, thf;                           // exclusive prefix of this thread within the tile
  OpSegAddF32::combine(wv, wf, xv, xf, thv, thf);

  if (warp == 0) {
    uint32_t ev, ef;
    bool ok = tile_lookback<OpSegAddF32>(status, tile, epoch, tv, tf, __float_as_uint(carry_in), failure, ev, ef);
    if (lane == 0) { s_pv = ev; s_pf = ef; s_ok = ok ? 1u : 0u; }
  }
  __syncthreads();
  if (!s_ok) return;
  uint32_t sv, sf2;
  OpSegAddF32::combine(s_pv, s_pf, thv, thf, sv, sf2);
  const float start = __uint_as_float(sv);

  {
    // elements before the thread's first segment start receive the incoming prefix
    const uint32_t first = fbits ? (uint32_t)(__ffs(fbits) - 1) : (uint32_t)SCAN_ITEMS;
    float4 *dst = reinterpret_cast<float4 *>(s_tile) + tid * (SCAN_ITEMS / 4);
#pragma unroll
    for (int j = 0; j < SCAN_ITEMS / 4; j++) {
      float4 v;
      v.x = (4 * j + 0 < first) ? start + x[4 * j + 0] : x[4 * j + 0];
      v.y = (4 * j + 1 < first) ? start + x[4 * j + 1] : x[4 * j + 1];
      v.z = (4 * j + 2 < first) ? start + x[4 * j + 2] : x[4 * j + 2];
      v.w = (4 * j + 3 < first) ? start + x[4 * j + 3] : x[4 * j + 3];
      dst[j] = v;
    }
  }
  if (bulk) {
    fence_proxy_async_smem();
    __syncthreads();
    if (tid == 0) {
      bulk_s2g(out + base, s_tile, SCAN_TILE * 4);
      bulk_commit();
      bulk_wait_read0();
    }
  } else {
    __syncthreads();
    for (int i = tid; i < count; i += SCAN_THREADS) out[base + i] = s_tile[i];
  }
}

// ---- filter / partition of u32 keys by the predicate (k & 7) < 3 ------------------------------
// out_true receives the selected keys at their stable rank; when PARTITION, out_false
// receives the rejected keys at theirs.  d_count[0] = number of selected keys.
template <bool PARTITION>
__global__ void __launch_bounds__(SCAN_THREADS)
compact_u32_kernel(const uint32_t *__restrict__ in, uint32_t *__restrict__ out_true,
                   uint32_t *__restrict__ out_false, int64_t n, uint32_t num_tiles, uint32_t *ticket,
                   uint64_t *status, uint32_t epoch, int *failure, int64_t *d_count) {
  __shared__ __align__(128) uint32_t s_tile[SCAN_TILE];
  __shared__ __align__(8) uint64_t s_bar;
  __shared__ uint32_t s_warp[SCAN_WARPS];
  __shared__ uint32_t s_slot, s_prefix, s_ok;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (ld_failure(failure) != FAIL_NONE) return;

  if (tid == 0) { mbar_init(&s_bar, 1); fence_mbar_init(); }
  const uint32_t tile = draw_tile(ticket, num_tiles, &s_slot);
  const int64_t base = (int64_t)tile * SCAN_TILE;
  const int count = (int)((n - base) < SCAN_TILE ? (n - base) : SCAN_TILE);
  const bool bulk = (count == SCAN_TILE) && aligned16(in + base);

  if (bulk) {
    if (tid == 0) {
      mbar_expect_tx(&s_bar, SCAN_TILE * 4);
      bulk_g2s(s_tile, in + base, SCAN_TILE * 4, &s_bar);
    }
    if (!mbar_wait_bounded(&s_bar, 0)) {
      atomicCAS(failure, FAIL_NONE, FAIL_BULK_COPY_TIMEOUT);
      return;
    }
  } else {
    for (int i = tid; i < SCAN_TILE; i += SCAN_THREADS) s_tile[i] = (i < count) ? in[base + i] : 0u;
    __syncthreads();
  }

  uint32_t x[SCAN_ITEMS];
  {
    const int4 *src = reinterpret_cast<const int4 *>(s_tile) + tid * (SCAN_ITEMS / 4);
#pragma unroll
    for (int j = 0; j < SCAN_ITEMS / 4; j++) {
      int4 v = src[j];
      x[4 * j + 0] = v.x; x[4 * j + 1] = v.y; x[4 * j + 2] = v.z; x[4 * j + 3] = v.w;
    }
  }
  const int first = tid * SCAN_ITEMS;                 // local index of the thread's first key
  uint32_t sel = 0;                                   // bit k: key k is selected
#pragma unroll
  for (int k = 0; k < SCAN_ITEMS; k++)
    if ((first + k < count) && ((x[k] & 7u) < 3u)) sel |= (1u << k);
  const uint32_t cnt = __popc(sel);

  const uint32_t incl = warp_incl_scan_add(cnt, lane);
  if (lane == 31) s_warp[warp] = incl;
  __syncthreads();                                    // also: every thread has its keys in registers
  uint32_t warp_excl = 0, tile_true = 0;
#pragma unroll
  for (int w = 0; w < SCAN_WARPS; w++) {
    uint32_t t = s_warp[w];
    if (w < warp) warp_excl += t;
    tile_true += t;
  }
  const uint32_t thread_excl = warp_excl + incl - cnt;

  if (warp == 0) {
    uint32_t ev, ef;
    bool ok = tile_lookback<OpAddU32>(status, tile, epoch, tile_true, 0u, 0u, failure, ev, ef);
    if (lane == 0) { s_prefix = ev; s_ok = ok ? 1u : 0u; }
  }

  // compact inside shared memory: selected keys first, in order; then the rejected
  {
    uint32_t t_pos = thread_excl;
    const int valid_before = first < count ? first : count;
    uint32_t f_pos = tile_true + (uint32_t)valid_before - thread_excl;
#pragma unroll
    for (int k = 0; k < SCAN_ITEMS; k++) {
      if (sel & (1u << k)) s_tile[t_pos++] = x[k];
      else if (PARTITION && (first + k < count)) s_tile[f_pos++] = x[k];
    }
  }
  __syncthreads();
  if (!s_ok) return;
  const int64_t true_before = (int64_t)s_prefix;      // selected keys in earlier tiles
  {
    uint32_t *dst = out_true + true_before;
    for (uint32_t i = tid; i < tile_true; i += SCAN_THREADS) dst[i] = s_tile[i];
  }
  if (PARTITION) {
    uint32_t *dst = out_false + (base - true_before);
    const uint32_t nf = (uint32_t)count - tile_true;
    for (uint32_t i = tid; i < nf; i += SCAN_THREADS) dst[i] = s_tile[tile_true + i];
  }
  if (tile == num_tiles - 1 && tid == 0) *d_count = true_before + (int64_t)tile_true;
}

// ---- host launchers --------------------------------------------------------------------

static inline uint32_t tiles_for(int64_t n) { return (uint32_t)((n + SCAN_TILE - 1) / SCAN_TILE); }

size_t lookback_scratch_bytes(int64_t n) {
  return 256 + (size_t)tiles_for(n) * sizeof(uint64_t);
}

static inline void split_scratch(void *scratch, uint32_t **ticket, uint64_t **status) {
  *ticket = reinterpret_cast<uint32_t *>(scratch);
  *status = reinterpret_cast<uint64_t *>(reinterpret_cast<char *>(scratch) + 256);
}

cudaError_t launch_scan_i32(const int32_t *in, int32_t *out, int64_t n, int32_t carry_in,
                            const int32_t *carry_vals, int carry_n, void *scratch,
                            uint32_t epoch, int *failure, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  uint32_t *ticket; uint64_t *status;
  split_scratch(scratch, &ticket, &status);
  const uint32_t nt = tiles_for(n);
  scan_i32_kernel<<<nt, SCAN_THREADS, 0, stream>>>(in, out, n, nt, ticket, status, epoch, failure,
                                                   (uint32_t)carry_in, reinterpret_cast<const uint32_t *>(carry_vals),
                                                   carry_n);
  return cudaGetLastError();
}

cudaError_t launch_segscan_f32(const uint8_t *flags, const float *in, float *out, int64_t n, float carry_in,
                               void *scratch, uint32_t epoch, int *failure, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  uint32_t *ticket; uint64_t *status;
  split_scratch(scratch, &ticket, &status);
  const uint32_t nt = tiles_for(n);
  segscan_f32_kernel<<<nt, SCAN_THREADS, 0, stream>>>(flags, in, out, n, nt, ticket, status, epoch, failure,
                                                      carry_in);
  return cudaGetLastError();
}

// ---- pieces of a segmented scan whose array is split across several devices ---------------
// Summary of a shard = inclusive prefix of its last tile: (value, "a segment starts somewhere
// in the shard").  Written as two 32-bit words {f32 bits, flag}.
__global__ void segscan_summary_kernel(const uint64_t *status, uint32_t last_tile, uint32_t *dst) {
  const uint64_t w = status[last_tile];
  dst[0] = status_value(w);
  dst[1] = status_flag(w);
}

// Position of the first segment start (n if none): CTAs walk 16 KiB chunks in ascending
// order and stop as soon as a start before their chunk is known.
__global__ void __launch_bounds__(256)
first_flag_kernel(const uint8_t *__restrict__ flags, int64_t n, unsigned long long *first) {
  constexpr int64_t CHUNK = 16384;
  for (int64_t c = blockIdx.x; c * CHUNK < n; c += gridDim.x) {
    const int64_t lo = c * CHUNK;
    if ((int64_t)*reinterpret_cast<volatile unsigned long long *>(first) < lo) return;
    const int64_t hi = lo + CHUNK < n ? lo + CHUNK : n;
    int64_t best = n;
    for (int64_t i = lo + threadIdx.x; i < hi; i += 256)
      if (flags[i]) { best = i; break; }
    if (best < n) atomicMin(first, (unsigned long long)best);
  }
}

// out[i] += carry for i before the first segment start, where carry is the fold of the
// summaries of the shards before this one under the lifted operator.
__global__ void __launch_bounds__(256)
apply_carry_kernel(float *__restrict__ out, const unsigned long long *first, const uint32_t *summaries, int rank) {
  uint32_t cv = 0, cf = 0;
  for (int q = 0; q < rank; q++) OpSegAddF32::combine(cv, cf, summaries[2 * q], summaries[2 * q + 1], cv, cf);
  const float carry = __uint_as_float(cv);
  const int64_t end = (int64_t)*first;
  const int64_t stride = (int64_t)gridDim.x * 256;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < end; i += stride) out[i] = carry + out[i];
}

cudaError_t launch_segscan_summary(void *scratch, int64_t n, uint32_t *dst, cudaStream_t stream) {
  if (n <= 0) return cudaMemsetAsync(dst, 0, 8, stream);   // (0, no flag): the identity
  uint32_t *ticket; uint64_t *status;
  split_scratch(scratch, &ticket, &status);
  segscan_summary_kernel<<<1, 1, 0, stream>>>(status, tiles_for(n) - 1, dst);
  return cudaGetLastError();
}

cudaError_t launch_segscan_apply_carry(float *out, const uint8_t *flags, int64_t n, const uint32_t *summaries,
                                       int rank, unsigned long long *d_first, int num_sms, cudaStream_t stream) {
  if (n <= 0 || rank <= 0) return cudaSuccess;
  const unsigned long long init = (unsigned long long)n;
  cudaError_t err = cudaMemcpyAsync(d_first, &init, sizeof(init), cudaMemcpyHostToDevice, stream);
  if (err != cudaSuccess) return err;
  int64_t chunks = (n + 16383) / 16384;
  int grid = (int)(chunks < (int64_t)num_sms * 4 ? chunks : (int64_t)num_sms * 4);
  first_flag_kernel<<<grid, 256, 0, stream>>>(flags, n, d_first);
  apply_carry_kernel<<<num_sms * 4, 256, 0, stream>>>(out, d_first, summaries, rank);
  return cudaGetLastError();
}

cudaError_t launch_compact_u32(bool partition, const uint32_t *in, uint32_t *out_true, uint32_t *out_false,
                               int64_t n, int64_t *d_count, void *scratch, uint32_t epoch, int *failure,
                               cudaStream_t stream) {
  if (n <= 0) return cudaMemsetAsync(d_count, 0, sizeof(int64_t), stream);
  uint32_t *ticket; uint64_t *status;
  split_scratch(scratch, &ticket, &status);
  const uint32_t nt = tiles_for(n);
  if (partition)
    compact_u32_kernel<true><<<nt, SCAN_THREADS, 0, stream>>>(in, out_true, out_false, n, nt, ticket, status,
                                                              epoch, failure, d_count);
  else
    compact_u32_kernel<false><<<nt, SCAN_THREADS, 0, stream>>>(in, out_true, out_false, n, nt, ticket, status,
                                                               epoch, failure, d_count);
  return cudaGetLastError();
}

// ---- scan (+) i32 without any allocation ---------------------------------------------------------
// Some hosts hand this library a GPU whose memory is already fully parcelled out by their
// own arena allocator, or run it inside a region of their program where a call that may
// synchronise the whole device or fail for lack of memory (cudaMalloc does both) is not
// acceptable, for instance a latency-bound service loop after start-up.  For them the tile
// ticket, the tile status words and the failure word of the look-back scan live in the
// fixed array below instead of in pooled memory.  The array is part of the loaded library
// image: every GPU that loads the library holds these ~103 KiB until the process exits.
constexpr int64_t NOALLOC_MAX_N = (int64_t)1 << 26;
constexpr uint32_t NOALLOC_MAX_TILES = (uint32_t)((NOALLOC_MAX_N + SCAN_TILE - 1) / SCAN_TILE);
constexpr size_t NOALLOC_HEAD = 512;     // [0,4) ticket, [256,260) failure word
constexpr size_t NOALLOC_BYTES = NOALLOC_HEAD + (size_t)NOALLOC_MAX_TILES * sizeof(uint64_t);
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_BYTES];

// In host code `g_noalloc_scratch` names a host-side shadow of the array, not device
// memory; the device address is asked for once per device, with that device current.
constexpr int NOALLOC_MAX_DEVICES = 64;
static std::mutex g_noalloc_lock;
static unsigned char *g_noalloc_ptr[NOALLOC_MAX_DEVICES];
static uint32_t g_noalloc_epoch[NOALLOC_MAX_DEVICES];

}  // namespace fb

extern "C" int futhark_b200_scan_i32_noalloc(const int32_t *in, int32_t *out, int64_t n, void *stream,
                                             int32_t *status_dev, char *errbuf, size_t errbuf_len) {
  using namespace fb;
  auto fail = [&](int code, const char *msg, const char *detail) {
    if (errbuf != nullptr && errbuf_len > 0) snprintf(errbuf, errbuf_len, "%s%s%s", msg, detail ? ": " : "", detail ? detail : "");
    return code;
  };
  if (n < 0) return fail(1, "futhark_b200_scan_i32_noalloc: negative length", nullptr);
  if (n > NOALLOC_MAX_N) {
    char d[96];
    snprintf(d, sizeof(d), "%lld elements requested, at most %lld fit the fixed scratch array", (long long)n, (long long)NOALLOC_MAX_N);
    return fail(1, "futhark_b200_scan_i32_noalloc: input too long", d);
  }
  int dev = -1;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return fail(1, "futhark_b200_scan_i32_noalloc: cudaGetDevice", cudaGetErrorString(err));
  if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) return fail(1, "futhark_b200_scan_i32_noalloc: device ordinal out of range", nullptr);
  unsigned char *base;
  uint32_t epoch;
  {
    std::lock_guard<std::mutex> g(g_noalloc_lock);
    if (g_noalloc_ptr[dev] == nullptr) {           // first call on this device: set-up
      void *p = nullptr;
      err = cudaGetSymbolAddress(&p, g_noalloc_scratch);
      if (err != cudaSuccess) return fail(1, "futhark_b200_scan_i32_noalloc: cudaGetSymbolAddress", cudaGetErrorString(err));
      g_noalloc_ptr[dev] = static_cast<unsigned char *>(p);
    }
    base = g_noalloc_ptr[dev];
    g_noalloc_epoch[dev] = (g_noalloc_epoch[dev] % ((1u << 29) - 1)) + 1;
    epoch = g_noalloc_epoch[dev];
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // The array keeps what the previous call left: the ticket and the failure word must start
  // at zero (an aborted call may have left either set); status words need no clearing, the
  // epoch tells this call's words from older ones.
  err = cudaMemsetAsync(base, 0, NOALLOC_HEAD, st);
  if (err != cudaSuccess) return fail(1, "futhark_b200_scan_i32_noalloc: cudaMemsetAsync", cudaGetErrorString(err));
  int *failure = reinterpret_cast<int *>(base + 256);
  if (n > 0) {
    const uint32_t nt = (uint32_t)((n + SCAN_TILE - 1) / SCAN_TILE);
    scan_i32_kernel<<<nt, SCAN_THREADS, 0, st>>>(in, out, n, nt, reinterpret_cast<uint32_t *>(base),
                                                 reinterpret_cast<uint64_t *>(base + NOALLOC_HEAD), epoch, failure, 0u, nullptr, 0);
    err = cudaGetLastError();
    if (err != cudaSuccess) return fail(1, "futhark_b200_scan_i32_noalloc: kernel launch", cudaGetErrorString(err));
  }
  if (status_dev != nullptr) {
    err = cudaMemcpyAsync(status_dev, failure, sizeof(int32_t), cudaMemcpyDeviceToDevice, st);
    if (err != cudaSuccess) return fail(1, "futhark_b200_scan_i32_noalloc: status copy", cudaGetErrorString(err));
  }
  return 0;
}

namespace fb {
}  // namespace fb
