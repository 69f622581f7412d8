// Single-pass decoupled look-back kernels: inclusive scan (+) over i32, flagged
// segmented inclusive scan (+) over f32, and filter / partition compaction of u32
// keys.  They replace the generated `segscan` kernel of the reference
// (src/Futhark/CodeGen/ImpGen/GPU/SegScan/SinglePass.hs:327-879) and, for
// compaction, the scan + scatter that prelude/soacs.fut:241-286 expands into.
//
// One persistent kernel, templated on what a tile computes.  Tiles hold 512 x 20 = 10240
// elements; every CTA owns two shared-memory stages, so the bulk load of its next tile is
// in flight while the current tile is processed:
//   1. thread 0 draws tile numbers from a ticket counter, so tile i starts only after
//      every tile < i has started -- the property that makes waiting on predecessors safe
//      (the reference draws its `dyn_id` the same way, :444-461).  A CTA draws the ticket
//      of its NEXT tile when it starts working on the current one, so the tiles being
//      worked on across the GPU at any moment are (nearly) consecutive;
//   2. a tile comes into shared memory with ONE bulk async copy (TMA) per array, awaited on
//      an mbarrier; a thread then owns 20 CONSECUTIVE elements = 5 x 16 bytes, a stride of
//      5 sixteen-byte units, which is odd, so the 128-bit shared-memory accesses are
//      bank-conflict free without padding;
//   3. per-thread sequential scan, warp-shuffle scan of thread totals, a second shuffle
//      scan over the 16 warp totals;
//   4. warp 0 publishes the tile aggregate and looks back over its predecessors, 128
//      status words per round trip (4 per lane); it waits only for the predecessors it
//      needs (up to the nearest one with a known prefix); every wait is bounded and polls
//      the failure word;
//   5. results go back into the stage and leave with one bulk async store (scan), or are
//      compacted in the stage and written as contiguous runs (compaction).
// A tile that is ragged (the last one) or whose global addresses are not 16-byte
// aligned uses plain guarded loads and stores instead of the bulk copies.
//
// Why tiles are this large and the look-back this wide: a tile at distance d from the
// nearest known prefix needs ceil(d / window) dependent L2 round trips, so the GPU as a
// whole cannot retire more than about window / round-trip tiles per unit time; at HBM
// speed that bound has to stay well above the tile rate.
#include <stdio.h>
#include <string.h>

#include <mutex>

#include "../../include/futhark_b200.h"
#include "common.cuh"
#include "kernels.h"

namespace fb {

constexpr int SCAN_THREADS = 512;
constexpr int SCAN_ITEMS = 20;
constexpr int SCAN_TILE = SCAN_THREADS * SCAN_ITEMS;  // 10240 elements
constexpr int SCAN_WARPS = SCAN_THREADS / 32;         // 16
constexpr int LB_PER_LANE = 8;                        // status words per lane per round
constexpr int LB_WINDOW = 32 * LB_PER_LANE;
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

// ---- look-back (warp 0 only, all 32 lanes) ---------------------------------------
// Publishes this tile's aggregate (or, when the tile's own prefix does not depend on
// its predecessors, its inclusive prefix), then combines predecessors from the
// nearest one backwards until one with a known inclusive prefix (or, for the
// segmented operator, one containing a segment start) is met.  Lane l looks at the
// predecessors j-8l .. j-8l-7 of each window.  Returns the exclusive prefix of the tile
// in (ev, ef) -- valid in every lane -- or false after a timeout.
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
  int64_t j = (int64_t)tile - 1;        // nearest predecessor of the current window
  uint32_t rounds = 0;
  // Waiting is done by ONE lane on ONE word (the nearest entry still missing): hundreds of
  // warps re-reading whole windows of the same few cache lines would saturate the L2
  // slice that holds them and delay the very stores they are waiting for.
  int64_t wait_idx = j;
  while (true) {
    // ---- wait until status[wait_idx] holds something (bounded)
    {
      uint32_t st = ST_PREFIX;
      while (true) {
        if (lane == 0 && wait_idx >= 0) st = status_state(ld_status(&status[wait_idx]), epoch);
        st = __shfl_sync(kFull, st, 0);
        if (st != ST_NONE) break;
        rounds++;
        if ((rounds & 63u) == 0) {
          int fl = (lane == 0) ? ld_failure(failure) : 0;
          fl = __shfl_sync(kFull, fl, 0);
          if (fl != FAIL_NONE) return false;
          if (rounds >= LOOKBACK_MAX_ROUNDS) {
            if (lane == 0) atomicCAS(failure, FAIL_NONE, FAIL_LOOKBACK_TIMEOUT);
            return false;
          }
        }
        __nanosleep(rounds < 8 ? 20 : (rounds < 64 ? 100 : 400));
      }
    }
    // ---- one wide read of the window: lane l takes the predecessors j-8l .. j-8l-7
    uint32_t v = 0, f = 0;              // this lane's ordered partial
    uint64_t w_q[LB_PER_LANE];
    const int64_t lane_first = j - (int64_t)(LB_PER_LANE * lane);
#pragma unroll
    for (int q = 0; q < LB_PER_LANE; q++) {
      const int64_t idx = lane_first - q;
      if (idx >= 0) w_q[q] = ld_status(&status[idx]);
      else           // before the array: virtual tile -1 carries the seed, the rest are identities
        w_q[q] = pack_status((idx == -1) ? carry_v : 0u, epoch, 0u, ST_PREFIX);
    }
    // nearest-first walk over the lane's entries
    bool lane_ready = true, lane_stop = false;
    int qend = LB_PER_LANE - 1, qhole = 0;
#pragma unroll
    for (int q = 0; q < LB_PER_LANE; q++) {
      if (lane_ready && !lane_stop) {
        const uint32_t st = status_state(w_q[q], epoch);
        if (st == ST_NONE) { lane_ready = false; qhole = q; }
        else if (st == ST_PREFIX || (Op::kHasFlag && status_flag(w_q[q]))) { lane_stop = true; qend = q; }
      }
    }
    const unsigned stop_mask = __ballot_sync(kFull, lane_ready && lane_stop);
    const unsigned not_ready = ~__ballot_sync(kFull, lane_ready);
    const int first_bad = not_ready ? (__ffs(not_ready) - 1) : 32;   // nearest lane with a hole
    const int p = stop_mask ? (__ffs(stop_mask) - 1) : 32;           // nearest lane with a stop
    if (first_bad < 32 && first_bad < p) {
      // a hole lies before any stop: wait for exactly that entry, then read the window again
      const int hole_q = __shfl_sync(kFull, qhole, first_bad);
      wait_idx = j - (int64_t)(LB_PER_LANE * first_bad + hole_q);
      continue;
    }
    {
      // ordered fold of this lane's entries: farther (higher q) on the left
      bool started = false;
#pragma unroll
      for (int q = LB_PER_LANE - 1; q >= 0; q--) {
        if (q <= qend) {
          const uint32_t qv = status_value(w_q[q]), qf = Op::kHasFlag ? status_flag(w_q[q]) : 0u;
          if (!started) { v = qv; f = qf; started = true; }
          else Op::combine(v, f, qv, qf, v, f);
        }
      }
    }
    if (lane > p) { v = 0; f = 0; }
    // ordered fold across lanes: lane l holds positions nearer than lane l+1, so the LEFT
    // operand comes from the higher lane.
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
    j -= LB_WINDOW;
    wait_idx = j;
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

// ---- the persistent look-back kernel -------------------------------------------------------------
// Progress: tickets are drawn in increasing order and a CTA processes its tiles in the
// order it drew them, so the smallest unfinished tile is always some CTA's current tile and
// waits only on finished ones.  The grid never exceeds what is resident at once.
#ifdef FB_TRACE
__device__ unsigned long long g_trace[32768 * 8];
__device__ __forceinline__ unsigned long long gtime() { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }
#define TRACE(slot) do { if (tid == 0 && tile < 32768u) g_trace[tile * 8 + (slot)] = gtime(); } while (0)
#define TRACEV(slot, val) do { if (tid == 0 && tile < 32768u) g_trace[tile * 8 + (slot)] = (val); } while (0)
#else
#define TRACE(slot) do {} while (0)
#define TRACEV(slot, val) do {} while (0)
#endif

enum ScanKind : int { K_SCAN_I32 = 0, K_SEGSCAN_F32 = 1, K_FILTER = 2, K_PARTITION = 3 };
constexpr int NSTAGE = 2;

template <int KIND> struct StageBytes { static constexpr int value = SCAN_TILE * 4; };
template <> struct StageBytes<K_SEGSCAN_F32> { static constexpr int value = SCAN_TILE * 4 + SCAN_TILE; };

struct LookbackArgs {
  const void *in;          // values / keys
  const uint8_t *flags;    // segmented scan only
  void *out;               // scan result, or the selected keys
  uint32_t *out_false;     // partition: the rejected keys
  int64_t n;
  uint32_t num_tiles;
  uint32_t *ticket;
  uint64_t *status;
  uint32_t epoch;
  int *failure;
  uint32_t carry_in;       // value bits of the seed (0 for compaction)
  const uint32_t *carry_vals;
  int carry_n;
  int64_t *d_count;        // compaction: number of selected keys
};

template <int KIND>
__global__ void __launch_bounds__(SCAN_THREADS, 2)
lookback_kernel(const LookbackArgs a) {
  constexpr int SB = StageBytes<KIND>::value;
  extern __shared__ __align__(128) unsigned char s_stages[];
  __shared__ __align__(8) uint64_t s_bar[NSTAGE];
  __shared__ uint32_t s_tid[NSTAGE];
  __shared__ uint32_t s_wv[SCAN_WARPS], s_wf[SCAN_WARPS];
  __shared__ uint32_t s_pv, s_pf, s_ok;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (ld_failure(a.failure) != FAIL_NONE) return;
  const uint32_t nt = a.num_tiles;
  // every CTA draws one ticket up front, one per tile it works on, and stops at its first
  // invalid ticket: nt valid draws + gridDim.x invalid ones in total
  const uint32_t last_draw = nt + gridDim.x - 1;
  const bool ptr_aligned = aligned16(a.in) && (KIND == K_FILTER || KIND == K_PARTITION || aligned16(a.out)) &&
                           (KIND != K_SEGSCAN_F32 || aligned16(a.flags));

  auto tile_is_bulk = [&](uint32_t t) -> bool {
    return ptr_aligned && ((int64_t)(t + 1) * SCAN_TILE <= a.n);
  };
  auto issue_load = [&](int s, uint32_t t) {   // one thread
    unsigned char *st = s_stages + s * SB;
    const int64_t base = (int64_t)t * SCAN_TILE;
    mbar_expect_tx(&s_bar[s], SB);
    bulk_g2s(st, reinterpret_cast<const uint32_t *>(a.in) + base, SCAN_TILE * 4, &s_bar[s]);
    if (KIND == K_SEGSCAN_F32) bulk_g2s(st + SCAN_TILE * 4, a.flags + base, SCAN_TILE, &s_bar[s]);
  };
  auto draw_and_load = [&](int s) {             // one thread
    uint32_t t = atomicAdd(a.ticket, 1u);
    if (t == last_draw) atomicExch(a.ticket, 0u);     // rewind for the next launch
    s_tid[s] = t;
    if (t < nt && tile_is_bulk(t)) issue_load(s, t);
  };

  if (tid == 0) {
    for (int s = 0; s < NSTAGE; s++) mbar_init(&s_bar[s], 1);
    fence_mbar_init();
    draw_and_load(0);
  }
  __syncthreads();

  uint32_t phases = 0;     // bit s: parity of stage s's next barrier completion
  for (uint32_t k = 0;; k++) {
    const int s = k % NSTAGE;
    const uint32_t tile = s_tid[s];
    if (tile >= nt) break;
    TRACE(0);
    TRACE(1);

    unsigned char *stage = s_stages + s * SB;
    uint32_t *s_tile = reinterpret_cast<uint32_t *>(stage);
    const int64_t base = (int64_t)tile * SCAN_TILE;
    const int count = (int)((a.n - base) < SCAN_TILE ? (a.n - base) : SCAN_TILE);
    const bool bulk = tile_is_bulk(tile);

    if (bulk) {
      const bool arrived = mbar_wait_bounded(&s_bar[s], (phases >> s) & 1u);
      phases ^= (1u << s);
      if (!__syncthreads_and(arrived)) {
        if (tid == 0) { atomicCAS(a.failure, FAIL_NONE, FAIL_BULK_COPY_TIMEOUT); bulk_wait_read0(); }
        return;
      }
    } else {
      const uint32_t *gin = reinterpret_cast<const uint32_t *>(a.in) + base;
      for (int i = tid; i < SCAN_TILE; i += SCAN_THREADS) s_tile[i] = (i < count) ? gin[i] : 0u;
      if (KIND == K_SEGSCAN_F32) {
        uint8_t *sf = stage + SCAN_TILE * 4;
        for (int i = tid; i < SCAN_TILE; i += SCAN_THREADS) sf[i] = (i < count) ? a.flags[base + i] : (uint8_t)0;
      }
      __syncthreads();
    }

    TRACE(2);
    // ---- each thread takes its 20 consecutive elements
    uint32_t x[SCAN_ITEMS];
    {
      const int4 *src = reinterpret_cast<const int4 *>(s_tile) + tid * (SCAN_ITEMS / 4);
#pragma unroll
      for (int j = 0; j < SCAN_ITEMS / 4; j++) {
        int4 v = src[j];
        x[4 * j + 0] = v.x; x[4 * j + 1] = v.y; x[4 * j + 2] = v.z; x[4 * j + 3] = v.w;
      }
    }
    const int first_local = tid * SCAN_ITEMS;

    // ---- in-thread pass: (pv, pf) = the thread's aggregate
    uint32_t pv, pf = 0, bits = 0;   // bits: segment starts (segmented scan) / selected keys (compaction)
    if (KIND == K_SCAN_I32) {
      uint32_t sum = 0;
#pragma unroll
      for (int q = 0; q < SCAN_ITEMS; q++) { sum += x[q]; x[q] = sum; }
      pv = sum;
    } else if (KIND == K_SEGSCAN_F32) {
      const uint32_t *s_flag = reinterpret_cast<const uint32_t *>(stage + SCAN_TILE * 4) + tid * (SCAN_ITEMS / 4);
      uint32_t fw[SCAN_ITEMS / 4];
#pragma unroll
      for (int j = 0; j < SCAN_ITEMS / 4; j++) fw[j] = s_flag[j];
      float acc = 0.0f;
#pragma unroll
      for (int q = 0; q < SCAN_ITEMS; q++) {
        const uint32_t fl = (fw[q >> 2] >> (8 * (q & 3))) & 0xffu;
        const float v = __uint_as_float(x[q]);
        if (fl) { acc = v; bits |= (1u << q); } else acc = acc + v;
        x[q] = __float_as_uint(acc);
      }
      pv = __float_as_uint(acc);
      pf = bits ? 1u : 0u;
    } else {
#pragma unroll
      for (int q = 0; q < SCAN_ITEMS; q++)
        if ((first_local + q < count) && ((x[q] & 7u) < 3u)) bits |= (1u << q);
      pv = __popc(bits);
    }

    // ---- block scan of the thread aggregates: shuffle scan in the warp, then every warp
    //      scans the 16 warp totals with shuffles
    uint32_t thv, thf = 0, tv, tf = 0;    // thread's exclusive prefix in the tile; tile aggregate
    if (KIND == K_SEGSCAN_F32) {
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        uint32_t lv = __shfl_up_sync(kFull, pv, o);
        uint32_t lf = __shfl_up_sync(kFull, pf, o);
        if (lane >= o) OpSegAddF32::combine(lv, lf, pv, pf, pv, pf);
      }
      if (lane == 31) { s_wv[warp] = pv; s_wf[warp] = pf; }
      uint32_t xv = __shfl_up_sync(kFull, pv, 1), xf = __shfl_up_sync(kFull, pf, 1);
      if (lane == 0) { xv = 0; xf = 0; }
      __syncthreads();
      uint32_t wv = (lane < SCAN_WARPS) ? s_wv[lane] : 0u, wf = (lane < SCAN_WARPS) ? s_wf[lane] : 0u;
#pragma unroll
      for (int o = 1; o < SCAN_WARPS; o <<= 1) {
        uint32_t lv = __shfl_up_sync(kFull, wv, o);
        uint32_t lf = __shfl_up_sync(kFull, wf, o);
        if (lane >= o) OpSegAddF32::combine(lv, lf, wv, wf, wv, wf);
      }
      tv = __shfl_sync(kFull, wv, SCAN_WARPS - 1);
      tf = __shfl_sync(kFull, wf, SCAN_WARPS - 1);
      uint32_t bv = __shfl_sync(kFull, wv, warp > 0 ? warp - 1 : 0), bf = __shfl_sync(kFull, wf, warp > 0 ? warp - 1 : 0);
      if (warp == 0) { bv = 0; bf = 0; }
      OpSegAddF32::combine(bv, bf, xv, xf, thv, thf);
    } else {
      const uint32_t own_v = pv;
      const uint32_t incl = warp_incl_scan_add(pv, lane);
      if (lane == 31) s_wv[warp] = incl;
      __syncthreads();
      uint32_t wv = (lane < SCAN_WARPS) ? s_wv[lane] : 0u;
      wv = warp_incl_scan_add(wv, lane);
      tv = __shfl_sync(kFull, wv, SCAN_WARPS - 1);
      uint32_t bv = __shfl_sync(kFull, wv, warp > 0 ? warp - 1 : 0);
      if (warp == 0) bv = 0;
      thv = bv + incl - own_v;
    }

    TRACE(3);
    // ---- look-back (warp 0); the other warps go on to whatever does not need the prefix
    if (warp == 0) {
      uint32_t ev, ef, cin = a.carry_in;
      if (KIND == K_SCAN_I32 && a.carry_vals != nullptr && tile < (uint32_t)LB_WINDOW)
        for (int q = 0; q < a.carry_n; q++) cin += a.carry_vals[q];
      bool ok;
      if (KIND == K_SEGSCAN_F32) ok = tile_lookback<OpSegAddF32>(a.status, tile, a.epoch, tv, tf, cin, a.failure, ev, ef);
      else ok = tile_lookback<OpAddU32>(a.status, tile, a.epoch, tv, 0u, cin, a.failure, ev, ef);
      if (lane == 0) { s_pv = ev; s_pf = ef; s_ok = ok ? 1u : 0u; }
      TRACE(4);
      // Only now is the next ticket drawn: this CTA will start that tile within about a
      // microsecond (the write-out below), so no tile is claimed long before it is worked
      // on -- a tile claimed early by a CTA that is still waiting in a look-back would
      // hold up every tile after it.  The other stage's last bulk store must have finished
      // reading shared memory before the stage is refilled.
      if (tid == 0 && ok) {
        bulk_wait_read0();
        draw_and_load(s ^ 1);
      }
    }

    if (KIND == K_FILTER || KIND == K_PARTITION) {
      // compact inside the stage (every thread holds its keys in registers since the barrier
      // above): selected keys first, in order, then the rejected ones
      uint32_t t_pos = thv;
      const int valid_before = first_local < count ? first_local : count;
      uint32_t f_pos = tv + (uint32_t)valid_before - thv;
#pragma unroll
      for (int q = 0; q < SCAN_ITEMS; q++) {
        if (bits & (1u << q)) s_tile[t_pos++] = x[q];
        else if (KIND == K_PARTITION && (first_local + q < count)) s_tile[f_pos++] = x[q];
      }
    }
    __syncthreads();
    if (!s_ok) {
      if (tid == 0) bulk_wait_read0();
      return;
    }

    if (KIND == K_SCAN_I32 || KIND == K_SEGSCAN_F32) {
      int4 *dst = reinterpret_cast<int4 *>(s_tile) + tid * (SCAN_ITEMS / 4);
      if (KIND == K_SCAN_I32) {
        const uint32_t start = s_pv + thv;
#pragma unroll
        for (int j = 0; j < SCAN_ITEMS / 4; j++) {
          int4 v;
          v.x = start + x[4 * j + 0]; v.y = start + x[4 * j + 1]; v.z = start + x[4 * j + 2]; v.w = start + x[4 * j + 3];
          dst[j] = v;
        }
      } else {
        uint32_t sv, sf2;
        OpSegAddF32::combine(s_pv, s_pf, thv, thf, sv, sf2);
        const float start = __uint_as_float(sv);
        // elements before the thread's first segment start receive the incoming prefix
        const int first = bits ? (__ffs(bits) - 1) : SCAN_ITEMS;
#pragma unroll
        for (int j = 0; j < SCAN_ITEMS / 4; j++) {
          float r[4];
#pragma unroll
          for (int e = 0; e < 4; e++) {
            const float v = __uint_as_float(x[4 * j + e]);
            r[e] = (4 * j + e < first) ? start + v : v;
          }
          int4 v; v.x = __float_as_int(r[0]); v.y = __float_as_int(r[1]); v.z = __float_as_int(r[2]); v.w = __float_as_int(r[3]);
          dst[j] = v;
        }
      }
      uint32_t *gout = reinterpret_cast<uint32_t *>(a.out) + base;
      if (bulk) {
        fence_proxy_async_smem();
        __syncthreads();
        if (tid == 0) {
          bulk_s2g(gout, s_tile, SCAN_TILE * 4);
          bulk_commit();                       // waited for (read side) before the stage is refilled
        }
      } else {
        __syncthreads();
        for (int i = tid; i < count; i += SCAN_THREADS) gout[i] = s_tile[i];
      }
    } else {
      const int64_t true_before = (int64_t)s_pv;        // selected keys in earlier tiles
      uint32_t *dst = reinterpret_cast<uint32_t *>(a.out) + true_before;
      for (uint32_t i = tid; i < tv; i += SCAN_THREADS) dst[i] = s_tile[i];
      if (KIND == K_PARTITION) {
        uint32_t *dstf = a.out_false + (base - true_before);
        const uint32_t nf = (uint32_t)count - tv;
        for (uint32_t i = tid; i < nf; i += SCAN_THREADS) dstf[i] = s_tile[tv + i];
      }
      if (tile == nt - 1 && tid == 0) *a.d_count = true_before + (int64_t)tv;
    }
    TRACE(5);
    TRACEV(6, (unsigned long long)blockIdx.x);
    // No barrier here: s_tid[s ^ 1] was written before the barrier that followed the look-back,
    // and the stage just used is refilled only after the barriers of the next iteration.
  }
  if (tid == 0) bulk_wait_read0();     // shared memory must outlive the last bulk store's reads
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

// Grid of the persistent kernel: what is resident at once (occupancy x SMs), at most one
// CTA per tile.  The occupancy query allocates nothing and is cached per kind.
template <int KIND>
static cudaError_t launch_lookback(LookbackArgs a, cudaStream_t stream) {
  constexpr int SB = StageBytes<KIND>::value;
  constexpr size_t smem = (size_t)NSTAGE * SB;
  static int ctas_per_sm_dev[64], num_sms_dev[64];     // per device ordinal (function attributes are per device)
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  int &ctas_per_sm = ctas_per_sm_dev[dev], &num_sms = num_sms_dev[dev];
  if (ctas_per_sm == 0) {
    cudaError_t err = cudaFuncSetAttribute(lookback_kernel<KIND>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return err;
    int occ = 0, sms = 0;
    err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (err != cudaSuccess) return err;
    err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, lookback_kernel<KIND>, SCAN_THREADS, smem);
    if (err != cudaSuccess) return err;
    if (occ < 1) return cudaErrorLaunchOutOfResources;
    num_sms = sms;
    ctas_per_sm = occ;
  }
  const uint32_t resident = (uint32_t)(ctas_per_sm * num_sms);
  const uint32_t grid = a.num_tiles < resident ? a.num_tiles : resident;
  lookback_kernel<KIND><<<grid, SCAN_THREADS, smem, stream>>>(a);
  return cudaGetLastError();
}

static LookbackArgs make_args(const void *in, const uint8_t *flags, void *out, uint32_t *out_false, int64_t n,
                              void *scratch, uint32_t epoch, int *failure) {
  LookbackArgs a;
  a.in = in; a.flags = flags; a.out = out; a.out_false = out_false; a.n = n;
  a.num_tiles = tiles_for(n);
  split_scratch(scratch, &a.ticket, &a.status);
  a.epoch = epoch; a.failure = failure;
  a.carry_in = 0; a.carry_vals = nullptr; a.carry_n = 0; a.d_count = nullptr;
  return a;
}

cudaError_t launch_scan_i32(const int32_t *in, int32_t *out, int64_t n, int32_t carry_in,
                            const int32_t *carry_vals, int carry_n, void *scratch,
                            uint32_t epoch, int *failure, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  LookbackArgs a = make_args(in, nullptr, out, nullptr, n, scratch, epoch, failure);
  a.carry_in = (uint32_t)carry_in;
  a.carry_vals = reinterpret_cast<const uint32_t *>(carry_vals);
  a.carry_n = carry_n;
  return launch_lookback<K_SCAN_I32>(a, stream);
}

cudaError_t launch_segscan_f32(const uint8_t *flags, const float *in, float *out, int64_t n, float carry_in,
                               void *scratch, uint32_t epoch, int *failure, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  LookbackArgs a = make_args(in, flags, out, nullptr, n, scratch, epoch, failure);
  uint32_t bits;
  memcpy(&bits, &carry_in, 4);
  a.carry_in = bits;
  return launch_lookback<K_SEGSCAN_F32>(a, stream);
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
  LookbackArgs a = make_args(in, nullptr, out_true, out_false, n, scratch, epoch, failure);
  a.d_count = d_count;
  return partition ? launch_lookback<K_PARTITION>(a, stream) : launch_lookback<K_FILTER>(a, stream);
}

// ---- scan (+) i32 without any allocation ---------------------------------------------------------
// Some hosts hand this library a GPU whose memory is already fully parcelled out by their
// own arena allocator, or run it inside a region of their program where a call that may
// synchronise the whole device or fail for lack of memory (cudaMalloc does both) is not
// acceptable, for instance a latency-bound service loop after start-up.  For them the tile
// ticket, the tile status words and the failure word of the look-back scan live in the
// fixed array below instead of in pooled memory.  The array is part of the loaded library
// image: every GPU that loads the library holds these ~52 KiB until the process exits.
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
    LookbackArgs a;
    a.in = in; a.flags = nullptr; a.out = out; a.out_false = nullptr; a.n = n;
    a.num_tiles = (uint32_t)((n + SCAN_TILE - 1) / SCAN_TILE);
    a.ticket = reinterpret_cast<uint32_t *>(base);
    a.status = reinterpret_cast<uint64_t *>(base + NOALLOC_HEAD);
    a.epoch = epoch; a.failure = failure;
    a.carry_in = 0; a.carry_vals = nullptr; a.carry_n = 0; a.d_count = nullptr;
    err = launch_lookback<K_SCAN_I32>(a, st);
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

#ifdef FB_TRACE
extern "C" __attribute__((visibility("default"))) int fb_debug_copy_trace(void *host, size_t bytes) {
  return (int)cudaMemcpyFromSymbol(host, fb::g_trace, bytes);
}
#endif
