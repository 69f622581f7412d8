// Single-pass scan kernels: inclusive scan (+) over i32, flagged segmented inclusive scan
// (+) over f32, and filter / partition compaction of u32 keys.  They replace the generated
// `segscan` kernel of the reference
// (src/Futhark/CodeGen/ImpGen/GPU/SegScan/SinglePass.hs:327-879) and, for compaction, the
// scan + scatter that prelude/soacs.fut:241-286 expands into.
//
// One persistent kernel, templated on what a tile computes; one CTA per SM.  A tile holds
// 512 x 20 = 10240 elements.  Like the reference's kernel it makes a single pass over
// memory and hands prefixes between tiles through one status word per tile (value and
// state in one 64-bit word, no fence in between, :628-660 there), and tiles are numbered
// by a ticket counter so that tile i is claimed only after every tile < i (:444-461).
// Where it differs:
//
//   * A CTA keeps a ring of shared-memory stages (5, or 4 for the segmented scan) and has
//     a tile in every one of them: being loaded (one bulk async copy, TMA, per array,
//     awaited on an mbarrier), scanned and waiting for its prefix, or being written out
//     (one bulk async store).  A tile that waits for its prefix costs no registers and no
//     thread: the CTA scans its next tile meanwhile.  So the wait for predecessors, which
//     grows with the number of tiles in flight, is covered by ~200 KB of tiles per SM.
//
//   * No tile looks back over its predecessors.  The first CTA to arrive does no tiles
//     at all: its warp 0 is the PROPAGATOR, which walks the status words once, in order,
//     256 per round trip, turning the published tile aggregates into inclusive prefixes
//     as soon as a contiguous run of them is there.  A tile therefore waits on one word
//     only (its predecessor's prefix).  The classic scheme -- every tile folds the
//     aggregates of all unresolved predecessors itself -- needs a number of dependent L2
//     round trips per tile that grows with the tiles in flight, and on 148 SMs the
//     re-reading of the same few cache lines by hundreds of warps saturates the L2 slice
//     that holds them.
//
//   * A thread owns 20 CONSECUTIVE elements = 5 x 16 bytes, an odd stride in 16-byte
//     units, so the 128-bit shared-memory accesses are conflict-free without padding;
//     in-thread sequential scan, shuffle scan of the thread totals, second shuffle scan
//     over the 16 warp totals.
//
// Progress: the propagator exists as soon as any CTA runs.  It needs the aggregates in
// tile order; a claimed tile always has a stage and a load in flight and is scanned
// without waiting for anything else, and a CTA whose stages are all taken by tiles that
// wait for prefixes holds only tiles whose predecessors are all claimed.  Every wait is
// bounded and polls the failure word.
//
// A tile that is ragged (the last one) or whose global addresses are not 16-byte aligned
// uses plain guarded loads and stores instead of the bulk copies.
#include <stdio.h>
#include <string.h>

#include <mutex>
#include <type_traits>

#include "../../include/futhark_b200.h"
#include "common.cuh"
#include "kernels.h"

namespace fb {

constexpr int SCAN_THREADS = 512;
constexpr int SCAN_ITEMS = 20;
constexpr int SCAN_TILE = SCAN_THREADS * SCAN_ITEMS;  // 10240 elements
constexpr int SCAN_WARPS = SCAN_THREADS / 32;         // 16
constexpr int PROP_PER_LANE = 8;                      // status words per lane per round of the propagator
constexpr int PROP_WINDOW = 32 * PROP_PER_LANE;
constexpr uint32_t WAIT_MAX_ROUNDS = 1u << 22;        // idle polls before a wait gives up

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

__device__ __forceinline__ bool aligned16(const void *p) { return (((uintptr_t)p) & 15u) == 0; }

#ifdef FB_TRACE
__device__ unsigned long long g_trace[32768 * 8];
__device__ __forceinline__ unsigned long long gtime() { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }
#define TRACE(tile, slot) do { if (threadIdx.x == 0 && (tile) < 32768u) g_trace[(tile) * 8 + (slot)] = gtime(); } while (0)
#else
#define TRACE(tile, slot) do {} while (0)
#endif

// ---- the propagator (one warp in the whole grid) --------------------------------------------
// Walks the status words in tile order.  For every contiguous run of published aggregates
// it writes the inclusive prefixes back.  `seed` is the exclusive prefix of tile 0.
template <typename Op>
__device__ void run_propagator(uint64_t *status, uint32_t nt, uint32_t epoch, uint32_t seed, int *failure) {
  const int lane = threadIdx.x & 31;
  uint32_t run_v = seed, run_f = 0;     // inclusive prefix of tile pos-1
  uint32_t pos = 0, idle = 0;
  while (pos < nt) {
    uint64_t w[PROP_PER_LANE];
    const uint32_t first = pos + PROP_PER_LANE * lane;
    int ready = 0;                      // leading published entries of this lane
    bool open = true;
#pragma unroll
    for (int q = 0; q < PROP_PER_LANE; q++) {
      const uint32_t idx = first + q;
      w[q] = (idx < nt) ? ld_status(&status[idx]) : 0ull;
    }
#pragma unroll
    for (int q = 0; q < PROP_PER_LANE; q++) {
      const bool ok = (first + q < nt) && (status_state(w[q], epoch) != ST_NONE);
      if (open && ok) ready++; else open = false;
    }
    const unsigned partial = __ballot_sync(kFull, ready < PROP_PER_LANE);
    const int stop_lane = partial ? (__ffs(partial) - 1) : 32;      // first lane with a gap
    const int stop_ready = __shfl_sync(kFull, ready, stop_lane & 31);
    const uint32_t run = (stop_lane == 32) ? (uint32_t)PROP_WINDOW : (uint32_t)(PROP_PER_LANE * stop_lane + stop_ready);
    if (run == 0) {
      idle++;
      if ((idle & 255u) == 0) {
        int fl = (lane == 0) ? ld_failure(failure) : 0;
        if (__shfl_sync(kFull, fl, 0) != FAIL_NONE) return;
        if (idle >= WAIT_MAX_ROUNDS) {
          if (lane == 0) atomicCAS(failure, FAIL_NONE, FAIL_LOOKBACK_TIMEOUT);
          return;
        }
      }
      if (idle > 64) __nanosleep(100);
      continue;
    }
    idle = 0;
    const int mine = (lane < stop_lane) ? PROP_PER_LANE : (lane == stop_lane ? stop_ready : 0);
    // in-lane inclusive fold of the aggregates, then exclusive scan across lanes
    uint32_t iv[PROP_PER_LANE], iflag[PROP_PER_LANE];
    uint32_t tv = 0, tf = 0;            // lane total (identity if the lane has nothing)
#pragma unroll
    for (int q = 0; q < PROP_PER_LANE; q++) {
      if (q < mine) {
        const uint32_t av = status_value(w[q]), af = Op::kHasFlag ? status_flag(w[q]) : 0u;
        if (q == 0) { tv = av; tf = af; } else Op::combine(tv, tf, av, af, tv, tf);
      }
      iv[q] = tv; iflag[q] = tf;
    }
    uint32_t sv = tv, sf = tf;          // inclusive scan of lane totals
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      uint32_t lv = __shfl_up_sync(kFull, sv, o), lf = __shfl_up_sync(kFull, sf, o);
      if (lane >= o) Op::combine(lv, lf, sv, sf, sv, sf);
    }
    uint32_t ev = __shfl_up_sync(kFull, sv, 1), ef = __shfl_up_sync(kFull, sf, 1);
    if (lane == 0) { ev = run_v; ef = run_f; } else Op::combine(run_v, run_f, ev, ef, ev, ef);
    // ev/ef: inclusive prefix of the tile just before this lane's first entry
#pragma unroll
    for (int q = 0; q < PROP_PER_LANE; q++) {
      if (q < mine) {
        uint32_t pv, pf;
        Op::combine(ev, ef, iv[q], iflag[q], pv, pf);
        st_status(&status[first + q], pack_status(pv, epoch, pf, ST_PREFIX));
#ifdef FB_TRACE
        if (first + q < 32768u) g_trace[(first + q) * 8 + 7] = gtime();
#endif
      }
    }
    // new running prefix = inclusive prefix of the last tile of the run
    uint32_t lastv, lastf;
    Op::combine(run_v, run_f, __shfl_sync(kFull, sv, 31), __shfl_sync(kFull, sf, 31), lastv, lastf);
    run_v = lastv; run_f = lastf;
    pos += run;
  }
}

// ---- the persistent kernel ---------------------------------------------------------------------------
enum ScanKind : int { K_SCAN_I32 = 0, K_SEGSCAN_F32 = 1, K_FILTER = 2, K_PARTITION = 3 };

template <int KIND> struct StageCfg { static constexpr int bytes = SCAN_TILE * 4; static constexpr int stages = 5; };
template <> struct StageCfg<K_SEGSCAN_F32> { static constexpr int bytes = SCAN_TILE * 4 + SCAN_TILE; static constexpr int stages = 4; };

// 32-bit load that goes to L2 (never served from a stale L1 line)
__device__ __forceinline__ int ld_stream_relaxed(const void *p) {
  int v;
  asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

struct LookbackArgs {
  const void *in;          // values / keys
  const uint8_t *flags;    // segmented scan only
  void *out;               // scan result, or the selected keys
  uint32_t *out_false;     // partition: the rejected keys
  int64_t n;
  uint32_t num_tiles;
  uint32_t *ticket;        // [0] tile tickets, [1] role counter
  uint64_t *status;
  uint32_t epoch;
  int *failure;
  uint32_t carry_in;       // value bits of the seed (0 for compaction)
  const uint32_t *carry_vals;
  int carry_n;
  int64_t *d_count;        // compaction: number of selected keys
};

enum : uint32_t { ACT_IDLE = 0, ACT_SCAN = 1, ACT_FINISH = 2, ACT_FIXUP = 3, ACT_DONE = 4, ACT_FAIL = 5 };
enum : uint32_t { SLOT_FREE = 0, SLOT_LOADING = 1, SLOT_LOADED = 2, SLOT_WAITING = 3, SLOT_STORING = 4 };
constexpr int PENDING_MAX = 32;           // scanned tiles of one CTA that may wait for their prefix
constexpr uint32_t HEAD_MAX = 2048;       // segmented scan: longest head patched in global memory

// Bulk-store groups complete in order; waits for all but the newest `newer` groups to be
// complete (written, not only read).
__device__ __forceinline__ void bulk_wait_all_but(uint32_t newer) {
  if (newer == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  else if (newer == 1) asm volatile("cp.async.bulk.wait_group 1;" ::: "memory");
  else if (newer == 2) asm volatile("cp.async.bulk.wait_group 2;" ::: "memory");
  else asm volatile("cp.async.bulk.wait_group 3;" ::: "memory");
}

template <int KIND>
__global__ void __launch_bounds__(SCAN_THREADS, 1)
lookback_kernel(const LookbackArgs a) {
  constexpr int SB = StageCfg<KIND>::bytes;
  constexpr int NST = StageCfg<KIND>::stages;
  using Op = typename std::conditional<KIND == K_SEGSCAN_F32, OpSegAddF32, OpAddU32>::type;
  extern __shared__ __align__(128) unsigned char s_stages[];
  __shared__ __align__(8) uint64_t s_bar[NST];
  // bookkeeping, touched by thread 0 only (shared memory because it is indexed dynamically)
  __shared__ uint32_t s_slot_state[NST], s_slot_tile[NST], s_slot_phase[NST];
  __shared__ uint32_t s_lq[NST];                       // slots in the order their tiles were claimed
  __shared__ uint32_t s_pq_tile[PENDING_MAX], s_pq_info[PENDING_MAX], s_pq_seq[PENDING_MAX];
  // per-action communication
  __shared__ uint32_t s_wv[SCAN_WARPS], s_wf[SCAN_WARPS], s_ff[SCAN_WARPS];
  __shared__ uint32_t s_act, s_slot, s_tile_id, s_info, s_pv, s_pf, s_role, s_agg_v, s_agg_f, s_fix, s_fix_tile;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (ld_failure(a.failure) != FAIL_NONE) return;
  const uint32_t nt = a.num_tiles;

  // ---- role: the first CTA to arrive propagates prefixes, all others work on tiles
  if (tid == 0) {
    const uint32_t r = atomicAdd(&a.ticket[1], 1u);
    if (r == gridDim.x - 1) atomicExch(&a.ticket[1], 0u);     // rewind for the next launch
    s_role = r;
  }
  __syncthreads();
  if (s_role == 0 && gridDim.x > 1) {
    if (warp == 0) {
      uint32_t seed = a.carry_in;
      if (KIND == K_SCAN_I32 && a.carry_vals != nullptr)
        for (int q = 0; q < a.carry_n; q++) seed += a.carry_vals[q];
      run_propagator<Op>(a.status, nt, a.epoch, seed, a.failure);
    }
    return;
  }
  // A grid of one CTA has no propagator: the lone worker carries the running prefix itself.
  const bool self_propagate = (gridDim.x == 1);
  const uint32_t workers = self_propagate ? 1u : gridDim.x - 1;
  const uint32_t last_draw = nt + workers - 1;   // every worker ends on exactly one invalid ticket
  const bool ptr_aligned = aligned16(a.in) && (KIND == K_FILTER || KIND == K_PARTITION || aligned16(a.out)) &&
                           (KIND != K_SEGSCAN_F32 || aligned16(a.flags));
  auto tile_is_bulk = [&](uint32_t t) -> bool { return ptr_aligned && ((int64_t)(t + 1) * SCAN_TILE <= a.n); };

  // thread 0's private counters
  uint32_t lq_head = 0, lq_tail = 0;          // claimed tiles not yet scanned: s_lq[lq_head % NST ..]
  uint32_t pq_head = 0, pq_tail = 0;          // scanned tiles waiting for their prefix
  uint32_t stores_committed = 0;              // bulk-store groups committed so far
  uint32_t last_store_slot = 0;
  uint32_t n_storing = 0, store_age = 0;      // slots in SLOT_STORING; decisions since the last store was committed
  bool in_hand = false;                       // a ticket has been drawn but not yet given a stage
  uint32_t next_ticket = 0;
  bool exhausted = false;
  uint32_t self_v = a.carry_in, self_f = 0;   // running prefix of a lone worker
  uint32_t idle = 0;
  // The status word of the oldest waiting tile's predecessor is read at the START of every
  // action and looked at when the action is over, so the L2 round trip overlaps the work.
  uint64_t polled_w = 0;
  uint32_t polled_idx = 0xffffffffu;

  if (tid == 0) {
    for (int s = 0; s < NST; s++) { mbar_init(&s_bar[s], 1); s_slot_state[s] = SLOT_FREE; s_slot_phase[s] = 0; }
    fence_mbar_init();
    if (self_propagate && KIND == K_SCAN_I32 && a.carry_vals != nullptr)
      for (int q = 0; q < a.carry_n; q++) self_v += a.carry_vals[q];
  }
  __syncthreads();

  while (true) {
    // ================= thread 0 decides what the CTA does next =================
    if (tid == 0) {
      // Stages whose bulk store was committed before the action that just ended have had time
      // to be read; this wait is then (nearly) free.
      // (stores finish in order: wait_group.read 1 leaves only the newest one possibly reading)
      if (n_storing > 0 && store_age > 0) {
        bulk_wait_read0();
        for (int s = 0; s < NST; s++) if (s_slot_state[s] == SLOT_STORING) s_slot_state[s] = SLOT_FREE;
        n_storing = 0;
      } else if (n_storing >= 2) {
        bulk_wait_read1();
        for (int s = 0; s < NST; s++)
          if (s_slot_state[s] == SLOT_STORING && s != (int)last_store_slot) s_slot_state[s] = SLOT_FREE;
        n_storing = 1;
      }
      store_age++;
      // Put the ticket drawn during the last action (if any) into a free stage.
      auto place_ticket = [&]() {
        const uint32_t t = next_ticket;
        if (t == last_draw) { atomicExch(&a.ticket[0], 0u); }   // rewind for the next launch (once)
        if (t >= nt) { exhausted = true; in_hand = false; return; }
        int fs = -1;
        for (int s = 0; s < NST; s++) if (s_slot_state[s] == SLOT_FREE) { fs = s; break; }
        if (fs < 0) return;
        in_hand = false;
        s_slot_state[fs] = SLOT_LOADING; s_slot_tile[fs] = t;
        TRACE(t, 4);
#ifdef FB_TRACE
        if (t < 32768u) g_trace[t * 8 + 6] = blockIdx.x;
#endif
        if (tile_is_bulk(t)) {
          unsigned char *st = s_stages + fs * SB;
          const int64_t tb = (int64_t)t * SCAN_TILE;
          mbar_expect_tx(&s_bar[fs], SB);
          bulk_g2s(st, reinterpret_cast<const uint32_t *>(a.in) + tb, SCAN_TILE * 4, &s_bar[fs]);
          if (KIND == K_SEGSCAN_F32) bulk_g2s(st + SCAN_TILE * 4, a.flags + tb, SCAN_TILE, &s_bar[fs]);
        }
        s_lq[lq_tail % NST] = fs; lq_tail++;
      };
      if (in_hand) place_ticket();
      uint32_t act = ACT_IDLE, slot = 0;
      // is the next claimed tile loaded?
      int scan_slot = -1;
      if (lq_head != lq_tail) {
        const int s = (int)s_lq[lq_head % NST];
        if (s_slot_state[s] == SLOT_LOADING &&
            (!tile_is_bulk(s_slot_tile[s]) || mbar_try_wait(&s_bar[s], s_slot_phase[s]))) {
          if (tile_is_bulk(s_slot_tile[s])) s_slot_phase[s] ^= 1u;   // the barrier's next completion has the other parity
          s_slot_state[s] = SLOT_LOADED;
          TRACE(s_slot_tile[s], 5);
        }
        if (s_slot_state[s] == SLOT_LOADED) scan_slot = s;
      }
      // Oldest tile waiting for its prefix: is the prefix there?  (The inclusive prefix of the
      // predecessor; for the segmented operator a predecessor that contains a segment start
      // supplies it with its aggregate alone.)
      bool have = false;
      uint32_t ptile = 0, pinfo = 0;
      if (pq_head != pq_tail) {
        const uint32_t e = pq_head % PENDING_MAX;
        ptile = s_pq_tile[e]; pinfo = s_pq_info[e];
        if (self_propagate) { s_pv = self_v; s_pf = self_f; have = true; }
        else if (ptile == 0) {
          uint32_t seed = a.carry_in;
          if (KIND == K_SCAN_I32 && a.carry_vals != nullptr) for (int q = 0; q < a.carry_n; q++) seed += a.carry_vals[q];
          s_pv = seed; s_pf = 0; have = true;
        } else {
          // the word read during the previous action, or a fresh read when there is nothing to scan
          uint64_t w = (polled_idx == ptile - 1) ? polled_w : 0ull;
          auto usable = [&](uint64_t ww) -> bool {
            const uint32_t st = status_state(ww, a.epoch);
            return st == ST_PREFIX || (Op::kHasFlag && st == ST_AGG && status_flag(ww));
          };
          if (!usable(w) && scan_slot < 0) w = ld_status(&a.status[ptile - 1]);
          if (usable(w)) { s_pv = status_value(w); s_pf = Op::kHasFlag ? status_flag(w) : 0u; have = true; }
        }
      }
      s_fix = 0;
      if (scan_slot >= 0 && !(have && !(pinfo & 0x80000000u))) {
        // Scan, unless a tile that still sits in a stage can be finished: finishing frees the
        // stage for the next load (measured: better than scanning first).
        act = ACT_SCAN; slot = (uint32_t)scan_slot; s_tile_id = s_slot_tile[scan_slot];
        if (have && (pinfo & 0x80000000u)) {
          // a stored tile's head can be patched along the way (its loads overlap the scan)
          const uint32_t newer = stores_committed - s_pq_seq[pq_head % PENDING_MAX];
          bulk_wait_all_but(newer > 3 ? 3 : newer);
          s_fix = 1; s_fix_tile = ptile; s_info = pinfo;
        }
      } else if (have) {
        s_tile_id = ptile; s_info = pinfo;
        if (pinfo & 0x80000000u) {             // already stored: patch its head in global memory
          act = ACT_FIXUP;
          const uint32_t newer = stores_committed - s_pq_seq[pq_head % PENDING_MAX];
          bulk_wait_all_but(newer > 3 ? 3 : newer);
        } else { act = ACT_FINISH; slot = pinfo & 0xffu; }
      }
      if (act == ACT_IDLE) {
        if (exhausted && !in_hand && pq_head == pq_tail && lq_head == lq_tail) act = ACT_DONE;
        else {
          // nothing to compute: this is the time for the blocking bits of housekeeping
          bool did = false;
          if (n_storing > 0) {
            bulk_wait_read0();
            for (int s = 0; s < NST; s++) if (s_slot_state[s] == SLOT_STORING) s_slot_state[s] = SLOT_FREE;
            n_storing = 0; did = true;
          }
          if (!in_hand && !exhausted && pq_tail - pq_head + (lq_tail - lq_head) < PENDING_MAX) {
            bool any_free = false;
            for (int s = 0; s < NST; s++) any_free |= (s_slot_state[s] == SLOT_FREE);
            if (any_free) { next_ticket = atomicAdd(&a.ticket[0], 1u); in_hand = true; }
          }
          if (in_hand) { place_ticket(); did = did || !in_hand; }
          if (!did) {
            idle++;
            if ((idle & 255u) == 0 && ld_failure(a.failure) != FAIL_NONE) act = ACT_FAIL;
            if (idle >= WAIT_MAX_ROUNDS) { atomicCAS(a.failure, FAIL_NONE, FAIL_LOOKBACK_TIMEOUT); act = ACT_FAIL; }
            if (act == ACT_IDLE && idle > 4) __nanosleep(idle < 64 ? 20 : 100);
          }
        }
      } else idle = 0;
      s_act = act; s_slot = slot;
    }
    __syncthreads();
    const uint32_t act = s_act;
    const int s = (int)s_slot;
    if (act == ACT_DONE) break;
    if (act == ACT_FAIL) {
      // drain: bulk stores must finish reading shared memory; loads in flight are awaited with a limit
      if (tid == 0) {
        bulk_wait_read0();
        for (uint32_t c = lq_head; c != lq_tail; c++) {
          const int q = (int)s_lq[c % NST];
          if (s_slot_state[q] == SLOT_LOADING && tile_is_bulk(s_slot_tile[q])) (void)mbar_wait_bounded(&s_bar[q], s_slot_phase[q], 1u << 16);
        }
      }
      return;
    }
    if (act == ACT_IDLE) { __syncthreads(); continue; }
    const uint32_t tile = s_tile_id;
    if (tid == 0 && !in_hand && !exhausted && pq_tail - pq_head + (lq_tail - lq_head) < PENDING_MAX) {
      // Draw the next ticket now if a stage is (or is about to be) free: the atomic's round trip
      // overlaps the action, and the tile gets its stage at the next decision.
      bool room = (act == ACT_FINISH) || n_storing > 0;
      for (int q = 0; q < NST; q++) room |= (s_slot_state[q] == SLOT_FREE);
      if (room) {
        next_ticket = atomicAdd(&a.ticket[0], 1u);     // looked at only when the action is over
        in_hand = true;
      }
    }
    if (tid == 0 && !self_propagate) {
      // which tile will be the oldest one waiting once this action is over?
      polled_idx = 0xffffffffu;
      uint32_t t = 0xffffffffu;
      const uint32_t h = pq_head + ((act == ACT_FINISH || act == ACT_FIXUP || s_fix) ? 1u : 0u);
      if (h != pq_tail) t = s_pq_tile[h % PENDING_MAX];
      else if (act == ACT_SCAN) t = tile;
      if (t != 0xffffffffu && t > 0) { polled_idx = t - 1; polled_w = ld_status(&a.status[t - 1]); }
    }

    unsigned char *stage = s_stages + s * SB;
    uint32_t *s_tile = reinterpret_cast<uint32_t *>(stage);
    const int64_t base = (int64_t)tile * SCAN_TILE;
    const int count = (int)((a.n - base) < SCAN_TILE ? (a.n - base) : SCAN_TILE);
    const bool bulk = tile_is_bulk(tile);

    if (act == ACT_SCAN) {
      // ================= local scan of a freshly loaded tile =================
      TRACE(tile, 0);
      // piggy-backed fix-up of an already stored tile: read its head now, write it at the end
      const bool fix = (KIND == K_SEGSCAN_F32) && s_fix;
      float fixv[HEAD_MAX / SCAN_THREADS];
      float *fixg = nullptr;
      uint32_t fix_head = 0;
      float fix_add = 0.f;
      if (fix) {
        fix_head = s_info & 0x7fffffffu;
        fix_add = __uint_as_float(s_pv);
        fixg = reinterpret_cast<float *>(a.out) + (int64_t)s_fix_tile * SCAN_TILE;
#pragma unroll
        for (int q = 0; q < (int)(HEAD_MAX / SCAN_THREADS); q++) {
          const uint32_t i = tid + q * SCAN_THREADS;
          fixv[q] = (i < fix_head) ? __uint_as_float((uint32_t)ld_stream_relaxed(&fixg[i])) : 0.f;
        }
      }
      if (!bulk) {
        const uint32_t *gin = reinterpret_cast<const uint32_t *>(a.in) + base;
        for (int i = tid; i < SCAN_TILE; i += SCAN_THREADS) s_tile[i] = (i < count) ? gin[i] : 0u;
        if (KIND == K_SEGSCAN_F32) {
          uint8_t *sf = stage + SCAN_TILE * 4;
          for (int i = tid; i < SCAN_TILE; i += SCAN_THREADS) sf[i] = (i < count) ? a.flags[base + i] : (uint8_t)0;
        }
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
      const int first_local = tid * SCAN_ITEMS;
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

      // block scan of the thread aggregates
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

      // publish the tile aggregate as early as possible
      if (tid == 0) {
        if (self_propagate) { s_agg_v = tv; s_agg_f = tf; }   // folded into the running prefix when the tile is finished
        else st_status(&a.status[tile], pack_status(tv, a.epoch, tf, ST_AGG));
      }

      // tile-local results back into the stage
      if (KIND == K_SCAN_I32 || KIND == K_SEGSCAN_F32) {
        int4 *dst = reinterpret_cast<int4 *>(s_tile) + tid * (SCAN_ITEMS / 4);
        if (KIND == K_SCAN_I32) {
#pragma unroll
          for (int j = 0; j < SCAN_ITEMS / 4; j++) {
            int4 v;
            v.x = thv + x[4 * j + 0]; v.y = thv + x[4 * j + 1]; v.z = thv + x[4 * j + 2]; v.w = thv + x[4 * j + 3];
            dst[j] = v;
          }
        } else {
          // elements before the thread's first segment start continue the thread's exclusive prefix
          const float start = __uint_as_float(thv);
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
          // index of the first segment start in the tile: the incoming prefix applies before it
          uint32_t ff = bits ? (uint32_t)(first_local + first) : (uint32_t)SCAN_TILE;
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) { uint32_t t2 = __shfl_xor_sync(kFull, ff, o); ff = t2 < ff ? t2 : ff; }
          if (lane == 0) s_ff[warp] = ff;
          fence_proxy_async_smem();            // the stage may be bulk-stored right after the barrier
        }
      } else {
        // compact inside the stage: selected keys first, in order, then the rejected ones
        // (every thread took its keys into registers before the barrier of the block scan)
        uint32_t t_pos = thv;
        const int valid_before = first_local < count ? first_local : count;
        uint32_t f_pos = tv + (uint32_t)valid_before - thv;
#pragma unroll
        for (int q = 0; q < SCAN_ITEMS; q++) {
          if (bits & (1u << q)) s_tile[t_pos++] = x[q];
          else if (KIND == K_PARTITION && (first_local + q < count)) s_tile[f_pos++] = x[q];
        }
      }
      if (fix) {
#pragma unroll
        for (int q = 0; q < (int)(HEAD_MAX / SCAN_THREADS); q++) {
          const uint32_t i = tid + q * SCAN_THREADS;
          if (i < fix_head) fixg[i] = fix_add + fixv[q];
        }
      }
      __syncthreads();
      if (tid == 0) {
        if (fix) pq_head++;
        uint32_t info = (uint32_t)s;            // waits in its stage
        uint32_t state = SLOT_WAITING;
        if (KIND == K_SEGSCAN_F32) {
          uint32_t head = SCAN_TILE;
          for (int wq = 0; wq < SCAN_WARPS; wq++) head = s_ff[wq] < head ? s_ff[wq] : head;
          if (bulk && head <= HEAD_MAX && !self_propagate) {
            // Only the `head` elements before the first segment start depend on the incoming
            // prefix: write the tile out now and patch those few in global memory later, so
            // that the stage is free again at once.
            bulk_s2g(reinterpret_cast<uint32_t *>(a.out) + base, s_tile, SCAN_TILE * 4);
            bulk_commit();
            stores_committed++;
            state = SLOT_STORING; n_storing++; store_age = 0; last_store_slot = (uint32_t)s;
            info = 0x80000000u | head;
          } else {
            info = (uint32_t)s | (head << 8);    // finish from the stage: prefix applies to [0, head)
          }
        } else if (KIND == K_FILTER || KIND == K_PARTITION) {
          info = (uint32_t)s | (tv << 8);        // selected count of the tile
        }
        s_slot_state[s] = state;
        const uint32_t e = pq_tail % PENDING_MAX;
        s_pq_tile[e] = tile; s_pq_info[e] = info; s_pq_seq[e] = stores_committed;
        pq_tail++; lq_head++;
      }
      TRACE(tile, 1);
    } else if (act == ACT_FINISH) {
      // ================= finish from the stage: apply the incoming prefix and write out =================
      TRACE(tile, 2);
      const uint32_t pv_in = s_pv;
      const uint32_t extra = s_info >> 8;       // segmented scan: head length; compaction: selected count
      if (KIND == K_SCAN_I32) {
        int4 *p4 = reinterpret_cast<int4 *>(s_tile);
#pragma unroll
        for (int j = 0; j < SCAN_ITEMS / 4; j++) {
          int4 v = p4[tid + j * SCAN_THREADS];
          v.x += pv_in; v.y += pv_in; v.z += pv_in; v.w += pv_in;
          p4[tid + j * SCAN_THREADS] = v;
        }
      } else if (KIND == K_SEGSCAN_F32) {
        const float add = __uint_as_float(pv_in);
        float *pf32 = reinterpret_cast<float *>(s_tile);
        for (uint32_t i = tid; i < extra; i += SCAN_THREADS) pf32[i] = add + pf32[i];
      }
      if (KIND == K_SCAN_I32 || KIND == K_SEGSCAN_F32) {
        uint32_t *gout = reinterpret_cast<uint32_t *>(a.out) + base;
        if (bulk) {
          fence_proxy_async_smem();
          __syncthreads();
          if (tid == 0) {
            bulk_s2g(gout, s_tile, SCAN_TILE * 4);
            bulk_commit();
            stores_committed++;
            s_slot_state[s] = SLOT_STORING; n_storing++; store_age = 0; last_store_slot = (uint32_t)s;
          }
        } else {
          __syncthreads();
          for (int i = tid; i < count; i += SCAN_THREADS) gout[i] = s_tile[i];
          __syncthreads();
          if (tid == 0) s_slot_state[s] = SLOT_FREE;
        }
      } else {
        const uint32_t tile_true = extra;
        const int64_t true_before = (int64_t)pv_in;       // selected keys in earlier tiles
        uint32_t *dst = reinterpret_cast<uint32_t *>(a.out) + true_before;
        for (uint32_t i = tid; i < tile_true; i += SCAN_THREADS) dst[i] = s_tile[i];
        if (KIND == K_PARTITION) {
          uint32_t *dstf = a.out_false + (base - true_before);
          const uint32_t nf = (uint32_t)count - tile_true;
          for (uint32_t i = tid; i < nf; i += SCAN_THREADS) dstf[i] = s_tile[tile_true + i];
        }
        if (tile == nt - 1 && tid == 0) *a.d_count = true_before + (int64_t)tile_true;
        __syncthreads();
        if (tid == 0) s_slot_state[s] = SLOT_FREE;
      }
      if (tid == 0) {
        if (self_propagate) {
          uint32_t nv, nf2;
          Op::combine(self_v, self_f, s_agg_v, s_agg_f, nv, nf2);   // a lone worker finishes each tile right after scanning it
          self_v = nv; self_f = nf2;
          st_status(&a.status[tile], pack_status(nv, a.epoch, nf2, ST_PREFIX));   // the shard summary reads the last one
        }
        pq_head++;
      }
      TRACE(tile, 3);
    } else {
      // ================= fix-up: the tile was stored already; add the prefix to its head =================
      TRACE(tile, 2);
      if (KIND == K_SEGSCAN_F32) {
        const uint32_t head = s_info & 0x7fffffffu;
        const float add = __uint_as_float(s_pv);
        float *g = reinterpret_cast<float *>(a.out) + base;
        // thread 0 waited for the tile's bulk store to complete before the barrier above
        for (uint32_t i = tid; i < head; i += SCAN_THREADS) {
          const float old = __uint_as_float((uint32_t)ld_stream_relaxed(&g[i]));
          g[i] = add + old;
        }
      }
      __syncthreads();
      if (tid == 0) pq_head++;
      TRACE(tile, 3);
    }
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
  constexpr size_t smem = (size_t)StageCfg<KIND>::stages * StageCfg<KIND>::bytes;
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
  // one propagator CTA + workers; a single tile runs as one self-propagating worker
  const uint32_t resident = (uint32_t)(ctas_per_sm * num_sms);
  uint32_t grid = a.num_tiles + 1 < resident ? a.num_tiles + 1 : resident;
  if (a.num_tiles <= 1 || grid < 2) grid = 1;
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
