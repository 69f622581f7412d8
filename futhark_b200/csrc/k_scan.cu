// Single-pass scan kernels: scans, flagged and regular segmented scans, scans with a fused
// map body and post-operation, and filter / partition compaction.  They replace the generated
// `segscan` kernel of the reference
// (src/Futhark/CodeGen/ImpGen/GPU/SegScan/SinglePass.hs:327-879) and, for compaction, the
// scan + scatter that prelude/soacs.fut:241-323 expands into.
//
// One persistent kernel, templated on a specification type (scan_specs.cuh) that supplies
// operator, map body, post-operation, flag source and predicate; 8 worker warps and one
// scheduler warp per CTA, 4 CTAs per SM.  A tile holds 256 x 20 = 5120 elements.  Like the
// reference's kernel it hands
// prefixes between tiles through one status word per tile (value and state in one 64-bit
// word, :628-660 there) and numbers its work by a global counter, so that what a tile
// depends on has always been claimed by a running CTA before it (:444-461).  Where it
// differs:
//
//   * A tile is visited twice.  Visit A only computes the tile's aggregate and publishes
//     it.  Visit B, drawn from the same counter about 20 MiB of input later, scans the
//     tile, adds its exclusive prefix and stores.  Visit A reads the tile from HBM and
//     leaves it in L2, where visit B finds it, so HBM traffic stays at one read and one
//     write per element.  Because the aggregates run that far ahead, the prefix a visit B
//     needs has long been published: in the steady state no tile waits for another, which
//     the look-back of the classic single-visit scheme cannot avoid once ~200 tiles finish
//     per microsecond (every resident tile then sits in that wait).
//
//   * No tile looks back over its predecessors.  The first CTA to arrive does no tiles:
//     its warp 0 is the PROPAGATOR, which walks the status words once, in order, 256 per
//     round trip, turning published aggregates into inclusive prefixes.  Visit B reads one
//     word, its predecessor's prefix.
//
//   * Loads run ahead of the threads.  The scheduler warp draws work items ahead and
//     starts a bulk async copy (TMA) per array of the next item's tile into the other of
//     two shared-memory buffers; an mbarrier hands the buffer to the workers when it has
//     landed.  A worker thread owns 20 CONSECUTIVE elements = 5 x 16 bytes, an odd stride in
//     16-byte units, so the 128-bit shared-memory accesses are conflict-free without
//     padding: sequential scan in the thread, one shuffle scan of the thread totals, 8 warp
//     totals through shared memory.  Visit B writes its results back into the buffer and
//     the scheduler sends it off with one bulk store; compaction ranks the keys, stages
//     them in the buffer at the 16-byte phase of their destination and the scheduler warp
//     copies the runs out as aligned vectors.
//
//   * The workers wait for little.  In a visit A they leave their warp totals in shared
//     memory, arrive at a named barrier and go on to the next tile; the scheduler warp waits
//     there, folds the totals and publishes the aggregate.  In a visit B they meet once (warp
//     totals and incoming prefix, which the scheduler fetched meanwhile), write their results
//     and arrive; drawing work, status polls, the store and the wait for the store to have
//     read its buffer are all the scheduler's.
//
// Progress: the propagator exists as soon as any CTA runs and needs the aggregates in
// tile order.  Visit A waits for nothing, and visit B of tile t is drawn after visit A of
// every tile <= t, so the lowest tile whose aggregate is missing always belongs to a CTA
// that is on its way to it.  Every wait is bounded and polls the failure word.
//
// A tile that is ragged (the last one) or whose global addresses are not 16-byte aligned
// is copied into the buffer by the threads with guarded loads, and copied out likewise.
#include <stdio.h>
#include <string.h>

#include <mutex>
#include <type_traits>

#include "../../include/futhark_b200.h"
#include "common.cuh"
#include "kernels.h"
#include "scan_specs.cuh"

namespace fb {

constexpr int SCAN_WORKERS = 256;                         // threads that work on the tiles
constexpr int SCAN_WARPS = SCAN_WORKERS / 32;
constexpr int SCAN_THREADS = SCAN_WORKERS + 32;           // ... and the scheduler warp
constexpr int SCAN_TILE_MIN = SCAN_WORKERS * 12;          // the smallest tile a specification may choose (V = 3): bounds the number of status words
// Named barriers of the tile kernel (0 is __syncthreads); the first two exist once per slot r of a ring of iterations.
constexpr int BAR_MID = 1;       // +r: visit B: the warp totals and the tile's incoming prefix are written (workers wait, the scheduler arrives)
constexpr int BAR_DONE = 5;      // +r: the workers are through with the iteration's buffer (workers arrive, the scheduler waits)
constexpr int BAR_WORKERS = 9;   // the workers among themselves (a tile copied in or out by the threads)
template <int ID, int COUNT>
__device__ __forceinline__ void bar_sync() { asm volatile("bar.sync %0, %1;" ::"n"(ID), "n"(COUNT) : "memory"); }
template <int ID, int COUNT>
__device__ __forceinline__ void bar_arrive() { asm volatile("bar.arrive %0, %1;" ::"n"(ID), "n"(COUNT) : "memory"); }
// barrier ID + r, r < 4 (the slot of the iteration in a small ring)
template <int ID, int COUNT>
__device__ __forceinline__ void bar_sync(int r) {
  switch (r) {
    case 0: bar_sync<ID, COUNT>(); break;
    case 1: bar_sync<ID + 1, COUNT>(); break;
    case 2: bar_sync<ID + 2, COUNT>(); break;
    default: bar_sync<ID + 3, COUNT>(); break;
  }
}
template <int ID, int COUNT>
__device__ __forceinline__ void bar_arrive(int r) {
  switch (r) {
    case 0: bar_arrive<ID, COUNT>(); break;
    case 1: bar_arrive<ID + 1, COUNT>(); break;
    case 2: bar_arrive<ID + 2, COUNT>(); break;
    default: bar_arrive<ID + 3, COUNT>(); break;
  }
}
template <int N>
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
constexpr int PROP_PER_LANE = 8;                          // status words per lane per round of the propagator
constexpr int PROP_WINDOW = 32 * PROP_PER_LANE;
constexpr uint32_t WAIT_MAX_ROUNDS = 1u << 22;            // idle polls before a wait gives up

template <typename S> struct TileOf {
  static constexpr int ITEMS = S::V * 4;
  static constexpr int TILE = SCAN_WORKERS * ITEMS;
  // bytes of a tile buffer; compaction stages with up to 9 words of padding, the flag bytes lie behind the values
  static constexpr int FO = S::kCompact ? TILE * 4 + 64 : TILE * 4;
  static constexpr int SB = S::kCompact ? TILE * 4 + 64 + (S::kFlagArray ? TILE : 0) : TILE * 4 + (S::kFlagArray ? TILE : 64);
};

__device__ __forceinline__ bool aligned16(const void *p) { return (((uintptr_t)p) & 15u) == 0; }


// ---- a shard's summary written into the other GPUs' memory ---------------------------------------
// Exchange buffer of a rank: PEER_RING generations of `world` slots of 4 words {value, flag,
// sequence number, -}; generation = sequence number mod PEER_RING.  Rank q writes slot q of the
// ranks behind it with ordinary peer stores, the sequence number last and with release
// semantics at system scope; the reader (apply_carry_peer_kernel) acquires it.
constexpr uint32_t PEER_RING = 16;
__device__ __forceinline__ void push_summary(uint32_t *const *bufs, int rank, int world, uint32_t seq, uint32_t v, uint32_t f) {
  for (int r = rank + 1; r < world; r++) {
    uint32_t *slot = bufs[r] + ((size_t)(seq % PEER_RING) * world + rank) * 4;
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(slot), "r"(v) : "memory");
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(slot + 1), "r"(f) : "memory");
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(slot + 2), "r"(seq) : "memory");
  }
}

// ---- the propagator (one warp in the whole grid) --------------------------------------------
// Walks the status words in tile order.  For every contiguous run of published aggregates
// it writes the inclusive prefixes back.  `seed` is the exclusive prefix of tile 0.
// When `shard_out` is given, the warp leaves there what a scan split over several devices
// needs of this shard: {value bits, flag} of the inclusive prefix of the last tile and the
// index of the first tile that contains a segment start (all ones if none does).
template <typename Op>
__device__ void run_propagator(uint64_t *status, uint32_t nt, uint32_t epoch, uint32_t seed, int *failure,
                               uint32_t *shard_out, uint32_t *const *peer_bufs, int peer_rank, int peer_world, uint32_t peer_seq) {
  const int lane = threadIdx.x & 31;
  uint32_t run_v = seed, run_f = 0;     // inclusive prefix of tile pos-1
  uint32_t pos = 0, idle = 0;
  uint32_t first_flagged = 0xffffffffu;
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
    uint32_t tv = Op::kIdentity, tf = 0;    // lane total (identity if the lane has nothing)
#pragma unroll
    for (int q = 0; q < PROP_PER_LANE; q++) {
      if (q < mine) {
        const uint32_t av = status_value(w[q]), af = Op::kHasFlag ? status_flag(w[q]) : 0u;
        if (q == 0) { tv = av; tf = af; } else Op::combine(tv, tf, av, af, tv, tf);
      }
      iv[q] = tv; iflag[q] = tf;
    }
    if (Op::kHasFlag && shard_out != nullptr && first_flagged == 0xffffffffu) {
      uint32_t cand = 0xffffffffu;
#pragma unroll
      for (int q = PROP_PER_LANE - 1; q >= 0; q--)
        if (q < mine && status_flag(w[q])) cand = first + q;
      first_flagged = __reduce_min_sync(kFull, cand);
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
      }
    }
    // new running prefix = inclusive prefix of the last tile of the run
    uint32_t lastv, lastf;
    Op::combine(run_v, run_f, __shfl_sync(kFull, sv, 31), __shfl_sync(kFull, sf, 31), lastv, lastf);
    run_v = lastv; run_f = lastf;
    pos += run;
  }
  if (shard_out != nullptr && lane == 0) {
    shard_out[0] = run_v; shard_out[1] = run_f; shard_out[2] = first_flagged; shard_out[3] = 0u;
    if (peer_bufs != nullptr) push_summary(peer_bufs, peer_rank, peer_world, peer_seq, run_v, run_f);
  }
}

// ---- the persistent tile kernel ------------------------------------------------------------------

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
  const int64_t *d_base;   // compaction of one piece of a longer array: selected keys in the pieces before (device word, or NULL)
  int64_t index_base;      // ... and the index of this piece's first key in the whole array
  int64_t seg_len;         // regular segmented scan: the length of every segment
  // a shard's summary pushed straight into the exchange buffers of the GPUs behind it (or peer_bufs == NULL)
  uint32_t *const *peer_bufs;   // device array [peer_world]: every rank's exchange buffer, peer-mapped
  int peer_rank, peer_world;
  uint32_t peer_seq;            // the call's sequence number (never 0)
  uint32_t *shard_out;     // segmented scan of one shard of a split array: 4 words, see run_propagator (or NULL)
};

// The warp totals of a tile, held in shared memory, folded in warp order by every thread for itself (eight
// broadcast reads and eight combines: a shorter chain than a shuffle scan over the same eight values).
// Returns the tile aggregate in (tv, tf) and the fold of the warps before `warp` in (bv, bf) (the identity
// for warp 0).
template <typename Op>
__device__ __forceinline__ void fold_warp_totals(const uint32_t *s_wv, const uint32_t *s_wf, int lane, int warp,
                                                 uint32_t &tv, uint32_t &tf, uint32_t &bv, uint32_t &bf) {
  static_assert(SCAN_WARPS == 8, "two 16-byte reads per array");
  if (Op::kHasFlag) {
    // (value, flag) pairs: measured slower this way (segmented scan of 2^27 f32: 239 us against 208 us), so
    // these keep the shuffle scan over the first eight lanes
    uint32_t wv = (lane < SCAN_WARPS) ? s_wv[lane] : Op::kIdentity;
    uint32_t wf = (lane < SCAN_WARPS) ? s_wf[lane] : 0u;
#pragma unroll
    for (int o = 1; o < SCAN_WARPS; o <<= 1) {
      const uint32_t lv = __shfl_up_sync(kFull, wv, o), lf = __shfl_up_sync(kFull, wf, o);
      if (lane >= o) Op::combine(lv, lf, wv, wf, wv, wf);
    }
    tv = __shfl_sync(kFull, wv, SCAN_WARPS - 1);
    tf = __shfl_sync(kFull, wf, SCAN_WARPS - 1);
    bv = __shfl_sync(kFull, wv, warp > 0 ? warp - 1 : 0);
    bf = __shfl_sync(kFull, wf, warp > 0 ? warp - 1 : 0);
    if (warp == 0) { bv = Op::kIdentity; bf = 0; }
    return;
  }
  const uint4 v0 = *reinterpret_cast<const uint4 *>(s_wv), v1 = *reinterpret_cast<const uint4 *>(s_wv + 4);
  const uint32_t wv[SCAN_WARPS] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
  uint32_t wf[SCAN_WARPS] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
  if (Op::kHasFlag) {
    const uint4 f0 = *reinterpret_cast<const uint4 *>(s_wf), f1 = *reinterpret_cast<const uint4 *>(s_wf + 4);
    wf[0] = f0.x; wf[1] = f0.y; wf[2] = f0.z; wf[3] = f0.w; wf[4] = f1.x; wf[5] = f1.y; wf[6] = f1.z; wf[7] = f1.w;
  }
  uint32_t av = Op::kIdentity, af = 0u;
  bv = Op::kIdentity; bf = 0u;
#pragma unroll
  for (int w = 0; w < SCAN_WARPS; w++) {
    if (w == warp) { bv = av; bf = af; }
    Op::combine(av, af, wv[w], wf[w], av, af);
  }
  tv = av; tf = af;
}

// Work item w of a launch -> (visit, tile).  The first `lead` items are visit A of tiles
// 0 .. lead-1; then visit A of tile lead+j alternates with visit B of tile j until the
// A visits run out; the remaining B visits follow.  Visit B of tile t is therefore drawn
// after visit A of every tile <= t, and in the steady state `lead` tiles behind the A visits.
struct WorkMap {
  uint32_t nt, lead;
  __device__ __forceinline__ uint32_t total() const { return 2u * nt; }
  __device__ __forceinline__ void decode(uint32_t w, bool &is_a, uint32_t &tile) const {
    if (w < lead) { is_a = true; tile = w; return; }
    const uint32_t k = w - lead, pairs = 2u * (nt - lead);
    if (k < pairs) { is_a = (k & 1u) == 0; tile = is_a ? lead + (k >> 1) : (k >> 1); }
    else { is_a = false; tile = (nt - lead) + (k - pairs); }
  }
};

template <typename S>
__global__ void __launch_bounds__(SCAN_THREADS, S::CTAS)
stream_kernel(const LookbackArgs a) {
  constexpr int V = S::V, ITEMS = TileOf<S>::ITEMS, TILE = TileOf<S>::TILE;
  using Op = typename S::Op;
  constexpr bool SEG = Op::kHasFlag;                   // the operator works on (flag, value) pairs
  constexpr bool HASF = S::kFlagArray;                 // a byte array is loaded with the values
  constexpr bool COMPACT = S::kCompact, PART = S::kPartition;
  constexpr bool ADD = std::is_same<Op, OpAddU32>::value;            // the operator is the wrapping add (counts included)
  constexpr bool REDO = !COMPACT && !SEG && (S::kHasPost || S::kExclusive);   // the second visit folds again from the prefix
  constexpr int FO = TileOf<S>::FO, SB = TileOf<S>::SB;
  // NBUF tile buffers; the tile of iteration it + DIST is fetched while iteration it computes.  What
  // belongs to one iteration (warp totals, prefix, named barriers) lives in slot it % RING: the
  // workers are never more than DIST iterations apart.
  constexpr int NBUF = S::NBUF, DIST = S::DIST, RING = DIST + 1, IR = DIST + 2;
  static_assert(DIST >= 1 && DIST < NBUF && RING <= 4, "ring sizes");
  static_assert(!SEG || HASF || S::kSegRegular, "a flagged operator needs a flag source");
  static_assert(!COMPACT || ADD, "compaction counts with the wrapping add");
  extern __shared__ __align__(128) unsigned char s_buf[];   // the tile buffers
  __shared__ __align__(8) uint64_t s_bar[NBUF];
  __shared__ uint32_t s_item[IR];        // work items of iterations it .. it+DIST+1: tile << 1 | visit A, or ITEM_NONE
  __shared__ __align__(16) uint32_t s_wv[RING][SCAN_WARPS], s_wf[RING][SCAN_WARPS];
  __shared__ uint32_t s_role;
  __shared__ volatile uint32_t s_fail;      // a worker's wait for a tile ran out
  __shared__ uint32_t s_ev[RING], s_ok[RING];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (ld_failure(a.failure) != FAIL_NONE) return;
  const uint32_t nt = a.num_tiles;

  // ---- role: with more than one CTA the first to arrive propagates prefixes, the others work on tiles
  if (tid == 0) {
    const uint32_t r = atomicAdd(&a.ticket[1], 1u);
    if (r == gridDim.x - 1) atomicExch(&a.ticket[1], 0u);     // rewind for the next launch
    s_role = r;
    s_fail = 0;
  }
  __syncthreads();
  uint32_t seed = a.carry_in;
  if (ADD && !COMPACT && a.carry_vals != nullptr)
    for (int q = 0; q < a.carry_n; q++) seed += a.carry_vals[q];
  const int64_t sel_base = (COMPACT && a.d_base != nullptr) ? *a.d_base : 0;   // selected keys in the pieces before this one
  const bool solo = (gridDim.x == 1);    // a lone CTA turns its own aggregates into prefixes
  if (s_role == 0 && !solo) {
    if (warp == 0) run_propagator<Op>(a.status, nt, a.epoch, seed, a.failure, a.shard_out, a.peer_bufs, a.peer_rank, a.peer_world, a.peer_seq);
    return;
  }
  const uint32_t workers = solo ? 1u : gridDim.x - 1;
  WorkMap wm;
  wm.nt = nt;
  wm.lead = nt < (uint32_t)S::LEAD ? nt : (uint32_t)S::LEAD;
  // Every CTA draws work items until it meets one past the end, so the counter ends at
  // total + workers; whoever draws that last value rewinds it for the next launch.
  const uint32_t last_value = wm.total() + workers - 1;
  const bool in_bulk = aligned16(a.in) && (!HASF || aligned16(a.flags));
  const bool out_bulk = !COMPACT && aligned16(a.out);
  constexpr uint32_t ITEM_NONE = 0xffffffffu;

  auto encode = [&](uint32_t w) -> uint32_t {     // work item -> what the threads need of it
    if (w >= wm.total()) return ITEM_NONE;
    bool ia;
    uint32_t t;
    wm.decode(w, ia, t);
    return (t << 1) | (ia ? 1u : 0u);
  };
  auto item_is_bulk = [&](uint32_t item) -> bool {
    return item != ITEM_NONE && in_bulk && ((int64_t)((item >> 1) + 1) * TILE <= a.n);
  };
  // Hands buffer b to the workers for `item`: by the copies' completion, or (no item, a ragged
  // tile, unaligned arrays: the workers copy the tile in themselves) at once.
  // L2 eviction priority (S::kStreamHints): a tile is dead in L2 once its visit B has read it, and the
  // results are written once; marking both "evict first" leaves the room to the tiles that wait between
  // their two visits.  Measured on 2^28 keys: filter 318 -> 308 us, partition 458 -> 431 us (DRAM reads of
  // the partition were 1.67 x the input without it); no effect on the scans, whose window fits anyway.
  const uint64_t pol_first = l2_policy_evict_first();
  auto load_hinted = [&](void *dst, const void *src, uint32_t bytes, uint64_t *bar, bool visit_a) {
    if (S::kStreamHints && !visit_a) bulk_g2s_hint(dst, src, bytes, bar, pol_first);
    else bulk_g2s(dst, src, bytes, bar);
  };
  auto store_hinted = [&](void *gdst, const void *src, uint32_t bytes) {
    if (S::kStreamHints) bulk_s2g_hint(gdst, src, bytes, pol_first);
    else bulk_s2g(gdst, src, bytes);
  };
  auto hand_over = [&](int b, uint32_t item) {
    if (item_is_bulk(item)) {
      unsigned char *dst = s_buf + b * SB;
      const int64_t tb = (int64_t)(item >> 1) * TILE;
      mbar_expect_tx(&s_bar[b], TILE * 4 + (HASF ? TILE : 0));
      load_hinted(dst, reinterpret_cast<const uint32_t *>(a.in) + tb, TILE * 4, &s_bar[b], (item & 1u) != 0);
      if (HASF) load_hinted(dst + FO, a.flags + tb, TILE, &s_bar[b], (item & 1u) != 0);
    } else {
      mbar_arrive(&s_bar[b]);
    }
  };
  auto draw = [&]() -> uint32_t {
    const uint32_t w = atomicAdd(&a.ticket[0], 1u);
    if (w == last_value) atomicExch(&a.ticket[0], 0u);
    return w;
  };
  // set-up by the scheduler's lane 0: the buffers' mbarriers, the first work items and copies
  if (warp == SCAN_WARPS && lane == 0) {
    for (int b = 0; b < NBUF; b++) mbar_init(&s_bar[b], 1);
    fence_mbar_init();
    uint32_t prev = 0;
    for (int k = 0; k <= DIST; k++) {      // a CTA stops drawing at its first item past the end
      prev = (prev != ITEM_NONE) ? encode(draw()) : ITEM_NONE;
      s_item[k] = prev;
    }
    __threadfence_block();
    for (int k = 0; k < DIST; k++) hand_over(k % NBUF, s_item[k]);
  }
  __syncthreads();

  // ================= the scheduler warp =================================================
  // Lane 0 draws the work items (two iterations ahead), starts the bulk async copy (TMA) of the
  // next iteration's tile into the buffer the previous iteration used, fetches the incoming
  // prefix of a visit B, and when the workers are through with the tile publishes its
  // aggregate (visit A) or sends the buffer off (visit B).  The workers never wait for any of
  // that except through the buffer's mbarrier and, in a visit B, for the prefix.
  if (warp == SCAN_WARPS) {
    uint32_t self_v = seed, self_f = 0;    // a lone CTA: running inclusive prefix
    uint32_t self_first = 0xffffffffu;     // ... and the first tile with a segment start
    bool failed = false;                   // lane 0: a wait ran out; draw nothing more
    volatile uint32_t *v_item = s_item;
    for (uint32_t it = 0;; it++) {
      const int r = (int)(it % RING);
      const uint32_t item = __shfl_sync(kFull, v_item[it % IR], 0);
      if (item == ITEM_NONE) break;
      const bool is_a = (item & 1u) != 0;
      const uint32_t tile = item >> 1;
      const int64_t base = (int64_t)tile * TILE;
      const int count = (int)((a.n - base) < TILE ? (a.n - base) : TILE);
      const bool full = (count == TILE);
      uint32_t ahead = ITEM_NONE;          // lane 0: the item DIST iterations on, the newest known
      uint32_t raw = 0xffffffffu, ev = seed, ok = 1;
      if (lane == 0) {
        uint64_t pw = 0;
        ahead = v_item[(it + DIST) % IR];
        if (ahead != ITEM_NONE && !failed) raw = draw();              // the item after that; its round trip to L2 ...
        if (!is_a && tile > 0) pw = ld_status(&a.status[tile - 1]);  // ... and this one overlap the wait below
        // The buffer of iteration it + DIST was last used NBUF iterations earlier: the workers left it
        // before that iteration's last barrier, and the bulk stores since then may still be reading.
        bulk_wait_read<NBUF - 1 - DIST>();
        hand_over((int)((it + DIST) % NBUF), ahead);
        if (!is_a) {
          // the exclusive prefix of the tile (normally there long ago: visit A runs `lead` tiles ahead)
          if (tile > 0) {
            uint32_t polls = 0;
            while (true) {
              const uint32_t st = status_state(pw, a.epoch);
              if (st == ST_PREFIX || (SEG && st == ST_AGG && status_flag(pw))) break;
              polls++;
              if ((polls & 63u) == 0 && (ld_failure(a.failure) != FAIL_NONE || polls >= WAIT_MAX_ROUNDS)) {
                atomicCAS(a.failure, FAIL_NONE, FAIL_LOOKBACK_TIMEOUT);
                ok = 0;
                break;
              }
              if (polls > 4) __nanosleep(polls > 64 ? 200 : 40);
              pw = ld_status(&a.status[tile - 1]);
            }
            ev = status_value(pw);
          }
          s_ev[r] = ev; s_ok[r] = ok;
          __threadfence_block();
        }
      }
      __syncwarp();
      if (!is_a) bar_arrive<BAR_MID, SCAN_THREADS>(r);     // the prefix is there
      bar_sync<BAR_DONE, SCAN_THREADS>(r);                 // the workers are through with the buffer
      ok = __shfl_sync(kFull, ok, 0);
      if (s_fail) ok = 0;
      uint32_t tv, tf, bv, bf;
      fold_warp_totals<Op>(s_wv[r], s_wf[r], lane, 0, tv, tf, bv, bf);
      uint32_t *s_tile = reinterpret_cast<uint32_t *>(s_buf + (it % NBUF) * SB);
      if (is_a) {
        if (lane == 0) {
          if (solo) {
            if (SEG && tf && self_first == 0xffffffffu) self_first = tile;
            Op::combine(self_v, self_f, tv, tf, self_v, self_f);
            st_status(&a.status[tile], pack_status(self_v, a.epoch, self_f, ST_PREFIX));
          } else {
            st_status(&a.status[tile], pack_status(tv, a.epoch, tf, ST_AGG));
          }
        }
      } else if (!COMPACT) {
        if (ok && full && out_bulk && lane == 0) {
          store_hinted(reinterpret_cast<uint32_t *>(a.out) + base, s_tile, TILE * 4);
          bulk_commit();
        }
      } else if (ok) {
        // Each run leaves as one bulk store of its 16-byte aligned body, issued by lane 0, plus up
        // to three keys in front and behind, stored by the other lanes.  (Same arithmetic as the
        // workers' staging below.)
        ev = __shfl_sync(kFull, ev, 0);
        const uint32_t tile_true = tv;
        const int64_t true_before = sel_base + (int64_t)ev;
        uint32_t *dst = reinterpret_cast<uint32_t *>(a.out) + true_before;
        uint32_t *dstf = PART ? a.out_false + (a.index_base + base - true_before) : nullptr;
        const uint32_t pad_t = (uint32_t)((reinterpret_cast<uintptr_t>(dst) >> 2) & 3u);
        const uint32_t pad_f = PART ? (uint32_t)((reinterpret_cast<uintptr_t>(dstf) >> 2) & 3u) : 0u;
        const uint32_t start_f = ((pad_t + tile_true + 3u) & ~3u) + pad_f;
        auto send_run = [&](uint32_t *g, uint32_t s0, uint32_t len, int lane0) {
          // g and s_tile + s0 are congruent modulo 16 bytes
          uint32_t h = (4u - (s0 & 3u)) & 3u;
          if (h > len) h = len;
          const uint32_t nvec = (len - h) >> 2, tail0 = h + (nvec << 2);
          const uint32_t l = (uint32_t)(lane - lane0);               // lanes lane0 .. lane0+2 take the ends
          if (l < h) g[l] = s_tile[s0 + l];
          if (l < len - tail0) g[tail0 + l] = s_tile[s0 + tail0 + l];
          if (lane == 0 && nvec > 0) store_hinted(g + h, s_tile + s0 + h, nvec << 4);
        };
        send_run(dst, pad_t, tile_true, 0);
        if (PART) send_run(dstf, start_f, (uint32_t)count - tile_true, 4);
        if (lane == 0) bulk_commit();
        __syncwarp();                      // lane 0 fills the buffer again only after these lanes have read their keys
        if (tile == nt - 1 && lane == 0) *a.d_count = true_before + (int64_t)tile_true;
      }
      if (lane == 0) {
        if (!ok) failed = true;
        const uint32_t drawn = (ahead != ITEM_NONE && !failed) ? encode(raw) : ITEM_NONE;
        v_item[(it + DIST + 1) % IR] = drawn;      // (the slot of the previous iteration's item)
        __threadfence_block();
      }
    }
    if (lane == 0) {
      if (solo && a.shard_out != nullptr && !failed) {
        a.shard_out[0] = self_v; a.shard_out[1] = self_f; a.shard_out[2] = self_first; a.shard_out[3] = 0u;
        if (a.peer_bufs != nullptr) push_summary(a.peer_bufs, a.peer_rank, a.peer_world, a.peer_seq, self_v, self_f);
      }
      bulk_wait_read0();                   // shared memory must outlive the last bulk store's reads
    }
    return;
  }

  // ================= the worker warps =====================================================
  for (uint32_t it = 0;; it++) {
    const int nb = (int)(it % NBUF), r = (int)(it % RING);
    // the buffer is ours once its mbarrier completes (once every NBUF iterations); the iteration's
    // item was written before that
    if (!mbar_wait_bounded(&s_bar[nb], (it / NBUF) & 1u)) {
      atomicCAS(a.failure, FAIL_NONE, FAIL_BULK_COPY_TIMEOUT);
      s_fail = 1;
    }
    const uint32_t item = reinterpret_cast<volatile uint32_t *>(s_item)[it % IR];
    if (item == ITEM_NONE) break;
    const bool is_a = (item & 1u) != 0;
    const uint32_t tile = item >> 1;

    // ---- the tile: in the buffer, by the bulk copy or (ragged / unaligned) copied in by the threads
    unsigned char *buf = s_buf + nb * SB;
    uint32_t *s_tile = reinterpret_cast<uint32_t *>(buf);
    const int64_t base = (int64_t)tile * TILE;
    const int count = (int)((a.n - base) < TILE ? (a.n - base) : TILE);
    const bool full = (count == TILE);
    if (!(full && in_bulk)) {
      const uint32_t *gin = reinterpret_cast<const uint32_t *>(a.in) + base;
      for (int i = tid; i < TILE; i += SCAN_WORKERS) s_tile[i] = (i < count) ? gin[i] : 0u;     // (what lies past `count` is masked below)
      if (HASF) {
        unsigned char *sfb = buf + FO;
        for (int i = tid; i < TILE; i += SCAN_WORKERS) sfb[i] = (i < count) ? a.flags[base + i] : (unsigned char)0;
      }
      fence_proxy_async_smem();          // a later bulk copy lands in this buffer: order it after these stores
      bar_sync<BAR_WORKERS, SCAN_WORKERS>();
    }
    // A thread owns ITEMS consecutive elements = V 16-byte vectors; V is odd, so the 128-bit
    // shared-memory accesses of a warp are conflict-free.
    uint32_t x[ITEMS];
    {
      const int4 *s4 = reinterpret_cast<const int4 *>(s_tile) + tid * V;
#pragma unroll
      for (int j = 0; j < V; j++) {
        const int4 q = s4[j];
        x[4 * j + 0] = q.x; x[4 * j + 1] = q.y; x[4 * j + 2] = q.z; x[4 * j + 3] = q.w;
      }
    }
    using mask_t = typename std::conditional<(ITEMS > 32), unsigned long long, uint32_t>::type;
    static_assert(ITEMS <= 64 && (SEG ? ITEMS <= 32 : true), "one bit per element of the thread");
    // elements of this thread that exist (the last tile may be ragged)
    const int valid = full ? ITEMS : (count - tid * ITEMS < 0 ? 0 : (count - tid * ITEMS > ITEMS ? ITEMS : count - tid * ITEMS));
    mask_t bits = 0;                     // segment starts (segmented scan) / selected keys (compaction)
    uint32_t tv_thread, tf_thread = 0;   // the thread's aggregate
    uint32_t fw[HASF ? V : 1];           // the thread's flag bytes
    if (HASF) {
      const uint32_t *sf = reinterpret_cast<const uint32_t *>(buf + FO) + tid * V;
#pragma unroll
      for (int j = 0; j < V; j++) fw[j] = sf[j];
    }
    if (COMPACT) {
#pragma unroll
      for (int q = 0; q < ITEMS; q++) {
        const uint32_t fl = HASF ? (fw[q >> 2] >> (8 * (q & 3))) & 0xffu : 0u;
        if (S::pred(x[q], fl)) bits |= (mask_t)1 << q;
      }
      if (!full) bits &= (valid >= ITEMS) ? ~(mask_t)0 : (((mask_t)1 << valid) - 1);
      tv_thread = (ITEMS > 32) ? (uint32_t)__popcll((unsigned long long)bits) : (uint32_t)__popc((uint32_t)bits);
    } else {
      // the map body, and the neutral element behind the end of a ragged tile
      if (!REDO) {                                   // (REDO keeps the elements for the post-operation and maps on the fly)
#pragma unroll
        for (int q = 0; q < ITEMS; q++) x[q] = S::map(x[q]);
      }
      if (!full) {                                   // only the last tile: nothing of this on the common path
#pragma unroll
        for (int q = 0; q < ITEMS; q++)
          if (q >= valid) x[q] = Op::kIdentity;
      }
      if (SEG) {
        // head flags: from the byte array, or computed from the position inside the regular segment
        int64_t pos = 0;
        if (S::kSegRegular) pos = (base + (int64_t)tid * ITEMS) % a.seg_len;
        uint32_t acc = Op::kIdentity, accf = 0;
        if (is_a) {
          // only the thread's aggregate is wanted: no record of where the segments start, nothing kept per element
#pragma unroll
          for (int q = 0; q < ITEMS; q++) {
            bool fl;
            if (S::kSegRegular) { fl = (pos == 0); pos = (pos + 1 == a.seg_len) ? 0 : pos + 1; }
            else fl = ((fw[q >> 2] >> (8 * (q & 3))) & 0xffu) != 0;
            Op::combine(acc, accf, x[q], fl ? 1u : 0u, acc, accf);
          }
          tv_thread = acc;
          tf_thread = accf;
        } else {
#pragma unroll
          for (int q = 0; q < ITEMS; q++) {
            bool fl;
            if (S::kSegRegular) { fl = (pos == 0); pos = (pos + 1 == a.seg_len) ? 0 : pos + 1; }
            else fl = ((fw[q >> 2] >> (8 * (q & 3))) & 0xffu) != 0;
            if (fl) bits |= (mask_t)1 << q;
            Op::combine(acc, accf, x[q], fl ? 1u : 0u, acc, accf);
            x[q] = acc;
          }
          tv_thread = acc;
          tf_thread = bits ? 1u : 0u;
        }
      } else if (is_a || REDO) {
        // (a ragged tile is the last one: its test of every element is kept off the common path)
        auto fold = [&](auto ragged) {
          uint32_t s = REDO ? S::map(x[0]) : x[0], sf = 0;
          if (REDO && decltype(ragged)::value && valid < 1) s = Op::kIdentity;
#pragma unroll
          for (int q = 1; q < ITEMS; q++) {
            uint32_t y = REDO ? S::map(x[q]) : x[q];
            if (REDO && decltype(ragged)::value && q >= valid) y = Op::kIdentity;
            Op::combine(s, sf, y, 0u, s, sf);
          }
          return s;
        };
        tv_thread = (REDO && !full) ? fold(std::true_type{}) : fold(std::false_type{});
      } else {
        uint32_t sf = 0;
#pragma unroll
        for (int q = 1; q < ITEMS; q++) Op::combine(x[q - 1], 0u, x[q], 0u, x[q], sf);
        tv_thread = x[ITEMS - 1];
      }
    }
    uint32_t xv = Op::kIdentity, xf = 0; // what precedes this thread inside its warp
    if (ADD && is_a) {
      // only the tile's aggregate is wanted, and the order does not matter
      const uint32_t t = warp_sum(tv_thread);
      if (lane == 31) s_wv[r][warp] = t;
    } else {
      // scan of the thread aggregates across the warp
      uint32_t iv = tv_thread, ifl = tf_thread;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t lv = __shfl_up_sync(kFull, iv, o);
        const uint32_t lf = SEG ? __shfl_up_sync(kFull, ifl, o) : 0u;
        if (lane >= o) Op::combine(lv, lf, iv, ifl, iv, ifl);
      }
      xv = __shfl_up_sync(kFull, iv, 1); xf = SEG ? __shfl_up_sync(kFull, ifl, 1) : 0u;
      if (lane == 0) { xv = Op::kIdentity; xf = 0; }
      if (lane == 31) { s_wv[r][warp] = iv; if (SEG) s_wf[r][warp] = ifl; }
    }
    if (is_a) {
      // the scheduler folds the warp totals and publishes the aggregate; nobody waits here
      __threadfence_block();
      bar_arrive<BAR_DONE, SCAN_THREADS>(r);
      continue;
    }
    bar_sync<BAR_MID, SCAN_THREADS>(r);         // all warp totals and the tile's incoming prefix are there
    if (s_ok[r]) {         // (set by the scheduler before the barrier: the same for every worker)
      uint32_t tv, tf, bv, bf;
      fold_warp_totals<Op>(s_wv[r], s_wf[r], lane, warp, tv, tf, bv, bf);
      const uint32_t ev = s_ev[r];
      uint32_t lv, lf;
      Op::combine(bv, bf, xv, xf, lv, lf);                           // what precedes this thread inside the tile
      if (!COMPACT) {
        // what precedes this thread: the tile's incoming prefix, then its left neighbours
        uint32_t pv, pf;
        Op::combine(ev, 0u, lv, lf, pv, pf);
        if (SEG) {
          // only the elements in front of the thread's first segment start take it: element q does if no
          // start lies at or before it (one test of the start bits against a constant mask)
#pragma unroll
          for (int q = 0; q < ITEMS; q++) {
            if (((uint32_t)bits & ((2u << q) - 1u)) == 0u) {
              uint32_t of;
              Op::combine(pv, pf, x[q], 0u, x[q], of);
            }
          }
        } else if (REDO) {
          // fold once more, from the prefix: element q receives post(scan up to q, element q); for
          // an exclusive scan, the scan up to q - 1
          auto refold = [&](auto ragged) {
            uint32_t sv = pv, sf = 0;
#pragma unroll
            for (int q = 0; q < ITEMS; q++) {
              uint32_t y = S::map(x[q]);
              if (decltype(ragged)::value && q >= valid) y = Op::kIdentity;
              if (S::kExclusive) { const uint32_t o = S::post(sv, x[q]); Op::combine(sv, sf, y, 0u, sv, sf); x[q] = o; }
              else { Op::combine(sv, sf, y, 0u, sv, sf); x[q] = S::post(sv, x[q]); }
            }
          };
          if (full) refold(std::false_type{}); else refold(std::true_type{});
        } else {
#pragma unroll
          for (int q = 0; q < ITEMS; q++) { uint32_t of; Op::combine(pv, 0u, x[q], 0u, x[q], of); }
        }
        int4 *s4 = reinterpret_cast<int4 *>(s_tile) + tid * V;
#pragma unroll
        for (int j = 0; j < V; j++) {
          int4 q; q.x = x[4 * j + 0]; q.y = x[4 * j + 1]; q.z = x[4 * j + 2]; q.w = x[4 * j + 3];
          s4[j] = q;
        }
        if (!(full && out_bulk)) {
          // ragged tile or unaligned result: the threads copy it out themselves
          uint32_t *gout = reinterpret_cast<uint32_t *>(a.out) + base;
          bar_sync<BAR_WORKERS, SCAN_WORKERS>();
          for (int i = tid; i < count; i += SCAN_WORKERS) gout[i] = s_tile[i];
        }
      } else {
        // Keys back into the buffer, selected first, each group in order; the scheduler sends the
        // runs.  Each group is staged at the same offset modulo 4 as its destination, so that the
        // body of a run moves as aligned 16-byte vectors on both sides.
        const uint32_t tile_true = tv;
        const int64_t true_before = sel_base + (int64_t)ev;         // selected keys in earlier tiles (and pieces); a piece has < 2^31 keys
        uint32_t *dst = reinterpret_cast<uint32_t *>(a.out) + true_before;
        uint32_t *dstf = PART ? a.out_false + (a.index_base + base - true_before) : nullptr;
        const uint32_t pad_t = (uint32_t)((reinterpret_cast<uintptr_t>(dst) >> 2) & 3u);
        const uint32_t pad_f = PART ? (uint32_t)((reinterpret_cast<uintptr_t>(dstf) >> 2) & 3u) : 0u;
        const uint32_t start_f = ((pad_t + tile_true + 3u) & ~3u) + pad_f;     // first rejected key in the buffer
        uint32_t rank = lv;
        const uint32_t first_ord = (uint32_t)tid * ITEMS;
        if (full) {
#pragma unroll
          for (int q = 0; q < ITEMS; q++) {
            if ((bits >> q) & 1u) s_tile[pad_t + rank++] = x[q];
            else if (PART) s_tile[start_f + first_ord + q - rank] = x[q];
          }
        } else {                                     // the last tile: keys past the end are not staged
#pragma unroll
          for (int q = 0; q < ITEMS; q++) {
            if ((bits >> q) & 1u) s_tile[pad_t + rank++] = x[q];
            else if (PART && first_ord + q < (uint32_t)count) s_tile[start_f + first_ord + q - rank] = x[q];
          }
        }
      }
    }
    // what the threads wrote is read by the scheduler's bulk store, and the buffer is filled again by a bulk copy
    fence_proxy_async_smem();
    __threadfence_block();
    bar_arrive<BAR_DONE, SCAN_THREADS>(r);
  }
}

// ---- host launchers --------------------------------------------------------------------

template <typename S>
static inline uint32_t tiles_for(int64_t n) { return (uint32_t)((n + TileOf<S>::TILE - 1) / TileOf<S>::TILE); }

size_t lookback_scratch_bytes(int64_t n) {
  return 256 + (size_t)((n + SCAN_TILE_MIN - 1) / SCAN_TILE_MIN) * sizeof(uint64_t);
}

static inline void split_scratch(void *scratch, uint32_t **ticket, uint64_t **status) {
  *ticket = reinterpret_cast<uint32_t *>(scratch);
  *status = reinterpret_cast<uint64_t *>(reinterpret_cast<char *>(scratch) + 256);
}

// Grid of the persistent kernel: what is resident at once (occupancy x SMs) and at most one
// worker per tile, plus the propagator.  The occupancy query allocates nothing and is
// cached per specification and device.
template <typename S>
static cudaError_t launch_stream(LookbackArgs a, cudaStream_t stream, int grid_cap = 0) {
  constexpr int TILE = TileOf<S>::TILE;
  constexpr size_t smem = (size_t)S::NBUF * TileOf<S>::SB;
  static int ctas_per_sm_dev[64], num_sms_dev[64];     // per device ordinal (function attributes are per device)
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= 63;
  int &ctas_per_sm = ctas_per_sm_dev[dev], &num_sms = num_sms_dev[dev];
  if (ctas_per_sm == 0) {
    cudaError_t err = cudaFuncSetAttribute(stream_kernel<S>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return err;
    int occ = 0, sms = 0;
    err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (err != cudaSuccess) return err;
    err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, stream_kernel<S>, SCAN_THREADS, smem);
    if (err != cudaSuccess) return err;
    if (occ < 1) return cudaErrorLaunchOutOfResources;
    num_sms = sms;
    ctas_per_sm = occ;
  }
  const uint32_t resident = (uint32_t)(ctas_per_sm * num_sms);
  uint32_t grid = 2 * a.num_tiles + 1 < resident ? 2 * a.num_tiles + 1 : resident;
  if (grid_cap >= 2 && (uint32_t)grid_cap < grid) grid = (uint32_t)grid_cap;   // the <entry>.segscan_num_tblocks tuning parameter
  if (a.num_tiles <= 1 || grid < 2) grid = 1;          // a single tile: one CTA that propagates for itself
  stream_kernel<S><<<grid, SCAN_THREADS, smem, stream>>>(a);
  return cudaGetLastError();
}

template <typename S>
static LookbackArgs make_args(const void *in, const uint8_t *flags, void *out, uint32_t *out_false, int64_t n,
                              void *scratch, uint32_t epoch, int *failure) {
  LookbackArgs a;
  a.in = in; a.flags = flags; a.out = out; a.out_false = out_false; a.n = n;
  a.num_tiles = tiles_for<S>(n);
  split_scratch(scratch, &a.ticket, &a.status);
  a.epoch = epoch; a.failure = failure;
  a.carry_in = S::kCompact ? 0u : S::Op::kIdentity; a.carry_vals = nullptr; a.carry_n = 0; a.d_count = nullptr; a.shard_out = nullptr;
  a.d_base = nullptr; a.index_base = 0; a.seg_len = 1;
  a.peer_bufs = nullptr; a.peer_rank = 0; a.peer_world = 0; a.peer_seq = 0;
  return a;
}

cudaError_t launch_scan_i32(const int32_t *in, int32_t *out, int64_t n, int32_t carry_in,
                            const int32_t *carry_vals, int carry_n, void *scratch,
                            uint32_t epoch, int *failure, cudaStream_t stream, int grid_cap) {
  if (n <= 0) return cudaSuccess;
  LookbackArgs a = make_args<SpecScanAddI32>(in, nullptr, out, nullptr, n, scratch, epoch, failure);
  a.carry_in = (uint32_t)carry_in;
  a.carry_vals = reinterpret_cast<const uint32_t *>(carry_vals);
  a.carry_n = carry_n;
  return launch_stream<SpecScanAddI32>(a, stream, grid_cap);
}

// Scans that differ from the above only in their specification: 0 exclusive (+), 1 inclusive max,
// 2 the scanomap step of tests/soacs/scan4.fut, seeded with seed_host plus the device value at `seed` (may be NULL).
cudaError_t launch_scan_variant_i32(int variant, const int32_t *in, int32_t *out, int64_t n, int32_t seed_host, const int32_t *seed,
                                    void *scratch, uint32_t epoch, int *failure, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  switch (variant) {
    case 0: return launch_stream<SpecExscanAddI32>(make_args<SpecExscanAddI32>(in, nullptr, out, nullptr, n, scratch, epoch, failure), stream);
    case 1: return launch_stream<SpecScanMaxI32>(make_args<SpecScanMaxI32>(in, nullptr, out, nullptr, n, scratch, epoch, failure), stream);
    case 2: {
      LookbackArgs a = make_args<SpecScanomapStepI32>(in, nullptr, out, nullptr, n, scratch, epoch, failure);
      a.carry_in = (uint32_t)seed_host;
      a.carry_vals = reinterpret_cast<const uint32_t *>(seed);
      a.carry_n = seed != nullptr ? 1 : 0;
      return launch_stream<SpecScanomapStepI32>(a, stream);
    }
    default: return cudaErrorInvalidValue;
  }
}

cudaError_t launch_exscan_i32(const int32_t *in, int32_t *out, int64_t n, void *scratch,
                              uint32_t epoch, int *failure, cudaStream_t stream) {
  return launch_scan_variant_i32(0, in, out, n, 0, nullptr, scratch, epoch, failure, stream);
}

// map (scan (+) 0) over [rows][cols] i32: one scan over rows * cols elements whose head flags are
// computed from the index (SegScan/SinglePass.hs:471-482, 594-599).
cudaError_t launch_segscan_rows_i32(const int32_t *in, int32_t *out, int64_t rows, int64_t cols, void *scratch,
                                    uint32_t epoch, int *failure, cudaStream_t stream) {
  if (rows * cols <= 0) return cudaSuccess;
  LookbackArgs a = make_args<SpecSegRowsAddI32>(in, nullptr, out, nullptr, rows * cols, scratch, epoch, failure);
  a.seg_len = cols;
  return launch_stream<SpecSegRowsAddI32>(a, stream);
}

// ---- pieces of a segmented scan whose array is split across several devices ---------------
// A shard's scan leaves a 4-word summary (see run_propagator): {value bits, flag} of its last
// inclusive prefix, and the index of its first tile that holds a segment start.  An empty
// shard has the identity (0, no flag, no such tile).
__global__ void shard_identity_kernel(uint32_t *dst, uint32_t *const *peer_bufs, int rank, int world, uint32_t seq) {
  dst[0] = 0u; dst[1] = 0u; dst[2] = 0xffffffffu; dst[3] = 0u;
  if (peer_bufs != nullptr) push_summary(peer_bufs, rank, world, seq, 0u, 0u);
}

cudaError_t launch_segscan_f32(const uint8_t *flags, const float *in, float *out, int64_t n, float carry_in,
                               uint32_t *shard_out, void *scratch, uint32_t epoch, int *failure, cudaStream_t stream, int grid_cap,
                               const PeerPush *peer) {
  if (n <= 0) {
    if (shard_out != nullptr) {
      shard_identity_kernel<<<1, 1, 0, stream>>>(shard_out, peer ? peer->bufs : nullptr, peer ? peer->rank : 0, peer ? peer->world : 0,
                                                 peer ? peer->seq : 0u);
      return cudaGetLastError();
    }
    return cudaSuccess;
  }
  LookbackArgs a = make_args<SpecSegScanAddF32>(in, flags, out, nullptr, n, scratch, epoch, failure);
  uint32_t bits;
  memcpy(&bits, &carry_in, 4);
  a.carry_in = bits;
  a.shard_out = shard_out;
  if (peer != nullptr && shard_out != nullptr) { a.peer_bufs = peer->bufs; a.peer_rank = peer->rank; a.peer_world = peer->world; a.peer_seq = peer->seq; }
  return launch_stream<SpecSegScanAddF32>(a, stream, grid_cap);
}

// out[i] = carry + out[i] for every i before the shard's first segment start, where carry is
// the fold of the summaries of the shards before this one under the lifted operator.  The
// summary of this shard names the first tile with a segment start: everything before that
// tile takes the carry (grid-stride, 16-byte vectors where the array allows), and the last
// CTA finds the start inside that one tile and finishes the elements in front of it.
// With peer_seq != 0 the summaries of the shards in front are not gathered by a collective: the
// GPUs that hold them write them into this GPU's exchange buffer (push_summary), and thread 0 of
// every CTA waits, bounded, until the sequence number of each has arrived.  `summaries` then is the
// generation of the ring this call uses, `own` the shard's own 4-word summary.
__global__ void __launch_bounds__(256)
apply_carry_kernel(float *__restrict__ out, const uint8_t *__restrict__ flags, int64_t n, const uint32_t *summaries, const uint32_t *own,
                   int rank, uint32_t peer_seq, int *failure) {
  constexpr int64_t TILE = TileOf<SpecSegScanAddF32>::TILE;
  __shared__ int s_first;
  __shared__ uint32_t s_cv, s_ok;
  if (peer_seq != 0u) {
    if (threadIdx.x == 0) {
      uint32_t cv = 0, cf = 0, ok = 1;
      for (int q = 0; q < rank && ok; q++) {
        const uint32_t *slot = summaries + 4 * q;
        uint32_t polls = 0, got = 0;
        while (true) {
          asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(got) : "l"(slot + 2) : "memory");
          if (got == peer_seq) break;
          polls++;
          if ((polls & 255u) == 0 && (ld_failure(failure) != FAIL_NONE || polls >= (1u << 21))) {
            atomicCAS(failure, FAIL_NONE, FAIL_PEER_TIMEOUT);
            ok = 0;
            break;
          }
          __nanosleep(polls > 32 ? 500 : 50);
        }
        if (ok) OpSegAddF32::combine(cv, cf, slot[0], slot[1], cv, cf);
      }
      s_cv = cv; s_ok = ok;
    }
    __syncthreads();
    if (!s_ok) return;
  } else if (threadIdx.x == 0) {
    uint32_t cv = 0, cf = 0;
    for (int q = 0; q < rank; q++) OpSegAddF32::combine(cv, cf, summaries[4 * q], summaries[4 * q + 1], cv, cf);
    s_cv = cv;
  }
  __syncthreads();
  const float carry = __uint_as_float(s_cv);
  const uint32_t ft = own[2];
  const int64_t tile_lo = (ft == 0xffffffffu || (int64_t)ft * TILE > n) ? n : (int64_t)ft * TILE;
  const int64_t gtid = (int64_t)blockIdx.x * 256 + threadIdx.x, stride = (int64_t)gridDim.x * 256;
  if (aligned16(out)) {
    float4 *o4 = reinterpret_cast<float4 *>(out);
    const int64_t nv = tile_lo >> 2;
    for (int64_t i = gtid; i < nv; i += stride) {
      float4 v = o4[i];
      v.x = carry + v.x; v.y = carry + v.y; v.z = carry + v.z; v.w = carry + v.w;
      o4[i] = v;
    }
    for (int64_t i = (nv << 2) + gtid; i < tile_lo; i += stride) out[i] = carry + out[i];
  } else {
    for (int64_t i = gtid; i < tile_lo; i += stride) out[i] = carry + out[i];
  }
  if (blockIdx.x == gridDim.x - 1 && tile_lo < n) {
    const int count = (int)((n - tile_lo) < TILE ? (n - tile_lo) : TILE);
    if (threadIdx.x == 0) s_first = count;
    __syncthreads();
    for (int i = threadIdx.x; i < count; i += 256)
      if (flags[tile_lo + i]) { atomicMin(&s_first, i); break; }
    __syncthreads();
    const int first = s_first;
    for (int i = threadIdx.x; i < first; i += 256) out[tile_lo + i] = carry + out[tile_lo + i];
  }
}

cudaError_t launch_segscan_apply_carry(float *out, const uint8_t *flags, int64_t n, const uint32_t *summaries,
                                       int rank, int num_sms, cudaStream_t stream) {
  if (n <= 0 || rank <= 0) return cudaSuccess;
  apply_carry_kernel<<<num_sms * 4, 256, 0, stream>>>(out, flags, n, summaries, summaries + 4 * rank, rank, 0u, nullptr);
  return cudaGetLastError();
}

cudaError_t launch_segscan_apply_carry_peer(float *out, const uint8_t *flags, int64_t n, const uint32_t *my_buf, const uint32_t *own, int rank,
                                            int world, uint32_t seq, int *failure, int num_sms, cudaStream_t stream) {
  if (n <= 0 || rank <= 0) return cudaSuccess;
  const uint32_t *generation = my_buf + (size_t)(seq % PEER_RING) * world * 4;
  apply_carry_kernel<<<num_sms * 4, 256, 0, stream>>>(out, flags, n, generation, own, rank, seq, failure);
  return cudaGetLastError();
}

size_t peer_exchange_bytes(int world) { return (size_t)PEER_RING * world * 16; }

// Compaction of n 4-byte keys under the predicate `which` (COMPACT_* of kernels.h).  Pieces of
// at most 2^30 keys are launched one behind the other: inside a piece ranks are 32-bit, across
// pieces the number of keys selected so far travels in *d_count (a 64-bit device word), so the
// count is 64-bit like the reference's (prelude/soacs.fut:241-253).  `epochs` holds one fresh
// epoch per piece (compact_pieces_needed(n) of them).
template <typename S>
static cudaError_t compact_pieces(const uint32_t *in, const uint8_t *flags, uint32_t *out_true, uint32_t *out_false, int64_t n,
                                  int64_t *d_count, void *scratch, const uint32_t *epochs, int *failure, cudaStream_t stream) {
  constexpr int64_t PIECE = (int64_t)1 << 30;
  cudaError_t err = cudaSuccess;
  for (int64_t lo = 0; lo < n && err == cudaSuccess; lo += PIECE) {
    const int64_t len = n - lo < PIECE ? n - lo : PIECE;
    LookbackArgs a = make_args<S>(in + lo, flags != nullptr ? flags + lo : nullptr, out_true, out_false, len, scratch, epochs[lo >> 30], failure);
    a.d_count = d_count;
    a.d_base = lo > 0 ? d_count : nullptr;
    a.index_base = lo;
    err = launch_stream<S>(a, stream);
  }
  return err;
}

int compact_pieces_needed(int64_t n) { return n <= 0 ? 1 : (int)((n + ((int64_t)1 << 30) - 1) >> 30); }

cudaError_t launch_compact(int which, const void *in, const uint8_t *flags, void *out_true, void *out_false,
                           int64_t n, int64_t *d_count, void *scratch, const uint32_t *epochs, int *failure, cudaStream_t stream) {
  if (n <= 0) return cudaMemsetAsync(d_count, 0, sizeof(int64_t), stream);
  const uint32_t *k = reinterpret_cast<const uint32_t *>(in);
  uint32_t *t = reinterpret_cast<uint32_t *>(out_true), *f = reinterpret_cast<uint32_t *>(out_false);
  switch (which) {
    case COMPACT_FILTER_LOW3_U32: return compact_pieces<SpecFilterLow3U32>(k, nullptr, t, f, n, d_count, scratch, epochs, failure, stream);
    case COMPACT_PARTITION_LOW3_U32: return compact_pieces<SpecPartitionLow3U32>(k, nullptr, t, f, n, d_count, scratch, epochs, failure, stream);
    case COMPACT_FILTER_POS_I32: return compact_pieces<SpecFilterPosI32>(k, nullptr, t, f, n, d_count, scratch, epochs, failure, stream);
    case COMPACT_PARTITION_EVEN_I32: return compact_pieces<SpecPartitionEvenI32>(k, nullptr, t, f, n, d_count, scratch, epochs, failure, stream);
    case COMPACT_PARTITION_DIV3_I32: return compact_pieces<SpecPartitionDiv3I32>(k, nullptr, t, f, n, d_count, scratch, epochs, failure, stream);
    case COMPACT_FILTER_BY_FLAG_I32: return compact_pieces<SpecFilterByFlagI32>(k, flags, t, f, n, d_count, scratch, epochs, failure, stream);
    default: return cudaErrorInvalidValue;
  }
}

// ---- classes of a three-way partition of pairs ----------------------------------------------------
// partition2 (\(x, y) -> x < y) (\(x, y) -> x == y) (zip xs ys) (tests/soacs/partition2.fut;
// prelude/soacs.fut:293-323): the class of a pair is written as three keep-flag arrays, `pitch`
// bytes apart, and each component of each group is then one filter by flags.
__global__ void __launch_bounds__(256)
classify_pairs_lt_eq_kernel(const int32_t *__restrict__ xs, const int32_t *__restrict__ ys, int64_t n, int64_t pitch,
                            uint8_t *__restrict__ keep) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const int32_t x = xs[i], y = ys[i];
    const int cls = x < y ? 0 : (x == y ? 1 : 2);
    keep[i] = cls == 0;
    keep[pitch + i] = cls == 1;
    keep[2 * pitch + i] = cls == 2;
  }
}

cudaError_t launch_classify_pairs_lt_eq(const int32_t *xs, const int32_t *ys, int64_t n, int64_t pitch, uint8_t *keep, int num_sms,
                                        cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  int64_t want = (n + 255) / 256;
  const int64_t cap = (int64_t)num_sms * 8;
  classify_pairs_lt_eq_kernel<<<(int)(want < cap ? want : cap), 256, 0, stream>>>(xs, ys, n, pitch, keep);
  return cudaGetLastError();
}

// ---- a wait that runs out, on purpose -------------------------------------------------------------
// One warp waits, as visit B of a tile does, for a status word that nothing will publish
// under this epoch, with a small poll limit; when the limit is reached it records
// FAIL_LOOKBACK_TIMEOUT in the failure word and returns.  This is how the failure protocol
// (failure word -> futhark_context_sync -> FUTHARK_PROGRAM_ERROR -> scratch reset) is exercised
// on a GPU without faulting, trapping or hanging anything.
__global__ void expire_wait_kernel(const uint64_t *status, uint32_t epoch, uint32_t max_polls, int *failure) {
  if (threadIdx.x != 0) return;
  for (uint32_t polls = 0; polls < max_polls; polls++) {
    if (status_state(ld_status(status), epoch) != ST_NONE) return;      // never happens: nobody publishes under this epoch
    __nanosleep(100);
  }
  atomicCAS(failure, FAIL_NONE, FAIL_LOOKBACK_TIMEOUT);
}

cudaError_t launch_expire_wait(void *scratch, uint32_t epoch, uint32_t max_polls, int *failure, cudaStream_t stream) {
  uint32_t *ticket; uint64_t *status;
  split_scratch(scratch, &ticket, &status);
  expire_wait_kernel<<<1, 32, 0, stream>>>(status, epoch, max_polls > 100000u ? 100000u : max_polls, failure);
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
constexpr uint32_t NOALLOC_MAX_TILES = (uint32_t)((NOALLOC_MAX_N + TileOf<SpecScanAddI32>::TILE - 1) / TileOf<SpecScanAddI32>::TILE);
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
  // Visit B of a tile stores while visit A of later tiles still reads: the scan is not safe in place.
  if (n > 0) {
    const uintptr_t ib = reinterpret_cast<uintptr_t>(in), ob = reinterpret_cast<uintptr_t>(out);
    const uintptr_t bytes = (uintptr_t)n * sizeof(int32_t);
    if (ib < ob + bytes && ob < ib + bytes)
      return fail(1, "futhark_b200_scan_i32_noalloc: `in` and `out` overlap", "the scan cannot run in place; pass disjoint buffers");
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
    a.num_tiles = tiles_for<SpecScanAddI32>(n);
    a.ticket = reinterpret_cast<uint32_t *>(base);
    a.status = reinterpret_cast<uint64_t *>(base + NOALLOC_HEAD);
    a.epoch = epoch; a.failure = failure;
    a.carry_in = 0; a.carry_vals = nullptr; a.carry_n = 0; a.d_count = nullptr; a.shard_out = nullptr;
    a.d_base = nullptr; a.index_base = 0; a.seg_len = 1;
    a.peer_bufs = nullptr; a.peer_rank = 0; a.peer_world = 0; a.peer_seq = 0;
    err = launch_stream<SpecScanAddI32>(a, st);
    if (err != cudaSuccess) return fail(1, "futhark_b200_scan_i32_noalloc: kernel launch", cudaGetErrorString(err));
  }
  if (status_dev != nullptr) {
    err = cudaMemcpyAsync(status_dev, failure, sizeof(int32_t), cudaMemcpyDeviceToDevice, st);
    if (err != cudaSuccess) return fail(1, "futhark_b200_scan_i32_noalloc: status copy", cudaGetErrorString(err));
  }
  return 0;
}


