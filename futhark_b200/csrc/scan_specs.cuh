// Specifications for the single-pass tile kernel of k_scan.cu (`stream_kernel<Spec>`).
//
// The reference generates one SegScan kernel per program from the operator, the fused map
// body, the post-operation and the index space (src/Futhark/CodeGen/ImpGen/GPU/SegScan.hs:17-90,
// SegScan/SinglePass.hs:327-879; filter and partition are scans with a scatter as post-operation,
// prelude/soacs.fut:241-323).  Here the kernel is written once and a specification type supplies
// those pieces; a new scan, segmented scan, filter or partition entry point is a new
// specification, not a new kernel:
//
//   Op            the operator on (value bits, flag) pairs: combine(), kHasFlag, and kIdentity, the
//                 bits of its neutral element (pads a ragged tile, seeds the scan)
//   map(x)        the map body fused in front of the scan (scanomap), on the element's bits
//   kHasPost / post(scanned, x)   post-operation on (scan result, original element)
//   kExclusive    the result is shifted by one element (exscan)
//   kFlagArray    a byte array travels with the values: the head flags of a flagged segmented
//                 scan, or the keep-flags of a filter
//   kSegRegular   segmented scan over segments of one length (the innermost dimension of the
//                 index space): the head flag is computed from the element's index
//   kCompact / kPartition / pred(key, flag byte)   compaction: keep the keys that satisfy
//                 pred, in order; a partition also keeps the others, behind them
//   V, CTAS, LEAD tile geometry: a thread owns V 16-byte vectors (V odd), CTAS CTAs per SM,
//                 aggregates run LEAD tiles ahead of the scans
//   kStreamHints  L2 eviction priority "first" for what visit B reads and for what is stored
//   NBUF, DIST    tile buffers per CTA, and how many iterations ahead a tile is fetched (DIST < NBUF)
#pragma once
#include <stdint.h>

#include "common.cuh"

namespace fb {

// ---- operators on (value bits, flag) pairs -----------------------------------------
struct OpAddU32 {  // wrapping integer add; the flag is unused (always 0)
  static __device__ __forceinline__ void combine(uint32_t lv, uint32_t lf, uint32_t rv, uint32_t rf,
                                                 uint32_t &ov, uint32_t &of) {
    ov = lv + rv; of = 0; (void)lf; (void)rf;
  }
  static constexpr bool kHasFlag = false;
  static constexpr uint32_t kIdentity = 0u;
};
struct OpMaxI32 {  // signed maximum
  static __device__ __forceinline__ void combine(uint32_t lv, uint32_t lf, uint32_t rv, uint32_t rf,
                                                 uint32_t &ov, uint32_t &of) {
    ov = (uint32_t)max((int32_t)lv, (int32_t)rv); of = 0; (void)lf; (void)rf;
  }
  static constexpr bool kHasFlag = false;
  static constexpr uint32_t kIdentity = 0x80000000u;   // i32.lowest
};
struct OpSegAddF32 {  // (f1,v1) (+) (f2,v2) = (f1|f2, f2 ? v2 : v1+v2) on f32 bit patterns
  static __device__ __forceinline__ void combine(uint32_t lv, uint32_t lf, uint32_t rv, uint32_t rf,
                                                 uint32_t &ov, uint32_t &of) {
    float s = __uint_as_float(lv) + __uint_as_float(rv);
    ov = rf ? rv : __float_as_uint(s);
    of = lf | rf;
  }
  static constexpr bool kHasFlag = true;
  static constexpr uint32_t kIdentity = 0u;            // (false, 0.0)
};
struct OpSegAddI32 {  // the same lifting of the wrapping integer add
  static __device__ __forceinline__ void combine(uint32_t lv, uint32_t lf, uint32_t rv, uint32_t rf,
                                                 uint32_t &ov, uint32_t &of) {
    ov = rf ? rv : lv + rv;
    of = lf | rf;
  }
  static constexpr bool kHasFlag = true;
  static constexpr uint32_t kIdentity = 0u;            // (false, 0)
};

// ---- what every specification starts from ----------------------------------------------
struct SpecDefaults {
  using Op = OpAddU32;
  static constexpr bool kHasPost = false, kExclusive = false, kFlagArray = false, kSegRegular = false;
  static constexpr bool kCompact = false, kPartition = false;
  // visit B's loads and the stores ask L2 to evict their lines first.  It pays where tiles would otherwise leave
  // L2 between the visits (the compactions); for the scans it changes nothing that lasts: 95.0 -> 95.6 us (i32),
  // 205.5 -> 202.7 us (flagged f32), and the reduction that runs behind the flagged scan takes 108.7 -> 113.3 us.
  static constexpr bool kStreamHints = false;
  // Measured on 2^26 i32 (scan) / 2^27 f32 with flags (segmented scan), V x CTAS x NBUF x DIST:
  // 5x4x2x1 97 / 213 us; 5x5x2x1 102 / 219 us; 5x3x3x2 102 / 274 us; 5x3x3x1 105 / 295 us;
  // 3x4x4x2 120 / 318 us; 3x4x3x2 119 / 279 us; 3x5x3x2 123 / 285 us; 7x3x2x1 112 / 260 us.
  static constexpr int V = 5, CTAS = 4, LEAD = 1024;
  static constexpr int NBUF = 2, DIST = 1;
  static __device__ __forceinline__ uint32_t map(uint32_t x) { return x; }
  static __device__ __forceinline__ uint32_t post(uint32_t scanned, uint32_t x) { (void)x; return scanned; }
  static __device__ __forceinline__ bool pred(uint32_t key, uint32_t flag) { (void)key; (void)flag; return false; }
};

// ---- scans ---------------------------------------------------------------------------------
struct SpecScanAddI32 : SpecDefaults {};                                        // scan (+) 0 xs
struct SpecExscanAddI32 : SpecDefaults { static constexpr bool kExclusive = true; };
struct SpecScanMaxI32 : SpecDefaults {                                           // scan i32.max i32.lowest xs
  using Op = OpMaxI32;
};
struct SpecSegScanAddF32 : SpecDefaults {                                        // flagged segmented scan (+) over f32 (tests/soacs/scan2.fut:7-17)
  using Op = OpSegAddF32;
  static constexpr bool kFlagArray = true;
};
struct SpecSegRowsAddI32 : SpecDefaults {                                        // map (scan (+) 0) xss: regular segments (tests/intrablock/segscan0.fut)
  using Op = OpSegAddI32;
  static constexpr bool kSegRegular = true;
};
// One round of tests/soacs/scan4.fut: xs' = map2 (+) (map (+ sum) (scan (+) 0 (map (+1) xs))) xs.
// The map body (+1) sits in front of the scan, `sum` seeds it, and the post-operation adds
// the element itself: a scanomap with a post-operation (SinglePass.hs:841-876).
struct SpecScanomapStepI32 : SpecDefaults {
  static constexpr bool kHasPost = true;
  static __device__ __forceinline__ uint32_t map(uint32_t x) { return x + 1u; }
  static __device__ __forceinline__ uint32_t post(uint32_t scanned, uint32_t x) { return scanned + x; }
};

// ---- compaction -----------------------------------------------------------------------------
// Tiles of 9216 keys (V = 9), 3 CTAs per SM: the second visit does much more per tile than a
// scan's.  Measured on 2^28 keys (filter / partition): 323 / 461 us; tiles of 5120 keys with 4 CTAs
// per SM 393 / 492 us (no better with a lead of 1536 or 2048 tiles); 7168 keys 368 / 481 us.  With the eviction
// hints (308 / 431 us) a lead of 704 / 768 / 896 / 1280 tiles gives 311 / 308 / 308 / 309 and 438 / 432 / 429 / 440 us.
// Tile sizes again with the hints: 5120 keys x 4 CTAs 369 / 478 us, 7168 x 3 349 / 468 us, 11264 x 2 348 / 510 us.
struct SpecCompact : SpecDefaults {
  static constexpr bool kCompact = true;
  static constexpr int V = 9, CTAS = 3, NBUF = 2, DIST = 1;
  static constexpr bool kStreamHints = true;
};
struct SpecFilterLow3U32 : SpecCompact {                                         // filter (\k -> (k & 7) < 3) ks
  static __device__ __forceinline__ bool pred(uint32_t key, uint32_t) { return (key & 7u) < 3u; }
};
struct SpecPartitionLow3U32 : SpecFilterLow3U32 { static constexpr bool kPartition = true; };
struct SpecFilterPosI32 : SpecCompact {                                          // filter (0 <) xs (tests/soacs/filter1.fut)
  static __device__ __forceinline__ bool pred(uint32_t key, uint32_t) { return (int32_t)key > 0; }
};
// The two predicates of tests/soacs/partition1.fut; partition2 p q = partition p, then
// partition q on what p rejected.  Futhark's % is the floored modulus: x % m == 0 iff the
// truncated remainder is 0 as well.
struct SpecPartitionEvenI32 : SpecCompact {
  static constexpr bool kPartition = true;
  static __device__ __forceinline__ bool pred(uint32_t key, uint32_t) { return (key & 1u) == 0u; }
};
struct SpecPartitionDiv3I32 : SpecCompact {
  static constexpr bool kPartition = true;
  static __device__ __forceinline__ bool pred(uint32_t key, uint32_t) { return ((int32_t)key % 3) == 0; }
};
// filter over zip xs keep by the second component (tests/soacs/filter3.fut): the keep-flags
// travel with the keys, so the tile is smaller (5120 keys, 4 CTAs per SM)
struct SpecFilterByFlagI32 : SpecDefaults {
  static constexpr bool kCompact = true, kFlagArray = true, kStreamHints = true;
  static constexpr int V = 5, CTAS = 4, NBUF = 2, DIST = 1;
  static __device__ __forceinline__ bool pred(uint32_t, uint32_t flag) { return flag != 0u; }
};

}  // namespace fb
