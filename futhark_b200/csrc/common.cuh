// Device-side helpers shared by every kernel file: 128-bit streaming loads, warp
// shuffles, bulk-async (TMA) copies with bounded mbarrier waits, and the packed
// tile-status word of the single-pass look-back scans.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace fb {

// ---- status codes written to the context's device failure word ------------------
// 0 means "no failure".  Kernels never trap or spin without bound: a wait that
// exceeds its limit stores one of these codes and the whole grid drains.
enum FailureCode : int {
  FAIL_NONE = 0,
  FAIL_LOOKBACK_TIMEOUT = 1,   // a tile waited too long for its predecessors
  FAIL_BULK_COPY_TIMEOUT = 2,  // an mbarrier wait on a bulk copy ran out
  FAIL_MMA_TIMEOUT = 3,        // an mbarrier wait in the tensor-core pipeline ran out
  FAIL_PEER_TIMEOUT = 4,       // a wait for the summary of another GPU's shard ran out
};

constexpr int kWarp = 32;
constexpr unsigned kFull = 0xffffffffu;

// ---- streaming global loads (read once: bypass L1 allocation) --------------------
__device__ __forceinline__ int4 ld_stream_v4(const void *p) {
  int4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.s32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ int ld_stream_b32(const void *p) {
  int v;
  asm volatile("ld.global.nc.L1::no_allocate.s32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ void st_stream_v4(void *p, int4 v) {
  asm volatile("st.global.cs.v4.s32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

// ---- warp primitives ------------------------------------------------------------
template <typename T>
__device__ __forceinline__ T warp_sum(T v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(kFull, v, o);
  return v;
}
// Ordered float sum (lane 0 .. lane 31 association as a balanced tree, fixed shape).
__device__ __forceinline__ float warp_sum_down(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(kFull, v, o);
  return v;  // valid in lane 0
}
// Inclusive scan across the warp.
__device__ __forceinline__ uint32_t warp_incl_scan_add(uint32_t v, int lane) {
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    uint32_t t = __shfl_up_sync(kFull, v, o);
    if (lane >= o) v += t;
  }
  return v;
}

// ---- shared-memory addresses and mbarriers ------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_inval(uint64_t *bar) {
  asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Makes mbarrier initialisation visible to the async proxy (TMA / tensor core).
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// Orders generic-proxy shared-memory writes before later async-proxy reads.
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Non-blocking test of a phase (try_wait may suspend the thread for a while).
__device__ __forceinline__ bool mbar_test_wait(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait: returns false when the limit ran out (the caller records a failure
// code and leaves without touching the data the copy was to deliver).
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity, uint32_t max_polls = (1u << 22)) {
  for (uint32_t i = 0; i < max_polls; i++) {
    if (mbar_try_wait(bar, parity)) return true;
    if (i > 64) __nanosleep(64);
  }
  return false;
}

// ---- bulk async copies (TMA, untiled): both addresses 16-byte aligned, size % 16 == 0
__device__ __forceinline__ void bulk_g2s(void *smem_dst, const void *gsrc, uint32_t bytes, uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void bulk_s2g(void *gdst, const void *smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               ::"l"(gdst), "r"(smem_u32(smem_src)), "r"(bytes) : "memory");
}
// The same copies with an L2 eviction priority for the lines they touch (createpolicy; 1.0 = all of them).
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void bulk_g2s_hint(void *smem_dst, const void *gsrc, uint32_t bytes, uint64_t *bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
      ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void bulk_s2g_hint(void *gdst, const void *smem_src, uint32_t bytes, uint64_t policy) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group.L2::cache_hint [%0], [%1], %2, %3;"
               ::"l"(gdst), "r"(smem_u32(smem_src)), "r"(bytes), "l"(policy) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Waits until the bulk stores of this thread have finished READING shared memory.
__device__ __forceinline__ void bulk_wait_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// Same, but the most recently committed group may still be reading.
__device__ __forceinline__ void bulk_wait_read1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }

// ---- packed tile status of the single-pass look-back scans ------------------------
// One 64-bit word per tile: low 32 bits = value, high 32 bits = tag.  The tag is
// (epoch << 3) | (flag << 2) | state, state 0 = nothing yet, 1 = tile aggregate,
// 2 = inclusive prefix.  A 64-bit relaxed store publishes value and state at once, so
// no fence is needed between them.  The epoch changes with every launch: words left
// over from earlier launches read as "nothing yet", so the array is never cleared.
constexpr uint32_t ST_NONE = 0, ST_AGG = 1, ST_PREFIX = 2;

__device__ __forceinline__ uint64_t pack_status(uint32_t value, uint32_t epoch, uint32_t flag, uint32_t state) {
  return ((uint64_t)((epoch << 3) | (flag << 2) | state) << 32) | (uint64_t)value;
}
__device__ __forceinline__ void st_status(uint64_t *p, uint64_t w) {
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ uint64_t ld_status(const uint64_t *p) {
  uint64_t w;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
  return w;
}
__device__ __forceinline__ int ld_failure(const int *p) {
  int v;
  asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// state of a word under this launch's epoch (ST_NONE if the word is stale)
__device__ __forceinline__ uint32_t status_state(uint64_t w, uint32_t epoch) {
  uint32_t tag = (uint32_t)(w >> 32);
  return ((tag >> 3) == epoch) ? (tag & 3u) : ST_NONE;
}
__device__ __forceinline__ uint32_t status_flag(uint64_t w) { return ((uint32_t)(w >> 32) >> 2) & 1u; }
__device__ __forceinline__ uint32_t status_value(uint64_t w) { return (uint32_t)w; }

}  // namespace fb
