// Batched dense contraction C[b] = A[b] x B[b], f16 inputs, f32 accumulation, on the
// 5th-generation tensor cores (tcgen05.mma with the accumulator in tensor memory).  Two
// kernels: the one described first works with one CTA per 128 x 256 tile and takes any shape
// the bulk tensor copies can address; where M and N are multiples of 256 the second one, further
// down, puts a pair of CTAs on a 256 x 256 tile (tcgen05.mma.cta_group::2).
// Replaces the block/register-tiled SIMT kernel the reference generates for a
// map-map-reduce nest (src/Futhark/Optimise/BlkRegTiling.hs:68-140,727-743;
// src/Futhark/CodeGen/ImpGen/GPU/Block.hs:687-722).
//
// One persistent CTA per SM, 6 warps:
//   warp 0      producer: TMA tile loads (A: 128 x 64 K-major, B: 64 x 256 N-major, both
//               128-byte swizzled) into a 4-stage shared-memory ring, one mbarrier per stage
//   warp 1      allocates 512 TMEM columns (two 128 x 256 f32 accumulators) and issues
//               tcgen05.mma M128 N256 K16; tcgen05.commit hands stages back to the
//               producer and finished accumulators to the epilogue
//   warps 2-5   epilogue: tcgen05.ld of the accumulator (one TMEM lane = one row per
//               thread, the next 32-column chunk in flight while this one is handled),
//               staged in shared memory and written to C by bulk tensor stores (TMA), so
//               the warps never wait for the memory system; runs while the next tile's
//               MMAs fill the other accumulator
// B is consumed as it lies in memory ([K][N], N contiguous) through the "MN-major"
// operand layout, so no transpose pass is needed.  No multicast is used anywhere.
// Every mbarrier wait is bounded; a wait that runs out stores a failure code, and all
// roles drain and meet at the final barrier so that TMEM is always released.
//
// Shapes the TMA path cannot take (K or N not a multiple of 8, or unaligned bases) go
// to a plain one-thread-per-output kernel.
#include <cuda.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "kernels.h"

namespace fb {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK * 2;            // 16 KiB
constexpr int B_STAGE_BYTES = BK * BN * 2;            // 32 KiB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int B_NBLOCK_BYTES = BK * 64 * 2;           // one 64-wide slab of N: 8 KiB
constexpr int BMM_THREADS = 192;
constexpr int EPI_PITCH = 36;                         // plain-store path: floats per staged row, 32 + 4 of padding
constexpr int EPI_CHUNK_BYTES = 32 * 32 * 4;          // one 32 x 32 f32 chunk
constexpr int EPI_BYTES = 4 * 2 * EPI_CHUNK_BYTES;    // two chunk buffers per epilogue warp (the plain path needs 4.5 KiB of them)
constexpr int BMM_SMEM = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 1024 /*barriers*/ + EPI_BYTES;
constexpr uint32_t TMEM_COLS = 512;

// ---- tcgen05 / TMA wrappers ---------------------------------------------------------------
__device__ __forceinline__ void tma_load_3d(void *smem_dst, const CUtensorMap *tm, int x, int y, int z,
                                            uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(smem_u32(smem_dst)), "l"(tm), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap *tm, const void *smem_src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(tm), "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t *smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
               ::"r"(smem_u32(smem_slot)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns: thread l of the warp receives row (lane base + l)
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor (64-bit): start address, leading / stride byte
// offsets in 16-byte units, descriptor version 1, 128-byte swizzle.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;      // descriptor version for this architecture
  d |= (uint64_t)2 << 61;      // SWIZZLE_128B
  return d;
}
// Instruction descriptor: D = f32, A = B = f16, A K-major, B MN-major, N = 256, M = 128.
constexpr uint32_t BMM_IDESC = (1u << 4) | (0u << 7) | (0u << 10) | (0u << 15) | (1u << 16) |
                               ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

struct BmmBarriers {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  uint32_t failed;
};

__global__ void __launch_bounds__(BMM_THREADS, 1)
bmm_f16_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const __grid_constant__ CUtensorMap tmC, int c_by_tma,
                  float *__restrict__ C, int nb, int M, int N, int K, int *failure) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  BmmBarriers *bars = reinterpret_cast<BmmBarriers *>(smem + STAGES * STAGE_BYTES);
  float *epi = reinterpret_cast<float *>(smem + STAGES * STAGE_BYTES + 1024);    // 1024-byte aligned

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
  const int tiles_per_batch = tiles_m * tiles_n;
  const int64_t num_tiles = (int64_t)tiles_per_batch * nb;
  const int kblocks = (K + BK - 1) / BK;

  if (tid == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(&bars->full[s], 1); mbar_init(&bars->empty[s], 1); }
    for (int a = 0; a < 2; a++) { mbar_init(&bars->tmem_full[a], 1); mbar_init(&bars->tmem_empty[a], 128); }
    bars->failed = 0;
    fence_mbar_init();
  }
  if (warp == 1) { tmem_alloc(&bars->tmem_base, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  const bool poisoned = ld_failure(failure) != FAIL_NONE;   // uniform over the grid at entry

  if (!poisoned && kblocks > 0) {
    if (warp == 0) {
      // ---------------- producer ----------------
      if (lane == 0) {
        uint32_t it = 0;
        bool ok = true;
        for (int64_t t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
          const int batch = (int)(t / tiles_per_batch);
          const int r = (int)(t % tiles_per_batch);
          const int m0 = (r / tiles_n) * BM, n0 = (r % tiles_n) * BN;
          for (int kb = 0; kb < kblocks; kb++, it++) {
            const int s = it % STAGES;
            const uint32_t ph = (it / STAGES) & 1;
            if (!mbar_wait_bounded(&bars->empty[s], ph ^ 1)) { ok = false; break; }
            uint8_t *sa = smem + s * STAGE_BYTES;
            uint8_t *sb = sa + A_STAGE_BYTES;
            mbar_expect_tx(&bars->full[s], STAGE_BYTES);
            tma_load_3d(sa, &tmA, kb * BK, m0, batch, &bars->full[s]);
#pragma unroll
            for (int j = 0; j < BN / 64; j++)
              tma_load_3d(sb + j * B_NBLOCK_BYTES, &tmB, n0 + j * 64, kb * BK, batch, &bars->full[s]);
          }
        }
        if (!ok) { atomicCAS(failure, FAIL_NONE, FAIL_MMA_TIMEOUT); bars->failed = 1; }
      }
    } else if (warp == 1) {
      // ---------------- MMA issuer ----------------
      if (lane == 0) {
        uint32_t it = 0, tile_it = 0;
        bool ok = true;
        for (int64_t t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, tile_it++) {
          const uint32_t acc = tile_it & 1, acc_ph = (tile_it >> 1) & 1;
          if (!mbar_wait_bounded(&bars->tmem_empty[acc], acc_ph ^ 1)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + acc * BN;
          for (int kb = 0; kb < kblocks; kb++, it++) {
            const int s = it % STAGES;
            const uint32_t ph = (it / STAGES) & 1;
            if (!mbar_wait_bounded(&bars->full[s], ph)) { ok = false; break; }
            tc_fence_after();
            const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
            const uint32_t sb = sa + A_STAGE_BYTES;
            // A: K-major, rows of 128 bytes, 8-row groups 1024 bytes apart
            const uint64_t adesc = make_smem_desc(sa, 16, 1024);
            // B: N-major, 64-wide N slabs 8 KiB apart (leading), 8-row K groups 1024 bytes apart (stride)
            const uint64_t bdesc = make_smem_desc(sb, B_NBLOCK_BYTES, 1024);
#pragma unroll
            for (int k = 0; k < BK / 16; k++) {
              // K step of 16: A advances 32 bytes inside the swizzled row, B advances 16 rows
              tc_mma_f16(d_tmem, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 128), BMM_IDESC,
                         (kb > 0 || k > 0) ? 1u : 0u);
            }
            tc_commit(&bars->empty[s]);          // stage free once these MMAs have read it
          }
          if (ok) tc_commit(&bars->tmem_full[acc]);  // accumulator complete
        }
        if (!ok) { atomicCAS(failure, FAIL_NONE, FAIL_MMA_TIMEOUT); bars->failed = 1; }
      }
    } else {
      // ---------------- epilogue (warps 2..5) ----------------
      const int quarter = warp & 3;                 // TMEM lanes 32*quarter .. +31
      uint32_t tile_it = 0;
      bool ok = true;
      const bool vec_ok = ((N & 3) == 0) && ((((uintptr_t)C) & 15) == 0);
      for (int64_t t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, tile_it++) {
        const int batch = (int)(t / tiles_per_batch);
        const int r = (int)(t % tiles_per_batch);
        const int m0 = (r / tiles_n) * BM, n0 = (r % tiles_n) * BN;
        const uint32_t acc = tile_it & 1, acc_ph = (tile_it >> 1) & 1;
        // warp-uniform outcome: the TMEM loads below need the whole warp
        if (!__all_sync(kFull, mbar_wait_bounded(&bars->tmem_full[acc], acc_ph))) { ok = false; break; }
        tc_fence_after();
        // A thread receives 32 consecutive columns of ONE row from TMEM; written out like
        // that, every store instruction would touch 32 different cache lines.  The chunk is
        // therefore turned through shared memory so that 8 lanes write one full 128-byte line.
        float *stg = epi + (warp - 2) * (2 * EPI_CHUNK_BYTES / 4);
        const int rsub = lane >> 3, c4 = (lane & 7) * 4;
        // The TMEM load of the next chunk is in flight while this one is staged and stored.
        const uint32_t taddr0 = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN;
        auto emit = [&](const uint32_t (&v)[32], int c) {
#pragma unroll
          for (int q = 0; q < 8; q++) {
            float4 o;
            o.x = __uint_as_float(v[4 * q]); o.y = __uint_as_float(v[4 * q + 1]);
            o.z = __uint_as_float(v[4 * q + 2]); o.w = __uint_as_float(v[4 * q + 3]);
            *reinterpret_cast<float4 *>(stg + lane * EPI_PITCH + 4 * q) = o;
          }
          __syncwarp();
          const int col0 = n0 + c * 32;
#pragma unroll
          for (int p = 0; p < 8; p++) {
            const int rloc = p * 4 + rsub;
            const int row = m0 + quarter * 32 + rloc;
            const float4 o = *reinterpret_cast<const float4 *>(stg + rloc * EPI_PITCH + c4);
            if (row < M) {
              float *dst = C + ((int64_t)batch * M + row) * (int64_t)N + col0 + c4;
              if (vec_ok && col0 + c4 + 4 <= N) {
                asm volatile("st.global.cs.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(dst), "f"(o.x), "f"(o.y), "f"(o.z), "f"(o.w) : "memory");
              } else {
                if (col0 + c4 + 0 < N) dst[0] = o.x;
                if (col0 + c4 + 1 < N) dst[1] = o.y;
                if (col0 + c4 + 2 < N) dst[2] = o.z;
                if (col0 + c4 + 3 < N) dst[3] = o.w;
              }
            }
          }
          __syncwarp();
        };
        // With a tensor map for C the chunk leaves as one bulk tensor store (TMA) issued by lane
        // 0: the warp does not wait for the memory system at all.  The chunk is staged as the
        // 128-byte swizzle wants it (16-byte piece q of row r at position q ^ (r & 7)), which
        // also keeps the staging stores conflict-free.  Two buffers per warp: a buffer is
        // written again once the store issued from it two chunks ago has read it.
        auto emit_tma = [&](const uint32_t (&v)[32], int c) {
          float *buf = stg + (c & 1) * (EPI_CHUNK_BYTES / 4);
          if (lane == 0) bulk_wait_read1();
          __syncwarp();
#pragma unroll
          for (int q = 0; q < 8; q++) {
            float4 o;
            o.x = __uint_as_float(v[4 * q]); o.y = __uint_as_float(v[4 * q + 1]);
            o.z = __uint_as_float(v[4 * q + 2]); o.w = __uint_as_float(v[4 * q + 3]);
            *reinterpret_cast<float4 *>(buf + lane * 32 + ((q ^ (lane & 7)) << 2)) = o;
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_3d(&tmC, buf, n0 + c * 32, m0 + quarter * 32, batch);
            bulk_commit();
          }
        };
        uint32_t va[32], vb[32];
        tmem_ld_32x32(taddr0, va);
#pragma unroll 1
        for (int c = 0; c < BN / 32; c += 2) {
          tmem_ld_wait();
          tmem_ld_32x32(taddr0 + (c + 1) * 32, vb);
          if (c_by_tma) emit_tma(va, c); else emit(va, c);
          tmem_ld_wait();
          if (c + 2 < BN / 32) tmem_ld_32x32(taddr0 + (c + 2) * 32, va);
          if (c_by_tma) emit_tma(vb, c + 1); else emit(vb, c + 1);
        }
        tc_fence_before();
        mbar_arrive(&bars->tmem_empty[acc]);
      }
      if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // the bulk stores of this warp are complete
      if (!ok) { atomicCAS(failure, FAIL_NONE, FAIL_MMA_TIMEOUT); bars->failed = 1; }
    }
  }
  // ---------------- teardown: every thread arrives here, whatever happened ----------------
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---- the same contraction with CTA pairs: tcgen05.mma.cta_group::2 ---------------------------------
// Two CTAs of a cluster work on one 256 x 256 tile.  CTA r of the pair loads rows r*128 .. +128 of
// the A tile and columns r*128 .. +128 of the B tile into its own shared memory (its own,
// non-multicast bulk tensor copies), and holds rows r*128 .. +128 of the accumulator in its own
// tensor memory; one thread of the pair's first CTA issues M256 N256 K16 instructions that read
// both CTAs' shared memory.  Per instruction a CTA therefore brings 128 x 64 + 64 x 128 operand
// elements from L2 for 128 x 256 x 64 multiply-adds of its own, against 128 x 64 + 64 x 256 in the
// one-CTA kernel above: the L2 -> SM traffic, which bounds that kernel, drops by a third.
//
// Barriers: full[s] lives in the first CTA and collects the bytes of both CTAs' copies (the second
// CTA's copies name it by its cluster address); empty[s] and tmem_full[a] exist in both CTAs and
// are signalled in both by one tcgen05.commit with a CTA mask; tmem_empty[a] lives in the first
// CTA and counts the epilogue threads of both.  Every wait is bounded.  The pair meets at a
// cluster barrier after setting its barriers up and again before anything is torn down, so that
// no CTA signals into a partner that has left.
constexpr int P_STAGES = 6;                            // (5 stages measured the same: 133 us on 64 x 1024^3)
constexpr int P_A_BYTES = BM * BK * 2;                 // 128 x 64 f16: 16 KiB
constexpr int P_B_BYTES = BK * 128 * 2;                // 64 x 128 f16 as two 64-wide slabs: 16 KiB
constexpr int P_STAGE_BYTES = P_A_BYTES + P_B_BYTES;
constexpr int BMM2_SMEM = P_STAGES * P_STAGE_BYTES + 1024 + 1024 + EPI_BYTES;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// bulk tensor copy into this CTA's shared memory whose completion is counted by a barrier given by
// its cluster address (it may be the partner's)
__device__ __forceinline__ void tma_load_3d_pair(void *smem_dst, const CUtensorMap *tm, int x, int y, int z, uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(smem_u32(smem_dst)), "l"(tm), "r"(x), "r"(y), "r"(z), "r"(bar_cluster_addr)
      : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void tc2_commit_both(uint64_t *bar) {     // arrives on `bar` in both CTAs of the pair
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void tc2_mma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Instruction descriptor of the pair: D = f32, A = B = f16, A K-major, B MN-major, N = 256, M = 256.
constexpr uint32_t BMM2_IDESC = (1u << 4) | (0u << 7) | (0u << 10) | (0u << 15) | (1u << 16) |
                                ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);

struct Bmm2Barriers {
  uint64_t full[P_STAGES];        // used in the first CTA only
  uint64_t empty[P_STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];         // used in the first CTA only
  uint32_t tmem_base;
  uint32_t failed;
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(BMM_THREADS, 1)
bmm_f16_tc2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                   const __grid_constant__ CUtensorMap tmC, int nb, int M, int N, int K, int *failure) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  Bmm2Barriers *bars = reinterpret_cast<Bmm2Barriers *>(smem + P_STAGES * P_STAGE_BYTES);
  float *epi = reinterpret_cast<float *>(smem + P_STAGES * P_STAGE_BYTES + 1024);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_ctarank();             // 0: issues the instructions of the pair
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  const int tiles_m = M / 256, tiles_n = N / 256;      // the launcher takes this kernel only for multiples of 256
  const int tiles_per_batch = tiles_m * tiles_n;
  const int64_t num_tiles = (int64_t)tiles_per_batch * nb;
  const int kblocks = (K + BK - 1) / BK;

  if (tid == 0) {
    for (int s = 0; s < P_STAGES; s++) { mbar_init(&bars->full[s], 1); mbar_init(&bars->empty[s], 1); }
    for (int a = 0; a < 2; a++) { mbar_init(&bars->tmem_full[a], 1); mbar_init(&bars->tmem_empty[a], 256); }
    bars->failed = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                                  // both CTAs' barriers exist before either signals the other's
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  const bool poisoned = ld_failure(failure) != FAIL_NONE;

  if (!poisoned && kblocks > 0) {
    if (warp == 0) {
      // ---------------- producer: this CTA's half of A and of B ----------------
      if (lane == 0) {
        uint32_t it = 0;
        bool ok = true;
        for (int64_t t = pair; t < num_tiles && ok; t += npairs) {
          const int batch = (int)(t / tiles_per_batch);
          const int r = (int)(t % tiles_per_batch);
          const int m0 = (r / tiles_n) * 256 + (int)rank * 128, n0 = (r % tiles_n) * 256 + (int)rank * 128;
          for (int kb = 0; kb < kblocks; kb++, it++) {
            const int s = it % P_STAGES;
            const uint32_t ph = (it / P_STAGES) & 1;
            if (!mbar_wait_bounded(&bars->empty[s], ph ^ 1)) { ok = false; break; }
            uint8_t *sa = smem + s * P_STAGE_BYTES;
            uint8_t *sb = sa + P_A_BYTES;
            const uint32_t full0 = map_to_cta(smem_u32(&bars->full[s]), 0);      // the first CTA's barrier
            if (rank == 0) mbar_expect_tx(&bars->full[s], 2 * P_STAGE_BYTES);     // both CTAs' bytes
            tma_load_3d_pair(sa, &tmA, kb * BK, m0, batch, full0);
            tma_load_3d_pair(sb, &tmB, n0, kb * BK, batch, full0);
            tma_load_3d_pair(sb + B_NBLOCK_BYTES, &tmB, n0 + 64, kb * BK, batch, full0);
          }
        }
        if (!ok) { atomicCAS(failure, FAIL_NONE, FAIL_MMA_TIMEOUT); bars->failed = 1; }
      }
    } else if (warp == 1) {
      // ---------------- MMA issuer: one thread of the first CTA ----------------
      if (lane == 0 && rank == 0) {
        uint32_t it = 0, tile_it = 0;
        bool ok = true;
        for (int64_t t = pair; t < num_tiles && ok; t += npairs, tile_it++) {
          const uint32_t acc = tile_it & 1, acc_ph = (tile_it >> 1) & 1;
          if (!mbar_wait_bounded(&bars->tmem_empty[acc], acc_ph ^ 1)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + acc * 256;
          for (int kb = 0; kb < kblocks; kb++, it++) {
            const int s = it % P_STAGES;
            const uint32_t ph = (it / P_STAGES) & 1;
            if (!mbar_wait_bounded(&bars->full[s], ph)) { ok = false; break; }
            tc_fence_after();
            const uint32_t sa = smem_u32(smem + s * P_STAGE_BYTES);
            const uint32_t sb = sa + P_A_BYTES;
            const uint64_t adesc = make_smem_desc(sa, 16, 1024);
            const uint64_t bdesc = make_smem_desc(sb, B_NBLOCK_BYTES, 1024);
#pragma unroll
            for (int k = 0; k < BK / 16; k++)
              tc2_mma_f16(d_tmem, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 128), BMM2_IDESC, (kb > 0 || k > 0) ? 1u : 0u);
            tc2_commit_both(&bars->empty[s]);          // the stage is free in both CTAs once these instructions have read it
          }
          if (ok) tc2_commit_both(&bars->tmem_full[acc]);
        }
        if (!ok) { atomicCAS(failure, FAIL_NONE, FAIL_MMA_TIMEOUT); bars->failed = 1; }
      }
    } else {
      // ---------------- epilogue (warps 2..5): this CTA's 128 rows of the tile ----------------
      const int quarter = warp & 3;
      uint32_t tile_it = 0;
      bool ok = true;
      float *stg = epi + (warp - 2) * (2 * EPI_CHUNK_BYTES / 4);
      for (int64_t t = pair; t < num_tiles && ok; t += npairs, tile_it++) {
        const int batch = (int)(t / tiles_per_batch);
        const int r = (int)(t % tiles_per_batch);
        const int m0 = (r / tiles_n) * 256 + (int)rank * 128, n0 = (r % tiles_n) * 256;
        const uint32_t acc = tile_it & 1, acc_ph = (tile_it >> 1) & 1;
        if (!__all_sync(kFull, mbar_wait_bounded(&bars->tmem_full[acc], acc_ph))) { ok = false; break; }
        tc_fence_after();
        const uint32_t taddr0 = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * 256;
        auto emit_tma = [&](const uint32_t (&v)[32], int c) {
          float *buf = stg + (c & 1) * (EPI_CHUNK_BYTES / 4);
          if (lane == 0) bulk_wait_read1();
          __syncwarp();
#pragma unroll
          for (int q = 0; q < 8; q++) {
            float4 o;
            o.x = __uint_as_float(v[4 * q]); o.y = __uint_as_float(v[4 * q + 1]);
            o.z = __uint_as_float(v[4 * q + 2]); o.w = __uint_as_float(v[4 * q + 3]);
            *reinterpret_cast<float4 *>(buf + lane * 32 + ((q ^ (lane & 7)) << 2)) = o;
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_3d(&tmC, buf, n0 + c * 32, m0 + quarter * 32, batch);
            bulk_commit();
          }
        };
        uint32_t va[32], vb[32];
        tmem_ld_32x32(taddr0, va);
#pragma unroll 1
        for (int c = 0; c < 256 / 32; c += 2) {
          tmem_ld_wait();
          tmem_ld_32x32(taddr0 + (c + 1) * 32, vb);
          emit_tma(va, c);
          tmem_ld_wait();
          if (c + 2 < 256 / 32) tmem_ld_32x32(taddr0 + (c + 2) * 32, va);
          emit_tma(vb, c + 1);
        }
        tc_fence_before();
        mbar_arrive_cluster(map_to_cta(smem_u32(&bars->tmem_empty[acc]), 0));
      }
      if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
      if (!ok) { atomicCAS(failure, FAIL_NONE, FAIL_MMA_TIMEOUT); bars->failed = 1; }
    }
  }
  // ---------------- teardown: every thread of both CTAs arrives here, whatever happened ----------------
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                                  // nobody signals into a partner that has left
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ---- plain kernel for shapes the TMA path cannot take -----------------------------------------
__global__ void __launch_bounds__(256)
bmm_f16_simple_kernel(const __half *__restrict__ A, const __half *__restrict__ B, float *__restrict__ C,
                      int64_t nb, int64_t M, int64_t K, int64_t N) {
  const int64_t total = nb * M * N;
  const int64_t stride = (int64_t)gridDim.x * 256;
  for (int64_t o = (int64_t)blockIdx.x * 256 + threadIdx.x; o < total; o += stride) {
    const int64_t b = o / (M * N), r = o % (M * N), i = r / N, j = r % N;
    const __half *a = A + (b * M + i) * K;
    const __half *bp = B + b * K * N + j;
    float acc = 0.f;
    for (int64_t k = 0; k < K; k++) acc = __fadd_rn(acc, __fmul_rn(__half2float(a[k]), __half2float(bp[k * N])));
    C[o] = acc;
  }
}

// ---- host side ----------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// dims are innermost first; strides (bytes) for dims 1..2
static bool make_map_3d(CUtensorMap *tm, const void *base, uint64_t d0, uint64_t d1, uint64_t d2, uint32_t b0,
                        uint32_t b1, bool f32 = false) {
  EncodeTiledFn enc = get_encode_fn();
  if (enc == nullptr) return false;
  const uint64_t es = f32 ? 4 : 2;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {d0 * es, d0 * d1 * es};
  cuuint32_t box[3] = {b0, b1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(tm, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void *>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

cudaError_t launch_bmm_f16(const uint16_t *A, const uint16_t *B, float *C, int64_t nb, int64_t m, int64_t k,
                           int64_t n, int *failure, cudaStream_t stream) {
  if (nb * m * n <= 0) return cudaSuccess;
  if (k <= 0) return cudaMemsetAsync(C, 0, (size_t)(nb * m * n) * sizeof(float), stream);
  const bool tma_ok = (k % 8 == 0) && (n % 8 == 0) && ((((uintptr_t)A) | ((uintptr_t)B)) & 15) == 0 &&
                      m < (1ll << 31) && n < (1ll << 31) && k < (1ll << 31) && nb < (1ll << 31) &&
                      m * n >= 128 * 64;
  if (tma_ok) {
    CUtensorMap tmA, tmB;
    if (make_map_3d(&tmA, A, (uint64_t)k, (uint64_t)m, (uint64_t)nb, BK, BM) &&
        make_map_3d(&tmB, B, (uint64_t)n, (uint64_t)k, (uint64_t)nb, 64, BK)) {
      cudaError_t err = cudaFuncSetAttribute(bmm_f16_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BMM_SMEM);
      if (err != cudaSuccess) return err;
      int dev = 0, sms = 0;
      cudaGetDevice(&dev);
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
      const int64_t tiles = ((m + BM - 1) / BM) * ((n + BN - 1) / BN) * nb;
      const int grid = (int)(tiles < sms ? tiles : sms);
      // C leaves by bulk tensor stores where a map can describe it (rows a multiple of 16 bytes, aligned base)
      CUtensorMap tmC = tmA;
      const int c_by_tma = ((n % 4 == 0) && ((((uintptr_t)C) & 15) == 0) &&
                            make_map_3d(&tmC, C, (uint64_t)n, (uint64_t)m, (uint64_t)nb, 32, 32, true)) ? 1 : 0;
      // tiles of 256 x 256 on CTA pairs where the shape is made of them
      if (c_by_tma && m % 256 == 0 && n % 256 == 0 && sms >= 2) {
        err = cudaFuncSetAttribute(bmm_f16_tc2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BMM2_SMEM);
        if (err != cudaSuccess) return err;
        const int64_t tiles2 = (m / 256) * (n / 256) * nb;
        int pairs = sms / 2;
        if (tiles2 < pairs) pairs = (int)tiles2;
        bmm_f16_tc2_kernel<<<2 * pairs, BMM_THREADS, BMM2_SMEM, stream>>>(tmA, tmB, tmC, (int)nb, (int)m, (int)n, (int)k, failure);
        return cudaGetLastError();
      }
      bmm_f16_tc_kernel<<<grid, BMM_THREADS, BMM_SMEM, stream>>>(tmA, tmB, tmC, c_by_tma, C, (int)nb, (int)m, (int)n, (int)k, failure);
      return cudaGetLastError();
    }
  }
  const int64_t total = nb * m * n;
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  bmm_f16_simple_kernel<<<(int)blocks, 256, 0, stream>>>(reinterpret_cast<const __half *>(A),
                                                         reinterpret_cast<const __half *>(B), C, nb, m, k, n);
  return cudaGetLastError();
}

}  // namespace fb
