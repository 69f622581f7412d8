// Generalised histogram (reduce_by_index) over 32-bit values.  Replaces the generated
// seghist_local / seghist_global kernels of the reference
// (src/Futhark/CodeGen/ImpGen/GPU/SegHist.hs:377-1188).
//
// The kernels are templated on the operator (HistOpKind, kernels.h).  What an operator
// supplies is what the reference's atomic-update choice supplies (ImpGen/GPU/Base.hs:720-905,
// the table of ImpGen/GPU.hs:46-90): its neutral element, how a value is combined into a bin
// atomically (a native 32-bit atomic where there is one: add, min, max, and, or, xor, f32 add;
// f32 max as unsigned max on an order-preserving key of the float; a compare-and-swap loop
// for what has none, here the integer product), and how two partial bins are folded.
// Indices outside [0,B) are skipped (SegHist.hs:450-455); NaN weights are skipped by the
// f32 max, as fmaxf drops them (rts/c/scalar.h:932).
//
// Strategies, by number of bins B (CAP = 57344 bins = 224 KiB of shared memory):
//   B <= CAP      one CTA per SM holds C = 2^k <= 32 private copies of the histogram in
//                 shared memory, laid out [bin][copy] with copy = lane mod C; for C = 32
//                 every lane owns a bank, so a warp never conflicts with itself no matter
//                 how skewed the indices are.  Copies are folded and flushed to the
//                 result with one global atomic per non-neutral bin.
//   B <= 4*CAP    the bins are cut into P = ceil(B/CAP) ranges; P consecutive CTAs read
//                 the same input chunk at the same time (the re-reads are served by L2)
//                 and each keeps only the indices of its range: one pass over HBM, P
//                 passes over L2, whose bandwidth bounds this path.  (One histogram per
//                 cluster of P CTAs in distributed shared memory, every element handled
//                 once, was measured three times slower at P = 2: shared-memory atomics
//                 across a cluster run at about one per three cycles and SM.)
//   larger        global atomics into the result, which stays L2-resident for the sizes of
//                 interest (2^20 bins = 4 MiB), behind a per-CTA cache in shared memory:
//                 16384 (bin, value) slots, a bin owning the slot it hashes to if it gets
//                 there first.  With skewed indices the hot bins claim their slots at once
//                 and are accumulated on chip; their updates would otherwise queue up on
//                 single L2 addresses.  A CTA that sees few hits (uniform indices over many
//                 more bins than slots) stops looking into the cache.
#include <cuda_fp16.h>

#include "common.cuh"
#include "kernels.h"

namespace fb {

constexpr int HIST_THREADS = 1024;
constexpr int64_t HIST_CAP_BINS = 57344;        // 224 KiB / 4
constexpr uint32_t KEY_NEG_INF = 0x007FFFFFu;   // key of -inf

__device__ __forceinline__ uint32_t f32_key(uint32_t bits) {
  return bits ^ ((uint32_t)((int32_t)bits >> 31) | 0x80000000u);     // a shift and one three-input logic operation
}
// Seen through the key, a NaN with the sign bit set lies below -inf (it can never win a maximum) and one
// without lies above +inf: one comparison on the key finds the only NaNs that matter.
constexpr uint32_t KEY_POS_INF = 0xFF800000u;
__device__ __forceinline__ bool key_is_winning_nan(uint32_t key) { return key > KEY_POS_INF; }
__device__ __forceinline__ uint32_t key_f32(uint32_t key) {
  return (key & 0x80000000u) ? (key ^ 0x80000000u) : ~key;
}

template <int OP>
__device__ __host__ __forceinline__ constexpr uint32_t neutral() {
  return OP == HOP_MAX_F32 ? KEY_NEG_INF
       : OP == HOP_MIN_I32 ? 0x7FFFFFFFu
       : OP == HOP_MAX_I32 ? 0x80000000u
       : OP == HOP_MIN_U32 ? 0xFFFFFFFFu
       : OP == HOP_AND_I32 ? 0xFFFFFFFFu
       : OP == HOP_MUL_I32 ? 1u
       : 0u;                       // add (i32, f32: +0.0), u32 max, or, xor
}

// update of a bin, in shared or in global memory (generic address)
template <int OP>
__device__ __forceinline__ void upd_bin(uint32_t *p, uint32_t w) {
  if (OP == HOP_ADD_I32) atomicAdd(p, w);              // result unused: compiles to a reduction
  else if (OP == HOP_MAX_F32 || OP == HOP_MAX_U32) atomicMax(p, w);
  else if (OP == HOP_MIN_U32) atomicMin(p, w);
  else if (OP == HOP_MIN_I32) atomicMin(reinterpret_cast<int *>(p), (int)w);
  else if (OP == HOP_MAX_I32) atomicMax(reinterpret_cast<int *>(p), (int)w);
  else if (OP == HOP_AND_I32) atomicAnd(p, w);
  else if (OP == HOP_OR_I32) atomicOr(p, w);
  else if (OP == HOP_XOR_I32) atomicXor(p, w);
  else if (OP == HOP_ADD_F32) atomicAdd(reinterpret_cast<float *>(p), __uint_as_float(w));
  else {                                               // no native atomic: compare-and-swap until nobody interfered (Base.hs:844-905)
    uint32_t old = *reinterpret_cast<volatile uint32_t *>(p), assumed;
    do {
      assumed = old;
      old = atomicCAS(p, assumed, assumed * w);
    } while (old != assumed);
  }
}
template <int OP>
__device__ __forceinline__ void upd_shared(uint32_t *p, uint32_t w) { upd_bin<OP>(p, w); }
template <int OP>
__device__ __forceinline__ void upd_global(uint32_t *p, uint32_t w) { upd_bin<OP>(p, w); }
// two partial bins folded (the private copies of a CTA)
template <int OP>
__device__ __forceinline__ uint32_t fold_bins(uint32_t a, uint32_t b) {
  if (OP == HOP_ADD_I32) return a + b;
  if (OP == HOP_MAX_F32 || OP == HOP_MAX_U32) return a > b ? a : b;
  if (OP == HOP_MIN_U32) return a < b ? a : b;
  if (OP == HOP_MIN_I32) return (uint32_t)min((int)a, (int)b);
  if (OP == HOP_MAX_I32) return (uint32_t)max((int)a, (int)b);
  if (OP == HOP_AND_I32) return a & b;
  if (OP == HOP_OR_I32) return a | b;
  if (OP == HOP_XOR_I32) return a ^ b;
  if (OP == HOP_ADD_F32) return __float_as_uint(__uint_as_float(a) + __uint_as_float(b));
  return a * b;
}
// weight as stored in the accumulator; `skip` set for a NaN under the f32 max
template <int OP>
__device__ __forceinline__ uint32_t prep(uint32_t wbits, bool &skip) {
  if (OP != HOP_MAX_F32) { skip = false; return wbits; }
  const uint32_t key = f32_key(wbits);
  skip = key_is_winning_nan(key);
  return key;
}

// One update of a bin range [lo, lo + nb) held in shared memory (nb <= 57344, lo < 2^31).  A
// single unsigned comparison covers "below the range", "above it" and negative indices; the
// weight is only looked at for an index inside the range.
template <int OP>
__device__ __forceinline__ void upd_range(uint32_t *s_hist, int32_t bin, uint32_t wbits, int32_t lo, uint32_t nb,
                                          int log2c, uint32_t copy) {
  const uint32_t b = (uint32_t)(bin - lo);
  if (b < nb) {
    bool skip;
    const uint32_t w = prep<OP>(wbits, skip);
    if (!skip) upd_shared<OP>(&s_hist[(b << log2c) + copy], w);
  }
}

// ---- shared-memory path ------------------------------------------------------------------
// grid = groups * P CTAs; CTA (g, p) streams the vectors of group g and keeps bins in
// [p*range, min(B, (p+1)*range)).  log2c = log2 of the number of private copies.
template <int OP, bool VEC>
__global__ void __launch_bounds__(HIST_THREADS, 1)
hist_smem_kernel(const int32_t *__restrict__ bins, const uint32_t *__restrict__ ws, int64_t n, int64_t B,
                 int P, int64_t range, int log2c, uint32_t *__restrict__ out) {
  extern __shared__ __align__(16) uint32_t s_hist[];
  const int tid = threadIdx.x;
  const int p = blockIdx.x % P;
  const int64_t g = blockIdx.x / P, groups = gridDim.x / P;
  const int64_t bin_lo = (int64_t)p * range;
  const int64_t bin_hi = (bin_lo + range < B) ? bin_lo + range : B;
  const uint32_t nb = (uint32_t)(bin_hi - bin_lo);
  const uint32_t C = 1u << log2c;
  const uint32_t copy = (uint32_t)(tid & 31) & (C - 1);
  const uint32_t total = nb << log2c;
  for (uint32_t i = tid; i < total; i += HIST_THREADS) s_hist[i] = neutral<OP>();
  __syncthreads();

  if (VEC) {
    const int4 *bv = reinterpret_cast<const int4 *>(bins);
    const int4 *wv = reinterpret_cast<const int4 *>(ws);
    const int64_t nvec = n >> 2;
    const int64_t stride = groups * HIST_THREADS;
    int64_t i = g * HIST_THREADS + tid;
    for (; i + stride < nvec; i += 2 * stride) {
      int4 b0 = ld_stream_v4(bv + i), w0 = ld_stream_v4(wv + i);
      int4 b1 = ld_stream_v4(bv + i + stride), w1 = ld_stream_v4(wv + i + stride);
      const int bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
      const int ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
      for (int k = 0; k < 8; k++) upd_range<OP>(s_hist, bb[k], (uint32_t)ww[k], (int32_t)bin_lo, nb, log2c, copy);
    }
    for (; i < nvec; i += stride) {
      int4 b0 = ld_stream_v4(bv + i), w0 = ld_stream_v4(wv + i);
      const int bb[4] = {b0.x, b0.y, b0.z, b0.w};
      const int ww[4] = {w0.x, w0.y, w0.z, w0.w};
#pragma unroll
      for (int k = 0; k < 4; k++) upd_range<OP>(s_hist, bb[k], (uint32_t)ww[k], (int32_t)bin_lo, nb, log2c, copy);
    }
    // fewer than four trailing elements: the first group's CTAs take them
    if (g == 0) {
      const int64_t j = (nvec << 2) + tid;
      if (j < n) {
        const int64_t b = (int64_t)bins[j] - bin_lo;
        bool skip;
        const uint32_t w = prep<OP>(ws[j], skip);
        if (b >= 0 && b < (int64_t)nb && !skip) upd_shared<OP>(&s_hist[((uint32_t)b << log2c) + copy], w);
      }
    }
  } else {
    const int64_t stride = groups * HIST_THREADS;
    for (int64_t i = g * HIST_THREADS + tid; i < n; i += stride) {
      const int64_t b = (int64_t)bins[i] - bin_lo;
      bool skip;
      const uint32_t w = prep<OP>(ws[i], skip);
      if (b >= 0 && b < (int64_t)nb && !skip) upd_shared<OP>(&s_hist[((uint32_t)b << log2c) + copy], w);
    }
  }
  __syncthreads();
  // fold the copies and flush
  for (uint32_t b = tid; b < nb; b += HIST_THREADS) {
    uint32_t acc = neutral<OP>();
    for (uint32_t c = 0; c < C; c++) {
      // rotate the starting copy per bin so the lanes of a warp hit different banks
      const uint32_t v = s_hist[(b << log2c) + ((c + b) & (C - 1))];
      acc = fold_bins<OP>(acc, v);
    }
    if (acc != neutral<OP>()) upd_global<OP>(&out[bin_lo + b], acc);
  }
}

// ---- shared-memory path with the input staged through shared memory ----------------------------
// With P bin ranges every CTA needs P times the input bandwidth of its share of the result,
// so the bytes in flight per SM must grow P-fold too, and the registers of 1024 threads cannot
// hold them.  Where the histogram leaves room (two ranges of <= 33536 bins), every thread
// keeps HIST_STAGES 16-byte copies of indices and of weights in flight straight into shared
// memory (cp.async), three rounds ahead of its own reading; a thread reads back only what it
// copied itself, so no barrier is involved.  One private copy of the bins (log2c = 0).  With
// skewed indices (Zipf 1.1 over 65536 bins) the CTA whose range holds the most frequent bins
// runs ~13 % longer than its partner, falls behind it, and re-reads from HBM what has left L2
// meanwhile (measured: 1.47x the input), which then bounds the kernel.  Measured and not kept:
// combining equal bins across the warp first (match.any + warp reduction, 10x slower); the four
// most frequent bins of a CTA combined in registers (no faster, and slower for uniform
// indices); the CTAs of a group paced by a cluster barrier (Zipf 12 % faster, uniform max 9 %
// slower, three and four ranges slower; the same with the pair meeting only every 8th round and
// arriving 4 rounds before it waits: add 405 / 502 us, max 502 / 527 us for uniform / Zipf indices against
// 354 / 548 and 412 / 506 unpaced, so it is the cluster launch that costs); the CTAs of a group paced through progress counters
// in global memory, a CTA waiting only when it is more than 12-16 rounds ahead (uniform AND
// Zipf 3.4x - 6.5x slower: in this kernel a global load or store queues behind the SM's
// outstanding input requests for several microseconds, during which the grid streams ~50 MB,
// so a counter is that stale when it is read, which is most of what L2 can keep for the slower
// CTA; and a check that waits for its load drains the CTA's copy pipeline each time).  Cutting
// the bins by residue (bin mod P) instead of into contiguous ranges does not change the
// picture for this workload: the rank -> bin permutation already scatters the frequent bins
// over both ranges, and what makes one CTA slower is the single most frequent bin (12 % of
// all updates under Zipf 1.1), which lands in one CTA whatever the split.
constexpr int HIST_STAGES = 3;
constexpr int HIST_STAGE_BYTES = HIST_THREADS * 32;       // 16 bytes of indices + 16 bytes of weights per thread

__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int OP>
__global__ void __launch_bounds__(HIST_THREADS, 1)
hist_smem_async_kernel(const int32_t *__restrict__ bins, const uint32_t *__restrict__ ws, int64_t n, int64_t B,
                       int P, int64_t range, uint32_t *__restrict__ out) {
  extern __shared__ __align__(16) uint32_t s_hist[];
  const int tid = threadIdx.x;
  const int p = blockIdx.x % P;
  const int64_t g = blockIdx.x / P, groups = gridDim.x / P;
  const int64_t bin_lo = (int64_t)p * range;
  const int64_t bin_hi = (bin_lo + range < B) ? bin_lo + range : B;
  const uint32_t nb = (uint32_t)(bin_hi - bin_lo);
  // stages behind the histogram (range is a multiple of 4: 16-byte aligned)
  unsigned char *s_stage = reinterpret_cast<unsigned char *>(s_hist + range);
  for (uint32_t i = tid; i < nb; i += HIST_THREADS) s_hist[i] = neutral<OP>();
  __syncthreads();

  const int4 *bv = reinterpret_cast<const int4 *>(bins);
  const int4 *wv = reinterpret_cast<const int4 *>(ws);
  const int64_t nvec = n >> 2;
  const int64_t stride = groups * HIST_THREADS;
  const int64_t first = g * HIST_THREADS + tid;
  auto issue = [&](int64_t i, int s) {              // this thread's two vectors of round i into stage s
    if (i < nvec) {
      unsigned char *d = s_stage + s * HIST_STAGE_BYTES + tid * 16;
      cp_async16(d, bv + i);
      cp_async16(d + HIST_THREADS * 16, wv + i);
    }
    cp_async_commit();                               // an empty group keeps the count of groups in step
  };
#pragma unroll
  for (int s = 0; s < HIST_STAGES - 1; s++) issue(first + s * stride, s);
  int s = 0;
  for (int64_t i = first; i < nvec; i += stride) {
    int sn = s + HIST_STAGES - 1;
    if (sn >= HIST_STAGES) sn -= HIST_STAGES;
    issue(i + (HIST_STAGES - 1) * stride, sn);
    cp_async_wait<HIST_STAGES - 1>();
    const unsigned char *d = s_stage + s * HIST_STAGE_BYTES + tid * 16;
    const int4 b0 = *reinterpret_cast<const int4 *>(d);
    const int4 w0 = *reinterpret_cast<const int4 *>(d + HIST_THREADS * 16);
    const int bb[4] = {b0.x, b0.y, b0.z, b0.w};
    const int ww[4] = {w0.x, w0.y, w0.z, w0.w};
#pragma unroll
    for (int k = 0; k < 4; k++) upd_range<OP>(s_hist, bb[k], (uint32_t)ww[k], (int32_t)bin_lo, nb, 0, 0u);
    if (++s == HIST_STAGES) s = 0;
  }
  cp_async_wait<0>();
  if (g == 0) {                                      // fewer than four trailing elements
    const int64_t j = (nvec << 2) + tid;
    if (j < n) {
      const int64_t b = (int64_t)bins[j] - bin_lo;
      bool skip;
      const uint32_t w = prep<OP>(ws[j], skip);
      if (b >= 0 && b < (int64_t)nb && !skip) upd_shared<OP>(&s_hist[(uint32_t)b], w);
    }
  }
  __syncthreads();
  for (uint32_t b = tid; b < nb; b += HIST_THREADS) {
    const uint32_t v = s_hist[b];
    if (v != neutral<OP>()) upd_global<OP>(&out[bin_lo + b], v);
  }
}

// ---- global atomics behind a per-CTA cache of hot bins ---------------------------------------------
constexpr int HC_LOG2_SLOTS = 14;
constexpr uint32_t HC_SLOTS = 1u << HC_LOG2_SLOTS;       // 16384 x (tag, value) = 128 KiB
constexpr int32_t HC_EMPTY = -1;
constexpr int HC_PROBE_ROUNDS = 8;                       // grid-stride rounds after which the hit rate is judged

template <int OP>
__global__ void __launch_bounds__(HIST_THREADS, 1)
hist_cached_kernel(const int32_t *__restrict__ bins, const uint32_t *__restrict__ ws, int64_t n, int64_t B,
                   uint32_t *__restrict__ out) {
  extern __shared__ __align__(16) uint32_t s_mem[];
  int32_t *s_tag = reinterpret_cast<int32_t *>(s_mem);
  uint32_t *s_val = s_mem + HC_SLOTS;
  __shared__ uint32_t s_hits, s_seen;
  const int tid = threadIdx.x;
  for (uint32_t i = tid; i < HC_SLOTS; i += HIST_THREADS) { s_tag[i] = HC_EMPTY; s_val[i] = neutral<OP>(); }
  if (tid == 0) { s_hits = 0; s_seen = 0; }
  __syncthreads();

  uint32_t hits = 0, seen = 0;
  auto update = [&](int32_t bin, uint32_t wbits, bool use_cache) {
    bool skip;
    const uint32_t w = prep<OP>(wbits, skip);
    if (bin < 0 || (int64_t)bin >= B || skip) return;
    if (use_cache) {
      seen++;
      const uint32_t slot = ((uint32_t)bin * 0x9E3779B1u) >> (32 - HC_LOG2_SLOTS);
      int32_t t = *reinterpret_cast<volatile int32_t *>(&s_tag[slot]);
      if (t == HC_EMPTY) {
        const int32_t old = atomicCAS(&s_tag[slot], HC_EMPTY, bin);
        t = (old == HC_EMPTY) ? bin : old;
      }
      if (t == bin) { upd_shared<OP>(&s_val[slot], w); hits++; return; }
    }
    upd_global<OP>(&out[bin], w);
  };

  const bool vec = ((((uintptr_t)bins) | ((uintptr_t)ws)) & 15) == 0;
  const int64_t stride = (int64_t)gridDim.x * HIST_THREADS;
  bool use_cache = true;
  if (vec) {
    const int4 *bv = reinterpret_cast<const int4 *>(bins);
    const int4 *wv = reinterpret_cast<const int4 *>(ws);
    const int64_t nvec = n >> 2;
    int64_t i = (int64_t)blockIdx.x * HIST_THREADS + tid;
    int round = 0;
    // the hit rate is judged only where every thread of the CTA makes that many rounds
    const bool probe = (int64_t)blockIdx.x * HIST_THREADS + (HIST_THREADS - 1) + (int64_t)HC_PROBE_ROUNDS * stride < nvec;
    for (; i < nvec; i += stride, round++) {
      if (probe && round == HC_PROBE_ROUNDS) {
        atomicAdd(&s_hits, hits); atomicAdd(&s_seen, seen);
        __syncthreads();
        use_cache = (uint64_t)s_hits * 4u >= (uint64_t)s_seen;       // keep the cache if >= 25% of the updates hit
      }
      const int4 b0 = ld_stream_v4(bv + i), w0 = ld_stream_v4(wv + i);
      update(b0.x, w0.x, use_cache); update(b0.y, w0.y, use_cache);
      update(b0.z, w0.z, use_cache); update(b0.w, w0.w, use_cache);
    }
    if (blockIdx.x == 0) {               // fewer than four trailing elements
      const int64_t j = (nvec << 2) + tid;
      if (j < n) update(bins[j], ws[j], false);
    }
  } else {
    for (int64_t i = (int64_t)blockIdx.x * HIST_THREADS + tid; i < n; i += stride) update(bins[i], ws[i], true);
  }
  __syncthreads();
  for (uint32_t i = tid; i < HC_SLOTS; i += HIST_THREADS) {
    const int32_t t = s_tag[i];
    const uint32_t v = s_val[i];
    if (t != HC_EMPTY && v != neutral<OP>()) upd_global<OP>(&out[t], v);
  }
}

__global__ void fill_u32_kernel(uint32_t *p, int64_t n, uint32_t v) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) p[i] = v;
}
__global__ void decode_keys_kernel(uint32_t *p, int64_t n) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) p[i] = key_f32(p[i]);
}

static int grid_for(int64_t n, int threads, int cap) {
  int64_t want = (n + threads - 1) / threads;
  if (want < 1) want = 1;
  return (int)(want < cap ? want : cap);
}

template <int OP>
static cudaError_t launch_hist_op(int64_t B, const int32_t *bins, const uint32_t *ws, int64_t n, uint32_t *out,
                                  const uint32_t *dest, int num_sms, cudaStream_t stream) {
  // the result starts at the neutral element (hist, prelude/soacs.fut:132-133) or as a copy of the
  // destination (reduce_by_index, :117-130)
  cudaError_t err;
  if (dest != nullptr) {
    err = cudaMemcpyAsync(out, dest, (size_t)B * 4, cudaMemcpyDeviceToDevice, stream);
  } else {
    fill_u32_kernel<<<grid_for(B, 256, num_sms * 8), 256, 0, stream>>>(out, B, neutral<OP>());
    err = cudaGetLastError();
  }
  if (err != cudaSuccess) return err;
  if (n > 0) {
    const int64_t P64 = (B + HIST_CAP_BINS - 1) / HIST_CAP_BINS;
    if (P64 <= 4 && P64 <= num_sms) {
      const int P = (int)P64;
      const int64_t range = (B + P - 1) / P;
      int log2c = 0;
      while (log2c < 5 && (range << (log2c + 1)) <= HIST_CAP_BINS) log2c++;
      const size_t smem = (size_t)(range << log2c) * sizeof(uint32_t);
      const bool vec = ((((uintptr_t)bins) | ((uintptr_t)ws)) & 15) == 0;
      int64_t max_groups = (n / 4 + HIST_THREADS - 1) / HIST_THREADS;
      if (max_groups < 1) max_groups = 1;
      int64_t groups = num_sms / P;
      if (groups > max_groups) groups = max_groups;
      const int grid = (int)groups * P;
      const int64_t range4 = (range + 3) & ~(int64_t)3;
      const size_t smem_async = (size_t)range4 * sizeof(uint32_t) + (size_t)HIST_STAGES * HIST_STAGE_BYTES;
      if (P > 1 && vec && smem_async <= (size_t)HIST_CAP_BINS * 4) {
        auto kern = hist_smem_async_kernel<OP>;
        err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(HIST_CAP_BINS * 4));
        if (err != cudaSuccess) return err;
        kern<<<grid, HIST_THREADS, smem_async, stream>>>(bins, ws, n, B, P, range4, out);
      } else {
        auto kern = vec ? hist_smem_kernel<OP, true> : hist_smem_kernel<OP, false>;
        err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(HIST_CAP_BINS * 4));
        if (err != cudaSuccess) return err;
        kern<<<grid, HIST_THREADS, smem, stream>>>(bins, ws, n, B, P, range, log2c, out);
      }
    } else {
      auto kern = hist_cached_kernel<OP>;
      const size_t smem = (size_t)HC_SLOTS * 8;
      err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (err != cudaSuccess) return err;
      int64_t want = (n / 4 + HIST_THREADS - 1) / HIST_THREADS;
      if (want < 1) want = 1;
      const int grid = (int)(want < num_sms ? want : num_sms);
      kern<<<grid, HIST_THREADS, smem, stream>>>(bins, ws, n, B, out);
    }
    err = cudaGetLastError();
    if (err != cudaSuccess) return err;
  }
  if (OP == HOP_MAX_F32) {
    decode_keys_kernel<<<grid_for(B, 256, num_sms * 8), 256, 0, stream>>>(out, B);
    err = cudaGetLastError();
  }
  return err;
}

cudaError_t launch_hist(int op, int64_t B, const int32_t *bins, const void *weights, int64_t n, void *out,
                        const void *dest, int num_sms, cudaStream_t stream) {
  if (B <= 0) return cudaSuccess;
  const uint32_t *w = reinterpret_cast<const uint32_t *>(weights), *d = reinterpret_cast<const uint32_t *>(dest);
  uint32_t *o = reinterpret_cast<uint32_t *>(out);
  switch (op) {
    case HOP_ADD_I32: return launch_hist_op<HOP_ADD_I32>(B, bins, w, n, o, d, num_sms, stream);
    case HOP_MAX_F32: return dest != nullptr ? cudaErrorInvalidValue : launch_hist_op<HOP_MAX_F32>(B, bins, w, n, o, d, num_sms, stream);
    case HOP_MIN_I32: return launch_hist_op<HOP_MIN_I32>(B, bins, w, n, o, d, num_sms, stream);
    case HOP_MAX_I32: return launch_hist_op<HOP_MAX_I32>(B, bins, w, n, o, d, num_sms, stream);
    case HOP_MIN_U32: return launch_hist_op<HOP_MIN_U32>(B, bins, w, n, o, d, num_sms, stream);
    case HOP_MAX_U32: return launch_hist_op<HOP_MAX_U32>(B, bins, w, n, o, d, num_sms, stream);
    case HOP_AND_I32: return launch_hist_op<HOP_AND_I32>(B, bins, w, n, o, d, num_sms, stream);
    case HOP_OR_I32: return launch_hist_op<HOP_OR_I32>(B, bins, w, n, o, d, num_sms, stream);
    case HOP_XOR_I32: return launch_hist_op<HOP_XOR_I32>(B, bins, w, n, o, d, num_sms, stream);
    case HOP_ADD_F32: return launch_hist_op<HOP_ADD_F32>(B, bins, w, n, o, d, num_sms, stream);
    case HOP_MUL_I32: return launch_hist_op<HOP_MUL_I32>(B, bins, w, n, o, d, num_sms, stream);
    default: return cudaErrorInvalidValue;
  }
}

// ---- index spaces with more than one dimension -----------------------------------------------------
// A histogram per row of [rows][cols] (segment dimension of the SegHist, SegHist.hs:97-148) is one
// histogram over rows * B bins whose index carries the row; reduce_by_index_2d
// (prelude/soacs.fut:149-152) is one over n * m bins.  These kernels write that flat index, -1 for
// what is out of range in any dimension.
__global__ void __launch_bounds__(256)
flatten_rows_index_kernel(const int32_t *__restrict__ is, int64_t n, int64_t cols, int64_t B, int32_t *__restrict__ flat) {
  const int64_t stride = (int64_t)gridDim.x * 256;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += stride) {
    const int32_t b = is[i];
    flat[i] = (b >= 0 && (int64_t)b < B) ? (int32_t)((i / cols) * B + b) : -1;
  }
}
__global__ void __launch_bounds__(256)
flatten_2d_index_kernel(const int64_t *__restrict__ is, const int64_t *__restrict__ js, int64_t n, int64_t N, int64_t M,
                        int32_t *__restrict__ flat) {
  const int64_t stride = (int64_t)gridDim.x * 256;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += stride) {
    const int64_t a = is[i], b = js[i];
    flat[i] = (a >= 0 && a < N && b >= 0 && b < M) ? (int32_t)(a * M + b) : -1;
  }
}
__global__ void __launch_bounds__(256)
flatten_3d_index_kernel(const int64_t *__restrict__ is, const int64_t *__restrict__ js, const int64_t *__restrict__ ks, int64_t n, int64_t K,
                        int64_t M, int64_t L, int32_t *__restrict__ flat) {
  const int64_t stride = (int64_t)gridDim.x * 256;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += stride) {
    const int64_t a = is[i], b = js[i], c = ks[i];
    flat[i] = (a >= 0 && a < K && b >= 0 && b < M && c >= 0 && c < L) ? (int32_t)((a * M + b) * L + c) : -1;
  }
}
// a 2-D histogram per row of [rows][cols] index pairs: flat = (row * N + x) * M + y
__global__ void __launch_bounds__(256)
flatten_rows_2d_index_kernel(const int32_t *__restrict__ xs, const int32_t *__restrict__ ys, int64_t n, int64_t cols, int64_t N, int64_t M,
                             int32_t *__restrict__ flat) {
  const int64_t stride = (int64_t)gridDim.x * 256;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += stride) {
    const int64_t x = xs[i], y = ys[i];
    flat[i] = (x >= 0 && x < N && y >= 0 && y < M) ? (int32_t)(((i / cols) * N + x) * M + y) : -1;
  }
}
cudaError_t launch_flatten_3d_index(const int64_t *is, const int64_t *js, const int64_t *ks, int64_t n, int64_t K, int64_t M, int64_t L,
                                    int32_t *flat, int num_sms, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  flatten_3d_index_kernel<<<grid_for(n, 256, num_sms * 8), 256, 0, stream>>>(is, js, ks, n, K, M, L, flat);
  return cudaGetLastError();
}
cudaError_t launch_flatten_rows_2d_index(const int32_t *xs, const int32_t *ys, int64_t n, int64_t cols, int64_t N, int64_t M, int32_t *flat,
                                         int num_sms, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  flatten_rows_2d_index_kernel<<<grid_for(n, 256, num_sms * 8), 256, 0, stream>>>(xs, ys, n, cols, N, M, flat);
  return cudaGetLastError();
}
cudaError_t launch_flatten_rows_index(const int32_t *is, int64_t n, int64_t cols, int64_t B, int32_t *flat, int num_sms, cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  flatten_rows_index_kernel<<<grid_for(n, 256, num_sms * 8), 256, 0, stream>>>(is, n, cols, B, flat);
  return cudaGetLastError();
}
cudaError_t launch_flatten_2d_index(const int64_t *is, const int64_t *js, int64_t n, int64_t N, int64_t M, int32_t *flat, int num_sms,
                                    cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  flatten_2d_index_kernel<<<grid_for(n, 256, num_sms * 8), 256, 0, stream>>>(is, js, n, N, M, flat);
  return cudaGetLastError();
}

// ---- 8-byte values: atomics straight to the result in global memory --------------------------------
// The reference's histKernelGlobal (SegHist.hs:377-560) with one sub-histogram: every update is an
// atomic on the result array, a native one where the hardware has it for the operator and type
// (Base.hs:720-760 picks; f64 addition is native here).  The result starts as a copy of dest.
__global__ void __launch_bounds__(256) hist_global_add_f64_kernel(const int32_t *__restrict__ bins, const double *__restrict__ vs, int64_t n,
                                                                 int64_t B, double *out) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const int32_t b = bins[i];
    if (b >= 0 && (int64_t)b < B) atomicAdd(&out[b], vs[i]);
  }
}
cudaError_t launch_hist_add_f64(int64_t B, const int32_t *bins, const double *vs, int64_t n, double *out, const double *dest, int num_sms,
                                cudaStream_t stream) {
  if (B <= 0) return cudaSuccess;
  cudaError_t err = cudaMemcpyAsync(out, dest, (size_t)B * sizeof(double), cudaMemcpyDeviceToDevice, stream);
  if (err != cudaSuccess || n <= 0) return err;
  int64_t grid = (n + 255) / 256;
  if (grid > (int64_t)num_sms * 8) grid = (int64_t)num_sms * 8;
  hist_global_add_f64_kernel<<<(int)grid, 256, 0, stream>>>(bins, vs, n, B, out);
  return cudaGetLastError();
}

// ---- 1- and 2-byte values: compare-and-swap on the 32-bit word that holds the element ---------------
// What the reference generates for element types without an atomic of their own (Base.hs:844-905): read
// the word, combine inside it, try to swap it in, repeat while somebody else got there first.
struct SwAddI8 {
  using V = uint8_t; using I = int8_t;
  static __device__ __forceinline__ uint32_t combine(uint32_t cur, uint32_t v) { return (cur + v) & 0xffu; }
};
struct SwAddI16 {
  using V = uint16_t; using I = int16_t;
  static __device__ __forceinline__ uint32_t combine(uint32_t cur, uint32_t v) { return (cur + v) & 0xffffu; }
};
// f32 -> binary16 bits by truncation (round toward zero), NaN payloads cut to their top ten bits: the
// arithmetic of the reference's table-driven float2halfbits (rts/c/half.h:220-228)
__device__ __forceinline__ uint32_t float_to_half_trunc(float f) {
  const uint32_t bits = __float_as_uint(f), sign = (bits >> 16) & 0x8000u, e = (bits >> 23) & 0xffu, m = bits & 0x7fffffu;
  if (e == 255u) return sign | 0x7c00u | (m >> 13);
  if (e > 142u) return sign | 0x7c00u;                               // 2^16 and beyond: infinity
  if (e >= 113u) return sign | ((e - 112u) << 10) | (m >> 13);      // normal numbers
  if (e >= 103u) return sign | ((0x0400u >> (113u - e)) + (m >> (126u - e)));   // subnormal numbers
  return sign;
}
struct SwAddF16 {
  using V = uint16_t; using I = int16_t;
  static __device__ __forceinline__ uint32_t combine(uint32_t cur, uint32_t v) {
    const float s = __half2float(__ushort_as_half((unsigned short)cur)) + __half2float(__ushort_as_half((unsigned short)v));
    return float_to_half_trunc(s);
  }
};
template <class S>
__global__ void __launch_bounds__(256) hist_global_cas_kernel(const typename S::I *__restrict__ bins, const typename S::V *__restrict__ vs,
                                                             int64_t n, int64_t B, typename S::V *out) {
  using V = typename S::V;
  constexpr uint32_t BITS = 8 * sizeof(V), MASK = (1u << BITS) - 1u;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const int64_t b = (int64_t)bins[i];                             // sign-extended, as i64.i8 / i64.i16
    if (b < 0 || b >= B) continue;
    const uintptr_t addr = reinterpret_cast<uintptr_t>(out + b);
    uint32_t *word = reinterpret_cast<uint32_t *>(addr & ~(uintptr_t)3);
    const uint32_t shift = (uint32_t)(addr & 3u) * 8u;
    const uint32_t v = (uint32_t)vs[i];
    uint32_t old = *reinterpret_cast<volatile uint32_t *>(word), assumed;
    do {
      assumed = old;
      const uint32_t nv = S::combine((assumed >> shift) & MASK, v);
      old = atomicCAS(word, assumed, (assumed & ~(MASK << shift)) | (nv << shift));
    } while (old != assumed);
  }
}
template <class S>
static cudaError_t launch_hist_cas(int64_t B, const void *bins, const void *vs, int64_t n, void *out, const void *dest, int num_sms, cudaStream_t stream,
                                   int fill_byte = 0) {      // dest == NULL: every byte of the result starts as fill_byte
  using V = typename S::V;
  if (B <= 0) return cudaSuccess;
  cudaError_t err = dest != nullptr ? cudaMemcpyAsync(out, dest, (size_t)B * sizeof(V), cudaMemcpyDeviceToDevice, stream)
                                    : cudaMemsetAsync(out, fill_byte, (size_t)B * sizeof(V), stream);
  if (err != cudaSuccess || n <= 0) return err;
  int64_t grid = (n + 255) / 256;
  if (grid > (int64_t)num_sms * 8) grid = (int64_t)num_sms * 8;
  hist_global_cas_kernel<S><<<(int)grid, 256, 0, stream>>>(reinterpret_cast<const typename S::I *>(bins), reinterpret_cast<const V *>(vs), n, B,
                                                          reinterpret_cast<V *>(out));
  return cudaGetLastError();
}
// `out` must be readable and writable up to the next multiple of 4 bytes (pooled blocks are)
cudaError_t launch_hist_add_subword(int kind, int64_t B, const void *bins, const void *vs, int64_t n, void *out, const void *dest, int num_sms,
                                    cudaStream_t stream) {
  switch (kind) {
    case 0: return launch_hist_cas<SwAddI8>(B, bins, vs, n, out, dest, num_sms, stream);
    case 1: return launch_hist_cas<SwAddI16>(B, bins, vs, n, out, dest, num_sms, stream);
    default: return launch_hist_cas<SwAddF16>(B, bins, vs, n, out, dest, num_sms, stream);
  }
}

// ---- 1- and 2-byte integers under min, max, and, or, xor; indices are i32 -----------------------------
// tests/hist/{min,max,and,or,xor}{8,16}.fut: the same compare-and-swap loop on the containing word under
// other operators; signed minimum and maximum compare the sign-extended sub-words.
template <typename VT, int OP>
struct SwNarrow {
  using V = VT; using I = int32_t;
  static __device__ __forceinline__ uint32_t combine(uint32_t cur, uint32_t v) {
    constexpr int SH = 32 - 8 * (int)sizeof(VT);
    constexpr uint32_t MASK = 0xffffffffu >> SH;
    const int32_t sc = (int32_t)(cur << SH) >> SH, sv = (int32_t)(v << SH) >> SH;
    if (OP == NOP_MIN_S) return (uint32_t)(sv < sc ? sv : sc) & MASK;
    if (OP == NOP_MAX_S) return (uint32_t)(sv > sc ? sv : sc) & MASK;
    if (OP == NOP_MIN_U) return v < cur ? v : cur;
    if (OP == NOP_MAX_U) return v > cur ? v : cur;
    if (OP == NOP_AND) return cur & v;
    if (OP == NOP_OR) return cur | v;
    return cur ^ v;
  }
};
template <typename VT>
static cudaError_t launch_hist_narrow_t(int op, int64_t B, const void *bins, const void *vs, int64_t n, void *out, const void *dest,
                                        int num_sms, cudaStream_t stream) {
  switch (op) {
    case NOP_MIN_S: return launch_hist_cas<SwNarrow<VT, NOP_MIN_S>>(B, bins, vs, n, out, dest, num_sms, stream);
    case NOP_MAX_S: return launch_hist_cas<SwNarrow<VT, NOP_MAX_S>>(B, bins, vs, n, out, dest, num_sms, stream);
    case NOP_MIN_U: return launch_hist_cas<SwNarrow<VT, NOP_MIN_U>>(B, bins, vs, n, out, dest, num_sms, stream);
    case NOP_MAX_U: return launch_hist_cas<SwNarrow<VT, NOP_MAX_U>>(B, bins, vs, n, out, dest, num_sms, stream);
    case NOP_AND: return launch_hist_cas<SwNarrow<VT, NOP_AND>>(B, bins, vs, n, out, dest, num_sms, stream, 0xff);
    case NOP_OR: return launch_hist_cas<SwNarrow<VT, NOP_OR>>(B, bins, vs, n, out, dest, num_sms, stream);
    case NOP_XOR: return launch_hist_cas<SwNarrow<VT, NOP_XOR>>(B, bins, vs, n, out, dest, num_sms, stream);
    default: return cudaErrorInvalidValue;
  }
}
cudaError_t launch_hist_narrow(int op, int elem_bytes, int64_t B, const int32_t *bins, const void *vs, int64_t n, void *out, const void *dest,
                               int num_sms, cudaStream_t stream) {
  if (dest == nullptr && op != NOP_AND && op != NOP_OR && op != NOP_XOR) return cudaErrorInvalidValue;
  if (elem_bytes == 1) return launch_hist_narrow_t<uint8_t>(op, B, bins, vs, n, out, dest, num_sms, stream);
  if (elem_bytes == 2) return launch_hist_narrow_t<uint16_t>(op, B, bins, vs, n, out, dest, num_sms, stream);
  return cudaErrorInvalidValue;
}

// ---- 8-byte integers under and, or, xor, the i32 values widened in the kernel -------------------------
// hist (i64.&) (-1) n (map i64.i32 is) (map i64.i32 image) (tests/hist/and64.fut, xor64.fut): native 64-bit
// atomics on the result (Base.hs:720-760), which starts at the operator's neutral element.
template <int OP>
__global__ void __launch_bounds__(256) hist_global_bitop_i64_kernel(const int32_t *__restrict__ bins, const int32_t *__restrict__ vs, int64_t n,
                                                                   int64_t B, unsigned long long *out) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const int32_t b = bins[i];
    if (b < 0 || (int64_t)b >= B) continue;
    const unsigned long long v = (unsigned long long)(long long)vs[i];       // i64.i32 extends the sign
    if (OP == NOP_AND) atomicAnd(&out[b], v);
    else if (OP == NOP_OR) atomicOr(&out[b], v);
    else atomicXor(&out[b], v);
  }
}
cudaError_t launch_hist_bitop_i64(int op, int64_t B, const int32_t *bins, const int32_t *vs, int64_t n, int64_t *out, int num_sms,
                                  cudaStream_t stream) {
  if (B <= 0) return cudaSuccess;
  if (op != NOP_AND && op != NOP_OR && op != NOP_XOR) return cudaErrorInvalidValue;
  cudaError_t err = cudaMemsetAsync(out, op == NOP_AND ? 0xff : 0x00, (size_t)B * sizeof(int64_t), stream);
  if (err != cudaSuccess || n <= 0) return err;
  int64_t grid = (n + 255) / 256;
  if (grid > (int64_t)num_sms * 8) grid = (int64_t)num_sms * 8;
  unsigned long long *o = reinterpret_cast<unsigned long long *>(out);
  if (op == NOP_AND) hist_global_bitop_i64_kernel<NOP_AND><<<(int)grid, 256, 0, stream>>>(bins, vs, n, B, o);
  else if (op == NOP_OR) hist_global_bitop_i64_kernel<NOP_OR><<<(int)grid, 256, 0, stream>>>(bins, vs, n, B, o);
  else hist_global_bitop_i64_kernel<NOP_XOR><<<(int)grid, 256, 0, stream>>>(bins, vs, n, B, o);
  return cudaGetLastError();
}

// ---- a vectorised operator: every bin is a row of `m` values ----------------------------------------------
// reduce_by_index xs (map2 (+)) (replicate m 0) is vss (tests/hist/array.fut; HistOp's operator shape,
// src/Futhark/IR/SegOp.hs:102-115): the update of row is[i] by the vector vss[i] is m scalar updates, so it is
// one histogram over n * m bins whose indices this kernel writes: flat[i * m + j] = is[i] * m + j, or -1.
__global__ void __launch_bounds__(256)
flatten_vec_index_kernel(const int64_t *__restrict__ is, int64_t k, int64_t n, int64_t m, int32_t *__restrict__ flat) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x, total = k * m;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride) {
    const int64_t i = t / m, j = t - i * m, b = is[i];
    flat[t] = (b >= 0 && b < n) ? (int32_t)(b * m + j) : -1;
  }
}
cudaError_t launch_flatten_vec_index(const int64_t *is, int64_t k, int64_t n, int64_t m, int32_t *flat, int num_sms, cudaStream_t stream) {
  if (k * m <= 0) return cudaSuccess;
  flatten_vec_index_kernel<<<grid_for(k * m, 256, num_sms * 8), 256, 0, stream>>>(is, k, n, m, flat);
  return cudaGetLastError();
}

// The same under a segment dimension (tests/hist/segmented_arr.fut): a histogram of k-vectors per row of
// [rows][cols] indices; flat[(r * cols + i) * k + j] = (r * m + iss[r][i]) * k + j, or -1.
__global__ void __launch_bounds__(256)
flatten_rows_vec_index_kernel(const int32_t *__restrict__ iss, int64_t elems, int64_t cols, int64_t m, int64_t k, int32_t *__restrict__ flat) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x, total = elems * k;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride) {
    const int64_t e = t / k, j = t - e * k, r = e / cols, b = iss[e];
    flat[t] = (b >= 0 && b < m) ? (int32_t)((r * m + b) * k + j) : -1;
  }
}
cudaError_t launch_flatten_rows_vec_index(const int32_t *iss, int64_t rows, int64_t cols, int64_t m, int64_t k, int32_t *flat, int num_sms,
                                          cudaStream_t stream) {
  const int64_t total = rows * cols * k;
  if (total <= 0) return cudaSuccess;
  flatten_rows_vec_index_kernel<<<grid_for(total, 256, num_sms * 8), 256, 0, stream>>>(iss, rows * cols, cols, m, k, flat);
  return cudaGetLastError();
}

// ---- an operator on pairs: the smaller first component wins and carries its second along ----------------
// tests/hist/tuple_partial.fut:19-22: op (x0, y0) (x1, y1) = if x0 != -1 && (x1 == -1 || x0 < x1) then (x0, y0)
// else (x1, y1), neutral (-1, -1).  The reference guards such an update with a lock per bin
// (atomicUpdateLocking, Base.hs:769-842); here a pair is one 64-bit word, updated by compare-and-swap, and
// the two result arrays are written from the words afterwards.  Where two updates of a bin have equal first
// components the operator keeps its right operand, so, as in the reference, the order decides.
__global__ void __launch_bounds__(256)
hist_minpair_kernel(const int32_t *__restrict__ bins, const int32_t *__restrict__ v0, const int32_t *__restrict__ v1, int64_t n, int64_t B,
                    unsigned long long *__restrict__ packed) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const int32_t b = bins[i];
    if (b < 0 || (int64_t)b >= B) continue;
    const int32_t x1 = v0[i];
    const unsigned long long mine = ((unsigned long long)(uint32_t)x1 << 32) | (uint32_t)v1[i];
    unsigned long long old = *reinterpret_cast<volatile unsigned long long *>(&packed[b]), assumed;
    do {
      assumed = old;
      const int32_t x0 = (int32_t)(uint32_t)(assumed >> 32);
      if (x0 != -1 && (x1 == -1 || x0 < x1)) break;                 // the bin keeps what it has
      old = atomicCAS(&packed[b], assumed, mine);
    } while (old != assumed);
  }
}
__global__ void __launch_bounds__(256) unpack_pairs_kernel(const unsigned long long *__restrict__ packed, int64_t B, int32_t *__restrict__ out0,
                                                          int32_t *__restrict__ out1) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; b < B; b += stride) {
    const unsigned long long w = packed[b];
    out0[b] = (int32_t)(uint32_t)(w >> 32);
    out1[b] = (int32_t)(uint32_t)w;
  }
}
// `packed`: B 8-byte words of scratch
cudaError_t launch_hist_minpair_i32(int64_t B, const int32_t *bins, const int32_t *v0, const int32_t *v1, int64_t n, void *packed, int32_t *out0,
                                    int32_t *out1, int num_sms, cudaStream_t stream) {
  if (B <= 0) return cudaSuccess;
  unsigned long long *p = reinterpret_cast<unsigned long long *>(packed);
  cudaError_t err = cudaMemsetAsync(p, 0xff, (size_t)B * 8, stream);          // (-1, -1) everywhere
  if (err != cudaSuccess) return err;
  if (n > 0) {
    hist_minpair_kernel<<<grid_for(n, 256, num_sms * 8), 256, 0, stream>>>(bins, v0, v1, n, B, p);
    err = cudaGetLastError();
    if (err != cudaSuccess) return err;
  }
  unpack_pairs_kernel<<<grid_for(B, 256, num_sms * 8), 256, 0, stream>>>(p, B, out0, out1);
  return cudaGetLastError();
}

}  // namespace fb
