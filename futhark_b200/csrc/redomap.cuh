// A fused redomap (map body + one or several reduction operators in one pass over HBM) as a
// kernel template over a *specification* type, so that a new entry point of this shape needs
// a specification and not a new kernel.  The reference fuses an arbitrary map body and up to
// 25 operators into one generated segred_nonseg kernel
// (src/Futhark/CodeGen/ImpGen/GPU/SegRed.hs:99-100,129-145,327-394) and keeps the operand order
// of non-commutative operators by reading windows through shared memory (:836-921).
//
// A specification provides
//   using Acc                      the accumulator: all operators' values side by side, a
//                                  trivially copyable struct of 1..4 32-bit words
//   static constexpr bool commutative
//   static constexpr int NIN       1 or 2 input arrays of 4-byte elements (map or map2)
//   static Acc neutral()           the neutral element(s)
//   static Acc map(uint32_t bits [, uint32_t bits2])   the map body on one element of each input
//   static Acc combine(Acc l, Acc r)   l (+) r, associative
//
// Operand order.  Every warp owns a contiguous run of *steps* (a step = 32 * K vectors of
// 16 bytes per input, read coalesced; K = RM_K, or 2 or 3 with two inputs to bound the registers).
// A commutative specification folds each lane's vectors as they come.  Otherwise a step goes through a warp-private shared-memory area that turns the
// coalesced layout into a blocked one (lane l then holds vectors l*K .. l*K+K-1 of each input; K
// is odd, which makes these 16-byte reads conflict-free), the lane folds its 4*K consecutive
// elements left to right and a shuffle tree that keeps lane order folds the 32 lanes.  Warp,
// CTA and grid partials are folded in index order as well.
#pragma once
#include <string.h>
#include <type_traits>

#include "common.cuh"

namespace fb {

constexpr int RM_THREADS = 256;
constexpr int RM_WARPS = RM_THREADS / 32;
constexpr int RM_K = 5;
constexpr int RM_MAX_BLOCKS = 4096;
// vectors per lane, input and step: 2 with two inputs to bound the registers, 3 when their operand
// order matters as well (odd: the blocked 16-byte reads of the transposition are conflict-free)
template <class Spec> struct RedomapK { static constexpr int K = Spec::NIN == 2 ? (Spec::commutative ? 2 : 3) : RM_K; };

template <class Acc>
__device__ __forceinline__ Acc shfl_down_acc(const Acc &a, int d) {
  static_assert(sizeof(Acc) % 4 == 0 && sizeof(Acc) <= 16, "an accumulator is 1..4 32-bit words");
  constexpr int W = sizeof(Acc) / 4;
  uint32_t w[W];
  memcpy(w, &a, sizeof(Acc));
#pragma unroll
  for (int i = 0; i < W; i++) w[i] = __shfl_down_sync(kFull, w[i], d);
  Acc r;
  memcpy(&r, w, sizeof(Acc));
  return r;
}

// Fold of the 32 lanes' values in lane order; the result is in lane 0.
template <class Spec>
__device__ __forceinline__ typename Spec::Acc warp_fold_ordered(typename Spec::Acc a, int lane) {
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const typename Spec::Acc o = shfl_down_acc(a, d);
    if (lane + d < 32) a = Spec::combine(a, o);
  }
  return a;
}

template <class Spec>
__device__ __forceinline__ typename Spec::Acc fold_vec(typename Spec::Acc a, const int4 &v) {
  a = Spec::combine(a, Spec::map((uint32_t)v.x));
  a = Spec::combine(a, Spec::map((uint32_t)v.y));
  a = Spec::combine(a, Spec::map((uint32_t)v.z));
  a = Spec::combine(a, Spec::map((uint32_t)v.w));
  return a;
}
template <class Spec>
__device__ __forceinline__ typename Spec::Acc fold_vec(typename Spec::Acc a, const uint32_t &v) {
  return Spec::combine(a, Spec::map(v));
}
template <class Spec>
__device__ __forceinline__ typename Spec::Acc fold_vec(typename Spec::Acc a, const int4 &v, const int4 &w) {
  a = Spec::combine(a, Spec::map((uint32_t)v.x, (uint32_t)w.x));
  a = Spec::combine(a, Spec::map((uint32_t)v.y, (uint32_t)w.y));
  a = Spec::combine(a, Spec::map((uint32_t)v.z, (uint32_t)w.z));
  a = Spec::combine(a, Spec::map((uint32_t)v.w, (uint32_t)w.w));
  return a;
}
template <class Spec>
__device__ __forceinline__ typename Spec::Acc fold_vec(typename Spec::Acc a, const uint32_t &v, const uint32_t &w) {
  return Spec::combine(a, Spec::map(v, w));
}

// VEC: the inputs are 16-byte aligned and read as int4; the n % 4 last elements are folded in by
// the thread that writes the result.  Otherwise one element per load.
template <class Spec, bool VEC>
__global__ void __launch_bounds__(RM_THREADS)
redomap_kernel(const uint32_t *__restrict__ in, const uint32_t *__restrict__ in2, int64_t n,
               typename Spec::Acc *__restrict__ d_out, uint32_t *ticket, typename Spec::Acc *partials) {
  using Acc = typename Spec::Acc;
  using Vec = typename std::conditional<VEC, int4, uint32_t>::type;
  constexpr bool ORDERED = !Spec::commutative;
  constexpr int NIN = Spec::NIN;
  static_assert(NIN == 1 || NIN == 2, "one or two input arrays");
  constexpr int K = RedomapK<Spec>::K;
  __shared__ Vec s_tr[ORDERED ? RM_WARPS * 32 * K * NIN : 1];
  __shared__ Acc s_warp[RM_WARPS];
  __shared__ uint32_t s_last;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const Vec *vec = reinterpret_cast<const Vec *>(in);
  const Vec *vec2 = reinterpret_cast<const Vec *>(in2);
  const int64_t nvec = VEC ? (n >> 2) : n;
  constexpr int64_t STEP = 32 * K;
  const int64_t steps = (nvec + STEP - 1) / STEP;
  const int64_t nwarps = (int64_t)gridDim.x * RM_WARPS;
  const int64_t per = (steps + nwarps - 1) / nwarps;
  const int64_t s0 = ((int64_t)blockIdx.x * RM_WARPS + warp) * per;
  const int64_t s1 = s0 + per < steps ? s0 + per : steps;

  auto ld = [&](const Vec *p) {
    if constexpr (VEC) return ld_stream_v4(p);
    else return *p;
  };
  Acc acc = Spec::neutral();              // ORDERED: meaningful in lane 0 only
  Vec cur[NIN][K], nxt[NIN][K];
  auto load = [&](Vec (&v)[NIN][K], int64_t s) {
    const int64_t base = s * STEP + lane;
    if (base - lane + STEP <= nvec) {
#pragma unroll
      for (int j = 0; j < K; j++) {
        v[0][j] = ld(vec + base + j * 32);
        if constexpr (NIN == 2) v[1][j] = ld(vec2 + base + j * 32);
      }
    }
  };
  if (s0 < s1) load(cur, s0);
  for (int64_t s = s0; s < s1; s++) {
    if (s + 1 < s1) load(nxt, s + 1);
    const int64_t base = s * STEP;
    if (base + STEP <= nvec) {
      if constexpr (ORDERED) {
        Vec *mine = s_tr + warp * (32 * K * NIN);
        __syncwarp();
#pragma unroll
        for (int j = 0; j < K; j++) {
          mine[j * 32 + lane] = cur[0][j];
          if constexpr (NIN == 2) mine[32 * K + j * 32 + lane] = cur[1][j];
        }
        __syncwarp();
        Acc a = Spec::neutral();
#pragma unroll
        for (int j = 0; j < K; j++) {
          if constexpr (NIN == 2) a = fold_vec<Spec>(a, mine[lane * K + j], mine[32 * K + lane * K + j]);
          else a = fold_vec<Spec>(a, mine[lane * K + j]);
        }
        a = warp_fold_ordered<Spec>(a, lane);
        acc = Spec::combine(acc, a);
      } else {
#pragma unroll
        for (int j = 0; j < K; j++) {
          if constexpr (NIN == 2) acc = fold_vec<Spec>(acc, cur[0][j], cur[1][j]);
          else acc = fold_vec<Spec>(acc, cur[0][j]);
        }
      }
    } else {
      // the one ragged step at the end of the input: row by row, absent vectors count as neutral
      for (int j = 0; j < K; j++) {
        const int64_t idx = base + j * 32 + lane;
        Acc a = Spec::neutral();
        if (idx < nvec) {
          if constexpr (NIN == 2) a = fold_vec<Spec>(a, vec[idx], vec2[idx]);
          else a = fold_vec<Spec>(a, vec[idx]);
        }
        if (ORDERED) { a = warp_fold_ordered<Spec>(a, lane); acc = Spec::combine(acc, a); }
        else acc = Spec::combine(acc, a);
      }
    }
#pragma unroll
    for (int j = 0; j < K; j++) {
      cur[0][j] = nxt[0][j];
      if constexpr (NIN == 2) cur[1][j] = nxt[1][j];
    }
  }
  if (!ORDERED) acc = warp_fold_ordered<Spec>(acc, lane);
  if (lane == 0) s_warp[warp] = acc;
  __syncthreads();
  if (warp == 0) {
    Acc b = (lane < RM_WARPS) ? s_warp[lane] : Spec::neutral();
    b = warp_fold_ordered<Spec>(b, lane);
    if (lane == 0) {
      partials[blockIdx.x] = b;
      __threadfence();
      const uint32_t t = atomicAdd(ticket, 1u);
      s_last = (t == gridDim.x - 1) ? 1u : 0u;
    }
  }
  __syncthreads();
  if (!s_last) return;
  // the CTA that drew the last ticket folds the per-CTA partials, each thread a contiguous range
  __threadfence();
  const int P = (int)gridDim.x;
  const int c = (P + RM_THREADS - 1) / RM_THREADS;
  Acc r = Spec::neutral();
  for (int j = tid * c; j < (tid + 1) * c && j < P; j++) {
    Acc p;
    const volatile uint32_t *src = reinterpret_cast<const volatile uint32_t *>(&partials[j]);
    uint32_t w[sizeof(Acc) / 4];
#pragma unroll
    for (int i = 0; i < (int)(sizeof(Acc) / 4); i++) w[i] = src[i];
    memcpy(&p, w, sizeof(Acc));
    r = Spec::combine(r, p);
  }
  r = warp_fold_ordered<Spec>(r, lane);
  __syncthreads();
  if (lane == 0) s_warp[warp] = r;
  __syncthreads();
  if (warp == 0) {
    Acc b = (lane < RM_WARPS) ? s_warp[lane] : Spec::neutral();
    b = warp_fold_ordered<Spec>(b, lane);
    if (lane == 0) {
      if (VEC)
        for (int64_t i = nvec << 2; i < n; i++) {
          if constexpr (NIN == 2) b = Spec::combine(b, Spec::map(in[i], in2[i]));
          else b = Spec::combine(b, Spec::map(in[i]));
        }
      *d_out = b;
      *ticket = 0u;
    }
  }
}

// `scratch`: a ticket word (zero before the first launch; every launch leaves it zero) and,
// 256 bytes further, room for RM_MAX_BLOCKS accumulators of 16 bytes.
template <class Spec>
cudaError_t launch_redomap(const void *in, const void *in2, int64_t n, void *d_out, void *scratch, int num_sms, cudaStream_t stream) {
  using Acc = typename Spec::Acc;
  constexpr int K = RedomapK<Spec>::K;
  uint32_t *ticket = reinterpret_cast<uint32_t *>(scratch);
  Acc *partials = reinterpret_cast<Acc *>(reinterpret_cast<char *>(scratch) + 256);
  const bool vec = ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(in2)) & 15) == 0;
  static int occ_v = 0, occ_s = 0;
  int &occ = vec ? occ_v : occ_s;
  if (occ == 0) {
    cudaError_t err = vec ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, redomap_kernel<Spec, true>, RM_THREADS, 0)
                          : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, redomap_kernel<Spec, false>, RM_THREADS, 0);
    if (err != cudaSuccess) return err;
    if (occ < 1) occ = 1;
  }
  const int64_t nvec = vec ? (n >> 2) : n;
  const int64_t steps = (nvec + 32 * K - 1) / (32 * K);
  int64_t want = (steps + RM_WARPS - 1) / RM_WARPS;
  int blocks = num_sms * occ;
  if (blocks > RM_MAX_BLOCKS) blocks = RM_MAX_BLOCKS;
  if (want < blocks) blocks = want < 1 ? 1 : (int)want;
  const uint32_t *p = reinterpret_cast<const uint32_t *>(in), *p2 = reinterpret_cast<const uint32_t *>(in2);
  Acc *out = reinterpret_cast<Acc *>(d_out);
  if (vec) redomap_kernel<Spec, true><<<blocks, RM_THREADS, 0, stream>>>(p, p2, n, out, ticket, partials);
  else redomap_kernel<Spec, false><<<blocks, RM_THREADS, 0, stream>>>(p, p2, n, out, ticket, partials);
  return cudaGetLastError();
}

}  // namespace fb
