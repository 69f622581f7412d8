// Specifications for the fused-redomap kernel template (redomap.cuh) and their launchers.
//
//   mss_i32        maximum segment sum: a map body producing a 4-tuple and a NON-commutative
//                  operator on 4-tuples of i32 (the program of tests/mss.fut:6-20)
//   dotprod_f32    reduce (+) 0 (map2 (*) xs ys): a map body over two inputs
//   prod_of_sums_i32   reduce (*) 1 (map2 (+) xs ys) (tests/modules/functor1.fut:30-33)
//   dotprod_i32, product_i32   the programs of tests/soacs/reduce2.fut and reduce1.fut
//   affine_f32     composition of affine maps over (zip as bs): two inputs AND a non-commutative
//                  operator on pairs
//   sum_i32_f32    two reductions fused horizontally over one input, the second behind a map
//                  body: (i32.sum xs, f32.sum (map f32.i32 xs))
//                  (the program of tests/fusion/red-red-fusion.fut:5)
//
// Integer arithmetic wraps like the reference's (rts/c/scalar.h:29: add32 is an unsigned add).
#include "kernels.h"
#include "redomap.cuh"

namespace fb {

__device__ __forceinline__ int32_t wadd(int32_t a, int32_t b) { return (int32_t)((uint32_t)a + (uint32_t)b); }

struct SpecMss {
  // x = best segment sum, y = best prefix sum, z = best suffix sum, w = total
  using Acc = int4;
  static constexpr bool commutative = false;
  static constexpr int NIN = 1;
  __device__ __forceinline__ static Acc neutral() { return make_int4(0, 0, 0, 0); }
  __device__ __forceinline__ static Acc map(uint32_t bits) {
    const int32_t x = (int32_t)bits, m = max(x, 0);
    return make_int4(m, m, m, x);
  }
  __device__ __forceinline__ static Acc combine(const Acc &l, const Acc &r) {
    Acc o;
    o.x = max(l.x, max(r.x, wadd(l.z, r.y)));
    o.y = max(l.y, wadd(l.w, r.y));
    o.z = max(r.z, wadd(l.z, r.w));
    o.w = wadd(l.w, r.w);
    return o;
  }
};

struct SumI32F32 { uint32_t s; float f; };
struct SpecSumI32F32 {
  using Acc = SumI32F32;
  static constexpr bool commutative = true;
  static constexpr int NIN = 1;
  __device__ __forceinline__ static Acc neutral() { Acc a; a.s = 0u; a.f = 0.0f; return a; }
  __device__ __forceinline__ static Acc map(uint32_t bits) { Acc a; a.s = bits; a.f = (float)(int32_t)bits; return a; }
  __device__ __forceinline__ static Acc combine(const Acc &l, const Acc &r) { Acc a; a.s = l.s + r.s; a.f = l.f + r.f; return a; }
};

// reduce (+) 0 (map2 (*) xs ys) over f32: the dot product
struct AccF32 { float v; };
struct SpecDotF32 {
  using Acc = AccF32;
  static constexpr bool commutative = true;
  static constexpr int NIN = 2;
  __device__ __forceinline__ static Acc neutral() { Acc a; a.v = 0.0f; return a; }
  __device__ __forceinline__ static Acc map(uint32_t x, uint32_t y) { Acc a; a.v = __fmul_rn(__uint_as_float(x), __uint_as_float(y)); return a; }
  __device__ __forceinline__ static Acc combine(const Acc &l, const Acc &r) { Acc a; a.v = __fadd_rn(l.v, r.v); return a; }
};

// reduce (*) 1 (map2 (+) xs ys) over i32 (the DotProd functor of tests/modules/functor1.fut:30-33 at Int)
struct AccI32 { uint32_t v; };
struct SpecProdOfSumsI32 {
  using Acc = AccI32;
  static constexpr bool commutative = true;
  static constexpr int NIN = 2;
  __device__ __forceinline__ static Acc neutral() { Acc a; a.v = 1u; return a; }
  __device__ __forceinline__ static Acc map(uint32_t x, uint32_t y) { Acc a; a.v = x + y; return a; }
  __device__ __forceinline__ static Acc combine(const Acc &l, const Acc &r) { Acc a; a.v = l.v * r.v; return a; }
};

// reduce (+) 0 (map2 (*) xs ys) over i32 (tests/soacs/reduce2.fut:11-12)
struct SpecDotI32 {
  using Acc = AccI32;
  static constexpr bool commutative = true;
  static constexpr int NIN = 2;
  __device__ __forceinline__ static Acc neutral() { Acc a; a.v = 0u; return a; }
  __device__ __forceinline__ static Acc map(uint32_t x, uint32_t y) { Acc a; a.v = x * y; return a; }
  __device__ __forceinline__ static Acc combine(const Acc &l, const Acc &r) { Acc a; a.v = l.v + r.v; return a; }
};
// reduce (*) 1 xs over i32 (tests/soacs/reduce1.fut:8)
struct SpecProductI32 {
  using Acc = AccI32;
  static constexpr bool commutative = true;
  static constexpr int NIN = 1;
  __device__ __forceinline__ static Acc neutral() { Acc a; a.v = 1u; return a; }
  __device__ __forceinline__ static Acc map(uint32_t x) { Acc a; a.v = x; return a; }
  __device__ __forceinline__ static Acc combine(const Acc &l, const Acc &r) { Acc a; a.v = l.v * r.v; return a; }
};
// reduce (\(a1,b1) (a2,b2) -> (a1*a2, b1*a2+b2)) (1,0) (zip as bs): the composition of the affine maps
// x -> a*x + b, a NON-commutative operator on pairs over two inputs.  Its second component is the last
// value of the recurrence x_i = a_i * x_(i-1) + b_i from x = 0.  No fused multiply-add, as in the
// reference's C (compiled without contraction).
struct AccAffine { float a, b; };
struct SpecAffineF32 {
  using Acc = AccAffine;
  static constexpr bool commutative = false;
  static constexpr int NIN = 2;
  __device__ __forceinline__ static Acc neutral() { Acc r; r.a = 1.0f; r.b = 0.0f; return r; }
  __device__ __forceinline__ static Acc map(uint32_t a, uint32_t b) { Acc r; r.a = __uint_as_float(a); r.b = __uint_as_float(b); return r; }
  __device__ __forceinline__ static Acc combine(const Acc &l, const Acc &r) {
    Acc o; o.a = __fmul_rn(l.a, r.a); o.b = __fadd_rn(__fmul_rn(l.b, r.a), r.b); return o;
  }
};

static_assert(RM_MAX_BLOCKS == 4096, "reduce_scratch_bytes() holds 4096 partials of 16 bytes");

cudaError_t launch_mss_i32(const int32_t *in, int64_t n, int32_t *d_out4, void *scratch, int num_sms, cudaStream_t stream) {
  return launch_redomap<SpecMss>(in, nullptr, n, d_out4, scratch, num_sms, stream);
}
cudaError_t launch_sum_i32_f32(const int32_t *in, int64_t n, void *d_out2, void *scratch, int num_sms, cudaStream_t stream) {
  return launch_redomap<SpecSumI32F32>(in, nullptr, n, d_out2, scratch, num_sms, stream);
}
cudaError_t launch_dotprod_f32(const float *xs, const float *ys, int64_t n, float *d_out, void *scratch, int num_sms, cudaStream_t stream) {
  return launch_redomap<SpecDotF32>(xs, ys, n, d_out, scratch, num_sms, stream);
}
cudaError_t launch_prod_of_sums_i32(const int32_t *xs, const int32_t *ys, int64_t n, int32_t *d_out, void *scratch, int num_sms, cudaStream_t stream) {
  return launch_redomap<SpecProdOfSumsI32>(xs, ys, n, d_out, scratch, num_sms, stream);
}

cudaError_t launch_dotprod_i32(const int32_t *xs, const int32_t *ys, int64_t n, int32_t *d_out, void *scratch, int num_sms, cudaStream_t stream) {
  return launch_redomap<SpecDotI32>(xs, ys, n, d_out, scratch, num_sms, stream);
}
cudaError_t launch_product_i32(const int32_t *xs, int64_t n, int32_t *d_out, void *scratch, int num_sms, cudaStream_t stream) {
  return launch_redomap<SpecProductI32>(xs, nullptr, n, d_out, scratch, num_sms, stream);
}
cudaError_t launch_affine_f32(const float *as, const float *bs, int64_t n, float *d_out2, void *scratch, int num_sms, cudaStream_t stream) {
  return launch_redomap<SpecAffineF32>(as, bs, n, d_out2, scratch, num_sms, stream);
}

}  // namespace fb
