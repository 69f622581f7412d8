/* CPU oracle, second part: the entry points that put the scan, compaction and histogram
 * kernels under other operators, predicates and index spaces.
 *
 * TEST INFRASTRUCTURE ONLY, like oracle.c: used by the parity tests, never by the shipped
 * library.  Every function restates the Futhark definition of its entry point literally
 * (sequential loops; these entry points are not part of the timed baseline).
 *
 * Parity status: pinned against the reference's own known-answer tests
 * tests/soacs/filter1.fut, filter3.fut, partition1.fut, scan4.fut,
 * tests/hist/and.fut, or.fut, xor.fut, min.fut, max.fut, f32.fut, segmented.fut, hist2d.fut.
 * tests/intrablock/segscan0.fut carries no values ("auto output"); the regular segmented scan
 * of i32 is fixed by its definition alone (integer arithmetic), as is scan i32.max.
 *
 * Scalar semantics follow rts/c/scalar.h: add32 / mul32 wrap (:29, :41), smin/smax/umin/umax
 * (:96-167), and/or/xor (:199-229), fadd32 (:865).  Futhark's x % m is the floored modulus
 * (smod32, scalar.h:352-361): it is 0 exactly when the C remainder is 0.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static int32_t wadd(int32_t a, int32_t b) { return (int32_t)((uint32_t)a + (uint32_t)b); }

/* scan i32.max i32.lowest xs (prelude/soacs.fut:176-178 with the operator of scalar.h:146) */
void orc_scan_max_i32(const int32_t *xs, int64_t n, int32_t *out) {
  int32_t acc = INT32_MIN;
  for (int64_t i = 0; i < n; i++) { acc = xs[i] > acc ? xs[i] : acc; out[i] = acc; }
}

/* map (scan (+) 0) xss (tests/intrablock/segscan0.fut:8-10) */
void orc_segscan_rows_i32(const int32_t *xss, int64_t rows, int64_t cols, int32_t *out) {
  for (int64_t r = 0; r < rows; r++) {
    int32_t acc = 0;
    for (int64_t c = 0; c < cols; c++) { acc = wadd(acc, xss[r * cols + c]); out[r * cols + c] = acc; }
  }
}

/* scan (map2 (+)) (replicate k 0) xss for xss: [m][k]i32 (tests/soacs/scan-with-map.fut:13-16 with a all
 * zeros, tests/soacs/scan5.fut:8): the accumulator is a whole row, rows are combined element by element */
void orc_scan_map2_add_i32(const int32_t *xss, int64_t m, int64_t k, int32_t *out) {
  for (int64_t i = 0; i < m; i++)
    for (int64_t j = 0; j < k; j++)
      out[i * k + j] = wadd(i > 0 ? out[(i - 1) * k + j] : 0, xss[i * k + j]);
}

/* reduce_by_index dest (+) 0f64 (map i64.i32 is) vs (tests/hist/f64.fut:40-41), in input order */
void orc_reduce_by_index_add_f64(double *dest, int64_t n, const int32_t *is, const double *vs, int64_t m) {
  for (int64_t i = 0; i < m; i++)
    if (is[i] >= 0 && (int64_t)is[i] < n) dest[is[i]] = dest[is[i]] + vs[i];
}

/* reduce (+) 0 (map2 (*) a b) (tests/soacs/reduce2.fut:11-12) and reduce (*) 1 a (tests/soacs/reduce1.fut:8):
 * mul32 and add32 wrap (rts/c/scalar.h:29-60) */
int32_t orc_dotprod_i32(const int32_t *xs, const int32_t *ys, int64_t n) {
  uint32_t acc = 0;
  for (int64_t i = 0; i < n; i++) acc += (uint32_t)xs[i] * (uint32_t)ys[i];
  return (int32_t)acc;
}
int32_t orc_product_i32(const int32_t *xs, int64_t n) {
  uint32_t acc = 1;
  for (int64_t i = 0; i < n; i++) acc *= (uint32_t)xs[i];
  return (int32_t)acc;
}

/* (reduce (\(a1,b1) (a2,b2) -> (a1*a2, b1*a2+b2)) (1,0) (zip as bs)).1, folded from the left */
float orc_linrec_last_f32(const float *as, const float *bs, int64_t n) {
  float a = 1.0f, b = 0.0f;
  for (int64_t i = 0; i < n; i++) { b = b * as[i] + bs[i]; a = a * as[i]; }
  return b;
}

/* reduce_by_index dest (+) 0 (map i64.iN is) vs over i8 and i16 (tests/hist/i8.fut:49-50, i16.fut): add8 / add16 wrap
 * (rts/c/scalar.h:21-27) */
void orc_reduce_by_index_add_i8(int8_t *dest, int64_t n, const int8_t *is, const int8_t *vs, int64_t m) {
  for (int64_t i = 0; i < m; i++)
    if (is[i] >= 0 && (int64_t)is[i] < n) dest[is[i]] = (int8_t)((uint8_t)dest[is[i]] + (uint8_t)vs[i]);
}
void orc_reduce_by_index_add_i16(int16_t *dest, int64_t n, const int16_t *is, const int16_t *vs, int64_t m) {
  for (int64_t i = 0; i < m; i++)
    if (is[i] >= 0 && (int64_t)is[i] < n) dest[is[i]] = (int16_t)((uint16_t)dest[is[i]] + (uint16_t)vs[i]);
}

/* reduce_by_index dest op ne (map i64.i32 is) vs over 1- and 2-byte integers (tests/hist/{min,max,and,or,xor}{8,16}.fut),
 * sequentially.  op: 0 smin, 1 smax, 2 umin, 3 umax (rts/c/scalar.h:486-505), 4 and, 5 or, 6 xor. */
#define ORC_RBI_NARROW(NAME, ST, UT)                                                                                      \
  void NAME(int op, ST *dest, int64_t n, const int32_t *is, const ST *vs, int64_t m) {                                    \
    for (int64_t i = 0; i < m; i++) {                                                                                     \
      if (is[i] < 0 || (int64_t)is[i] >= n) continue;                                                                     \
      const ST a = dest[is[i]], b = vs[i];                                                                                \
      ST r;                                                                                                               \
      switch (op) {                                                                                                       \
        case 0: r = a < b ? a : b; break;                                                                                 \
        case 1: r = a < b ? b : a; break;                                                                                 \
        case 2: r = (ST)((UT)a < (UT)b ? (UT)a : (UT)b); break;                                                           \
        case 3: r = (ST)((UT)a < (UT)b ? (UT)b : (UT)a); break;                                                           \
        case 4: r = (ST)(a & b); break;                                                                                   \
        case 5: r = (ST)(a | b); break;                                                                                   \
        default: r = (ST)(a ^ b); break;                                                                                  \
      }                                                                                                                   \
      dest[is[i]] = r;                                                                                                    \
    }                                                                                                                     \
  }
ORC_RBI_NARROW(orc_reduce_by_index_narrow8, int8_t, uint8_t)
ORC_RBI_NARROW(orc_reduce_by_index_narrow16, int16_t, uint16_t)

/* reduce_by_index xs (map2 (+)) (replicate m 0) is vss (tests/hist/array.fut:6-11): the bins are rows of m values */
void orc_reduce_by_index_vec_add_i32(int32_t *dest, int64_t n, int64_t m, const int64_t *is, const int32_t *vss, int64_t k) {
  for (int64_t i = 0; i < k; i++) {
    if (is[i] < 0 || is[i] >= n) continue;
    for (int64_t j = 0; j < m; j++) dest[is[i] * m + j] = (int32_t)((uint32_t)dest[is[i] * m + j] + (uint32_t)vss[i * m + j]);
  }
}

/* map2 (\is vss -> hist (map2 (+)) (replicate k 0) m (map i64.i32 is) vss) iss vsss (tests/hist/segmented_arr.fut:8-9);
 * out is [rows][m][k], zeroed here */
void orc_hist_rows_vec_add_i32(int32_t *out, int64_t rows, int64_t cols, int64_t m, int64_t k, const int32_t *iss, const int32_t *vsss) {
  for (int64_t t = 0; t < rows * m * k; t++) out[t] = 0;
  for (int64_t r = 0; r < rows; r++)
    for (int64_t i = 0; i < cols; i++) {
      const int64_t b = iss[r * cols + i];
      if (b < 0 || b >= m) continue;
      for (int64_t j = 0; j < k; j++)
        out[(r * m + b) * k + j] = (int32_t)((uint32_t)out[(r * m + b) * k + j] + (uint32_t)vsss[(r * cols + i) * k + j]);
    }
}

/* tests/hist/tuple_partial.fut:19-28: dest[b] = operator dest[b] (vs0[i], vs1[i]) in the order of the input, from
 * (-1, -1); operator (x0, y0) (x1, y1) = if x0 != -1 && (x1 == -1 || x0 < x1) then (x0, y0) else (x1, y1) */
void orc_reduce_by_index_minpair_i32(int32_t *out0, int32_t *out1, int64_t m, const int32_t *is, const int32_t *vs0, const int32_t *vs1,
                                     int64_t n) {
  for (int64_t b = 0; b < m; b++) { out0[b] = -1; out1[b] = -1; }
  for (int64_t i = 0; i < n; i++) {
    if (is[i] < 0 || (int64_t)is[i] >= m) continue;
    const int32_t x0 = out0[is[i]], x1 = vs0[i];
    if (!(x0 != -1 && (x1 == -1 || x0 < x1))) { out0[is[i]] = x1; out1[is[i]] = vs1[i]; }
  }
}

/* main of tests/segredomap/ex1-comm.fut:11-15: per row the sum of i64.f32 x (fptosi_f32_i64, rts/c/scalar.h:975-981: 0 for NaN
 * and infinities; wrapping addition) and the row of f64.f32 (-x) */
void orc_segredomap_sum_neg_f32(const float *xss, int64_t rows, int64_t cols, int64_t *sums, double *neg) {
  for (int64_t r = 0; r < rows; r++) {
    uint64_t acc = 0;
    for (int64_t i = 0; i < cols; i++) {
      const float x = xss[r * cols + i];
      if (!(x != x) && !(x == INFINITY || x == -INFINITY)) acc += (uint64_t)(int64_t)x;
      neg[r * cols + i] = (double)(-x);
    }
    sums[r] = (int64_t)acc;
  }
}

/* reduce_comm (map2 (+)) (replicate m 0) xss (tests/soacs/reduce4.fut:6-7): column sums, wrapping */
void orc_reduce_map2_add_i32(const int32_t *xss, int64_t rows, int64_t cols, int32_t *out) {
  for (int64_t c = 0; c < cols; c++) out[c] = 0;
  for (int64_t r = 0; r < rows; r++)
    for (int64_t c = 0; c < cols; c++) out[c] = (int32_t)((uint32_t)out[c] + (uint32_t)xss[r * cols + c]);
}

/* hist op ne n (map i64.i32 is) (map i64.i32 vs) over i64 (tests/hist/and64.fut, xor64.fut); op: 4 and, 5 or, 6 xor;
 * dest must hold the neutral element on entry */
void orc_hist_bitop_i64(int op, int64_t *dest, int64_t n, const int32_t *is, const int32_t *vs, int64_t m) {
  for (int64_t i = 0; i < m; i++) {
    if (is[i] < 0 || (int64_t)is[i] >= n) continue;
    const int64_t v = (int64_t)vs[i];
    if (op == 4) dest[is[i]] &= v;
    else if (op == 5) dest[is[i]] |= v;
    else dest[is[i]] ^= v;
  }
}

/* f32 -> binary16 bits the way the reference's C code narrows (rts/c/half.h:220-228: a table lookup whose
 * arithmetic this is): truncation, NaN payloads cut to their top ten bits */
uint16_t orc_float_to_half_trunc(float f) {
  union { float x; uint32_t y; } u;
  u.x = f;
  const uint32_t bits = u.y, sign = (bits >> 16) & 0x8000u, e = (bits >> 23) & 0xffu, m = bits & 0x7fffffu;
  if (e == 255u) return (uint16_t)(sign | 0x7c00u | (m >> 13));
  if (e > 142u) return (uint16_t)(sign | 0x7c00u);
  if (e >= 113u) return (uint16_t)(sign | ((e - 112u) << 10) | (m >> 13));
  if (e >= 103u) return (uint16_t)(sign | ((0x0400u >> (113u - e)) + (m >> (126u - e))));
  return (uint16_t)sign;
}
float orc_half_to_float(uint16_t h);     /* oracle.c */
/* tests/hist/f16.fut:40-41 under the C code's f16: values are widened to f32, added there and narrowed back
 * when they are stored (rts/c/scalar_f16.h:16-46) */
void orc_reduce_by_index_add_f16(uint16_t *dest, int64_t n, const int16_t *is, const uint16_t *vs, int64_t m) {
  for (int64_t i = 0; i < m; i++)
    if (is[i] >= 0 && (int64_t)is[i] < n)
      dest[is[i]] = orc_float_to_half_trunc(orc_half_to_float(dest[is[i]]) + orc_half_to_float(vs[i]));
}

/* reduce_by_index_3d dest (+) 0 (zip3 is js ks) vs (prelude/soacs.fut:153-154; tests/hist/hist3d.fut:8-9) */
void orc_reduce_by_index_3d_add_i32(int32_t *dest, int64_t K, int64_t M, int64_t L, const int64_t *is, const int64_t *js, const int64_t *ks,
                                    const int32_t *vs, int64_t n) {
  for (int64_t i = 0; i < n; i++)
    if (is[i] >= 0 && is[i] < K && js[i] >= 0 && js[i] < M && ks[i] >= 0 && ks[i] < L) {
      int32_t *d = &dest[(is[i] * M + js[i]) * L + ks[i]];
      *d = wadd(*d, vs[i]);
    }
}

/* tests/hist/segmented_2d.fut:18-24: per row, reduce_by_index_2d of ones over (x, y) pairs into [n][m] zeros */
void orc_hist_rows_2d_add_i32(int64_t N, int64_t M, const int32_t *xss, const int32_t *yss, int64_t rows, int64_t cols, int32_t *out) {
  for (int64_t i = 0; i < rows * N * M; i++) out[i] = 0;
  for (int64_t r = 0; r < rows; r++)
    for (int64_t c = 0; c < cols; c++) {
      const int64_t x = xss[r * cols + c], y = yss[r * cols + c];
      if (x >= 0 && x < N && y >= 0 && y < M) out[(r * N + x) * M + y] = wadd(out[(r * N + x) * M + y], 1);
    }
}

/* tests/soacs/scan4.fut:11-22, statement by statement */
static void scan4_step(const int32_t *xs, int64_t n, int32_t *out) {
  int32_t bits_sum = 0;
  for (int64_t i = 0; i < n; i++) bits_sum = wadd(bits_sum, wadd(xs[i], 1));   /* reduce (+) 0 (map (+1) xs) */
  int32_t ps = 0;
  for (int64_t i = 0; i < n; i++) {
    ps = wadd(ps, wadd(xs[i], 1));                    /* ps1 = scan (+) 0 bits */
    out[i] = wadd(wadd(ps, bits_sum), xs[i]);         /* map2 (+) (map (+ bits_sum) ps1) xs */
  }
}
void orc_scanomap_steps_i32(const int32_t *xs, int64_t n, int32_t *out) {
  int32_t *tmp = (int32_t *)malloc((size_t)(n > 0 ? n : 1) * sizeof(int32_t));
  scan4_step(xs, n, tmp);
  scan4_step(tmp, n, out);
  free(tmp);
}

/* filter (0 <) xs (tests/soacs/filter1.fut:14; prelude/soacs.fut:241-253) */
int64_t orc_filter_pos_i32(const int32_t *xs, int64_t n, int32_t *out) {
  int64_t k = 0;
  for (int64_t i = 0; i < n; i++) if (0 < xs[i]) out[k++] = xs[i];
  return k;
}

/* (unzip (filter (.1) (zip xs keep))).0 (tests/soacs/filter3.fut:11-19) */
int64_t orc_filter_by_flag_i32(const int32_t *xs, const uint8_t *keep, int64_t n, int32_t *out) {
  int64_t k = 0;
  for (int64_t i = 0; i < n; i++) if (keep[i]) out[k++] = xs[i];
  return k;
}

/* partition2 (x % 2 == 0) (x % 3 == 0) xs (tests/soacs/partition1.fut:13-18; prelude/soacs.fut:293-323):
 * out = group 0 ++ group 1 ++ group 2, each in original order; counts[0..2] their sizes. */
void orc_partition2_i32(const int32_t *xs, int64_t n, int32_t *out, int64_t *counts) {
  int64_t c[3] = {0, 0, 0};
  for (int64_t i = 0; i < n; i++) c[xs[i] % 2 == 0 ? 0 : (xs[i] % 3 == 0 ? 1 : 2)]++;
  int64_t o[3] = {0, c[0], c[0] + c[1]};
  for (int64_t i = 0; i < n; i++) out[o[xs[i] % 2 == 0 ? 0 : (xs[i] % 3 == 0 ? 1 : 2)]++] = xs[i];
  memcpy(counts, c, sizeof(c));
}

/* main of tests/soacs/partition2.fut:16-21: partition2 (x < y) (x == y) over zip xs ys, the three groups
 * unzipped (prelude/soacs.fut:293-323: a pair goes to the first group whose predicate holds, else to the
 * third; every group keeps the original order).  outx / outy = the first / second components of
 * group 0 ++ group 1 ++ group 2; counts[0..2] the group sizes. */
void orc_partition2_pairs_i32(const int32_t *xs, const int32_t *ys, int64_t n, int32_t *outx, int32_t *outy, int64_t *counts) {
  int64_t c[3] = {0, 0, 0};
  for (int64_t i = 0; i < n; i++) c[xs[i] < ys[i] ? 0 : (xs[i] == ys[i] ? 1 : 2)]++;
  int64_t o[3] = {0, c[0], c[0] + c[1]};
  for (int64_t i = 0; i < n; i++) {
    const int64_t at = o[xs[i] < ys[i] ? 0 : (xs[i] == ys[i] ? 1 : 2)]++;
    outx[at] = xs[i];
    outy[at] = ys[i];
  }
  memcpy(counts, c, sizeof(c));
}

/* reduce_by_index dest op ne is vs over 32-bit values (prelude/soacs.fut:117-130): dest is updated
 * in place; indices outside [0, B) are ignored.  op: 0 add i32, 2 min i32, 3 max i32, 4 min u32,
 * 5 max u32, 6 and, 7 or, 8 xor, 9 add f32 (sequential order), 10 mul i32 (numbering of the
 * library's operator list; 1, the f32 max, is orc_hist_max_f32 in oracle.c). */
void orc_reduce_by_index_32(int op, uint32_t *dest, int64_t B, const int32_t *is, const uint32_t *vs, int64_t n) {
  for (int64_t i = 0; i < n; i++) {
    const int64_t b = (int64_t)is[i];
    if (b < 0 || b >= B) continue;
    const uint32_t a = dest[b], v = vs[i];
    uint32_t r;
    switch (op) {
      case 0: r = a + v; break;
      case 2: r = (uint32_t)((int32_t)a < (int32_t)v ? (int32_t)a : (int32_t)v); break;
      case 3: r = (uint32_t)((int32_t)a > (int32_t)v ? (int32_t)a : (int32_t)v); break;
      case 4: r = a < v ? a : v; break;
      case 5: r = a > v ? a : v; break;
      case 6: r = a & v; break;
      case 7: r = a | v; break;
      case 8: r = a ^ v; break;
      case 9: { float fa, fv; memcpy(&fa, &a, 4); memcpy(&fv, &v, 4); fa = fa + fv; memcpy(&r, &fa, 4); break; }
      default: r = a * v; break;
    }
    dest[b] = r;
  }
}

/* map2 (\is vs -> hist (+) 0 m is vs) iss vss (tests/hist/segmented.fut:9-10) */
void orc_hist_rows_add_i32(int64_t m, const int32_t *iss, const int32_t *vss, int64_t rows, int64_t cols, int32_t *out) {
  memset(out, 0, (size_t)(rows * m) * sizeof(int32_t));
  for (int64_t r = 0; r < rows; r++)
    for (int64_t c = 0; c < cols; c++) {
      const int64_t b = (int64_t)iss[r * cols + c];
      if (b >= 0 && b < m) out[r * m + b] = wadd(out[r * m + b], vss[r * cols + c]);
    }
}

/* reduce_by_index_2d dest (+) 0 (zip is js) vs (prelude/soacs.fut:149-152): dest [N][M] updated in place */
void orc_reduce_by_index_2d_add_i32(int32_t *dest, int64_t N, int64_t M, const int64_t *is, const int64_t *js, const int32_t *vs, int64_t n) {
  for (int64_t i = 0; i < n; i++)
    if (is[i] >= 0 && is[i] < N && js[i] >= 0 && js[i] < M) dest[is[i] * M + js[i]] = wadd(dest[is[i] * M + js[i]], vs[i]);
}

/* scan (+) 0 over i64 (add64 wraps, scalar.h:33) */
void orc_scan_i64(const int64_t *xs, int64_t n, int64_t *out) {
  uint64_t acc = 0;
  for (int64_t i = 0; i < n; i++) { acc += (uint64_t)xs[i]; out[i] = (int64_t)acc; }
}

/* map (.1) (scan (\(a1,b1) (a2,b2) -> (a1*a2, b1*a2+b2)) (1,0) (zip as bs)), evaluated left to right in
 * f32 (products and sums rounded separately: no contraction), and in f64 for the tolerance check */
void orc_linrec_f32(const float *as, const float *bs, int64_t n, float *out) {
  float a = 1.0f, b = 0.0f;
  for (int64_t i = 0; i < n; i++) {
    const float na = a * as[i], t = b * as[i];
    b = t + bs[i];
    a = na;
    out[i] = b;
  }
}
void orc_linrec_f64(const float *as, const float *bs, int64_t n, double *out, double *cond) {
  double x = 0.0, c = 0.0;          /* c: the same recurrence on absolute values bounds the rounding error */
  for (int64_t i = 0; i < n; i++) {
    x = (double)as[i] * x + (double)bs[i];
    c = (as[i] < 0 ? -(double)as[i] : (double)as[i]) * c + (bs[i] < 0 ? -(double)bs[i] : (double)bs[i]);
    out[i] = x;
    cond[i] = c;
  }
}
