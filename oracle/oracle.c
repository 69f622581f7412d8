/* CPU oracle for the SegOp hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is a plain-C restatement of the algorithms
 * that the reference's `futhark multicore` backend generates for the fixed entry
 * points of the library.  It is used by the parity tests, by the smoke check and as the timed CPU
 * baseline; the shipped library never links, loads or calls it.
 *
 * Parity status: pinned against the known-answer vectors that the reference's own
 * tests carry for these paths (tests/soacs/scan0.fut, reduce0.fut, filter1.fut,
 * partition1.fut, tests/hist/simple.fut, max.fut, large.fut,
 * tests/segredomap/segsum-comm.fut, tests/soacs/segreduce-iota.fut,
 * tests/reg-tiling/mmm.fut, tests/mss.fut, tests/soacs/exscan0.fut, exscan1.fut,
 * tests/modules/functor1.fut, tests/tokens.fut).  For the flagged f32 segmented
 * scan and the f16-input contraction the reference holds one known answer each on
 * exactly representable values (tests/tokens.fut: a flagged segmented scan of 0/1
 * values; tests/reg-tiling/mmm.fut: a product of small integers) and otherwise
 * "auto output" only, so for their rounding on general data this oracle is
 * "parity unpinned": it follows the reference's operator definitions but cannot
 * be checked against reference-produced values there.
 *
 * Scalar semantics follow rts/c/scalar.h: add32 is an unsigned add (:29), fmax32
 * is fmaxf (:932), f16 values are widened exactly to f32 before arithmetic
 * (rts/c/scalar_f16.h:402, rts/c/half.h:230).
 *
 * Build: gcc -O3 -std=c99 -ffp-contract=off -fopenmp -shared -fPIC
 * (-ffp-contract=off mirrors the reference's ISO-mode `cc -O3 -std=c99` build,
 * src/Futhark/Actions.hs:445, which forbids fusing a*b+c).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static int pick_threads(int requested) {
#ifdef _OPENMP
  int hw = omp_get_max_threads();
#else
  int hw = 1;
#endif
  if (requested <= 0) return hw;
  return requested;
}

int orc_max_threads(void) { return pick_threads(0); }

/* Contiguous chunk [lo,hi) of subtask t out of k over n iterations: the static
 * split the reference's scheduler hands to its workers (rts/c/scheduler.h:803-830:
 * iterations/nsubtasks each, the remainder spread one per leading subtask). */
static void chunk_of(int64_t n, int k, int t, int64_t *lo, int64_t *hi) {
  int64_t base = n / k, rem = n % k;
  *lo = t * base + (t < rem ? t : rem);
  *hi = *lo + base + (t < rem ? 1 : 0);
}

/* ---- reduce (+) 0 over i32 -------------------------------------------------
 * Multicore/SegRed.hs:95-125 picks the non-segmented path; stage one
 * (:297-320) folds each subtask's contiguous chunk from the neutral element,
 * stage two (:345-376) folds the per-subtask partials in subtask order. */
int32_t orc_reduce_i32(const int32_t *xs, int64_t n, int nthreads) {
  int k = pick_threads(nthreads);
  if (n < k) k = n > 0 ? (int)n : 1;
  uint32_t *part = (uint32_t *)calloc((size_t)k, sizeof(uint32_t));
#pragma omp parallel for num_threads(k) schedule(static, 1)
  for (int t = 0; t < k; t++) {
    int64_t lo, hi;
    chunk_of(n, k, t, &lo, &hi);
    uint32_t acc = 0;
    for (int64_t i = lo; i < hi; i++) acc += (uint32_t)xs[i];
    part[t] = acc;
  }
  uint32_t r = 0;
  for (int t = 0; t < k; t++) r += part[t];
  free(part);
  return (int32_t)r;
}

/* ---- inclusive scan (+) 0 over i32 ----------------------------------------
 * Multicore/SegScan.hs:407-566: the array is cut into blocks of
 * 64 KiB / sizeof(elem) elements (:24-25,424-427); each block is scanned
 * sequentially, block aggregates are combined by a look-back (:509-559).  For a
 * wrapping integer add every association gives the same bits, so the blocks are
 * processed here in two deterministic phases. */
#define ORC_SCAN_BLOCK_BYTES 65536

void orc_scan_i32(const int32_t *xs, int64_t n, int32_t *out, int nthreads) {
  if (n <= 0) return; /* SegScan.hs:76: nothing is emitted for an empty array */
  int k = pick_threads(nthreads);
  const int64_t blk = ORC_SCAN_BLOCK_BYTES / (int64_t)sizeof(int32_t);
  int64_t nb = (n + blk - 1) / blk;
  uint32_t *agg = (uint32_t *)malloc((size_t)nb * sizeof(uint32_t));
#pragma omp parallel for num_threads(k) schedule(static)
  for (int64_t b = 0; b < nb; b++) {
    int64_t lo = b * blk, hi = lo + blk < n ? lo + blk : n;
    uint32_t acc = 0;
    for (int64_t i = lo; i < hi; i++) acc += (uint32_t)xs[i];
    agg[b] = acc;
  }
  uint32_t run = 0;
  for (int64_t b = 0; b < nb; b++) { uint32_t a = agg[b]; agg[b] = run; run += a; }
#pragma omp parallel for num_threads(k) schedule(static)
  for (int64_t b = 0; b < nb; b++) {
    int64_t lo = b * blk, hi = lo + blk < n ? lo + blk : n;
    uint32_t acc = agg[b];
    for (int64_t i = lo; i < hi; i++) { acc += (uint32_t)xs[i]; out[i] = (int32_t)acc; }
  }
  free(agg);
}

/* ---- exclusive scan (+) 0 over i32 -----------------------------------------
 * prelude/soacs.fut:212-215: the inclusive scan scattered one place to the right
 * over an array of neutral elements; the last inclusive value falls off the end. */
void orc_exscan_i32(const int32_t *xs, int64_t n, int32_t *out, int nthreads) {
  if (n <= 0) return;
  int32_t *incl = (int32_t *)malloc((size_t)n * sizeof(int32_t));
  orc_scan_i32(xs, n, incl, nthreads);
  out[0] = 0;
  memcpy(out + 1, incl, (size_t)(n - 1) * sizeof(int32_t));
  free(incl);
}

/* ---- maximum segment sum: redomap with a non-commutative 4-tuple operator ------
 * The program of tests/mss.fut:6-20.  Multicore/SegRed.hs:297-320, 345-376: every
 * subtask folds its contiguous chunk left to right from the neutral element, the
 * per-subtask partials are folded in subtask order.  i32 additions wrap
 * (rts/c/scalar.h:29), max is the signed maximum (smax32, :262). */
typedef struct { int32_t mss, mis, mcs, ts; } orc_mss_t;
static int32_t wadd32(int32_t a, int32_t b) { return (int32_t)((uint32_t)a + (uint32_t)b); }
static int32_t smax32(int32_t a, int32_t b) { return a < b ? b : a; }
static orc_mss_t mss_op(orc_mss_t x, orc_mss_t y) {
  orc_mss_t r;
  r.mss = smax32(x.mss, smax32(y.mss, wadd32(x.mcs, y.mis)));
  r.mis = smax32(x.mis, wadd32(x.ts, y.mis));
  r.mcs = smax32(y.mcs, wadd32(x.mcs, y.ts));
  r.ts = wadd32(x.ts, y.ts);
  return r;
}
int32_t orc_mss_i32(const int32_t *xs, int64_t n, int nthreads) {
  int k = pick_threads(nthreads);
  if (n < k) k = n > 0 ? (int)n : 1;
  orc_mss_t *part = (orc_mss_t *)calloc((size_t)k, sizeof(orc_mss_t));
#pragma omp parallel for num_threads(k) schedule(static, 1)
  for (int t = 0; t < k; t++) {
    int64_t lo, hi;
    chunk_of(n, k, t, &lo, &hi);
    orc_mss_t acc = {0, 0, 0, 0};
    for (int64_t i = lo; i < hi; i++) {
      int32_t m = smax32(xs[i], 0);
      orc_mss_t e = {m, m, m, xs[i]};
      acc = mss_op(acc, e);
    }
    part[t] = acc;
  }
  orc_mss_t r = {0, 0, 0, 0};
  for (int t = 0; t < k; t++) r = mss_op(r, part[t]);
  free(part);
  return r.mss;
}

/* ---- two reductions fused over one input -------------------------------------
 * The program of tests/fusion/red-red-fusion.fut:5: (i32.sum xs, f32.sum (map f32.i32 xs)),
 * one SegRed with two operators; chunking as above.  f32.i32 is sitofp_i32_f32
 * (rts/c/scalar.h: a C cast). */
void orc_sum_i32_f32(const int32_t *xs, int64_t n, int32_t *out_i, float *out_f, int nthreads) {
  int k = pick_threads(nthreads);
  if (n < k) k = n > 0 ? (int)n : 1;
  uint32_t *pi = (uint32_t *)calloc((size_t)k, sizeof(uint32_t));
  float *pf = (float *)calloc((size_t)k, sizeof(float));
#pragma omp parallel for num_threads(k) schedule(static, 1)
  for (int t = 0; t < k; t++) {
    int64_t lo, hi;
    chunk_of(n, k, t, &lo, &hi);
    uint32_t ai = 0;
    float af = 0.0f;
    for (int64_t i = lo; i < hi; i++) { ai += (uint32_t)xs[i]; af += (float)xs[i]; }
    pi[t] = ai; pf[t] = af;
  }
  uint32_t ri = 0;
  float rf = 0.0f;
  for (int t = 0; t < k; t++) { ri += pi[t]; rf += pf[t]; }
  free(pi); free(pf);
  *out_i = (int32_t)ri;
  *out_f = rf;
}

/* ---- redomaps over two inputs ---------------------------------------------------
 * reduce (+) 0 (map2 (*) xs ys) over f32, and reduce (*) 1 (map2 (+) xs ys) over i32 (the
 * DotProd functor of tests/modules/functor1.fut:30-33); chunking as for the other
 * reductions (Multicore/SegRed.hs:297-320, 345-376).  The product and the sum are separate
 * roundings: the build forbids contraction into a fused multiply-add. */
float orc_dotprod_f32(const float *xs, const float *ys, int64_t n, int nthreads) {
  int k = pick_threads(nthreads);
  if (n < k) k = n > 0 ? (int)n : 1;
  float *part = (float *)calloc((size_t)k, sizeof(float));
#pragma omp parallel for num_threads(k) schedule(static, 1)
  for (int t = 0; t < k; t++) {
    int64_t lo, hi;
    chunk_of(n, k, t, &lo, &hi);
    float acc = 0.0f;
    for (int64_t i = lo; i < hi; i++) acc += xs[i] * ys[i];
    part[t] = acc;
  }
  float r = 0.0f;
  for (int t = 0; t < k; t++) r += part[t];
  free(part);
  return r;
}

int32_t orc_prod_of_sums_i32(const int32_t *xs, const int32_t *ys, int64_t n, int nthreads) {
  int k = pick_threads(nthreads);
  if (n < k) k = n > 0 ? (int)n : 1;
  uint32_t *part = (uint32_t *)calloc((size_t)k, sizeof(uint32_t));
#pragma omp parallel for num_threads(k) schedule(static, 1)
  for (int t = 0; t < k; t++) {
    int64_t lo, hi;
    chunk_of(n, k, t, &lo, &hi);
    uint32_t acc = 1;
    for (int64_t i = lo; i < hi; i++) acc *= (uint32_t)xs[i] + (uint32_t)ys[i];
    part[t] = acc;
  }
  uint32_t r = 1;
  for (int t = 0; t < k; t++) r *= part[t];
  free(part);
  return (int32_t)r;
}

/* ---- flagged segmented inclusive scan (+) over f32 --------------------------
 * The program scans (flag,value) pairs with the lifted operator of
 * tests/soacs/scan2.fut:7-17:  (f1,v1) (+) (f2,v2) = (f1||f2, f2 ? v2 : v1+v2),
 * neutral (false, 0).  Same block structure as orc_scan_i32; the float
 * association is: sequential inside a block, block aggregates folded in block
 * order.  (The reference's own association depends on thread timing.) */
void orc_segscan_f32(const uint8_t *flags, const float *xs, int64_t n, float *out, int nthreads) {
  if (n <= 0) return;
  int k = pick_threads(nthreads);
  const int64_t blk = ORC_SCAN_BLOCK_BYTES / (int64_t)(sizeof(float) + 1);
  int64_t nb = (n + blk - 1) / blk;
  float *aggv = (float *)malloc((size_t)nb * sizeof(float));
  uint8_t *aggf = (uint8_t *)malloc((size_t)nb);
#pragma omp parallel for num_threads(k) schedule(static)
  for (int64_t b = 0; b < nb; b++) {
    int64_t lo = b * blk, hi = lo + blk < n ? lo + blk : n;
    float acc = 0.0f; uint8_t f = 0;
    for (int64_t i = lo; i < hi; i++) {
      if (flags[i]) { acc = xs[i]; f = 1; } else acc = acc + xs[i];
    }
    aggv[b] = acc; aggf[b] = f;
  }
  float run = 0.0f;
  for (int64_t b = 0; b < nb; b++) {
    float a = aggv[b]; uint8_t f = aggf[b];
    aggv[b] = run;                     /* exclusive prefix of the block */
    run = f ? a : run + a;
  }
#pragma omp parallel for num_threads(k) schedule(static)
  for (int64_t b = 0; b < nb; b++) {
    int64_t lo = b * blk, hi = lo + blk < n ? lo + blk : n;
    float acc = aggv[b];
    for (int64_t i = lo; i < hi; i++) {
      if (flags[i]) acc = xs[i]; else acc = acc + xs[i];
      out[i] = acc;
    }
  }
  free(aggv); free(aggf);
}

/* Sequential f64-accumulated version of the same scan, for tolerance checks. */
void orc_segscan_f32_seq64(const uint8_t *flags, const float *xs, int64_t n, double *out) {
  double acc = 0.0;
  for (int64_t i = 0; i < n; i++) {
    if (flags[i]) acc = (double)xs[i]; else acc += (double)xs[i];
    out[i] = acc;
  }
}

/* ---- irregular segmented reduce (+) over f32, segments given by offsets -----
 * One sequential left fold per segment [off[s], off[s+1]), parallel over the
 * segments (Multicore/SegRed.hs:382-443); an empty segment yields the neutral
 * element, as the reference's flattened form does
 * (src/Futhark/Pass/Flatten/Builtins.hs:595-600). */
void orc_segreduce_f32(const int64_t *offsets, int64_t nseg, const float *xs, float *out, int nthreads) {
  int k = pick_threads(nthreads);
#pragma omp parallel for num_threads(k) schedule(static)
  for (int64_t s = 0; s < nseg; s++) {
    float acc = 0.0f;
    for (int64_t i = offsets[s]; i < offsets[s + 1]; i++) acc = acc + xs[i];
    out[s] = acc;
  }
}

/* ---- regular segmented reduce: map (reduce (+) 0) over rows -----------------
 * Multicore/SegRed.hs:382-443: parallel over rows, sequential fold per row. */
void orc_rowsum_f32(const float *xss, int64_t rows, int64_t cols, float *out, int nthreads) {
  int k = pick_threads(nthreads);
#pragma omp parallel for num_threads(k) schedule(static)
  for (int64_t r = 0; r < rows; r++) {
    float acc = 0.0f;
    const float *row = xss + r * cols;
    for (int64_t c = 0; c < cols; c++) acc = acc + row[c];
    out[r] = acc;
  }
}

/* ---- generalised histogram -------------------------------------------------
 * Multicore/SegHist.hs:50-77 chooses per-subtask private histograms when
 * num_threads * B <= n and atomic updates otherwise; :187-320 is the
 * private-histogram form (every copy starts at the neutral element, then a
 * segmented reduce over the copies); :263-265 is the bounds check: an index
 * outside [0,B) is skipped.  Both forms give the same bits for a wrapping i32
 * add and for f32 max, so the atomic form is restated as a sequential loop. */
void orc_hist_add_i32(int64_t B, const int32_t *is, const int32_t *ws, int64_t n, int32_t *out, int nthreads) {
  int k = pick_threads(nthreads);
  if (B <= 0) return;
  if ((int64_t)k * B <= n && k > 1) {
    uint32_t *priv = (uint32_t *)calloc((size_t)k * (size_t)B, sizeof(uint32_t));
#pragma omp parallel for num_threads(k) schedule(static, 1)
    for (int t = 0; t < k; t++) {
      int64_t lo, hi; chunk_of(n, k, t, &lo, &hi);
      uint32_t *h = priv + (size_t)t * (size_t)B;
      for (int64_t i = lo; i < hi; i++) {
        int64_t b = (int64_t)is[i];
        if (b >= 0 && b < B) h[b] += (uint32_t)ws[i];
      }
    }
#pragma omp parallel for num_threads(k) schedule(static)
    for (int64_t b = 0; b < B; b++) {
      uint32_t acc = 0;
      for (int t = 0; t < k; t++) acc += priv[(size_t)t * (size_t)B + (size_t)b];
      out[b] = (int32_t)acc;
    }
    free(priv);
  } else {
    uint32_t *o = (uint32_t *)out;
    for (int64_t b = 0; b < B; b++) o[b] = 0;
    for (int64_t i = 0; i < n; i++) {
      int64_t b = (int64_t)is[i];
      if (b >= 0 && b < B) o[b] += (uint32_t)ws[i];
    }
  }
}

/* hist f32.max f32.lowest: neutral is -inf (prelude/math.fut:1203), the
 * operator is fmaxf, which drops a NaN operand (rts/c/scalar.h:932). */
void orc_hist_max_f32(int64_t B, const int32_t *is, const float *ws, int64_t n, float *out, int nthreads) {
  int k = pick_threads(nthreads);
  if (B <= 0) return;
  if ((int64_t)k * B <= n && k > 1) {
    float *priv = (float *)malloc((size_t)k * (size_t)B * sizeof(float));
#pragma omp parallel for num_threads(k) schedule(static, 1)
    for (int t = 0; t < k; t++) {
      int64_t lo, hi; chunk_of(n, k, t, &lo, &hi);
      float *h = priv + (size_t)t * (size_t)B;
      for (int64_t b = 0; b < B; b++) h[b] = -INFINITY;
      for (int64_t i = lo; i < hi; i++) {
        int64_t b = (int64_t)is[i];
        if (b >= 0 && b < B) h[b] = fmaxf(h[b], ws[i]);
      }
    }
#pragma omp parallel for num_threads(k) schedule(static)
    for (int64_t b = 0; b < B; b++) {
      float acc = -INFINITY;
      for (int t = 0; t < k; t++) acc = fmaxf(acc, priv[(size_t)t * (size_t)B + (size_t)b]);
      out[b] = acc;
    }
    free(priv);
  } else {
    for (int64_t b = 0; b < B; b++) out[b] = -INFINITY;
    for (int64_t i = 0; i < n; i++) {
      int64_t b = (int64_t)is[i];
      if (b >= 0 && b < B) out[b] = fmaxf(out[b], ws[i]);
    }
  }
}

/* reduce_by_index dest (+) 0 is ws: starts from dest instead of the neutral
 * element (prelude/soacs.fut:145-146); used to replay tests/hist/simple.fut. */
void orc_reduce_by_index_add_i32(int32_t *dest, int64_t B, const int32_t *is, const int32_t *ws, int64_t n) {
  uint32_t *o = (uint32_t *)dest;
  for (int64_t i = 0; i < n; i++) {
    int64_t b = (int64_t)is[i];
    if (b >= 0 && b < B) o[b] += (uint32_t)ws[i];
  }
}

/* ---- filter / partition ----------------------------------------------------
 * prelude/soacs.fut:241-253: flags = map p; offsets = inclusive scan (+) of the
 * i64 flags; element i with p true goes to out[offsets[i]-1]; the count is the
 * last offset.  The predicate of the fixed program is (k & 7) < 3, unsigned. */
static inline int pred_u32(uint32_t k) { return (k & 7u) < 3u; }

int64_t orc_filter_u32(const uint32_t *ks, int64_t n, uint32_t *out, int nthreads) {
  if (n <= 0) return 0;
  int k = pick_threads(nthreads);
  if (n < k) k = 1;
  int64_t *cnt = (int64_t *)calloc((size_t)k + 1, sizeof(int64_t));
#pragma omp parallel for num_threads(k) schedule(static, 1)
  for (int t = 0; t < k; t++) {
    int64_t lo, hi; chunk_of(n, k, t, &lo, &hi);
    int64_t c = 0;
    for (int64_t i = lo; i < hi; i++) c += pred_u32(ks[i]);
    cnt[t + 1] = c;
  }
  for (int t = 0; t < k; t++) cnt[t + 1] += cnt[t];
#pragma omp parallel for num_threads(k) schedule(static, 1)
  for (int t = 0; t < k; t++) {
    int64_t lo, hi; chunk_of(n, k, t, &lo, &hi);
    int64_t off = cnt[t];                 /* = inclusive scan value before lo */
    for (int64_t i = lo; i < hi; i++)
      if (pred_u32(ks[i])) { off += 1; out[off - 1] = ks[i]; }
  }
  int64_t total = cnt[k];
  free(cnt);
  return total;
}

/* prelude/soacs.fut:261-286: partition p as = (selected, rejected), both in
 * original order; `out` receives the selected keys in [0,k) and the rejected
 * keys in [k,n); the split count k is returned. */
int64_t orc_partition_u32(const uint32_t *ks, int64_t n, uint32_t *out, int nthreads) {
  if (n <= 0) return 0;
  int k = pick_threads(nthreads);
  if (n < k) k = 1;
  int64_t *cnt = (int64_t *)calloc((size_t)k + 1, sizeof(int64_t));
#pragma omp parallel for num_threads(k) schedule(static, 1)
  for (int t = 0; t < k; t++) {
    int64_t lo, hi; chunk_of(n, k, t, &lo, &hi);
    int64_t c = 0;
    for (int64_t i = lo; i < hi; i++) c += pred_u32(ks[i]);
    cnt[t + 1] = c;
  }
  for (int t = 0; t < k; t++) cnt[t + 1] += cnt[t];
  int64_t total = cnt[k];
#pragma omp parallel for num_threads(k) schedule(static, 1)
  for (int t = 0; t < k; t++) {
    int64_t lo, hi; chunk_of(n, k, t, &lo, &hi);
    int64_t ot = cnt[t];
    int64_t of = total + (lo - cnt[t]);
    for (int64_t i = lo; i < hi; i++) {
      if (pred_u32(ks[i])) out[ot++] = ks[i]; else out[of++] = ks[i];
    }
  }
  free(cnt);
  return total;
}

/* ---- f16 -> f32 (binary16 bits to float), exact widening --------------------
 * Restates what rts/c/half.h:230 computes (its table-driven conversion is an
 * exact widening, so any exact widening gives the same bits). */
float orc_half_to_float(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1Fu;
  uint32_t man = h & 0x3FFu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) bits = sign;
    else {
      int e = -1;
      do { e++; man <<= 1; } while ((man & 0x400u) == 0);
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
    }
  } else if (exp == 31) bits = sign | 0x7F800000u | (man << 13);
  else bits = sign | ((exp + (127 - 15)) << 23) | (man << 13);
  float f; memcpy(&f, &bits, 4);
  return f;
}

/* ---- batched contraction ---------------------------------------------------
 * Nested maps around a sequential inner redomap
 * (src/Futhark/Pass/ExtractMulticore.hs:177-193): for every (b,i,j) a left fold
 * over k of f32(A[b,i,k]) * f32(B[b,k,j]) in f32, multiply and add rounded
 * separately (no FMA).  A: [nb][m][kk], B: [nb][kk][n], C: [nb][m][n], row-major. */
void orc_bmm_f16(const uint16_t *A, const uint16_t *Bm, int64_t nb, int64_t m, int64_t kk, int64_t n,
                 float *C, int nthreads) {
  int k = pick_threads(nthreads);
  if (nb * m * n <= 0) return;
  /* Widen once; B is transposed so the inner loop is unit-stride (no change in
   * the arithmetic or its order). */
  float *Bt = (float *)malloc((size_t)(kk > 0 ? kk : 1) * (size_t)n * sizeof(float));
  float *Af = (float *)malloc((size_t)(kk > 0 ? kk : 1) * (size_t)m * sizeof(float));
  for (int64_t b = 0; b < nb; b++) {
    const uint16_t *Ab = A + b * m * kk, *Bb = Bm + b * kk * n;
    float *Cb = C + b * m * n;
#pragma omp parallel for num_threads(k) schedule(static)
    for (int64_t j = 0; j < n; j++)
      for (int64_t q = 0; q < kk; q++) Bt[j * kk + q] = orc_half_to_float(Bb[q * n + j]);
#pragma omp parallel for num_threads(k) schedule(static)
    for (int64_t i = 0; i < m; i++)
      for (int64_t q = 0; q < kk; q++) Af[i * kk + q] = orc_half_to_float(Ab[i * kk + q]);
#pragma omp parallel for num_threads(k) schedule(static)
    for (int64_t i = 0; i < m; i++) {
      const float *ar = Af + i * kk;
      for (int64_t j = 0; j < n; j++) {
        const float *bc = Bt + j * kk;
        float acc = 0.0f;
        for (int64_t q = 0; q < kk; q++) { float p = ar[q] * bc[q]; acc = acc + p; }
        Cb[i * n + j] = acc;
      }
    }
  }
  free(Bt); free(Af);
}

/* Same contraction for f32 inputs; replays tests/reg-tiling/mmm.fut:6-12. */
void orc_mm_f32(const float *A, const float *Bm, int64_t m, int64_t kk, int64_t n, float *C) {
  for (int64_t i = 0; i < m; i++)
    for (int64_t j = 0; j < n; j++) {
      float acc = 0.0f;
      for (int64_t q = 0; q < kk; q++) { float p = A[i * kk + q] * Bm[q * n + j]; acc = acc + p; }
      C[i * n + j] = acc;
    }
}

/* Scalar shims so tests can compare against the reference's own headers. */
uint32_t orc_add32(uint32_t a, uint32_t b) { return a + b; }
float orc_fmax32(float a, float b) { return fmaxf(a, b); }
