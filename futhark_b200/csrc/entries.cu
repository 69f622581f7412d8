// The entry points: argument checks, result allocation, kernel launches on the context's
// stream, packing of results into fresh array objects.  They stand where the reference's
// generated futhark_entry_* wrappers and futrts_entry_* host functions stand
// (src/Futhark/CodeGen/Backends/GenericC/EntryPoints.hs:133-223,
//  src/Futhark/CodeGen/ImpGen/GPU.hs:175-188).
#include <stdlib.h>

#include <string>

#include "common.cuh"
#include "kernels.h"
#include "runtime.h"

#define PROV(x) x

static std::string kv(const char *k, int64_t v) { return std::string("\"") + k + "\":" + std::to_string(v); }

static int bad_sizes(futhark_context *ctx) {
  // same text as EntryPoints.hs:171-174
  fb_set_error(ctx, "Error: entry point arguments have invalid sizes.\n");
  return 1;
}

template <typename ARR>
static ARR *make_1d(futhark_context *ctx, int64_t n, size_t elem, const char *desc, int *rc) {
  ARR *arr = (ARR *)malloc(sizeof(ARR));
  if (arr == nullptr) { *rc = 1; return nullptr; }
  arr->shape[0] = n;
  *rc = fb_alloc(ctx, (size_t)n * elem, desc, &arr->mem);
  if (*rc != FUTHARK_SUCCESS) { free(arr); return nullptr; }
  return arr;
}

template <typename T>
static inline T *dptr(const memblock_device &m) { return reinterpret_cast<T *>((uintptr_t)m.mem); }

static int not_ready(futhark_context *ctx) {
  fb_set_error(ctx, "The context failed to initialise; no entry point can run.");
  return 1;
}

// Launch a fused redomap whose result is `bytes` of scalars, read them back and wait
// (scalar results are synchronous: Backends/GPU.hs:269-281).
template <typename LAUNCH>
static int scalar_redomap(futhark_context *ctx, const char *name, const char *prov, int64_t n, size_t bytes, LAUNCH launch) {
  int rc;
  {
    LaunchScope ls(ctx, name, prov, "{" + kv("n", n) + "}");
    rc = fb_cuda_check(ctx, launch(), name);
  }
  if (rc) return rc;
  rc = fb_cuda_check(ctx, cudaMemcpyAsync(ctx->h_scalar, ctx->d_scalar, bytes, cudaMemcpyDeviceToHost, ctx->stream), "scalar read");
  if (rc) return rc;
  return fb_cuda_check(ctx, cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize");
}

extern "C" {

int futhark_entry_scan_i32(struct futhark_context *ctx, struct futhark_i32_1d **out0, const struct futhark_i32_1d *in0) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  const int64_t n = in0->shape[0];
  int rc;
  futhark_i32_1d *out = make_1d<futhark_i32_1d>(ctx, n, 4, "scan_i32.out", &rc);
  if (out == nullptr) return rc;
  if (n > 0) {
    rc = fb_ensure_lookback_scratch(ctx, fb::lookback_scratch_bytes(n));
    if (rc == 0) {
      LaunchScope ls(ctx, "scan_i32.segscan", PROV("scan (+) 0 xs"), "{" + kv("n", n) + "}");
      rc = fb_cuda_check(ctx, fb::launch_scan_i32(dptr<int32_t>(in0->mem), dptr<int32_t>(out->mem), n, 0, nullptr, 0, ctx->lookback_scratch,
                                                  fb_next_epoch(ctx), ctx->d_failure, ctx->stream,
                                                  (int)fb_tuning(ctx, "scan_i32.segscan_num_tblocks")), "scan_i32");
      ctx->failure_is_an_option = true;
    }
    if (rc != 0) { fb_unref(ctx, &out->mem); free(out); return rc; }
  }
  *out0 = out;
  return FUTHARK_SUCCESS;
}

int futhark_entry_reduce_i32(struct futhark_context *ctx, int32_t *out0, const struct futhark_i32_1d *in0) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  const int64_t n = in0->shape[0];
  int rc;
  {
    LaunchScope ls(ctx, "reduce_i32.segred_nonseg", PROV("reduce (+) 0 xs"), "{" + kv("n", n) + "}");
    rc = fb_cuda_check(ctx, fb::launch_reduce_i32(dptr<int32_t>(in0->mem), n, reinterpret_cast<int32_t *>(ctx->d_scalar),
                                                  ctx->reduce_scratch, ctx->num_sms, ctx->stream,
                                                  (int)fb_tuning(ctx, "reduce_i32.segred_num_tblocks")), "reduce_i32");
  }
  if (rc) return rc;
  // scalar result: read back and wait (Backends/GPU.hs:269-281)
  rc = fb_cuda_check(ctx, cudaMemcpyAsync(ctx->h_scalar, ctx->d_scalar, sizeof(int32_t), cudaMemcpyDeviceToHost, ctx->stream), "scalar read");
  if (rc) return rc;
  rc = fb_cuda_check(ctx, cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize");
  if (rc) return rc;
  *out0 = *reinterpret_cast<int32_t *>(ctx->h_scalar);
  return FUTHARK_SUCCESS;
}

// exscan (+) 0 xs: the same single-pass kernel as scan_i32 with the write-back shifted by one
// (the reference composes it from a scan and a scatter, prelude/soacs.fut:212-215).
int futhark_entry_exscan_i32(struct futhark_context *ctx, struct futhark_i32_1d **out0, const struct futhark_i32_1d *in0) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  const int64_t n = in0->shape[0];
  int rc;
  futhark_i32_1d *out = make_1d<futhark_i32_1d>(ctx, n, 4, "exscan_i32.out", &rc);
  if (out == nullptr) return rc;
  if (n > 0) {
    rc = fb_ensure_lookback_scratch(ctx, fb::lookback_scratch_bytes(n));
    if (rc == 0) {
      LaunchScope ls(ctx, "exscan_i32.segscan", PROV("exscan (+) 0 xs"), "{" + kv("n", n) + "}");
      rc = fb_cuda_check(ctx, fb::launch_exscan_i32(dptr<int32_t>(in0->mem), dptr<int32_t>(out->mem), n, ctx->lookback_scratch,
                                                    fb_next_epoch(ctx), ctx->d_failure, ctx->stream), "exscan_i32");
      ctx->failure_is_an_option = true;
    }
    if (rc != 0) { fb_unref(ctx, &out->mem); free(out); return rc; }
  }
  *out0 = out;
  return FUTHARK_SUCCESS;
}

// Maximum segment sum (tests/mss.fut): map body to 4-tuples, non-commutative tuple operator,
// first component of the result.
int futhark_entry_mss_i32(struct futhark_context *ctx, int32_t *out0, const struct futhark_i32_1d *in0) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  const int64_t n = in0->shape[0];
  int rc = scalar_redomap(ctx, "mss_i32.segred_nonseg", PROV("(reduce redOp (0,0,0,0) (map mapOp xs)).0"), n, 16, [&] {
    return fb::launch_mss_i32(dptr<int32_t>(in0->mem), n, reinterpret_cast<int32_t *>(ctx->d_scalar), ctx->reduce_scratch, ctx->num_sms, ctx->stream);
  });
  if (rc) return rc;
  *out0 = reinterpret_cast<int32_t *>(ctx->h_scalar)[0];
  return FUTHARK_SUCCESS;
}

// Two reductions fused over one input (tests/fusion/red-red-fusion.fut): (i32.sum xs, f32.sum (map f32.i32 xs)).
int futhark_entry_sum_i32_f32(struct futhark_context *ctx, struct futhark_opaque_tup2_i32_f32 **out0, const struct futhark_i32_1d *in0) {
  if (!ctx->ready) return not_ready(ctx);
  const int64_t n = in0->shape[0];
  int rc;
  int32_t s_i = 0;
  float s_f = 0.0f;
  {
    CtxGuard g(ctx);             // the staging words are read before the lock is given up
    rc = scalar_redomap(ctx, "sum_i32_f32.segred_nonseg", PROV("(i32.sum xs, f32.sum (map f32.i32 xs))"), n, 8, [&] {
      return fb::launch_sum_i32_f32(dptr<int32_t>(in0->mem), n, ctx->d_scalar, ctx->reduce_scratch, ctx->num_sms, ctx->stream);
    });
    s_i = reinterpret_cast<int32_t *>(ctx->h_scalar)[0];
    s_f = reinterpret_cast<float *>(ctx->h_scalar)[1];
  }
  if (rc) return rc;
  return futhark_new_opaque_tup2_i32_f32(ctx, out0, s_i, s_f);
}

// reduce (+) 0 (map2 (*) xs ys): a redomap whose map body takes two inputs.
int futhark_entry_dotprod_f32(struct futhark_context *ctx, float *out0, const struct futhark_f32_1d *in0, const struct futhark_f32_1d *in1) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  const int64_t n = in0->shape[0];
  if (in1->shape[0] != n) return bad_sizes(ctx);
  int rc = scalar_redomap(ctx, "dotprod_f32.segred_nonseg", PROV("reduce (+) 0 (map2 (*) xs ys)"), n, 4, [&] {
    return fb::launch_dotprod_f32(dptr<float>(in0->mem), dptr<float>(in1->mem), n, reinterpret_cast<float *>(ctx->d_scalar), ctx->reduce_scratch, ctx->num_sms, ctx->stream);
  });
  if (rc) return rc;
  *out0 = reinterpret_cast<float *>(ctx->h_scalar)[0];
  return FUTHARK_SUCCESS;
}

// reduce (*) 1 (map2 (+) xs ys) (tests/modules/functor1.fut:30-33 at i32).
int futhark_entry_prod_of_sums_i32(struct futhark_context *ctx, int32_t *out0, const struct futhark_i32_1d *in0, const struct futhark_i32_1d *in1) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  const int64_t n = in0->shape[0];
  if (in1->shape[0] != n) return bad_sizes(ctx);
  int rc = scalar_redomap(ctx, "prod_of_sums_i32.segred_nonseg", PROV("reduce (*) 1 (map2 (+) xs ys)"), n, 4, [&] {
    return fb::launch_prod_of_sums_i32(dptr<int32_t>(in0->mem), dptr<int32_t>(in1->mem), n, reinterpret_cast<int32_t *>(ctx->d_scalar), ctx->reduce_scratch, ctx->num_sms, ctx->stream);
  });
  if (rc) return rc;
  *out0 = reinterpret_cast<int32_t *>(ctx->h_scalar)[0];
  return FUTHARK_SUCCESS;
}

// reduce (+) 0 (map2 (*) xs ys) over i32 (tests/soacs/reduce2.fut) and reduce (*) 1 xs (tests/soacs/reduce1.fut)
int futhark_entry_dotprod_i32(struct futhark_context *ctx, int32_t *out0, const struct futhark_i32_1d *in0, const struct futhark_i32_1d *in1) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  const int64_t n = in0->shape[0];
  if (in1->shape[0] != n) return bad_sizes(ctx);
  int rc = scalar_redomap(ctx, "dotprod_i32.segred_nonseg", PROV("reduce (+) 0 (map2 (*) xs ys)"), n, 4, [&] {
    return fb::launch_dotprod_i32(dptr<int32_t>(in0->mem), dptr<int32_t>(in1->mem), n, reinterpret_cast<int32_t *>(ctx->d_scalar), ctx->reduce_scratch, ctx->num_sms, ctx->stream);
  });
  if (rc) return rc;
  *out0 = reinterpret_cast<int32_t *>(ctx->h_scalar)[0];
  return FUTHARK_SUCCESS;
}
int futhark_entry_product_i32(struct futhark_context *ctx, int32_t *out0, const struct futhark_i32_1d *in0) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  const int64_t n = in0->shape[0];
  int rc = scalar_redomap(ctx, "product_i32.segred_nonseg", PROV("reduce (*) 1 xs"), n, 4, [&] {
    return fb::launch_product_i32(dptr<int32_t>(in0->mem), n, reinterpret_cast<int32_t *>(ctx->d_scalar), ctx->reduce_scratch, ctx->num_sms, ctx->stream);
  });
  if (rc) return rc;
  *out0 = reinterpret_cast<int32_t *>(ctx->h_scalar)[0];
  return FUTHARK_SUCCESS;
}

// (reduce (\(a1,b1) (a2,b2) -> (a1*a2, b1*a2+b2)) (1,0) (zip as bs)).1: a non-commutative operator on pairs
// over two inputs; the last value of the recurrence that linrec_f32 scans.
int futhark_entry_linrec_last_f32(struct futhark_context *ctx, float *out0, const struct futhark_f32_1d *in0, const struct futhark_f32_1d *in1) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  const int64_t n = in0->shape[0];
  if (in1->shape[0] != n) return bad_sizes(ctx);
  int rc = scalar_redomap(ctx, "linrec_last_f32.segred_nonseg", PROV("(reduce compose (1,0) (zip as bs)).1"), n, 8, [&] {
    return fb::launch_affine_f32(dptr<float>(in0->mem), dptr<float>(in1->mem), n, reinterpret_cast<float *>(ctx->d_scalar), ctx->reduce_scratch, ctx->num_sms, ctx->stream);
  });
  if (rc) return rc;
  *out0 = reinterpret_cast<float *>(ctx->h_scalar)[1];
  return FUTHARK_SUCCESS;
}

// The caller holds the context's lock.  shard_out (device, 4 words, or NULL): see launch_segscan_f32.
int segscan_f32_locked(futhark_context *ctx, struct futhark_f32_1d **out0, const struct futhark_bool_1d *in0,
                       const struct futhark_f32_1d *in1, uint32_t *shard_out, const fb::PeerPush *peer) {
  const int64_t n = in1->shape[0];
  if (in0->shape[0] != n) return bad_sizes(ctx);
  int rc;
  futhark_f32_1d *out = make_1d<futhark_f32_1d>(ctx, n, 4, "segscan_f32.out", &rc);
  if (out == nullptr) return rc;
  rc = n > 0 ? fb_ensure_lookback_scratch(ctx, fb::lookback_scratch_bytes(n)) : 0;
  if (rc == 0 && (n > 0 || shard_out != nullptr)) {
    LaunchScope ls(ctx, "segscan_f32.segscan", PROV("scan lifted(+) (false,0) (zip flags xs)"), "{" + kv("n", n) + "}");
    rc = fb_cuda_check(ctx, fb::launch_segscan_f32(dptr<uint8_t>(in0->mem), dptr<float>(in1->mem), dptr<float>(out->mem), n, 0.0f, shard_out,
                                                   ctx->lookback_scratch, fb_next_epoch(ctx), ctx->d_failure, ctx->stream,
                                                   (int)fb_tuning(ctx, "segscan_f32.segscan_num_tblocks"), peer), "segscan_f32");
    ctx->failure_is_an_option = true;
  }
  if (rc != 0) { fb_unref(ctx, &out->mem); free(out); return rc; }
  *out0 = out;
  return FUTHARK_SUCCESS;
}

int futhark_entry_segscan_f32(struct futhark_context *ctx, struct futhark_f32_1d **out0, const struct futhark_bool_1d *in0,
                              const struct futhark_f32_1d *in1) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  return segscan_f32_locked(ctx, out0, in0, in1, nullptr, nullptr);
}

int futhark_entry_segreduce_f32(struct futhark_context *ctx, struct futhark_f32_1d **out0, const struct futhark_i64_1d *in0,
                                const struct futhark_bool_1d *in1, const struct futhark_f32_1d *in2) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  const int64_t n = in2->shape[0];
  if (in1->shape[0] != n) return bad_sizes(ctx);
  const int64_t nseg = in0->shape[0] > 0 ? in0->shape[0] - 1 : 0;
  int rc;
  futhark_f32_1d *out = make_1d<futhark_f32_1d>(ctx, nseg, 4, "segreduce_f32.out", &rc);
  if (out == nullptr) return rc;
  if (nseg > 0) {
    LaunchScope ls(ctx, "segreduce_f32.segred", PROV("map (reduce (+) 0) over offsets"), "{" + kv("n", n) + "," + kv("segments", nseg) + "}");
    rc = fb_cuda_check(ctx, fb::launch_segreduce_f32(dptr<int64_t>(in0->mem), nseg, dptr<float>(in2->mem), n, dptr<float>(out->mem),
                                                     ctx->reduce_scratch, ctx->d_failure, ctx->num_sms, ctx->stream), "segreduce_f32");
    ctx->failure_is_an_option = true;
    if (rc != 0) { fb_unref(ctx, &out->mem); free(out); return rc; }
  }
  *out0 = out;
  return FUTHARK_SUCCESS;
}

int futhark_entry_rowsum_f32(struct futhark_context *ctx, struct futhark_f32_1d **out0, const struct futhark_f32_2d *in0) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  const int64_t rows = in0->shape[0], cols = in0->shape[1];
  int rc;
  futhark_f32_1d *out = make_1d<futhark_f32_1d>(ctx, rows, 4, "rowsum_f32.out", &rc);
  if (out == nullptr) return rc;
  if (rows > 0) {
    LaunchScope ls(ctx, "rowsum_f32.segred", PROV("map (reduce (+) 0) xss"), "{" + kv("rows", rows) + "," + kv("cols", cols) + "}");
    rc = fb_cuda_check(ctx, fb::launch_rowsum_f32(dptr<float>(in0->mem), rows, cols, dptr<float>(out->mem), ctx->num_sms, ctx->stream,
                                                  fb_tuning(ctx, "rowsum_f32.suff_outer_par"), (int)fb_tuning(ctx, "rowsum_f32.segred_num_tblocks")), "rowsum_f32");
    if (rc != 0) { fb_unref(ctx, &out->mem); free(out); return rc; }
  }
  *out0 = out;
  return FUTHARK_SUCCESS;
}

// hist op ne B is ws (dest == NULL) or reduce_by_index dest op ne is ws: any operator of fb::HistOpKind
// over 32-bit values.  `is_raw` are the bin indices as i32 on the device.
static int hist_launch(futhark_context *ctx, int op, void **out_arr, int64_t B, const memblock_device *dest, const int32_t *is_raw,
                       int64_t n, const memblock_device &ws, int64_t ws_len, const char *name) {
  if (ws_len != n) return bad_sizes(ctx);
  if (B < 0) {
    // a negative size is a program error in the reference (array construction with a negative length)
    fb_set_error(ctx, "Error: negative histogram size %lld.\n", (long long)B);
    return FUTHARK_PROGRAM_ERROR;
  }
  int rc;
  futhark_i32_1d *out = make_1d<futhark_i32_1d>(ctx, B, 4, name, &rc);   // the same layout for every 4-byte element type
  if (out == nullptr) return rc;
  if (B > 0) {
    LaunchScope ls(ctx, name, PROV("hist op ne B (map i64.i32 is) ws"), "{" + kv("n", n) + "," + kv("bins", B) + "}");
    ctx->launch_count += (op == fb::HOP_MAX_F32 ? 2 : 1);   // the fill (and, for the f32 max, the key decode) besides the histogram kernel
    rc = fb_cuda_check(ctx, fb::launch_hist(op, B, is_raw, dptr<void>(ws), n, dptr<void>(out->mem), dest ? dptr<void>(*dest) : nullptr,
                                            ctx->num_sms, ctx->stream), name);
    if (rc != 0) { fb_unref(ctx, &out->mem); free(out); return rc; }
  }
  *out_arr = out;
  return FUTHARK_SUCCESS;
}

static int hist_common(futhark_context *ctx, int op, void **out_arr, int64_t B, const futhark_i32_1d *is, const memblock_device &ws,
                       int64_t ws_len, const char *name) {
  return hist_launch(ctx, op, out_arr, B, nullptr, dptr<int32_t>(is->mem), is->shape[0], ws, ws_len, name);
}

int futhark_entry_hist_add_i32(struct futhark_context *ctx, struct futhark_i32_1d **out0, const int64_t in0, const struct futhark_i32_1d *in1,
                               const struct futhark_i32_1d *in2) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  void *o = nullptr;
  int rc = hist_common(ctx, fb::HOP_ADD_I32, &o, in0, in1, in2->mem, in2->shape[0], "hist_add_i32.seghist");
  if (rc == 0) *out0 = (futhark_i32_1d *)o;
  return rc;
}

int futhark_entry_hist_max_f32(struct futhark_context *ctx, struct futhark_f32_1d **out0, const int64_t in0, const struct futhark_i32_1d *in1,
                               const struct futhark_f32_1d *in2) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  void *o = nullptr;
  int rc = hist_common(ctx, fb::HOP_MAX_F32, &o, in0, in1, in2->mem, in2->shape[0], "hist_max_f32.seghist");
  if (rc == 0) *out0 = (futhark_f32_1d *)o;   // futhark_i32_1d and futhark_f32_1d have the same layout
  return rc;
}

// ---- the histogram kernels under other operators (tests/hist/{and,or,xor,min,max,f32}.fut) --------
#define FB_HIST_ENTRY(NAME, OP, ARR)                                                                                          \
  int futhark_entry_hist_##NAME(struct futhark_context *ctx, struct futhark_##ARR **out0, const int64_t in0,                   \
                                const struct futhark_i32_1d *in1, const struct futhark_##ARR *in2) {                         \
    if (!ctx->ready) return not_ready(ctx);                                                                                   \
    CtxGuard g(ctx);                                                                                                          \
    void *o = nullptr;                                                                                                        \
    int rc = hist_common(ctx, OP, &o, in0, in1, in2->mem, in2->shape[0], "hist_" #NAME ".seghist");                           \
    if (rc == 0) *out0 = (futhark_##ARR *)o;                                                                                  \
    return rc;                                                                                                                \
  }
FB_HIST_ENTRY(and_i32, fb::HOP_AND_I32, i32_1d)
FB_HIST_ENTRY(or_i32, fb::HOP_OR_I32, i32_1d)
FB_HIST_ENTRY(xor_i32, fb::HOP_XOR_I32, i32_1d)
FB_HIST_ENTRY(mul_i32, fb::HOP_MUL_I32, i32_1d)

// reduce_by_index dest op ne (map i64.i32 is) vs: the result starts as a copy of dest
#define FB_RBI_ENTRY(NAME, OP, ARR)                                                                                           \
  int futhark_entry_reduce_by_index_##NAME(struct futhark_context *ctx, struct futhark_##ARR **out0,                          \
                                           const struct futhark_##ARR *in0, const struct futhark_i32_1d *in1,                 \
                                           const struct futhark_##ARR *in2) {                                                 \
    if (!ctx->ready) return not_ready(ctx);                                                                                   \
    CtxGuard g(ctx);                                                                                                          \
    void *o = nullptr;                                                                                                        \
    int rc = hist_launch(ctx, OP, &o, in0->shape[0], &in0->mem, dptr<int32_t>(in1->mem), in1->shape[0], in2->mem,              \
                         in2->shape[0], "reduce_by_index_" #NAME ".seghist");                                                 \
    if (rc == 0) *out0 = (futhark_##ARR *)o;                                                                                  \
    return rc;                                                                                                                \
  }
FB_RBI_ENTRY(min_i32, fb::HOP_MIN_I32, i32_1d)
FB_RBI_ENTRY(max_i32, fb::HOP_MAX_I32, i32_1d)
FB_RBI_ENTRY(min_u32, fb::HOP_MIN_U32, u32_1d)
FB_RBI_ENTRY(max_u32, fb::HOP_MAX_U32, u32_1d)
FB_RBI_ENTRY(add_f32, fb::HOP_ADD_F32, f32_1d)

// reduce_by_index dest (+) 0f64 (map i64.i32 is) vs (tests/hist/f64.fut): 8-byte values take the route of
// atomics on the result in global memory (SegHist.hs:377-560)
int futhark_entry_reduce_by_index_add_f64(struct futhark_context *ctx, struct futhark_f64_1d **out0, const struct futhark_f64_1d *in0,
                                          const struct futhark_i32_1d *in1, const struct futhark_f64_1d *in2) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  const int64_t B = in0->shape[0], n = in1->shape[0];
  if (in2->shape[0] != n) return bad_sizes(ctx);
  int rc;
  futhark_f64_1d *out = make_1d<futhark_f64_1d>(ctx, B, 8, "reduce_by_index_add_f64.out", &rc);
  if (out == nullptr) return rc;
  if (B > 0) {
    LaunchScope ls(ctx, "reduce_by_index_add_f64.seghist", PROV("reduce_by_index dest (+) 0f64 (map i64.i32 is) vs"), "{" + kv("n", n) + "," + kv("bins", B) + "}");
    rc = fb_cuda_check(ctx, fb::launch_hist_add_f64(B, dptr<int32_t>(in1->mem), dptr<double>(in2->mem), n, dptr<double>(out->mem), dptr<double>(in0->mem),
                                                    ctx->num_sms, ctx->stream), "reduce_by_index_add_f64");
    if (rc != 0) { fb_unref(ctx, &out->mem); free(out); return rc; }
  }
  *out0 = out;
  return FUTHARK_SUCCESS;
}

// reduce_by_index dest (+) 0 (map i64.iN is) vs over i8, i16 and f16 (tests/hist/i8.fut, i16.fut, f16.fut): element
// types without an atomic of their own take a compare-and-swap loop on the containing word (Base.hs:844-905)
#define FB_RBI_SUBWORD_ENTRY(NAME, KIND, ARR, IARR, ES)                                                                        \
  int futhark_entry_reduce_by_index_add_##NAME(struct futhark_context *ctx, struct futhark_##ARR **out0,                      \
                                               const struct futhark_##ARR *in0, const struct futhark_##IARR *in1,              \
                                               const struct futhark_##ARR *in2) {                                             \
    if (!ctx->ready) return not_ready(ctx);                                                                                   \
    CtxGuard g(ctx);                                                                                                          \
    const int64_t B = in0->shape[0], n = in1->shape[0];                                                                       \
    if (in2->shape[0] != n) return bad_sizes(ctx);                                                                            \
    int rc;                                                                                                                   \
    futhark_##ARR *out = make_1d<futhark_##ARR>(ctx, B, ES, "reduce_by_index_add_" #NAME ".out", &rc);                        \
    if (out == nullptr) return rc;                                                                                            \
    if (B > 0) {                                                                                                              \
      LaunchScope ls(ctx, "reduce_by_index_add_" #NAME ".seghist", PROV("reduce_by_index dest (+) 0 is vs"),                  \
                     "{" + kv("n", n) + "," + kv("bins", B) + "}");                                                           \
      rc = fb_cuda_check(ctx, fb::launch_hist_add_subword(KIND, B, dptr<void>(in1->mem), dptr<void>(in2->mem), n, dptr<void>(out->mem), \
                                                          dptr<void>(in0->mem), ctx->num_sms, ctx->stream),                   \
                         "reduce_by_index_add_" #NAME);                                                                       \
      if (rc != 0) { fb_unref(ctx, &out->mem); free(out); return rc; }                                                        \
    }                                                                                                                         \
    *out0 = out;                                                                                                              \
    return FUTHARK_SUCCESS;                                                                                                   \
  }
FB_RBI_SUBWORD_ENTRY(i8, 0, i8_1d, i8_1d, 1)
FB_RBI_SUBWORD_ENTRY(i16, 1, i16_1d, i16_1d, 2)
FB_RBI_SUBWORD_ENTRY(f16, 2, f16_1d, i16_1d, 2)

// ---- histograms over 1-, 2- and 8-byte integers with i32 indices ---------------------------------------
// tests/hist/{and,or,xor}{8,16}.fut, {min,max}{8,16}.fut: compare-and-swap on the containing word
// (Base.hs:844-905); tests/hist/{and,xor}64.fut: native 64-bit atomics, the i32 values widened in the kernel.
// dest == NULL: hist op ne B is vs; otherwise reduce_by_index dest op ne is vs.
static int hist_narrow(futhark_context *ctx, int op, int es, void **out_arr, int64_t B, const memblock_device *dest, const futhark_i32_1d *is,
                       const memblock_device &vs, int64_t vs_len, const char *name) {
  const int64_t n = is->shape[0];
  if (vs_len != n) return bad_sizes(ctx);
  if (B < 0) {
    fb_set_error(ctx, "Error: negative histogram size %lld.\n", (long long)B);
    return FUTHARK_PROGRAM_ERROR;
  }
  int rc;
  futhark_i8_1d *out = make_1d<futhark_i8_1d>(ctx, B, (size_t)es, name, &rc);     // the same layout for every one-dimensional array
  if (out == nullptr) return rc;
  if (B > 0) {
    LaunchScope ls(ctx, name, PROV("hist / reduce_by_index over sub-word integers"), "{" + kv("n", n) + "," + kv("bins", B) + "}");
    rc = fb_cuda_check(ctx, fb::launch_hist_narrow(op, es, B, dptr<int32_t>(is->mem), dptr<void>(vs), n, dptr<void>(out->mem),
                                                   dest ? dptr<void>(*dest) : nullptr, ctx->num_sms, ctx->stream), name);
    if (rc != 0) { fb_unref(ctx, &out->mem); free(out); return rc; }
  }
  *out_arr = out;
  return FUTHARK_SUCCESS;
}
#define FB_HIST_NARROW_ENTRY(NAME, OP, ARR, ES)                                                                               \
  int futhark_entry_hist_##NAME(struct futhark_context *ctx, struct futhark_##ARR **out0, const int64_t in0,                   \
                                const struct futhark_i32_1d *in1, const struct futhark_##ARR *in2) {                         \
    if (!ctx->ready) return not_ready(ctx);                                                                                   \
    CtxGuard g(ctx);                                                                                                          \
    void *o = nullptr;                                                                                                        \
    int rc = hist_narrow(ctx, OP, ES, &o, in0, nullptr, in1, in2->mem, in2->shape[0], "hist_" #NAME ".seghist");              \
    if (rc == 0) *out0 = (futhark_##ARR *)o;                                                                                  \
    return rc;                                                                                                                \
  }
FB_HIST_NARROW_ENTRY(and_i8, fb::NOP_AND, i8_1d, 1)
FB_HIST_NARROW_ENTRY(or_i8, fb::NOP_OR, i8_1d, 1)
FB_HIST_NARROW_ENTRY(xor_i8, fb::NOP_XOR, i8_1d, 1)
FB_HIST_NARROW_ENTRY(and_i16, fb::NOP_AND, i16_1d, 2)
FB_HIST_NARROW_ENTRY(or_i16, fb::NOP_OR, i16_1d, 2)
FB_HIST_NARROW_ENTRY(xor_i16, fb::NOP_XOR, i16_1d, 2)
FB_HIST_NARROW_ENTRY(or_bool, fb::NOP_OR, bool_1d, 1)      // hist (||) false (tests/hist/lor.fut): a bool is one byte holding 0 or 1
#define FB_RBI_NARROW_ENTRY(NAME, OP, ARR, ES)                                                                                \
  int futhark_entry_reduce_by_index_##NAME(struct futhark_context *ctx, struct futhark_##ARR **out0,                          \
                                           const struct futhark_##ARR *in0, const struct futhark_i32_1d *in1,                 \
                                           const struct futhark_##ARR *in2) {                                                 \
    if (!ctx->ready) return not_ready(ctx);                                                                                   \
    CtxGuard g(ctx);                                                                                                          \
    void *o = nullptr;                                                                                                        \
    int rc = hist_narrow(ctx, OP, ES, &o, in0->shape[0], &in0->mem, in1, in2->mem, in2->shape[0],                             \
                         "reduce_by_index_" #NAME ".seghist");                                                                \
    if (rc == 0) *out0 = (futhark_##ARR *)o;                                                                                  \
    return rc;                                                                                                                \
  }
FB_RBI_NARROW_ENTRY(min_i8, fb::NOP_MIN_S, i8_1d, 1)
FB_RBI_NARROW_ENTRY(max_i8, fb::NOP_MAX_S, i8_1d, 1)
FB_RBI_NARROW_ENTRY(min_u8, fb::NOP_MIN_U, u8_1d, 1)
FB_RBI_NARROW_ENTRY(max_u8, fb::NOP_MAX_U, u8_1d, 1)
FB_RBI_NARROW_ENTRY(min_i16, fb::NOP_MIN_S, i16_1d, 2)
FB_RBI_NARROW_ENTRY(max_i16, fb::NOP_MAX_S, i16_1d, 2)
FB_RBI_NARROW_ENTRY(min_u16, fb::NOP_MIN_U, u16_1d, 2)
FB_RBI_NARROW_ENTRY(max_u16, fb::NOP_MAX_U, u16_1d, 2)

#define FB_HIST_I64_ENTRY(NAME, OP)                                                                                           \
  int futhark_entry_hist_##NAME(struct futhark_context *ctx, struct futhark_i64_1d **out0, const int64_t in0,                  \
                                const struct futhark_i32_1d *in1, const struct futhark_i32_1d *in2) {                        \
    if (!ctx->ready) return not_ready(ctx);                                                                                   \
    CtxGuard g(ctx);                                                                                                          \
    const int64_t n = in1->shape[0];                                                                                          \
    if (in2->shape[0] != n) return bad_sizes(ctx);                                                                            \
    if (in0 < 0) { fb_set_error(ctx, "Error: negative histogram size %lld.\n", (long long)in0); return FUTHARK_PROGRAM_ERROR; } \
    int rc;                                                                                                                   \
    futhark_i64_1d *out = make_1d<futhark_i64_1d>(ctx, in0, 8, "hist_" #NAME ".out", &rc);                                    \
    if (out == nullptr) return rc;                                                                                            \
    if (in0 > 0) {                                                                                                            \
      LaunchScope ls(ctx, "hist_" #NAME ".seghist", PROV("hist op ne B (map i64.i32 is) (map i64.i32 vs)"),                   \
                     "{" + kv("n", n) + "," + kv("bins", (int64_t)in0) + "}");                                                \
      rc = fb_cuda_check(ctx, fb::launch_hist_bitop_i64(OP, in0, dptr<int32_t>(in1->mem), dptr<int32_t>(in2->mem), n,          \
                                                        dptr<int64_t>(out->mem), ctx->num_sms, ctx->stream), "hist_" #NAME);   \
      if (rc != 0) { fb_unref(ctx, &out->mem); free(out); return rc; }                                                        \
    }                                                                                                                         \
    *out0 = out;                                                                                                              \
    return FUTHARK_SUCCESS;                                                                                                   \
  }
FB_HIST_I64_ENTRY(and_i64, fb::NOP_AND)
FB_HIST_I64_ENTRY(or_i64, fb::NOP_OR)
FB_HIST_I64_ENTRY(xor_i64, fb::NOP_XOR)

// reduce_by_index xs (map2 (+)) (replicate m 0) is vss (tests/hist/array.fut, array_novec.fut): the bins are
// rows; one histogram over n * m bins behind a kernel that spreads every row index over its m elements
int futhark_entry_reduce_by_index_vec_add_i32(struct futhark_context *ctx, struct futhark_i32_2d **out0, const struct futhark_i32_2d *in0,
                                              const struct futhark_i64_1d *in1, const struct futhark_i32_2d *in2) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  const int64_t N = in0->shape[0], M = in0->shape[1], k = in1->shape[0];
  if (in2->shape[0] != k || in2->shape[1] != M) return bad_sizes(ctx);
  if (N * M >= (1ll << 31)) { fb_set_error(ctx, "reduce_by_index_vec_add_i32: %lld bins exceed 2^31-1.", (long long)(N * M)); return 1; }
  memblock_device flat;
  int rc = fb_alloc(ctx, (size_t)(k * M) * 4, "reduce_by_index_vec.flat_index", &flat);
  if (rc != 0) return rc;
  void *o = nullptr;
  ctx->launch_count++;
  rc = fb_cuda_check(ctx, fb::launch_flatten_vec_index(dptr<int64_t>(in1->mem), k, N, M, dptr<int32_t>(flat), ctx->num_sms, ctx->stream),
                     "flatten_vec_index");
  if (rc == 0) rc = hist_launch(ctx, fb::HOP_ADD_I32, &o, N * M, &in0->mem, dptr<int32_t>(flat), k * M, in2->mem, k * M, "reduce_by_index_vec_add_i32.seghist");
  fb_unref(ctx, &flat);
  if (rc != 0) return rc;
  futhark_i32_1d *h = (futhark_i32_1d *)o;
  futhark_i32_2d *out = (futhark_i32_2d *)malloc(sizeof(futhark_i32_2d));
  if (out == nullptr) { fb_unref(ctx, &h->mem); free(h); return 1; }
  out->mem = h->mem; out->shape[0] = N; out->shape[1] = M;
  free(h);
  *out0 = out;
  return FUTHARK_SUCCESS;
}

// map2 (\is vss -> hist (map2 (+)) (replicate k 0) m (map i64.i32 is) vss) iss vsss (tests/hist/segmented_arr.fut): a
// segment dimension over a histogram whose bins are k-vectors; one histogram over rows * m * k bins
int futhark_entry_hist_rows_vec_add_i32(struct futhark_context *ctx, struct futhark_i32_3d **out0, const int64_t in0, const struct futhark_i32_2d *in1,
                                        const struct futhark_i32_3d *in2) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  const int64_t m = in0, rows = in1->shape[0], cols = in1->shape[1], k = in2->shape[2];
  if (in2->shape[0] != rows || in2->shape[1] != cols) return bad_sizes(ctx);
  if (m < 0) { fb_set_error(ctx, "Error: negative histogram size %lld.\n", (long long)m); return FUTHARK_PROGRAM_ERROR; }
  if (rows * m * k >= (1ll << 31)) { fb_set_error(ctx, "hist_rows_vec_add_i32: %lld bins exceed 2^31-1.", (long long)(rows * m * k)); return 1; }
  const int64_t n = rows * cols * k;
  memblock_device flat;
  int rc = fb_alloc(ctx, (size_t)n * 4, "hist_rows_vec.flat_index", &flat);
  if (rc != 0) return rc;
  void *o = nullptr;
  ctx->launch_count++;
  rc = fb_cuda_check(ctx, fb::launch_flatten_rows_vec_index(dptr<int32_t>(in1->mem), rows, cols, m, k, dptr<int32_t>(flat), ctx->num_sms, ctx->stream),
                     "flatten_rows_vec_index");
  if (rc == 0) rc = hist_launch(ctx, fb::HOP_ADD_I32, &o, rows * m * k, nullptr, dptr<int32_t>(flat), n, in2->mem, n, "hist_rows_vec_add_i32.seghist");
  fb_unref(ctx, &flat);
  if (rc != 0) return rc;
  futhark_i32_1d *h = (futhark_i32_1d *)o;
  futhark_i32_3d *out = (futhark_i32_3d *)malloc(sizeof(futhark_i32_3d));
  if (out == nullptr) { fb_unref(ctx, &h->mem); free(h); return 1; }
  out->mem = h->mem; out->shape[0] = rows; out->shape[1] = m; out->shape[2] = k;
  free(h);
  *out0 = out;
  return FUTHARK_SUCCESS;
}

// main of tests/hist/tuple_partial.fut:24-28: reduce_by_index (replicate m (-1, -1)) operator (-1, -1) (map i64.i32 is)
// (zip vs0 vs1), unzipped; the operator keeps the pair with the smaller first component.  A pair is one 64-bit
// word updated by compare-and-swap (the reference takes a lock per bin for such an operator, Base.hs:769-842).
int futhark_entry_reduce_by_index_minpair_i32(struct futhark_context *ctx, struct futhark_opaque_tup2_arr1d_i32_arr1d_i32 **out0, const int64_t in0,
                                              const struct futhark_i32_1d *in1, const struct futhark_i32_1d *in2,
                                              const struct futhark_i32_1d *in3) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  const int64_t B = in0, n = in1->shape[0];
  if (in2->shape[0] != n || in3->shape[0] != n) return bad_sizes(ctx);
  if (B < 0) { fb_set_error(ctx, "Error: negative histogram size %lld.\n", (long long)B); return FUTHARK_PROGRAM_ERROR; }
  int rc;
  futhark_i32_1d *a = make_1d<futhark_i32_1d>(ctx, B, 4, "reduce_by_index_minpair_i32.out0", &rc);
  if (a == nullptr) return rc;
  futhark_i32_1d *b = make_1d<futhark_i32_1d>(ctx, B, 4, "reduce_by_index_minpair_i32.out1", &rc);
  if (b == nullptr) { fb_unref(ctx, &a->mem); free(a); return rc; }
  auto *p = (futhark_opaque_tup2_arr1d_i32_arr1d_i32 *)malloc(sizeof(futhark_opaque_tup2_arr1d_i32_arr1d_i32));
  memblock_device packed;
  rc = p == nullptr ? 1 : fb_alloc(ctx, (size_t)(B > 0 ? B : 1) * 8, "reduce_by_index_minpair_i32.packed", &packed);
  if (rc == 0) {
    if (B > 0) {
      LaunchScope ls(ctx, "reduce_by_index_minpair_i32.seghist", PROV("reduce_by_index dest op (-1, -1) is (zip vs0 vs1)"),
                     "{" + kv("n", n) + "," + kv("bins", B) + "}");
      ctx->launch_count += 1;
      rc = fb_cuda_check(ctx, fb::launch_hist_minpair_i32(B, dptr<int32_t>(in1->mem), dptr<int32_t>(in2->mem), dptr<int32_t>(in3->mem), n,
                                                          dptr<void>(packed), dptr<int32_t>(a->mem), dptr<int32_t>(b->mem), ctx->num_sms, ctx->stream),
                         "reduce_by_index_minpair_i32");
    }
    fb_unref(ctx, &packed);
  }
  if (rc != 0) {
    fb_unref(ctx, &a->mem); free(a);
    fb_unref(ctx, &b->mem); free(b);
    free(p);
    return rc;
  }
  p->v[0] = a; p->v[1] = b;
  *out0 = p;
  return FUTHARK_SUCCESS;
}

int futhark_free_opaque_tup2_arr1d_i32_arr1d_i32(struct futhark_context *ctx, struct futhark_opaque_tup2_arr1d_i32_arr1d_i32 *obj) {
  if (obj == nullptr) return 0;
  for (int i = 0; i < 2; i++) futhark_free_i32_1d(ctx, obj->v[i]);
  free(obj);
  return 0;
}
int futhark_new_opaque_tup2_arr1d_i32_arr1d_i32(struct futhark_context *ctx, struct futhark_opaque_tup2_arr1d_i32_arr1d_i32 **out,
                                                const struct futhark_i32_1d *v0, const struct futhark_i32_1d *v1) {
  CtxGuard g(ctx);
  auto *p = (futhark_opaque_tup2_arr1d_i32_arr1d_i32 *)malloc(sizeof(futhark_opaque_tup2_arr1d_i32_arr1d_i32));
  if (p == nullptr) return 1;
  const futhark_i32_1d *src[2] = {v0, v1};
  for (int i = 0; i < 2; i++) {
    p->v[i] = (futhark_i32_1d *)malloc(sizeof(futhark_i32_1d));
    if (p->v[i] == nullptr) return 1;
    *p->v[i] = *src[i];
    fb_ref(&p->v[i]->mem);         // the record shares the blocks of its fields (docs/c-api.rst:366-381)
  }
  *out = p;
  return 0;
}
static int project_tup2_i32(futhark_context *ctx, futhark_i32_1d **out, const futhark_opaque_tup2_arr1d_i32_arr1d_i32 *obj, int i) {
  CtxGuard g(ctx);
  futhark_i32_1d *a = (futhark_i32_1d *)malloc(sizeof(futhark_i32_1d));
  if (a == nullptr) return 1;
  *a = *obj->v[i];
  fb_ref(&a->mem);          // the projection shares the block (docs/c-api.rst:383-391)
  *out = a;
  return 0;
}
int futhark_project_opaque_tup2_arr1d_i32_arr1d_i32_0(struct futhark_context *ctx, struct futhark_i32_1d **out,
                                                      const struct futhark_opaque_tup2_arr1d_i32_arr1d_i32 *obj) { return project_tup2_i32(ctx, out, obj, 0); }
int futhark_project_opaque_tup2_arr1d_i32_arr1d_i32_1(struct futhark_context *ctx, struct futhark_i32_1d **out,
                                                      const struct futhark_opaque_tup2_arr1d_i32_arr1d_i32 *obj) { return project_tup2_i32(ctx, out, obj, 1); }

// main of tests/segredomap/ex1-comm.fut:11-15: unzip (map (\xs -> (reduce_comm (+) 0 (map i64.f32 xs), map (\x -> f64.f32 (-x)) xs)) xss):
// a segmented redomap whose body also returns a mapped array (a map-out result, SegRed.hs:138-143)
int futhark_entry_segredomap_sum_neg_f32(struct futhark_context *ctx, struct futhark_opaque_tup2_arr1d_i64_arr2d_f64 **out0,
                                         const struct futhark_f32_2d *in0) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  const int64_t rows = in0->shape[0], cols = in0->shape[1];
  int rc;
  futhark_i64_1d *sums = make_1d<futhark_i64_1d>(ctx, rows, 8, "segredomap_sum_neg_f32.sums", &rc);
  if (sums == nullptr) return rc;
  futhark_f64_2d *neg = (futhark_f64_2d *)malloc(sizeof(futhark_f64_2d));
  auto *p = (futhark_opaque_tup2_arr1d_i64_arr2d_f64 *)malloc(sizeof(futhark_opaque_tup2_arr1d_i64_arr2d_f64));
  rc = (neg == nullptr || p == nullptr) ? 1 : fb_alloc(ctx, (size_t)(rows * cols) * 8, "segredomap_sum_neg_f32.neg", &neg->mem);
  if (rc != 0) { fb_unref(ctx, &sums->mem); free(sums); free(neg); free(p); return rc; }
  neg->shape[0] = rows; neg->shape[1] = cols;
  {
    LaunchScope ls(ctx, "segredomap_sum_neg_f32.segred", PROV("map (\\xs -> (reduce (+) 0 (map i64.f32 xs), map (f64.f32 <-< f32.neg) xs)) xss"),
                   "{" + kv("rows", rows) + "," + kv("cols", cols) + "}");
    rc = fb_cuda_check(ctx, fb::launch_rowsum_mapout(dptr<float>(in0->mem), rows, cols, dptr<int64_t>(sums->mem), dptr<double>(neg->mem), ctx->num_sms,
                                                     ctx->stream), "segredomap_sum_neg_f32");
  }
  if (rc != 0) { fb_unref(ctx, &sums->mem); free(sums); fb_unref(ctx, &neg->mem); free(neg); free(p); return rc; }
  p->v0 = sums; p->v1 = neg;
  *out0 = p;
  return FUTHARK_SUCCESS;
}
int futhark_free_opaque_tup2_arr1d_i64_arr2d_f64(struct futhark_context *ctx, struct futhark_opaque_tup2_arr1d_i64_arr2d_f64 *obj) {
  if (obj == nullptr) return 0;
  futhark_free_i64_1d(ctx, obj->v0);
  futhark_free_f64_2d(ctx, obj->v1);
  free(obj);
  return 0;
}
int futhark_new_opaque_tup2_arr1d_i64_arr2d_f64(struct futhark_context *ctx, struct futhark_opaque_tup2_arr1d_i64_arr2d_f64 **out,
                                                const struct futhark_i64_1d *v0, const struct futhark_f64_2d *v1) {
  CtxGuard g(ctx);
  auto *p = (futhark_opaque_tup2_arr1d_i64_arr2d_f64 *)malloc(sizeof(futhark_opaque_tup2_arr1d_i64_arr2d_f64));
  if (p == nullptr) return 1;
  p->v0 = (futhark_i64_1d *)malloc(sizeof(futhark_i64_1d));
  p->v1 = (futhark_f64_2d *)malloc(sizeof(futhark_f64_2d));
  if (p->v0 == nullptr || p->v1 == nullptr) return 1;
  *p->v0 = *v0; fb_ref(&p->v0->mem);           // the record shares the blocks of its fields (docs/c-api.rst:366-381)
  *p->v1 = *v1; fb_ref(&p->v1->mem);
  *out = p;
  return 0;
}
int futhark_project_opaque_tup2_arr1d_i64_arr2d_f64_0(struct futhark_context *ctx, struct futhark_i64_1d **out,
                                                      const struct futhark_opaque_tup2_arr1d_i64_arr2d_f64 *obj) {
  CtxGuard g(ctx);
  futhark_i64_1d *a = (futhark_i64_1d *)malloc(sizeof(futhark_i64_1d));
  if (a == nullptr) return 1;
  *a = *obj->v0; fb_ref(&a->mem);              // the projection shares the block (docs/c-api.rst:383-391)
  *out = a;
  return 0;
}
int futhark_project_opaque_tup2_arr1d_i64_arr2d_f64_1(struct futhark_context *ctx, struct futhark_f64_2d **out,
                                                      const struct futhark_opaque_tup2_arr1d_i64_arr2d_f64 *obj) {
  CtxGuard g(ctx);
  futhark_f64_2d *a = (futhark_f64_2d *)malloc(sizeof(futhark_f64_2d));
  if (a == nullptr) return 1;
  *a = *obj->v1; fb_ref(&a->mem);
  *out = a;
  return 0;
}

// reduce (map2 (+)) (replicate m 0) xss (tests/soacs/reduce4.fut, reduce5.fut): an operator on whole rows; the
// reduction is interchanged with the inner map (src/Futhark/Transform/ISRWIM.hs) and every column reduced
int futhark_entry_reduce_map2_add_i32(struct futhark_context *ctx, struct futhark_i32_1d **out0, const struct futhark_i32_2d *in0) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  const int64_t rows = in0->shape[0], cols = in0->shape[1];
  int rc;
  futhark_i32_1d *out = make_1d<futhark_i32_1d>(ctx, cols, 4, "reduce_map2_add_i32.out", &rc);
  if (out == nullptr) return rc;
  if (cols > 0) {
    LaunchScope ls(ctx, "reduce_map2_add_i32.segred", PROV("reduce (map2 (+)) (replicate m 0) xss"), "{" + kv("rows", rows) + "," + kv("cols", cols) + "}");
    rc = fb_cuda_check(ctx, fb::launch_colsum_i32(dptr<int32_t>(in0->mem), rows, cols, dptr<int32_t>(out->mem), ctx->num_sms, ctx->stream),
                       "reduce_map2_add_i32");
    if (rc != 0) { fb_unref(ctx, &out->mem); free(out); return rc; }
  }
  *out0 = out;
  return FUTHARK_SUCCESS;
}

// map2 (\is vs -> hist (+) 0 m (map i64.i32 is) vs) iss vss (tests/hist/segmented.fut: a SegHist with a
// segment dimension, SegHist.hs:97-148): one histogram over rows * m bins whose index carries the row.
int futhark_entry_hist_rows_add_i32(struct futhark_context *ctx, struct futhark_i32_2d **out0, const int64_t in0,
                                    const struct futhark_i32_2d *in1, const struct futhark_i32_2d *in2) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  const int64_t rows = in1->shape[0], cols = in1->shape[1], m = in0;
  if (in2->shape[0] != rows || in2->shape[1] != cols) return bad_sizes(ctx);
  if (m < 0) { fb_set_error(ctx, "Error: negative histogram size %lld.\n", (long long)m); return FUTHARK_PROGRAM_ERROR; }
  if (rows * m >= (1ll << 31)) { fb_set_error(ctx, "hist_rows_add_i32: %lld bins in all exceed 2^31-1.", (long long)(rows * m)); return 1; }
  memblock_device flat;
  int rc = fb_alloc(ctx, (size_t)(rows * cols) * 4, "hist_rows.flat_index", &flat);
  if (rc != 0) return rc;
  void *o = nullptr;
  ctx->launch_count++;
  rc = fb_cuda_check(ctx, fb::launch_flatten_rows_index(dptr<int32_t>(in1->mem), rows * cols, cols, m, dptr<int32_t>(flat), ctx->num_sms, ctx->stream),
                     "flatten_rows_index");
  if (rc == 0) rc = hist_launch(ctx, fb::HOP_ADD_I32, &o, rows * m, nullptr, dptr<int32_t>(flat), rows * cols, in2->mem, rows * cols,
                                "hist_rows_add_i32.seghist");
  fb_unref(ctx, &flat);
  if (rc != 0) return rc;
  futhark_i32_1d *h = (futhark_i32_1d *)o;
  futhark_i32_2d *out = (futhark_i32_2d *)malloc(sizeof(futhark_i32_2d));
  if (out == nullptr) { fb_unref(ctx, &h->mem); free(h); return 1; }
  out->mem = h->mem; out->shape[0] = rows; out->shape[1] = m;
  free(h);
  *out0 = out;
  return FUTHARK_SUCCESS;
}

// reduce_by_index_2d dest (+) 0 (zip is js) vs (prelude/soacs.fut:149-152; tests/hist/hist2d.fut).
int futhark_entry_reduce_by_index_2d_add_i32(struct futhark_context *ctx, struct futhark_i32_2d **out0, const struct futhark_i32_2d *in0,
                                             const struct futhark_i64_1d *in1, const struct futhark_i64_1d *in2,
                                             const struct futhark_i32_1d *in3) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  const int64_t N = in0->shape[0], M = in0->shape[1], n = in1->shape[0];
  if (in2->shape[0] != n || in3->shape[0] != n) return bad_sizes(ctx);
  if (N * M >= (1ll << 31)) { fb_set_error(ctx, "reduce_by_index_2d_add_i32: %lld bins exceed 2^31-1.", (long long)(N * M)); return 1; }
  memblock_device flat;
  int rc = fb_alloc(ctx, (size_t)n * 4, "reduce_by_index_2d.flat_index", &flat);
  if (rc != 0) return rc;
  void *o = nullptr;
  ctx->launch_count++;
  rc = fb_cuda_check(ctx, fb::launch_flatten_2d_index(dptr<int64_t>(in1->mem), dptr<int64_t>(in2->mem), n, N, M, dptr<int32_t>(flat), ctx->num_sms,
                                                      ctx->stream), "flatten_2d_index");
  if (rc == 0) rc = hist_launch(ctx, fb::HOP_ADD_I32, &o, N * M, &in0->mem, dptr<int32_t>(flat), n, in3->mem, n, "reduce_by_index_2d_add_i32.seghist");
  fb_unref(ctx, &flat);
  if (rc != 0) return rc;
  futhark_i32_1d *h = (futhark_i32_1d *)o;
  futhark_i32_2d *out = (futhark_i32_2d *)malloc(sizeof(futhark_i32_2d));
  if (out == nullptr) { fb_unref(ctx, &h->mem); free(h); return 1; }
  out->mem = h->mem; out->shape[0] = N; out->shape[1] = M;
  free(h);
  *out0 = out;
  return FUTHARK_SUCCESS;
}

// reduce_by_index_3d dest (+) 0 (zip3 is js ks) vs (prelude/soacs.fut:153-154, tests/hist/hist3d.fut): one histogram
// over k * m * l bins behind a kernel that flattens the index triples
int futhark_entry_reduce_by_index_3d_add_i32(struct futhark_context *ctx, struct futhark_i32_3d **out0, const struct futhark_i32_3d *in0,
                                             const struct futhark_i64_1d *in1, const struct futhark_i64_1d *in2,
                                             const struct futhark_i64_1d *in3, const struct futhark_i32_1d *in4) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  const int64_t K = in0->shape[0], M = in0->shape[1], L = in0->shape[2], n = in1->shape[0];
  if (in2->shape[0] != n || in3->shape[0] != n || in4->shape[0] != n) return bad_sizes(ctx);
  if (K * M * L >= (1ll << 31)) { fb_set_error(ctx, "reduce_by_index_3d_add_i32: %lld bins exceed 2^31-1.", (long long)(K * M * L)); return 1; }
  memblock_device flat;
  int rc = fb_alloc(ctx, (size_t)n * 4, "reduce_by_index_3d.flat_index", &flat);
  if (rc != 0) return rc;
  void *o = nullptr;
  ctx->launch_count++;
  rc = fb_cuda_check(ctx, fb::launch_flatten_3d_index(dptr<int64_t>(in1->mem), dptr<int64_t>(in2->mem), dptr<int64_t>(in3->mem), n, K, M, L,
                                                      dptr<int32_t>(flat), ctx->num_sms, ctx->stream), "flatten_3d_index");
  if (rc == 0) rc = hist_launch(ctx, fb::HOP_ADD_I32, &o, K * M * L, &in0->mem, dptr<int32_t>(flat), n, in4->mem, n, "reduce_by_index_3d_add_i32.seghist");
  fb_unref(ctx, &flat);
  if (rc != 0) return rc;
  futhark_i32_1d *h = (futhark_i32_1d *)o;
  futhark_i32_3d *out = (futhark_i32_3d *)malloc(sizeof(futhark_i32_3d));
  if (out == nullptr) { fb_unref(ctx, &h->mem); free(h); return 1; }
  out->mem = h->mem; out->shape[0] = K; out->shape[1] = M; out->shape[2] = L;
  free(h);
  *out0 = out;
  return FUTHARK_SUCCESS;
}

// tests/hist/segmented_2d.fut: a 2-D histogram of ones per row of index pairs (a segment dimension over
// reduce_by_index_2d, SegHist.hs:97-148): one histogram over rows * n * m bins
int futhark_entry_hist_rows_2d_add_i32(struct futhark_context *ctx, struct futhark_i32_3d **out0, const int64_t in0, const int64_t in1,
                                       const struct futhark_i32_2d *in2, const struct futhark_i32_2d *in3) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  const int64_t N = in0, M = in1, rows = in2->shape[0], cols = in2->shape[1], n = rows * cols;
  if (in3->shape[0] != rows || in3->shape[1] != cols) return bad_sizes(ctx);
  if (N < 0 || M < 0) { fb_set_error(ctx, "Error: negative histogram size %lld x %lld.\n", (long long)N, (long long)M); return FUTHARK_PROGRAM_ERROR; }
  if (rows * N * M >= (1ll << 31)) { fb_set_error(ctx, "hist_rows_2d_add_i32: %lld bins in all exceed 2^31-1.", (long long)(rows * N * M)); return 1; }
  memblock_device flat, ones;
  int rc = fb_alloc(ctx, (size_t)n * 4, "hist_rows_2d.flat_index", &flat);
  if (rc != 0) return rc;
  rc = fb_alloc(ctx, (size_t)n * 4, "hist_rows_2d.ones", &ones);
  if (rc != 0) { fb_unref(ctx, &flat); return rc; }
  void *o = nullptr;
  ctx->launch_count += 2;
  rc = fb_cuda_check(ctx, fb::launch_replicate(4, dptr<void>(ones), n, 1ull, ctx->num_sms, ctx->stream), "replicate");
  if (rc == 0)
    rc = fb_cuda_check(ctx, fb::launch_flatten_rows_2d_index(dptr<int32_t>(in2->mem), dptr<int32_t>(in3->mem), n, cols, N, M, dptr<int32_t>(flat),
                                                             ctx->num_sms, ctx->stream), "flatten_rows_2d_index");
  if (rc == 0) rc = hist_launch(ctx, fb::HOP_ADD_I32, &o, rows * N * M, nullptr, dptr<int32_t>(flat), n, ones, n, "hist_rows_2d_add_i32.seghist");
  fb_unref(ctx, &flat);
  fb_unref(ctx, &ones);
  if (rc != 0) return rc;
  futhark_i32_1d *h = (futhark_i32_1d *)o;
  futhark_i32_3d *out = (futhark_i32_3d *)malloc(sizeof(futhark_i32_3d));
  if (out == nullptr) { fb_unref(ctx, &h->mem); free(h); return 1; }
  out->mem = h->mem; out->shape[0] = rows; out->shape[1] = N; out->shape[2] = M;
  free(h);
  *out0 = out;
  return FUTHARK_SUCCESS;
}

// ---- compaction entry points -----------------------------------------------------------------------
// Shared by every filter and partition: one look-back pass per 2^30 keys, then the count is read back
// so the result shapes can be filled in.  ARR is any one-dimensional array struct of 4-byte elements.
}  // extern "C"
template <typename ARR>
static int compact_common(futhark_context *ctx, int which, bool partition, const char *name, const memblock_device &in, int64_t n,
                          const uint8_t *flags, ARR **sel, ARR **rej) {
  const int pieces = fb::compact_pieces_needed(n);
  if (pieces > 64) {
    fb_set_error(ctx, "filter/partition: %lld elements exceed the supported 2^36 per call.", (long long)n);
    return 1;
  }
  int rc;
  ARR *t = make_1d<ARR>(ctx, n, 4, name, &rc);
  if (t == nullptr) return rc;
  ARR *f = nullptr;
  if (partition) {
    f = make_1d<ARR>(ctx, n, 4, name, &rc);
    if (f == nullptr) { fb_unref(ctx, &t->mem); free(t); return rc; }
  }
  const int64_t piece_n = n < ((int64_t)1 << 30) ? n : ((int64_t)1 << 30);
  rc = fb_ensure_lookback_scratch(ctx, fb::lookback_scratch_bytes(piece_n));
  if (rc == 0) {
    LaunchScope ls(ctx, name, PROV("scan (+) of predicate flags with scatter post-op"), "{" + kv("n", n) + "}");
    uint32_t epochs[64];
    for (int i = 0; i < pieces; i++) epochs[i] = fb_next_epoch(ctx);
    ctx->launch_count += pieces - 1;
    rc = fb_cuda_check(ctx, fb::launch_compact(which, dptr<void>(in), flags, dptr<void>(t->mem), f ? dptr<void>(f->mem) : nullptr,
                                               n, ctx->d_scalar, ctx->lookback_scratch, epochs, ctx->d_failure, ctx->stream),
                       "compact");
    ctx->failure_is_an_option = true;
  }
  if (rc == 0) rc = fb_cuda_check(ctx, cudaMemcpyAsync(ctx->h_scalar, ctx->d_scalar, sizeof(int64_t), cudaMemcpyDeviceToHost, ctx->stream), "count read");
  if (rc == 0) rc = fb_cuda_check(ctx, cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize");
  int64_t count = 0;
  if (rc == 0) {
    count = ctx->h_scalar[0];
    if (count < 0 || count > n) {   // only possible after a device-side failure; sync reports it
      count = 0;
    }
  }
  if (rc != 0) {
    fb_unref(ctx, &t->mem); free(t);
    if (f) { fb_unref(ctx, &f->mem); free(f); }
    return rc;
  }
  t->shape[0] = count;
  *sel = t;
  if (partition) { f->shape[0] = n - count; *rej = f; }
  return FUTHARK_SUCCESS;
}
extern "C" {

int futhark_entry_filter_u32(struct futhark_context *ctx, struct futhark_u32_1d **out0, const struct futhark_u32_1d *in0) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  futhark_u32_1d *sel = nullptr;
  int rc = compact_common<futhark_u32_1d>(ctx, fb::COMPACT_FILTER_LOW3_U32, false, "filter_u32.segscan", in0->mem, in0->shape[0], nullptr, &sel, nullptr);
  if (rc == 0) *out0 = sel;
  return rc;
}

int futhark_entry_partition_u32(struct futhark_context *ctx, struct futhark_opaque_tup2_arr1d_u32_arr1d_u32 **out0,
                                const struct futhark_u32_1d *in0) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  futhark_u32_1d *sel = nullptr, *rej = nullptr;
  int rc = compact_common<futhark_u32_1d>(ctx, fb::COMPACT_PARTITION_LOW3_U32, true, "partition_u32.segscan", in0->mem, in0->shape[0], nullptr, &sel, &rej);
  if (rc != 0) return rc;
  auto *p = (futhark_opaque_tup2_arr1d_u32_arr1d_u32 *)malloc(sizeof(futhark_opaque_tup2_arr1d_u32_arr1d_u32));
  if (p == nullptr) return 1;
  p->v0 = sel;
  p->v1 = rej;
  *out0 = p;
  return FUTHARK_SUCCESS;
}

// filter (0 <) xs (tests/soacs/filter1.fut): the compaction kernel under another predicate.
int futhark_entry_filter_pos_i32(struct futhark_context *ctx, struct futhark_i32_1d **out0, const struct futhark_i32_1d *in0) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  futhark_i32_1d *sel = nullptr;
  int rc = compact_common<futhark_i32_1d>(ctx, fb::COMPACT_FILTER_POS_I32, false, "filter_pos_i32.segscan", in0->mem, in0->shape[0], nullptr, &sel, nullptr);
  if (rc == 0) *out0 = sel;
  return rc;
}

// (filter (.1) (zip xs keep)).0 (tests/soacs/filter3.fut): the predicate reads a second array.
int futhark_entry_filter_by_flag_i32(struct futhark_context *ctx, struct futhark_i32_1d **out0, const struct futhark_i32_1d *in0,
                                     const struct futhark_bool_1d *in1) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  if (in1->shape[0] != in0->shape[0]) return bad_sizes(ctx);
  futhark_i32_1d *sel = nullptr;
  int rc = compact_common<futhark_i32_1d>(ctx, fb::COMPACT_FILTER_BY_FLAG_I32, false, "filter_by_flag_i32.segscan", in0->mem, in0->shape[0],
                                          dptr<uint8_t>(in1->mem), &sel, nullptr);
  if (rc == 0) *out0 = sel;
  return rc;
}

// partition2 (\x -> x % 2 == 0) (\x -> x % 3 == 0) xs (tests/soacs/partition1.fut; prelude/soacs.fut:293-323):
// a partition by the first predicate, then a partition of what it rejected by the second.  All
// three groups keep the original order.
int futhark_entry_partition2_i32(struct futhark_context *ctx, struct futhark_opaque_tup3_arr1d_i32_arr1d_i32_arr1d_i32 **out0,
                                 const struct futhark_i32_1d *in0) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  futhark_i32_1d *c0 = nullptr, *rest = nullptr, *c1 = nullptr, *c2 = nullptr;
  int rc = compact_common<futhark_i32_1d>(ctx, fb::COMPACT_PARTITION_EVEN_I32, true, "partition2_i32.segscan", in0->mem, in0->shape[0], nullptr, &c0, &rest);
  if (rc != 0) return rc;
  rc = compact_common<futhark_i32_1d>(ctx, fb::COMPACT_PARTITION_DIV3_I32, true, "partition2_i32.segscan", rest->mem, rest->shape[0], nullptr, &c1, &c2);
  fb_unref(ctx, &rest->mem); free(rest);
  if (rc != 0) { fb_unref(ctx, &c0->mem); free(c0); return rc; }
  auto *p = (futhark_opaque_tup3_arr1d_i32_arr1d_i32_arr1d_i32 *)malloc(sizeof(futhark_opaque_tup3_arr1d_i32_arr1d_i32_arr1d_i32));
  if (p == nullptr) return 1;
  p->v[0] = c0; p->v[1] = c1; p->v[2] = c2;
  *out0 = p;
  return FUTHARK_SUCCESS;
}

int futhark_free_opaque_tup3_arr1d_i32_arr1d_i32_arr1d_i32(struct futhark_context *ctx, struct futhark_opaque_tup3_arr1d_i32_arr1d_i32_arr1d_i32 *obj) {
  if (obj == nullptr) return 0;
  for (int i = 0; i < 3; i++) futhark_free_i32_1d(ctx, obj->v[i]);
  free(obj);
  return 0;
}

int futhark_new_opaque_tup3_arr1d_i32_arr1d_i32_arr1d_i32(struct futhark_context *ctx, struct futhark_opaque_tup3_arr1d_i32_arr1d_i32_arr1d_i32 **out,
                                                          const struct futhark_i32_1d *v0, const struct futhark_i32_1d *v1, const struct futhark_i32_1d *v2) {
  CtxGuard g(ctx);
  auto *p = (futhark_opaque_tup3_arr1d_i32_arr1d_i32_arr1d_i32 *)malloc(sizeof(futhark_opaque_tup3_arr1d_i32_arr1d_i32_arr1d_i32));
  if (p == nullptr) return 1;
  const futhark_i32_1d *src[3] = {v0, v1, v2};
  for (int i = 0; i < 3; i++) {
    p->v[i] = (futhark_i32_1d *)malloc(sizeof(futhark_i32_1d));
    if (p->v[i] == nullptr) return 1;
    *p->v[i] = *src[i];
    fb_ref(&p->v[i]->mem);         // the record shares the blocks of its fields (docs/c-api.rst:366-381)
  }
  *out = p;
  return 0;
}

static int project_tup3(futhark_context *ctx, futhark_i32_1d **out, const futhark_opaque_tup3_arr1d_i32_arr1d_i32_arr1d_i32 *obj, int i) {
  CtxGuard g(ctx);
  futhark_i32_1d *a = (futhark_i32_1d *)malloc(sizeof(futhark_i32_1d));
  if (a == nullptr) return 1;
  *a = *obj->v[i];
  fb_ref(&a->mem);          // the projection shares the block (docs/c-api.rst:383-391)
  *out = a;
  return 0;
}
int futhark_project_opaque_tup3_arr1d_i32_arr1d_i32_arr1d_i32_0(struct futhark_context *ctx, struct futhark_i32_1d **out,
                                                                const struct futhark_opaque_tup3_arr1d_i32_arr1d_i32_arr1d_i32 *obj) { return project_tup3(ctx, out, obj, 0); }
int futhark_project_opaque_tup3_arr1d_i32_arr1d_i32_arr1d_i32_1(struct futhark_context *ctx, struct futhark_i32_1d **out,
                                                                const struct futhark_opaque_tup3_arr1d_i32_arr1d_i32_arr1d_i32 *obj) { return project_tup3(ctx, out, obj, 1); }
int futhark_project_opaque_tup3_arr1d_i32_arr1d_i32_arr1d_i32_2(struct futhark_context *ctx, struct futhark_i32_1d **out,
                                                                const struct futhark_opaque_tup3_arr1d_i32_arr1d_i32_arr1d_i32 *obj) { return project_tup3(ctx, out, obj, 2); }

// partition2 (\(x, y) -> x < y) (\(x, y) -> x == y) (zip xs ys), unzipped (tests/soacs/partition2.fut;
// prelude/soacs.fut:293-323): one kernel writes the class of every pair as three arrays of keep-flags,
// and each component of each group is a filter by its flags, so all six arrays keep the original order.
#define FB_TUP6 futhark_opaque_tup6_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32
int futhark_entry_partition2_pairs_i32(struct futhark_context *ctx, struct FB_TUP6 **out0, const struct futhark_i32_1d *in0,
                                       const struct futhark_i32_1d *in1) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  const int64_t n = in0->shape[0];
  if (in1->shape[0] != n) return bad_sizes(ctx);
  const int64_t pitch = (n + 255) & ~(int64_t)255;          // every flag array starts on a 256-byte boundary
  memblock_device keep;
  int rc = fb_alloc(ctx, (size_t)(3 * pitch > 0 ? 3 * pitch : 1), "partition2_pairs_i32.keep", &keep);
  if (rc != 0) return rc;
  ctx->launch_count++;
  rc = fb_cuda_check(ctx, fb::launch_classify_pairs_lt_eq(dptr<int32_t>(in0->mem), dptr<int32_t>(in1->mem), n, pitch, dptr<uint8_t>(keep),
                                                          ctx->num_sms, ctx->stream), "classify_pairs");
  futhark_i32_1d *part[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  for (int k = 0; k < 6 && rc == 0; k++) {
    const futhark_i32_1d *src = (k & 1) ? in1 : in0;
    rc = compact_common<futhark_i32_1d>(ctx, fb::COMPACT_FILTER_BY_FLAG_I32, false, "partition2_pairs_i32.segscan", src->mem, n,
                                        dptr<uint8_t>(keep) + (k >> 1) * pitch, &part[k], nullptr);
  }
  fb_unref(ctx, &keep);
  FB_TUP6 *p = rc == 0 ? (FB_TUP6 *)malloc(sizeof(FB_TUP6)) : nullptr;
  if (p == nullptr) {
    for (int k = 0; k < 6; k++) if (part[k] != nullptr) { fb_unref(ctx, &part[k]->mem); free(part[k]); }
    return rc != 0 ? rc : 1;
  }
  for (int k = 0; k < 6; k++) p->v[k] = part[k];
  *out0 = p;
  return FUTHARK_SUCCESS;
}

int futhark_free_opaque_tup6_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32(struct futhark_context *ctx, struct FB_TUP6 *obj) {
  if (obj == nullptr) return 0;
  for (int i = 0; i < 6; i++) futhark_free_i32_1d(ctx, obj->v[i]);
  free(obj);
  return 0;
}

int futhark_new_opaque_tup6_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32(
    struct futhark_context *ctx, struct FB_TUP6 **out, const struct futhark_i32_1d *v0, const struct futhark_i32_1d *v1,
    const struct futhark_i32_1d *v2, const struct futhark_i32_1d *v3, const struct futhark_i32_1d *v4, const struct futhark_i32_1d *v5) {
  CtxGuard g(ctx);
  FB_TUP6 *p = (FB_TUP6 *)malloc(sizeof(FB_TUP6));
  if (p == nullptr) return 1;
  const futhark_i32_1d *src[6] = {v0, v1, v2, v3, v4, v5};
  for (int i = 0; i < 6; i++) {
    p->v[i] = (futhark_i32_1d *)malloc(sizeof(futhark_i32_1d));
    if (p->v[i] == nullptr) return 1;
    *p->v[i] = *src[i];
    fb_ref(&p->v[i]->mem);         // the record shares the blocks of its fields (docs/c-api.rst:366-381)
  }
  *out = p;
  return 0;
}

static int project_tup6(futhark_context *ctx, futhark_i32_1d **out, const FB_TUP6 *obj, int i) {
  CtxGuard g(ctx);
  futhark_i32_1d *a = (futhark_i32_1d *)malloc(sizeof(futhark_i32_1d));
  if (a == nullptr) return 1;
  *a = *obj->v[i];
  fb_ref(&a->mem);          // the projection shares the block (docs/c-api.rst:383-391)
  *out = a;
  return 0;
}
#define FB_TUP6_PROJECT(I)                                                                                             \
  int futhark_project_opaque_tup6_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_##I(                     \
      struct futhark_context *ctx, struct futhark_i32_1d **out, const struct FB_TUP6 *obj) {                           \
    return project_tup6(ctx, out, obj, I);                                                                             \
  }
FB_TUP6_PROJECT(0)
FB_TUP6_PROJECT(1)
FB_TUP6_PROJECT(2)
FB_TUP6_PROJECT(3)
FB_TUP6_PROJECT(4)
FB_TUP6_PROJECT(5)
#undef FB_TUP6_PROJECT
#undef FB_TUP6

// ---- scans under other specifications of the single-pass kernel -------------------------------------
}  // extern "C"
template <typename ARR>
static int scan_like(futhark_context *ctx, ARR **out0, const ARR *in0, int64_t n, const char *name, const char *prov,
                     cudaError_t (*launch)(futhark_context *, const ARR *, ARR *, int64_t)) {
  ARR *out = (ARR *)malloc(sizeof(ARR));
  if (out == nullptr) return 1;
  *out = *in0;                                   // same shape
  int rc = fb_alloc(ctx, (size_t)n * 4, name, &out->mem);
  if (rc != 0) { free(out); return rc; }
  if (n > 0) {
    rc = fb_ensure_lookback_scratch(ctx, fb::lookback_scratch_bytes(n));
    if (rc == 0) {
      LaunchScope ls(ctx, name, prov, "{" + kv("n", n) + "}");
      rc = fb_cuda_check(ctx, launch(ctx, in0, out, n), name);
      ctx->failure_is_an_option = true;
    }
    if (rc != 0) { fb_unref(ctx, &out->mem); free(out); return rc; }
  }
  *out0 = out;
  return FUTHARK_SUCCESS;
}
extern "C" {

// scan i32.max i32.lowest xs
int futhark_entry_scan_max_i32(struct futhark_context *ctx, struct futhark_i32_1d **out0, const struct futhark_i32_1d *in0) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  return scan_like<futhark_i32_1d>(ctx, out0, in0, in0->shape[0], "scan_max_i32.segscan", PROV("scan i32.max i32.lowest xs"),
                                   [](futhark_context *c, const futhark_i32_1d *in, futhark_i32_1d *out, int64_t n) {
                                     return fb::launch_scan_variant_i32(1, dptr<int32_t>(in->mem), dptr<int32_t>(out->mem), n, 0, nullptr, c->lookback_scratch,
                                                                        fb_next_epoch(c), c->d_failure, c->stream);
                                   });
}

// map (scan (+) 0) xss (tests/intrablock/segscan0.fut): a regular segmented scan, one launch over all rows.
int futhark_entry_segscan_rows_i32(struct futhark_context *ctx, struct futhark_i32_2d **out0, const struct futhark_i32_2d *in0) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  return scan_like<futhark_i32_2d>(ctx, out0, in0, in0->shape[0] * in0->shape[1], "segscan_rows_i32.segscan", PROV("map (scan (+) 0) xss"),
                                   [](futhark_context *c, const futhark_i32_2d *in, futhark_i32_2d *out, int64_t) {
                                     return fb::launch_segscan_rows_i32(dptr<int32_t>(in->mem), dptr<int32_t>(out->mem), in->shape[0], in->shape[1],
                                                                        c->lookback_scratch, fb_next_epoch(c), c->d_failure, c->stream);
                                   });
}

// tests/soacs/scan4.fut: two rounds of  xs' = map2 (+) (map (+ sum) (scan (+) 0 (map (+1) xs))) xs  with
// sum = reduce (+) 0 (map (+1) xs).  Per round one reduction (sum of xs; the n ones are added on the
// host side of the seed) and one scan kernel with the map body and the post-operation fused in.
int futhark_entry_scanomap_steps_i32(struct futhark_context *ctx, struct futhark_i32_1d **out0, const struct futhark_i32_1d *in0) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  const int64_t n = in0->shape[0];
  futhark_i32_1d *mid = nullptr;
  auto round = [](futhark_context *c, const futhark_i32_1d *in, futhark_i32_1d *out, int64_t n) -> cudaError_t {
    int32_t *sum = reinterpret_cast<int32_t *>(c->d_scalar + 2);
    cudaError_t err = fb::launch_reduce_i32(dptr<int32_t>(in->mem), n, sum, c->reduce_scratch, c->num_sms, c->stream);
    if (err != cudaSuccess) return err;
    c->launch_count++;
    return fb::launch_scan_variant_i32(2, dptr<int32_t>(in->mem), dptr<int32_t>(out->mem), n, (int32_t)(uint32_t)n, sum, c->lookback_scratch,
                                       fb_next_epoch(c), c->d_failure, c->stream);
  };
  int rc = scan_like<futhark_i32_1d>(ctx, &mid, in0, n, "scanomap_steps_i32.segscan", PROV("scan (+) 0 (map (+1) xs), post-op (+ sum + x)"), round);
  if (rc != 0) return rc;
  rc = scan_like<futhark_i32_1d>(ctx, out0, mid, n, "scanomap_steps_i32.segscan", PROV("scan (+) 0 (map (+1) xs), post-op (+ sum + x)"), round);
  fb_unref(ctx, &mid->mem); free(mid);
  return rc;
}

// scan (+) 0 over i64, and a scan over pairs: operators the single-pass kernel's 32-bit status
// word cannot carry go through the two-pass route (SegScan/TwoPass.hs:621-682).
int futhark_entry_scan_i64(struct futhark_context *ctx, struct futhark_i64_1d **out0, const struct futhark_i64_1d *in0) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  const int64_t n = in0->shape[0];
  int rc;
  futhark_i64_1d *out = make_1d<futhark_i64_1d>(ctx, n, 8, "scan_i64.out", &rc);
  if (out == nullptr) return rc;
  if (n > 0) {
    LaunchScope ls(ctx, "scan_i64.scan_stage1-3", PROV("scan (+) 0 xs"), "{" + kv("n", n) + "}");
    ctx->launch_count += 2;
    rc = fb_cuda_check(ctx, fb::launch_scan_i64(dptr<int64_t>(in0->mem), dptr<int64_t>(out->mem), n, ctx->reduce_scratch, ctx->num_sms, ctx->stream), "scan_i64");
    if (rc != 0) { fb_unref(ctx, &out->mem); free(out); return rc; }
  }
  *out0 = out;
  return FUTHARK_SUCCESS;
}

int futhark_entry_linrec_f32(struct futhark_context *ctx, struct futhark_f32_1d **out0, const struct futhark_f32_1d *in0,
                             const struct futhark_f32_1d *in1) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  const int64_t n = in0->shape[0];
  if (in1->shape[0] != n) return bad_sizes(ctx);
  int rc;
  futhark_f32_1d *out = make_1d<futhark_f32_1d>(ctx, n, 4, "linrec_f32.out", &rc);
  if (out == nullptr) return rc;
  if (n > 0) {
    LaunchScope ls(ctx, "linrec_f32.scan_stage1-3", PROV("map (.1) (scan compose (1,0) (zip as bs))"), "{" + kv("n", n) + "}");
    ctx->launch_count += 2;
    rc = fb_cuda_check(ctx, fb::launch_linrec_f32(dptr<float>(in0->mem), dptr<float>(in1->mem), dptr<float>(out->mem), n, ctx->reduce_scratch,
                                                  ctx->num_sms, ctx->stream), "linrec_f32");
    if (rc != 0) { fb_unref(ctx, &out->mem); free(out); return rc; }
  }
  *out0 = out;
  return FUTHARK_SUCCESS;
}

int futhark_entry_bmm_f16(struct futhark_context *ctx, struct futhark_f32_3d **out0, const struct futhark_f16_3d *in0,
                          const struct futhark_f16_3d *in1) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  const int64_t nb = in0->shape[0], m = in0->shape[1], k = in0->shape[2], n = in1->shape[2];
  if (in1->shape[0] != nb || in1->shape[1] != k) return bad_sizes(ctx);
  futhark_f32_3d *out = (futhark_f32_3d *)malloc(sizeof(futhark_f32_3d));
  if (out == nullptr) return 1;
  out->shape[0] = nb; out->shape[1] = m; out->shape[2] = n;
  int rc = fb_alloc(ctx, (size_t)(nb * m * n) * 4, "bmm_f16.out", &out->mem);
  if (rc != 0) { free(out); return rc; }
  {
    LaunchScope ls(ctx, "bmm_f16.segmap_intrablock", PROV("map2 (matmul) A B"),
                   "{" + kv("batch", nb) + "," + kv("m", m) + "," + kv("k", k) + "," + kv("n", n) + "}");
    rc = fb_cuda_check(ctx, fb::launch_bmm_f16(dptr<uint16_t>(in0->mem), dptr<uint16_t>(in1->mem), dptr<float>(out->mem), nb, m, k, n,
                                               ctx->d_failure, ctx->stream), "bmm_f16");
    ctx->failure_is_an_option = true;
  }
  if (rc != 0) { fb_unref(ctx, &out->mem); free(out); return rc; }
  *out0 = out;
  return FUTHARK_SUCCESS;
}

static int transpose_common(futhark_context *ctx, int64_t nb, int64_t rows, int64_t cols, const memblock_device &in, memblock_device *out) {
  int rc = fb_alloc(ctx, (size_t)(nb * rows * cols) * 4, "transpose_f32.out", out);
  if (rc != 0) return rc;
  if (nb * rows * cols > 0) {
    LaunchScope ls(ctx, "transpose_f32.map_transpose_4b", PROV("map transpose xsss"),
                   "{" + kv("batch", nb) + "," + kv("rows", rows) + "," + kv("cols", cols) + "}");
    rc = fb_cuda_check(ctx, fb::launch_transpose_b32(dptr<void>(in), dptr<void>(*out), nb, rows, cols, ctx->num_sms, ctx->stream), "transpose_f32");
    if (rc != 0) fb_unref(ctx, out);
  }
  return rc;
}

int futhark_entry_transpose_f32(struct futhark_context *ctx, struct futhark_f32_2d **out0, const struct futhark_f32_2d *in0) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  futhark_f32_2d *out = (futhark_f32_2d *)malloc(sizeof(futhark_f32_2d));
  if (out == nullptr) return 1;
  out->shape[0] = in0->shape[1]; out->shape[1] = in0->shape[0];
  int rc = transpose_common(ctx, 1, in0->shape[0], in0->shape[1], in0->mem, &out->mem);
  if (rc != 0) { free(out); return rc; }
  *out0 = out;
  return FUTHARK_SUCCESS;
}

int futhark_entry_transpose_f32_3d(struct futhark_context *ctx, struct futhark_f32_3d **out0, const struct futhark_f32_3d *in0) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  futhark_f32_3d *out = (futhark_f32_3d *)malloc(sizeof(futhark_f32_3d));
  if (out == nullptr) return 1;
  out->shape[0] = in0->shape[0]; out->shape[1] = in0->shape[2]; out->shape[2] = in0->shape[1];
  int rc = transpose_common(ctx, in0->shape[0], in0->shape[1], in0->shape[2], in0->mem, &out->mem);
  if (rc != 0) { free(out); return rc; }
  *out0 = out;
  return FUTHARK_SUCCESS;
}

// scan (map2 (+)) (replicate k 0) xss over xss: [m][k]i32 (tests/soacs/scan-with-map.fut, scan5.fut): a scan
// whose operator works on whole rows.  The rows' elements never meet, so the scan is interchanged with
// the inner map, as the reference does before it extracts kernels (src/Futhark/Transform/ISRWIM.hs):
// transpose, one regular segmented scan over the k columns laid out as rows, transpose back.
int futhark_entry_scan_map2_add_i32(struct futhark_context *ctx, struct futhark_i32_2d **out0, const struct futhark_i32_2d *in0) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  const int64_t m = in0->shape[0], k = in0->shape[1];
  futhark_i32_2d *out = (futhark_i32_2d *)malloc(sizeof(futhark_i32_2d));
  if (out == nullptr) return 1;
  out->shape[0] = m; out->shape[1] = k;
  memblock_device cols, scanned;
  int rc = transpose_common(ctx, 1, m, k, in0->mem, &cols);                    // [k][m]
  if (rc != 0) { free(out); return rc; }
  rc = fb_alloc(ctx, (size_t)(m * k) * 4, "scan_map2_add_i32.scanned", &scanned);
  if (rc != 0) { fb_unref(ctx, &cols); free(out); return rc; }
  if (m * k > 0) {
    rc = fb_ensure_lookback_scratch(ctx, fb::lookback_scratch_bytes(m * k));
    if (rc == 0) {
      LaunchScope ls(ctx, "scan_map2_add_i32.segscan", PROV("scan (map2 (+)) (replicate k 0) xss"), "{" + kv("m", m) + "," + kv("k", k) + "}");
      rc = fb_cuda_check(ctx, fb::launch_segscan_rows_i32(dptr<int32_t>(cols), dptr<int32_t>(scanned), k, m, ctx->lookback_scratch,
                                                          fb_next_epoch(ctx), ctx->d_failure, ctx->stream), "scan_map2_add_i32");
      ctx->failure_is_an_option = true;
    }
  }
  fb_unref(ctx, &cols);
  if (rc == 0) rc = transpose_common(ctx, 1, k, m, scanned, &out->mem);        // [m][k]
  fb_unref(ctx, &scanned);
  if (rc != 0) { free(out); return rc; }
  *out0 = out;
  return FUTHARK_SUCCESS;
}

// map transpose over f16 (the `transpose b` of the matrix product, tests/reg-tiling/mmm.fut:17-21), and
// transposition of 8-byte and 1-byte elements: rts/opencl/transpose.cl:3-277 at the other widths.
static int transpose_sized(futhark_context *ctx, int es, int64_t nb, int64_t rows, int64_t cols, const memblock_device &in, memblock_device *out,
                           const char *name) {
  int rc = fb_alloc(ctx, (size_t)(nb * rows * cols) * es, name, out);
  if (rc != 0) return rc;
  if (nb * rows * cols > 0) {
    LaunchScope ls(ctx, name, PROV("map transpose xsss"), "{" + kv("batch", nb) + "," + kv("rows", rows) + "," + kv("cols", cols) + "," + kv("elem_size", es) + "}");
    rc = fb_cuda_check(ctx, fb::launch_transpose(es, dptr<void>(in), dptr<void>(*out), nb, rows, cols, ctx->num_sms, ctx->stream), name);
    if (rc != 0) fb_unref(ctx, out);
  }
  return rc;
}

int futhark_entry_transpose_f16_3d(struct futhark_context *ctx, struct futhark_f16_3d **out0, const struct futhark_f16_3d *in0) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  futhark_f16_3d *out = (futhark_f16_3d *)malloc(sizeof(futhark_f16_3d));
  if (out == nullptr) return 1;
  out->shape[0] = in0->shape[0]; out->shape[1] = in0->shape[2]; out->shape[2] = in0->shape[1];
  int rc = transpose_sized(ctx, 2, in0->shape[0], in0->shape[1], in0->shape[2], in0->mem, &out->mem, "transpose_f16_3d.map_transpose_2b");
  if (rc != 0) { free(out); return rc; }
  *out0 = out;
  return FUTHARK_SUCCESS;
}

int futhark_entry_transpose_i64(struct futhark_context *ctx, struct futhark_i64_2d **out0, const struct futhark_i64_2d *in0) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  futhark_i64_2d *out = (futhark_i64_2d *)malloc(sizeof(futhark_i64_2d));
  if (out == nullptr) return 1;
  out->shape[0] = in0->shape[1]; out->shape[1] = in0->shape[0];
  int rc = transpose_sized(ctx, 8, 1, in0->shape[0], in0->shape[1], in0->mem, &out->mem, "transpose_i64.map_transpose_8b");
  if (rc != 0) { free(out); return rc; }
  *out0 = out;
  return FUTHARK_SUCCESS;
}

int futhark_entry_transpose_bool(struct futhark_context *ctx, struct futhark_bool_2d **out0, const struct futhark_bool_2d *in0) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  futhark_bool_2d *out = (futhark_bool_2d *)malloc(sizeof(futhark_bool_2d));
  if (out == nullptr) return 1;
  out->shape[0] = in0->shape[1]; out->shape[1] = in0->shape[0];
  int rc = transpose_sized(ctx, 1, 1, in0->shape[0], in0->shape[1], in0->mem, &out->mem, "transpose_bool.map_transpose_1b");
  if (rc != 0) { free(out); return rc; }
  *out0 = out;
  return FUTHARK_SUCCESS;
}

// replicate n v and iota n: the fills the compiler puts around SegOps (ImpGen/GPU/Base.hs:1342-1436)
int futhark_entry_replicate_i32(struct futhark_context *ctx, struct futhark_i32_1d **out0, const int64_t in0, const int32_t in1) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  if (in0 < 0) { fb_set_error(ctx, "Error: negative array size %lld.\n", (long long)in0); return FUTHARK_PROGRAM_ERROR; }
  int rc;
  futhark_i32_1d *out = make_1d<futhark_i32_1d>(ctx, in0, 4, "replicate_i32.out", &rc);
  if (out == nullptr) return rc;
  if (in0 > 0) {
    LaunchScope ls(ctx, "replicate_i32.replicate", PROV("replicate n v"), "{" + kv("n", in0) + "}");
    rc = fb_cuda_check(ctx, fb::launch_replicate(4, dptr<void>(out->mem), in0, (uint32_t)in1, ctx->num_sms, ctx->stream), "replicate_i32");
    if (rc != 0) { fb_unref(ctx, &out->mem); free(out); return rc; }
  }
  *out0 = out;
  return FUTHARK_SUCCESS;
}

int futhark_entry_iota_i64(struct futhark_context *ctx, struct futhark_i64_1d **out0, const int64_t in0) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  if (in0 < 0) { fb_set_error(ctx, "Error: negative array size %lld.\n", (long long)in0); return FUTHARK_PROGRAM_ERROR; }
  int rc;
  futhark_i64_1d *out = make_1d<futhark_i64_1d>(ctx, in0, 8, "iota_i64.out", &rc);
  if (out == nullptr) return rc;
  if (in0 > 0) {
    LaunchScope ls(ctx, "iota_i64.iota", PROV("iota n"), "{" + kv("n", in0) + "}");
    rc = fb_cuda_check(ctx, fb::launch_iota(8, dptr<void>(out->mem), in0, 0, 1, ctx->num_sms, ctx->stream), "iota_i64");
    if (rc != 0) { fb_unref(ctx, &out->mem); free(out); return rc; }
  }
  *out0 = out;
  return FUTHARK_SUCCESS;
}

int futhark_b200_debug_expire_wait(struct futhark_context *ctx, int max_polls) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  int rc = fb_ensure_lookback_scratch(ctx, fb::lookback_scratch_bytes(1));
  if (rc != 0) return rc;
  ctx->launch_count++;
  rc = fb_cuda_check(ctx, fb::launch_expire_wait(ctx->lookback_scratch, fb_next_epoch(ctx), (uint32_t)(max_polls < 1 ? 1 : max_polls),
                                                 ctx->d_failure, ctx->stream), "expire_wait");
  ctx->failure_is_an_option = true;
  return rc;
}

// ---- strided copies between device arrays (extension; the reference's lmad_copy_gpu2gpu) -------

int futhark_b200_lmad_classify(int r, const int64_t *dst_strides, const int64_t *src_strides, const int64_t *shape, int64_t *knm) {
  if (r < 0 || r > fb::LMAD_MAX_RANK) return -2;
  int64_t ns[fb::LMAD_MAX_RANK], nd[fb::LMAD_MAX_RANK], nsrc[fb::LMAD_MAX_RANK];
  const int m = fb::lmad_normalise(r, dst_strides, src_strides, shape, ns, nd, nsrc);
  int64_t nb = 0, rows = 0, cols = 0;
  const int kind = fb::lmad_classify(m, ns, nd, nsrc, &nb, &rows, &cols);
  if (knm != nullptr) { knm[0] = nb; knm[1] = rows; knm[2] = cols; }
  return kind;
}

int futhark_b200_lmad_copy(struct futhark_context *ctx, int elem_size, int r, CUdeviceptr dst, int64_t dst_offset,
                           const int64_t *dst_strides, CUdeviceptr src, int64_t src_offset, const int64_t *src_strides,
                           const int64_t *shape) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  if (r < 0 || r > fb::LMAD_MAX_RANK || (elem_size != 1 && elem_size != 2 && elem_size != 4 && elem_size != 8)) {
    fb_set_error(ctx, "lmad_copy: the rank must be 0..8 and the element size 1, 2, 4 or 8 bytes.\n");
    return 1;
  }
  int64_t total = 1;
  for (int i = 0; i < r; i++) {
    if (shape[i] < 0) return bad_sizes(ctx);
    total *= shape[i];
  }
  if (total == 0) return FUTHARK_SUCCESS;
  int kind = futhark_b200_lmad_classify(r, dst_strides, src_strides, shape, nullptr);
  const char *name = kind == fb::LMAD_FLAT ? "copy_dev_to_dev" : kind == fb::LMAD_TRANSPOSE ? "lmad_copy.map_transpose" : "lmad_copy.general";
  LaunchScope ls(ctx, name, PROV("copy"), "{" + kv("elements", total) + "," + kv("elem_size", elem_size) + "}");
  return fb_cuda_check(ctx, fb::launch_lmad_copy(elem_size, r, reinterpret_cast<void *>((uintptr_t)dst), dst_offset, dst_strides,
                                                 reinterpret_cast<const void *>((uintptr_t)src), src_offset, src_strides, shape,
                                                 ctx->num_sms, ctx->stream, nullptr), "lmad_copy");
}

// ---- shard-local pieces for arrays split across several contexts (extensions) -------------------

int futhark_b200_reduce_i32_to_device(struct futhark_context *ctx, CUdeviceptr dst, const struct futhark_i32_1d *in0) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  LaunchScope ls(ctx, "reduce_i32.segred_nonseg", PROV("reduce (+) 0 xs"), "{" + kv("n", in0->shape[0]) + "}");
  return fb_cuda_check(ctx, fb::launch_reduce_i32(dptr<int32_t>(in0->mem), in0->shape[0], reinterpret_cast<int32_t *>((uintptr_t)dst),
                                                  ctx->reduce_scratch, ctx->num_sms, ctx->stream), "reduce_i32");
}

int futhark_b200_entry_scan_i32_carried(struct futhark_context *ctx, struct futhark_i32_1d **out0, const struct futhark_i32_1d *in0,
                                        CUdeviceptr carries, int num_carries) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  const int64_t n = in0->shape[0];
  int rc;
  futhark_i32_1d *out = make_1d<futhark_i32_1d>(ctx, n, 4, "scan_i32.out", &rc);
  if (out == nullptr) return rc;
  if (n > 0) {
    rc = fb_ensure_lookback_scratch(ctx, fb::lookback_scratch_bytes(n));
    if (rc == 0) {
      LaunchScope ls(ctx, "scan_i32.segscan", PROV("scan (+) carry xs"), "{" + kv("n", n) + "}");
      rc = fb_cuda_check(ctx, fb::launch_scan_i32(dptr<int32_t>(in0->mem), dptr<int32_t>(out->mem), n, 0,
                                                  reinterpret_cast<const int32_t *>((uintptr_t)carries), num_carries,
                                                  ctx->lookback_scratch, fb_next_epoch(ctx), ctx->d_failure, ctx->stream), "scan_i32");
      ctx->failure_is_an_option = true;
    }
    if (rc != 0) { fb_unref(ctx, &out->mem); free(out); return rc; }
  }
  *out0 = out;
  return FUTHARK_SUCCESS;
}

int futhark_b200_entry_segscan_f32_shard(struct futhark_context *ctx, struct futhark_f32_1d **out0, CUdeviceptr summary_dst,
                                         const struct futhark_bool_1d *in0, const struct futhark_f32_1d *in1) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  // the scan kernel writes the summary itself: one launch, one critical section
  return segscan_f32_locked(ctx, out0, in0, in1, reinterpret_cast<uint32_t *>((uintptr_t)summary_dst), nullptr);
}

int futhark_b200_segscan_f32_apply_carries(struct futhark_context *ctx, struct futhark_f32_1d *out, const struct futhark_bool_1d *in0,
                                           CUdeviceptr summaries, int rank) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  if (out->shape[0] != in0->shape[0]) return bad_sizes(ctx);
  if (rank <= 0 || out->shape[0] <= 0) return FUTHARK_SUCCESS;
  LaunchScope ls(ctx, "segscan_f32.apply_carry", PROV("carry of the shards before this one"), "{" + kv("n", out->shape[0]) + "}");
  return fb_cuda_check(ctx, fb::launch_segscan_apply_carry(dptr<float>(out->mem), dptr<uint8_t>(in0->mem), out->shape[0],
                                                           reinterpret_cast<const uint32_t *>((uintptr_t)summaries), rank,
                                                           ctx->num_sms, ctx->stream),
                       "segscan carry");
}

}  // extern "C"
