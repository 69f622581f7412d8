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
                                                  fb_next_epoch(ctx), ctx->d_failure, ctx->stream), "scan_i32");
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
                                                  ctx->reduce_scratch, ctx->num_sms, ctx->stream), "reduce_i32");
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

// The caller holds the context's lock.  shard_out (device, 4 words, or NULL): see launch_segscan_f32.
static int segscan_f32_locked(futhark_context *ctx, struct futhark_f32_1d **out0, const struct futhark_bool_1d *in0,
                              const struct futhark_f32_1d *in1, uint32_t *shard_out) {
  const int64_t n = in1->shape[0];
  if (in0->shape[0] != n) return bad_sizes(ctx);
  int rc;
  futhark_f32_1d *out = make_1d<futhark_f32_1d>(ctx, n, 4, "segscan_f32.out", &rc);
  if (out == nullptr) return rc;
  rc = n > 0 ? fb_ensure_lookback_scratch(ctx, fb::lookback_scratch_bytes(n)) : 0;
  if (rc == 0 && (n > 0 || shard_out != nullptr)) {
    LaunchScope ls(ctx, "segscan_f32.segscan", PROV("scan lifted(+) (false,0) (zip flags xs)"), "{" + kv("n", n) + "}");
    rc = fb_cuda_check(ctx, fb::launch_segscan_f32(dptr<uint8_t>(in0->mem), dptr<float>(in1->mem), dptr<float>(out->mem), n, 0.0f, shard_out,
                                                   ctx->lookback_scratch, fb_next_epoch(ctx), ctx->d_failure, ctx->stream), "segscan_f32");
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
  return segscan_f32_locked(ctx, out0, in0, in1, nullptr);
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
    rc = fb_cuda_check(ctx, fb::launch_rowsum_f32(dptr<float>(in0->mem), rows, cols, dptr<float>(out->mem), ctx->num_sms, ctx->stream), "rowsum_f32");
    if (rc != 0) { fb_unref(ctx, &out->mem); free(out); return rc; }
  }
  *out0 = out;
  return FUTHARK_SUCCESS;
}

static int hist_common(futhark_context *ctx, int op, void **out_arr, int64_t B, const futhark_i32_1d *is, const memblock_device &ws,
                       int64_t ws_len, const char *name) {
  const int64_t n = is->shape[0];
  if (ws_len != n) return bad_sizes(ctx);
  if (B < 0) {
    // a negative size is a program error in the reference (array construction with a negative length)
    fb_set_error(ctx, "Error: negative histogram size %lld.\n", (long long)B);
    return FUTHARK_PROGRAM_ERROR;
  }
  int rc;
  futhark_i32_1d *out = make_1d<futhark_i32_1d>(ctx, B, 4, name, &rc);   // same layout for the f32 result
  if (out == nullptr) return rc;
  if (B > 0) {
    LaunchScope ls(ctx, name, PROV("hist op ne B (map i64.i32 is) ws"), "{" + kv("n", n) + "," + kv("bins", B) + "}");
    ctx->launch_count += (op == 1 ? 2 : 1);   // the fill (and, for max, the key decode) besides the histogram kernel
    rc = fb_cuda_check(ctx, fb::launch_hist(op, B, dptr<int32_t>(is->mem), dptr<void>(ws), n, dptr<void>(out->mem), ctx->num_sms, ctx->stream), name);
    if (rc != 0) { fb_unref(ctx, &out->mem); free(out); return rc; }
  }
  *out_arr = out;
  return FUTHARK_SUCCESS;
}

int futhark_entry_hist_add_i32(struct futhark_context *ctx, struct futhark_i32_1d **out0, const int64_t in0, const struct futhark_i32_1d *in1,
                               const struct futhark_i32_1d *in2) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  void *o = nullptr;
  int rc = hist_common(ctx, 0, &o, in0, in1, in2->mem, in2->shape[0], "hist_add_i32.seghist");
  if (rc == 0) *out0 = (futhark_i32_1d *)o;
  return rc;
}

int futhark_entry_hist_max_f32(struct futhark_context *ctx, struct futhark_f32_1d **out0, const int64_t in0, const struct futhark_i32_1d *in1,
                               const struct futhark_f32_1d *in2) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  void *o = nullptr;
  int rc = hist_common(ctx, 1, &o, in0, in1, in2->mem, in2->shape[0], "hist_max_f32.seghist");
  if (rc == 0) *out0 = (futhark_f32_1d *)o;   // futhark_i32_1d and futhark_f32_1d have the same layout
  return rc;
}

// Shared by filter and partition: one look-back pass, then the count is read back so the
// result shapes can be filled in.
static int compact_common(futhark_context *ctx, bool partition, const futhark_u32_1d *in, futhark_u32_1d **sel, futhark_u32_1d **rej) {
  const int64_t n = in->shape[0];
  if (n >= (1ll << 31)) {
    fb_set_error(ctx, "filter/partition: %lld elements exceed the supported 2^31-1 per call.", (long long)n);
    return 1;
  }
  int rc;
  futhark_u32_1d *t = make_1d<futhark_u32_1d>(ctx, n, 4, partition ? "partition_u32.selected" : "filter_u32.out", &rc);
  if (t == nullptr) return rc;
  futhark_u32_1d *f = nullptr;
  if (partition) {
    f = make_1d<futhark_u32_1d>(ctx, n, 4, "partition_u32.rejected", &rc);
    if (f == nullptr) { fb_unref(ctx, &t->mem); free(t); return rc; }
  }
  rc = fb_ensure_lookback_scratch(ctx, fb::lookback_scratch_bytes(n));
  if (rc == 0) {
    LaunchScope ls(ctx, partition ? "partition_u32.segscan" : "filter_u32.segscan", PROV("scan (+) of predicate flags with scatter post-op"),
                   "{" + kv("n", n) + "}");
    rc = fb_cuda_check(ctx, fb::launch_compact_u32(partition, dptr<uint32_t>(in->mem), dptr<uint32_t>(t->mem), f ? dptr<uint32_t>(f->mem) : nullptr,
                                                   n, ctx->d_scalar, ctx->lookback_scratch, fb_next_epoch(ctx), ctx->d_failure, ctx->stream),
                       "compact_u32");
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

int futhark_entry_filter_u32(struct futhark_context *ctx, struct futhark_u32_1d **out0, const struct futhark_u32_1d *in0) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  futhark_u32_1d *sel = nullptr;
  int rc = compact_common(ctx, false, in0, &sel, nullptr);
  if (rc == 0) *out0 = sel;
  return rc;
}

int futhark_entry_partition_u32(struct futhark_context *ctx, struct futhark_opaque_tup2_arr1d_u32_arr1d_u32 **out0,
                                const struct futhark_u32_1d *in0) {
  if (!ctx->ready) return not_ready(ctx);
  CtxGuard g(ctx);
  futhark_u32_1d *sel = nullptr, *rej = nullptr;
  int rc = compact_common(ctx, true, in0, &sel, &rej);
  if (rc != 0) return rc;
  auto *p = (futhark_opaque_tup2_arr1d_u32_arr1d_u32 *)malloc(sizeof(futhark_opaque_tup2_arr1d_u32_arr1d_u32));
  if (p == nullptr) return 1;
  p->v0 = sel;
  p->v1 = rej;
  *out0 = p;
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
  if (kind == fb::LMAD_TRANSPOSE && elem_size != 4) kind = fb::LMAD_GENERAL;
  const char *name = kind == fb::LMAD_FLAT ? "copy_dev_to_dev" : kind == fb::LMAD_TRANSPOSE ? "lmad_copy.map_transpose_4b" : "lmad_copy.general";
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
  return segscan_f32_locked(ctx, out0, in0, in1, reinterpret_cast<uint32_t *>((uintptr_t)summary_dst));
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
