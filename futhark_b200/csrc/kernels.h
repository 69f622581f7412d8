// Host-callable launchers of the sm_100a kernels.  Plain pointers and sizes only;
// every launcher enqueues on the given stream and returns the launch status.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace fb {

// ---- look-back family (k_scan.cu) ---------------------------------------------------
// `scratch` must hold lookback_scratch_bytes(n) bytes, zeroed once when allocated;
// `epoch` must differ from the epochs of earlier launches that used the same scratch
// (1 .. 2^29-1); `failure` is the context's device failure word.
size_t lookback_scratch_bytes(int64_t n);
// The scan starts from carry_in plus, when carry_vals is not NULL, the sum of the carry_n
// device values it points to.
cudaError_t launch_scan_i32(const int32_t *in, int32_t *out, int64_t n, int32_t carry_in,
                            const int32_t *carry_vals, int carry_n, void *scratch,
                            uint32_t epoch, int *failure, cudaStream_t stream, int grid_cap = 0);
// Exclusive scan: out[0] = 0, out[i] = in[0] + ... + in[i-1] (prelude/soacs.fut:212-215).
cudaError_t launch_exscan_i32(const int32_t *in, int32_t *out, int64_t n, void *scratch,
                              uint32_t epoch, int *failure, cudaStream_t stream);
// A bounded wait on a status word that is never published: records FAIL_LOOKBACK_TIMEOUT.
cudaError_t launch_expire_wait(void *scratch, uint32_t epoch, uint32_t max_polls, int *failure, cudaStream_t stream);
// Flagged segmented scan.  With shard_out != NULL the kernel also leaves the 4-word summary of
// the array seen as one shard of a longer one: {f32 bits, flag} of its last inclusive prefix, the
// index of its first 5120-element tile that holds a segment start (all ones if none), 0.
// With `peer` the scan kernel also writes {f32 bits, flag, seq} of the summary into the exchange buffers
// (peer-mapped, peer_exchange_bytes(world) each) of the ranks behind this one.
struct PeerPush {
  uint32_t *const *bufs;   // device array [world] of every rank's exchange buffer as this GPU addresses it
  int rank, world;
  uint32_t seq;            // sequence number of the call, the same on every rank, never 0
};
size_t peer_exchange_bytes(int world);
cudaError_t launch_segscan_f32(const uint8_t *flags, const float *in, float *out, int64_t n, float carry_in,
                               uint32_t *shard_out, void *scratch, uint32_t epoch, int *failure, cudaStream_t stream, int grid_cap = 0,
                               const PeerPush *peer = nullptr);
// The carry kernel fed by peer stores instead of a gathered array: it waits (bounded; FAIL_PEER_TIMEOUT) for
// the summaries of ranks 0..rank-1 of call `seq` in this rank's own exchange buffer; `own` is this shard's summary.
cudaError_t launch_segscan_apply_carry_peer(float *out, const uint8_t *flags, int64_t n, const uint32_t *my_buf, const uint32_t *own, int rank,
                                            int world, uint32_t seq, int *failure, int num_sms, cudaStream_t stream);
// Adds the fold of summaries[0..rank) (4 words per shard) to out[0 .. first segment start),
// the first start being located through summaries[rank].
cudaError_t launch_segscan_apply_carry(float *out, const uint8_t *flags, int64_t n, const uint32_t *summaries,
                                       int rank, int num_sms, cudaStream_t stream);
// Scans given by another specification of the same kernel (scan_specs.cuh): variant 0 exclusive
// (+), 1 inclusive i32.max, 2 the scanomap step of tests/soacs/scan4.fut seeded with seed_host + *seed.
cudaError_t launch_scan_variant_i32(int variant, const int32_t *in, int32_t *out, int64_t n, int32_t seed_host, const int32_t *seed,
                                    void *scratch, uint32_t epoch, int *failure, cudaStream_t stream);
// map (scan (+) 0) xss over [rows][cols] i32 (regular segments, head flags from the index).
cudaError_t launch_segscan_rows_i32(const int32_t *in, int32_t *out, int64_t rows, int64_t cols, void *scratch,
                                    uint32_t epoch, int *failure, cudaStream_t stream);
// Compaction of 4-byte keys.  `which` names the predicate and whether the rejected keys are
// kept (out_false); COMPACT_FILTER_BY_FLAG_I32 keeps in[i] where flags[i] != 0.  *d_count
// receives the number of selected keys.  The keys are worked off in pieces of 2^30; `epochs`
// holds one fresh epoch for each of the compact_pieces_needed(n) pieces.
enum CompactKind : int {
  COMPACT_FILTER_LOW3_U32 = 0, COMPACT_PARTITION_LOW3_U32 = 1, COMPACT_FILTER_POS_I32 = 2,
  COMPACT_PARTITION_EVEN_I32 = 3, COMPACT_PARTITION_DIV3_I32 = 4, COMPACT_FILTER_BY_FLAG_I32 = 5,
};
int compact_pieces_needed(int64_t n);
cudaError_t launch_compact(int which, const void *in, const uint8_t *flags, void *out_true, void *out_false,
                           int64_t n, int64_t *d_count, void *scratch, const uint32_t *epochs, int *failure, cudaStream_t stream);

// keep[c * pitch + i] = 1 if the pair (xs[i], ys[i]) is of class c (0: x < y, 1: x == y, 2: neither), else 0
cudaError_t launch_classify_pairs_lt_eq(const int32_t *xs, const int32_t *ys, int64_t n, int64_t pitch, uint8_t *keep, int num_sms,
                                        cudaStream_t stream);

// ---- two-pass scans for 8-byte and tuple operators (k_twopass.cu) ---------------------------
// `scratch`: the reduce scratch (at least twopass_scratch_bytes()).
size_t twopass_scratch_bytes();
cudaError_t launch_scan_i64(const int64_t *in, int64_t *out, int64_t n, void *scratch, int num_sms, cudaStream_t stream);
// out[i] = x_i of the recurrence x_i = as[i] * x_{i-1} + bs[i], x_{-1} = 0: the second component of the
// scan of the pairs (as[i], bs[i]) under composition of affine maps
cudaError_t launch_linrec_f32(const float *as, const float *bs, float *out, int64_t n, void *scratch, int num_sms, cudaStream_t stream);

// ---- reductions (k_reduce.cu) ---------------------------------------------------------
// `scratch` must hold reduce_scratch_bytes() bytes, zeroed once when allocated.
size_t reduce_scratch_bytes();
// grid_cap (> 0) bounds the number of CTAs; suff_outer_par: with at least that many rows one warp takes a
// row whatever its length (the outer parallelism suffices), with fewer a long row is shared by a CTA.
// grid_cap / block_cap: 0 = the launcher's own choice (the *_num_tblocks tuning parameters).
cudaError_t launch_reduce_i32(const int32_t *in, int64_t n, int32_t *d_out, void *scratch, int num_sms,
                              cudaStream_t stream, int block_cap = 0);
cudaError_t launch_rowsum_f32(const float *in, int64_t rows, int64_t cols, float *out, int num_sms,
                              cudaStream_t stream, int64_t suff_outer_par = 32768, int block_cap = 0);
// out[s] = sum of xs[offsets[s] .. offsets[s+1]) for s < nseg (offsets ascending, clamped to [0, n]); `scratch` as above.
cudaError_t launch_segreduce_f32(const int64_t *offsets, int64_t nseg, const float *xs, int64_t n, float *out,
                                 void *scratch, int *failure, int num_sms, cudaStream_t stream);

// sums[r] = sum of i64.f32 of row r (wrapping), neg[r][i] = f64.f32 (-in[r][i]): a segmented redomap with a map-out result
cudaError_t launch_rowsum_mapout(const float *in, int64_t rows, int64_t cols, int64_t *sums, double *neg, int num_sms, cudaStream_t stream);
// out[c] = sum over the rows of in[r][c] (wrapping): a reduction with an operator on whole rows
cudaError_t launch_colsum_i32(const int32_t *in, int64_t rows, int64_t cols, int32_t *out, int num_sms, cudaStream_t stream);

// ---- fused redomaps (k_redomap.cu; the kernel template is redomap.cuh) -----------------------
// `scratch` as for the reductions.  mss: d_out4 receives the operator's 4-tuple (best segment
// sum first).  sum_i32_f32: d_out2 receives {i32 sum, f32 sum of the converted elements}.
cudaError_t launch_mss_i32(const int32_t *in, int64_t n, int32_t *d_out4, void *scratch, int num_sms, cudaStream_t stream);
cudaError_t launch_sum_i32_f32(const int32_t *in, int64_t n, void *d_out2, void *scratch, int num_sms, cudaStream_t stream);
// map2 bodies: the f32 dot product, and the product of the element-wise sums of two i32 arrays
cudaError_t launch_dotprod_f32(const float *xs, const float *ys, int64_t n, float *d_out, void *scratch, int num_sms, cudaStream_t stream);
cudaError_t launch_prod_of_sums_i32(const int32_t *xs, const int32_t *ys, int64_t n, int32_t *d_out, void *scratch, int num_sms, cudaStream_t stream);
cudaError_t launch_dotprod_i32(const int32_t *xs, const int32_t *ys, int64_t n, int32_t *d_out, void *scratch, int num_sms, cudaStream_t stream);
cudaError_t launch_product_i32(const int32_t *xs, int64_t n, int32_t *d_out, void *scratch, int num_sms, cudaStream_t stream);
// d_out2: the pair (a, b) of the composed affine map
cudaError_t launch_affine_f32(const float *as, const float *bs, int64_t n, float *d_out2, void *scratch, int num_sms, cudaStream_t stream);

// ---- histograms (k_hist.cu) -------------------------------------------------------------
// out[b] = fold of the weights whose index is b, over 32-bit values; `out` holds B 4-byte bins.
// dest == NULL: the bins start at the operator's neutral element (hist); otherwise `out`
// starts as a copy of the B values at dest (reduce_by_index; not offered for HOP_MAX_F32).
enum HistOpKind : int {
  HOP_ADD_I32 = 0, HOP_MAX_F32 = 1, HOP_MIN_I32 = 2, HOP_MAX_I32 = 3, HOP_MIN_U32 = 4, HOP_MAX_U32 = 5,
  HOP_AND_I32 = 6, HOP_OR_I32 = 7, HOP_XOR_I32 = 8, HOP_ADD_F32 = 9, HOP_MUL_I32 = 10,
};
cudaError_t launch_hist(int op, int64_t B, const int32_t *bins, const void *weights, int64_t n, void *out,
                        const void *dest, int num_sms, cudaStream_t stream);
// flat[i * m + j] = is[i] * m + j, or -1 where is[i] is outside [0, n): a histogram whose bins are rows of m values
cudaError_t launch_flatten_vec_index(const int64_t *is, int64_t k, int64_t n, int64_t m, int32_t *flat, int num_sms, cudaStream_t stream);
// flat[(r * cols + i) * k + j] = (r * m + iss[r][i]) * k + j, or -1: one histogram of k-vectors per row
cudaError_t launch_flatten_rows_vec_index(const int32_t *iss, int64_t rows, int64_t cols, int64_t m, int64_t k, int32_t *flat, int num_sms,
                                          cudaStream_t stream);
// the minimum of the first components carrying the second along, neutral (-1, -1); `packed`: B 8-byte words
cudaError_t launch_hist_minpair_i32(int64_t B, const int32_t *bins, const int32_t *v0, const int32_t *v1, int64_t n, void *packed, int32_t *out0,
                                    int32_t *out1, int num_sms, cudaStream_t stream);
// 1- and 2-byte integers (elem_bytes) under an operator of NarrowOp, by compare-and-swap on the containing
// word; dest == NULL (and, or, xor only): the bins start at the operator's neutral element.  `out` must be
// readable and writable up to the next multiple of 4 bytes.
enum NarrowOp : int { NOP_MIN_S = 0, NOP_MAX_S = 1, NOP_MIN_U = 2, NOP_MAX_U = 3, NOP_AND = 4, NOP_OR = 5, NOP_XOR = 6 };
cudaError_t launch_hist_narrow(int op, int elem_bytes, int64_t B, const int32_t *bins, const void *vs, int64_t n, void *out, const void *dest,
                               int num_sms, cudaStream_t stream);
// and / or / xor over i64 bins of sign-extended i32 values, from the neutral element
cudaError_t launch_hist_bitop_i64(int op, int64_t B, const int32_t *bins, const int32_t *vs, int64_t n, int64_t *out, int num_sms,
                                  cudaStream_t stream);
// flat[i] = (is[i] * M + js[i]) * L + ks[i], or -1 out of range: reduce_by_index_3d
cudaError_t launch_flatten_3d_index(const int64_t *is, const int64_t *js, const int64_t *ks, int64_t n, int64_t K, int64_t M, int64_t L,
                                    int32_t *flat, int num_sms, cudaStream_t stream);
// flat[i] = ((i / cols) * N + xs[i]) * M + ys[i], or -1 out of range: a 2-D histogram per row
cudaError_t launch_flatten_rows_2d_index(const int32_t *xs, const int32_t *ys, int64_t n, int64_t cols, int64_t N, int64_t M, int32_t *flat,
                                         int num_sms, cudaStream_t stream);
// reduce_by_index dest (+) 0 is vs over f64: atomics on the result in global memory
cudaError_t launch_hist_add_f64(int64_t B, const int32_t *bins, const double *vs, int64_t n, double *out, const double *dest, int num_sms,
                                cudaStream_t stream);
// reduce_by_index dest (+) 0 is vs over 1- and 2-byte values (kind 0: i8 with i8 indices, 1: i16 with i16 indices,
// 2: f16 with i16 indices): a compare-and-swap loop on the containing 32-bit word
cudaError_t launch_hist_add_subword(int kind, int64_t B, const void *bins, const void *vs, int64_t n, void *out, const void *dest, int num_sms,
                                    cudaStream_t stream);
// flat[i] = (i / cols) * B + is[i], or -1 if is[i] is outside [0, B): a histogram per row
cudaError_t launch_flatten_rows_index(const int32_t *is, int64_t n, int64_t cols, int64_t B, int32_t *flat, int num_sms, cudaStream_t stream);
// flat[i] = is[i] * M + js[i], or -1 if either index is out of range: reduce_by_index_2d
cudaError_t launch_flatten_2d_index(const int64_t *is, const int64_t *js, int64_t n, int64_t N, int64_t M, int32_t *flat, int num_sms,
                                    cudaStream_t stream);

// ---- layout operations (k_layout.cu) ----------------------------------------------------------
// out[b][c][r] = in[b][r][c] for 4-byte elements.
cudaError_t launch_transpose_b32(const void *in, void *out, int64_t nb, int64_t rows, int64_t cols, int num_sms,
                                 cudaStream_t stream);
// The same for elements of 1, 2, 4 or 8 bytes.
cudaError_t launch_transpose(int elem_size, const void *in, void *out, int64_t nb, int64_t rows, int64_t cols, int num_sms,
                             cudaStream_t stream);
// dst[i] = value (elements of 1, 2, 4 or 8 bytes, given as bits); dst[i] = start + i * step in that integer width.
cudaError_t launch_replicate(int elem_size, void *dst, int64_t n, uint64_t value_bits, int num_sms, cudaStream_t stream);
cudaError_t launch_iota(int elem_size, void *dst, int64_t n, int64_t start, int64_t step, int num_sms, cudaStream_t stream);

// Strided copy between two device arrays given as LMADs (offset + one stride per dimension, in
// elements) over a common shape of rank <= LMAD_MAX_RANK; elem_size 1, 2, 4 or 8.  *kind_out
// (may be NULL) receives the route taken.  The two host-side steps are exported for tests:
// lmad_normalise returns the rank of the normal form, lmad_classify the route for it.
constexpr int LMAD_MAX_RANK = 8;
enum LmadKind : int { LMAD_NOTHING = -1, LMAD_GENERAL = 0, LMAD_TRANSPOSE = 1, LMAD_FLAT = 2 };
int lmad_normalise(int r, const int64_t *dst_strides, const int64_t *src_strides, const int64_t *shape,
                   int64_t *n_shape, int64_t *n_dst, int64_t *n_src);
int lmad_classify(int r, const int64_t *shape, const int64_t *dst, const int64_t *src, int64_t *nb, int64_t *rows,
                  int64_t *cols);
cudaError_t launch_lmad_copy(int elem_size, int r, void *dst, int64_t dst_offset, const int64_t *dst_strides,
                             const void *src, int64_t src_offset, const int64_t *src_strides, const int64_t *shape,
                             int num_sms, cudaStream_t stream, int *kind_out);

// ---- batched f16 contraction (k_bmm.cu) ------------------------------------------------
cudaError_t launch_bmm_f16(const uint16_t *A, const uint16_t *B, float *C, int64_t nb, int64_t m, int64_t k,
                           int64_t n, int *failure, cudaStream_t stream);

}  // namespace fb
