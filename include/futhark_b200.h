/* futhark_b200.h -- C API of the B200-native SegOp core.
 *
 * The symbols below are the ones `futhark cuda --library` generates for a program
 * with the entry points listed at the end of this file; each declaration
 * cites the place in the reference (diku-dk/futhark v0.28.0) that defines the
 * interface it replaces.  A host program written against the generated header of
 * that program links against libfuthark_b200.so unchanged.
 *
 * Conventions (docs/c-api.rst):
 *  - every function is asynchronous with respect to the device unless stated;
 *    results are valid after futhark_context_sync() returns 0      (:176-180, :580-596)
 *  - values are reference counted; every value returned by a `new`, an entry
 *    point or a projection must be freed exactly once               (:249-254, :598-601)
 *  - all public calls on one context are serialised by a lock
 *    (src/Futhark/CodeGen/Backends/GenericC/Monad.hs:707-714)
 *  - f16 data crosses the API as uint16_t binary16 bits             (:229-233)
 *  - bool is one byte, 0 or 1 (docs/binary-data-format.rst)
 *  - multi-dimensional arrays are row-major                         (:262-266)
 */
#ifndef FUTHARK_B200_H
#define FUTHARK_B200_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>
#include <stdio.h>

#ifdef FUTHARK_B200_NO_CUDA_H
typedef unsigned long long CUdeviceptr;   /* same underlying type as in <cuda.h> */
#else
#include <cuda.h>                          /* the generated header includes it too
                                              (src/Futhark/CodeGen/Backends/CCUDA.hs:134-138) */
#endif

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default)   /* the library is built with hidden visibility */
#endif

/* ---- error codes: rts/c/errors.h:1-3, docs/c-api.rst:37-58 ----------------- */
#define FUTHARK_SUCCESS 0
#define FUTHARK_PROGRAM_ERROR 2
#define FUTHARK_OUT_OF_MEMORY 3

/* ---- configuration: rts/c/context.h:95-163, docs/c-api.rst:60-145 ---------- */
struct futhark_context_config;
struct futhark_context_config *futhark_context_config_new(void);
void futhark_context_config_free(struct futhark_context_config *cfg);
void futhark_context_config_set_debugging(struct futhark_context_config *cfg, int flag);
void futhark_context_config_set_profiling(struct futhark_context_config *cfg, int flag);
void futhark_context_config_set_logging(struct futhark_context_config *cfg, int flag);
int futhark_context_config_set_tuning_param(struct futhark_context_config *cfg,
                                            const char *param_name, size_t new_value);
int futhark_get_tuning_param_count(void);
const char *futhark_get_tuning_param_name(int i);
const char *futhark_get_tuning_param_class(int i);
void futhark_context_config_set_cache_file(struct futhark_context_config *cfg, const char *f);

/* GPU configuration: rts/c/backends/cuda.h:134-179, rts/c/gpu.h:54-91,
 * src/Futhark/CodeGen/Backends/CCUDA.hs:46-51.  The kernels of this library are
 * compiled ahead of time for sm_100a, so the NVRTC / PTX / program-text setters
 * are accepted and ignored. */
void futhark_context_config_set_device(struct futhark_context_config *cfg, const char *s);
void futhark_context_config_set_unified_memory(struct futhark_context_config *cfg, int flag);
void futhark_context_config_set_default_thread_block_size(struct futhark_context_config *cfg, int size);
void futhark_context_config_set_default_group_size(struct futhark_context_config *cfg, int size);
void futhark_context_config_set_default_grid_size(struct futhark_context_config *cfg, int num);
void futhark_context_config_set_default_num_groups(struct futhark_context_config *cfg, int num);
void futhark_context_config_set_default_tile_size(struct futhark_context_config *cfg, int size);
void futhark_context_config_set_default_reg_tile_size(struct futhark_context_config *cfg, int size);
void futhark_context_config_set_default_registers(struct futhark_context_config *cfg, int size);
void futhark_context_config_set_default_cache(struct futhark_context_config *cfg, int size);
void futhark_context_config_set_default_threshold(struct futhark_context_config *cfg, int size);
const char *futhark_context_config_get_program(struct futhark_context_config *cfg);
void futhark_context_config_set_program(struct futhark_context_config *cfg, const char *s);
void futhark_context_config_add_nvrtc_option(struct futhark_context_config *cfg, const char *opt);
void futhark_context_config_dump_ptx_to(struct futhark_context_config *cfg, const char *s);
void futhark_context_config_load_ptx_from(struct futhark_context_config *cfg, const char *s);

/* ---- context: rts/c/context.h:89-211, rts/c/backends/cuda.h:719-861,
 *      src/Futhark/CodeGen/Backends/GenericC.hs:603-640 ---------------------- */
struct futhark_context;
struct futhark_context *futhark_context_new(struct futhark_context_config *cfg);
void futhark_context_free(struct futhark_context *ctx);
int futhark_context_sync(struct futhark_context *ctx);
char *futhark_context_get_error(struct futhark_context *ctx);   /* caller frees; clears */
void futhark_context_set_logging_file(struct futhark_context *ctx, FILE *f);
void futhark_context_pause_profiling(struct futhark_context *ctx);
void futhark_context_unpause_profiling(struct futhark_context *ctx);
char *futhark_context_report(struct futhark_context *ctx);      /* caller frees; JSON */
int futhark_context_clear_caches(struct futhark_context *ctx);

/* ---- arrays: src/Futhark/CodeGen/Backends/GenericC/Types.hs:61-250,
 *      docs/c-api.rst:256-315; raw pointers are CUdeviceptr (CCUDA.hs:105-107) - */
#define FUTHARK_B200_ARRAY_COMMON(NAME, CT)                                                    \
  struct futhark_##NAME;                                                                       \
  int futhark_free_##NAME(struct futhark_context *ctx, struct futhark_##NAME *arr);            \
  int futhark_values_##NAME(struct futhark_context *ctx, struct futhark_##NAME *arr, CT *data);\
  CUdeviceptr futhark_values_raw_##NAME(struct futhark_context *ctx, struct futhark_##NAME *arr);\
  const int64_t *futhark_shape_##NAME(struct futhark_context *ctx, struct futhark_##NAME *arr);

#define FUTHARK_B200_ARRAY_1D(NAME, CT)                                                        \
  FUTHARK_B200_ARRAY_COMMON(NAME, CT)                                                          \
  struct futhark_##NAME *futhark_new_##NAME(struct futhark_context *ctx, const CT *data,       \
                                            int64_t dim0);                                     \
  struct futhark_##NAME *futhark_new_raw_##NAME(struct futhark_context *ctx, CUdeviceptr data, \
                                                int64_t dim0);                                 \
  int futhark_index_##NAME(struct futhark_context *ctx, CT *out, struct futhark_##NAME *arr,   \
                           int64_t i0);

#define FUTHARK_B200_ARRAY_2D(NAME, CT)                                                        \
  FUTHARK_B200_ARRAY_COMMON(NAME, CT)                                                          \
  struct futhark_##NAME *futhark_new_##NAME(struct futhark_context *ctx, const CT *data,       \
                                            int64_t dim0, int64_t dim1);                       \
  struct futhark_##NAME *futhark_new_raw_##NAME(struct futhark_context *ctx, CUdeviceptr data, \
                                                int64_t dim0, int64_t dim1);                   \
  int futhark_index_##NAME(struct futhark_context *ctx, CT *out, struct futhark_##NAME *arr,   \
                           int64_t i0, int64_t i1);

#define FUTHARK_B200_ARRAY_3D(NAME, CT)                                                        \
  FUTHARK_B200_ARRAY_COMMON(NAME, CT)                                                          \
  struct futhark_##NAME *futhark_new_##NAME(struct futhark_context *ctx, const CT *data,       \
                                            int64_t dim0, int64_t dim1, int64_t dim2);         \
  struct futhark_##NAME *futhark_new_raw_##NAME(struct futhark_context *ctx, CUdeviceptr data, \
                                                int64_t dim0, int64_t dim1, int64_t dim2);     \
  int futhark_index_##NAME(struct futhark_context *ctx, CT *out, struct futhark_##NAME *arr,   \
                           int64_t i0, int64_t i1, int64_t i2);

FUTHARK_B200_ARRAY_1D(i32_1d, int32_t)
FUTHARK_B200_ARRAY_1D(i64_1d, int64_t)
FUTHARK_B200_ARRAY_1D(u32_1d, uint32_t)
FUTHARK_B200_ARRAY_1D(f32_1d, float)
FUTHARK_B200_ARRAY_1D(bool_1d, bool)
FUTHARK_B200_ARRAY_2D(f32_2d, float)
FUTHARK_B200_ARRAY_2D(i32_2d, int32_t)
FUTHARK_B200_ARRAY_2D(bool_2d, bool)
FUTHARK_B200_ARRAY_2D(i64_2d, int64_t)
FUTHARK_B200_ARRAY_2D(f64_2d, double)
FUTHARK_B200_ARRAY_1D(f64_1d, double)
FUTHARK_B200_ARRAY_1D(i8_1d, int8_t)
FUTHARK_B200_ARRAY_1D(i16_1d, int16_t)
FUTHARK_B200_ARRAY_1D(f16_1d, uint16_t)   /* binary16 bit patterns, as for f16_3d */
FUTHARK_B200_ARRAY_1D(u8_1d, uint8_t)
FUTHARK_B200_ARRAY_1D(u16_1d, uint16_t)
FUTHARK_B200_ARRAY_3D(f32_3d, float)
FUTHARK_B200_ARRAY_3D(i32_3d, int32_t)
FUTHARK_B200_ARRAY_3D(f16_3d, uint16_t)

/* ---- opaque tuple returned by partition: naming per
 *      src/Futhark/CodeGen/Backends/SimpleRep.hs:152-158; functions per
 *      docs/c-api.rst:317-438 (free, store, restore, new, project) ------------ */
struct futhark_opaque_tup2_arr1d_u32_arr1d_u32;
int futhark_free_opaque_tup2_arr1d_u32_arr1d_u32(struct futhark_context *ctx,
                                                 struct futhark_opaque_tup2_arr1d_u32_arr1d_u32 *obj);
int futhark_store_opaque_tup2_arr1d_u32_arr1d_u32(struct futhark_context *ctx,
                                                  const struct futhark_opaque_tup2_arr1d_u32_arr1d_u32 *obj,
                                                  void **p, size_t *n);
struct futhark_opaque_tup2_arr1d_u32_arr1d_u32 *
futhark_restore_opaque_tup2_arr1d_u32_arr1d_u32(struct futhark_context *ctx, const void *p);
int futhark_new_opaque_tup2_arr1d_u32_arr1d_u32(struct futhark_context *ctx,
                                                struct futhark_opaque_tup2_arr1d_u32_arr1d_u32 **out,
                                                const struct futhark_u32_1d *v0,
                                                const struct futhark_u32_1d *v1);
int futhark_project_opaque_tup2_arr1d_u32_arr1d_u32_0(struct futhark_context *ctx,
                                                      struct futhark_u32_1d **out,
                                                      const struct futhark_opaque_tup2_arr1d_u32_arr1d_u32 *obj);
int futhark_project_opaque_tup2_arr1d_u32_arr1d_u32_1(struct futhark_context *ctx,
                                                      struct futhark_u32_1d **out,
                                                      const struct futhark_opaque_tup2_arr1d_u32_arr1d_u32 *obj);

/* ---- opaque triple of i32 arrays returned by partition2_i32 (same naming rule); `free`
 *      releases the three arrays, `new` and the projections share them (docs/c-api.rst:366-391) ---------- */
struct futhark_opaque_tup3_arr1d_i32_arr1d_i32_arr1d_i32;
int futhark_free_opaque_tup3_arr1d_i32_arr1d_i32_arr1d_i32(struct futhark_context *ctx,
                                                           struct futhark_opaque_tup3_arr1d_i32_arr1d_i32_arr1d_i32 *obj);
int futhark_new_opaque_tup3_arr1d_i32_arr1d_i32_arr1d_i32(struct futhark_context *ctx,
                                                          struct futhark_opaque_tup3_arr1d_i32_arr1d_i32_arr1d_i32 **out,
                                                          const struct futhark_i32_1d *v0, const struct futhark_i32_1d *v1,
                                                          const struct futhark_i32_1d *v2);
int futhark_project_opaque_tup3_arr1d_i32_arr1d_i32_arr1d_i32_0(struct futhark_context *ctx, struct futhark_i32_1d **out,
                                                                const struct futhark_opaque_tup3_arr1d_i32_arr1d_i32_arr1d_i32 *obj);
int futhark_project_opaque_tup3_arr1d_i32_arr1d_i32_arr1d_i32_1(struct futhark_context *ctx, struct futhark_i32_1d **out,
                                                                const struct futhark_opaque_tup3_arr1d_i32_arr1d_i32_arr1d_i32 *obj);
int futhark_project_opaque_tup3_arr1d_i32_arr1d_i32_arr1d_i32_2(struct futhark_context *ctx, struct futhark_i32_1d **out,
                                                                const struct futhark_opaque_tup3_arr1d_i32_arr1d_i32_arr1d_i32 *obj);

/* ---- opaque pair ([]i64, [][]f64) returned by segredomap_sum_neg_f32 (same naming rule and functions) ---------- */
struct futhark_opaque_tup2_arr1d_i64_arr2d_f64;
int futhark_free_opaque_tup2_arr1d_i64_arr2d_f64(struct futhark_context *ctx,
                                                 struct futhark_opaque_tup2_arr1d_i64_arr2d_f64 *obj);
int futhark_new_opaque_tup2_arr1d_i64_arr2d_f64(struct futhark_context *ctx,
                                                struct futhark_opaque_tup2_arr1d_i64_arr2d_f64 **out,
                                                const struct futhark_i64_1d *v0, const struct futhark_f64_2d *v1);
int futhark_project_opaque_tup2_arr1d_i64_arr2d_f64_0(struct futhark_context *ctx, struct futhark_i64_1d **out,
                                                      const struct futhark_opaque_tup2_arr1d_i64_arr2d_f64 *obj);
int futhark_project_opaque_tup2_arr1d_i64_arr2d_f64_1(struct futhark_context *ctx, struct futhark_f64_2d **out,
                                                      const struct futhark_opaque_tup2_arr1d_i64_arr2d_f64 *obj);

/* ---- opaque pair of i32 arrays returned by reduce_by_index_minpair_i32 (same naming rule and functions) ---------- */
struct futhark_opaque_tup2_arr1d_i32_arr1d_i32;
int futhark_free_opaque_tup2_arr1d_i32_arr1d_i32(struct futhark_context *ctx,
                                                 struct futhark_opaque_tup2_arr1d_i32_arr1d_i32 *obj);
int futhark_new_opaque_tup2_arr1d_i32_arr1d_i32(struct futhark_context *ctx,
                                                struct futhark_opaque_tup2_arr1d_i32_arr1d_i32 **out,
                                                const struct futhark_i32_1d *v0, const struct futhark_i32_1d *v1);
int futhark_project_opaque_tup2_arr1d_i32_arr1d_i32_0(struct futhark_context *ctx, struct futhark_i32_1d **out,
                                                      const struct futhark_opaque_tup2_arr1d_i32_arr1d_i32 *obj);
int futhark_project_opaque_tup2_arr1d_i32_arr1d_i32_1(struct futhark_context *ctx, struct futhark_i32_1d **out,
                                                      const struct futhark_opaque_tup2_arr1d_i32_arr1d_i32 *obj);

/* ---- opaque 6-tuple of i32 arrays returned by partition2_pairs_i32 (same naming rule, the name
 *      findPrettyName of src/Futhark/CodeGen/Backends/SimpleRep.hs:145-175 gives the type
 *      ([]i32, []i32, []i32, []i32, []i32, []i32)); same functions as the triple ---------- */
struct futhark_opaque_tup6_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32;
int futhark_free_opaque_tup6_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32(
    struct futhark_context *ctx, struct futhark_opaque_tup6_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32 *obj);
int futhark_new_opaque_tup6_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32(
    struct futhark_context *ctx, struct futhark_opaque_tup6_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32 **out,
    const struct futhark_i32_1d *v0, const struct futhark_i32_1d *v1, const struct futhark_i32_1d *v2,
    const struct futhark_i32_1d *v3, const struct futhark_i32_1d *v4, const struct futhark_i32_1d *v5);
int futhark_project_opaque_tup6_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_0(
    struct futhark_context *ctx, struct futhark_i32_1d **out, const struct futhark_opaque_tup6_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32 *obj);
int futhark_project_opaque_tup6_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_1(
    struct futhark_context *ctx, struct futhark_i32_1d **out, const struct futhark_opaque_tup6_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32 *obj);
int futhark_project_opaque_tup6_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_2(
    struct futhark_context *ctx, struct futhark_i32_1d **out, const struct futhark_opaque_tup6_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32 *obj);
int futhark_project_opaque_tup6_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_3(
    struct futhark_context *ctx, struct futhark_i32_1d **out, const struct futhark_opaque_tup6_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32 *obj);
int futhark_project_opaque_tup6_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_4(
    struct futhark_context *ctx, struct futhark_i32_1d **out, const struct futhark_opaque_tup6_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32 *obj);
int futhark_project_opaque_tup6_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_5(
    struct futhark_context *ctx, struct futhark_i32_1d **out, const struct futhark_opaque_tup6_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32 *obj);

/* ---- opaque tuple (i32, f32) returned by sum_i32_f32: same naming and functions; its
 *      fields are scalars, so `new` takes and the projections return them by value ---------- */
struct futhark_opaque_tup2_i32_f32;
int futhark_free_opaque_tup2_i32_f32(struct futhark_context *ctx, struct futhark_opaque_tup2_i32_f32 *obj);
int futhark_store_opaque_tup2_i32_f32(struct futhark_context *ctx, const struct futhark_opaque_tup2_i32_f32 *obj,
                                      void **p, size_t *n);
struct futhark_opaque_tup2_i32_f32 *futhark_restore_opaque_tup2_i32_f32(struct futhark_context *ctx, const void *p);
int futhark_new_opaque_tup2_i32_f32(struct futhark_context *ctx, struct futhark_opaque_tup2_i32_f32 **out,
                                    const int32_t v0, const float v1);
int futhark_project_opaque_tup2_i32_f32_0(struct futhark_context *ctx, int32_t *out,
                                          const struct futhark_opaque_tup2_i32_f32 *obj);
int futhark_project_opaque_tup2_i32_f32_1(struct futhark_context *ctx, float *out,
                                          const struct futhark_opaque_tup2_i32_f32 *obj);

/* ---- entry points: src/Futhark/CodeGen/Backends/GenericC/EntryPoints.hs:133-223.
 * One out-parameter each (a tuple result is one opaque value); array results are allocated by the callee and owned by
 * the caller; on error the out-parameter is untouched.  The Futhark source of each
 * entry is given; the kernels that implement them replace what
 * src/Futhark/CodeGen/ImpGen/GPU/{SegRed,SegScan/SinglePass,SegHist,SegMap}.hs
 * would have generated. */

/* entry scan_i32 (xs: []i32): []i32 = scan (+) 0 xs
 * replaces the segscan kernel of ImpGen/GPU/SegScan/SinglePass.hs:327-879 */
int futhark_entry_scan_i32(struct futhark_context *ctx, struct futhark_i32_1d **out0,
                           const struct futhark_i32_1d *in0);

/* entry reduce_i32 (xs: []i32): i32 = reduce (+) 0 xs
 * replaces segred_nonseg, ImpGen/GPU/SegRed.hs:327-394.  The scalar result is read
 * back, so this call synchronises (Backends/GPU.hs:269-281). */
int futhark_entry_reduce_i32(struct futhark_context *ctx, int32_t *out0,
                             const struct futhark_i32_1d *in0);

/* entry segscan_f32 (flags: []bool) (xs: []f32): []f32
 *   = (unzip (scan (\(f1,x) (f2,y) -> (f1||f2, if f2 then y else x+y)) (false,0) (zip flags xs))).1
 * (the idiom of tests/soacs/scan2.fut:7-17); replaces the pair scan through
 * SinglePass.hs:327-879. */
int futhark_entry_segscan_f32(struct futhark_context *ctx, struct futhark_f32_1d **out0,
                              const struct futhark_bool_1d *in0, const struct futhark_f32_1d *in1);

/* entry segreduce_f32 (offsets: []i64) (flags: []bool) (xs: []f32): []f32
 * Segment s covers xs[offsets[s] .. offsets[s+1]); result length = length offsets - 1;
 * an empty segment gives 0.  Replaces the flagged scan + gather of
 * src/Futhark/Pass/Flatten/Builtins.hs:582-602. */
int futhark_entry_segreduce_f32(struct futhark_context *ctx, struct futhark_f32_1d **out0,
                                const struct futhark_i64_1d *in0, const struct futhark_bool_1d *in1,
                                const struct futhark_f32_1d *in2);

/* entry rowsum_f32 (xss: [][]f32): []f32 = map (reduce (+) 0) xss
 * (tests/segredomap/segsum-comm.fut:9-10); replaces segred_small / segred_large,
 * ImpGen/GPU/SegRed.hs:396-636. */
int futhark_entry_rowsum_f32(struct futhark_context *ctx, struct futhark_f32_1d **out0,
                             const struct futhark_f32_2d *in0);

/* entry segredomap_sum_neg_f32 [m][n] (xss: [m][n]f32): ([m]i64, [m][n]f64) =
 *   unzip (map (\xs -> (reduce_comm (+) 0 (map i64.f32 xs), map (\x -> f64.f32 (-x)) xs)) xss)
 * (main of tests/segredomap/ex1-comm.fut:11-15: a segmented redomap whose body also returns a mapped array; the
 * threads write that map-out result while they read, src/Futhark/CodeGen/ImpGen/GPU/SegRed.hs:138-143). */
int futhark_entry_segredomap_sum_neg_f32(struct futhark_context *ctx,
                                         struct futhark_opaque_tup2_arr1d_i64_arr2d_f64 **out0,
                                         const struct futhark_f32_2d *in0);

/* entry reduce_map2_add_i32 [n][m] (xss: [n][m]i32): [m]i32 = reduce_comm (map2 (+)) (replicate m 0) xss
 * (tests/soacs/reduce4.fut, reduce5.fut: a reduction whose operator works on whole rows; it is interchanged
 * with the inner map, src/Futhark/Transform/ISRWIM.hs, and every column is reduced on its own). */
int futhark_entry_reduce_map2_add_i32(struct futhark_context *ctx, struct futhark_i32_1d **out0,
                                      const struct futhark_i32_2d *in0);

/* entry hist_add_i32 (B: i64) (is: []i32) (ws: []i32): [B]i32
 *   = hist (+) 0 B (map i64.i32 is) ws            (prelude/soacs.fut:132-133)
 * entry hist_max_f32 (B: i64) (is: []i32) (ws: []f32): [B]f32
 *   = hist f32.max f32.lowest B (map i64.i32 is) ws
 * Indices outside [0,B) are ignored.  Replace seghist_local / seghist_global,
 * ImpGen/GPU/SegHist.hs:377-1188. */
int futhark_entry_hist_add_i32(struct futhark_context *ctx, struct futhark_i32_1d **out0,
                               const int64_t in0, const struct futhark_i32_1d *in1,
                               const struct futhark_i32_1d *in2);
int futhark_entry_hist_max_f32(struct futhark_context *ctx, struct futhark_f32_1d **out0,
                               const int64_t in0, const struct futhark_i32_1d *in1,
                               const struct futhark_f32_1d *in2);

/* The histogram kernels under other operators and index spaces.  The reference chooses per
 * operator between a native atomic, a compare-and-swap loop and a lock
 * (src/Futhark/CodeGen/ImpGen/GPU/Base.hs:720-905, table ImpGen/GPU.hs:46-90); here the operator is
 * a template parameter of the same three kernels.  Indices are i32, widened to i64 as in
 * `map i64.i32 is`; out-of-range indices are ignored.
 *
 * entry hist_and_i32 (n: i64) (is: []i32) (vs: []i32): [n]i32 = hist (i32.&) (-1) n (map i64.i32 is) vs   (tests/hist/and.fut)
 * entry hist_or_i32  ... = hist (i32.|) 0 n ...                                                  (tests/hist/or.fut)
 * entry hist_xor_i32 ... = hist (i32.^) 0 n ...                                                  (tests/hist/xor.fut)
 * entry hist_mul_i32 ... = hist (i32.*) 1 n ...      (no native atomic: a compare-and-swap loop, Base.hs:844-905)
 * entry reduce_by_index_min_i32 (dest: *[n]i32) (is: []i32) (vs: []i32): [n]i32 =
 *   reduce_by_index dest i32.min i32.highest (map i64.i32 is) vs        (tests/hist/min.fut, first result)
 * entry reduce_by_index_min_u32 ... u32.min u32.highest ...            (tests/hist/min.fut, second result)
 * entry reduce_by_index_max_i32, reduce_by_index_max_u32 ... max / lowest (tests/hist/max.fut)
 * entry reduce_by_index_add_f32 (dest: *[n]f32) (is: []i32) (vs: []f32): [n]f32 =
 *   reduce_by_index dest (+) 0f32 (map i64.i32 is) vs                   (tests/hist/f32.fut; NaN propagates)
 * entry reduce_by_index_add_f64 (dest: *[n]f64) (is: []i32) (vs: []f64): [n]f64 =
 *   reduce_by_index dest (+) 0f64 (map i64.i32 is) vs                   (tests/hist/f64.fut; 8-byte values go
 *   the route of atomics on the result in global memory, SegHist.hs:377-560)
 * entry reduce_by_index_add_i8 (dest: *[n]i8) (is: []i8) (vs: []i8): [n]i8 =
 *   reduce_by_index dest (+) 0i8 (map i64.i8 is) vs                     (tests/hist/i8.fut)
 * entry reduce_by_index_add_i16 (dest: *[n]i16) (is: []i16) (vs: []i16): [n]i16   (tests/hist/i16.fut)
 * entry reduce_by_index_add_f16 (dest: *[n]f16) (is: []i16) (vs: []f16): [n]f16   (tests/hist/f16.fut)
 *   1- and 2-byte values have no atomic of their own: a compare-and-swap loop on the 32-bit word that
 *   holds the element (Base.hs:844-905).  f16 values are added as f32 and narrowed by truncation, as
 *   the reference's C code does it (rts/c/scalar_f16.h:16-46, rts/c/half.h:220-228).
 * entry hist_{and,or,xor}_{i8,i16} (n: i64) (is: []i32) (vs: []t): [n]t = hist (t.&) (-1) n (map i64.i32 is) vs, ...
 *   (tests/hist/and8.fut, and16.fut, or8.fut, or16.fut, xor8.fut, xor16.fut)
 * entry hist_or_bool (n: i64) (is: []i32) (vs: []bool): [n]bool = hist (||) false n (map i64.i32 is) vs   (tests/hist/lor.fut)
 * entry reduce_by_index_{min,max}_{i8,u8,i16,u16} (dest: *[n]t) (is: []i32) (vs: []t): [n]t =
 *   reduce_by_index dest t.min t.highest (map i64.i32 is) vs, ...      (the two results of tests/hist/min8.fut,
 *   min16.fut, max8.fut, max16.fut; the same compare-and-swap loop, signed operators on the sign-extended sub-word)
 * entry reduce_by_index_vec_add_i32 [n][m][k] (xs: *[n][m]i32) (is: [k]i64) (vss: [k][m]i32): [n][m]i32 =
 *   reduce_by_index xs (map2 (+)) (replicate m 0) is vss               (tests/hist/array.fut, array_novec.fut: the
 *   bins are rows, HistOp's operator shape, src/Futhark/IR/SegOp.hs:102-115; one histogram over n * m bins)
 * entry hist_rows_vec_add_i32 [r][c][k] (m: i64) (iss: [r][c]i32) (vsss: [r][c][k]i32): [r][m][k]i32 =
 *   map2 (\is vss -> hist (map2 (+)) (replicate k 0) m (map i64.i32 is) vss) iss vsss   (tests/hist/segmented_arr.fut:
 *   a segment dimension over a histogram whose bins are vectors)
 * entry reduce_by_index_minpair_i32 (m: i64) (is: []i32) (vs0: []i32) (vs1: []i32): ([m]i32, [m]i32) =
 *   main of tests/hist/tuple_partial.fut:24-28: an operator on pairs (the smaller first component wins and
 *   carries its second along; neutral (-1, -1)).  The reference locks the bin (Base.hs:769-842); here the
 *   pair is one 64-bit word updated by compare-and-swap.
 * entry hist_{and,or,xor}_i64 (n: i64) (is: []i32) (vs: []i32): [n]i64 =
 *   hist (i64.&) (-1) n (map i64.i32 is) (map i64.i32 vs), ...         (tests/hist/and64.fut, xor64.fut: native
 *   64-bit atomics on the result, the widening of the values fused into the kernel)
 * entry hist_rows_add_i32 (m: i64) (iss: [][]i32) (vss: [][]i32): [][m]i32 =
 *   map2 (\is vs -> hist (+) 0 m (map i64.i32 is) vs) iss vss           (tests/hist/segmented.fut: the segment
 *   dimension of a SegHist, SegHist.hs:97-148)
 * entry reduce_by_index_2d_add_i32 (dest: *[n][m]i32) (is: []i64) (js: []i64) (vs: []i32): [n][m]i32 =
 *   reduce_by_index_2d dest (+) 0 (zip is js) vs                        (prelude/soacs.fut:149-152; tests/hist/hist2d.fut)
 * entry reduce_by_index_3d_add_i32 (dest: *[k][m][l]i32) (is: []i64) (js: []i64) (ks: []i64) (vs: []i32): [k][m][l]i32 =
 *   reduce_by_index_3d dest (+) 0 (zip3 is js ks) vs                    (prelude/soacs.fut:153-154; tests/hist/hist3d.fut)
 * entry hist_rows_2d_add_i32 (n: i64) (m: i64) (xss: [][]i32) (yss: [][]i32): [][n][m]i32 =
 *   map2 (\xs ys -> reduce_by_index_2d (replicate n (replicate m 0)) (+) 0 (zip (map i64.i32 xs) (map i64.i32 ys))
 *                                      (map (const 1) xs)) xss yss      (tests/hist/segmented_2d.fut: a segment
 *   dimension over a 2-D histogram) */
#define FUTHARK_B200_HIST_ENTRY(NAME, ARR)                                                          \
  int futhark_entry_hist_##NAME(struct futhark_context *ctx, struct futhark_##ARR **out0,           \
                                const int64_t in0, const struct futhark_i32_1d *in1,               \
                                const struct futhark_##ARR *in2);
FUTHARK_B200_HIST_ENTRY(and_i32, i32_1d)
FUTHARK_B200_HIST_ENTRY(or_i32, i32_1d)
FUTHARK_B200_HIST_ENTRY(xor_i32, i32_1d)
FUTHARK_B200_HIST_ENTRY(mul_i32, i32_1d)
#define FUTHARK_B200_RBI_ENTRY(NAME, ARR)                                                           \
  int futhark_entry_reduce_by_index_##NAME(struct futhark_context *ctx, struct futhark_##ARR **out0,\
                                           const struct futhark_##ARR *in0,                        \
                                           const struct futhark_i32_1d *in1,                       \
                                           const struct futhark_##ARR *in2);
FUTHARK_B200_RBI_ENTRY(min_i32, i32_1d)
FUTHARK_B200_RBI_ENTRY(max_i32, i32_1d)
FUTHARK_B200_RBI_ENTRY(min_u32, u32_1d)
FUTHARK_B200_RBI_ENTRY(max_u32, u32_1d)
FUTHARK_B200_RBI_ENTRY(add_f32, f32_1d)
FUTHARK_B200_RBI_ENTRY(add_f64, f64_1d)
int futhark_entry_reduce_by_index_add_i8(struct futhark_context *ctx, struct futhark_i8_1d **out0,
                                         const struct futhark_i8_1d *in0, const struct futhark_i8_1d *in1,
                                         const struct futhark_i8_1d *in2);
int futhark_entry_reduce_by_index_add_i16(struct futhark_context *ctx, struct futhark_i16_1d **out0,
                                          const struct futhark_i16_1d *in0, const struct futhark_i16_1d *in1,
                                          const struct futhark_i16_1d *in2);
int futhark_entry_reduce_by_index_add_f16(struct futhark_context *ctx, struct futhark_f16_1d **out0,
                                          const struct futhark_f16_1d *in0, const struct futhark_i16_1d *in1,
                                          const struct futhark_f16_1d *in2);
FUTHARK_B200_HIST_ENTRY(and_i8, i8_1d)
FUTHARK_B200_HIST_ENTRY(or_i8, i8_1d)
FUTHARK_B200_HIST_ENTRY(xor_i8, i8_1d)
FUTHARK_B200_HIST_ENTRY(and_i16, i16_1d)
FUTHARK_B200_HIST_ENTRY(or_i16, i16_1d)
FUTHARK_B200_HIST_ENTRY(xor_i16, i16_1d)
FUTHARK_B200_HIST_ENTRY(or_bool, bool_1d)
FUTHARK_B200_RBI_ENTRY(min_i8, i8_1d)
FUTHARK_B200_RBI_ENTRY(max_i8, i8_1d)
FUTHARK_B200_RBI_ENTRY(min_u8, u8_1d)
FUTHARK_B200_RBI_ENTRY(max_u8, u8_1d)
FUTHARK_B200_RBI_ENTRY(min_i16, i16_1d)
FUTHARK_B200_RBI_ENTRY(max_i16, i16_1d)
FUTHARK_B200_RBI_ENTRY(min_u16, u16_1d)
FUTHARK_B200_RBI_ENTRY(max_u16, u16_1d)
#define FUTHARK_B200_HIST_I64_ENTRY(NAME)                                                           \
  int futhark_entry_hist_##NAME(struct futhark_context *ctx, struct futhark_i64_1d **out0,          \
                                const int64_t in0, const struct futhark_i32_1d *in1,               \
                                const struct futhark_i32_1d *in2);
FUTHARK_B200_HIST_I64_ENTRY(and_i64)
FUTHARK_B200_HIST_I64_ENTRY(or_i64)
FUTHARK_B200_HIST_I64_ENTRY(xor_i64)
int futhark_entry_reduce_by_index_vec_add_i32(struct futhark_context *ctx, struct futhark_i32_2d **out0,
                                              const struct futhark_i32_2d *in0, const struct futhark_i64_1d *in1,
                                              const struct futhark_i32_2d *in2);
int futhark_entry_hist_rows_vec_add_i32(struct futhark_context *ctx, struct futhark_i32_3d **out0,
                                        const int64_t in0, const struct futhark_i32_2d *in1,
                                        const struct futhark_i32_3d *in2);
int futhark_entry_reduce_by_index_minpair_i32(struct futhark_context *ctx,
                                              struct futhark_opaque_tup2_arr1d_i32_arr1d_i32 **out0,
                                              const int64_t in0, const struct futhark_i32_1d *in1,
                                              const struct futhark_i32_1d *in2, const struct futhark_i32_1d *in3);
int futhark_entry_hist_rows_add_i32(struct futhark_context *ctx, struct futhark_i32_2d **out0,
                                    const int64_t in0, const struct futhark_i32_2d *in1,
                                    const struct futhark_i32_2d *in2);
int futhark_entry_reduce_by_index_2d_add_i32(struct futhark_context *ctx, struct futhark_i32_2d **out0,
                                             const struct futhark_i32_2d *in0,
                                             const struct futhark_i64_1d *in1,
                                             const struct futhark_i64_1d *in2,
                                             const struct futhark_i32_1d *in3);
int futhark_entry_reduce_by_index_3d_add_i32(struct futhark_context *ctx, struct futhark_i32_3d **out0,
                                             const struct futhark_i32_3d *in0,
                                             const struct futhark_i64_1d *in1,
                                             const struct futhark_i64_1d *in2,
                                             const struct futhark_i64_1d *in3,
                                             const struct futhark_i32_1d *in4);
int futhark_entry_hist_rows_2d_add_i32(struct futhark_context *ctx, struct futhark_i32_3d **out0,
                                       const int64_t in0, const int64_t in1,
                                       const struct futhark_i32_2d *in2, const struct futhark_i32_2d *in3);

/* entry filter_u32 (ks: []u32): []u32 = filter (\k -> (k & 7) < 3) ks
 * entry partition_u32 (ks: []u32): ([]u32, []u32) = partition (\k -> (k & 7) < 3) ks
 * (prelude/soacs.fut:241-286: stable; the split count is shape[0] of field 0).
 * Both read the result size back, so they synchronise.  Counts are 64-bit as in the
 * reference: more than 2^31 keys are worked off in pieces of 2^30 inside one call. */
int futhark_entry_filter_u32(struct futhark_context *ctx, struct futhark_u32_1d **out0,
                             const struct futhark_u32_1d *in0);
int futhark_entry_partition_u32(struct futhark_context *ctx,
                                struct futhark_opaque_tup2_arr1d_u32_arr1d_u32 **out0,
                                const struct futhark_u32_1d *in0);

/* entry bmm_f16 (A: [b][m][k]f16) (B: [b][k][n]f16): [b][m][n]f32
 *   = map2 (\a b -> map (\ar -> map (\bc -> f32.sum (map2 (\x y -> f32.f16 x * f32.f16 y) ar bc))
 *                                   (transpose b)) a) A B
 * (shape of tests/reg-tiling/mmm.fut:17-21); replaces the block/register-tiled
 * segmap_intrablock of src/Futhark/Optimise/BlkRegTiling.hs:68-140. */
int futhark_entry_bmm_f16(struct futhark_context *ctx, struct futhark_f32_3d **out0,
                          const struct futhark_f16_3d *in0, const struct futhark_f16_3d *in1);

/* entry transpose_f32 (xss: [][]f32): [][]f32 = transpose xss
 * entry transpose_f32_3d (xsss: [][][]f32): [][][]f32 = map transpose xsss
 * A manifest transposition: the reference's compiler turns it into a call of the runtime's
 * map_transpose_4b kernels (rts/opencl/transpose.cl:3-275, launched through
 * rts/c/gpu.h gpu_map_transpose_4b), which it also inserts around SegOps (row-major
 * coalescing, the transposed operand of a matrix product). */
int futhark_entry_transpose_f32(struct futhark_context *ctx, struct futhark_f32_2d **out0,
                                const struct futhark_f32_2d *in0);
int futhark_entry_transpose_f32_3d(struct futhark_context *ctx, struct futhark_f32_3d **out0,
                                   const struct futhark_f32_3d *in0);
/* The other element widths of the reference's transposition kernels (rts/opencl/transpose.cl:3-277,
 * instantiated for 1, 2, 4 and 8 bytes at rts/c/gpu.h:145-168): `map transpose` over f16 (the
 * `transpose b` of the f16 matrix product), `transpose` over i64 and over bool. */
int futhark_entry_transpose_f16_3d(struct futhark_context *ctx, struct futhark_f16_3d **out0,
                                   const struct futhark_f16_3d *in0);
int futhark_entry_transpose_i64(struct futhark_context *ctx, struct futhark_i64_2d **out0,
                                const struct futhark_i64_2d *in0);
int futhark_entry_transpose_bool(struct futhark_context *ctx, struct futhark_bool_2d **out0,
                                 const struct futhark_bool_2d *in0);
/* entry replicate_i32 (n: i64) (v: i32): [n]i32 = replicate n v;  entry iota_i64 (n: i64): [n]i64 = iota n:
 * the fills the reference's compiler emits around SegOps (src/Futhark/CodeGen/ImpGen/GPU/Base.hs:1342-1436). */
int futhark_entry_replicate_i32(struct futhark_context *ctx, struct futhark_i32_1d **out0,
                                const int64_t in0, const int32_t in1);
int futhark_entry_iota_i64(struct futhark_context *ctx, struct futhark_i64_1d **out0, const int64_t in0);

/* Other scans, segmented scans, filters and partitions: the same single-pass kernel under other
 * specifications (operator, fused map body, post-operation, flag source, predicate), where the
 * reference generates a kernel per program from the same pieces (src/Futhark/CodeGen/ImpGen/GPU/
 * SegScan.hs:17-90, SegScan/SinglePass.hs:327-879; prelude/soacs.fut:241-323).
 *
 * entry scan_max_i32 (xs: []i32): []i32 = scan i32.max i32.lowest xs
 * entry segscan_rows_i32 (xss: [][]i32): [][]i32 = map (scan (+) 0) xss   (tests/intrablock/segscan0.fut;
 *   a regular segmented scan: the innermost dimension is the segment, SegScan/SinglePass.hs:471-482,594-599)
 * entry scanomap_steps_i32 (xs: []i32): []i32 = main of tests/soacs/scan4.fut:20-22: two rounds of
 *   xs' = map2 (+) (map (+ sum) (scan (+) 0 (map (+1) xs))) xs, sum = reduce (+) 0 (map (+1) xs):
 *   the map body in front of the scan and the post-operation behind it run inside the scan kernel
 * entry filter_pos_i32 (xs: []i32): []i32 = filter (0 <) xs                (tests/soacs/filter1.fut)
 * entry filter_by_flag_i32 (xs: []i32) (keep: []bool): []i32 = (unzip (filter (.1) (zip xs keep))).0
 *   (tests/soacs/filter3.fut: the predicate reads a second array)
 * entry partition2_i32 (xs: []i32): ([]i32, []i32, []i32) =
 *   partition2 (\x -> x % 2 == 0) (\x -> x % 3 == 0) xs   (tests/soacs/partition1.fut; prelude/soacs.fut:293-323)
 * entry partition2_pairs_i32 [n] (xs: [n]i32) (ys: [n]i32): ([]i32, []i32, []i32, []i32, []i32, []i32) =
 *   main of tests/soacs/partition2.fut:16-21: partition2 (\(x, y) -> x < y) (\(x, y) -> x == y) (zip xs ys),
 *   each of the three groups unzipped (a three-way partition of an array of tuples)
 * entry scan_map2_add_i32 [m][k] (xss: [m][k]i32): [m][k]i32 = scan (map2 (+)) (replicate k 0) xss
 *   (tests/soacs/scan-with-map.fut, scan5.fut: an operator on whole rows; the scan is interchanged with the
 *   inner map and runs as a regular segmented scan over the transposed array) */
int futhark_entry_scan_max_i32(struct futhark_context *ctx, struct futhark_i32_1d **out0,
                               const struct futhark_i32_1d *in0);
int futhark_entry_segscan_rows_i32(struct futhark_context *ctx, struct futhark_i32_2d **out0,
                                   const struct futhark_i32_2d *in0);
int futhark_entry_scan_map2_add_i32(struct futhark_context *ctx, struct futhark_i32_2d **out0,
                                    const struct futhark_i32_2d *in0);
int futhark_entry_scanomap_steps_i32(struct futhark_context *ctx, struct futhark_i32_1d **out0,
                                     const struct futhark_i32_1d *in0);
int futhark_entry_filter_pos_i32(struct futhark_context *ctx, struct futhark_i32_1d **out0,
                                 const struct futhark_i32_1d *in0);
int futhark_entry_filter_by_flag_i32(struct futhark_context *ctx, struct futhark_i32_1d **out0,
                                     const struct futhark_i32_1d *in0, const struct futhark_bool_1d *in1);
int futhark_entry_partition2_i32(struct futhark_context *ctx,
                                 struct futhark_opaque_tup3_arr1d_i32_arr1d_i32_arr1d_i32 **out0,
                                 const struct futhark_i32_1d *in0);
int futhark_entry_partition2_pairs_i32(
    struct futhark_context *ctx, struct futhark_opaque_tup6_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32 **out0,
    const struct futhark_i32_1d *in0, const struct futhark_i32_1d *in1);

/* Scans whose operator works on 8-byte values or on tuples take the two-pass route (three
 * launches: per-block scan, scan of the block carries, carry distribution), as the reference's do
 * when its single-pass kernel does not apply (src/Futhark/CodeGen/ImpGen/GPU/SegScan.hs:51-90,
 * SegScan/TwoPass.hs:146-682).
 *
 * entry scan_i64 (xs: []i64): []i64 = scan (+) 0 xs
 * entry linrec_f32 (as: []f32) (bs: []f32): []f32 =
 *   map (.1) (scan (\(a1,b1) (a2,b2) -> (a1*a2, b1*a2+b2)) (1,0) (zip as bs))
 *   (a non-commutative operator on pairs: out[i] = as[i] * out[i-1] + bs[i], out[-1] = 0) */
int futhark_entry_scan_i64(struct futhark_context *ctx, struct futhark_i64_1d **out0,
                           const struct futhark_i64_1d *in0);
int futhark_entry_linrec_f32(struct futhark_context *ctx, struct futhark_f32_1d **out0,
                             const struct futhark_f32_1d *in0, const struct futhark_f32_1d *in1);

/* Fused and multi-operator SegOps.  The reference generates ONE kernel for a map body fused
 * with one or several reduction operators (src/Futhark/CodeGen/ImpGen/GPU/SegRed.hs:99-100,
 * 129-145) and keeps operand order for non-commutative operators (:836-921); here one kernel
 * template takes the body and the operators as a specification type.
 *
 * entry exscan_i32 (xs: []i32): []i32 = exscan (+) 0 xs          (prelude/soacs.fut:212-215;
 *   tests/soacs/exscan0.fut, exscan1.fut): out[0] = 0, out[i] = xs[0] + ... + xs[i-1].
 * entry mss_i32 (xs: []i32): i32 = (reduce redOp (0,0,0,0) (map mapOp xs)).0, the maximum
 *   segment sum of tests/mss.fut:6-20: a 4-tuple-valued, non-commutative operator.
 * entry sum_i32_f32 (xs: []i32): (i32, f32) = (i32.sum xs, f32.sum (map f32.i32 xs)), the
 *   horizontally fused pair of tests/fusion/red-red-fusion.fut:5.
 * entry dotprod_f32 (xs: []f32) (ys: []f32): f32 = reduce (+) 0 (map2 (*) xs ys): a map body over two
 *   inputs fused into the reduction (the shape of every dot product in the programs under tests/tiling).
 * entry prod_of_sums_i32 (xs: []i32) (ys: []i32): i32 = reduce (*) 1 (map2 (+) xs ys), the DotProd
 *   functor of tests/modules/functor1.fut:30-33 applied to i32 (known answer :3-4).
 * entry dotprod_i32 (xs: []i32) (ys: []i32): i32 = reduce (+) 0 (map2 (*) xs ys)   (tests/soacs/reduce2.fut)
 * entry product_i32 (xs: []i32): i32 = reduce (*) 1 xs                             (tests/soacs/reduce1.fut)
 * entry linrec_last_f32 (as: []f32) (bs: []f32): f32 =
 *   (reduce (\(a1,b1) (a2,b2) -> (a1*a2, b1*a2+b2)) (1,0) (zip as bs)).1: a non-commutative operator on
 *   pairs over two inputs (operand order kept as in SegRed.hs:836-921); equals last (linrec_f32 as bs).
 * Those with scalar results read them back, so they synchronise. */
int futhark_entry_exscan_i32(struct futhark_context *ctx, struct futhark_i32_1d **out0,
                             const struct futhark_i32_1d *in0);
int futhark_entry_mss_i32(struct futhark_context *ctx, int32_t *out0,
                          const struct futhark_i32_1d *in0);
int futhark_entry_sum_i32_f32(struct futhark_context *ctx, struct futhark_opaque_tup2_i32_f32 **out0,
                              const struct futhark_i32_1d *in0);
int futhark_entry_dotprod_f32(struct futhark_context *ctx, float *out0,
                              const struct futhark_f32_1d *in0, const struct futhark_f32_1d *in1);
int futhark_entry_prod_of_sums_i32(struct futhark_context *ctx, int32_t *out0,
                                   const struct futhark_i32_1d *in0, const struct futhark_i32_1d *in1);
int futhark_entry_dotprod_i32(struct futhark_context *ctx, int32_t *out0,
                              const struct futhark_i32_1d *in0, const struct futhark_i32_1d *in1);
int futhark_entry_product_i32(struct futhark_context *ctx, int32_t *out0,
                              const struct futhark_i32_1d *in0);
int futhark_entry_linrec_last_f32(struct futhark_context *ctx, float *out0,
                                  const struct futhark_f32_1d *in0, const struct futhark_f32_1d *in1);

/* ---- extensions (prefix futhark_b200_): not part of the reference's generated API ----
 * The reference keeps its one CUDA stream private (rts/c/backends/cuda.h:219); a host
 * program that shares a process with other CUDA code needs it to order its own work
 * (events, copies, collectives) against the entry points. */

/* The context's stream, as a cudaStream_t / CUstream handle.  Every entry point, copy and
 * kernel of the context is enqueued on it. */
void *futhark_b200_context_get_stream(struct futhark_context *ctx);
/* Ordinal of the CUDA device the context runs on. */
int futhark_b200_context_get_device(struct futhark_context *ctx);
/* Number of kernel launches issued by the context so far. */
int64_t futhark_b200_context_get_launch_count(struct futhark_context *ctx);

/* Failure-path check that faults nothing: enqueues one warp that waits, like a scan tile,
 * for a tile status word that is never published, gives up after `max_polls` polls of
 * ~100 ns (at most 100000) and records the look-back time-out in the context's failure
 * word.  The next futhark_context_sync then returns FUTHARK_PROGRAM_ERROR with a message,
 * clears the failure and resets the scan scratch, as after a real time-out
 * (the global_failure protocol of rts/c/backends/cuda.h:719-754); the context stays usable. */
int futhark_b200_debug_expire_wait(struct futhark_context *ctx, int max_polls);

/* Strided copy between two arrays in device memory, each described by an LMAD: an offset and
 * one stride per dimension of the common `shape`, all counted in elements of elem_size (1, 2, 4
 * or 8) bytes; rank 0..8.  For every index I below shape:
 *     dst[dst_offset + sum_i I_i * dst_strides[i]] = src[src_offset + sum_i I_i * src_strides[i]]
 * It stands where the reference's generated code calls lmad_copy_gpu2gpu_{1,2,4,8}b
 * (rts/c/gpu.h:540-586; host-side twin rts/c/copy.h:60-268) for the layout changes the compiler
 * inserts around SegOps, and routes the copy the same way: a batched transposition (of 4-byte
 * elements) to the tiled transposition kernel, a copy between equal dense layouts to one
 * device-to-device copy, the rest to a general strided kernel (rts/opencl/copy.cl:3-83).
 * Strides may be zero or negative on the source; the destination index must be injective.
 * Asynchronous, on the context's stream.
 *
 * futhark_b200_lmad_classify is the host-only routing decision for 4-byte elements
 * (0 general, 1 batched transposition, 2 flat copy; -2 bad rank); for a transposition
 * knm (may be NULL) receives {arrays, rows, columns of the source matrix}. */
int futhark_b200_lmad_copy(struct futhark_context *ctx, int elem_size, int r,
                           CUdeviceptr dst, int64_t dst_offset, const int64_t *dst_strides,
                           CUdeviceptr src, int64_t src_offset, const int64_t *src_strides,
                           const int64_t *shape);
int futhark_b200_lmad_classify(int r, const int64_t *dst_strides, const int64_t *src_strides,
                               const int64_t *shape, int64_t *knm);

/* Host-side values in the two formats of the reference's compiled executables: the textual
 * value syntax and the binary data format (docs/binary-data-format.rst; the behaviour of
 * rts/c/values.h:18-845: read_array/read_scalar, write_array/write_scalar, end_of_input).
 * Readers are typed like the reference's: the caller names the element type ("i8" ... "u64",
 * "f16", "f32", "f64", "bool") and the rank its entry point expects; text or binary is detected
 * per value (a leading 'b'), text elements may omit the type suffix, `--` comments are skipped.
 * Unlike the reference, which ends the process, a malformed or mismatching value returns 1 and
 * leaves a message for futhark_b200_value_error().  f16 data is binary16 bits. */
struct futhark_b200_value {
  char type[8];        /* element type name */
  int32_t rank;        /* 0 for a scalar */
  int64_t shape[8];
  void *data;          /* row-major elements, malloc'd by the readers */
};
int futhark_b200_value_read(FILE *f, const char *type, int rank, struct futhark_b200_value *out);
int futhark_b200_value_write(FILE *f, const struct futhark_b200_value *v, int binary);
void futhark_b200_value_free(struct futhark_b200_value *v);
/* 0 when nothing but blanks and comments remains (rts/c/values.h:713-722) */
int futhark_b200_value_end_of_input(FILE *f);
const char *futhark_b200_value_error(void);
/* The same over memory: *consumed receives the bytes read; *buf is malloc'd. */
int futhark_b200_value_read_mem(const void *buf, size_t len, size_t *consumed, const char *type,
                                int rank, struct futhark_b200_value *out);
int futhark_b200_value_write_mem(const struct futhark_b200_value *v, int binary, void **buf,
                                 size_t *len);

/* Shard-local pieces, for one logical array split into contiguous shards over several
 * contexts (one per GPU).  The reference is single-device (rts/c/backends/cuda.h:219) and has
 * no counterpart.  All are asynchronous; device pointers passed in must belong to the
 * context's device and be ordered on the context's stream.
 *
 *  reduce_i32_to_device    writes reduce (+) 0 of the shard to *dst (one i32 on the device)
 *  entry_scan_i32_carried  scan (+) of the shard started from the sum of the num_carries i32
 *                          values at `carries` (the totals of the shards before this one)
 *  entry_segscan_f32_shard the segmented scan of the shard alone, plus its 16-byte summary at
 *                          summary_dst, written by the scan kernel itself: {f32 bits of the last
 *                          element, 1 if any segment starts in the shard else 0, index of the
 *                          first 5120-element tile of the shard that holds a segment start (all
 *                          ones if none), 0}
 *  segscan_f32_apply_carries  given the summaries of all shards (4 x u32 each, in rank order),
 *                          adds the carry of shards 0..rank-1 to the elements of `out` that
 *                          precede the shard's first segment start (one kernel; shard `rank`'s
 *                          own summary tells it where to look for that start) */
int futhark_b200_reduce_i32_to_device(struct futhark_context *ctx, CUdeviceptr dst,
                                      const struct futhark_i32_1d *in0);
int futhark_b200_entry_scan_i32_carried(struct futhark_context *ctx, struct futhark_i32_1d **out0,
                                        const struct futhark_i32_1d *in0, CUdeviceptr carries,
                                        int num_carries);
int futhark_b200_entry_segscan_f32_shard(struct futhark_context *ctx, struct futhark_f32_1d **out0,
                                         CUdeviceptr summary_dst, const struct futhark_bool_1d *in0,
                                         const struct futhark_f32_1d *in1);
int futhark_b200_segscan_f32_apply_carries(struct futhark_context *ctx, struct futhark_f32_1d *out,
                                           const struct futhark_bool_1d *in0, CUdeviceptr summaries,
                                           int rank);

/* The sharded operations through the C ABI: a group is one rank of a set of contexts (one per
 * GPU, in one process or several) that hold contiguous shards of one logical array.  Each
 * operation runs the shard-local entry points above plus, where it has an exchange step, one
 * NCCL collective on the context's own stream (NCCL is looked up at run time in the libnccl.so.2
 * of the process; the library does not link it).  No counterpart in the reference, which is
 * single-device (rts/c/backends/cuda.h:219).
 *
 *  group_unique_id   fills 128 bytes (an ncclUniqueId) on ONE rank; the host program hands them
 *                    to the others (MPI, a file, a socket, torch.distributed ...)
 *  group_new         joins the group: ncclCommInitRank on the context's device; collective
 *  group_from_comm   or: borrows a communicator (ncclComm_t) the host already has
 *  group_unavailable NULL, or why NCCL could not be loaded
 *  group_reduce_i32  the sum over all shards, on every rank (synchronous, like every scalar result)
 *  group_scan_i32    this rank's shard of the scan of the whole array
 *  group_segscan_f32 this rank's shard of the flagged segmented scan of the whole array
 *  group_segscan_f32_begin / _finish   the same in two halves: the shard's scan, and the carry; what
 *                    the host enqueues between them runs while the summaries travel
 *  group_enable_peer_exchange   collective, once: from then on the summaries of the segmented scan
 *                    are written by the scan kernels straight into the other GPUs' memory (peer
 *                    stores over NVLink, buffers swapped as CUDA IPC handles) and awaited by the
 *                    carry kernels with a bounded wait, instead of gathered by a collective
 *  group_hist_*      the histogram of the whole array, on every rank
 *  group_filter_u32 / group_partition_u32   this rank's part of the result, with the offsets at
 *                    which it lies in the logical result (selected keys of all ranks first, then
 *                    the rejected ones) and the total number of selected keys
 *  group_bmm_f16     whole batches per rank: the local contraction */
struct futhark_b200_group;
int futhark_b200_group_unique_id(void *id_out, size_t len);
const char *futhark_b200_group_unavailable(void);
struct futhark_b200_group *futhark_b200_group_new(struct futhark_context *ctx, const void *unique_id,
                                                  int rank, int world);
struct futhark_b200_group *futhark_b200_group_from_comm(struct futhark_context *ctx, void *nccl_comm,
                                                        int rank, int world);
void futhark_b200_group_free(struct futhark_b200_group *g);
int futhark_b200_group_rank(const struct futhark_b200_group *g);
int futhark_b200_group_size(const struct futhark_b200_group *g);
int futhark_b200_group_reduce_i32(struct futhark_b200_group *g, int32_t *out0, const struct futhark_i32_1d *in0);
int futhark_b200_group_scan_i32(struct futhark_b200_group *g, struct futhark_i32_1d **out0,
                                const struct futhark_i32_1d *in0);
int futhark_b200_group_segscan_f32(struct futhark_b200_group *g, struct futhark_f32_1d **out0,
                                   const struct futhark_bool_1d *in0, const struct futhark_f32_1d *in1);
int futhark_b200_group_segscan_f32_begin(struct futhark_b200_group *g, const struct futhark_bool_1d *in0,
                                         const struct futhark_f32_1d *in1);
int futhark_b200_group_segscan_f32_finish(struct futhark_b200_group *g, struct futhark_f32_1d **out0,
                                          const struct futhark_bool_1d *in0);
int futhark_b200_group_enable_peer_exchange(struct futhark_b200_group *g);
int futhark_b200_group_hist_add_i32(struct futhark_b200_group *g, struct futhark_i32_1d **out0, const int64_t in0,
                                    const struct futhark_i32_1d *in1, const struct futhark_i32_1d *in2);
int futhark_b200_group_hist_max_f32(struct futhark_b200_group *g, struct futhark_f32_1d **out0, const int64_t in0,
                                    const struct futhark_i32_1d *in1, const struct futhark_f32_1d *in2);
int futhark_b200_group_filter_u32(struct futhark_b200_group *g, struct futhark_u32_1d **out0, int64_t *offset,
                                  int64_t *total, const struct futhark_u32_1d *in0);
int futhark_b200_group_partition_u32(struct futhark_b200_group *g,
                                     struct futhark_opaque_tup2_arr1d_u32_arr1d_u32 **out0,
                                     int64_t *sel_offset, int64_t *rej_offset, int64_t *total_selected,
                                     const struct futhark_u32_1d *in0);
int futhark_b200_group_bmm_f16(struct futhark_b200_group *g, struct futhark_f32_3d **out0,
                               const struct futhark_f16_3d *in0, const struct futhark_f16_3d *in1);

/* Inclusive scan (+) over n i32 values in device memory, in -> out, with no allocation of
 * any kind.  It has no counterpart in the reference, whose entry points always allocate
 * their results and temporaries from the context's pool (rts/c/gpu.h:240-316).
 *
 * Who needs it: a host that cannot let this library allocate -- because the GPU's memory is
 * already divided up by the host's own allocator, or because the call sits in a part of the
 * host program (a latency-bound loop after start-up, say) where a device-wide
 * synchronisation or an out-of-memory failure from cudaMalloc cannot be tolerated.  The
 * caller supplies `in` and `out` (device pointers, 4-byte aligned; 16-byte alignment is
 * faster; the two ranges must not overlap -- the scan does not work in place, and an
 * overlapping pair is refused with a non-zero return); the scan's temporaries (a tile counter and one 8-byte status word per tile of
 * 5120 elements) live in a fixed ~103 KiB array inside the library image, which every GPU
 * that loads the library keeps until the process exits.
 *
 * Limits and rules:
 *  - n must be <= 2^26 = 67108864 (what the fixed array has room for); a longer input is
 *    refused with a non-zero return and a message in errbuf;
 *  - the work is enqueued on `stream` (a cudaStream_t; NULL = the default stream) of the
 *    CURRENT device and the function returns without waiting;
 *  - if status_dev is not NULL, one i32 is written there (device memory) after the scan:
 *    0 = complete, otherwise a wait inside the kernel hit its limit and `out` is incomplete;
 *  - the first call on each device looks up the array's device address; make that first
 *    call before starting any stream capture;
 *  - all calls share the one array: two calls whose GPU work may overlap (different
 *    streams, different threads) race on it and give wrong results -- serialise them;
 *  - errbuf (may be NULL) receives a NUL-terminated message when the return value is not 0. */
int futhark_b200_scan_i32_noalloc(const int32_t *in, int32_t *out, int64_t n, void *stream,
                                  int32_t *status_dev, char *errbuf, size_t errbuf_len);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* FUTHARK_B200_H */
