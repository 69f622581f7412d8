// What the two front-ends (the executable and the server) know about the library: its array
// types, its entry points with their parameter and result types, and a uniform representation
// of the values they pass around.  It plays the part of the manifest-driven tables that the
// reference generates into every program (src/Futhark/CodeGen/Backends/GenericC/Server.hs:
// one `struct type` with restore/store/free functions per type and one `struct entry_point` per
// entry; GenericC/CLI.hs for the executable).  Plain C++ on the library's C ABI.
#pragma once
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <functional>
#include <string>
#include <vector>

#define FUTHARK_B200_NO_CUDA_H
#include "../../include/futhark_b200.h"

namespace fe {

struct PrimType { const char *name; size_t size; };
static const PrimType PRIMS[] = {{"i8", 1}, {"i16", 2}, {"i32", 4}, {"i64", 8}, {"u8", 1}, {"u16", 2}, {"u32", 4},
                                 {"u64", 8}, {"f16", 2}, {"f32", 4}, {"f64", 8}, {"bool", 1}};
inline const PrimType *prim_type(const std::string &name) {
  for (const PrimType &p : PRIMS)
    if (name == p.name) return &p;
  return nullptr;
}

// An array type of the C API behind type-erased functions.
struct ArrayType {
  const char *name;      // as the server protocol prints it: "[]i32", "[][][]f16"
  const char *elem;
  int rank;
  size_t elem_size;
  void *(*make)(futhark_context *, const void *, const int64_t *);
  int (*values)(futhark_context *, void *, void *);
  const int64_t *(*shape)(futhark_context *, void *);
  int (*release)(futhark_context *, void *);
};

#define FE_DIMS_1 s[0]
#define FE_DIMS_2 s[0], s[1]
#define FE_DIMS_3 s[0], s[1], s[2]
#define FE_ARRAY(T, CT, R, NAME, ELEM)                                                                              \
  {NAME, ELEM, R, sizeof(CT),                                                                                       \
   [](futhark_context *c, const void *d, const int64_t *s) -> void * { return futhark_new_##T##_##R##d(c, (const CT *)d, FE_DIMS_##R); }, \
   [](futhark_context *c, void *a, void *d) { return futhark_values_##T##_##R##d(c, (futhark_##T##_##R##d *)a, (CT *)d); },              \
   [](futhark_context *c, void *a) { return futhark_shape_##T##_##R##d(c, (futhark_##T##_##R##d *)a); },                                 \
   [](futhark_context *c, void *a) { return futhark_free_##T##_##R##d(c, (futhark_##T##_##R##d *)a); }}

static const ArrayType ARRAYS[] = {
    FE_ARRAY(i32, int32_t, 1, "[]i32", "i32"),   FE_ARRAY(i64, int64_t, 1, "[]i64", "i64"), FE_ARRAY(u32, uint32_t, 1, "[]u32", "u32"),
    FE_ARRAY(f32, float, 1, "[]f32", "f32"),     FE_ARRAY(bool, bool, 1, "[]bool", "bool"), FE_ARRAY(f32, float, 2, "[][]f32", "f32"),
    FE_ARRAY(f32, float, 3, "[][][]f32", "f32"), FE_ARRAY(f16, uint16_t, 3, "[][][]f16", "f16"),
    FE_ARRAY(f64, double, 1, "[]f64", "f64"),    FE_ARRAY(i32, int32_t, 2, "[][]i32", "i32"), FE_ARRAY(i64, int64_t, 2, "[][]i64", "i64"),
    FE_ARRAY(bool, bool, 2, "[][]bool", "bool"), FE_ARRAY(i8, int8_t, 1, "[]i8", "i8"), FE_ARRAY(i16, int16_t, 1, "[]i16", "i16"),
    FE_ARRAY(f16, uint16_t, 1, "[]f16", "f16"), FE_ARRAY(i32, int32_t, 3, "[][][]i32", "i32"),
    FE_ARRAY(u8, uint8_t, 1, "[]u8", "u8"), FE_ARRAY(u16, uint16_t, 1, "[]u16", "u16"),
    FE_ARRAY(f64, double, 2, "[][]f64", "f64"),
};
inline const ArrayType *array_type(const std::string &name) {
  for (const ArrayType &a : ARRAYS)
    if (name == a.name) return &a;
  return nullptr;
}

struct RecordType;

// A value: a scalar held on the host, an array held on the device, or a record (an opaque object
// of the C API whose fields are reached by projection).
struct Value {
  std::string type;
  const ArrayType *array = nullptr;
  const RecordType *record = nullptr;
  void *arr = nullptr;                       // the array or opaque object
  unsigned char scalar[8] = {0, 0, 0, 0, 0, 0, 0, 0};
};

// The record types entry points return (tuples: fields named 0, 1, ... as in the C API).
struct RecordType {
  const char *name;
  std::vector<const char *> fields;
  int (*release)(futhark_context *, void *);
  int (*project)(futhark_context *, const void *obj, int field, Value &out);   // a new reference / the scalar
  int (*make)(futhark_context *, const std::vector<const Value *> &fields, void **obj);
};

inline int release(futhark_context *ctx, Value &v) {
  int rc = 0;
  if (v.arr != nullptr) rc = v.record != nullptr ? v.record->release(ctx, v.arr) : v.array->release(ctx, v.arr);
  v.arr = nullptr;
  return rc;
}

inline void set_array(Value &v, const char *type, void *arr) {
  v.type = type;
  v.array = array_type(type);
  v.arr = arr;
}
template <typename T>
inline void set_scalar(Value &v, const char *type, T x) {
  v.type = type;
  memcpy(v.scalar, &x, sizeof(T));
}
template <typename T>
inline T scalar_of(const Value &v) {
  T x;
  memcpy(&x, v.scalar, sizeof(T));
  return x;
}

static const RecordType RECORDS[] = {
    {"([]u32, []u32)", {"[]u32", "[]u32"},
     [](futhark_context *c, void *o) { return futhark_free_opaque_tup2_arr1d_u32_arr1d_u32(c, (futhark_opaque_tup2_arr1d_u32_arr1d_u32 *)o); },
     [](futhark_context *c, const void *o, int k, Value &out) {
       futhark_u32_1d *a = nullptr;
       const auto *obj = (const futhark_opaque_tup2_arr1d_u32_arr1d_u32 *)o;
       const int rc = k == 0 ? futhark_project_opaque_tup2_arr1d_u32_arr1d_u32_0(c, &a, obj) : futhark_project_opaque_tup2_arr1d_u32_arr1d_u32_1(c, &a, obj);
       if (!rc) set_array(out, "[]u32", a);
       return rc;
     },
     [](futhark_context *c, const std::vector<const Value *> &f, void **obj) {
       return futhark_new_opaque_tup2_arr1d_u32_arr1d_u32(c, (futhark_opaque_tup2_arr1d_u32_arr1d_u32 **)obj, (const futhark_u32_1d *)f[0]->arr, (const futhark_u32_1d *)f[1]->arr);
     }},
    {"([]i64, [][]f64)", {"[]i64", "[][]f64"},
     [](futhark_context *c, void *o) { return futhark_free_opaque_tup2_arr1d_i64_arr2d_f64(c, (futhark_opaque_tup2_arr1d_i64_arr2d_f64 *)o); },
     [](futhark_context *c, const void *o, int k, Value &out) {
       const auto *obj = (const futhark_opaque_tup2_arr1d_i64_arr2d_f64 *)o;
       if (k == 0) {
         futhark_i64_1d *a = nullptr;
         const int rc = futhark_project_opaque_tup2_arr1d_i64_arr2d_f64_0(c, &a, obj);
         if (!rc) set_array(out, "[]i64", a);
         return rc;
       }
       futhark_f64_2d *a = nullptr;
       const int rc = futhark_project_opaque_tup2_arr1d_i64_arr2d_f64_1(c, &a, obj);
       if (!rc) set_array(out, "[][]f64", a);
       return rc;
     },
     [](futhark_context *c, const std::vector<const Value *> &f, void **obj) {
       return futhark_new_opaque_tup2_arr1d_i64_arr2d_f64(c, (futhark_opaque_tup2_arr1d_i64_arr2d_f64 **)obj, (const futhark_i64_1d *)f[0]->arr, (const futhark_f64_2d *)f[1]->arr);
     }},
    {"([]i32, []i32)", {"[]i32", "[]i32"},
     [](futhark_context *c, void *o) { return futhark_free_opaque_tup2_arr1d_i32_arr1d_i32(c, (futhark_opaque_tup2_arr1d_i32_arr1d_i32 *)o); },
     [](futhark_context *c, const void *o, int k, Value &out) {
       futhark_i32_1d *a = nullptr;
       const auto *obj = (const futhark_opaque_tup2_arr1d_i32_arr1d_i32 *)o;
       const int rc = k == 0 ? futhark_project_opaque_tup2_arr1d_i32_arr1d_i32_0(c, &a, obj) : futhark_project_opaque_tup2_arr1d_i32_arr1d_i32_1(c, &a, obj);
       if (!rc) set_array(out, "[]i32", a);
       return rc;
     },
     [](futhark_context *c, const std::vector<const Value *> &f, void **obj) {
       return futhark_new_opaque_tup2_arr1d_i32_arr1d_i32(c, (futhark_opaque_tup2_arr1d_i32_arr1d_i32 **)obj, (const futhark_i32_1d *)f[0]->arr, (const futhark_i32_1d *)f[1]->arr);
     }},
    {"([]i32, []i32, []i32)", {"[]i32", "[]i32", "[]i32"},
     [](futhark_context *c, void *o) { return futhark_free_opaque_tup3_arr1d_i32_arr1d_i32_arr1d_i32(c, (futhark_opaque_tup3_arr1d_i32_arr1d_i32_arr1d_i32 *)o); },
     [](futhark_context *c, const void *o, int k, Value &out) {
       futhark_i32_1d *a = nullptr;
       const auto *obj = (const futhark_opaque_tup3_arr1d_i32_arr1d_i32_arr1d_i32 *)o;
       const int rc = k == 0   ? futhark_project_opaque_tup3_arr1d_i32_arr1d_i32_arr1d_i32_0(c, &a, obj)
                      : k == 1 ? futhark_project_opaque_tup3_arr1d_i32_arr1d_i32_arr1d_i32_1(c, &a, obj)
                               : futhark_project_opaque_tup3_arr1d_i32_arr1d_i32_arr1d_i32_2(c, &a, obj);
       if (!rc) set_array(out, "[]i32", a);
       return rc;
     },
     [](futhark_context *c, const std::vector<const Value *> &f, void **obj) {
       return futhark_new_opaque_tup3_arr1d_i32_arr1d_i32_arr1d_i32(c, (futhark_opaque_tup3_arr1d_i32_arr1d_i32_arr1d_i32 **)obj, (const futhark_i32_1d *)f[0]->arr,
                                                                    (const futhark_i32_1d *)f[1]->arr, (const futhark_i32_1d *)f[2]->arr);
     }},
    {"([]i32, []i32, []i32, []i32, []i32, []i32)", {"[]i32", "[]i32", "[]i32", "[]i32", "[]i32", "[]i32"},
     [](futhark_context *c, void *o) { return futhark_free_opaque_tup6_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32(c, (futhark_opaque_tup6_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32 *)o); },
     [](futhark_context *c, const void *o, int k, Value &out) {
       using Project = int (*)(futhark_context *, futhark_i32_1d **, const futhark_opaque_tup6_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32 *);
       static const Project project[6] = {futhark_project_opaque_tup6_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_0, futhark_project_opaque_tup6_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_1, futhark_project_opaque_tup6_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_2,
                                          futhark_project_opaque_tup6_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_3, futhark_project_opaque_tup6_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_4, futhark_project_opaque_tup6_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_5};
       futhark_i32_1d *a = nullptr;
       const int rc = project[k](c, &a, (const futhark_opaque_tup6_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32 *)o);
       if (!rc) set_array(out, "[]i32", a);
       return rc;
     },
     [](futhark_context *c, const std::vector<const Value *> &f, void **obj) {
       return futhark_new_opaque_tup6_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32(c, (futhark_opaque_tup6_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32 **)obj, (const futhark_i32_1d *)f[0]->arr, (const futhark_i32_1d *)f[1]->arr,
                                (const futhark_i32_1d *)f[2]->arr, (const futhark_i32_1d *)f[3]->arr, (const futhark_i32_1d *)f[4]->arr,
                                (const futhark_i32_1d *)f[5]->arr);
     }},
    {"(i32, f32)", {"i32", "f32"},
     [](futhark_context *c, void *o) { return futhark_free_opaque_tup2_i32_f32(c, (futhark_opaque_tup2_i32_f32 *)o); },
     [](futhark_context *c, const void *o, int k, Value &out) {
       const auto *obj = (const futhark_opaque_tup2_i32_f32 *)o;
       int32_t a = 0;
       float b = 0;
       const int rc = k == 0 ? futhark_project_opaque_tup2_i32_f32_0(c, &a, obj) : futhark_project_opaque_tup2_i32_f32_1(c, &b, obj);
       if (!rc) { if (k == 0) set_scalar(out, "i32", a); else set_scalar(out, "f32", b); }
       return rc;
     },
     [](futhark_context *c, const std::vector<const Value *> &f, void **obj) {
       return futhark_new_opaque_tup2_i32_f32(c, (futhark_opaque_tup2_i32_f32 **)obj, scalar_of<int32_t>(*f[0]), scalar_of<float>(*f[1]));
     }},
};
inline const RecordType *record_type(const std::string &name) {
  for (const RecordType &r : RECORDS)
    if (name == r.name) return &r;
  return nullptr;
}
inline void set_record(Value &v, const char *type, void *obj) {
  v.type = type;
  v.record = record_type(type);
  v.arr = obj;
}

// Host value (as read from a file) -> value; arrays are uploaded.  Returns 0, or 1 with the
// context's error set / a type that is not transparent.
inline int from_host(futhark_context *ctx, const std::string &type, const futhark_b200_value &h, Value &out) {
  if (const ArrayType *a = array_type(type)) {
    void *arr = a->make(ctx, h.data, h.shape);
    if (arr == nullptr) return 1;
    set_array(out, a->name, arr);
    return 0;
  }
  if (const PrimType *p = prim_type(type)) {
    out.type = p->name;
    memcpy(out.scalar, h.data, p->size);
    return 0;
  }
  return 1;
}

// Value -> host value (malloc'd data; arrays are downloaded, the caller synchronises before use).
inline int to_host(futhark_context *ctx, const Value &v, futhark_b200_value &h) {
  memset(&h, 0, sizeof(h));
  if (v.array != nullptr) {
    snprintf(h.type, sizeof(h.type), "%s", v.array->elem);
    h.rank = v.array->rank;
    const int64_t *shape = v.array->shape(ctx, v.arr);
    size_t n = 1;
    for (int d = 0; d < h.rank; d++) { h.shape[d] = shape[d]; n *= (size_t)shape[d]; }
    h.data = calloc(n ? n : 1, v.array->elem_size);
    return v.array->values(ctx, v.arr, h.data);
  }
  const PrimType *p = prim_type(v.type);
  if (p == nullptr) return 1;
  snprintf(h.type, sizeof(h.type), "%s", p->name);
  h.rank = 0;
  h.data = calloc(1, 8);
  memcpy(h.data, v.scalar, p->size);
  return 0;
}

// "[][]f32" -> ("f32", 2); a scalar type has rank 0
inline void split_type(const std::string &type, std::string &elem, int &rank) {
  size_t i = 0;
  rank = 0;
  while (type.compare(i, 2, "[]") == 0) { i += 2; rank++; }
  elem = type.substr(i);
}

struct EntryPoint {
  const char *name;
  std::vector<const char *> ins;
  const char *out;
  std::function<int(futhark_context *, const std::vector<const Value *> &, Value &)> call;
};

#define FE_IN(i, T) ((const futhark_##T *)in[i]->arr)
// entry points of the shapes array -> array, (i64, array, array) -> array and (array, array[, array]) -> array
#define FE_E1(NAME, TI, SI, TO, SO) \
  {#NAME, {SI}, SO, [](C *c, In in, Value &o) { futhark_##TO *r = nullptr; int rc = futhark_entry_##NAME(c, &r, FE_IN(0, TI)); if (!rc) set_array(o, SO, r); return rc; }}
#define FE_E2(NAME, T0, S0, T1, S1, TO, SO) \
  {#NAME, {S0, S1}, SO, [](C *c, In in, Value &o) { futhark_##TO *r = nullptr; int rc = futhark_entry_##NAME(c, &r, FE_IN(0, T0), FE_IN(1, T1)); if (!rc) set_array(o, SO, r); return rc; }}
#define FE_E3(NAME, T0, S0, T1, S1, T2, S2, TO, SO) \
  {#NAME, {S0, S1, S2}, SO, [](C *c, In in, Value &o) { futhark_##TO *r = nullptr; int rc = futhark_entry_##NAME(c, &r, FE_IN(0, T0), FE_IN(1, T1), FE_IN(2, T2)); if (!rc) set_array(o, SO, r); return rc; }}
#define FE_EH(NAME, T1, S1, T2, S2, TO, SO) \
  {#NAME, {"i64", S1, S2}, SO, [](C *c, In in, Value &o) { futhark_##TO *r = nullptr; int rc = futhark_entry_##NAME(c, &r, scalar_of<int64_t>(*in[0]), FE_IN(1, T1), FE_IN(2, T2)); if (!rc) set_array(o, SO, r); return rc; }}

inline const std::vector<EntryPoint> &entry_points() {
  typedef futhark_context C;
  typedef const std::vector<const Value *> &In;
  static const std::vector<EntryPoint> table = {
      {"scan_i32", {"[]i32"}, "[]i32", [](C *c, In in, Value &o) { futhark_i32_1d *r = nullptr; int rc = futhark_entry_scan_i32(c, &r, FE_IN(0, i32_1d)); if (!rc) set_array(o, "[]i32", r); return rc; }},
      {"exscan_i32", {"[]i32"}, "[]i32", [](C *c, In in, Value &o) { futhark_i32_1d *r = nullptr; int rc = futhark_entry_exscan_i32(c, &r, FE_IN(0, i32_1d)); if (!rc) set_array(o, "[]i32", r); return rc; }},
      {"reduce_i32", {"[]i32"}, "i32", [](C *c, In in, Value &o) { int32_t r = 0; int rc = futhark_entry_reduce_i32(c, &r, FE_IN(0, i32_1d)); if (!rc) set_scalar(o, "i32", r); return rc; }},
      {"mss_i32", {"[]i32"}, "i32", [](C *c, In in, Value &o) { int32_t r = 0; int rc = futhark_entry_mss_i32(c, &r, FE_IN(0, i32_1d)); if (!rc) set_scalar(o, "i32", r); return rc; }},
      {"sum_i32_f32", {"[]i32"}, "(i32, f32)", [](C *c, In in, Value &o) { futhark_opaque_tup2_i32_f32 *r = nullptr; int rc = futhark_entry_sum_i32_f32(c, &r, FE_IN(0, i32_1d)); if (!rc) set_record(o, "(i32, f32)", r); return rc; }},
      {"dotprod_f32", {"[]f32", "[]f32"}, "f32", [](C *c, In in, Value &o) { float r = 0; int rc = futhark_entry_dotprod_f32(c, &r, FE_IN(0, f32_1d), FE_IN(1, f32_1d)); if (!rc) set_scalar(o, "f32", r); return rc; }},
      {"prod_of_sums_i32", {"[]i32", "[]i32"}, "i32", [](C *c, In in, Value &o) { int32_t r = 0; int rc = futhark_entry_prod_of_sums_i32(c, &r, FE_IN(0, i32_1d), FE_IN(1, i32_1d)); if (!rc) set_scalar(o, "i32", r); return rc; }},
      {"dotprod_i32", {"[]i32", "[]i32"}, "i32", [](C *c, In in, Value &o) { int32_t r = 0; int rc = futhark_entry_dotprod_i32(c, &r, FE_IN(0, i32_1d), FE_IN(1, i32_1d)); if (!rc) set_scalar(o, "i32", r); return rc; }},
      {"product_i32", {"[]i32"}, "i32", [](C *c, In in, Value &o) { int32_t r = 0; int rc = futhark_entry_product_i32(c, &r, FE_IN(0, i32_1d)); if (!rc) set_scalar(o, "i32", r); return rc; }},
      {"linrec_last_f32", {"[]f32", "[]f32"}, "f32", [](C *c, In in, Value &o) { float r = 0; int rc = futhark_entry_linrec_last_f32(c, &r, FE_IN(0, f32_1d), FE_IN(1, f32_1d)); if (!rc) set_scalar(o, "f32", r); return rc; }},
      {"segscan_f32", {"[]bool", "[]f32"}, "[]f32", [](C *c, In in, Value &o) { futhark_f32_1d *r = nullptr; int rc = futhark_entry_segscan_f32(c, &r, FE_IN(0, bool_1d), FE_IN(1, f32_1d)); if (!rc) set_array(o, "[]f32", r); return rc; }},
      {"segreduce_f32", {"[]i64", "[]bool", "[]f32"}, "[]f32", [](C *c, In in, Value &o) { futhark_f32_1d *r = nullptr; int rc = futhark_entry_segreduce_f32(c, &r, FE_IN(0, i64_1d), FE_IN(1, bool_1d), FE_IN(2, f32_1d)); if (!rc) set_array(o, "[]f32", r); return rc; }},
      {"rowsum_f32", {"[][]f32"}, "[]f32", [](C *c, In in, Value &o) { futhark_f32_1d *r = nullptr; int rc = futhark_entry_rowsum_f32(c, &r, FE_IN(0, f32_2d)); if (!rc) set_array(o, "[]f32", r); return rc; }},
      {"hist_add_i32", {"i64", "[]i32", "[]i32"}, "[]i32", [](C *c, In in, Value &o) { futhark_i32_1d *r = nullptr; int rc = futhark_entry_hist_add_i32(c, &r, scalar_of<int64_t>(*in[0]), FE_IN(1, i32_1d), FE_IN(2, i32_1d)); if (!rc) set_array(o, "[]i32", r); return rc; }},
      {"hist_max_f32", {"i64", "[]i32", "[]f32"}, "[]f32", [](C *c, In in, Value &o) { futhark_f32_1d *r = nullptr; int rc = futhark_entry_hist_max_f32(c, &r, scalar_of<int64_t>(*in[0]), FE_IN(1, i32_1d), FE_IN(2, f32_1d)); if (!rc) set_array(o, "[]f32", r); return rc; }},
      {"filter_u32", {"[]u32"}, "[]u32", [](C *c, In in, Value &o) { futhark_u32_1d *r = nullptr; int rc = futhark_entry_filter_u32(c, &r, FE_IN(0, u32_1d)); if (!rc) set_array(o, "[]u32", r); return rc; }},
      {"partition_u32", {"[]u32"}, "([]u32, []u32)", [](C *c, In in, Value &o) { futhark_opaque_tup2_arr1d_u32_arr1d_u32 *r = nullptr; int rc = futhark_entry_partition_u32(c, &r, FE_IN(0, u32_1d)); if (!rc) set_record(o, "([]u32, []u32)", r); return rc; }},
      {"bmm_f16", {"[][][]f16", "[][][]f16"}, "[][][]f32", [](C *c, In in, Value &o) { futhark_f32_3d *r = nullptr; int rc = futhark_entry_bmm_f16(c, &r, FE_IN(0, f16_3d), FE_IN(1, f16_3d)); if (!rc) set_array(o, "[][][]f32", r); return rc; }},
      {"transpose_f32", {"[][]f32"}, "[][]f32", [](C *c, In in, Value &o) { futhark_f32_2d *r = nullptr; int rc = futhark_entry_transpose_f32(c, &r, FE_IN(0, f32_2d)); if (!rc) set_array(o, "[][]f32", r); return rc; }},
      {"transpose_f32_3d", {"[][][]f32"}, "[][][]f32", [](C *c, In in, Value &o) { futhark_f32_3d *r = nullptr; int rc = futhark_entry_transpose_f32_3d(c, &r, FE_IN(0, f32_3d)); if (!rc) set_array(o, "[][][]f32", r); return rc; }},
      FE_E1(scan_max_i32, i32_1d, "[]i32", i32_1d, "[]i32"),
      FE_E1(scan_i64, i64_1d, "[]i64", i64_1d, "[]i64"),
      FE_E1(scanomap_steps_i32, i32_1d, "[]i32", i32_1d, "[]i32"),
      FE_E1(segscan_rows_i32, i32_2d, "[][]i32", i32_2d, "[][]i32"),
      FE_E1(scan_map2_add_i32, i32_2d, "[][]i32", i32_2d, "[][]i32"),
      FE_E1(filter_pos_i32, i32_1d, "[]i32", i32_1d, "[]i32"),
      FE_E1(transpose_f16_3d, f16_3d, "[][][]f16", f16_3d, "[][][]f16"),
      FE_E1(transpose_i64, i64_2d, "[][]i64", i64_2d, "[][]i64"),
      FE_E1(transpose_bool, bool_2d, "[][]bool", bool_2d, "[][]bool"),
      FE_E2(linrec_f32, f32_1d, "[]f32", f32_1d, "[]f32", f32_1d, "[]f32"),
      FE_E2(filter_by_flag_i32, i32_1d, "[]i32", bool_1d, "[]bool", i32_1d, "[]i32"),
      FE_EH(hist_and_i32, i32_1d, "[]i32", i32_1d, "[]i32", i32_1d, "[]i32"),
      FE_EH(hist_or_i32, i32_1d, "[]i32", i32_1d, "[]i32", i32_1d, "[]i32"),
      FE_EH(hist_xor_i32, i32_1d, "[]i32", i32_1d, "[]i32", i32_1d, "[]i32"),
      FE_EH(hist_mul_i32, i32_1d, "[]i32", i32_1d, "[]i32", i32_1d, "[]i32"),
      FE_EH(hist_rows_add_i32, i32_2d, "[][]i32", i32_2d, "[][]i32", i32_2d, "[][]i32"),
      FE_E3(reduce_by_index_min_i32, i32_1d, "[]i32", i32_1d, "[]i32", i32_1d, "[]i32", i32_1d, "[]i32"),
      FE_E3(reduce_by_index_max_i32, i32_1d, "[]i32", i32_1d, "[]i32", i32_1d, "[]i32", i32_1d, "[]i32"),
      FE_E3(reduce_by_index_min_u32, u32_1d, "[]u32", i32_1d, "[]i32", u32_1d, "[]u32", u32_1d, "[]u32"),
      FE_E3(reduce_by_index_max_u32, u32_1d, "[]u32", i32_1d, "[]i32", u32_1d, "[]u32", u32_1d, "[]u32"),
      FE_E3(reduce_by_index_add_f32, f32_1d, "[]f32", i32_1d, "[]i32", f32_1d, "[]f32", f32_1d, "[]f32"),
      FE_E3(reduce_by_index_add_f64, f64_1d, "[]f64", i32_1d, "[]i32", f64_1d, "[]f64", f64_1d, "[]f64"),
      FE_E3(reduce_by_index_add_i8, i8_1d, "[]i8", i8_1d, "[]i8", i8_1d, "[]i8", i8_1d, "[]i8"),
      FE_EH(hist_or_bool, i32_1d, "[]i32", bool_1d, "[]bool", bool_1d, "[]bool"),
      FE_EH(hist_and_i8, i32_1d, "[]i32", i8_1d, "[]i8", i8_1d, "[]i8"),
      FE_EH(hist_and_i16, i32_1d, "[]i32", i16_1d, "[]i16", i16_1d, "[]i16"),
      FE_EH(hist_and_i64, i32_1d, "[]i32", i32_1d, "[]i32", i64_1d, "[]i64"),
      FE_EH(hist_or_i8, i32_1d, "[]i32", i8_1d, "[]i8", i8_1d, "[]i8"),
      FE_EH(hist_or_i16, i32_1d, "[]i32", i16_1d, "[]i16", i16_1d, "[]i16"),
      FE_EH(hist_or_i64, i32_1d, "[]i32", i32_1d, "[]i32", i64_1d, "[]i64"),
      FE_EH(hist_xor_i8, i32_1d, "[]i32", i8_1d, "[]i8", i8_1d, "[]i8"),
      FE_EH(hist_xor_i16, i32_1d, "[]i32", i16_1d, "[]i16", i16_1d, "[]i16"),
      FE_EH(hist_xor_i64, i32_1d, "[]i32", i32_1d, "[]i32", i64_1d, "[]i64"),
      FE_E3(reduce_by_index_min_i8, i8_1d, "[]i8", i32_1d, "[]i32", i8_1d, "[]i8", i8_1d, "[]i8"),
      FE_E3(reduce_by_index_min_u8, u8_1d, "[]u8", i32_1d, "[]i32", u8_1d, "[]u8", u8_1d, "[]u8"),
      FE_E3(reduce_by_index_min_i16, i16_1d, "[]i16", i32_1d, "[]i32", i16_1d, "[]i16", i16_1d, "[]i16"),
      FE_E3(reduce_by_index_min_u16, u16_1d, "[]u16", i32_1d, "[]i32", u16_1d, "[]u16", u16_1d, "[]u16"),
      FE_E3(reduce_by_index_max_i8, i8_1d, "[]i8", i32_1d, "[]i32", i8_1d, "[]i8", i8_1d, "[]i8"),
      FE_E3(reduce_by_index_max_u8, u8_1d, "[]u8", i32_1d, "[]i32", u8_1d, "[]u8", u8_1d, "[]u8"),
      FE_E3(reduce_by_index_max_i16, i16_1d, "[]i16", i32_1d, "[]i32", i16_1d, "[]i16", i16_1d, "[]i16"),
      FE_E3(reduce_by_index_max_u16, u16_1d, "[]u16", i32_1d, "[]i32", u16_1d, "[]u16", u16_1d, "[]u16"),
      FE_E3(reduce_by_index_add_i16, i16_1d, "[]i16", i16_1d, "[]i16", i16_1d, "[]i16", i16_1d, "[]i16"),
      FE_E3(reduce_by_index_add_f16, f16_1d, "[]f16", i16_1d, "[]i16", f16_1d, "[]f16", f16_1d, "[]f16"),
      {"reduce_by_index_2d_add_i32", {"[][]i32", "[]i64", "[]i64", "[]i32"}, "[][]i32", [](C *c, In in, Value &o) { futhark_i32_2d *r = nullptr; int rc = futhark_entry_reduce_by_index_2d_add_i32(c, &r, FE_IN(0, i32_2d), FE_IN(1, i64_1d), FE_IN(2, i64_1d), FE_IN(3, i32_1d)); if (!rc) set_array(o, "[][]i32", r); return rc; }},
      {"reduce_by_index_3d_add_i32", {"[][][]i32", "[]i64", "[]i64", "[]i64", "[]i32"}, "[][][]i32", [](C *c, In in, Value &o) { futhark_i32_3d *r = nullptr; int rc = futhark_entry_reduce_by_index_3d_add_i32(c, &r, FE_IN(0, i32_3d), FE_IN(1, i64_1d), FE_IN(2, i64_1d), FE_IN(3, i64_1d), FE_IN(4, i32_1d)); if (!rc) set_array(o, "[][][]i32", r); return rc; }},
      {"hist_rows_2d_add_i32", {"i64", "i64", "[][]i32", "[][]i32"}, "[][][]i32", [](C *c, In in, Value &o) { futhark_i32_3d *r = nullptr; int rc = futhark_entry_hist_rows_2d_add_i32(c, &r, scalar_of<int64_t>(*in[0]), scalar_of<int64_t>(*in[1]), FE_IN(2, i32_2d), FE_IN(3, i32_2d)); if (!rc) set_array(o, "[][][]i32", r); return rc; }},
      {"partition2_i32", {"[]i32"}, "([]i32, []i32, []i32)", [](C *c, In in, Value &o) { futhark_opaque_tup3_arr1d_i32_arr1d_i32_arr1d_i32 *r = nullptr; int rc = futhark_entry_partition2_i32(c, &r, FE_IN(0, i32_1d)); if (!rc) set_record(o, "([]i32, []i32, []i32)", r); return rc; }},
      {"segredomap_sum_neg_f32", {"[][]f32"}, "([]i64, [][]f64)", [](C *c, In in, Value &o) { futhark_opaque_tup2_arr1d_i64_arr2d_f64 *r = nullptr; int rc = futhark_entry_segredomap_sum_neg_f32(c, &r, FE_IN(0, f32_2d)); if (!rc) set_record(o, "([]i64, [][]f64)", r); return rc; }},
      FE_E1(reduce_map2_add_i32, i32_2d, "[][]i32", i32_1d, "[]i32"),
      FE_E3(reduce_by_index_vec_add_i32, i32_2d, "[][]i32", i64_1d, "[]i64", i32_2d, "[][]i32", i32_2d, "[][]i32"),
      {"hist_rows_vec_add_i32", {"i64", "[][]i32", "[][][]i32"}, "[][][]i32", [](C *c, In in, Value &o) { futhark_i32_3d *r = nullptr; int rc = futhark_entry_hist_rows_vec_add_i32(c, &r, scalar_of<int64_t>(*in[0]), FE_IN(1, i32_2d), FE_IN(2, i32_3d)); if (!rc) set_array(o, "[][][]i32", r); return rc; }},
      {"reduce_by_index_minpair_i32", {"i64", "[]i32", "[]i32", "[]i32"}, "([]i32, []i32)", [](C *c, In in, Value &o) { futhark_opaque_tup2_arr1d_i32_arr1d_i32 *r = nullptr; int rc = futhark_entry_reduce_by_index_minpair_i32(c, &r, scalar_of<int64_t>(*in[0]), FE_IN(1, i32_1d), FE_IN(2, i32_1d), FE_IN(3, i32_1d)); if (!rc) set_record(o, "([]i32, []i32)", r); return rc; }},
      {"partition2_pairs_i32", {"[]i32", "[]i32"}, "([]i32, []i32, []i32, []i32, []i32, []i32)", [](C *c, In in, Value &o) { futhark_opaque_tup6_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32 *r = nullptr; int rc = futhark_entry_partition2_pairs_i32(c, &r, FE_IN(0, i32_1d), FE_IN(1, i32_1d)); if (!rc) set_record(o, "([]i32, []i32, []i32, []i32, []i32, []i32)", r); return rc; }},
      {"replicate_i32", {"i64", "i32"}, "[]i32", [](C *c, In in, Value &o) { futhark_i32_1d *r = nullptr; int rc = futhark_entry_replicate_i32(c, &r, scalar_of<int64_t>(*in[0]), scalar_of<int32_t>(*in[1])); if (!rc) set_array(o, "[]i32", r); return rc; }},
      {"iota_i64", {"i64"}, "[]i64", [](C *c, In in, Value &o) { futhark_i64_1d *r = nullptr; int rc = futhark_entry_iota_i64(c, &r, scalar_of<int64_t>(*in[0])); if (!rc) set_array(o, "[]i64", r); return rc; }},
  };
  return table;
}

inline const EntryPoint *entry_point(const std::string &name) {
  for (const EntryPoint &e : entry_points())
    if (name == e.name) return &e;
  return nullptr;
}

}  // namespace fe
