// The executable front-end: what `futhark cuda` (without --library) wraps around a program's
// entry points, for the entry points of libfuthark_b200.so.  It follows the generated main() of
// src/Futhark/CodeGen/Backends/GenericC/CLI.hs:28-470: the same options, input values read from
// standard input (text or binary, one per parameter, then end of input), an optional warm-up run
// and `-r` timed runs with the wall time of each (entry point + sync, in microseconds) written
// to the `-t` file, and the result of the last run printed to standard output in text or (`-b`)
// binary form, one value per line.  `futhark test` and `futhark bench` drive compiled programs
// through exactly this interface.
//
// Plain C++ on the library's C ABI; no CUDA code here.
#include <errno.h>
#include <getopt.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/time.h>

#include <functional>
#include <memory>
#include <string>
#include <vector>

#define FUTHARK_B200_NO_CUDA_H
#include "../../include/futhark_b200.h"

static void panic(int code, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vfprintf(stderr, fmt, ap);
  va_end(ap);
  exit(code);
}

static int64_t wall_usec() {
  struct timeval t;
  gettimeofday(&t, nullptr);
  return (int64_t)t.tv_sec * 1000000 + t.tv_usec;
}

typedef futhark_b200_value Val;

struct Param { const char *type; int rank; };

// One entry point: its parameter and result types as the manifest would list them, and a
// runner that packs host values into arrays, calls the entry and unpacks the results.
struct Entry {
  const char *name;
  std::vector<Param> ins, outs;
  // uploads happen in `pack`, outside the timed region, as in the generated code
  std::function<void(futhark_context *, const std::vector<Val> &)> pack;
  std::function<int(futhark_context *)> run;                       // the timed call
  std::function<void(futhark_context *, std::vector<Val> &)> fetch;  // results to host values
  std::function<void(futhark_context *)> free_outputs, free_inputs;
};

static void check(futhark_context *ctx, int rc) {
  if (rc != 0) {
    char *e = futhark_context_get_error(ctx);
    panic(1, "%s", e ? e : "unknown error\n");
  }
}

static Val host_val(const char *type, int rank, const int64_t *shape, size_t elem) {
  Val v;
  memset(&v, 0, sizeof(v));
  snprintf(v.type, sizeof(v.type), "%s", type);
  v.rank = rank;
  size_t n = 1;
  for (int d = 0; d < rank; d++) { v.shape[d] = shape[d]; n *= (size_t)shape[d]; }
  v.data = calloc(n ? n : 1, elem);
  return v;
}

// ---- array plumbing per array type of the API -----------------------------------------------------
#define ARR1(T, CT, NAME)                                                                                          \
  static futhark_##T##_1d *up_##T##_1d(futhark_context *c, const Val &v) {                                         \
    futhark_##T##_1d *a = futhark_new_##T##_1d(c, (const CT *)v.data, v.shape[0]);                                  \
    if (a == nullptr) check(c, 1);                                                                                 \
    return a;                                                                                                      \
  }                                                                                                                \
  [[maybe_unused]] static Val down_##T##_1d(futhark_context *c, futhark_##T##_1d *a) {                                            \
    Val v = host_val(NAME, 1, futhark_shape_##T##_1d(c, a), sizeof(CT));                                            \
    check(c, futhark_values_##T##_1d(c, a, (CT *)v.data));                                                         \
    return v;                                                                                                      \
  }
ARR1(i32, int32_t, "i32")
ARR1(i64, int64_t, "i64")
ARR1(u32, uint32_t, "u32")
ARR1(f32, float, "f32")
ARR1(bool, bool, "bool")

static futhark_f32_2d *up_f32_2d(futhark_context *c, const Val &v) {
  futhark_f32_2d *a = futhark_new_f32_2d(c, (const float *)v.data, v.shape[0], v.shape[1]);
  if (a == nullptr) check(c, 1);
  return a;
}
static Val down_f32_2d(futhark_context *c, futhark_f32_2d *a) {
  Val v = host_val("f32", 2, futhark_shape_f32_2d(c, a), 4);
  check(c, futhark_values_f32_2d(c, a, (float *)v.data));
  return v;
}
static futhark_f32_3d *up_f32_3d(futhark_context *c, const Val &v) {
  futhark_f32_3d *a = futhark_new_f32_3d(c, (const float *)v.data, v.shape[0], v.shape[1], v.shape[2]);
  if (a == nullptr) check(c, 1);
  return a;
}
static Val down_f32_3d(futhark_context *c, futhark_f32_3d *a) {
  Val v = host_val("f32", 3, futhark_shape_f32_3d(c, a), 4);
  check(c, futhark_values_f32_3d(c, a, (float *)v.data));
  return v;
}
static futhark_f16_3d *up_f16_3d(futhark_context *c, const Val &v) {
  futhark_f16_3d *a = futhark_new_f16_3d(c, (const uint16_t *)v.data, v.shape[0], v.shape[1], v.shape[2]);
  if (a == nullptr) check(c, 1);
  return a;
}

static Val scalar_val(const char *type, const void *src, size_t elem) {
  Val v = host_val(type, 0, nullptr, 8);
  memcpy(v.data, src, elem);
  return v;
}

// ---- the entry points ------------------------------------------------------------------------------
// array in -> array out, same element type and rank 1
template <typename A, typename UP, typename DOWN, typename FREE, typename CALL>
static Entry map1(const char *name, const char *t, UP up, DOWN down, FREE fr, CALL call) {
  struct St { A *in = nullptr, *out = nullptr; };
  auto st = std::make_shared<St>();
  Entry e;
  e.name = name;
  e.ins = {{t, 1}};
  e.outs = {{t, 1}};
  e.pack = [=](futhark_context *c, const std::vector<Val> &v) { st->in = up(c, v[0]); };
  e.run = [=](futhark_context *c) { return call(c, &st->out, st->in); };
  e.fetch = [=](futhark_context *c, std::vector<Val> &o) { o.push_back(down(c, st->out)); };
  e.free_outputs = [=](futhark_context *c) { if (st->out) { fr(c, st->out); st->out = nullptr; } };
  e.free_inputs = [=](futhark_context *c) { if (st->in) { fr(c, st->in); st->in = nullptr; } };
  return e;
}

static std::vector<Entry> make_entries() {
  std::vector<Entry> es;
  es.push_back(map1<futhark_i32_1d>("scan_i32", "i32", up_i32_1d, down_i32_1d, futhark_free_i32_1d, futhark_entry_scan_i32));
  es.push_back(map1<futhark_i32_1d>("exscan_i32", "i32", up_i32_1d, down_i32_1d, futhark_free_i32_1d, futhark_entry_exscan_i32));
  es.push_back(map1<futhark_u32_1d>("filter_u32", "u32", up_u32_1d, down_u32_1d, futhark_free_u32_1d, futhark_entry_filter_u32));

  {  // i32 array -> i32 scalar
    struct St { futhark_i32_1d *in = nullptr; int32_t out = 0; };
    for (int which = 0; which < 2; which++) {
      auto st = std::make_shared<St>();
      Entry e;
      e.name = which == 0 ? "reduce_i32" : "mss_i32";
      e.ins = {{"i32", 1}};
      e.outs = {{"i32", 0}};
      e.pack = [=](futhark_context *c, const std::vector<Val> &v) { st->in = up_i32_1d(c, v[0]); };
      e.run = [=](futhark_context *c) { return which == 0 ? futhark_entry_reduce_i32(c, &st->out, st->in) : futhark_entry_mss_i32(c, &st->out, st->in); };
      e.fetch = [=](futhark_context *, std::vector<Val> &o) { o.push_back(scalar_val("i32", &st->out, 4)); };
      e.free_outputs = [](futhark_context *) {};
      e.free_inputs = [=](futhark_context *c) { if (st->in) { futhark_free_i32_1d(c, st->in); st->in = nullptr; } };
      es.push_back(e);
    }
  }
  {  // i32 array -> (i32, f32)
    struct St { futhark_i32_1d *in = nullptr; int32_t o0 = 0; float o1 = 0; };
    auto st = std::make_shared<St>();
    Entry e;
    e.name = "sum_i32_f32";
    e.ins = {{"i32", 1}};
    e.outs = {{"i32", 0}, {"f32", 0}};
    e.pack = [=](futhark_context *c, const std::vector<Val> &v) { st->in = up_i32_1d(c, v[0]); };
    e.run = [=](futhark_context *c) { return futhark_entry_sum_i32_f32(c, &st->o0, &st->o1, st->in); };
    e.fetch = [=](futhark_context *, std::vector<Val> &o) { o.push_back(scalar_val("i32", &st->o0, 4)); o.push_back(scalar_val("f32", &st->o1, 4)); };
    e.free_outputs = [](futhark_context *) {};
    e.free_inputs = [=](futhark_context *c) { if (st->in) { futhark_free_i32_1d(c, st->in); st->in = nullptr; } };
    es.push_back(e);
  }
  {  // (flags, xs) -> f32 array
    struct St { futhark_bool_1d *f = nullptr; futhark_f32_1d *x = nullptr, *out = nullptr; };
    auto st = std::make_shared<St>();
    Entry e;
    e.name = "segscan_f32";
    e.ins = {{"bool", 1}, {"f32", 1}};
    e.outs = {{"f32", 1}};
    e.pack = [=](futhark_context *c, const std::vector<Val> &v) { st->f = up_bool_1d(c, v[0]); st->x = up_f32_1d(c, v[1]); };
    e.run = [=](futhark_context *c) { return futhark_entry_segscan_f32(c, &st->out, st->f, st->x); };
    e.fetch = [=](futhark_context *c, std::vector<Val> &o) { o.push_back(down_f32_1d(c, st->out)); };
    e.free_outputs = [=](futhark_context *c) { if (st->out) { futhark_free_f32_1d(c, st->out); st->out = nullptr; } };
    e.free_inputs = [=](futhark_context *c) {
      if (st->f) { futhark_free_bool_1d(c, st->f); st->f = nullptr; }
      if (st->x) { futhark_free_f32_1d(c, st->x); st->x = nullptr; }
    };
    es.push_back(e);
  }
  {  // (offsets, flags, xs) -> f32 array
    struct St { futhark_i64_1d *o = nullptr; futhark_bool_1d *f = nullptr; futhark_f32_1d *x = nullptr, *out = nullptr; };
    auto st = std::make_shared<St>();
    Entry e;
    e.name = "segreduce_f32";
    e.ins = {{"i64", 1}, {"bool", 1}, {"f32", 1}};
    e.outs = {{"f32", 1}};
    e.pack = [=](futhark_context *c, const std::vector<Val> &v) { st->o = up_i64_1d(c, v[0]); st->f = up_bool_1d(c, v[1]); st->x = up_f32_1d(c, v[2]); };
    e.run = [=](futhark_context *c) { return futhark_entry_segreduce_f32(c, &st->out, st->o, st->f, st->x); };
    e.fetch = [=](futhark_context *c, std::vector<Val> &o) { o.push_back(down_f32_1d(c, st->out)); };
    e.free_outputs = [=](futhark_context *c) { if (st->out) { futhark_free_f32_1d(c, st->out); st->out = nullptr; } };
    e.free_inputs = [=](futhark_context *c) {
      if (st->o) { futhark_free_i64_1d(c, st->o); st->o = nullptr; }
      if (st->f) { futhark_free_bool_1d(c, st->f); st->f = nullptr; }
      if (st->x) { futhark_free_f32_1d(c, st->x); st->x = nullptr; }
    };
    es.push_back(e);
  }
  {  // [][]f32 -> []f32 and [][]f32 -> [][]f32
    struct St { futhark_f32_2d *in = nullptr, *out2 = nullptr; futhark_f32_1d *out1 = nullptr; };
    for (int which = 0; which < 2; which++) {
      auto st = std::make_shared<St>();
      Entry e;
      e.name = which == 0 ? "rowsum_f32" : "transpose_f32";
      e.ins = {{"f32", 2}};
      e.outs = {{"f32", which == 0 ? 1 : 2}};
      e.pack = [=](futhark_context *c, const std::vector<Val> &v) { st->in = up_f32_2d(c, v[0]); };
      e.run = [=](futhark_context *c) { return which == 0 ? futhark_entry_rowsum_f32(c, &st->out1, st->in) : futhark_entry_transpose_f32(c, &st->out2, st->in); };
      e.fetch = [=](futhark_context *c, std::vector<Val> &o) { o.push_back(which == 0 ? down_f32_1d(c, st->out1) : down_f32_2d(c, st->out2)); };
      e.free_outputs = [=](futhark_context *c) {
        if (st->out1) { futhark_free_f32_1d(c, st->out1); st->out1 = nullptr; }
        if (st->out2) { futhark_free_f32_2d(c, st->out2); st->out2 = nullptr; }
      };
      e.free_inputs = [=](futhark_context *c) { if (st->in) { futhark_free_f32_2d(c, st->in); st->in = nullptr; } };
      es.push_back(e);
    }
  }
  {  // [][][]f32 -> [][][]f32
    struct St { futhark_f32_3d *in = nullptr, *out = nullptr; };
    auto st = std::make_shared<St>();
    Entry e;
    e.name = "transpose_f32_3d";
    e.ins = {{"f32", 3}};
    e.outs = {{"f32", 3}};
    e.pack = [=](futhark_context *c, const std::vector<Val> &v) { st->in = up_f32_3d(c, v[0]); };
    e.run = [=](futhark_context *c) { return futhark_entry_transpose_f32_3d(c, &st->out, st->in); };
    e.fetch = [=](futhark_context *c, std::vector<Val> &o) { o.push_back(down_f32_3d(c, st->out)); };
    e.free_outputs = [=](futhark_context *c) { if (st->out) { futhark_free_f32_3d(c, st->out); st->out = nullptr; } };
    e.free_inputs = [=](futhark_context *c) { if (st->in) { futhark_free_f32_3d(c, st->in); st->in = nullptr; } };
    es.push_back(e);
  }
  {  // (B, is, ws) -> histogram
    struct St { int64_t B = 0; futhark_i32_1d *is = nullptr, *wi = nullptr, *oi = nullptr; futhark_f32_1d *wf = nullptr, *of = nullptr; };
    for (int which = 0; which < 2; which++) {
      auto st = std::make_shared<St>();
      Entry e;
      e.name = which == 0 ? "hist_add_i32" : "hist_max_f32";
      e.ins = {{"i64", 0}, {"i32", 1}, {which == 0 ? "i32" : "f32", 1}};
      e.outs = {{which == 0 ? "i32" : "f32", 1}};
      e.pack = [=](futhark_context *c, const std::vector<Val> &v) {
        st->B = *(const int64_t *)v[0].data;
        st->is = up_i32_1d(c, v[1]);
        if (which == 0) st->wi = up_i32_1d(c, v[2]); else st->wf = up_f32_1d(c, v[2]);
      };
      e.run = [=](futhark_context *c) {
        return which == 0 ? futhark_entry_hist_add_i32(c, &st->oi, st->B, st->is, st->wi) : futhark_entry_hist_max_f32(c, &st->of, st->B, st->is, st->wf);
      };
      e.fetch = [=](futhark_context *c, std::vector<Val> &o) { o.push_back(which == 0 ? down_i32_1d(c, st->oi) : down_f32_1d(c, st->of)); };
      e.free_outputs = [=](futhark_context *c) {
        if (st->oi) { futhark_free_i32_1d(c, st->oi); st->oi = nullptr; }
        if (st->of) { futhark_free_f32_1d(c, st->of); st->of = nullptr; }
      };
      e.free_inputs = [=](futhark_context *c) {
        if (st->is) { futhark_free_i32_1d(c, st->is); st->is = nullptr; }
        if (st->wi) { futhark_free_i32_1d(c, st->wi); st->wi = nullptr; }
        if (st->wf) { futhark_free_f32_1d(c, st->wf); st->wf = nullptr; }
      };
      es.push_back(e);
    }
  }
  {  // []u32 -> ([]u32, []u32): the tuple's fields are printed one per line (CLI.hs:279-296)
    struct St { futhark_u32_1d *in = nullptr; futhark_opaque_tup2_arr1d_u32_arr1d_u32 *out = nullptr; };
    auto st = std::make_shared<St>();
    Entry e;
    e.name = "partition_u32";
    e.ins = {{"u32", 1}};
    e.outs = {{"u32", 1}, {"u32", 1}};
    e.pack = [=](futhark_context *c, const std::vector<Val> &v) { st->in = up_u32_1d(c, v[0]); };
    e.run = [=](futhark_context *c) { return futhark_entry_partition_u32(c, &st->out, st->in); };
    e.fetch = [=](futhark_context *c, std::vector<Val> &o) {
      futhark_u32_1d *a = nullptr, *b = nullptr;
      check(c, futhark_project_opaque_tup2_arr1d_u32_arr1d_u32_0(c, &a, st->out));
      check(c, futhark_project_opaque_tup2_arr1d_u32_arr1d_u32_1(c, &b, st->out));
      o.push_back(down_u32_1d(c, a));
      o.push_back(down_u32_1d(c, b));
      futhark_free_u32_1d(c, a);
      futhark_free_u32_1d(c, b);
    };
    e.free_outputs = [=](futhark_context *c) { if (st->out) { futhark_free_opaque_tup2_arr1d_u32_arr1d_u32(c, st->out); st->out = nullptr; } };
    e.free_inputs = [=](futhark_context *c) { if (st->in) { futhark_free_u32_1d(c, st->in); st->in = nullptr; } };
    es.push_back(e);
  }
  {  // ([b][m][k]f16, [b][k][n]f16) -> [b][m][n]f32
    struct St { futhark_f16_3d *a = nullptr, *b = nullptr; futhark_f32_3d *out = nullptr; };
    auto st = std::make_shared<St>();
    Entry e;
    e.name = "bmm_f16";
    e.ins = {{"f16", 3}, {"f16", 3}};
    e.outs = {{"f32", 3}};
    e.pack = [=](futhark_context *c, const std::vector<Val> &v) { st->a = up_f16_3d(c, v[0]); st->b = up_f16_3d(c, v[1]); };
    e.run = [=](futhark_context *c) { return futhark_entry_bmm_f16(c, &st->out, st->a, st->b); };
    e.fetch = [=](futhark_context *c, std::vector<Val> &o) { o.push_back(down_f32_3d(c, st->out)); };
    e.free_outputs = [=](futhark_context *c) { if (st->out) { futhark_free_f32_3d(c, st->out); st->out = nullptr; } };
    e.free_inputs = [=](futhark_context *c) {
      if (st->a) { futhark_free_f16_3d(c, st->a); st->a = nullptr; }
      if (st->b) { futhark_free_f16_3d(c, st->b); st->b = nullptr; }
    };
    es.push_back(e);
  }
  return es;
}

static const char *USAGE =
    "  -t/--write-runtime-to FILE Print the time taken to execute the program to the indicated file, an integral number of microseconds.\n"
    "  -r/--runs INT              Perform NUM runs of the program.\n"
    "  -D/--debugging             Perform possibly expensive internal correctness checks and verbose logging.\n"
    "  -L/--log                   Print various low-overhead logging information to stderr while running.\n"
    "  -P/--profile               Enable the collection of profiling information.\n"
    "  -e/--entry-point NAME      The entry point to run.\n"
    "  -b/--binary-output         Print the program result in the binary output format.\n"
    "  -n/--no-print-result       Do not print the program result.\n"
    "  -h/--help                  Print help information and exit.\n"
    "  --print-params             Print all tuning parameters that can be set with --param or --tuning.\n"
    "  --param ASSIGNMENT         Set a tuning parameter to the given value.\n"
    "  --tuning FILE              Read size=value assignments from the given file.\n"
    "  --cache-file FILE          Store program cache here.\n"
    "  -d/--device NAME           Use the first device whose name contains the given string.\n"
    "  --list-entry-points        Print the entry points with their parameter and result types and exit.\n";

int main(int argc, char **argv) {
  std::vector<Entry> entries = make_entries();
  futhark_context_config *cfg = futhark_context_config_new();
  const char *entry_point = "main";
  const char *runtime_path = nullptr;
  int num_runs = 1, perform_warmup = 0, binary_output = 0, print_result = 1, profile = 0;
  static struct option longopts[] = {
      {"write-runtime-to", required_argument, nullptr, 't'}, {"runs", required_argument, nullptr, 'r'},
      {"debugging", no_argument, nullptr, 'D'},              {"log", no_argument, nullptr, 'L'},
      {"profile", no_argument, nullptr, 'P'},                {"entry-point", required_argument, nullptr, 'e'},
      {"binary-output", no_argument, nullptr, 'b'},          {"no-print-result", no_argument, nullptr, 'n'},
      {"help", no_argument, nullptr, 'h'},                   {"print-params", no_argument, nullptr, 1},
      {"param", required_argument, nullptr, 2},              {"tuning", required_argument, nullptr, 3},
      {"cache-file", required_argument, nullptr, 4},         {"device", required_argument, nullptr, 'd'},
      {"list-entry-points", no_argument, nullptr, 5},        {nullptr, 0, nullptr, 0}};
  int ch;
  while ((ch = getopt_long(argc, argv, ":t:r:DLPe:bnhd:", longopts, nullptr)) != -1) {
    switch (ch) {
      case 't': runtime_path = optarg; break;
      case 'r':
        num_runs = atoi(optarg);
        perform_warmup = 1;
        if (num_runs <= 0) panic(1, "Need a positive number of runs, not %s\n", optarg);
        break;
      case 'D': futhark_context_config_set_debugging(cfg, 1); break;
      case 'L': futhark_context_config_set_logging(cfg, 1); break;
      case 'P': futhark_context_config_set_profiling(cfg, 1); profile = 1; break;
      case 'e': entry_point = optarg; break;
      case 'b': binary_output = 1; break;
      case 'n': print_result = 0; break;
      case 'd': futhark_context_config_set_device(cfg, optarg); break;
      case 'h': printf("Usage: %s [OPTION]...\nOptions:\n\n%s\nFor more information, consult the Futhark User's Guide or the man pages.\n", argv[0], USAGE); return 0;
      case 1:
        for (int i = 0; i < futhark_get_tuning_param_count(); i++) printf("%s (%s)\n", futhark_get_tuning_param_name(i), futhark_get_tuning_param_class(i));
        return 0;
      case 2: {
        char *eq = strstr(optarg, "=");
        if (eq == nullptr) panic(1, "Invalid argument for --parameter option: %s\n", optarg);
        *eq = 0;
        if (futhark_context_config_set_tuning_param(cfg, optarg, (size_t)atoi(eq + 1)) != 0) panic(1, "Unknown tuning parameter: %s\n", optarg);
        break;
      }
      case 3: {  // lines of name=value (rts/c/tuning.h)
        FILE *f = fopen(optarg, "r");
        if (f == nullptr) panic(1, "When loading tuning file '%s': cannot open file\n", optarg);
        char line[512];
        while (fgets(line, sizeof(line), f)) {
          char *eq = strstr(line, "=");
          if (eq == nullptr) continue;
          *eq = 0;
          if (futhark_context_config_set_tuning_param(cfg, line, (size_t)atoi(eq + 1)) != 0)
            panic(1, "When loading tuning file '%s': Unknown name '%s'\n", optarg, line);
        }
        fclose(f);
        break;
      }
      case 4: futhark_context_config_set_cache_file(cfg, optarg); break;
      case 5:
        for (const Entry &e : entries) {
          printf("%s:", e.name);
          for (const Param &p : e.ins) { printf(" "); for (int d = 0; d < p.rank; d++) printf("[]"); printf("%s", p.type); }
          printf(" ->");
          for (const Param &p : e.outs) { printf(" "); for (int d = 0; d < p.rank; d++) printf("[]"); printf("%s", p.type); }
          printf("\n");
        }
        return 0;
      case ':': panic(-1, "Missing argument for option %s\n", argv[optind - 1]);
      default: panic(-1, "Unknown option: %s\n", argv[optind - 1]);
    }
  }
  if (optind != argc) panic(1, "Excess non-option: %s\n", argv[optind]);

  const Entry *entry = nullptr;
  for (const Entry &e : entries)
    if (strcmp(e.name, entry_point) == 0) entry = &e;
  if (entry == nullptr) {
    fprintf(stderr, "No entry point '%s'.  Select another with --entry-point.  Options are:\n", entry_point);
    for (const Entry &e : entries) fprintf(stderr, "%s\n", e.name);
    return 1;
  }

  FILE *runtime_file = nullptr;
  if (runtime_path != nullptr) {
    runtime_file = fopen(runtime_path, "w");
    if (runtime_file == nullptr) panic(1, "Cannot open %s: %s\n", runtime_path, strerror(errno));
  }

  futhark_context *ctx = futhark_context_new(cfg);
  {
    char *err = futhark_context_get_error(ctx);
    if (err != nullptr) panic(1, "Error during context initialisation:\n%s", err);
  }
  futhark_context_pause_profiling(ctx);       // initialisation is not profiled (CLI.hs:385-386)

  // read the arguments, then insist on the end of the input (CLI.hs:388-394)
  std::vector<Val> inputs(entry->ins.size());
  for (size_t i = 0; i < entry->ins.size(); i++) {
    if (futhark_b200_value_read(stdin, entry->ins[i].type, entry->ins[i].rank, &inputs[i]) != 0) {
      std::string t;
      for (int d = 0; d < entry->ins[i].rank; d++) t += "[]";
      panic(1, "Error when reading input #%d of type %s%s (errno: %s).\n%s\n", (int)i, t.c_str(), entry->ins[i].type, strerror(errno),
            futhark_b200_value_error());
    }
  }
  if (futhark_b200_value_end_of_input(stdin) != 0) panic(1, "Expected EOF on stdin after reading input for \"%s\".\n", entry->name);

  auto run_once = [&](bool timed, bool profiled) {
    entry->pack(ctx, inputs);
    check(ctx, futhark_context_sync(ctx));
    if (profiled) futhark_context_unpause_profiling(ctx);
    const int64_t t0 = wall_usec();
    check(ctx, entry->run(ctx));
    check(ctx, futhark_context_sync(ctx));
    if (profiled) futhark_context_pause_profiling(ctx);
    const int64_t t1 = wall_usec();
    if (timed && runtime_file != nullptr) {
      fprintf(runtime_file, "%lld\n", (long long)(t1 - t0));
      fflush(runtime_file);
    }
    entry->free_inputs(ctx);
  };
  if (perform_warmup) {
    run_once(false, false);
    entry->free_outputs(ctx);
  }
  for (int run = 0; run < num_runs; run++) {
    run_once(true, run == num_runs - 1);       // only the last run is profiled
    if (run < num_runs - 1) entry->free_outputs(ctx);
  }
  for (Val &v : inputs) futhark_b200_value_free(&v);

  if (print_result) {
    std::vector<Val> outs;
    entry->fetch(ctx, outs);
    check(ctx, futhark_context_sync(ctx));
    for (Val &v : outs) {
      futhark_b200_value_write(stdout, &v, binary_output);
      puts("");
      futhark_b200_value_free(&v);
    }
  }
  entry->free_outputs(ctx);
  if (runtime_file != nullptr) fclose(runtime_file);
  if (profile) {
    char *report = futhark_context_report(ctx);
    fputs(report, stderr);
    free(report);
  }
  futhark_context_free(ctx);
  futhark_context_config_free(cfg);
  return 0;
}
