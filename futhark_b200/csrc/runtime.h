// Internal definitions of the host runtime behind the C API: configuration,
// context, device memory pool, reference-counted memory blocks, array objects,
// launch records for the profiling report.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/futhark_b200.h"

// ---- tuning parameters (names and classes are enumerable through the API) --------------
struct TuningParam {
  const char *name;
  const char *klass;
  int64_t def;
};
extern const TuningParam kTuningParams[];
extern const int kNumTuningParams;

struct futhark_context_config {
  int in_use = 0;
  int debugging = 0, profiling = 0, logging = 0;
  int unified_memory = 0;
  std::string cache_fname;
  std::string device;          // "" = best device, "#k" = index, else name substring
  std::string program;         // kept only so get_program/set_program round-trip
  std::vector<std::string> nvrtc_options;
  std::string dump_ptx_to, load_ptx_from;
  int64_t default_block_size = 256, default_grid_size = 0, default_tile_size = 32,
          default_reg_tile_size = 2, default_registers = 0, default_cache = 0, default_threshold = 32768;
  std::vector<int64_t> tuning;  // one value per kTuningParams entry
};

// A reference-counted block of device memory; the same four fields as the struct the
// reference generates for its arrays (GenericC.hs:155-266).
struct memblock_device {
  int *references;     // NULL for borrowed (raw) memory
  CUdeviceptr mem;
  int64_t size;
  const char *desc;
};

struct LaunchRecord {
  const char *name;
  const char *provenance;
  cudaEvent_t start, stop;
  std::string details;   // JSON object text
};

struct futhark_context {
  futhark_context_config *cfg = nullptr;
  std::mutex lock;             // serialises every public call on the context
  std::mutex error_lock;
  char *error = nullptr;       // first unread error (malloc'd)
  FILE *log = nullptr;
  int debugging = 0, logging = 0, profiling = 0, profiling_paused = 0;
  bool ready = false;          // backend set-up succeeded

  int device = 0;
  int num_sms = 0;
  cudaStream_t stream = nullptr;
  // Device-to-host copies of array values run on a stream of their own, ordered after the
  // work enqueued so far, so that they overlap later uploads and kernels; futhark_context_sync
  // waits for both streams, and a block freed while such a copy is pending makes the main
  // stream wait for it before the block can be reused.
  cudaStream_t copy_stream = nullptr;
  cudaEvent_t ev_main = nullptr, ev_copy = nullptr;
  bool copies_pending = false;
  std::string device_name;

  // pool: freed blocks by size (rts/c/gpu.h:240-316 semantics: smallest block that fits,
  // at most 2x waste unless below 4 KiB; on allocation failure cached blocks are
  // released and the allocation retried)
  std::multimap<size_t, void *> free_blocks;
  int64_t cur_mem = 0, peak_mem = 0;

  // device words shared by the kernels
  int *d_failure = nullptr;        // 0 = ok, else fb::FailureCode
  bool failure_is_an_option = false;
  void *lookback_scratch = nullptr;
  size_t lookback_scratch_bytes = 0;
  void *reduce_scratch = nullptr;
  int64_t *d_scalar = nullptr;     // device staging for scalar results (8 x 8 bytes)
  int64_t *h_scalar = nullptr;     // pinned host mirror
  uint32_t epoch = 0;
  int64_t launch_count = 0;       // kernels launched so far

  std::vector<LaunchRecord> events;
};

// ---- internal helpers (runtime.cu) ---------------------------------------------------------
void fb_set_error(futhark_context *ctx, const char *fmt, ...);
int fb_cuda_check(futhark_context *ctx, cudaError_t err, const char *what);   // 0 or an error code
int fb_alloc(futhark_context *ctx, size_t bytes, const char *desc, memblock_device *out);
void fb_unref(futhark_context *ctx, memblock_device *mb);
void fb_ref(memblock_device *mb);
int fb_ensure_lookback_scratch(futhark_context *ctx, size_t bytes);
uint32_t fb_next_epoch(futhark_context *ctx);
int64_t fb_tuning(futhark_context *ctx, const char *name);   // value of a tuning parameter (its default if never set)

// The flagged segmented scan with the context's lock held (entries.cu); shard_out / peer: see kernels.h.
namespace fb { struct PeerPush; }
struct futhark_f32_1d;
struct futhark_bool_1d;
extern "C" int segscan_f32_locked(futhark_context *ctx, struct futhark_f32_1d **out0, const struct futhark_bool_1d *in0,
                                  const struct futhark_f32_1d *in1, uint32_t *shard_out, const fb::PeerPush *peer);

// RAII guard: lock + make the context's device current
struct CtxGuard {
  futhark_context *ctx;
  int prev_device = -1;
  explicit CtxGuard(futhark_context *c);
  ~CtxGuard();
};

// Profiling scope around one kernel launch (no-op unless profiling is on and unpaused)
struct LaunchScope {
  futhark_context *ctx;
  bool active = false;
  LaunchRecord rec;
  LaunchScope(futhark_context *c, const char *name, const char *provenance, const std::string &details);
  ~LaunchScope();
};

// ---- array objects -------------------------------------------------------------------------------
#define FB_DEFINE_ARRAY_STRUCT(NAME, RANK) \
  struct futhark_##NAME {                  \
    memblock_device mem;                   \
    int64_t shape[RANK];                   \
  };
FB_DEFINE_ARRAY_STRUCT(i32_1d, 1)
FB_DEFINE_ARRAY_STRUCT(i64_1d, 1)
FB_DEFINE_ARRAY_STRUCT(u32_1d, 1)
FB_DEFINE_ARRAY_STRUCT(f32_1d, 1)
FB_DEFINE_ARRAY_STRUCT(bool_1d, 1)
FB_DEFINE_ARRAY_STRUCT(f32_2d, 2)
FB_DEFINE_ARRAY_STRUCT(i32_2d, 2)
FB_DEFINE_ARRAY_STRUCT(bool_2d, 2)
FB_DEFINE_ARRAY_STRUCT(i64_2d, 2)
FB_DEFINE_ARRAY_STRUCT(f64_2d, 2)
FB_DEFINE_ARRAY_STRUCT(f64_1d, 1)
FB_DEFINE_ARRAY_STRUCT(i8_1d, 1)
FB_DEFINE_ARRAY_STRUCT(i16_1d, 1)
FB_DEFINE_ARRAY_STRUCT(f16_1d, 1)
FB_DEFINE_ARRAY_STRUCT(u8_1d, 1)
FB_DEFINE_ARRAY_STRUCT(u16_1d, 1)
FB_DEFINE_ARRAY_STRUCT(f32_3d, 3)
FB_DEFINE_ARRAY_STRUCT(i32_3d, 3)
FB_DEFINE_ARRAY_STRUCT(f16_3d, 3)

struct futhark_opaque_tup2_arr1d_u32_arr1d_u32 {
  futhark_u32_1d *v0;
  futhark_u32_1d *v1;
};

struct futhark_opaque_tup3_arr1d_i32_arr1d_i32_arr1d_i32 {
  futhark_i32_1d *v[3];
};

struct futhark_opaque_tup2_arr1d_i64_arr2d_f64 {
  futhark_i64_1d *v0;
  futhark_f64_2d *v1;
};

struct futhark_opaque_tup2_arr1d_i32_arr1d_i32 {
  futhark_i32_1d *v[2];
};

struct futhark_opaque_tup6_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32_arr1d_i32 {
  futhark_i32_1d *v[6];
};

struct futhark_opaque_tup2_i32_f32 {
  int32_t v0;
  float v1;
};
