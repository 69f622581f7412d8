// Host runtime behind the C API: configuration objects, context life cycle, device
// selection, the device memory pool, array objects, the sticky error string, sync with
// failure-word decoding, and the JSON profiling report.  It stands where the reference's
// rts/c/context.h, rts/c/gpu.h, rts/c/free_list.h, rts/c/event_list.h and
// rts/c/backends/cuda.h stand; the interface is theirs, the implementation is not.
#include "runtime.h"

#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

#include <sstream>

#include "common.cuh"
#include "kernels.h"

// ---- tuning parameters ---------------------------------------------------------------------
// Names follow the reference's "<entry>.<kernel>_<what>" scheme and its size classes
// (rts/c/backends/cuda.h:552-596).  Five of them act: the four *_num_tblocks of the persistent
// scan / reduce grids cap the number of CTAs (0 = as many as are resident at once), and
// rowsum_f32.suff_outer_par is the threshold at which the outer parallelism of a row
// reduction is taken to suffice (one warp per row whatever the row length; below it a long
// row is shared by a CTA): the version choice of src/Futhark/CodeGen/Backends/GPU.hs:147-156.
// The others (block sizes, tile sizes) name shapes that are fixed in these kernels; they are
// accepted, stored and reported so that tuning files written for the reference load without error.
const TuningParam kTuningParams[] = {
    {"builtin#replicate_i32.tblock_size", "thread_block_size", 256},
    {"scan_i32.segscan_tblock_size", "thread_block_size", 256},
    {"scan_i32.segscan_num_tblocks", "grid_size", 0},
    {"reduce_i32.segred_tblock_size", "thread_block_size", 256},
    {"reduce_i32.segred_num_tblocks", "grid_size", 0},
    {"segscan_f32.segscan_tblock_size", "thread_block_size", 256},
    {"segscan_f32.segscan_num_tblocks", "grid_size", 0},
    {"segreduce_f32.segred_tblock_size", "thread_block_size", 256},
    {"rowsum_f32.segred_tblock_size", "thread_block_size", 256},
    {"rowsum_f32.segred_num_tblocks", "grid_size", 0},
    {"rowsum_f32.suff_outer_par", "threshold(def, )", 32768},
    {"hist_add_i32.seghist_tblock_size", "thread_block_size", 1024},
    {"hist_add_i32.seghist_num_tblocks", "grid_size", 0},
    {"hist_max_f32.seghist_tblock_size", "thread_block_size", 1024},
    {"filter_u32.segscan_tblock_size", "thread_block_size", 256},
    {"partition_u32.segscan_tblock_size", "thread_block_size", 256},
    {"bmm_f16.tile_size", "tile_size", 128},
    {"bmm_f16.reg_tile_size", "reg_tile_size", 1},
};
const int kNumTuningParams = (int)(sizeof(kTuningParams) / sizeof(kTuningParams[0]));

// ---- errors -------------------------------------------------------------------------------------
void fb_set_error(futhark_context *ctx, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  char buf[1024];
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  std::lock_guard<std::mutex> g(ctx->error_lock);
  if (ctx->error == nullptr) ctx->error = strdup(buf);   // the first error sticks (rts/c/context.h:5-13)
}

int fb_cuda_check(futhark_context *ctx, cudaError_t err, const char *what) {
  if (err == cudaSuccess) return FUTHARK_SUCCESS;
  (void)cudaGetLastError();   // clear the sticky per-thread error
  if (err == cudaErrorMemoryAllocation) {
    fb_set_error(ctx, "Failed to allocate device memory (%s).", what);
    return FUTHARK_OUT_OF_MEMORY;
  }
  fb_set_error(ctx, "CUDA call failed: %s: %s", what, cudaGetErrorString(err));
  return 1;
}

// ---- guards -------------------------------------------------------------------------------------
CtxGuard::CtxGuard(futhark_context *c) : ctx(c) {
  ctx->lock.lock();
  if (cudaGetDevice(&prev_device) != cudaSuccess) prev_device = -1;
  if (prev_device != ctx->device) cudaSetDevice(ctx->device);
}
CtxGuard::~CtxGuard() {
  if (prev_device >= 0 && prev_device != ctx->device) cudaSetDevice(prev_device);
  ctx->lock.unlock();
}

LaunchScope::LaunchScope(futhark_context *c, const char *name, const char *provenance, const std::string &details)
    : ctx(c) {
  ctx->launch_count++;
  if (ctx->logging) fprintf(ctx->log, "Event: %s\n  at: %s\n  %s\n", name, provenance, details.c_str());
  if (!ctx->profiling || ctx->profiling_paused) return;
  rec.name = name;
  rec.provenance = provenance;
  rec.details = details;
  if (cudaEventCreate(&rec.start) != cudaSuccess) return;
  if (cudaEventCreate(&rec.stop) != cudaSuccess) { cudaEventDestroy(rec.start); return; }
  cudaEventRecord(rec.start, ctx->stream);
  active = true;
}
LaunchScope::~LaunchScope() {
  if (!active) return;
  cudaEventRecord(rec.stop, ctx->stream);
  ctx->events.push_back(rec);
  if (ctx->debugging) {   // -D style: every launch is synchronous and its time is logged
    cudaEventSynchronize(rec.stop);
    float ms = 0;
    cudaEventElapsedTime(&ms, rec.start, rec.stop);
    fprintf(ctx->log, "  runtime: %.1fus\n", ms * 1000.0f);
  }
}

// ---- memory pool ----------------------------------------------------------------------------------
static cudaError_t raw_alloc(futhark_context *ctx, size_t bytes, void **p) {
  if (ctx->cfg->unified_memory) return cudaMallocManaged(p, bytes);
  return cudaMalloc(p, bytes);
}

int fb_alloc(futhark_context *ctx, size_t bytes, const char *desc, memblock_device *out) {
  if (bytes < 256) bytes = 256;
  bytes = (bytes + 255) & ~(size_t)255;
  void *p = nullptr;
  size_t got = bytes;
  // smallest cached block that fits and wastes at most half (or is tiny)
  auto it = ctx->free_blocks.lower_bound(bytes);
  if (it != ctx->free_blocks.end() && (it->first < 4096 || it->first < bytes * 2)) {
    p = it->second;
    got = it->first;
    ctx->free_blocks.erase(it);
    if (ctx->debugging) fprintf(ctx->log, "Allocation of %zu bytes (%s) served from the pool (%zu).\n", bytes, desc, got);
  } else {
    cudaError_t err = raw_alloc(ctx, bytes, &p);
    while (err == cudaErrorMemoryAllocation && !ctx->free_blocks.empty()) {
      (void)cudaGetLastError();
      // out of memory: release cached blocks one at a time and retry (rts/c/gpu.h:289-305)
      auto victim = std::prev(ctx->free_blocks.end());
      cudaStreamSynchronize(ctx->stream);
      cudaFree(victim->second);
      ctx->free_blocks.erase(victim);
      err = raw_alloc(ctx, bytes, &p);
    }
    int rc = fb_cuda_check(ctx, err, desc);
    if (rc != FUTHARK_SUCCESS) {
      if (rc == FUTHARK_OUT_OF_MEMORY) {
        std::lock_guard<std::mutex> g(ctx->error_lock);
        free(ctx->error);
        char buf[256];
        snprintf(buf, sizeof(buf), "Failed to allocate memory in space 'device'.\nAttempted allocation: %12lld bytes\nCurrently allocated:  %12lld bytes\n",
                 (long long)bytes, (long long)ctx->cur_mem);
        ctx->error = strdup(buf);
      }
      return rc;
    }
    if (ctx->debugging) fprintf(ctx->log, "Allocated %zu bytes (%s) from the driver.\n", bytes, desc);
  }
  out->references = (int *)malloc(sizeof(int));
  *out->references = 1;
  out->mem = (CUdeviceptr)(uintptr_t)p;
  out->size = (int64_t)got;
  out->desc = desc;
  ctx->cur_mem += (int64_t)got;
  if (ctx->cur_mem > ctx->peak_mem) ctx->peak_mem = ctx->cur_mem;
  return FUTHARK_SUCCESS;
}

void fb_ref(memblock_device *mb) {
  if (mb->references != nullptr) (*mb->references)++;
}

void fb_unref(futhark_context *ctx, memblock_device *mb) {
  if (mb->references == nullptr) return;   // borrowed memory is never freed by us
  if (--(*mb->references) == 0) {
    // Stream order makes immediate reuse safe: every consumer of the old contents was
    // enqueued on the main stream before any producer of the new contents will be -- except
    // a value copy still pending on the copy stream, which the main stream now waits for.
    if (ctx->copies_pending) {
      cudaEventRecord(ctx->ev_copy, ctx->copy_stream);
      cudaStreamWaitEvent(ctx->stream, ctx->ev_copy, 0);
      ctx->copies_pending = false;
    }
    ctx->free_blocks.emplace((size_t)mb->size, (void *)(uintptr_t)mb->mem);
    ctx->cur_mem -= mb->size;
    free(mb->references);
  }
  mb->references = nullptr;
  mb->mem = 0;
}

static int release_pool(futhark_context *ctx) {
  cudaStreamSynchronize(ctx->stream);
  for (auto &kv : ctx->free_blocks) cudaFree(kv.second);
  ctx->free_blocks.clear();
  return FUTHARK_SUCCESS;
}

int fb_ensure_lookback_scratch(futhark_context *ctx, size_t bytes) {
  if (bytes <= ctx->lookback_scratch_bytes) return FUTHARK_SUCCESS;
  size_t want = bytes < (1u << 20) ? (1u << 20) : bytes * 2;
  void *p = nullptr;
  int rc = fb_cuda_check(ctx, cudaMalloc(&p, want), "look-back scratch");
  if (rc != FUTHARK_SUCCESS) return rc;
  rc = fb_cuda_check(ctx, cudaMemsetAsync(p, 0, want, ctx->stream), "look-back scratch clear");
  if (rc != FUTHARK_SUCCESS) { cudaFree(p); return rc; }
  if (ctx->lookback_scratch != nullptr) {
    cudaStreamSynchronize(ctx->stream);
    cudaFree(ctx->lookback_scratch);
  }
  ctx->lookback_scratch = p;
  ctx->lookback_scratch_bytes = want;
  return FUTHARK_SUCCESS;
}

int64_t fb_tuning(futhark_context *ctx, const char *name) {
  for (int i = 0; i < kNumTuningParams; i++)
    if (strcmp(name, kTuningParams[i].name) == 0)
      return (ctx->cfg != nullptr && (int)ctx->cfg->tuning.size() > i) ? ctx->cfg->tuning[i] : kTuningParams[i].def;
  return 0;
}

uint32_t fb_next_epoch(futhark_context *ctx) {
  ctx->epoch = (ctx->epoch % ((1u << 29) - 1)) + 1;   // 1 .. 2^29-1, never 0
  return ctx->epoch;
}

// ---- configuration ----------------------------------------------------------------------------------
extern "C" {

struct futhark_context_config *futhark_context_config_new(void) {
  futhark_context_config *cfg = new (std::nothrow) futhark_context_config();
  if (cfg == nullptr) return nullptr;
  cfg->tuning.resize(kNumTuningParams);
  for (int i = 0; i < kNumTuningParams; i++) cfg->tuning[i] = kTuningParams[i].def;
  return cfg;
}
void futhark_context_config_free(struct futhark_context_config *cfg) { delete cfg; }
void futhark_context_config_set_debugging(struct futhark_context_config *cfg, int flag) {
  cfg->profiling = cfg->logging = cfg->debugging = flag;   // rts/c/context.h:95-97
}
void futhark_context_config_set_profiling(struct futhark_context_config *cfg, int flag) { cfg->profiling = flag; }
void futhark_context_config_set_logging(struct futhark_context_config *cfg, int flag) { cfg->logging = flag; }
void futhark_context_config_set_cache_file(struct futhark_context_config *cfg, const char *f) { cfg->cache_fname = f ? f : ""; }
int futhark_get_tuning_param_count(void) { return kNumTuningParams; }
const char *futhark_get_tuning_param_name(int i) { return (i >= 0 && i < kNumTuningParams) ? kTuningParams[i].name : nullptr; }
const char *futhark_get_tuning_param_class(int i) { return (i >= 0 && i < kNumTuningParams) ? kTuningParams[i].klass : nullptr; }

int futhark_context_config_set_tuning_param(struct futhark_context_config *cfg, const char *param_name, size_t new_value) {
  for (int i = 0; i < kNumTuningParams; i++)
    if (strcmp(param_name, kTuningParams[i].name) == 0) { cfg->tuning[i] = (int64_t)new_value; return 0; }
  // the default_* pseudo-parameters of rts/c/gpu.h:93-135
  if (strcmp(param_name, "default_thread_block_size") == 0 || strcmp(param_name, "default_group_size") == 0) { cfg->default_block_size = (int64_t)new_value; return 0; }
  if (strcmp(param_name, "default_grid_size") == 0 || strcmp(param_name, "default_num_groups") == 0) { cfg->default_grid_size = (int64_t)new_value; return 0; }
  if (strcmp(param_name, "default_threshold") == 0) { cfg->default_threshold = (int64_t)new_value; return 0; }
  if (strcmp(param_name, "default_tile_size") == 0) { cfg->default_tile_size = (int64_t)new_value; return 0; }
  if (strcmp(param_name, "default_reg_tile_size") == 0) { cfg->default_reg_tile_size = (int64_t)new_value; return 0; }
  return 1;
}

void futhark_context_config_set_device(struct futhark_context_config *cfg, const char *s) { cfg->device = s ? s : ""; }
void futhark_context_config_set_unified_memory(struct futhark_context_config *cfg, int flag) { cfg->unified_memory = flag; }
void futhark_context_config_set_default_thread_block_size(struct futhark_context_config *cfg, int size) { cfg->default_block_size = size; }
void futhark_context_config_set_default_group_size(struct futhark_context_config *cfg, int size) { cfg->default_block_size = size; }
void futhark_context_config_set_default_grid_size(struct futhark_context_config *cfg, int num) { cfg->default_grid_size = num; }
void futhark_context_config_set_default_num_groups(struct futhark_context_config *cfg, int num) { cfg->default_grid_size = num; }
void futhark_context_config_set_default_tile_size(struct futhark_context_config *cfg, int size) { cfg->default_tile_size = size; }
void futhark_context_config_set_default_reg_tile_size(struct futhark_context_config *cfg, int size) { cfg->default_reg_tile_size = size; }
void futhark_context_config_set_default_registers(struct futhark_context_config *cfg, int size) { cfg->default_registers = size; }
void futhark_context_config_set_default_cache(struct futhark_context_config *cfg, int size) { cfg->default_cache = size; }
void futhark_context_config_set_default_threshold(struct futhark_context_config *cfg, int size) { cfg->default_threshold = size; }
const char *futhark_context_config_get_program(struct futhark_context_config *cfg) { return cfg->program.c_str(); }
void futhark_context_config_set_program(struct futhark_context_config *cfg, const char *s) { cfg->program = s ? s : ""; }
void futhark_context_config_add_nvrtc_option(struct futhark_context_config *cfg, const char *opt) { if (opt) cfg->nvrtc_options.push_back(opt); }
void futhark_context_config_dump_ptx_to(struct futhark_context_config *cfg, const char *s) { cfg->dump_ptx_to = s ? s : ""; }
void futhark_context_config_load_ptx_from(struct futhark_context_config *cfg, const char *s) { cfg->load_ptx_from = s ? s : ""; }

// ---- context ------------------------------------------------------------------------------------------
// Device choice: "#k" picks device k, any other non-empty string the first device whose
// name contains it, the empty string the device with the highest compute capability
// (rts/c/backends/cuda.h:253-314).
static int pick_device(futhark_context *ctx) {
  int count = 0;
  cudaError_t err = cudaGetDeviceCount(&count);
  if (err != cudaSuccess || count == 0) {
    (void)cudaGetLastError();
    fb_set_error(ctx, "No CUDA device available: %s", err == cudaSuccess ? "device count is 0" : cudaGetErrorString(err));
    return -1;
  }
  const std::string &want = ctx->cfg->device;
  if (!want.empty() && want[0] == '#') {
    int k = atoi(want.c_str() + 1);
    if (k < 0 || k >= count) { fb_set_error(ctx, "Device %s does not exist (%d devices).", want.c_str(), count); return -1; }
    return k;
  }
  int best = -1, best_cc = -1;
  for (int d = 0; d < count; d++) {
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, d) != cudaSuccess) continue;
    if (!want.empty()) {
      if (strstr(prop.name, want.c_str()) != nullptr) return d;
      continue;
    }
    int cc = prop.major * 10 + prop.minor;
    if (cc > best_cc) { best_cc = cc; best = d; }
  }
  if (best < 0) fb_set_error(ctx, "No device matches '%s'.", want.c_str());
  return best;
}

static int backend_setup(futhark_context *ctx) {
  int dev = pick_device(ctx);
  if (dev < 0) return 1;
  ctx->device = dev;
  int rc = fb_cuda_check(ctx, cudaSetDevice(dev), "cudaSetDevice");
  if (rc) return rc;
  cudaDeviceProp prop;
  rc = fb_cuda_check(ctx, cudaGetDeviceProperties(&prop, dev), "cudaGetDeviceProperties");
  if (rc) return rc;
  ctx->device_name = prop.name;
  ctx->num_sms = prop.multiProcessorCount;
  if (prop.major != 10) {
    fb_set_error(ctx, "Device '%s' has compute capability %d.%d; this library contains sm_100a code only.",
                 prop.name, prop.major, prop.minor);
    return 1;
  }
  if (ctx->logging)
    fprintf(ctx->log, "Using device #%d: %s (compute capability %d.%d, %d SMs, %zu MiB, %zu KiB shared memory per block, %d KiB L2)\n",
            dev, prop.name, prop.major, prop.minor, prop.multiProcessorCount, prop.totalGlobalMem >> 20,
            prop.sharedMemPerBlockOptin >> 10, prop.l2CacheSize >> 10);
  rc = fb_cuda_check(ctx, cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking), "cudaStreamCreate");
  if (rc) return rc;
  rc = fb_cuda_check(ctx, cudaStreamCreateWithFlags(&ctx->copy_stream, cudaStreamNonBlocking), "cudaStreamCreate");
  if (rc) return rc;
  rc = fb_cuda_check(ctx, cudaEventCreateWithFlags(&ctx->ev_main, cudaEventDisableTiming), "cudaEventCreate");
  if (rc) return rc;
  rc = fb_cuda_check(ctx, cudaEventCreateWithFlags(&ctx->ev_copy, cudaEventDisableTiming), "cudaEventCreate");
  if (rc) return rc;
  rc = fb_cuda_check(ctx, cudaMalloc((void **)&ctx->d_failure, 256), "failure word");
  if (rc) return rc;
  rc = fb_cuda_check(ctx, cudaMemsetAsync(ctx->d_failure, 0, 256, ctx->stream), "failure word clear");
  if (rc) return rc;
  rc = fb_cuda_check(ctx, cudaMalloc(&ctx->reduce_scratch, fb::reduce_scratch_bytes()), "reduce scratch");
  if (rc) return rc;
  rc = fb_cuda_check(ctx, cudaMemsetAsync(ctx->reduce_scratch, 0, fb::reduce_scratch_bytes(), ctx->stream), "reduce scratch clear");
  if (rc) return rc;
  rc = fb_cuda_check(ctx, cudaMalloc((void **)&ctx->d_scalar, 64), "scalar staging");
  if (rc) return rc;
  rc = fb_cuda_check(ctx, cudaMallocHost((void **)&ctx->h_scalar, 64), "pinned scalar staging");
  if (rc) return rc;
  rc = fb_ensure_lookback_scratch(ctx, 1u << 20);
  if (rc) return rc;
  return fb_cuda_check(ctx, cudaStreamSynchronize(ctx->stream), "initial sync");
}

struct futhark_context *futhark_context_new(struct futhark_context_config *cfg) {
  futhark_context *ctx = new (std::nothrow) futhark_context();
  if (ctx == nullptr) return nullptr;
  ctx->cfg = cfg;
  cfg->in_use = 1;
  ctx->debugging = cfg->debugging;
  ctx->logging = cfg->logging;
  ctx->profiling = cfg->profiling;
  ctx->log = stderr;
  int prev = -1;
  if (cudaGetDevice(&prev) != cudaSuccess) { (void)cudaGetLastError(); prev = -1; }
  // On failure the context is still returned; the caller finds out through
  // futhark_context_get_error (docs/c-api.rst:161-166).
  ctx->ready = (backend_setup(ctx) == 0);
  if (prev >= 0 && ctx->ready && prev != ctx->device) cudaSetDevice(prev);
  return ctx;
}

void futhark_context_free(struct futhark_context *ctx) {
  if (ctx == nullptr) return;
  if (ctx->ready) {
    int prev = -1;
    cudaGetDevice(&prev);
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    release_pool(ctx);
    for (auto &r : ctx->events) { cudaEventDestroy(r.start); cudaEventDestroy(r.stop); }
    cudaFree(ctx->d_failure);
    cudaFree(ctx->reduce_scratch);
    cudaFree(ctx->lookback_scratch);
    cudaFree(ctx->d_scalar);
    cudaFreeHost(ctx->h_scalar);
    cudaStreamSynchronize(ctx->copy_stream);
    cudaStreamDestroy(ctx->copy_stream);
    cudaEventDestroy(ctx->ev_main);
    cudaEventDestroy(ctx->ev_copy);
    cudaStreamDestroy(ctx->stream);
    if (prev >= 0 && prev != ctx->device) cudaSetDevice(prev);
  }
  free(ctx->error);
  ctx->cfg->in_use = 0;
  delete ctx;
}

static const char *failure_text(int code) {
  switch (code) {
    case fb::FAIL_LOOKBACK_TIMEOUT: return "a scan tile waited too long for its predecessors (look-back wait limit reached)";
    case fb::FAIL_BULK_COPY_TIMEOUT: return "a bulk shared-memory copy did not complete within its wait limit";
    case fb::FAIL_MMA_TIMEOUT: return "the tensor-core pipeline did not make progress within its wait limit";
    case fb::FAIL_PEER_TIMEOUT: return "the summary of another GPU's shard did not arrive within the wait limit";
    default: return "unknown device failure code";
  }
}

int futhark_context_sync(struct futhark_context *ctx) {
  if (!ctx->ready) return 1;
  CtxGuard g(ctx);
  int rc = fb_cuda_check(ctx, cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize");
  if (rc) return rc;
  rc = fb_cuda_check(ctx, cudaStreamSynchronize(ctx->copy_stream), "cudaStreamSynchronize");
  if (rc) return rc;
  ctx->copies_pending = false;
  if (ctx->failure_is_an_option) {
    // Same protocol as rts/c/backends/cuda.h:719-754: read the failure word, and if it
    // is set, reset it and report a program error.
    int code = 0;
    rc = fb_cuda_check(ctx, cudaMemcpyAsync(&code, ctx->d_failure, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream), "failure word read");
    if (rc) return rc;
    rc = fb_cuda_check(ctx, cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize");
    if (rc) return rc;
    ctx->failure_is_an_option = false;
    if (code != fb::FAIL_NONE) {
      cudaMemsetAsync(ctx->d_failure, 0, sizeof(int), ctx->stream);
      // tickets and status words may be left half-way: start them afresh
      cudaMemsetAsync(ctx->lookback_scratch, 0, ctx->lookback_scratch_bytes, ctx->stream);
      cudaStreamSynchronize(ctx->stream);
      fb_set_error(ctx, "Device-side failure %d: %s.", code, failure_text(code));
      return FUTHARK_PROGRAM_ERROR;
    }
  }
  return FUTHARK_SUCCESS;
}

void *futhark_b200_context_get_stream(struct futhark_context *ctx) { return (void *)ctx->stream; }
int futhark_b200_context_get_device(struct futhark_context *ctx) { return ctx->device; }
int64_t futhark_b200_context_get_launch_count(struct futhark_context *ctx) { return ctx->launch_count; }

char *futhark_context_get_error(struct futhark_context *ctx) {
  std::lock_guard<std::mutex> g(ctx->error_lock);
  char *e = ctx->error;
  ctx->error = nullptr;
  return e;
}
void futhark_context_set_logging_file(struct futhark_context *ctx, FILE *f) { ctx->log = f; }
void futhark_context_pause_profiling(struct futhark_context *ctx) { ctx->profiling_paused = 1; }
void futhark_context_unpause_profiling(struct futhark_context *ctx) { ctx->profiling_paused = 0; }

int futhark_context_clear_caches(struct futhark_context *ctx) {
  if (!ctx->ready) return 1;
  CtxGuard g(ctx);
  return release_pool(ctx);
}

static void json_escape(std::ostringstream &os, const char *s) {
  os << '"';
  for (; *s; s++) {
    if (*s == '"' || *s == '\\') os << '\\' << *s;
    else if (*s == '\n') os << "\\n";
    else os << *s;
  }
  os << '"';
}

// JSON of the shape {"memory":{...},"events":[{name,provenance,duration,details}]}, duration
// in microseconds (rts/c/event_list.h:150-179, GenericC.hs:610-630).  Reported events are
// consumed.
char *futhark_context_report(struct futhark_context *ctx) {
  if (!ctx->ready) return strdup("{}");
  CtxGuard g(ctx);
  cudaStreamSynchronize(ctx->stream);
  std::ostringstream os;
  os << "{\"memory\":{\"device\":" << ctx->peak_mem << "},\"events\":[";
  bool first = true;
  for (auto &r : ctx->events) {
    float ms = 0;
    cudaEventElapsedTime(&ms, r.start, r.stop);
    if (!first) os << ',';
    first = false;
    os << "{\"name\":";
    json_escape(os, r.name);
    os << ",\"provenance\":";
    json_escape(os, r.provenance);
    os << ",\"duration\":" << (double)ms * 1000.0 << ",\"details\":" << (r.details.empty() ? "{}" : r.details) << "}";
    cudaEventDestroy(r.start);
    cudaEventDestroy(r.stop);
  }
  ctx->events.clear();
  os << "]}";
  return strdup(os.str().c_str());
}

}  // extern "C"

// ---- arrays ------------------------------------------------------------------------------------------
// new: allocate + asynchronous host-to-device copy; values: asynchronous device-to-host
// copy; index: one element; raw: borrow a device pointer.  (GenericC/Types.hs:61-250)
template <typename ARR, int RANK>
static ARR *array_new(futhark_context *ctx, const void *data, const int64_t *dims, size_t elem, const char *desc) {
  if (!ctx->ready) return nullptr;
  ARR *arr = (ARR *)malloc(sizeof(ARR));
  if (arr == nullptr) return nullptr;
  CtxGuard g(ctx);
  int64_t n = 1;
  for (int i = 0; i < RANK; i++) {
    if (dims[i] < 0) { fb_set_error(ctx, "Negative array dimension."); free(arr); return nullptr; }
    arr->shape[i] = dims[i];
    n *= dims[i];
  }
  if (fb_alloc(ctx, (size_t)n * elem, desc, &arr->mem) != FUTHARK_SUCCESS) { free(arr); return nullptr; }
  if (n > 0) {
    cudaError_t err = cudaMemcpyAsync((void *)(uintptr_t)arr->mem.mem, data, (size_t)n * elem, cudaMemcpyHostToDevice, ctx->stream);
    if (fb_cuda_check(ctx, err, "host-to-device copy") != 0) { fb_unref(ctx, &arr->mem); free(arr); return nullptr; }
  }
  return arr;
}

template <typename ARR, int RANK>
static ARR *array_new_raw(futhark_context *ctx, CUdeviceptr data, const int64_t *dims, size_t elem) {
  ARR *arr = (ARR *)malloc(sizeof(ARR));
  if (arr == nullptr) return nullptr;
  int64_t n = 1;
  for (int i = 0; i < RANK; i++) { arr->shape[i] = dims[i]; n *= dims[i]; }
  arr->mem.references = nullptr;
  arr->mem.mem = data;
  arr->mem.size = n * (int64_t)elem;
  arr->mem.desc = "raw";
  (void)ctx;
  return arr;
}

template <typename ARR>
static int array_free(futhark_context *ctx, ARR *arr) {
  if (arr == nullptr) return 0;
  CtxGuard g(ctx);
  fb_unref(ctx, &arr->mem);
  free(arr);
  return 0;
}

template <typename ARR, int RANK>
static int array_values(futhark_context *ctx, ARR *arr, void *out, size_t elem) {
  CtxGuard g(ctx);
  int64_t n = 1;
  for (int i = 0; i < RANK; i++) n *= arr->shape[i];
  if (n == 0) return 0;
  // after everything enqueued so far, beside everything enqueued later
  int rc = fb_cuda_check(ctx, cudaEventRecord(ctx->ev_main, ctx->stream), "cudaEventRecord");
  if (rc) return rc;
  rc = fb_cuda_check(ctx, cudaStreamWaitEvent(ctx->copy_stream, ctx->ev_main, 0), "cudaStreamWaitEvent");
  if (rc) return rc;
  ctx->copies_pending = true;
  return fb_cuda_check(ctx, cudaMemcpyAsync(out, (const void *)(uintptr_t)arr->mem.mem, (size_t)n * elem, cudaMemcpyDeviceToHost, ctx->copy_stream),
                       "device-to-host copy");
}

template <typename ARR, int RANK>
static int array_index(futhark_context *ctx, void *out, ARR *arr, const int64_t *idx, size_t elem) {
  int64_t flat = 0;
  for (int i = 0; i < RANK; i++) {
    if (idx[i] < 0 || idx[i] >= arr->shape[i]) { fb_set_error(ctx, "Index out of bounds."); return 1; }
    flat = flat * arr->shape[i] + idx[i];
  }
  CtxGuard g(ctx);
  return fb_cuda_check(ctx, cudaMemcpyAsync(out, (const char *)(uintptr_t)arr->mem.mem + flat * elem, elem, cudaMemcpyDeviceToHost, ctx->stream),
                       "device-to-host copy");
}

#define FB_ARRAY_COMMON(NAME, CT, RANK)                                                                        \
  int futhark_free_##NAME(struct futhark_context *ctx, struct futhark_##NAME *arr) { return array_free(ctx, arr); } \
  int futhark_values_##NAME(struct futhark_context *ctx, struct futhark_##NAME *arr, CT *data) {                \
    return array_values<futhark_##NAME, RANK>(ctx, arr, data, sizeof(CT));                                      \
  }                                                                                                            \
  CUdeviceptr futhark_values_raw_##NAME(struct futhark_context *ctx, struct futhark_##NAME *arr) { (void)ctx; return arr->mem.mem; } \
  const int64_t *futhark_shape_##NAME(struct futhark_context *ctx, struct futhark_##NAME *arr) { (void)ctx; return arr->shape; }

#define FB_ARRAY_1D(NAME, CT)                                                                                  \
  FB_ARRAY_COMMON(NAME, CT, 1)                                                                                 \
  struct futhark_##NAME *futhark_new_##NAME(struct futhark_context *ctx, const CT *data, int64_t dim0) {       \
    int64_t d[1] = {dim0};                                                                                     \
    return array_new<futhark_##NAME, 1>(ctx, data, d, sizeof(CT), #NAME);                                      \
  }                                                                                                            \
  struct futhark_##NAME *futhark_new_raw_##NAME(struct futhark_context *ctx, CUdeviceptr data, int64_t dim0) { \
    int64_t d[1] = {dim0};                                                                                     \
    return array_new_raw<futhark_##NAME, 1>(ctx, data, d, sizeof(CT));                                         \
  }                                                                                                            \
  int futhark_index_##NAME(struct futhark_context *ctx, CT *out, struct futhark_##NAME *arr, int64_t i0) {     \
    int64_t i[1] = {i0};                                                                                       \
    return array_index<futhark_##NAME, 1>(ctx, out, arr, i, sizeof(CT));                                       \
  }

#define FB_ARRAY_2D(NAME, CT)                                                                                  \
  FB_ARRAY_COMMON(NAME, CT, 2)                                                                                 \
  struct futhark_##NAME *futhark_new_##NAME(struct futhark_context *ctx, const CT *data, int64_t dim0, int64_t dim1) { \
    int64_t d[2] = {dim0, dim1};                                                                               \
    return array_new<futhark_##NAME, 2>(ctx, data, d, sizeof(CT), #NAME);                                      \
  }                                                                                                            \
  struct futhark_##NAME *futhark_new_raw_##NAME(struct futhark_context *ctx, CUdeviceptr data, int64_t dim0, int64_t dim1) { \
    int64_t d[2] = {dim0, dim1};                                                                               \
    return array_new_raw<futhark_##NAME, 2>(ctx, data, d, sizeof(CT));                                         \
  }                                                                                                            \
  int futhark_index_##NAME(struct futhark_context *ctx, CT *out, struct futhark_##NAME *arr, int64_t i0, int64_t i1) { \
    int64_t i[2] = {i0, i1};                                                                                   \
    return array_index<futhark_##NAME, 2>(ctx, out, arr, i, sizeof(CT));                                       \
  }

#define FB_ARRAY_3D(NAME, CT)                                                                                  \
  FB_ARRAY_COMMON(NAME, CT, 3)                                                                                 \
  struct futhark_##NAME *futhark_new_##NAME(struct futhark_context *ctx, const CT *data, int64_t dim0, int64_t dim1, int64_t dim2) { \
    int64_t d[3] = {dim0, dim1, dim2};                                                                         \
    return array_new<futhark_##NAME, 3>(ctx, data, d, sizeof(CT), #NAME);                                      \
  }                                                                                                            \
  struct futhark_##NAME *futhark_new_raw_##NAME(struct futhark_context *ctx, CUdeviceptr data, int64_t dim0, int64_t dim1, int64_t dim2) { \
    int64_t d[3] = {dim0, dim1, dim2};                                                                         \
    return array_new_raw<futhark_##NAME, 3>(ctx, data, d, sizeof(CT));                                         \
  }                                                                                                            \
  int futhark_index_##NAME(struct futhark_context *ctx, CT *out, struct futhark_##NAME *arr, int64_t i0, int64_t i1, int64_t i2) { \
    int64_t i[3] = {i0, i1, i2};                                                                               \
    return array_index<futhark_##NAME, 3>(ctx, out, arr, i, sizeof(CT));                                       \
  }

extern "C" {
FB_ARRAY_1D(i32_1d, int32_t)
FB_ARRAY_1D(i64_1d, int64_t)
FB_ARRAY_1D(u32_1d, uint32_t)
FB_ARRAY_1D(f32_1d, float)
FB_ARRAY_1D(bool_1d, bool)
FB_ARRAY_2D(f32_2d, float)
FB_ARRAY_2D(i32_2d, int32_t)
FB_ARRAY_2D(bool_2d, bool)
FB_ARRAY_2D(i64_2d, int64_t)
FB_ARRAY_2D(f64_2d, double)
FB_ARRAY_1D(f64_1d, double)
FB_ARRAY_1D(i8_1d, int8_t)
FB_ARRAY_1D(i16_1d, int16_t)
FB_ARRAY_1D(f16_1d, uint16_t)
FB_ARRAY_1D(u8_1d, uint8_t)
FB_ARRAY_1D(u16_1d, uint16_t)
FB_ARRAY_3D(f32_3d, float)
FB_ARRAY_3D(i32_3d, int32_t)
FB_ARRAY_3D(f16_3d, uint16_t)

// ---- the opaque pair returned by partition (docs/c-api.rst:317-438) --------------------------------
typedef struct futhark_opaque_tup2_arr1d_u32_arr1d_u32 pair_t;

static futhark_u32_1d *alias_u32(const futhark_u32_1d *src) {
  futhark_u32_1d *a = (futhark_u32_1d *)malloc(sizeof(futhark_u32_1d));
  if (a == nullptr) return nullptr;
  *a = *src;
  fb_ref(&a->mem);
  return a;
}

int futhark_free_opaque_tup2_arr1d_u32_arr1d_u32(struct futhark_context *ctx, pair_t *obj) {
  if (obj == nullptr) return 0;
  futhark_free_u32_1d(ctx, obj->v0);
  futhark_free_u32_1d(ctx, obj->v1);
  free(obj);
  return 0;
}

int futhark_new_opaque_tup2_arr1d_u32_arr1d_u32(struct futhark_context *ctx, pair_t **out, const struct futhark_u32_1d *v0,
                                                const struct futhark_u32_1d *v1) {
  pair_t *p = (pair_t *)malloc(sizeof(pair_t));
  if (p == nullptr) return 1;
  {
    CtxGuard g(ctx);
    p->v0 = alias_u32(v0);
    p->v1 = alias_u32(v1);
  }
  *out = p;
  return 0;
}

int futhark_project_opaque_tup2_arr1d_u32_arr1d_u32_0(struct futhark_context *ctx, struct futhark_u32_1d **out, const pair_t *obj) {
  CtxGuard g(ctx);
  *out = alias_u32(obj->v0);
  return *out == nullptr;
}
int futhark_project_opaque_tup2_arr1d_u32_arr1d_u32_1(struct futhark_context *ctx, struct futhark_u32_1d **out, const pair_t *obj) {
  CtxGuard g(ctx);
  *out = alias_u32(obj->v1);
  return *out == nullptr;
}

// Serialised form: for each field the binary data format of docs/binary-data-format.rst
// ('b', version 2, rank 1, " u32", int64 length, then the elements).
static const size_t kHdr = 1 + 1 + 1 + 4 + 8;
int futhark_store_opaque_tup2_arr1d_u32_arr1d_u32(struct futhark_context *ctx, const pair_t *obj, void **p, size_t *n) {
  const int64_t n0 = obj->v0->shape[0], n1 = obj->v1->shape[0];
  const size_t total = 2 * kHdr + (size_t)(n0 + n1) * 4;
  *n = total;
  if (p == nullptr) return 0;
  if (*p == nullptr) *p = malloc(total);
  if (*p == nullptr) return 1;
  unsigned char *o = (unsigned char *)*p;
  const futhark_u32_1d *f[2] = {obj->v0, obj->v1};
  int rc = 0;
  for (int i = 0; i < 2; i++) {
    const int64_t len = f[i]->shape[0];
    *o++ = 'b'; *o++ = 2; *o++ = 1;
    memcpy(o, " u32", 4); o += 4;
    memcpy(o, &len, 8); o += 8;
    rc |= futhark_values_u32_1d(ctx, const_cast<futhark_u32_1d *>(f[i]), (uint32_t *)o);
    o += (size_t)len * 4;
  }
  return rc;
}

pair_t *futhark_restore_opaque_tup2_arr1d_u32_arr1d_u32(struct futhark_context *ctx, const void *p) {
  const unsigned char *s = (const unsigned char *)p;
  futhark_u32_1d *f[2] = {nullptr, nullptr};
  for (int i = 0; i < 2; i++) {
    if (s[0] != 'b' || s[1] != 2 || s[2] != 1 || memcmp(s + 3, " u32", 4) != 0) {
      fb_set_error(ctx, "Cannot restore value: malformed header.");
      if (f[0]) futhark_free_u32_1d(ctx, f[0]);
      return nullptr;
    }
    int64_t len;
    memcpy(&len, s + 7, 8);
    s += kHdr;
    f[i] = futhark_new_u32_1d(ctx, (const uint32_t *)s, len);
    if (f[i] == nullptr) { if (f[0]) futhark_free_u32_1d(ctx, f[0]); return nullptr; }
    s += (size_t)len * 4;
  }
  pair_t *out = (pair_t *)malloc(sizeof(pair_t));
  out->v0 = f[0];
  out->v1 = f[1];
  return out;
}

// ---- the opaque pair of scalars returned by sum_i32_f32: same functions, host-side fields -----------
typedef struct futhark_opaque_tup2_i32_f32 spair_t;

int futhark_free_opaque_tup2_i32_f32(struct futhark_context *ctx, spair_t *obj) {
  (void)ctx;
  free(obj);
  return 0;
}

int futhark_new_opaque_tup2_i32_f32(struct futhark_context *ctx, spair_t **out, const int32_t v0, const float v1) {
  (void)ctx;
  spair_t *p = (spair_t *)malloc(sizeof(spair_t));
  if (p == nullptr) return 1;
  p->v0 = v0;
  p->v1 = v1;
  *out = p;
  return 0;
}

int futhark_project_opaque_tup2_i32_f32_0(struct futhark_context *ctx, int32_t *out, const spair_t *obj) {
  (void)ctx;
  *out = obj->v0;
  return 0;
}
int futhark_project_opaque_tup2_i32_f32_1(struct futhark_context *ctx, float *out, const spair_t *obj) {
  (void)ctx;
  *out = obj->v1;
  return 0;
}

// Serialised form: the two scalars in the binary data format ('b', version 2, rank 0, type, value).
static const size_t kScalarHdr = 1 + 1 + 1 + 4;
int futhark_store_opaque_tup2_i32_f32(struct futhark_context *ctx, const spair_t *obj, void **p, size_t *n) {
  (void)ctx;
  const size_t total = 2 * (kScalarHdr + 4);
  *n = total;
  if (p == nullptr) return 0;
  if (*p == nullptr) *p = malloc(total);
  if (*p == nullptr) return 1;
  unsigned char *o = (unsigned char *)*p;
  *o++ = 'b'; *o++ = 2; *o++ = 0; memcpy(o, " i32", 4); o += 4; memcpy(o, &obj->v0, 4); o += 4;
  *o++ = 'b'; *o++ = 2; *o++ = 0; memcpy(o, " f32", 4); o += 4; memcpy(o, &obj->v1, 4);
  return 0;
}

spair_t *futhark_restore_opaque_tup2_i32_f32(struct futhark_context *ctx, const void *p) {
  const unsigned char *s = (const unsigned char *)p;
  const unsigned char *t = s + kScalarHdr + 4;
  if (s[0] != 'b' || s[1] != 2 || s[2] != 0 || memcmp(s + 3, " i32", 4) != 0 || t[0] != 'b' || t[1] != 2 || t[2] != 0 ||
      memcmp(t + 3, " f32", 4) != 0) {
    fb_set_error(ctx, "Cannot restore value: malformed header.");
    return nullptr;
  }
  spair_t *out = (spair_t *)malloc(sizeof(spair_t));
  if (out == nullptr) return nullptr;
  memcpy(&out->v0, s + kScalarHdr, 4);
  memcpy(&out->v1, t + kScalarHdr, 4);
  return out;
}

}  // extern "C"
