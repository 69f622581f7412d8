// One logical array split into contiguous shards over several contexts (one per GPU, one
// process or thread each), through the C ABI: the shard-local kernels of this library plus one
// NCCL collective where the operation has an exchange step.  The reference is single-device
// (rts/c/backends/cuda.h:219 picks one device per context), so this layer has no counterpart
// there; it is what a C host program links against instead of driving the exchange itself.
//
//   reduce          local reduce -> all-reduce (sum) of one i32
//   scan            local reduce -> all-gather of the shard totals -> local scan seeded with the
//                   totals of the shards in front
//   segmented scan  local scan, whose kernel also writes the shard's 16-byte summary ->
//                   all-gather of the summaries -> one kernel adds the carry in front of the
//                   shard's first segment start
//   histogram       local histogram -> all-reduce (sum / max) over the bins
//   filter, partition   local compaction -> all-gather of the counts; the result stays sharded
//   contraction     whole batches per shard: no exchange
//
// NCCL is not linked: its six entry points are looked up at run time in the libnccl.so.2 the
// process already has (or can load), so the library itself has no dependency on it and a
// single-GPU user never touches it.  Every collective runs on the context's own stream, in
// order with the kernels: no host synchronisation between them.
#include <dlfcn.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include <mutex>
#include <string>

#include "common.cuh"
#include "kernels.h"
#include "runtime.h"

namespace {

// The part of NCCL's public C API that is used (nccl.h: stable names, types and enumerators).
struct NcclUniqueId { char internal[128]; };
typedef void *NcclComm;
enum { NCCL_INT32 = 2, NCCL_INT64 = 4, NCCL_FLOAT32 = 7 };      // ncclDataType_t
enum { NCCL_SUM = 0, NCCL_MAX = 2 };                            // ncclRedOp_t

struct NcclApi {
  int (*GetUniqueId)(NcclUniqueId *) = nullptr;
  int (*CommInitRank)(NcclComm *, int, NcclUniqueId, int) = nullptr;
  int (*CommDestroy)(NcclComm) = nullptr;
  int (*AllReduce)(const void *, void *, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
  int (*AllGather)(const void *, void *, size_t, int, NcclComm, cudaStream_t) = nullptr;
  const char *(*GetErrorString)(int) = nullptr;
  std::string why;            // why it could not be loaded
  bool ok = false;
};

NcclApi &nccl() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    void *h = nullptr;
    const char *env = getenv("FUTHARK_B200_NCCL");
    if (env != nullptr && env[0] != 0) h = dlopen(env, RTLD_NOW | RTLD_GLOBAL);
    if (h == nullptr) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);       // the copy the process already has
    if (h == nullptr) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (h == nullptr) { api.why = std::string("libnccl.so.2 could not be loaded: ") + dlerror(); return; }
    auto sym = [&](const char *name) -> void * {
      void *p = dlsym(h, name);
      if (p == nullptr && api.why.empty()) api.why = std::string("libnccl.so.2 lacks ") + name;
      return p;
    };
    api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
    api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
    api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
    api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(sym("ncclAllReduce"));
    api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
    api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
    api.ok = api.why.empty();
  });
  return api;
}

}  // namespace

struct futhark_b200_group {
  futhark_context *ctx;
  NcclComm comm;
  bool owns_comm;
  int rank, world;
  int32_t *d_xchg;          // exchange area on the device: 4 words per rank, then 4 of this rank
  // exchange by peer stores (futhark_b200_group_enable_peer_exchange)
  uint32_t *peer_buf = nullptr;        // this rank's buffer, written by the ranks in front
  uint32_t **d_peer_bufs = nullptr;    // device array: every rank's buffer as this GPU addresses it
  void *opened[64] = {nullptr};        // IPC mappings to close
  uint32_t seq = 0;                    // sequence number of the last segmented scan
  struct Pending { futhark_f32_1d *out; uint32_t seq; } pending = {nullptr, 0};
};

static int group_check(futhark_b200_group *g, int rc, const char *what) {
  if (rc == 0) return 0;
  fb_set_error(g->ctx, "NCCL call failed: %s: %s", what, nccl().GetErrorString ? nccl().GetErrorString(rc) : "?");
  return 1;
}

template <typename T>
static inline T *gdptr(const memblock_device &m) { return reinterpret_cast<T *>((uintptr_t)m.mem); }

extern "C" {

int futhark_b200_group_unique_id(void *id_out, size_t len) {
  if (!nccl().ok || len < sizeof(NcclUniqueId)) return 1;
  return nccl().GetUniqueId(reinterpret_cast<NcclUniqueId *>(id_out)) == 0 ? 0 : 1;
}

const char *futhark_b200_group_unavailable(void) { return nccl().ok ? nullptr : nccl().why.c_str(); }

static futhark_b200_group *group_make(futhark_context *ctx, NcclComm comm, bool owns, int rank, int world) {
  futhark_b200_group *g = new (std::nothrow) futhark_b200_group();
  if (g == nullptr) return nullptr;
  g->ctx = ctx; g->comm = comm; g->owns_comm = owns; g->rank = rank; g->world = world; g->d_xchg = nullptr;
  CtxGuard guard(ctx);
  if (cudaMalloc((void **)&g->d_xchg, (size_t)(world + 1) * 16) != cudaSuccess) {
    fb_set_error(ctx, "group: could not allocate the exchange area");
    if (owns) nccl().CommDestroy(comm);
    delete g;
    return nullptr;
  }
  return g;
}

struct futhark_b200_group *futhark_b200_group_new(struct futhark_context *ctx, const void *unique_id, int rank, int world) {
  if (!ctx->ready) { fb_set_error(ctx, "The context failed to initialise; no group can be made."); return nullptr; }
  if (!nccl().ok) { fb_set_error(ctx, "group: %s", nccl().why.c_str()); return nullptr; }
  if (world < 1 || rank < 0 || rank >= world) { fb_set_error(ctx, "group: rank %d of %d", rank, world); return nullptr; }
  NcclUniqueId id;
  memcpy(&id, unique_id, sizeof(id));
  NcclComm comm = nullptr;
  int rc;
  {
    CtxGuard guard(ctx);          // the communicator belongs to the context's device
    rc = nccl().CommInitRank(&comm, world, id, rank);
  }
  if (rc != 0) { fb_set_error(ctx, "ncclCommInitRank failed: %s", nccl().GetErrorString(rc)); return nullptr; }
  return group_make(ctx, comm, true, rank, world);
}

struct futhark_b200_group *futhark_b200_group_from_comm(struct futhark_context *ctx, void *nccl_comm, int rank, int world) {
  if (!ctx->ready) { fb_set_error(ctx, "The context failed to initialise; no group can be made."); return nullptr; }
  if (!nccl().ok) { fb_set_error(ctx, "group: %s", nccl().why.c_str()); return nullptr; }
  return group_make(ctx, nccl_comm, false, rank, world);
}

void futhark_b200_group_free(struct futhark_b200_group *g) {
  if (g == nullptr) return;
  {
    CtxGuard guard(g->ctx);
    cudaStreamSynchronize(g->ctx->stream);
    for (int r = 0; r < 64; r++)
      if (g->opened[r] != nullptr) cudaIpcCloseMemHandle(g->opened[r]);
    if (g->d_peer_bufs != nullptr) cudaFree(g->d_peer_bufs);
    if (g->peer_buf != nullptr) cudaFree(g->peer_buf);
    cudaFree(g->d_xchg);
    if (g->owns_comm) nccl().CommDestroy(g->comm);
  }
  delete g;
}

int futhark_b200_group_rank(const struct futhark_b200_group *g) { return g->rank; }
int futhark_b200_group_size(const struct futhark_b200_group *g) { return g->world; }

int futhark_b200_group_reduce_i32(struct futhark_b200_group *g, int32_t *out0, const struct futhark_i32_1d *in0) {
  futhark_context *ctx = g->ctx;
  int rc = futhark_b200_reduce_i32_to_device(ctx, (CUdeviceptr)(uintptr_t)g->d_xchg, in0);
  if (rc != 0) return rc;
  CtxGuard guard(ctx);
  rc = group_check(g, nccl().AllReduce(g->d_xchg, g->d_xchg, 1, NCCL_INT32, NCCL_SUM, g->comm, ctx->stream), "all-reduce of the shard sums");
  if (rc != 0) return rc;
  rc = fb_cuda_check(ctx, cudaMemcpyAsync(ctx->h_scalar, g->d_xchg, 4, cudaMemcpyDeviceToHost, ctx->stream), "scalar read");
  if (rc == 0) rc = fb_cuda_check(ctx, cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize");   // a scalar result is synchronous
  if (rc == 0) *out0 = *reinterpret_cast<int32_t *>(ctx->h_scalar);
  return rc;
}

int futhark_b200_group_scan_i32(struct futhark_b200_group *g, struct futhark_i32_1d **out0, const struct futhark_i32_1d *in0) {
  futhark_context *ctx = g->ctx;
  int32_t *mine = g->d_xchg + 4 * g->world;
  int rc = futhark_b200_reduce_i32_to_device(ctx, (CUdeviceptr)(uintptr_t)mine, in0);
  if (rc != 0) return rc;
  {
    CtxGuard guard(ctx);
    rc = group_check(g, nccl().AllGather(mine, g->d_xchg, 1, NCCL_INT32, g->comm, ctx->stream), "all-gather of the shard totals");
  }
  if (rc != 0) return rc;
  return futhark_b200_entry_scan_i32_carried(ctx, out0, in0, (CUdeviceptr)(uintptr_t)g->d_xchg, g->rank);
}

// ---- the summaries of the segmented scan exchanged by peer stores instead of a collective ------------
// Collective over the group, once: every rank allocates an exchange buffer, the ranks swap the
// buffers' IPC handles (one all-gather), and each maps the others' buffers.  From then on the
// scan kernel of a rank writes its shard's summary straight into the buffers of the ranks
// behind it, and a rank's carry kernel waits for the summaries of the ranks in front: no
// collective, no second stream, nothing between the kernels of a step.  The buffers hold 16
// generations; every eighth call the ranks meet in a one-word all-reduce on their streams, so no
// rank runs more than eight calls ahead of another and a generation is never overwritten before
// it was read.  Needs one process per GPU, or peer access between the GPUs of one process.
int futhark_b200_group_enable_peer_exchange(struct futhark_b200_group *g) {
  futhark_context *ctx = g->ctx;
  if (g->d_peer_bufs != nullptr) return 0;
  if (g->world > 64) { fb_set_error(ctx, "group: peer exchange supports at most 64 ranks"); return 1; }
  CtxGuard guard(ctx);
  struct Card { cudaIpcMemHandle_t handle; long long pid; unsigned long long ptr; int device; int pad; };
  const size_t bytes = fb::peer_exchange_bytes(g->world);
  int rc = fb_cuda_check(ctx, cudaMalloc((void **)&g->peer_buf, bytes), "peer exchange buffer");
  if (rc == 0) rc = fb_cuda_check(ctx, cudaMemset(g->peer_buf, 0, bytes), "peer exchange buffer");
  Card mine;
  memset(&mine, 0, sizeof(mine));
  if (rc == 0) rc = fb_cuda_check(ctx, cudaIpcGetMemHandle(&mine.handle, g->peer_buf), "cudaIpcGetMemHandle");
  if (rc != 0) return rc;
  mine.pid = (long long)getpid();
  mine.ptr = (unsigned long long)(uintptr_t)g->peer_buf;
  mine.device = ctx->device;
  Card *d_cards = nullptr, *h_cards = (Card *)malloc(sizeof(Card) * (size_t)g->world);
  rc = fb_cuda_check(ctx, cudaMalloc((void **)&d_cards, sizeof(Card) * (size_t)(g->world + 1)), "handle exchange");
  if (rc == 0) rc = fb_cuda_check(ctx, cudaMemcpyAsync(d_cards + g->world, &mine, sizeof(Card), cudaMemcpyHostToDevice, ctx->stream), "handle exchange");
  if (rc == 0) rc = group_check(g, nccl().AllGather(d_cards + g->world, d_cards, sizeof(Card), 0 /* ncclInt8 */, g->comm, ctx->stream), "all-gather of the buffer handles");
  if (rc == 0) rc = fb_cuda_check(ctx, cudaMemcpyAsync(h_cards, d_cards, sizeof(Card) * (size_t)g->world, cudaMemcpyDeviceToHost, ctx->stream), "handle exchange");
  if (rc == 0) rc = fb_cuda_check(ctx, cudaStreamSynchronize(ctx->stream), "handle exchange");
  uint32_t *bufs[64];
  for (int r = 0; r < g->world && rc == 0; r++) {
    if (r == g->rank) { bufs[r] = g->peer_buf; continue; }
    if (h_cards[r].pid == mine.pid) {                 // a rank in this process: its pointer is valid here once peer access is on
      int can = 0;
      cudaDeviceCanAccessPeer(&can, ctx->device, h_cards[r].device);
      if (!can) { fb_set_error(ctx, "group: GPU %d cannot address the memory of GPU %d", ctx->device, h_cards[r].device); rc = 1; break; }
      cudaError_t e = cudaDeviceEnablePeerAccess(h_cards[r].device, 0);
      if (e == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); e = cudaSuccess; }
      rc = fb_cuda_check(ctx, e, "cudaDeviceEnablePeerAccess");
      bufs[r] = reinterpret_cast<uint32_t *>((uintptr_t)h_cards[r].ptr);
    } else {
      void *p = nullptr;
      rc = fb_cuda_check(ctx, cudaIpcOpenMemHandle(&p, h_cards[r].handle, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
      g->opened[r] = p;
      bufs[r] = reinterpret_cast<uint32_t *>(p);
    }
  }
  if (rc == 0) rc = fb_cuda_check(ctx, cudaMalloc((void **)&g->d_peer_bufs, sizeof(uint32_t *) * (size_t)g->world), "peer table");
  if (rc == 0) rc = fb_cuda_check(ctx, cudaMemcpy(g->d_peer_bufs, bufs, sizeof(uint32_t *) * (size_t)g->world, cudaMemcpyHostToDevice), "peer table");
  // nobody writes into a buffer before every rank has mapped everything: one more collective
  if (rc == 0) rc = group_check(g, nccl().AllReduce(g->d_xchg, g->d_xchg, 1, NCCL_INT32, NCCL_SUM, g->comm, ctx->stream), "barrier");
  if (rc == 0) rc = fb_cuda_check(ctx, cudaStreamSynchronize(ctx->stream), "barrier");
  cudaFree(d_cards);
  free(h_cards);
  if (rc != 0 && g->d_peer_bufs != nullptr) { cudaFree(g->d_peer_bufs); g->d_peer_bufs = nullptr; }
  return rc;
}

// The segmented scan in two halves, so that the host can put other work of the step between the
// shard's scan (which sends the summary off) and the carry (which needs the others' summaries).
int futhark_b200_group_segscan_f32_begin(struct futhark_b200_group *g, const struct futhark_bool_1d *in0, const struct futhark_f32_1d *in1) {
  futhark_context *ctx = g->ctx;
  if (g->pending.out != nullptr) { fb_set_error(ctx, "group: a segmented scan is already in progress"); return 1; }
  CtxGuard guard(ctx);
  int32_t *mine = g->d_xchg + 4 * g->world;
  g->seq = g->seq == 0xfffffffeu ? 1u : g->seq + 1u;
  int rc = 0;
  futhark_f32_1d *out = nullptr;
  if (g->d_peer_bufs != nullptr) {
    if ((g->seq & 7u) == 0u)       // keep the ranks within eight calls of each other (see enable_peer_exchange)
      rc = group_check(g, nccl().AllReduce(g->d_xchg, g->d_xchg, 1, NCCL_INT32, NCCL_SUM, g->comm, ctx->stream), "pacing all-reduce");
    fb::PeerPush peer = {g->d_peer_bufs, g->rank, g->world, g->seq};
    if (rc == 0) rc = segscan_f32_locked(ctx, &out, in0, in1, reinterpret_cast<uint32_t *>(mine), &peer);
  } else {
    rc = segscan_f32_locked(ctx, &out, in0, in1, reinterpret_cast<uint32_t *>(mine), nullptr);
    if (rc == 0) rc = group_check(g, nccl().AllGather(mine, g->d_xchg, 4, NCCL_INT32, g->comm, ctx->stream), "all-gather of the shard summaries");
    if (rc != 0 && out != nullptr) { fb_unref(ctx, &out->mem); free(out); out = nullptr; }
  }
  if (rc != 0) return rc;
  g->pending.out = out;
  g->pending.seq = g->seq;
  return 0;
}

int futhark_b200_group_segscan_f32_finish(struct futhark_b200_group *g, struct futhark_f32_1d **out0, const struct futhark_bool_1d *in0) {
  futhark_context *ctx = g->ctx;
  futhark_f32_1d *out = g->pending.out;
  if (out == nullptr) { fb_set_error(ctx, "group: no segmented scan in progress"); return 1; }
  g->pending.out = nullptr;
  int rc;
  if (g->d_peer_bufs != nullptr) {
    CtxGuard guard(ctx);
    if (g->rank > 0 && out->shape[0] > 0) ctx->launch_count++;
    rc = fb_cuda_check(ctx, fb::launch_segscan_apply_carry_peer(gdptr<float>(out->mem), gdptr<uint8_t>(in0->mem), out->shape[0], g->peer_buf,
                                                                reinterpret_cast<const uint32_t *>(g->d_xchg + 4 * g->world), g->rank, g->world,
                                                                g->pending.seq, ctx->d_failure, ctx->num_sms, ctx->stream), "segscan carry");
    ctx->failure_is_an_option = true;
  } else {
    rc = futhark_b200_segscan_f32_apply_carries(ctx, out, in0, (CUdeviceptr)(uintptr_t)g->d_xchg, g->rank);
  }
  if (rc != 0) { futhark_free_f32_1d(ctx, out); return rc; }
  *out0 = out;
  return 0;
}

int futhark_b200_group_segscan_f32(struct futhark_b200_group *g, struct futhark_f32_1d **out0, const struct futhark_bool_1d *in0,
                                   const struct futhark_f32_1d *in1) {
  int rc = futhark_b200_group_segscan_f32_begin(g, in0, in1);
  if (rc != 0) return rc;
  return futhark_b200_group_segscan_f32_finish(g, out0, in0);
}

int futhark_b200_group_hist_add_i32(struct futhark_b200_group *g, struct futhark_i32_1d **out0, const int64_t in0,
                                    const struct futhark_i32_1d *in1, const struct futhark_i32_1d *in2) {
  futhark_context *ctx = g->ctx;
  futhark_i32_1d *out = nullptr;
  int rc = futhark_entry_hist_add_i32(ctx, &out, in0, in1, in2);
  if (rc != 0) return rc;
  if (in0 > 0) {
    CtxGuard guard(ctx);
    rc = group_check(g, nccl().AllReduce(gdptr<void>(out->mem), gdptr<void>(out->mem), (size_t)in0, NCCL_INT32, NCCL_SUM, g->comm, ctx->stream),
                     "all-reduce of the bins");
  }
  if (rc != 0) { futhark_free_i32_1d(ctx, out); return rc; }
  *out0 = out;
  return 0;
}

int futhark_b200_group_hist_max_f32(struct futhark_b200_group *g, struct futhark_f32_1d **out0, const int64_t in0,
                                    const struct futhark_i32_1d *in1, const struct futhark_f32_1d *in2) {
  futhark_context *ctx = g->ctx;
  futhark_f32_1d *out = nullptr;
  int rc = futhark_entry_hist_max_f32(ctx, &out, in0, in1, in2);
  if (rc != 0) return rc;
  if (in0 > 0) {
    CtxGuard guard(ctx);
    rc = group_check(g, nccl().AllReduce(gdptr<void>(out->mem), gdptr<void>(out->mem), (size_t)in0, NCCL_FLOAT32, NCCL_MAX, g->comm, ctx->stream),
                     "all-reduce of the bins");
  }
  if (rc != 0) { futhark_free_f32_1d(ctx, out); return rc; }
  *out0 = out;
  return 0;
}

// counts[0 .. k) of this rank -> where its pieces lie in the logical concatenation
static int gather_counts(futhark_b200_group *g, const int64_t *mine, int k, int64_t *all /* world * k */) {
  futhark_context *ctx = g->ctx;
  CtxGuard guard(ctx);
  int64_t *d = reinterpret_cast<int64_t *>(g->d_xchg);                 // 16 bytes per rank: up to two counts
  int64_t *dm = d + 2 * g->world;
  int rc = fb_cuda_check(ctx, cudaMemcpyAsync(dm, mine, (size_t)k * 8, cudaMemcpyHostToDevice, ctx->stream), "counts to the device");
  if (rc == 0) rc = group_check(g, nccl().AllGather(dm, d, (size_t)k, NCCL_INT64, g->comm, ctx->stream), "all-gather of the counts");
  if (rc == 0) rc = fb_cuda_check(ctx, cudaMemcpyAsync(all, d, (size_t)k * g->world * 8, cudaMemcpyDeviceToHost, ctx->stream), "counts to the host");
  if (rc == 0) rc = fb_cuda_check(ctx, cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize");
  return rc;
}

int futhark_b200_group_filter_u32(struct futhark_b200_group *g, struct futhark_u32_1d **out0, int64_t *offset, int64_t *total,
                                  const struct futhark_u32_1d *in0) {
  futhark_context *ctx = g->ctx;
  if (g->world > 1024) { fb_set_error(ctx, "group: more than 1024 ranks"); return 1; }
  futhark_u32_1d *out = nullptr;
  int rc = futhark_entry_filter_u32(ctx, &out, in0);
  if (rc != 0) return rc;
  int64_t mine = futhark_shape_u32_1d(ctx, out)[0], all[1024];
  rc = gather_counts(g, &mine, 1, all);
  if (rc != 0) { futhark_free_u32_1d(ctx, out); return rc; }
  int64_t off = 0, tot = 0;
  for (int r = 0; r < g->world; r++) { if (r < g->rank) off += all[r]; tot += all[r]; }
  *offset = off; *total = tot; *out0 = out;
  return 0;
}

int futhark_b200_group_partition_u32(struct futhark_b200_group *g, struct futhark_opaque_tup2_arr1d_u32_arr1d_u32 **out0,
                                     int64_t *sel_offset, int64_t *rej_offset, int64_t *total_selected, const struct futhark_u32_1d *in0) {
  futhark_context *ctx = g->ctx;
  if (g->world > 512) { fb_set_error(ctx, "group: more than 512 ranks"); return 1; }
  futhark_opaque_tup2_arr1d_u32_arr1d_u32 *pair = nullptr;
  int rc = futhark_entry_partition_u32(ctx, &pair, in0);
  if (rc != 0) return rc;
  int64_t mine[2] = {pair->v0->shape[0], pair->v1->shape[0]}, all[1024];
  rc = gather_counts(g, mine, 2, all);
  if (rc != 0) { futhark_free_opaque_tup2_arr1d_u32_arr1d_u32(ctx, pair); return rc; }
  int64_t so = 0, ro = 0, ts = 0;
  for (int r = 0; r < g->world; r++) { if (r < g->rank) { so += all[2 * r]; ro += all[2 * r + 1]; } ts += all[2 * r]; }
  *sel_offset = so; *rej_offset = ts + ro; *total_selected = ts; *out0 = pair;
  return 0;
}

// the contraction is sharded by whole batches: nothing to exchange
int futhark_b200_group_bmm_f16(struct futhark_b200_group *g, struct futhark_f32_3d **out0, const struct futhark_f16_3d *in0,
                               const struct futhark_f16_3d *in1) {
  return futhark_entry_bmm_f16(g->ctx, out0, in0, in1);
}

}  // extern "C"
