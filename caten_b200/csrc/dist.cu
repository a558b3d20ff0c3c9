// Multi-GPU plane of the C ABI: one process per GPU, sequences sharded, weights replicated.
// Two collectives exist on this path and both are thin NCCL calls on the context's stream:
// the broadcast of the packed weight arena from one rank at load, and the all-gather of the
// next-token ids.  Sequences never interact (external/llm/layers.lisp:35-51), so nothing else
// crosses NVLink.  The reference has no distributed component (its multi-device support is a
// roadmap item); these entry points exist so that a Common Lisp host, which cannot reach
// torch.distributed, can shard a batch through CFFI.
//
// NCCL is bound at run time (dlopen of libnccl.so.2) with the handful of prototypes declared
// here, so the library neither needs NCCL's header to build nor NCCL itself to load on a
// single-GPU host.  When the process has already loaded an NCCL (PyTorch bundles one), dlopen
// returns that copy.
#include <dlfcn.h>
#include <string.h>

#include <mutex>

#include "common.cuh"

namespace cb {

// The part of NCCL's public C API used here (nccl.h, stable since 2.x).
typedef struct { char internal[128]; } NcclUniqueId;
typedef void *NcclComm;
enum { NCCL_SUCCESS = 0, NCCL_UINT8 = 1, NCCL_INT64 = 4 };
struct NcclApi {
  void *handle = nullptr;
  int (*GetUniqueId)(NcclUniqueId *) = nullptr;
  int (*CommInitRank)(NcclComm *, int, NcclUniqueId, int) = nullptr;
  int (*CommDestroy)(NcclComm) = nullptr;
  int (*Broadcast)(const void *, void *, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
  int (*AllGather)(const void *, void *, size_t, int, NcclComm, cudaStream_t) = nullptr;
  const char *(*GetErrorString)(int) = nullptr;
  std::string why;  // why binding failed
};

static NcclApi *nccl_api() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    for (const char *name : {"libnccl.so.2", "libnccl.so"}) {
      api.handle = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
      if (api.handle) break;
    }
    if (!api.handle) { api.why = "libnccl.so.2 not found (dlopen)"; return; }
    auto sym = [&](const char *n) { void *p = dlsym(api.handle, n); if (!p && api.why.empty()) api.why = std::string("NCCL symbol missing: ") + n; return p; };
    api.GetUniqueId = (int (*)(NcclUniqueId *))sym("ncclGetUniqueId");
    api.CommInitRank = (int (*)(NcclComm *, int, NcclUniqueId, int))sym("ncclCommInitRank");
    api.CommDestroy = (int (*)(NcclComm))sym("ncclCommDestroy");
    api.Broadcast = (int (*)(const void *, void *, size_t, int, int, NcclComm, cudaStream_t))sym("ncclBroadcast");
    api.AllGather = (int (*)(const void *, void *, size_t, int, NcclComm, cudaStream_t))sym("ncclAllGather");
    api.GetErrorString = (const char *(*)(int))sym("ncclGetErrorString");
  });
  return &api;
}

static int nccl_fail(caten_b200_ctx *ctx, NcclApi *api, int rc, const char *what) {
  return fail(ctx, CATEN_B200_ECUDA, "%s: %s", what, api->GetErrorString ? api->GetErrorString(rc) : "NCCL error");
}

}  // namespace cb

using namespace cb;

extern "C" {

int caten_b200_dist_unique_id(void *id128) {
  if (!id128) return fail(nullptr, CATEN_B200_EINVAL, "dist_unique_id: NULL output");
  NcclApi *api = nccl_api();
  if (!api->why.empty()) return fail(nullptr, CATEN_B200_EUNSUPPORTED, "dist_unique_id: %s", api->why.c_str());
  NcclUniqueId id;
  const int rc = api->GetUniqueId(&id);
  if (rc != NCCL_SUCCESS) return nccl_fail(nullptr, api, rc, "ncclGetUniqueId");
  memcpy(id128, &id, sizeof id);
  return 0;
}

int caten_b200_dist_init(caten_b200_ctx *ctx, int rank, int world, const void *id128) {
  if (!ctx) return fail(nullptr, CATEN_B200_EINVAL, "dist_init: ctx is NULL");
  cudaSetDevice(ctx->device);
  if (world < 1 || rank < 0 || rank >= world) return fail(ctx, CATEN_B200_EINVAL, "dist_init: rank %d of %d", rank, world);
  if (ctx->dist_comm) return fail(ctx, CATEN_B200_EINVAL, "dist_init: this context already belongs to a group of %d", ctx->dist_world);
  if (world == 1) { ctx->dist_rank = 0; ctx->dist_world = 1; return 0; }  // replicas only: nothing to set up
  if (!id128) return fail(ctx, CATEN_B200_EINVAL, "dist_init: the group id is NULL");
  NcclApi *api = nccl_api();
  if (!api->why.empty()) return fail(ctx, CATEN_B200_EUNSUPPORTED, "dist_init: %s", api->why.c_str());
  NcclUniqueId id;
  memcpy(&id, id128, sizeof id);
  NcclComm comm = nullptr;
  const int rc = api->CommInitRank(&comm, world, id, rank);
  if (rc != NCCL_SUCCESS) return nccl_fail(ctx, api, rc, "ncclCommInitRank");
  ctx->dist_comm = comm;
  ctx->dist_rank = rank;
  ctx->dist_world = world;
  return 0;
}

int caten_b200_dist_finalize(caten_b200_ctx *ctx) {
  if (!ctx) return fail(nullptr, CATEN_B200_EINVAL, "dist_finalize: ctx is NULL");
  if (ctx->dist_comm) {
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    nccl_api()->CommDestroy(ctx->dist_comm);
    ctx->dist_comm = nullptr;
  }
  ctx->dist_world = 1;
  ctx->dist_rank = 0;
  return 0;
}

int caten_b200_dist_rank(caten_b200_ctx *ctx) { return ctx ? ctx->dist_rank : -1; }
int caten_b200_dist_world(caten_b200_ctx *ctx) { return ctx ? ctx->dist_world : -1; }

int caten_b200_dist_shard(int64_t batch, int world, int rank, int64_t *first, int64_t *count) {
  if (world < 1 || rank < 0 || rank >= world || batch < 0 || !first || !count)
    return fail(nullptr, CATEN_B200_EINVAL, "dist_shard: rank %d of %d, batch %lld", rank, world, (long long)batch);
  const int64_t base = batch / world, rem = batch % world;
  *count = base + (rank < rem ? 1 : 0);
  *first = rank * base + (rank < rem ? rank : rem);
  return 0;
}

int caten_b200_dist_bcast_weights(caten_b200_ctx *ctx, void *d_arena, size_t bytes, int root) {
  if (!ctx) return fail(nullptr, CATEN_B200_EINVAL, "dist_bcast_weights: ctx is NULL");
  cudaSetDevice(ctx->device);
  if (ctx->dist_world == 1) return 0;
  if (!ctx->dist_comm) return fail(ctx, CATEN_B200_EINVAL, "dist_bcast_weights: call caten_b200_dist_init first");
  if (bytes && !d_arena) return fail(ctx, CATEN_B200_EINVAL, "dist_bcast_weights: NULL buffer");
  if (root < 0 || root >= ctx->dist_world) return fail(ctx, CATEN_B200_EINVAL, "dist_bcast_weights: root %d of %d", root, ctx->dist_world);
  NcclApi *api = nccl_api();
  const int rc = api->Broadcast(d_arena, d_arena, bytes, NCCL_UINT8, root, ctx->dist_comm, ctx->stream);
  if (rc != NCCL_SUCCESS) return nccl_fail(ctx, api, rc, "ncclBroadcast");
  ctx->weights_pending = true;  // kernels that read weights early must not overtake the broadcast
  return 0;
}

int caten_b200_dist_gather_ids(caten_b200_ctx *ctx, const int64_t *d_local, int64_t n_per_rank, int64_t *d_all) {
  if (!ctx) return fail(nullptr, CATEN_B200_EINVAL, "dist_gather_ids: ctx is NULL");
  cudaSetDevice(ctx->device);
  if (n_per_rank < 0 || (n_per_rank && (!d_local || !d_all))) return fail(ctx, CATEN_B200_EINVAL, "dist_gather_ids: bad argument");
  if (ctx->dist_world == 1) {
    if (d_all != d_local) CB_CUDA(ctx, cudaMemcpyAsync(d_all, d_local, (size_t)n_per_rank * sizeof(int64_t), cudaMemcpyDeviceToDevice, ctx->stream));
    return 0;
  }
  if (!ctx->dist_comm) return fail(ctx, CATEN_B200_EINVAL, "dist_gather_ids: call caten_b200_dist_init first");
  NcclApi *api = nccl_api();
  const int rc = api->AllGather(d_local, d_all, (size_t)n_per_rank, NCCL_INT64, ctx->dist_comm, ctx->stream);
  if (rc != NCCL_SUCCESS) return nccl_fail(ctx, api, rc, "ncclAllGather");
  return 0;
}

}  // extern "C"
