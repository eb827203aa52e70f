// Expert parallelism: the communicator behind the two exchange steps of the MoE layer (see
// b200_moe_forward_ep in moe.cu).  NCCL is loaded at run time (dlopen of libnccl.so.2: the copy a host
// such as PyTorch has already loaded is reused, otherwise the system's), so the library has no link-time
// dependency on it and processes that never use expert parallelism never touch it.
//
//   dispatch = ncclAllGather of the ranks' token rows,
//   combine  = ncclReduceScatter (sum, f32) of the ranks' shares of every token's expert sum.
// Both are queued on the caller's stream; nothing synchronises.  b200_ep_wait is the host-side watchdog:
// it waits for the stream with a time limit, polls ncclCommGetAsyncError and aborts the communicator
// (ncclCommAbort) instead of waiting for ever when a peer has gone.
#include <cuda_bf16.h>
#include <dlfcn.h>
#include <nccl.h>

#include <cstring>

#include "common.h"

namespace {
struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
  ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*ReduceScatter)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  ncclResult_t (*GetVersion)(int*) = nullptr;
};
NcclApi g_nccl;

b200_status load_nccl() {
  if (g_nccl.handle) return B200_OK;
  const char* names[] = {getenv("DMLX_B200_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
  void* h = nullptr;
  for (const char* n : names) {
    if (!n || !*n) continue;
    h = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
    if (h) break;
  }
  if (!h) { b200_set_error("expert parallelism needs NCCL: libnccl.so.2 could not be loaded (%s)", dlerror()); return B200_ERR_UNSUPPORTED; }
#define SYM(field, name)                                                         \
  do {                                                                           \
    g_nccl.field = reinterpret_cast<decltype(g_nccl.field)>(dlsym(h, name));      \
    if (!g_nccl.field) { b200_set_error("NCCL symbol %s not found", name); dlclose(h); return B200_ERR_UNSUPPORTED; } \
  } while (0)
  SYM(GetUniqueId, "ncclGetUniqueId");
  SYM(CommInitRank, "ncclCommInitRank");
  SYM(CommDestroy, "ncclCommDestroy");
  SYM(CommAbort, "ncclCommAbort");
  SYM(CommGetAsyncError, "ncclCommGetAsyncError");
  SYM(AllGather, "ncclAllGather");
  SYM(ReduceScatter, "ncclReduceScatter");
  SYM(GetErrorString, "ncclGetErrorString");
  SYM(GetVersion, "ncclGetVersion");
#undef SYM
  g_nccl.handle = h;
  return B200_OK;
}

#define NCCL_TRY(expr)                                                                              \
  do {                                                                                              \
    ncclResult_t r_ = (expr);                                                                       \
    if (r_ != ncclSuccess && r_ != ncclInProgress) {                                                \
      b200_set_error("%s failed: %s", #expr, g_nccl.GetErrorString ? g_nccl.GetErrorString(r_) : "?"); \
      return B200_ERR_CUDA;                                                                         \
    }                                                                                               \
  } while (0)
}  // namespace

struct b200_ep {
  int rank = 0, world = 1;
  ncclComm_t comm = nullptr;
  cudaEvent_t mark = nullptr;
  bool aborted = false;
};

static_assert(sizeof(ncclUniqueId) == B200_EP_UNIQUE_ID_BYTES, "unique id size");

extern "C" {

b200_status b200_ep_unique_id(uint8_t* out) {
  b200_status st = load_nccl();
  if (st != B200_OK) return st;
  ncclUniqueId id;
  NCCL_TRY(g_nccl.GetUniqueId(&id));
  std::memcpy(out, &id, sizeof(id));
  return B200_OK;
}

b200_status b200_ep_create(int32_t rank, int32_t world, const uint8_t* unique_id, b200_ep** out) {
  *out = nullptr;
  b200_status st = b200_require_device();
  if (st != B200_OK) return st;
  if (world < 1 || rank < 0 || rank >= world || !unique_id) { b200_set_error("ep: rank %d of %d", rank, world); return B200_ERR_INVALID_ARGUMENT; }
  if ((st = load_nccl()) != B200_OK) return st;
  auto* ep = new b200_ep();
  ep->rank = rank;
  ep->world = world;
  ncclUniqueId id;
  std::memcpy(&id, unique_id, sizeof(id));
  ncclResult_t r = g_nccl.CommInitRank(&ep->comm, world, id, rank);
  if (r != ncclSuccess) {
    b200_set_error("ncclCommInitRank failed: %s", g_nccl.GetErrorString(r));
    delete ep;
    return B200_ERR_CUDA;
  }
  if (cudaEventCreateWithFlags(&ep->mark, cudaEventDisableTiming) != cudaSuccess) {
    b200_set_error("ep: event creation failed");
    g_nccl.CommDestroy(ep->comm);
    delete ep;
    return B200_ERR_CUDA;
  }
  *out = ep;
  return B200_OK;
}

void b200_ep_destroy(b200_ep* ep) {
  if (!ep) return;
  if (ep->comm && !ep->aborted) g_nccl.CommDestroy(ep->comm);
  if (ep->mark) cudaEventDestroy(ep->mark);
  delete ep;
}

int32_t b200_ep_rank(const b200_ep* ep) { return ep->rank; }
int32_t b200_ep_world(const b200_ep* ep) { return ep->world; }
int32_t b200_ep_nccl_version(void) {
  int v = 0;
  if (load_nccl() != B200_OK || g_nccl.GetVersion(&v) != ncclSuccess) return 0;
  return v;
}

b200_status b200_ep_dispatch(b200_ep* ep, const void* d_rows, void* d_rows_all, int32_t n_rows, int32_t hidden, void* stream) {
  if (ep->aborted) { b200_set_error("ep: the communicator was aborted"); return B200_ERR_DEVICE_FLAGGED; }
  if (n_rows <= 0) return B200_OK;
  NCCL_TRY(g_nccl.AllGather(d_rows, d_rows_all, (size_t)n_rows * hidden, ncclBfloat16, ep->comm, (cudaStream_t)stream));
  ++g_b200_launch_counter;
  return B200_OK;
}

b200_status b200_ep_combine(b200_ep* ep, const float* d_partial_all, float* d_sum, int32_t n_rows, int32_t hidden, void* stream) {
  if (ep->aborted) { b200_set_error("ep: the communicator was aborted"); return B200_ERR_DEVICE_FLAGGED; }
  if (n_rows <= 0) return B200_OK;
  NCCL_TRY(g_nccl.ReduceScatter(d_partial_all, d_sum, (size_t)n_rows * hidden, ncclFloat32, ncclSum, ep->comm, (cudaStream_t)stream));
  ++g_b200_launch_counter;
  return B200_OK;
}

b200_status b200_ep_abort(b200_ep* ep) {
  if (ep->comm && !ep->aborted) {
    g_nccl.CommAbort(ep->comm);
    ep->aborted = true;
  }
  return B200_OK;
}

}  // extern "C"

namespace {
int watch_done(void* ctx) { return cudaEventQuery(static_cast<b200_ep*>(ctx)->mark) != cudaErrorNotReady; }
int watch_error(void* ctx) {
  auto* ep = static_cast<b200_ep*>(ctx);
  ncclResult_t r = ncclSuccess;
  if (g_nccl.CommGetAsyncError(ep->comm, &r) != ncclSuccess) return 1;
  return r != ncclSuccess && r != ncclInProgress;
}
void watch_abort(void* ctx) { b200_ep_abort(static_cast<b200_ep*>(ctx)); }
}  // namespace

extern "C" b200_status b200_ep_wait(b200_ep* ep, void* stream, int32_t timeout_ms) {
  if (ep->aborted) { b200_set_error("ep: the communicator was aborted"); return B200_ERR_DEVICE_FLAGGED; }
  B200_CUDA_TRY(cudaEventRecord(ep->mark, (cudaStream_t)stream));
  b200_ep_watch_ops ops{watch_done, watch_error, watch_abort, ep};
  const int32_t r = b200_ep_watch(&ops, timeout_ms, 50);
  if (r == B200_EP_WATCH_DONE) {
    cudaError_t e = cudaEventQuery(ep->mark);
    if (e != cudaSuccess) { b200_set_error("ep: the stream ended with %s", cudaGetErrorString(e)); return B200_ERR_CUDA; }
    return B200_OK;
  }
  b200_set_error(r == B200_EP_WATCH_TIMEOUT ? "ep: collectives did not finish within %d ms; communicator aborted"
                                            : "ep: NCCL reported an asynchronous error; communicator aborted", timeout_ms);
  return B200_ERR_DEVICE_FLAGGED;
}
