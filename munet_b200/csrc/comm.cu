// NCCL-backed all-reduce behind the C ABI: the device-native form of
// Backend::all_reduce (src/core/backend.hpp:199; semantic = elementwise SUM over the
// participants, src/core/all_reduce_runtime.hpp:85-133), which the reference only
// implements by staging every buffer through host memory.
//
// One communicator per process and device (one process per GPU). NCCL is bound at run
// time with dlopen("libnccl.so.2") so that the library has no link-time dependency and
// shares the NCCL already loaded by the host process (torch's, when present).
// The collective runs over NVLink 5 / NVSwitch; the kernels here never read a peer's
// memory themselves.
#include "../../include/munet_b200.h"
#include <cstdio>
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <mutex>
#include <new>

namespace {

// The handful of NCCL declarations this file needs (stable since NCCL 2.10).
struct NcclUniqueId { char internal[128]; };
typedef struct ncclComm *NcclComm;
enum { kNcclInt32 = 2, kNcclFloat32 = 7, kNcclBfloat16 = 9, kNcclSum = 0, kNcclSuccess = 0 };

struct NcclApi {
  void *handle = nullptr;
  int (*GetUniqueId)(NcclUniqueId *) = nullptr;
  int (*CommInitRank)(NcclComm *, int, NcclUniqueId, int) = nullptr;
  int (*CommDestroy)(NcclComm) = nullptr;
  int (*CommAbort)(NcclComm) = nullptr;
  int (*AllReduce)(const void *, void *, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
  int (*CommGetAsyncError)(NcclComm, int *) = nullptr;
  const char *(*GetErrorString)(int) = nullptr;
  bool ok = false;
};

NcclApi &api() {
  static NcclApi a;
  static std::once_flag once;
  std::call_once(once, [] {
    // MUNET_B200_NCCL_LIBRARY names another library with the same entry points (a site build of
    // NCCL; the tests put a stand-in there whose collective never completes in time).
    const char *path = getenv("MUNET_B200_NCCL_LIBRARY");
    a.handle = dlopen((path && path[0]) ? path : "libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!a.handle)
      return;
    auto sym = [&](const char *n) { return dlsym(a.handle, n); };
    a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(sym("ncclGetUniqueId"));
    a.CommInitRank = reinterpret_cast<decltype(a.CommInitRank)>(sym("ncclCommInitRank"));
    a.CommDestroy = reinterpret_cast<decltype(a.CommDestroy)>(sym("ncclCommDestroy"));
    a.CommAbort = reinterpret_cast<decltype(a.CommAbort)>(sym("ncclCommAbort"));
    a.AllReduce = reinterpret_cast<decltype(a.AllReduce)>(sym("ncclAllReduce"));
    a.CommGetAsyncError = reinterpret_cast<decltype(a.CommGetAsyncError)>(sym("ncclCommGetAsyncError"));
    a.GetErrorString = reinterpret_cast<decltype(a.GetErrorString)>(sym("ncclGetErrorString"));
    a.ok = a.GetUniqueId && a.CommInitRank && a.CommDestroy && a.AllReduce && a.GetErrorString;
  });
  return a;
}

} // namespace

struct mu_comm {
  NcclComm comm = nullptr;
  int rank = 0, world = 1;
  bool aborted = false; // ncclCommAbort has run: the handle is gone, every later call fails
};

extern "C" {
int mu_set_error(mu_ctx *ctx, int code, const char *msg);

int mu_comm_unique_id(void *out, size_t capacity) {
  if (!out || capacity < sizeof(NcclUniqueId))
    return MU_ERR_INVALID;
  NcclApi &a = api();
  if (!a.ok)
    return MU_ERR_UNSUPPORTED;
  NcclUniqueId id;
  if (a.GetUniqueId(&id) != kNcclSuccess)
    return MU_ERR_CUDA;
  memcpy(out, &id, sizeof(id));
  return MU_OK;
}

int mu_comm_create(mu_ctx *ctx, const void *unique_id, int rank, int world, mu_comm **out) {
  if (!ctx || !unique_id || !out || world <= 0 || rank < 0 || rank >= world)
    return MU_ERR_INVALID;
  *out = nullptr;
  NcclApi &a = api();
  if (!a.ok)
    return mu_set_error(ctx, MU_ERR_UNSUPPORTED, "all_reduce: libnccl.so.2 could not be loaded");
  mu_comm *c = new (std::nothrow) mu_comm();
  if (!c)
    return MU_ERR_NOMEM;
  NcclUniqueId id;
  memcpy(&id, unique_id, sizeof(id));
  const int rc = a.CommInitRank(&c->comm, world, id, rank);
  if (rc != kNcclSuccess) {
    delete c;
    return mu_set_error(ctx, MU_ERR_CUDA, a.GetErrorString(rc));
  }
  c->rank = rank, c->world = world;
  *out = c;
  return MU_OK;
}

void mu_comm_destroy(mu_comm *comm) {
  if (!comm)
    return;
  if (comm->comm && !comm->aborted)
    api().CommDestroy(comm->comm);
  delete comm;
}

int mu_comm_rank(const mu_comm *comm) { return comm ? comm->rank : 0; }
int mu_comm_world(const mu_comm *comm) { return comm ? comm->world : 1; }

// In-place elementwise sum over every rank of the communicator, asynchronous on `stream`.
int mu_all_reduce_sum(mu_ctx *ctx, mu_comm *comm, void *buffer, long long n, int dtype,
                      void *stream) {
  if (!ctx)
    return MU_ERR_INVALID;
  if (n < 0)
    return mu_set_error(ctx, MU_ERR_INVALID, "all_reduce: negative element count");
  if (!comm || comm->world == 1 || n == 0)
    return MU_OK; // a single participant: the sum is the buffer itself
  if (!buffer)
    return mu_set_error(ctx, MU_ERR_INVALID, "all_reduce: null buffer");
  if (comm->aborted)
    return mu_set_error(ctx, MU_ERR_CUDA, "all_reduce: the communicator was aborted after a timeout");
  int nd;
  if (dtype == MU_F32) nd = kNcclFloat32;
  else if (dtype == MU_BF16) nd = kNcclBfloat16;
  else if (dtype == MU_I32) nd = kNcclInt32;
  else return mu_set_error(ctx, MU_ERR_UNSUPPORTED, "all_reduce: unsupported dtype");
  NcclApi &a = api();
  const int rc = a.AllReduce(buffer, buffer, static_cast<size_t>(n), nd, kNcclSum, comm->comm,
                             static_cast<cudaStream_t>(stream));
  if (rc != kNcclSuccess)
    return mu_set_error(ctx, MU_ERR_CUDA, a.GetErrorString(rc));
  return MU_OK;
}

// Non-blocking health check of the communicator (a failed or departed peer shows up
// here on the host; nothing waits on the device).
int mu_comm_check(mu_ctx *ctx, mu_comm *comm) {
  if (!ctx)
    return MU_ERR_INVALID;
  if (!comm || !comm->comm)
    return MU_OK;
  if (comm->aborted)
    return mu_set_error(ctx, MU_ERR_CUDA, "all_reduce: the communicator was aborted after a timeout");
  NcclApi &a = api();
  if (!a.CommGetAsyncError)
    return MU_OK;
  int async_err = 0;
  const int rc = a.CommGetAsyncError(comm->comm, &async_err);
  if (rc != kNcclSuccess || async_err != kNcclSuccess)
    return mu_set_error(ctx, MU_ERR_CUDA, a.GetErrorString(rc != kNcclSuccess ? rc : async_err));
  return MU_OK;
}

// Tear the communicator down without waiting for the peers (ncclCommAbort): collectives of this
// rank that are still in flight end, the handle becomes unusable.
int mu_comm_abort(mu_comm *comm) {
  if (!comm || !comm->comm || comm->aborted)
    return MU_OK;
  NcclApi &a = api();
  comm->aborted = true;
  if (a.CommAbort)
    a.CommAbort(comm->comm);
  return MU_OK;
}

// Host deadline around the collectives already enqueued on `stream`: polls the stream (and the
// communicator's asynchronous error) until the work has completed or `timeout_ms` has passed.
// The reference waits that long for every participant to arrive and then throws
// "all_reduce: timeout waiting for participants" (src/core/all_reduce_runtime.hpp:205-225,
// MUNET_ALLREDUCE_TIMEOUT_MS, default 10 s). A participant that never joins shows up here the
// same way: the collective cannot finish, the deadline passes, the communicator is aborted so
// that nothing of it stays on the device, and MU_ERR_TIMEOUT comes back with that message.
int mu_comm_wait(mu_ctx *ctx, mu_comm *comm, void *stream, int timeout_ms) {
  if (!ctx)
    return MU_ERR_INVALID;
  if (timeout_ms <= 0) {
    const char *env = getenv("MUNET_ALLREDUCE_TIMEOUT_MS");
    timeout_ms = env ? atoi(env) : 0;
    if (timeout_ms <= 0)
      timeout_ms = 10000;
  }
  const auto t0 = std::chrono::steady_clock::now();
  NcclApi &a = api();
  for (;;) {
    const cudaError_t q = cudaStreamQuery(static_cast<cudaStream_t>(stream));
    if (q == cudaSuccess)
      return MU_OK;
    if (q != cudaErrorNotReady)
      return mu_set_error(ctx, MU_ERR_CUDA, cudaGetErrorString(q));
    if (comm && comm->comm && !comm->aborted && a.CommGetAsyncError) {
      int async_err = 0;
      if (a.CommGetAsyncError(comm->comm, &async_err) == kNcclSuccess && async_err != kNcclSuccess) {
        mu_comm_abort(comm);
        return mu_set_error(ctx, MU_ERR_CUDA, a.GetErrorString(async_err));
      }
    }
    const auto waited = std::chrono::duration_cast<std::chrono::milliseconds>(
                            std::chrono::steady_clock::now() - t0).count();
    if (waited >= timeout_ms) {
      mu_comm_abort(comm);
      char msg[160];
      snprintf(msg, sizeof(msg), "all_reduce: timeout waiting for participants (waited %d ms)", timeout_ms);
      return mu_set_error(ctx, MU_ERR_TIMEOUT, msg);
    }
    std::this_thread::sleep_for(std::chrono::microseconds(200));
  }
}
}
