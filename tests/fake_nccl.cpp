// TEST INFRASTRUCTURE ONLY: a stand-in for libnccl.so.2 whose all-reduce behaves like a
// collective that a peer never joins — it cannot complete before the caller's deadline.
//
// Nothing waits on the GPU: the "collective" is a host function enqueued on the caller's
// stream that sleeps for FAKE_NCCL_STALL_MS (default 1500) and then returns, so the stream is
// merely not ready for that long and drains by itself afterwards. ncclCommAbort only records
// that it was called. tests/test_comm_deadline.py builds this file and points
// MUNET_B200_NCCL_LIBRARY at the result.
#include <atomic>
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <cuda_runtime.h>
#include <thread>

namespace {
std::atomic<int> g_aborts{0}, g_reduces{0};
int g_dummy_comm;
void CUDART_CB stall(void *) {
  const char *e = getenv("FAKE_NCCL_STALL_MS");
  const int ms = e ? atoi(e) : 1500;
  std::this_thread::sleep_for(std::chrono::milliseconds(ms));
}
} // namespace

extern "C" {
struct FakeId { char internal[128]; };
int ncclGetUniqueId(FakeId *id) { memset(id, 7, sizeof(*id)); return 0; }
int ncclCommInitRank(void **comm, int, FakeId, int) { *comm = &g_dummy_comm; return 0; }
int ncclCommDestroy(void *) { return 0; }
int ncclCommAbort(void *) { ++g_aborts; return 0; }
int ncclCommGetAsyncError(void *, int *err) { *err = 0; return 0; }
const char *ncclGetErrorString(int) { return "fake nccl error"; }
int ncclAllReduce(const void *, void *, size_t, int, int, void *, cudaStream_t stream) {
  ++g_reduces;
  return cudaLaunchHostFunc(stream, stall, nullptr) == cudaSuccess ? 0 : 1;
}
int fake_nccl_aborts() { return g_aborts.load(); }
int fake_nccl_reduces() { return g_reduces.load(); }
}
