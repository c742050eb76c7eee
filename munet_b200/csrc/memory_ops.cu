// Memory entry points of the C ABI that are not plain copies: fill, strided gather, and the
// event pair behind the profiler's "last kernel time".
//
// Backend::memset / to_contiguous / get_last_kernel_time_us (src/core/backend.hpp:207-232;
// CUDA reference src/backend/cuda_backend.cu:827-840, 946-961, 1709-1726).
#include "../../include/munet_b200.h"
#include <cstdio>
#include <cuda_runtime.h>
#include <mutex>
#include <unordered_map>

extern "C" {
int mu_set_error(mu_ctx *ctx, int code, const char *msg);
int mu_ctx_select_device(mu_ctx *ctx);
int mu_ctx_num_sms(const mu_ctx *ctx);
}

namespace {

constexpr int MAX_DIMS = 6;

struct GatherArgs {
  long long extent[MAX_DIMS]; // output extents, outermost first, padded with 1 in front
  long long stride[MAX_DIMS]; // source strides in elements, same order
  long long offset;           // source offset in elements
  long long total;            // output elements
};

// dst[linear] = src[offset + sum_d idx_d * stride_d]: the row-major walk of a strided view.
// One thread handles VEC consecutive output elements of the innermost dimension when that
// dimension is contiguous in the source (inner_contig), so permutes that keep the last axis
// (head split / merge) move 16 bytes per thread; any other view moves one element per thread.
template <typename T, int VEC>
__global__ void to_contiguous_kernel(const T *__restrict__ src, T *__restrict__ dst, GatherArgs a) {
  const long long n_vec = a.total / VEC;
  for (long long v = blockIdx.x * 1ll * blockDim.x + threadIdx.x; v < n_vec;
       v += 1ll * gridDim.x * blockDim.x) {
    long long rem = v * VEC, off = a.offset;
#pragma unroll
    for (int d = MAX_DIMS - 1; d >= 0; --d) {
      const long long e = a.extent[d];
      off += (rem % e) * a.stride[d];
      rem /= e;
    }
    if (VEC == 1) {
      dst[v] = src[off];
    } else {
      struct alignas(sizeof(T) * VEC) Pack { T x[VEC]; };
      *reinterpret_cast<Pack *>(dst + v * VEC) = *reinterpret_cast<const Pack *>(src + off);
    }
  }
}

template <typename T>
int launch_gather(const void *src, void *dst, const GatherArgs &a, bool inner_contig, int sms,
                  cudaStream_t st) {
  constexpr int VEC = 16 / sizeof(T);
  const long long inner = a.extent[MAX_DIMS - 1];
  bool vec = inner_contig && VEC > 1 && inner % VEC == 0 && a.offset % VEC == 0 &&
             (reinterpret_cast<uintptr_t>(src) & 15u) == 0 && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0;
  for (int d = 0; d < MAX_DIMS - 1 && vec; ++d)
    vec = a.stride[d] % VEC == 0;
  const long long work = vec ? a.total / VEC : a.total;
  const int threads = 256;
  long long blocks = (work + threads - 1) / threads;
  const long long cap = 1ll * sms * 16;
  if (blocks > cap)
    blocks = cap;
  if (blocks < 1)
    blocks = 1;
  if (vec)
    to_contiguous_kernel<T, VEC><<<static_cast<unsigned>(blocks), threads, 0, st>>>(
        static_cast<const T *>(src), static_cast<T *>(dst), a);
  else
    to_contiguous_kernel<T, 1><<<static_cast<unsigned>(blocks), threads, 0, st>>>(
        static_cast<const T *>(src), static_cast<T *>(dst), a);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

// Event pairs of mu_timer_*: one per context, created on first use.
struct Timer {
  cudaEvent_t start = nullptr, stop = nullptr;
  bool armed = false, closed = false;
};
std::mutex g_timer_mu;
std::unordered_map<const mu_ctx *, Timer> g_timers;

} // namespace

extern "C" {

int mu_memset(mu_ctx *ctx, void *ptr, int value, size_t bytes, void *stream) {
  if (!ctx)
    return MU_ERR_INVALID;
  if (bytes == 0)
    return MU_OK;
  if (!ptr)
    return mu_set_error(ctx, MU_ERR_INVALID, "memset: null pointer");
  if (mu_ctx_select_device(ctx) != MU_OK)
    return mu_set_error(ctx, MU_ERR_CUDA, "memset: cannot select device");
  const cudaError_t e = cudaMemsetAsync(ptr, value, bytes, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? MU_OK : mu_set_error(ctx, MU_ERR_CUDA, cudaGetErrorString(e));
}

int mu_to_contiguous(mu_ctx *ctx, const void *src, void *dst, int ndim, const int *shape,
                     const long long *strides, long long offset, int elem_size, void *stream) {
  if (!ctx)
    return MU_ERR_INVALID;
  if (ndim < 0 || ndim > MAX_DIMS)
    return mu_set_error(ctx, MU_ERR_UNSUPPORTED, "to_contiguous: at most 6 dimensions");
  if ((ndim > 0 && (!shape || !strides)) || offset < 0)
    return mu_set_error(ctx, MU_ERR_INVALID, "to_contiguous: bad shape/strides/offset");
  if (elem_size != 1 && elem_size != 2 && elem_size != 4 && elem_size != 8)
    return mu_set_error(ctx, MU_ERR_UNSUPPORTED, "to_contiguous: element size must be 1, 2, 4 or 8 bytes");
  GatherArgs a;
  a.offset = offset, a.total = 1;
  for (int d = 0; d < MAX_DIMS; ++d)
    a.extent[d] = 1, a.stride[d] = 0;
  for (int d = 0; d < ndim; ++d) {
    if (shape[d] < 0 || strides[d] < 0)
      return mu_set_error(ctx, MU_ERR_INVALID, "to_contiguous: negative extent or stride");
    a.extent[MAX_DIMS - ndim + d] = shape[d];
    a.stride[MAX_DIMS - ndim + d] = strides[d];
    a.total *= shape[d];
  }
  if (a.total == 0)
    return MU_OK;
  if (!src || !dst)
    return mu_set_error(ctx, MU_ERR_INVALID, "to_contiguous: null pointer");
  if (mu_ctx_select_device(ctx) != MU_OK)
    return mu_set_error(ctx, MU_ERR_CUDA, "to_contiguous: cannot select device");
  const bool inner_contig = ndim > 0 && (strides[ndim - 1] == 1 || shape[ndim - 1] == 1);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int sms = mu_ctx_num_sms(ctx);
  int rc;
  switch (elem_size) {
  case 1: rc = launch_gather<unsigned char>(src, dst, a, inner_contig, sms, st); break;
  case 2: rc = launch_gather<unsigned short>(src, dst, a, inner_contig, sms, st); break;
  case 4: rc = launch_gather<unsigned int>(src, dst, a, inner_contig, sms, st); break;
  default: rc = launch_gather<unsigned long long>(src, dst, a, inner_contig, sms, st); break;
  }
  return rc == 0 ? MU_OK : mu_set_error(ctx, MU_ERR_CUDA, cudaGetErrorString(cudaGetLastError()));
}

int mu_timer_begin(mu_ctx *ctx, void *stream) {
  if (!ctx)
    return MU_ERR_INVALID;
  if (mu_ctx_select_device(ctx) != MU_OK)
    return mu_set_error(ctx, MU_ERR_CUDA, "timer: cannot select device");
  std::lock_guard<std::mutex> lock(g_timer_mu);
  Timer &t = g_timers[ctx];
  if (!t.start && (cudaEventCreate(&t.start) != cudaSuccess || cudaEventCreate(&t.stop) != cudaSuccess))
    return mu_set_error(ctx, MU_ERR_CUDA, "timer: event creation failed");
  t.closed = false;
  t.armed = cudaEventRecord(t.start, static_cast<cudaStream_t>(stream)) == cudaSuccess;
  return t.armed ? MU_OK : mu_set_error(ctx, MU_ERR_CUDA, "timer: event record failed");
}

int mu_timer_end(mu_ctx *ctx, void *stream) {
  if (!ctx)
    return MU_ERR_INVALID;
  std::lock_guard<std::mutex> lock(g_timer_mu);
  auto it = g_timers.find(ctx);
  if (it == g_timers.end() || !it->second.armed)
    return mu_set_error(ctx, MU_ERR_INVALID, "timer: end without begin");
  it->second.closed = cudaEventRecord(it->second.stop, static_cast<cudaStream_t>(stream)) == cudaSuccess;
  return it->second.closed ? MU_OK : mu_set_error(ctx, MU_ERR_CUDA, "timer: event record failed");
}

double mu_timer_last_us(mu_ctx *ctx) {
  if (!ctx)
    return 0.0;
  std::lock_guard<std::mutex> lock(g_timer_mu);
  auto it = g_timers.find(ctx);
  if (it == g_timers.end() || !it->second.armed || !it->second.closed)
    return 0.0;
  float ms = 0.f;
  if (cudaEventSynchronize(it->second.stop) != cudaSuccess ||
      cudaEventElapsedTime(&ms, it->second.start, it->second.stop) != cudaSuccess) {
    cudaGetLastError();
    return 0.0;
  }
  return static_cast<double>(ms) * 1000.0;
}

// called by mu_ctx_destroy
void mu_timer_release(mu_ctx *ctx) {
  std::lock_guard<std::mutex> lock(g_timer_mu);
  auto it = g_timers.find(ctx);
  if (it == g_timers.end())
    return;
  if (it->second.start)
    cudaEventDestroy(it->second.start);
  if (it->second.stop)
    cudaEventDestroy(it->second.stop);
  g_timers.erase(it);
}

} // extern "C"
