// Tensor-parallel exchange over peer memory: the sum of the two ranks' partial results of a
// row-parallel Linear, fused with the bias and residual adds that follow it.
//
// Stands in for Backend::all_reduce (src/core/backend.hpp:199; sum semantic
// src/core/all_reduce_runtime.hpp:85-133) followed by the bias add of nn::Linear
// (src/nn/linear.hpp:28-34) and the residual add of the decoder block. Where the NCCL path
// runs a reduce-scatter + all-gather kernel and then a separate elementwise pass over the
// result, this kernel reads the local partial from HBM and the peer's partial straight over
// NVLink (plain peer loads, 16 bytes per thread and load) and writes the finished residual
// stream once: y = bf16(bf16(bf16(a + a_peer) + bias) + residual), the same rounding chain as the
// NCCL path (a bf16 sum, then one rounding per add), and bit-identical on both ranks because
// a + a_peer commutes.
//
// Hand-shake. Each rank owns two 64-bit counters that only its PEER writes (through the peer
// mapping of the same allocation):
//   READY  the peer's partial of exchange number n is complete   (written after its GEMM)
//   DONE   the peer has finished reading this rank's partial n   (written by its reduce kernel)
// Exchange numbers grow monotonically over the life of the engine (step * exchanges-per-forward +
// index), so a counter never has to be reset and `>=` is the only comparison. Every wait is
// bounded: when it runs out the kernel latches MU_DEV_TIMEOUT_OTHER in the context's status
// word and returns without touching peer memory. No kernel here uses TMA, multicast or multimem.
#include "../../include/munet_b200.h"
#include "common.h"
#include "ptx.cuh"
#include <cstring>

namespace mu {

struct PeerFlags {
  unsigned long long ready;   // written by the peer
  unsigned long long done;    // written by the peer
  unsigned long long step;    // forwards started on this rank (local)
  unsigned int ctas_left;     // reduce kernel: CTAs still running (local)
  unsigned int pad;
};

__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long *p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned long long *p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// Bounded wait until *flag >= want. Returns false after MU_WAIT_LIMIT_NS.
__device__ __forceinline__ bool wait_at_least(const unsigned long long *flag, unsigned long long want) {
  if (ld_acquire_sys(flag) >= want)
    return true;
  const unsigned long long t0 = globaltimer_ns();
  while (ld_acquire_sys(flag) < want) {
    if (globaltimer_ns() - t0 > MU_WAIT_LIMIT_NS)
      return false;
    __nanosleep(200);
  }
  return true;
}

// One thread: a new forward starts on this rank.
__global__ void peer_step_kernel(PeerFlags *mine) { mine->step += 1; }

// One thread, after the GEMM that produced partial number `index` of this forward: tell the
// peer. `per_step` = exchanges per forward.
__global__ void peer_signal_kernel(const PeerFlags *mine, PeerFlags *peer, unsigned per_step, unsigned index) {
  __threadfence_system(); // the GEMM's stores (earlier kernel on this stream) are visible system-wide
  st_release_sys(&peer->ready, (mine->step - 1) * per_step + index + 1);
}

// One thread, before a GEMM overwrites a partial buffer: the peer must have finished reading
// every earlier partial of this rank (`index` = number of exchanges of this forward issued so far).
__global__ void peer_wait_done_kernel(const PeerFlags *mine, unsigned per_step, unsigned index, int *status) {
  const unsigned long long want = (mine->step - 1) * per_step + index;
  if (!wait_at_least(&mine->done, want))
    atomicCAS(status, 0, MU_DEV_TIMEOUT_OTHER);
}

// One thread, before a kernel reads what the peer pushed for exchange `index`: the peer's READY.
__global__ void peer_wait_ready_kernel(const PeerFlags *mine, unsigned per_step, unsigned index, int *status) {
  const unsigned long long want = (mine->step - 1) * per_step + index + 1;
  if (!wait_at_least(&mine->ready, want))
    atomicCAS(status, 0, MU_DEV_TIMEOUT_OTHER);
}

// One thread, after the kernel that consumed what the peer pushed for exchange `index`: the peer may
// overwrite that receive buffer (exchanges without a reduce kernel, which otherwise writes DONE).
__global__ void peer_signal_done_kernel(const PeerFlags *mine, PeerFlags *peer, unsigned per_step, unsigned index) {
  __threadfence_system();
  st_release_sys(&peer->done, (mine->step - 1) * per_step + index + 1);
}

// y = bf16(bf16(bf16(a + a_peer) + bias[col]) + residual), n elements, `cols` per row, 8 elements
// per thread and step. bias / residual may be null. y may alias residual (in-place residual stream).
__global__ void __launch_bounds__(512)
peer_reduce_kernel(const uint4 *__restrict__ a, const uint4 *__restrict__ a_peer, const uint4 *bias,
                   const uint4 *residual, uint4 *y, long long n_vec, int cols_vec, PeerFlags *mine,
                   PeerFlags *peer, unsigned per_step, unsigned index, int *status) {
  __shared__ int go;
  const unsigned long long seq = (mine->step - 1) * per_step + index + 1;
  if (threadIdx.x == 0) {
    go = wait_at_least(&mine->ready, seq) ? 1 : 0;
    if (!go)
      atomicCAS(status, 0, MU_DEV_TIMEOUT_OTHER);
  }
  __syncthreads();
  if (go) {
    // Eight independent 16-byte peer loads per thread are in flight before the first one is used
    // (an NVLink round trip is a few microseconds). ld.cv: never served from a line this SM
    // cached during an earlier exchange at the same address.
    constexpr int U = 8;
    const long long stride = 1ll * gridDim.x * blockDim.x;
    // column (in 16-byte vectors) of element i0 + u * stride, kept by addition: one 64-bit
    // modulo per thread instead of one per vector
    const int cstep = static_cast<int>(stride % cols_vec);
    int c0 = static_cast<int>((1ll * blockIdx.x * blockDim.x + threadIdx.x) % cols_vec);
    for (long long i0 = 1ll * blockIdx.x * blockDim.x + threadIdx.x; i0 < n_vec; i0 += stride * U) {
      uint4 vp[U], va[U], vr[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
        if (i < n_vec)
          vp[u] = __ldcv(a_peer + i);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
        if (i < n_vec) {
          va[u] = a[i];
          vr[u] = residual ? residual[i] : make_uint4(0, 0, 0, 0);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + u * stride;
        const int col = c0;
        c0 += cstep;
        if (c0 >= cols_vec)
          c0 -= cols_vec;
        if (i >= n_vec)
          break;
        uint4 vb = make_uint4(0, 0, 0, 0);
        if (bias)
          vb = __ldg(bias + col);
        const uint32_t wa[4] = {va[u].x, va[u].y, va[u].z, va[u].w}, wp[4] = {vp[u].x, vp[u].y, vp[u].z, vp[u].w};
        const uint32_t wb[4] = {vb.x, vb.y, vb.z, vb.w}, wr[4] = {vr[u].x, vr[u].y, vr[u].z, vr[u].w};
        uint32_t wo[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          float lo = bf16_round(bf16_lo(wa[k]) + bf16_lo(wp[k]));
          float hi = bf16_round(bf16_hi(wa[k]) + bf16_hi(wp[k]));
          if (bias) {
            lo = bf16_round(lo + bf16_lo(wb[k]));
            hi = bf16_round(hi + bf16_hi(wb[k]));
          }
          if (residual) {
            lo = bf16_round(lo + bf16_lo(wr[k]));
            hi = bf16_round(hi + bf16_hi(wr[k]));
          }
          wo[k] = pack_bf16x2(lo, hi);
        }
        y[i] = make_uint4(wo[0], wo[1], wo[2], wo[3]);
      }
    }
  }
  // the last CTA to finish tells the peer that this rank is done reading its partial
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicSub(&mine->ctas_left, 1u) == 1u) {
      mine->ctas_left = gridDim.x; // re-armed for the next launch (launches are stream-ordered)
      __threadfence_system();
      if (go)
        st_release_sys(&peer->done, seq);
    }
  }
}

// One thread: arm the CTA counter for a grid of `ctas` (every reduce launch uses the same grid).
__global__ void peer_arm_kernel(PeerFlags *mine, unsigned ctas) { mine->ctas_left = ctas; }

} // namespace mu

extern "C" {
int mu_set_error(mu_ctx *ctx, int code, const char *msg);
int mu_ctx_select_device(mu_ctx *ctx);
int *mu_ctx_status_ptr(mu_ctx *ctx);
int mu_ctx_num_sms(const mu_ctx *ctx);

size_t mu_peer_flags_bytes(void) { return sizeof(mu::PeerFlags); }

int mu_ipc_export(mu_ctx *ctx, const void *device_ptr, void *handle_out, size_t capacity) {
  if (!ctx || !device_ptr || !handle_out || capacity < sizeof(cudaIpcMemHandle_t))
    return MU_ERR_INVALID;
  if (mu_ctx_select_device(ctx) != MU_OK)
    return mu_set_error(ctx, MU_ERR_CUDA, "ipc export: cannot select device");
  cudaIpcMemHandle_t h;
  const cudaError_t e = cudaIpcGetMemHandle(&h, const_cast<void *>(device_ptr));
  if (e != cudaSuccess)
    return mu_set_error(ctx, MU_ERR_CUDA, cudaGetErrorString(e));
  memcpy(handle_out, &h, sizeof(h));
  return MU_OK;
}

int mu_ipc_open(mu_ctx *ctx, const void *handle, void **peer_ptr) {
  if (!ctx || !handle || !peer_ptr)
    return MU_ERR_INVALID;
  *peer_ptr = nullptr;
  if (mu_ctx_select_device(ctx) != MU_OK)
    return mu_set_error(ctx, MU_ERR_CUDA, "ipc open: cannot select device");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  const cudaError_t e = cudaIpcOpenMemHandle(peer_ptr, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess)
    return mu_set_error(ctx, MU_ERR_CUDA, cudaGetErrorString(e));
  return MU_OK;
}

int mu_ipc_close(mu_ctx *ctx, void *peer_ptr) {
  if (!ctx)
    return MU_ERR_INVALID;
  if (!peer_ptr)
    return MU_OK;
  const cudaError_t e = cudaIpcCloseMemHandle(peer_ptr);
  return e == cudaSuccess ? MU_OK : mu_set_error(ctx, MU_ERR_CUDA, cudaGetErrorString(e));
}

// ---- launchers used by the executor (not part of the declared ABI) ----
int mu_peer_arm(mu_ctx *ctx, void *flags, unsigned ctas, void *stream) {
  if (mu_ctx_select_device(ctx) != MU_OK)
    return MU_ERR_CUDA;
  mu::peer_arm_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<mu::PeerFlags *>(flags), ctas);
  return cudaGetLastError() == cudaSuccess ? MU_OK : MU_ERR_CUDA;
}
int mu_peer_step(mu_ctx *ctx, void *flags, void *stream) {
  if (mu_ctx_select_device(ctx) != MU_OK)
    return MU_ERR_CUDA;
  mu::peer_step_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<mu::PeerFlags *>(flags));
  return cudaGetLastError() == cudaSuccess ? MU_OK : MU_ERR_CUDA;
}
int mu_peer_signal(mu_ctx *ctx, void *flags, void *peer_flags, unsigned per_step, unsigned index, void *stream) {
  if (mu_ctx_select_device(ctx) != MU_OK)
    return MU_ERR_CUDA;
  mu::peer_signal_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const mu::PeerFlags *>(flags), static_cast<mu::PeerFlags *>(peer_flags), per_step, index);
  return cudaGetLastError() == cudaSuccess ? MU_OK : MU_ERR_CUDA;
}
int mu_peer_wait_done(mu_ctx *ctx, void *flags, unsigned per_step, unsigned index, void *stream) {
  if (mu_ctx_select_device(ctx) != MU_OK)
    return MU_ERR_CUDA;
  mu::peer_wait_done_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const mu::PeerFlags *>(flags), per_step, index, mu_ctx_status_ptr(ctx));
  return cudaGetLastError() == cudaSuccess ? MU_OK : MU_ERR_CUDA;
}
int mu_peer_wait_ready(mu_ctx *ctx, void *flags, unsigned per_step, unsigned index, void *stream) {
  if (mu_ctx_select_device(ctx) != MU_OK)
    return MU_ERR_CUDA;
  mu::peer_wait_ready_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const mu::PeerFlags *>(flags), per_step, index, mu_ctx_status_ptr(ctx));
  return cudaGetLastError() == cudaSuccess ? MU_OK : MU_ERR_CUDA;
}
int mu_peer_signal_done(mu_ctx *ctx, void *flags, void *peer_flags, unsigned per_step, unsigned index, void *stream) {
  if (mu_ctx_select_device(ctx) != MU_OK)
    return MU_ERR_CUDA;
  mu::peer_signal_done_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const mu::PeerFlags *>(flags), static_cast<mu::PeerFlags *>(peer_flags), per_step, index);
  return cudaGetLastError() == cudaSuccess ? MU_OK : MU_ERR_CUDA;
}
// n elements of bf16 (n and cols multiples of 8, pointers 16-byte aligned); `ctas` = the grid
// every reduce launch of this engine uses (the CTA counter is armed for it).
int mu_peer_reduce(mu_ctx *ctx, const void *a, const void *a_peer, const void *bias, const void *residual,
                   void *y, long long n, int cols, void *flags, void *peer_flags, unsigned per_step,
                   unsigned index, unsigned ctas, void *stream) {
  if (!ctx || !a || !a_peer || !y || !flags || !peer_flags || n < 0 || cols <= 0 || (n % 8) || (cols % 8))
    return mu_set_error(ctx, MU_ERR_INVALID, "peer reduce: bad arguments");
  if (mu_ctx_select_device(ctx) != MU_OK)
    return MU_ERR_CUDA;
  mu::peer_reduce_kernel<<<ctas, 512, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4 *>(a), static_cast<const uint4 *>(a_peer), static_cast<const uint4 *>(bias),
      static_cast<const uint4 *>(residual), static_cast<uint4 *>(y), n / 8, cols / 8,
      static_cast<mu::PeerFlags *>(flags), static_cast<mu::PeerFlags *>(peer_flags), per_step, index,
      mu_ctx_status_ptr(ctx));
  return cudaGetLastError() == cudaSuccess ? MU_OK : MU_ERR_CUDA;
}
}
