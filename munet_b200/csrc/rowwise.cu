// HBM-bound row and elementwise kernels: LayerNorm, row softmax (optionally
// causal), embedding gather + positional add, fused elementwise chains and
// first-max argmax. One warp per row, 128-bit coalesced loads, the row cached
// in registers (one HBM read, one HBM write), warp-shuffle reductions only.
//
// Reference semantics:
//   LayerNorm  src/core/ops/normalization.cpp:172-206 (two-pass mean / biased
//              variance, eps inside the sqrt); the reference runs it on the
//              host for every backend — here it never leaves the device.
//   softmax    src/backend/cpu_backend.hpp:587-611, src/core/ops/activations.cpp:189-254
//   Embedding  src/nn/linear.hpp:92-131 (index path, bounds-checked)
//   GELU/Tanh  src/nn/activations.hpp:20-38 (compositions of mul/sigmoid)
#include "common.h"
#include "ptx.cuh"
#include "epilogue_math.cuh"
#include <cfloat>

namespace mu {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// A 16-byte vector of T viewed as floats.
template <typename T> struct Vec;
template <> struct Vec<float> {
  static constexpr int N = 4;
  __device__ static void load(const float *p, float (&f)[8]) {
    float4 v = *reinterpret_cast<const float4 *>(p);
    f[0] = v.x, f[1] = v.y, f[2] = v.z, f[3] = v.w;
  }
  __device__ static void store(float *p, const float (&f)[8]) {
    *reinterpret_cast<float4 *>(p) = make_float4(f[0], f[1], f[2], f[3]);
  }
  __device__ static float ld1(const float *p) { return *p; }
  __device__ static void st1(float *p, float v) { *p = v; }
};
template <> struct Vec<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static void load(const __nv_bfloat16 *p, float (&f)[8]) {
    uint4 v = *reinterpret_cast<const uint4 *>(p);
    f[0] = bf16_lo(v.x), f[1] = bf16_hi(v.x), f[2] = bf16_lo(v.y), f[3] = bf16_hi(v.y);
    f[4] = bf16_lo(v.z), f[5] = bf16_hi(v.z), f[6] = bf16_lo(v.w), f[7] = bf16_hi(v.w);
  }
  __device__ static void store(__nv_bfloat16 *p, const float (&f)[8]) {
    *reinterpret_cast<uint4 *>(p) = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]),
                                               pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
  }
  __device__ static float ld1(const __nv_bfloat16 *p) { return __bfloat162float(*p); }
  __device__ static void st1(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }
};

constexpr int ROW_WARPS = 8;  // warps (rows) per block
constexpr int MAXV = 8;       // 16-byte vectors cached per lane

// ---------------------------------------------------------------------------
// LayerNorm
// ---------------------------------------------------------------------------
template <typename T, bool VEC>
__global__ void __launch_bounds__(ROW_WARPS * 32)
layer_norm_kernel(const T *__restrict__ x, const T *__restrict__ gamma,
                  const T *__restrict__ beta, T *__restrict__ y, long long rows, int cols,
                  float eps) {
  constexpr int N = Vec<T>::N;
  const int lane = threadIdx.x & 31;
  const long long row = 1ll * blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
  if (row >= rows)
    return;
  const T *xr = x + row * cols;
  T *yr = y + row * cols;
  const float inv_n = 1.0f / static_cast<float>(cols);
  if (VEC) {
    const int nvec = cols / N;
    float c[MAXV][8];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = lane + i * 32;
      if (v < nvec) {
        Vec<T>::load(xr + v * N, c[i]);
#pragma unroll
        for (int e = 0; e < N; ++e)
          s += c[i][e];
      }
    }
    for (int v = lane + MAXV * 32; v < nvec; v += 32) { // rows longer than the register cache
      float t[8];
      Vec<T>::load(xr + v * N, t);
#pragma unroll
      for (int e = 0; e < N; ++e)
        s += t[e];
    }
    const float mean = warp_sum(s) * inv_n;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = lane + i * 32;
      if (v < nvec) {
#pragma unroll
        for (int e = 0; e < N; ++e) {
          const float d = c[i][e] - mean;
          q += d * d;
        }
      }
    }
    for (int v = lane + MAXV * 32; v < nvec; v += 32) {
      float t[8];
      Vec<T>::load(xr + v * N, t);
#pragma unroll
      for (int e = 0; e < N; ++e) {
        const float d = t[e] - mean;
        q += d * d;
      }
    }
    const float inv = rsqrtf(warp_sum(q) * inv_n + eps);
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = lane + i * 32;
      if (v < nvec) {
        float g[8], b[8], o[8];
        Vec<T>::load(gamma + v * N, g);
        Vec<T>::load(beta + v * N, b);
#pragma unroll
        for (int e = 0; e < N; ++e)
          o[e] = (c[i][e] - mean) * inv * g[e] + b[e];
        Vec<T>::store(yr + v * N, o);
      }
    }
    for (int v = lane + MAXV * 32; v < nvec; v += 32) {
      float t[8], g[8], b[8], o[8];
      Vec<T>::load(xr + v * N, t);
      Vec<T>::load(gamma + v * N, g);
      Vec<T>::load(beta + v * N, b);
#pragma unroll
      for (int e = 0; e < N; ++e)
        o[e] = (t[e] - mean) * inv * g[e] + b[e];
      Vec<T>::store(yr + v * N, o);
    }
  } else {
    float s = 0.f;
    for (int c = lane; c < cols; c += 32)
      s += Vec<T>::ld1(xr + c);
    const float mean = warp_sum(s) * inv_n;
    float q = 0.f;
    for (int c = lane; c < cols; c += 32) {
      const float d = Vec<T>::ld1(xr + c) - mean;
      q += d * d;
    }
    const float inv = rsqrtf(warp_sum(q) * inv_n + eps);
    for (int c = lane; c < cols; c += 32)
      Vec<T>::st1(yr + c, (Vec<T>::ld1(xr + c) - mean) * inv * Vec<T>::ld1(gamma + c) +
                              Vec<T>::ld1(beta + c));
  }
}

// ---------------------------------------------------------------------------
// Row softmax. causal_T > 0: row r only sees columns 0..(r % causal_T); the
// rest of the output row is written as exact zeros (what the reference's
// -1e9 fill turns into after exp). `scale` multiplies the input first.
// ---------------------------------------------------------------------------
template <typename T, bool VEC>
__global__ void __launch_bounds__(ROW_WARPS * 32)
softmax_kernel(const T *__restrict__ x, T *__restrict__ y, long long rows, int cols, float scale,
               int causal_T, int round_scaled) {
  constexpr int N = Vec<T>::N;
  const int lane = threadIdx.x & 31;
  const long long row = 1ll * blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
  if (row >= rows)
    return;
  const T *xr = x + row * cols;
  T *yr = y + row * cols;
  const int valid = causal_T > 0 ? static_cast<int>(row % causal_T) + 1 : cols;
  if (VEC) {
    const int nvec = cols / N;
    float c[MAXV][8];
    float mx = -FLT_MAX;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = lane + i * 32;
      if (v < nvec && v * N < valid) {
        Vec<T>::load(xr + v * N, c[i]);
#pragma unroll
        for (int e = 0; e < N; ++e) {
          float t = c[i][e] * scale;
          if (round_scaled)
            t = bf16_round(t);
          c[i][e] = t;
          if (v * N + e < valid)
            mx = fmaxf(mx, t);
        }
      }
    }
    mx = warp_max(mx);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = lane + i * 32;
      if (v < nvec && v * N < valid) {
#pragma unroll
        for (int e = 0; e < N; ++e) {
          const float p = (v * N + e < valid) ? __expf(c[i][e] - mx) : 0.f;
          c[i][e] = p;
          s += p;
        }
      }
    }
    const float inv = 1.0f / warp_sum(s);
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = lane + i * 32;
      if (v < nvec) {
        float o[8];
#pragma unroll
        for (int e = 0; e < N; ++e)
          o[e] = (v * N < valid) ? c[i][e] * inv : 0.f;
        Vec<T>::store(yr + v * N, o);
      }
    }
  } else {
    float mx = -FLT_MAX;
    for (int c = lane; c < valid; c += 32) {
      float t = Vec<T>::ld1(xr + c) * scale;
      if (round_scaled)
        t = bf16_round(t);
      mx = fmaxf(mx, t);
    }
    mx = warp_max(mx);
    float s = 0.f;
    for (int c = lane; c < valid; c += 32) {
      float t = Vec<T>::ld1(xr + c) * scale;
      if (round_scaled)
        t = bf16_round(t);
      s += __expf(t - mx);
    }
    const float inv = 1.0f / warp_sum(s);
    for (int c = lane; c < cols; c += 32) {
      float o = 0.f;
      if (c < valid) {
        float t = Vec<T>::ld1(xr + c) * scale;
        if (round_scaled)
          t = bf16_round(t);
        o = __expf(t - mx) * inv;
      }
      Vec<T>::st1(yr + c, o);
    }
  }
}

// ---------------------------------------------------------------------------
// Embedding gather (+ positional row add). One warp per token.
// ---------------------------------------------------------------------------
template <typename T, bool VEC>
__global__ void __launch_bounds__(ROW_WARPS * 32)
embedding_kernel(const int *__restrict__ ids, const T *__restrict__ table,
                 const T *__restrict__ pos, T *__restrict__ out, long long tokens, int T_len,
                 int V, int D, int *status) {
  constexpr int N = Vec<T>::N;
  const int lane = threadIdx.x & 31;
  const long long tok = 1ll * blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
  if (tok >= tokens)
    return;
  int id = ids[tok];
  const bool bad = id < 0 || id >= V;
  if (bad) {
    if (lane == 0)
      atomicCAS(status, 0, MU_DEV_BAD_INDEX);
    id = 0;
  }
  const T *src = table + 1ll * id * D;
  const T *pr = pos ? pos + 1ll * (tok % T_len) * D : nullptr;
  T *dst = out + tok * D;
  if (VEC) {
    for (int v = lane; v < D / N; v += 32) {
      float a[8], p[8];
      Vec<T>::load(src + v * N, a);
      if (pr) {
        Vec<T>::load(pr + v * N, p);
#pragma unroll
        for (int e = 0; e < N; ++e)
          a[e] += p[e];
      }
      if (bad) {
#pragma unroll
        for (int e = 0; e < N; ++e)
          a[e] = 0.f;
      }
      Vec<T>::store(dst + v * N, a);
    }
  } else {
    for (int c = lane; c < D; c += 32) {
      float a = Vec<T>::ld1(src + c);
      if (pr)
        a += Vec<T>::ld1(pr + c);
      Vec<T>::st1(dst + c, bad ? 0.f : a);
    }
  }
}

// ---------------------------------------------------------------------------
// Fused elementwise chain: y = act(x [+ bias[col]]) [+ residual], with the
// reference's per-op rounding for bf16. 128-bit vectors, grid-stride.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float chain_math(float x, float bias, float res, bool hb, bool hr,
                                            int act, bool bf) {
  if (hb) {
    x = bf ? bf16_round(x + bias) : __fadd_rn(x, bias);
  }
  if (act == ACT_RELU) {
    x = x > 0.f ? x : 0.f;
  } else if (act == ACT_GELU) {
    if (bf) {
      float t = bf16_round(x * bf16_round(1.702f));
      float s = bf16_round(1.0f / (1.0f + __expf(-t)));
      x = bf16_round(x * s);
    } else {
      float t = __fmul_rn(x, 1.702f);
      float s = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-t)));
      x = __fmul_rn(x, s);
    }
  } else if (act == ACT_SIGMOID) {
    x = bf ? bf16_round(1.0f / (1.0f + __expf(-x))) : __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-x)));
  } else if (act == ACT_TANH) {
    if (bf) {
      float t = bf16_round(x * 2.0f);
      float s = bf16_round(1.0f / (1.0f + __expf(-t)));
      x = bf16_round(s * 2.0f - 1.0f);
    } else {
      float t = __fmul_rn(x, 2.0f);
      float s = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-t)));
      x = __fadd_rn(__fmul_rn(s, 2.0f), -1.0f);
    }
  }
  if (hr) {
    x = bf ? bf16_round(x + res) : __fadd_rn(x, res);
  }
  return x;
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
eltwise_kernel(const T *__restrict__ x, const T *__restrict__ bias, const T *__restrict__ res,
               T *__restrict__ y, long long n, int cols, int act) {
  constexpr int N = Vec<T>::N;
  constexpr bool bf = sizeof(T) == 2;
  const long long stride = 1ll * gridDim.x * blockDim.x;
  long long i = 1ll * blockIdx.x * blockDim.x + threadIdx.x;
  if (VEC) {
    const long long nv = n / N;
    for (; i < nv; i += stride) {
      float a[8], b[8], r[8];
      Vec<T>::load(x + i * N, a);
      if (bias)
        Vec<T>::load(bias + (i * N) % cols, b);
      if (res)
        Vec<T>::load(res + i * N, r);
#pragma unroll
      for (int e = 0; e < N; ++e)
        a[e] = chain_math(a[e], bias ? b[e] : 0.f, res ? r[e] : 0.f, bias != nullptr,
                          res != nullptr, act, bf);
      Vec<T>::store(y + i * N, a);
    }
  } else {
    for (; i < n; i += stride) {
      const float b = bias ? Vec<T>::ld1(bias + i % cols) : 0.f;
      const float r = res ? Vec<T>::ld1(res + i) : 0.f;
      Vec<T>::st1(y + i, chain_math(Vec<T>::ld1(x + i), b, r, bias != nullptr, res != nullptr,
                                    act, bf));
    }
  }
}

// bf16 fast path of the chain above: activation fixed at compile time, pair arithmetic with
// packed converts (epilogue_math.cuh, the same code the GEMM epilogue runs), two 16-byte
// vectors per thread in flight.
template <int ACT>
__global__ void __launch_bounds__(256)
eltwise_bf16_vec_kernel(const uint4 *__restrict__ x, const __nv_bfloat16 *__restrict__ bias,
                        const uint4 *__restrict__ res, uint4 *__restrict__ y, long long nv, int cols) {
  const long long stride = 1ll * gridDim.x * blockDim.x;
  const bool hb = bias != nullptr, hr = res != nullptr;
  auto one = [&](long long i, uint4 xv, uint4 rv) {
    uint4 bv = make_uint4(0, 0, 0, 0);
    if (hb)
      bv = __ldg(reinterpret_cast<const uint4 *>(bias + (i * 8) % cols));
    const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w}, bw[4] = {bv.x, bv.y, bv.z, bv.w},
                   rw[4] = {rv.x, rv.y, rv.z, rv.w};
    uint32_t ow[4];
#pragma unroll
    for (int k = 0; k < 4; ++k)
      ow[k] = epi_pair<ACT, false>(bf16_lo(xw[k]), bf16_hi(xw[k]), bf16_lo(bw[k]), bf16_hi(bw[k]),
                                   bf16_lo(rw[k]), bf16_hi(rw[k]), 1.0f, false, hb, hr, true);
    __stcs(y + i, make_uint4(ow[0], ow[1], ow[2], ow[3]));
  };
  for (long long i = 1ll * blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += 2 * stride) {
    const long long i2 = i + stride;
    const bool two = i2 < nv;
    const uint4 z = make_uint4(0, 0, 0, 0);
    const uint4 xa = __ldcs(x + i), xb = two ? __ldcs(x + i2) : z;
    const uint4 ra = hr ? __ldcs(res + i) : z, rb = (hr && two) ? __ldcs(res + i2) : z;
    one(i, xa, ra);
    if (two)
      one(i2, xb, rb);
  }
}

// ---------------------------------------------------------------------------
// argmax over the last dim, first maximum wins (np.argmax rule). Warp per row.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(ROW_WARPS * 32)
argmax_kernel(const T *__restrict__ x, int *__restrict__ idx, long long rows, int cols) {
  const int lane = threadIdx.x & 31;
  const long long row = 1ll * blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
  if (row >= rows)
    return;
  const T *xr = x + row * cols;
  float best = -FLT_MAX;
  int bi = 0x7fffffff;
  for (int c = lane; c < cols; c += 32) {
    const float v = Vec<T>::ld1(xr + c);
    if (v > best || bi == 0x7fffffff) {
      best = v;
      bi = c;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > best || (ov == best && oi < bi))) {
      best = ov;
      bi = oi;
    }
  }
  if (lane == 0)
    idx[row] = bi;
}

// bf16 rows whose length is a multiple of 8: 16-byte streaming loads, four in flight per lane,
// and a packed maximum (one instruction per two values). The index is only searched for when a
// lane's chunk beats its running maximum, which happens O(log n) times per lane. Same answer as
// argmax_kernel: the smallest index of the maximum.
__global__ void __launch_bounds__(ROW_WARPS * 32)
argmax_bf16_vec_kernel(const __nv_bfloat16 *__restrict__ x, int *__restrict__ idx, long long rows,
                       int cols) {
  const int lane = threadIdx.x & 31;
  const long long row = 1ll * blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
  if (row >= rows)
    return;
  const uint4 *xr = reinterpret_cast<const uint4 *>(x + row * cols);
  const int nvec = cols / 8;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int v0 = lane; v0 < nvec; v0 += 128) {
    uint4 qv[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int vi = v0 + 32 * u;
      qv[u] = vi < nvec ? __ldcs(xr + vi) : make_uint4(0xFF80FF80u, 0xFF80FF80u, 0xFF80FF80u, 0xFF80FF80u);
    }
    uint32_t m2 = 0xFF80FF80u;
#pragma unroll
    for (int u = 0; u < 4; ++u)
      m2 = bf16x2_max(m2, bf16x2_max(bf16x2_max(qv[u].x, qv[u].y), bf16x2_max(qv[u].z, qv[u].w)));
    const float cm = fmaxf(bf16_lo(m2), bf16_hi(m2));
    if (cm > best) {
      best = cm;
      int found = 0x7fffffff;
#pragma unroll
      for (int u = 3; u >= 0; --u) { // descending, so the smallest index is written last
        const uint32_t w[4] = {qv[u].x, qv[u].y, qv[u].z, qv[u].w};
#pragma unroll
        for (int k = 3; k >= 0; --k) {
          const int base = (v0 + 32 * u) * 8 + 2 * k;
          if (bf16_hi(w[k]) == cm)
            found = base + 1;
          if (bf16_lo(w[k]) == cm)
            found = base;
        }
      }
      bi = found;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  }
  if (lane == 0)
    idx[row] = bi == 0x7fffffff ? 0 : bi; // every value was -inf (or NaN): the first index
}

// ---------------------------------------------------------------------------
// Host launchers
// ---------------------------------------------------------------------------
static bool al16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
static unsigned row_blocks(long long rows) {
  return static_cast<unsigned>((rows + ROW_WARPS - 1) / ROW_WARPS);
}

template <typename T>
static int ln_t(const void *x, const void *g, const void *b, void *y, long long rows, int cols,
                float eps, cudaStream_t st) {
  const bool vec = (cols % Vec<T>::N == 0) && al16(x) && al16(g) && al16(b) && al16(y);
  if (vec)
    layer_norm_kernel<T, true><<<row_blocks(rows), ROW_WARPS * 32, 0, st>>>(
        (const T *)x, (const T *)g, (const T *)b, (T *)y, rows, cols, eps);
  else
    layer_norm_kernel<T, false><<<row_blocks(rows), ROW_WARPS * 32, 0, st>>>(
        (const T *)x, (const T *)g, (const T *)b, (T *)y, rows, cols, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}
int launch_layer_norm_bf16_rows(const void *, const void *, const void *, void *, long long, int,
                                float, int *, int, cudaStream_t); // layer_norm_bf16.cu
int launch_layer_norm(const void *x, const void *g, const void *b, void *y, long long rows,
                      int cols, float eps, int dtype, int *status, int num_sms, cudaStream_t st) {
  if (rows <= 0)
    return 0;
  if (dtype == F32)
    return ln_t<float>(x, g, b, y, rows, cols, eps, st);
  if (dtype == BF16) {
    const int rc = launch_layer_norm_bf16_rows(x, g, b, y, rows, cols, eps, status, num_sms, st);
    return rc == 1 ? ln_t<__nv_bfloat16>(x, g, b, y, rows, cols, eps, st) : rc;
  }
  return 1;
}

template <typename T>
static int sm_t(const void *x, void *y, long long rows, int cols, float scale, int causal_T,
                int round_scaled, cudaStream_t st) {
  const bool vec = (cols % Vec<T>::N == 0) && al16(x) && al16(y) && cols <= MAXV * 32 * Vec<T>::N;
  if (vec)
    softmax_kernel<T, true><<<row_blocks(rows), ROW_WARPS * 32, 0, st>>>(
        (const T *)x, (T *)y, rows, cols, scale, causal_T, round_scaled);
  else
    softmax_kernel<T, false><<<row_blocks(rows), ROW_WARPS * 32, 0, st>>>(
        (const T *)x, (T *)y, rows, cols, scale, causal_T, round_scaled);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}
int launch_softmax(const void *x, void *y, long long rows, int cols, float scale, int causal_T,
                   int round_scaled, int dtype, cudaStream_t st) {
  if (rows <= 0)
    return 0;
  if (dtype == F32)
    return sm_t<float>(x, y, rows, cols, scale, causal_T, 0, st);
  if (dtype == BF16)
    return sm_t<__nv_bfloat16>(x, y, rows, cols, scale, causal_T, round_scaled, st);
  return 1;
}

template <typename T>
static int emb_t(const int *ids, const void *table, const void *pos, void *out, long long tokens,
                 int T_len, int V, int D, int *status, cudaStream_t st) {
  const bool vec = (D % Vec<T>::N == 0) && al16(table) && al16(out) && (!pos || al16(pos));
  if (vec)
    embedding_kernel<T, true><<<row_blocks(tokens), ROW_WARPS * 32, 0, st>>>(
        ids, (const T *)table, (const T *)pos, (T *)out, tokens, T_len, V, D, status);
  else
    embedding_kernel<T, false><<<row_blocks(tokens), ROW_WARPS * 32, 0, st>>>(
        ids, (const T *)table, (const T *)pos, (T *)out, tokens, T_len, V, D, status);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}
int launch_embedding(const int *ids, const void *table, const void *pos, void *out,
                     long long tokens, int T_len, int V, int D, int dtype, int *status,
                     cudaStream_t st) {
  if (tokens <= 0)
    return 0;
  if (dtype == F32)
    return emb_t<float>(ids, table, pos, out, tokens, T_len, V, D, status, st);
  if (dtype == BF16)
    return emb_t<__nv_bfloat16>(ids, table, pos, out, tokens, T_len, V, D, status, st);
  return 1;
}

template <typename T>
static int elt_t(const void *x, const void *bias, const void *res, void *y, long long n, int cols,
                 int act, int num_sms, cudaStream_t st) {
  const bool vec = (n % Vec<T>::N == 0) && (cols % Vec<T>::N == 0) && al16(x) && al16(y) &&
                   (!bias || al16(bias)) && (!res || al16(res));
  if constexpr (sizeof(T) == 2) {
    if (vec) {
      const long long nv = n / 8;
      long long nb = (nv + 511) / 512; // two vectors per thread and pass
      const long long capb = 1ll * num_sms * 8;
      if (nb > capb)
        nb = capb;
      if (nb < 1)
        nb = 1;
#define MU_ELT(A)                                                                                  \
  eltwise_bf16_vec_kernel<A><<<(unsigned)nb, 256, 0, st>>>((const uint4 *)x, (const __nv_bfloat16 *)bias, \
                                                           (const uint4 *)res, (uint4 *)y, nv, cols)
      switch (act) {
      case ACT_NONE: MU_ELT(ACT_NONE); break;
      case ACT_RELU: MU_ELT(ACT_RELU); break;
      case ACT_GELU: MU_ELT(ACT_GELU); break;
      case ACT_SIGMOID: MU_ELT(ACT_SIGMOID); break;
      case ACT_TANH: MU_ELT(ACT_TANH); break;
      default: return 1;
      }
#undef MU_ELT
      return cudaGetLastError() == cudaSuccess ? 0 : 2;
    }
  }
  const long long work = vec ? n / Vec<T>::N : n;
  long long blocks = (work + 255) / 256;
  const long long cap = 1ll * num_sms * 16;
  if (blocks > cap)
    blocks = cap;
  if (vec)
    eltwise_kernel<T, true><<<(unsigned)blocks, 256, 0, st>>>((const T *)x, (const T *)bias,
                                                              (const T *)res, (T *)y, n, cols, act);
  else
    eltwise_kernel<T, false><<<(unsigned)blocks, 256, 0, st>>>(
        (const T *)x, (const T *)bias, (const T *)res, (T *)y, n, cols, act);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}
int launch_eltwise(const void *x, const void *bias, const void *res, void *y, long long n,
                   int cols, int act, int dtype, int num_sms, cudaStream_t st) {
  if (n <= 0)
    return 0;
  if (cols <= 0)
    cols = 1;
  if (dtype == F32)
    return elt_t<float>(x, bias, res, y, n, cols, act, num_sms, st);
  if (dtype == BF16)
    return elt_t<__nv_bfloat16>(x, bias, res, y, n, cols, act, num_sms, st);
  return 1;
}

int launch_argmax(const void *x, int *idx, long long rows, int cols, int dtype, cudaStream_t st) {
  if (rows <= 0)
    return 0;
  if (dtype == F32)
    argmax_kernel<float><<<row_blocks(rows), ROW_WARPS * 32, 0, st>>>((const float *)x, idx, rows, cols);
  else if (dtype == BF16 && cols % 8 == 0 && al16(x))
    argmax_bf16_vec_kernel<<<row_blocks(rows), ROW_WARPS * 32, 0, st>>>((const __nv_bfloat16 *)x, idx,
                                                                      rows, cols);
  else if (dtype == BF16)
    argmax_kernel<__nv_bfloat16><<<row_blocks(rows), ROW_WARPS * 32, 0, st>>>(
        (const __nv_bfloat16 *)x, idx, rows, cols);
  else
    return 1;
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

} // namespace mu
