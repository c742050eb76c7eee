// Any-shape GEMM on CUDA cores: C = epilogue(A · B) for float32 or bfloat16
// operands with arbitrary (unaligned) leading dimensions and batch strides.
//
// Role: shapes the TMA/tcgen05 kernel cannot address (row strides that are not
// a multiple of 16 bytes, e.g. the 512→10 classifier of the MLP config) and all
// float32 matmuls that must reproduce the reference bit-for-bit.
//
// float32 mode reproduces the reference CPU kernel's rounding exactly
// (src/backend/cpu_backend.hpp:361-373): each output is a float sum over k in
// ascending order of separately rounded products (no fused multiply-add), so
// logits — and therefore argmax — are bit-identical to the reference.
// bfloat16 mode accumulates in fp32 with FMA.
#include "common.h"
#include "ptx.cuh"

namespace mu {

constexpr int ST = 64;  // tile M = tile N
constexpr int SK = 16;  // tile K

__device__ __forceinline__ float ld_elem(const void *p, long long i, bool bf) {
  return bf ? __bfloat162float(static_cast<const __nv_bfloat16 *>(p)[i])
            : static_cast<const float *>(p)[i];
}

__device__ __forceinline__ float act_f32_exact(float x, int act) {
  // float32 activation modules (src/backend/cpu_backend.hpp:493-520,
  // src/nn/activations.hpp:20-38): separate float ops, no contraction.
  if (act == ACT_RELU)
    return x > 0.f ? x : 0.f;
  if (act == ACT_GELU) {
    float t = __fmul_rn(x, 1.702f);
    float s = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-t)));
    return __fmul_rn(x, s);
  }
  if (act == ACT_SIGMOID)
    return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-x)));
  if (act == ACT_TANH) {
    float t = __fmul_rn(x, 2.0f);
    float s = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-t)));
    return __fadd_rn(__fmul_rn(s, 2.0f), -1.0f);
  }
  return x;
}

__device__ __forceinline__ float epi_bf16(float x, float bias, float res, bool hb, bool hr,
                                          float alpha, int act, bool rnd);

template <bool BF>
__global__ void __launch_bounds__(256) gemm_simt_kernel(SimtArgs g) {
  __shared__ float As[SK][ST + 1];
  __shared__ float Bs[SK][ST + 1];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int bt = blockIdx.z;
  const int m0 = blockIdx.y * ST, n0 = blockIdx.x * ST;
  const long long abase = 1ll * bt * g.a_batch, bbase = 1ll * bt * g.b_batch;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
      acc[i][j] = 0.f;

  for (int k0 = 0; k0 < g.sh.K; k0 += SK) {
    // A tile: 64 x 16, B tile: 16 x 64; 1024 elements each, 4 per thread
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = threadIdx.x + i * 256;
      {
        const int mm = e / SK, kk = e % SK; // k fastest: coalesced along K
        const int m = m0 + mm, k = k0 + kk;
        As[kk][mm] = (m < g.sh.M && k < g.sh.K) ? ld_elem(g.a, abase + 1ll * m * g.lda + k, BF) : 0.f;
      }
      if (g.b_kmajor) {
        const int nn = e / SK, kk = e % SK;
        const int n = n0 + nn, k = k0 + kk;
        Bs[kk][nn] = (n < g.sh.N && k < g.sh.K) ? ld_elem(g.b, bbase + 1ll * n * g.ldb + k, BF) : 0.f;
      } else {
        const int kk = e / ST, nn = e % ST; // n fastest
        const int n = n0 + nn, k = k0 + kk;
        Bs[kk][nn] = (n < g.sh.N && k < g.sh.K) ? ld_elem(g.b, bbase + 1ll * k * g.ldb + n, BF) : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < SK; ++kk) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        av[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        bv[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (BF)
            acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
          else // zero-padded k >= K adds +0.0f products: value-preserving
            acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(av[i], bv[j]));
        }
    }
    __syncthreads();
  }

  const Epilogue &ep = g.ep;
  const bool rnd = BF && ep.round_each;
  const float alpha = (rnd && ep.alpha != 1.0f) ? bf16_round(ep.alpha) : ep.alpha;
  const long long batch_off =
      1ll * (bt / ep.batch_div) * ep.batch_hi + 1ll * (bt % ep.batch_div) * ep.batch_lo;
  const int HD = ep.split_H * ep.split_D;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= g.sh.M)
      continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= g.sh.N)
        continue;
      long long off;
      if (ep.split_T > 0) {
        const int b = m / ep.split_T, t = m % ep.split_T;
        const int which = n / HD, rem = n % HD, h = rem / ep.split_D, d = rem % ep.split_D;
        off = which * ep.split_which_stride +
              ((1ll * b * ep.split_H + h) * ep.split_T + t) * ep.split_D + d;
      } else {
        off = batch_off + 1ll * m * ep.ldc + n;
      }
      float x = acc[i][j];
      if (BF) {
        const float bias = ep.bias ? ld_elem(ep.bias, n, true) : 0.f;
        const float res = ep.residual ? ld_elem(ep.residual, off, true) : 0.f;
        x = epi_bf16(x, bias, res, ep.bias != nullptr, ep.residual != nullptr, alpha, ep.act, rnd);
        static_cast<__nv_bfloat16 *>(ep.c)[off] = __float2bfloat16_rn(x);
      } else {
        if (ep.alpha != 1.0f)
          x = __fmul_rn(x, ep.alpha);
        if (ep.bias)
          x = __fadd_rn(x, static_cast<const float *>(ep.bias)[n]);
        x = act_f32_exact(x, ep.act);
        if (ep.residual)
          x = __fadd_rn(x, static_cast<const float *>(ep.residual)[off]);
        static_cast<float *>(ep.c)[off] = x;
      }
    }
  }
}

__device__ __forceinline__ float epi_bf16(float x, float bias, float res, bool hb, bool hr,
                                          float alpha, int act, bool rnd) {
  if (rnd)
    x = bf16_round(x);
  if (alpha != 1.0f) {
    x = x * alpha;
    if (rnd)
      x = bf16_round(x);
  }
  if (hb) {
    x = x + bias;
    if (rnd)
      x = bf16_round(x);
  }
  if (act == ACT_RELU) {
    x = fmaxf(x, 0.f);
  } else if (act == ACT_GELU) {
    const float c = rnd ? bf16_round(1.702f) : 1.702f;
    float t = x * c;
    if (rnd)
      t = bf16_round(t);
    float s = 1.0f / (1.0f + __expf(-t));
    if (rnd)
      s = bf16_round(s);
    x = x * s;
    if (rnd)
      x = bf16_round(x);
  } else if (act == ACT_SIGMOID) {
    x = 1.0f / (1.0f + __expf(-x));
    if (rnd)
      x = bf16_round(x);
  } else if (act == ACT_TANH) {
    float t = x * 2.0f;
    float s = 1.0f / (1.0f + __expf(-t));
    if (rnd)
      s = bf16_round(s);
    x = s * 2.0f - 1.0f;
    if (rnd)
      x = bf16_round(x);
  }
  if (hr) {
    x = x + res;
    if (rnd)
      x = bf16_round(x);
  }
  return x;
}

int launch_gemm_simt(const SimtArgs &g, cudaStream_t stream) {
  if (g.sh.M <= 0 || g.sh.N <= 0 || g.sh.batch <= 0)
    return 1;
  dim3 grid((g.sh.N + ST - 1) / ST, (g.sh.M + ST - 1) / ST, g.sh.batch);
  if (grid.y > 65535 || grid.z > 65535)
    return 1;
  if (g.is_bf16)
    gemm_simt_kernel<true><<<grid, 256, 0, stream>>>(g);
  else
    gemm_simt_kernel<false><<<grid, 256, 0, stream>>>(g);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

} // namespace mu
