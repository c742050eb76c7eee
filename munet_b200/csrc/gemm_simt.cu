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

// R x R outputs per thread, 16 x 16 threads: tiles of 16R x 16R. Small problems take small
// tiles so that the grid still covers the device (the 256 x 512 layer of the MLP config is 32
// tiles of 64 x 64 but 512 of 16 x 16); the sum over k of one output is sequential in any case.
template <bool BF, int R>
__global__ void __launch_bounds__(256) gemm_simt_kernel(SimtArgs g) {
  constexpr int ST = 16 * R;
  constexpr int PER = (ST * SK + 255) / 256; // tile elements per thread and operand
  __shared__ float As[SK][ST + 1];
  __shared__ float Bs[SK][ST + 1];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int bt = blockIdx.z;
  const int m0 = blockIdx.y * ST, n0 = blockIdx.x * ST;
  const long long abase = 1ll * bt * g.a_batch, bbase = 1ll * bt * g.b_batch;
  float acc[R][R];
#pragma unroll
  for (int i = 0; i < R; ++i)
#pragma unroll
    for (int j = 0; j < R; ++j)
      acc[i][j] = 0.f;

  float ra[PER], rb[PER];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = threadIdx.x + i * 256;
      ra[i] = rb[i] = 0.f;
      if (e < ST * SK) {
        {
          const int mm = e / SK, kk = e % SK; // k fastest: coalesced along K
          const int m = m0 + mm, k = k0 + kk;
          if (m < g.sh.M && k < g.sh.K)
            ra[i] = ld_elem(g.a, abase + 1ll * m * g.lda + k, BF);
        }
        if (g.b_kmajor) {
          const int nn = e / SK, kk = e % SK;
          const int n = n0 + nn, k = k0 + kk;
          if (n < g.sh.N && k < g.sh.K)
            rb[i] = ld_elem(g.b, bbase + 1ll * n * g.ldb + k, BF);
        } else {
          const int kk = e / ST, nn = e % ST; // n fastest
          const int n = n0 + nn, k = k0 + kk;
          if (n < g.sh.N && k < g.sh.K)
            rb[i] = ld_elem(g.b, bbase + 1ll * k * g.ldb + n, BF);
        }
      }
    }
  };
  auto stage = [&]() {
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = threadIdx.x + i * 256;
      if (e < ST * SK) {
        As[e % SK][e / SK] = ra[i];
        if (g.b_kmajor)
          Bs[e % SK][e / SK] = rb[i];
        else
          Bs[e / ST][e % ST] = rb[i];
      }
    }
  };

  // Small tiles (few warps' worth of work per k-tile) hide the global-load latency by fetching
  // the next k-tile during the multiply; for 64 x 64 tiles the extra registers cost more than
  // the overlap gains (1024^3 float32: 0.133 ms without, 0.150 ms with).
  constexpr bool PREFETCH = R < 4;
  if (PREFETCH)
    fetch(0);
  for (int k0 = 0; k0 < g.sh.K; k0 += SK) {
    if (!PREFETCH)
      fetch(k0);
    stage();
    __syncthreads();
    if (PREFETCH && k0 + SK < g.sh.K)
      fetch(k0 + SK); // in flight during the multiply below
#pragma unroll
    for (int kk = 0; kk < SK; ++kk) {
      float av[R], bv[R];
#pragma unroll
      for (int i = 0; i < R; ++i)
        av[i] = As[kk][ty * R + i];
#pragma unroll
      for (int j = 0; j < R; ++j)
        bv[j] = Bs[kk][tx * R + j];
#pragma unroll
      for (int i = 0; i < R; ++i)
#pragma unroll
        for (int j = 0; j < R; ++j) {
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
  for (int i = 0; i < R; ++i) {
    const int m = m0 + ty * R + i;
    if (m >= g.sh.M)
      continue;
#pragma unroll
    for (int j = 0; j < R; ++j) {
      const int n = n0 + tx * R + j;
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

template <int R> static int launch_simt_r(const SimtArgs &g, cudaStream_t stream) {
  constexpr int ST = 16 * R;
  dim3 grid((g.sh.N + ST - 1) / ST, (g.sh.M + ST - 1) / ST, g.sh.batch);
  if (grid.y > 65535 || grid.z > 65535)
    return 1;
  if (g.is_bf16)
    gemm_simt_kernel<true, R><<<grid, 256, 0, stream>>>(g);
  else
    gemm_simt_kernel<false, R><<<grid, 256, 0, stream>>>(g);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int launch_gemm_simt(const SimtArgs &g, cudaStream_t stream) {
  if (g.sh.M <= 0 || g.sh.N <= 0 || g.sh.batch <= 0)
    return 1;
  // the largest tile whose grid still gives every SM a CTA (measured: 1024^3 float32 0.13 ms on
  // 64 x 64 tiles, 0.19 ms on 32 x 32; the 256-row MLP 0.18 ms on 64 x 64, 0.09 ms on 16 x 16)
  auto ctas = [&](int st) {
    return 1ll * ((g.sh.N + st - 1) / st) * ((g.sh.M + st - 1) / st) * g.sh.batch;
  };
  if (ctas(64) >= 148)
    return launch_simt_r<4>(g, stream);
  if (ctas(32) >= 148)
    return launch_simt_r<2>(g, stream);
  return launch_simt_r<1>(g, stream);
}

} // namespace mu
