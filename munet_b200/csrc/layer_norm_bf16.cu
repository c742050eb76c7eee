// Persistent bf16 LayerNorm for the model widths (cols = 256 * VPL elements).
// Same arithmetic as layer_norm_kernel in rowwise.cu (two-pass mean / biased variance
// in fp32, eps inside the sqrt: src/core/ops/normalization.cpp:172-206); what changes
// is the data movement. The generic kernel has one row per warp in flight and its loads
// stop while the warp reduces and stores, so the bytes in flight per SM fall short of
// what HBM latency needs. Here every warp owns a ring of LN_STAGES row buffers in shared
// memory that one lane keeps full with untiled bulk copies (completion on an mbarrier per
// stage), so loads for the next rows are always outstanding, independent of registers.
// gamma and beta sit in shared memory once per block.
#include "common.h"
#include "ptx.cuh"
#include <cfloat>

namespace mu {

constexpr int LN_WARPS = 16;
constexpr int LN_SMEM_BUDGET = 200 * 1024; // ring + gamma/beta, below the 227 KB per-block limit

template <int VPL> struct LnCfg {
  static constexpr int COLS = VPL * 256;
  static constexpr int ROW_BYTES = COLS * 2;
  static constexpr int STAGES_FIT = (LN_SMEM_BUDGET - 2 * ROW_BYTES) / (LN_WARPS * ROW_BYTES);
  static constexpr int STAGES = STAGES_FIT > 8 ? 8 : STAGES_FIT;
  static constexpr int SMEM = 2 * ROW_BYTES + LN_WARPS * STAGES * ROW_BYTES + LN_WARPS * STAGES * 8;
  static_assert(STAGES >= 2, "row too wide for the shared-memory ring");
};

template <int VPL>
__global__ void __launch_bounds__(LN_WARPS * 32, 1)
layer_norm_bf16_rows_kernel(const __nv_bfloat16 *__restrict__ x, const __nv_bfloat16 *__restrict__ gamma,
                            const __nv_bfloat16 *__restrict__ beta, __nv_bfloat16 *__restrict__ y,
                            long long rows, float eps, int *status) {
  using Cfg = LnCfg<VPL>;
  constexpr int COLS = Cfg::COLS, ROW_BYTES = Cfg::ROW_BYTES, STAGES = Cfg::STAGES;
  extern __shared__ __align__(128) unsigned char ln_smem[];
  uint4 *sg = reinterpret_cast<uint4 *>(ln_smem);
  uint4 *sb = reinterpret_cast<uint4 *>(ln_smem + ROW_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  unsigned char *ring = ln_smem + 2 * ROW_BYTES + warp * STAGES * ROW_BYTES;
  uint64_t *bars = reinterpret_cast<uint64_t *>(ln_smem + 2 * ROW_BYTES + LN_WARPS * STAGES * ROW_BYTES) +
                   warp * STAGES;

  for (int i = threadIdx.x; i < COLS / 8; i += LN_WARPS * 32) {
    sg[i] = __ldg(reinterpret_cast<const uint4 *>(gamma) + i);
    sb[i] = __ldg(reinterpret_cast<const uint4 *>(beta) + i);
  }
  if (lane == 0) {
    for (int s = 0; s < STAGES; ++s)
      mbar_init(&bars[s], 1);
    fence_barrier_init();
  }
  __syncthreads();

  const long long stride = 1ll * gridDim.x * LN_WARPS;
  const long long first = 1ll * blockIdx.x * LN_WARPS + warp;
  if (lane == 0) { // fill the ring
    for (int s = 0; s < STAGES; ++s) {
      const long long r = first + s * stride;
      if (r < rows) {
        mbar_arrive_expect_tx(&bars[s], ROW_BYTES);
        bulk_load(ring + s * ROW_BYTES, x + r * COLS, ROW_BYTES, &bars[s]);
      }
    }
  }
  const float inv_n = 1.0f / static_cast<float>(COLS);
  int stage = 0;
  uint32_t parity = 0;
  for (long long row = first; row < rows; row += stride) {
    if (!mbar_wait(&bars[stage], parity)) {
      // The copy never landed: record it, give the warp's other copies in flight the same
      // bounded chance to land, and leave. No other warp waits on this one.
      if (lane == 0)
        atomicCAS(status, 0, MU_DEV_TIMEOUT_OTHER);
      for (int k = 1; k < STAGES; ++k) {
        if (row + k * stride >= rows)
          break;
        if (++stage == STAGES) {
          stage = 0;
          parity ^= 1u;
        }
        if (!mbar_wait(&bars[stage], parity))
          break;
      }
      return;
    }
    const uint4 *buf = reinterpret_cast<const uint4 *>(ring + stage * ROW_BYTES);
    uint4 cur[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i)
      cur[i] = buf[lane + i * 32];
    __syncwarp(); // every lane has its copy of the row: the stage may be refilled
    if (lane == 0) {
      const long long r = row + STAGES * stride;
      if (r < rows) {
        mbar_arrive_expect_tx(&bars[stage], ROW_BYTES);
        bulk_load(ring + stage * ROW_BYTES, x + r * COLS, ROW_BYTES, &bars[stage]);
      }
    }
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const uint32_t w[4] = {cur[i].x, cur[i].y, cur[i].z, cur[i].w};
#pragma unroll
      for (int k = 0; k < 4; ++k)
        s += bf16_lo(w[k]) + bf16_hi(w[k]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      s += __shfl_xor_sync(0xffffffffu, s, o);
    const float mean = s * inv_n;
    float qv = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const uint32_t w[4] = {cur[i].x, cur[i].y, cur[i].z, cur[i].w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float d0 = bf16_lo(w[k]) - mean, d1 = bf16_hi(w[k]) - mean;
        qv += d0 * d0 + d1 * d1;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      qv += __shfl_xor_sync(0xffffffffu, qv, o);
    const float inv = rsqrtf(qv * inv_n + eps);
    uint4 *yr = reinterpret_cast<uint4 *>(y + row * COLS);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const uint4 g = sg[lane + i * 32], b = sb[lane + i * 32];
      const uint32_t w[4] = {cur[i].x, cur[i].y, cur[i].z, cur[i].w};
      const uint32_t gw[4] = {g.x, g.y, g.z, g.w};
      const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
      uint32_t o[4];
#pragma unroll
      for (int k = 0; k < 4; ++k)
        o[k] = pack_bf16x2((bf16_lo(w[k]) - mean) * inv * bf16_lo(gw[k]) + bf16_lo(bw[k]),
                           (bf16_hi(w[k]) - mean) * inv * bf16_hi(gw[k]) + bf16_hi(bw[k]));
      __stcs(&yr[lane + i * 32], make_uint4(o[0], o[1], o[2], o[3]));
    }
    if (++stage == STAGES) {
      stage = 0;
      parity ^= 1u;
    }
  }
}

// Row softmax on the same ring (arithmetic of softmax_kernel in rowwise.cu: scale first, optional
// bf16 rounding of the scaled value, maximum, exp, sum, divide; causal_T > 0 limits row r to its
// first r % causal_T + 1 columns and writes exact zeros behind them).
template <int VPL>
__global__ void __launch_bounds__(LN_WARPS * 32, 1)
softmax_bf16_rows_kernel(const __nv_bfloat16 *__restrict__ x, __nv_bfloat16 *__restrict__ y,
                         long long rows, float scale, int causal_T, int round_scaled, int *status) {
  using Cfg = LnCfg<VPL>;
  constexpr int COLS = Cfg::COLS, ROW_BYTES = Cfg::ROW_BYTES, STAGES = Cfg::STAGES;
  extern __shared__ __align__(128) unsigned char ln_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  unsigned char *ring = ln_smem + 2 * ROW_BYTES + warp * STAGES * ROW_BYTES;
  uint64_t *bars = reinterpret_cast<uint64_t *>(ln_smem + 2 * ROW_BYTES + LN_WARPS * STAGES * ROW_BYTES) +
                   warp * STAGES;
  if (lane == 0) {
    for (int s = 0; s < STAGES; ++s)
      mbar_init(&bars[s], 1);
    fence_barrier_init();
  }
  __syncwarp();
  const long long stride = 1ll * gridDim.x * LN_WARPS;
  const long long first = 1ll * blockIdx.x * LN_WARPS + warp;
  if (lane == 0) {
    for (int s = 0; s < STAGES; ++s) {
      const long long r = first + s * stride;
      if (r < rows) {
        mbar_arrive_expect_tx(&bars[s], ROW_BYTES);
        bulk_load(ring + s * ROW_BYTES, x + r * COLS, ROW_BYTES, &bars[s]);
      }
    }
  }
  int stage = 0;
  uint32_t parity = 0;
  for (long long row = first; row < rows; row += stride) {
    if (!mbar_wait(&bars[stage], parity)) {
      if (lane == 0)
        atomicCAS(status, 0, MU_DEV_TIMEOUT_OTHER);
      for (int k = 1; k < STAGES; ++k) {
        if (row + k * stride >= rows)
          break;
        if (++stage == STAGES) {
          stage = 0;
          parity ^= 1u;
        }
        if (!mbar_wait(&bars[stage], parity))
          break;
      }
      return;
    }
    const uint4 *buf = reinterpret_cast<const uint4 *>(ring + stage * ROW_BYTES);
    uint4 cur[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i)
      cur[i] = buf[lane + i * 32];
    __syncwarp();
    if (lane == 0) {
      const long long r = row + STAGES * stride;
      if (r < rows) {
        mbar_arrive_expect_tx(&bars[stage], ROW_BYTES);
        bulk_load(ring + stage * ROW_BYTES, x + r * COLS, ROW_BYTES, &bars[stage]);
      }
    }
    const int valid = causal_T > 0 ? static_cast<int>(row % causal_T) + 1 : COLS;
    float p[VPL * 8];
    float mx = -FLT_MAX;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const uint32_t w[4] = {cur[i].x, cur[i].y, cur[i].z, cur[i].w};
      const int c0 = (lane + i * 32) * 8;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float t0 = bf16_lo(w[k]) * scale, t1 = bf16_hi(w[k]) * scale;
        if (round_scaled) {
          const uint32_t u = pack_bf16x2(t0, t1);
          t0 = bf16_lo(u), t1 = bf16_hi(u);
        }
        p[i * 8 + 2 * k] = t0, p[i * 8 + 2 * k + 1] = t1;
        if (c0 + 2 * k < valid)
          mx = fmaxf(mx, t0);
        if (c0 + 2 * k + 1 < valid)
          mx = fmaxf(mx, t1);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int c0 = (lane + i * 32) * 8;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float v = (c0 + e < valid) ? __expf(p[i * 8 + e] - mx) : 0.f;
        p[i * 8 + e] = v;
        s += v;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      s += __shfl_xor_sync(0xffffffffu, s, o);
    const float inv = 1.0f / s;
    uint4 *yr = reinterpret_cast<uint4 *>(y + row * COLS);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      uint32_t o[4];
#pragma unroll
      for (int k = 0; k < 4; ++k)
        o[k] = pack_bf16x2(p[i * 8 + 2 * k] * inv, p[i * 8 + 2 * k + 1] * inv);
      __stcs(&yr[lane + i * 32], make_uint4(o[0], o[1], o[2], o[3]));
    }
    if (++stage == STAGES) {
      stage = 0;
      parity ^= 1u;
    }
  }
}

template <int VPL>
static int sm_launch(const __nv_bfloat16 *x, __nv_bfloat16 *y, long long rows, float scale, int causal_T,
                     int round_scaled, int *status, unsigned blocks, cudaStream_t st) {
  auto kern = softmax_bf16_rows_kernel<VPL>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, LnCfg<VPL>::SMEM) !=
      cudaSuccess)
    return 2;
  kern<<<blocks, LN_WARPS * 32, LnCfg<VPL>::SMEM, st>>>(x, y, rows, scale, causal_T, round_scaled, status);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

// Returns 0 launched, 1 shape not covered here (caller uses the generic kernel), 2 failure.
int launch_softmax_bf16_rows(const void *x, void *y, long long rows, int cols, float scale, int causal_T,
                             int round_scaled, int *status, int num_sms, cudaStream_t st) {
  auto al = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  if (!al(x) || !al(y) || rows <= 0 || num_sms <= 0 || status == nullptr)
    return 1;
  long long blocks = (rows + LN_WARPS - 1) / LN_WARPS;
  if (blocks > num_sms)
    blocks = num_sms;
  const auto *xp = static_cast<const __nv_bfloat16 *>(x);
  auto *yp = static_cast<__nv_bfloat16 *>(y);
  const unsigned nb = static_cast<unsigned>(blocks);
  switch (cols) {
  case 256: return sm_launch<1>(xp, yp, rows, scale, causal_T, round_scaled, status, nb, st);
  case 512: return sm_launch<2>(xp, yp, rows, scale, causal_T, round_scaled, status, nb, st);
  case 1024: return sm_launch<4>(xp, yp, rows, scale, causal_T, round_scaled, status, nb, st);
  case 2048: return sm_launch<8>(xp, yp, rows, scale, causal_T, round_scaled, status, nb, st);
  default: return 1;
  }
}

template <int VPL>
static int ln_launch(const __nv_bfloat16 *x, const __nv_bfloat16 *g, const __nv_bfloat16 *b,
                     __nv_bfloat16 *y, long long rows, float eps, int *status, unsigned blocks,
                     cudaStream_t st) {
  auto kern = layer_norm_bf16_rows_kernel<VPL>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, LnCfg<VPL>::SMEM) !=
      cudaSuccess)
    return 2;
  kern<<<blocks, LN_WARPS * 32, LnCfg<VPL>::SMEM, st>>>(x, g, b, y, rows, eps, status);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

// Returns 0 launched, 1 shape not covered here (caller uses the generic kernel), 2 failure.
int launch_layer_norm_bf16_rows(const void *x, const void *g, const void *b, void *y, long long rows,
                                int cols, float eps, int *status, int num_sms, cudaStream_t st) {
  auto al = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  if (!al(x) || !al(g) || !al(b) || !al(y) || rows <= 0 || num_sms <= 0 || status == nullptr)
    return 1;
  long long blocks = (rows + LN_WARPS - 1) / LN_WARPS;
  if (blocks > num_sms)
    blocks = num_sms; // one persistent block per SM
  const auto *xp = static_cast<const __nv_bfloat16 *>(x), *gp = static_cast<const __nv_bfloat16 *>(g),
             *bp = static_cast<const __nv_bfloat16 *>(b);
  auto *yp = static_cast<__nv_bfloat16 *>(y);
  const unsigned nb = static_cast<unsigned>(blocks);
  switch (cols) {
  case 512: return ln_launch<2>(xp, gp, bp, yp, rows, eps, status, nb, st);
  case 1024: return ln_launch<4>(xp, gp, bp, yp, rows, eps, status, nb, st);
  case 2048: return ln_launch<8>(xp, gp, bp, yp, rows, eps, status, nb, st);
  default: return 1;
  }
}

} // namespace mu
