// float32 GEMM on the tensor cores for sm_100a: C = epilogue(A · B) with every float32 operand
// split into two TF32 numbers (hi = tf32(x), lo = x - hi) and the product formed as
//   hi·hi + lo·hi + hi·lo        (three tcgen05.mma kind::tf32 per k-step, fp32 accumulation in TMEM)
// which keeps ~2^-21 relative accuracy per product — float32-class, inside the 1e-4 tolerance of
// the float32 configs — at a third of the TF32 rate. The reference runs these products as scalar
// float loops (src/backend/cpu_backend.hpp:334-414, cuBLAS SGEMM on its CUDA backend); small
// problems keep that exact accumulation order on the CUDA-core kernel (gemm_simt.cu), the large
// ones (the Linear sweep at n >= 2048) come here.
//
// Two passes:
//   1. split kernels write hi/lo copies of A [M,K] and of B transposed to [N,K] (K-major for both
//      operands) into a scratch buffer of the context;
//   2. a persistent warp-specialised kernel, one CTA per SM, 320 threads:
//        warp 0    TMA producer: A_hi, A_lo [128 x 32] and B_hi, B_lo [256 x 32] fp32 tiles
//                  (128-byte rows, 128-byte swizzle), two-stage mbarrier ring
//        warp 1    tcgen05.mma issuer (M128 x N256 x K8), accumulators double-buffered in TMEM
//        warps 2-9 epilogue: tcgen05.ld, alpha / bias / activation / residual in fp32, swizzled
//                  staging box, TMA store (the residual arrives by TMA load into the same box)
// Every wait is bounded; a timeout latches the status word and the CTA unwinds.
#include "common.h"
#include "ptx.cuh"
#include <cuda.h>

namespace mu {

constexpr int T3_BM = 128, T3_BK = 32; // 32 fp32 = 128 bytes = one swizzle row
// The tensor core adds into its fp32 accumulator with truncation, a bias toward zero that grows
// linearly with K (measured: -1e-5 of the result's RMS per 2048 values of k, -4e-5 at K = 8192,
// beyond the 1e-4 bound on some elements). The K loop is therefore cut into chunks of
// T3_CHUNK_KB k-blocks (1024 values of k): each chunk accumulates in TMEM from zero and the
// epilogue warps sum the chunks in registers with round-to-nearest adds, which holds the bias at
// the one-chunk level (-5e-6, worst element at 0.19 of the bound) for any K.
constexpr int T3_CHUNK_KB = 32;
constexpr int T3_THREADS = 320;
constexpr int T3_A_BYTES = T3_BM * 128;
constexpr int T3_OUT_BOX = 32 * 128; // 32 rows x 32 fp32
// Column-tile width BN = 256 for wide outputs; 128 and 64 for the narrow ones (a convolution's
// output channels), where a 256-wide MMA would mostly multiply zero fill.
template <int BN> struct T3Cfg {
  static constexpr int B_BYTES = BN * 128;
  static constexpr int STAGE_BYTES = 2 * T3_A_BYTES + 2 * B_BYTES;
  static constexpr int STAGES = BN == 256 ? 2 : (BN == 128 ? 3 : 4);
  static constexpr int SMEM = STAGES * STAGE_BYTES + 8 * T3_OUT_BOX + 1024 + 256;
  static constexpr int NG = BN >= 64 ? BN / 64 : 1; // 32-column groups per epilogue warp
};

struct T3Args {
  int M, N, K;
  int act, has_bias, has_res;
  float alpha;
  const float *bias;
};

// Implicit-GEMM convolution (CONV = true): the A operand is never materialised. Row m of the
// im2col matrix is output pixel m of an NHWC image, column kk = (kh*k + kw)*iC + c; a k-block of 32
// columns is one filter tap and 32 input channels, i.e. a [bn, bh, W, 32] box of the NHWC input
// shifted by (kh - pad, kw - pad) — one 4-D TMA load, zero fill outside the image doing the padding.
// A 128-row tile is bn whole images (small images) or bh full rows of one image.
struct T3Conv {
  int icb;  // iC / 32: k-blocks per filter tap
  int k, pad;
  int H, bh, bn; // tile = bn images x bh rows x W columns = 128 pixels
};

// ---- pass 1: operand split ---------------------------------------------------------------
__device__ __forceinline__ float to_tf32(float x) {
  uint32_t u;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
  return __uint_as_float(u);
}

__global__ void __launch_bounds__(256)
split_tf32_kernel(const float *__restrict__ x, long long ldx, float *__restrict__ hi,
                  float *__restrict__ lo, long long rows, int cols) {
  const long long n = rows * cols;
  for (long long i = 1ll * blockIdx.x * blockDim.x + threadIdx.x; i < n; i += 1ll * gridDim.x * blockDim.x) {
    const float v = x[(i / cols) * ldx + (i % cols)];
    const float h = to_tf32(v);
    hi[i] = h;
    lo[i] = v - h; // exact in fp32; the tensor core drops its low 13 mantissa bits
  }
}

// w [K, N] (row stride ldw) -> hiT, loT [N, K]
__global__ void __launch_bounds__(256)
split_tf32_transpose_kernel(const float *__restrict__ w, long long ldw, float *__restrict__ hiT,
                            float *__restrict__ loT, int K, int N) {
  __shared__ float tile[32][33];
  const int k0 = blockIdx.y * 32, n0 = blockIdx.x * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5; // 32 x 8
  for (int r = ty; r < 32; r += 8) {
    const int k = k0 + r, n = n0 + tx;
    tile[r][tx] = (k < K && n < N) ? w[1ll * k * ldw + n] : 0.f;
  }
  __syncthreads();
  for (int r = ty; r < 32; r += 8) {
    const int n = n0 + r, k = k0 + tx;
    if (n < N && k < K) {
      const float v = tile[tx][r];
      const float h = to_tf32(v);
      hiT[1ll * n * K + k] = h;
      loT[1ll * n * K + k] = v - h;
    }
  }
}

// ---- pass 2: the GEMM ----------------------------------------------------------------------
__device__ __forceinline__ float t3_epilogue(float x, float b, float r, const T3Args &g) {
  if (g.alpha != 1.0f)
    x = __fmul_rn(x, g.alpha);
  if (g.has_bias)
    x = __fadd_rn(x, b);
  if (g.act == ACT_RELU) {
    x = x > 0.f ? x : 0.f;
  } else if (g.act == ACT_GELU) { // x * sigmoid(1.702 x), src/nn/activations.hpp:31-38
    const float t = __fmul_rn(x, 1.702f);
    x = __fmul_rn(x, __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-t))));
  } else if (g.act == ACT_SIGMOID) {
    x = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-x)));
  } else if (g.act == ACT_TANH) { // sigmoid(2x)*2 - 1, src/nn/activations.hpp:20-29
    const float s = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-__fmul_rn(x, 2.0f))));
    x = __fadd_rn(__fmul_rn(s, 2.0f), -1.0f);
  }
  if (g.has_res)
    x = __fadd_rn(x, r);
  return x;
}

__device__ __forceinline__ void t3_tma_load_2d(void *dst, const void *tmap, uint64_t *bar, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
               " [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(dst)),
               "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void t3_tma_store_2d(const void *tmap, const void *src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(tmap)),
               "r"(smem_u32(src)), "r"(c0), "r"(c1)
               : "memory");
}

template <int T3_BN, bool CONV>
__global__ void __launch_bounds__(T3_THREADS, 1)
gemm_tf32x3_kernel(const __grid_constant__ CUtensorMap tmAh, const __grid_constant__ CUtensorMap tmAl,
                   const __grid_constant__ CUtensorMap tmBh, const __grid_constant__ CUtensorMap tmBl,
                   const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmR,
                   T3Args g, T3Conv cv, int *status) {
  constexpr int T3_STAGES = T3Cfg<T3_BN>::STAGES, T3_STAGE_BYTES = T3Cfg<T3_BN>::STAGE_BYTES;
  constexpr int T3_B_BYTES = T3Cfg<T3_BN>::B_BYTES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t *out_stage = smem + T3_STAGES * T3_STAGE_BYTES;
  uint64_t *full_bar = reinterpret_cast<uint64_t *>(out_stage + 8 * T3_OUT_BOX);
  uint64_t *empty_bar = full_bar + T3_STAGES;
  uint64_t *tfull_bar = empty_bar + T3_STAGES;
  uint64_t *tempty_bar = tfull_bar + 2;
  uint64_t *res_bar = tempty_bar + 2;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(res_bar + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (g.M + T3_BM - 1) / T3_BM, tiles_n = (g.N + T3_BN - 1) / T3_BN;
  const int num_kb = (g.K + T3_BK - 1) / T3_BK;
  const long long total_tiles = 1ll * tiles_m * tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < T3_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull_bar[b], 1);
      mbar_init(&tempty_bar[b], 8);
    }
    for (int b = 0; b < 8; ++b)
      mbar_init(&res_bar[b], 1);
    fence_barrier_init();
    prefetch_tmap(&tmAh);
    prefetch_tmap(&tmAl);
    prefetch_tmap(&tmBh);
    prefetch_tmap(&tmBl);
    prefetch_tmap(&tmC);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (long long tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int nt = static_cast<int>(tile % tiles_n), mt = static_cast<int>(tile / tiles_n);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
            atomicCAS(status, 0, MU_DEV_TIMEOUT_PRODUCER);
            ok = false;
            break;
          }
          uint8_t *s = smem + stage * T3_STAGE_BYTES;
          mbar_arrive_expect_tx(&full_bar[stage], T3_STAGE_BYTES);
          if constexpr (CONV) {
            const int tap = kb / cv.icb, c0 = (kb % cv.icb) * T3_BK;
            const int kh = tap / cv.k, kw = tap % cv.k;
            int n0, h0;
            if (cv.bn > 1) {
              n0 = mt * cv.bn, h0 = 0;
            } else {
              const int per_image = cv.H / cv.bh;
              n0 = mt / per_image, h0 = (mt % per_image) * cv.bh;
            }
            tma_load_4d(s, &tmAh, &full_bar[stage], c0, kw - cv.pad, h0 + kh - cv.pad, n0);
            tma_load_4d(s + T3_A_BYTES, &tmAl, &full_bar[stage], c0, kw - cv.pad, h0 + kh - cv.pad, n0);
          } else {
            t3_tma_load_2d(s, &tmAh, &full_bar[stage], kb * T3_BK, mt * T3_BM);
            t3_tma_load_2d(s + T3_A_BYTES, &tmAl, &full_bar[stage], kb * T3_BK, mt * T3_BM);
          }
          t3_tma_load_2d(s + 2 * T3_A_BYTES, &tmBh, &full_bar[stage], kb * T3_BK, nt * T3_BN);
          t3_tma_load_2d(s + 2 * T3_A_BYTES + T3_B_BYTES, &tmBl, &full_bar[stage], kb * T3_BK, nt * T3_BN);
          if (++stage == T3_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok)
        for (int i = 0; i < 64; ++i)
          __nanosleep(1000);
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(2u, 0u, 0u, T3_BM, T3_BN); // tf32 x tf32 -> f32, both K-major
      int stage = 0, it = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (long long tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        for (int kb0 = 0; kb0 < num_kb && ok; kb0 += T3_CHUNK_KB, ++it) { // `it` counts chunks
          const int buf = it & 1;
          if (!mbar_wait(&tempty_bar[buf], ((static_cast<uint32_t>(it >> 1)) & 1) ^ 1)) {
            atomicCAS(status, 0, MU_DEV_TIMEOUT_MMA);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(buf * T3_BN);
          const int kb1 = min(kb0 + T3_CHUNK_KB, num_kb);
          for (int kb = kb0; kb < kb1; ++kb) {
            if (!mbar_wait(&full_bar[stage], phase)) {
              atomicCAS(status, 0, MU_DEV_TIMEOUT_MMA);
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t ah = smem_u32(smem + stage * T3_STAGE_BYTES), al = ah + T3_A_BYTES;
            const uint32_t bh = ah + 2 * T3_A_BYTES, bl = bh + T3_B_BYTES;
#pragma unroll
            for (int k = 0; k < T3_BK / 8; ++k) { // K = 8 per instruction = 32 bytes
              const uint64_t dah = make_smem_desc(ah + k * 32, 16, 1024), dal = make_smem_desc(al + k * 32, 16, 1024);
              const uint64_t dbh = make_smem_desc(bh + k * 32, 16, 1024), dbl = make_smem_desc(bl + k * 32, 16, 1024);
              umma_tf32(tmem_d, dal, dbh, idesc, ((kb - kb0) | k) != 0 ? 1u : 0u); // small terms first
              umma_tf32(tmem_d, dah, dbl, idesc, 1u);
              umma_tf32(tmem_d, dah, dbh, idesc, 1u);
            }
            umma_commit(&empty_bar[stage]);
            if (++stage == T3_STAGES) {
              stage = 0;
              phase ^= 1;
            }
          }
          if (ok)
            umma_commit(&tfull_bar[buf]);
        }
      }
    }
    __syncwarp();
  } else {
    const int q = warp & 3, half = (warp - 2) >> 2;
    uint8_t *buf = out_stage + (warp - 2) * T3_OUT_BOX;
    int it = 0, gcount = 0; // `it` counts K chunks, like the MMA warp
    bool ok = true;
    constexpr int NG = T3Cfg<T3_BN>::NG; // 32-column groups per warp
    for (long long tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      const int nt = static_cast<int>(tile % tiles_n), mt = static_cast<int>(tile / tiles_n);
      const int m0 = mt * T3_BM + q * 32;
      float acc[NG][32]; // running sum of the K chunks (0 + x is exact)
#pragma unroll
      for (int gi = 0; gi < NG; ++gi)
#pragma unroll
        for (int k = 0; k < 32; ++k)
          acc[gi][k] = 0.f;
      for (int kb0 = 0; kb0 < num_kb && ok; kb0 += T3_CHUNK_KB, ++it) {
        const int b = it & 1;
        if (!mbar_wait(&tfull_bar[b], (static_cast<uint32_t>(it >> 1)) & 1)) {
          atomicCAS(status, 0, MU_DEV_TIMEOUT_EPILOGUE);
          ok = false;
          break;
        }
        tc_fence_after();
        if (m0 < g.M) {
#pragma unroll
          for (int gi = 0; gi < NG; ++gi) {
            const int grp = half + 2 * gi;
            if (nt * T3_BN + grp * 32 < g.N) { // warp-uniform
              uint32_t r[32];
              tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                                static_cast<uint32_t>(b * T3_BN + grp * 32), r);
              tmem_ld_wait();
#pragma unroll
              for (int k = 0; k < 32; ++k)
                acc[gi][k] = __fadd_rn(acc[gi][k], __uint_as_float(r[k]));
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0)
          mbar_arrive(&tempty_bar[b]); // the next chunk may overwrite this accumulator
      }
      if (!ok)
        break;
      if (m0 < g.M) {
#pragma unroll
        for (int gi = 0; gi < NG; ++gi) {
          const int grp = half + 2 * gi;
          const int n0 = nt * T3_BN + grp * 32;
          if (n0 < g.N) {
            if (lane == 0) {
              bulk_wait_read<0>();
              if (g.has_res) {
                mbar_arrive_expect_tx(&res_bar[warp - 2], T3_OUT_BOX);
                t3_tma_load_2d(buf, &tmR, &res_bar[warp - 2], n0, m0);
              }
            }
            __syncwarp();
            if (g.has_res && !mbar_wait(&res_bar[warp - 2], gcount & 1)) {
              atomicCAS(status, 0, MU_DEV_TIMEOUT_EPILOGUE);
              ok = false;
            }
            if (ok) {
              uint8_t *row = buf + lane * 128;
#pragma unroll
              for (int cc = 0; cc < 8; ++cc) {
                float4 *slot = reinterpret_cast<float4 *>(row + ((cc ^ (lane & 7)) << 4));
                float4 bv = make_float4(0.f, 0.f, 0.f, 0.f), rv = bv;
                if (g.has_bias) {
                  const int n = n0 + cc * 4; // columns past N are clipped by the store: clamp the read
                  bv.x = n < g.N ? __ldg(g.bias + n) : 0.f;
                  bv.y = n + 1 < g.N ? __ldg(g.bias + n + 1) : 0.f;
                  bv.z = n + 2 < g.N ? __ldg(g.bias + n + 2) : 0.f;
                  bv.w = n + 3 < g.N ? __ldg(g.bias + n + 3) : 0.f;
                }
                if (g.has_res)
                  rv = *slot;
                float4 o;
                o.x = t3_epilogue(acc[gi][cc * 4 + 0], bv.x, rv.x, g);
                o.y = t3_epilogue(acc[gi][cc * 4 + 1], bv.y, rv.y, g);
                o.z = t3_epilogue(acc[gi][cc * 4 + 2], bv.z, rv.z, g);
                o.w = t3_epilogue(acc[gi][cc * 4 + 3], bv.w, rv.w, g);
                *slot = o;
              }
              fence_proxy_async();
              __syncwarp();
              if (lane == 0) {
                t3_tma_store_2d(&tmC, buf, n0, m0);
                bulk_commit();
              }
              ++gcount;
            }
          }
        }
      }
    }
    if (lane == 0)
      bulk_wait<0>();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1)
    tmem_dealloc(tmem_base, 512);
}

// ---- host ------------------------------------------------------------------------------------
typedef CUresult (*T3EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                               const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                               CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                               CUtensorMapFloatOOBfill);
static T3EncodeFn t3_encode_fn() {
  static T3EncodeFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &p, 12000, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<T3EncodeFn>(p);
  }
  return fn;
}
// fp32 matrix [rows, cols], row stride ld elements, box [brows x 32 columns], 128-byte swizzle
static bool t3_map(CUtensorMap *m, const void *base, unsigned long long cols, unsigned long long rows,
                   unsigned long long ld, unsigned brows) {
  T3EncodeFn fn = t3_encode_fn();
  if (!fn)
    return false;
  cuuint64_t dims[2] = {cols, rows}, strides[1] = {ld * 4ull};
  cuuint32_t box[2] = {32, brows}, es[2] = {1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void *>(base), dims, strides, box, es,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Scratch the split copies need, in bytes (256-byte aligned parts).
size_t gemm_tf32x3_scratch_bytes(int M, int N, int K) {
  auto up = [](size_t v) { return (v + 255) & ~static_cast<size_t>(255); };
  return 2 * up(static_cast<size_t>(M) * K * 4) + 2 * up(static_cast<size_t>(N) * K * 4);
}

template <int BN, bool CONV = false>
static int t3_launch(const CUtensorMap &tmAh, const CUtensorMap &tmAl, const float *bh, const float *bl,
                     const CUtensorMap &tmC, const CUtensorMap &tmR, const T3Args &g, int *status, int num_sms,
                     cudaStream_t st, T3Conv cv = T3Conv()) {
  CUtensorMap tmBh, tmBl;
  if (!t3_map(&tmBh, bh, g.K, g.N, g.K, BN) || !t3_map(&tmBl, bl, g.K, g.N, g.K, BN))
    return 2;
  auto kern = gemm_tf32x3_kernel<BN, CONV>;
  static PerDeviceOnce attr_set;
  if (attr_set.get() < 0) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, T3Cfg<BN>::SMEM) != cudaSuccess)
      return 2;
    attr_set.set(1);
  }
  const long long tiles = 1ll * ((g.M + T3_BM - 1) / T3_BM) * ((g.N + BN - 1) / BN);
  const unsigned grid = static_cast<unsigned>(tiles < num_sms ? tiles : num_sms);
  kern<<<grid, T3_THREADS, T3Cfg<BN>::SMEM, st>>>(tmAh, tmAl, tmBh, tmBl, tmC, tmR, g, cv, status);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

// NHWC fp32 image tensor [B, H, W, C] as a 4-D map, box [bn, bh, W, 32 channels], 128-byte swizzle:
// in shared memory the box is 128 rows of 128 bytes, the K-major A tile the MMA descriptors expect.
static bool t3_map_nhwc(CUtensorMap *m, const void *base, int B, int H, int W, int C, int bh, int bn) {
  T3EncodeFn fn = t3_encode_fn();
  if (!fn)
    return false;
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(C), static_cast<cuuint64_t>(W), static_cast<cuuint64_t>(H),
                        static_cast<cuuint64_t>(B)};
  cuuint64_t strides[3] = {4ull * C, 4ull * C * W, 4ull * C * W * H};
  cuuint32_t box[4] = {32, static_cast<cuuint32_t>(W), static_cast<cuuint32_t>(bh), static_cast<cuuint32_t>(bn)};
  cuuint32_t es[4] = {1, 1, 1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void *>(base), dims, strides, box, es,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Convolution (stride 1, "same" padding: output H x W = input H x W) as an implicit GEMM on inputs
// that are already split: xh, xl NHWC [B,H,W,iC]; wh, wl [oC][k][k][iC] (K-major, K = k*k*iC);
// c [B*H*W, oC] (NHWC output), bias + optional ReLU fused. Returns 0 ok, 1 when the geometry does
// not tile into 128-pixel boxes of whole rows (the caller falls back), 2 failure.
// Does the geometry tile into 128-pixel boxes of whole image rows?
bool conv_tf32x3_implicit_ok(int B, int H, int W, int iC, int oC, int k, int pad) {
  if (W <= 0 || W > 128 || 128 % W || iC % 32 || oC % 4 || 2 * pad != k - 1 || k > 15)
    return false;
  const int rows = 128 / W;
  if (rows <= H ? (H % rows != 0) : (rows % H != 0 || B % (rows / H) != 0))
    return false;
  const long long M = 1ll * B * H * W;
  return M <= 0x7fffffffll && M % 128 == 0;
}

int conv_tf32x3_implicit(const float *xh, const float *xl, const float *wh, const float *wl, float *c,
                         const float *bias, int relu, int B, int H, int W, int iC, int oC, int k, int pad,
                         int *status, int num_sms, cudaStream_t st) {
  if (!conv_tf32x3_implicit_ok(B, H, W, iC, oC, k, pad))
    return 1;
  const int rows = 128 / W;
  T3Conv cv;
  cv.icb = iC / 32, cv.k = k, cv.pad = pad, cv.H = H;
  if (rows <= H)
    cv.bh = rows, cv.bn = 1;
  else
    cv.bh = H, cv.bn = rows / H;
  const long long M = 1ll * B * H * W;
  auto al16 = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  if (!al16(xh) || !al16(xl) || !al16(wh) || !al16(wl) || !al16(c))
    return 1;
  CUtensorMap tmAh, tmAl, tmC;
  if (!t3_map_nhwc(&tmAh, xh, B, H, W, iC, cv.bh, cv.bn) || !t3_map_nhwc(&tmAl, xl, B, H, W, iC, cv.bh, cv.bn) ||
      !t3_map(&tmC, c, oC, M, oC, 32))
    return 2;
  T3Args g;
  g.M = static_cast<int>(M), g.N = oC, g.K = k * k * iC, g.act = relu ? ACT_RELU : ACT_NONE;
  g.has_bias = bias != nullptr, g.has_res = 0, g.alpha = 1.0f, g.bias = bias;
  if (oC > 128)
    return t3_launch<256, true>(tmAh, tmAl, wh, wl, tmC, tmC, g, status, num_sms, st, cv);
  if (oC > 64)
    return t3_launch<128, true>(tmAh, tmAl, wh, wl, tmC, tmC, g, status, num_sms, st, cv);
  return t3_launch<64, true>(tmAh, tmAl, wh, wl, tmC, tmC, g, status, num_sms, st, cv);
}

// The GEMM on operands that are already split: ah, al [M,K] and bh, bl [N,K], dense, K % 4 == 0.
// c and residual [M,N] with row stride ldc. Returns 0 ok, 1 outside the envelope, 2 failure.
int gemm_tf32x3_presplit(const float *ah, const float *al, const float *bh, const float *bl, float *c,
                         long long ldc, const float *bias, const float *residual, float alpha, int act, int M,
                         int N, int K, int *status, int num_sms, cudaStream_t st) {
  auto al16 = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  if (M <= 0 || N <= 0 || K <= 0 || (K % 4) || (ldc % 4) || !al16(c) || (residual && !al16(residual)) ||
      !al16(ah) || !al16(al) || !al16(bh) || !al16(bl))
    return 1;
  CUtensorMap tmAh, tmAl, tmC, tmR;
  if (!t3_map(&tmAh, ah, K, M, K, T3_BM) || !t3_map(&tmAl, al, K, M, K, T3_BM) || !t3_map(&tmC, c, N, M, ldc, 32))
    return 2;
  if (residual) {
    if (!t3_map(&tmR, residual, N, M, ldc, 32))
      return 2;
  } else {
    tmR = tmC;
  }
  T3Args g;
  g.M = M, g.N = N, g.K = K, g.act = act, g.has_bias = bias != nullptr, g.has_res = residual != nullptr;
  g.alpha = alpha, g.bias = bias;
  if (N > 128)
    return t3_launch<256>(tmAh, tmAl, bh, bl, tmC, tmR, g, status, num_sms, st);
  if (N > 64)
    return t3_launch<128>(tmAh, tmAl, bh, bl, tmC, tmR, g, status, num_sms, st);
  return t3_launch<64>(tmAh, tmAl, bh, bl, tmC, tmR, g, status, num_sms, st);
}

// Split only: x [rows, cols] with row stride ldx -> hi, lo dense [rows, cols].
void split_tf32(const float *x, long long ldx, float *hi, float *lo, long long rows, int cols, int num_sms,
                cudaStream_t st) {
  const unsigned eb = static_cast<unsigned>(num_sms > 0 ? num_sms * 16 : 1024);
  split_tf32_kernel<<<eb, 256, 0, st>>>(x, ldx, hi, lo, rows, cols);
}

// Returns 0 ok, 1 shape/alignment outside this kernel's envelope, 2 launch/encode failure.
// a [M,K] (row stride lda); b [K,N] (row stride ldb) or, with b_kmajor, [N,K]; c, residual [M,N]
// (row stride ldc).
int launch_gemm_tf32x3(const float *a, long long lda, const float *b, long long ldb, int b_kmajor, float *c,
                       long long ldc, const float *bias, const float *residual, float alpha, int act, int M,
                       int N, int K, void *scratch, int *status, int num_sms, cudaStream_t st) {
  if (M <= 0 || N <= 0 || K <= 0 || (K % 4) || !scratch)
    return 1;
  auto up = [](size_t v) { return (v + 255) & ~static_cast<size_t>(255); };
  uint8_t *s = static_cast<uint8_t *>(scratch);
  float *ah = reinterpret_cast<float *>(s), *alo = reinterpret_cast<float *>(s + up(1ull * M * K * 4));
  float *bh = reinterpret_cast<float *>(s + 2 * up(1ull * M * K * 4));
  float *bl = reinterpret_cast<float *>(s + 2 * up(1ull * M * K * 4) + up(1ull * N * K * 4));
  split_tf32(a, lda, ah, alo, M, K, num_sms, st);
  if (b_kmajor)
    split_tf32(b, ldb, bh, bl, N, K, num_sms, st);
  else
    split_tf32_transpose_kernel<<<dim3((N + 31) / 32, (K + 31) / 32), 256, 0, st>>>(b, ldb, bh, bl, K, N);
  return gemm_tf32x3_presplit(ah, alo, bh, bl, c, ldc, bias, residual, alpha, act, M, N, K, status, num_sms, st);
}

} // namespace mu
