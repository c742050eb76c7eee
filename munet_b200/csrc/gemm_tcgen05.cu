// bf16 GEMM for sm_100a: C = epilogue(A · B), fp32 accumulation in TMEM.
//
// The B200 replacement for the reference's `BackendBlasCapability::matmul` /
// `batched_matmul` (src/core/backend.hpp:250-260) fused with the broadcast bias
// add of nn::Linear (src/nn/linear.hpp:28-34), the activation module that
// follows it and the residual add of the decoder block.
//
// Structure (one persistent CTA per SM, 320 threads):
//   warp 0   TMA producer: A [128 x 64] and B [64 x BN] tiles, 128-byte swizzle,
//            STAGES-deep mbarrier ring. No cluster multicast anywhere.
//   warp 1   allocates TMEM and issues tcgen05.mma (kind::f16, M=128, N=BN, K=16)
//            from one thread; accumulators are double-buffered in TMEM so the
//            epilogue of tile i overlaps the main loop of tile i+1.
//   warps 2-9 epilogue (two per TMEM lane quarter, alternate 64-column groups): tcgen05.ld
//            32 lanes x 32 columns, scale / bias / activation / residual on packed pairs in
//            registers, result staged in a swizzled shared-memory box and written with one
//            TMA store per 32 x 64 box (the residual arrives in the same box by TMA load).
//            Outputs that no tensor map can address fall back to guarded 128-bit stores.
// A is row-major [M,K] (K-major operand). B is either row-major [K,N] as MuNet
// stores Linear weights (MN-major operand) or row-major [N,K] (K-major, "B
// transposed"). All operands may be batched through a third tensor-map dim.
// Tails in M, N and K are handled by TMA zero fill and guarded stores.
#include "common.h"
#include "ptx.cuh"
#include "epilogue_math.cuh"
#include <cuda.h>

namespace mu {

constexpr int BM = 128;
constexpr int BK = 64; // 64 bf16 = 128 bytes = one swizzle row
constexpr int GEMM_THREADS = 320; // TMA warp, MMA warp, 8 epilogue warps

// CTAS = 2: a cluster of two CTAs shares one 256 x BN tile (tcgen05 cta_group::2). Each CTA
// stages its own 128 rows of A and its own BN/2 columns of B, so a CTA moves a third less
// shared-memory traffic per FLOP and the ring is deeper.
template <int BN, int CTAS = 1> struct GemmCfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = (BN / CTAS) * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = CTAS == 2 ? (BN == 256 ? 6 : 8) : (BN == 256 ? 4 : (BN == 128 ? 6 : 8));
  static constexpr int TMEM_COLS = 2 * BN;
  // epilogue staging: one [32 rows x 64 cols] bf16 box (128-byte rows) per epilogue warp
  static constexpr int OUT_BOX_BYTES = 32 * 128;
  static constexpr int OUT_BYTES = 8 * OUT_BOX_BYTES;
  static constexpr int SMEM_BYTES =
      STAGES * STAGE_BYTES + OUT_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;
};

__device__ __forceinline__ float epi_math(float x, float bias, float res, bool has_bias,
                                          bool has_res, float alpha, int act, bool rnd) {
  if (rnd)
    x = bf16_round(x);
  if (alpha != 1.0f) {
    x = x * alpha;
    if (rnd)
      x = bf16_round(x);
  }
  if (has_bias) {
    x = x + bias;
    if (rnd)
      x = bf16_round(x);
  }
  if (act == ACT_RELU) {
    x = fmaxf(x, 0.0f);
  } else if (act == ACT_GELU) {
    // x * sigmoid(1.702 x): the reference's GELU (src/nn/activations.hpp:31-38)
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
    // sigmoid(2x)*2 - 1 (src/nn/activations.hpp:20-29)
    float t = x * 2.0f;
    float s = 1.0f / (1.0f + __expf(-t));
    if (rnd)
      s = bf16_round(s);
    x = s * 2.0f;
    x = x - 1.0f;
    if (rnd)
      x = bf16_round(x);
  }
  if (has_res) {
    x = x + res;
    if (rnd)
      x = bf16_round(x);
  }
  return x;
}

// One half (32 accumulator columns = four 16-byte chunks) of a staged 64-column
// group: optional residual is read from the staging row (where a TMA load put
// it), the result is written back to the same swizzled chunk.
template <int ACT>
__device__ __forceinline__ void epi_half(const uint32_t (&r)[32], uint8_t *row, int lane7,
                                         int half, const __nv_bfloat16 *bias, bool has_res,
                                         float alpha, bool has_alpha, bool rnd) {
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int cc = half * 4 + c;
    uint4 *slot = reinterpret_cast<uint4 *>(row + ((cc ^ lane7) << 4));
    uint4 bv = make_uint4(0, 0, 0, 0), rv = make_uint4(0, 0, 0, 0);
    if (bias)
      bv = __ldg(reinterpret_cast<const uint4 *>(bias) + cc);
    if (has_res)
      rv = *slot;
    const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w}, rw[4] = {rv.x, rv.y, rv.z, rv.w};
    uint32_t ow[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      ow[j] = epi_pair<ACT>(__uint_as_float(r[c * 8 + 2 * j]), __uint_as_float(r[c * 8 + 2 * j + 1]),
                            bf16_lo(bw[j]), bf16_hi(bw[j]), bf16_lo(rw[j]), bf16_hi(rw[j]), alpha,
                            has_alpha, bias != nullptr, has_res, rnd);
    *slot = make_uint4(ow[0], ow[1], ow[2], ow[3]);
  }
}

// Tile index -> (batch, row tile, column tile). Column tiles are grouped in panels of P: inside a
// panel the column index runs fastest, panels follow one another after all row tiles of the
// previous panel. CTAs running side by side then share the panel's slice of B (and a few rows of
// A) in L2; with every column tile in one sweep a B wider than L2 would be re-read from DRAM for
// each row tile (measured on the 32000-column head: 6.1 GB read for 0.2 GB of operands).
__device__ __forceinline__ void decode_tile(long long tile, int tiles_m, int tiles_n, int P, int &bt,
                                            int &mt, int &nt) {
  const long long per_batch = 1ll * tiles_m * tiles_n;
  bt = static_cast<int>(tile / per_batch);
  const long long t = tile % per_batch;
  const int panel = static_cast<int>(t / (1ll * P * tiles_m));
  const int r = static_cast<int>(t % (1ll * P * tiles_m));
  const int w = min(P, tiles_n - panel * P);
  mt = r / w;
  nt = panel * P + r % w;
}

template <int BN, bool B_KMAJOR, int CTAS>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA,
                         const __grid_constant__ CUtensorMap tmB,
                         const __grid_constant__ CUtensorMap tmC,
                         const __grid_constant__ CUtensorMap tmR, GemmShape sh, Epilogue ep,
                         int *status) {
  using Cfg = GemmCfg<BN, CTAS>;
  constexpr int STAGES = Cfg::STAGES;
  static_assert(CTAS == 1 || (CTAS == 2 && (BN == 256 || BN == 128)), "CTA pairs: 256 x 256 or 256 x 128 tiles");
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: required by the 128-byte swizzle atoms.
  uint8_t *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t *out_stage = smem + STAGES * Cfg::STAGE_BYTES;
  uint8_t *bar_base = out_stage + Cfg::OUT_BYTES;
  uint64_t *full_bar = reinterpret_cast<uint64_t *>(bar_base);
  uint64_t *empty_bar = full_bar + STAGES;
  uint64_t *tfull_bar = empty_bar + STAGES;
  uint64_t *tempty_bar = tfull_bar + 2;
  uint64_t *res_bar = tempty_bar + 2; // one per epilogue warp
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(res_bar + 8);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // rank of this CTA inside its pair; the leader (rank 0) owns the full/tempty barriers and
  // issues the MMAs. With CTAS == 1 every CTA is its own leader.
  const int rank = CTAS == 2 ? static_cast<int>(cluster_ctarank()) : 0;
  const bool leader = rank == 0;
  const int tiles_m = (sh.M + BM * CTAS - 1) / (BM * CTAS);
  const int tiles_n = (sh.N + BN - 1) / BN;
  const int num_kb = (sh.K + BK - 1) / BK;
  const long long total_tiles = 1ll * tiles_m * tiles_n * sh.batch;
  const long long tile0 = blockIdx.x / CTAS, tile_step = gridDim.x / CTAS;
  const int panel = (sh.panel_n > 0 && sh.panel_n < tiles_n) ? sh.panel_n : tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull_bar[b], 1);
      mbar_init(&tempty_bar[b], 8 * CTAS);
    }
    for (int b = 0; b < 8; ++b)
      mbar_init(&res_bar[b], 1);
    fence_barrier_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
    if (ep.tma_out) {
      prefetch_tmap(&tmC);
      if (ep.residual)
        prefetch_tmap(&tmR);
    }
  }
  if (warp == 1) {
    tmem_alloc_g<CTAS>(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish_g<CTAS>();
  }
  tc_fence_before();
  if constexpr (CTAS == 2)
    cluster_sync_all(); // the peer's barriers are initialised before anything signals them
  else
    __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const uint64_t b_policy = sh.b_evict_last ? l2_policy_evict_last() : 0ull;
      for (long long tile = tile0; tile < total_tiles && ok; tile += tile_step) {
        int nt, mt, bt;
        decode_tile(tile, tiles_m, tiles_n, panel, bt, mt, nt);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1)) {
            atomicCAS(status, 0, MU_DEV_TIMEOUT_PRODUCER);
            ok = false;
            break;
          }
          uint8_t *sa = smem + stage * Cfg::STAGE_BYTES;
          uint8_t *sb = sa + Cfg::A_BYTES;
          // the leader's barrier counts the bytes of both CTAs of a pair
          if (leader)
            mbar_arrive_expect_tx(&full_bar[stage], Cfg::STAGE_BYTES * CTAS);
          const int bta = sh.a_batched ? bt : 0, btb = sh.b_batched ? bt : 0;
          tma_load_3d_g<CTAS>(sa, &tmA, &full_bar[stage], kb * BK, (mt * CTAS + rank) * BM, bta);
          if (B_KMAJOR) {
            tma_load_3d_g<CTAS>(sb, &tmB, &full_bar[stage], kb * BK, nt * BN + rank * (BN / CTAS), btb);
          } else {
            const int c0 = nt * BN + rank * (BN / CTAS) + bt * sh.b_col_per_batch;
            if (sh.b_evict_last) {
#pragma unroll
              for (int j = 0; j < BN / CTAS / 64; ++j)
                tma_load_3d_g_hint<CTAS>(sb + j * 8192, &tmB, &full_bar[stage], c0 + j * 64, kb * BK, btb,
                                         b_policy);
            } else {
#pragma unroll
              for (int j = 0; j < BN / CTAS / 64; ++j)
                tma_load_3d_g<CTAS>(sb + j * 8192, &tmB, &full_bar[stage], c0 + j * 64, kb * BK, btb);
            }
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) {
        // let copies already in flight land before the CTA's memory is released
        for (int i = 0; i < 64; ++i)
          __nanosleep(1000);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = make_idesc(1u, 0u, B_KMAJOR ? 0u : 1u, BM * CTAS, BN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (long long tile = tile0; tile < total_tiles && ok; tile += tile_step, ++it) {
        const int buf = it & 1;
        const uint32_t use = static_cast<uint32_t>(it >> 1);
        if (!mbar_wait(&tempty_bar[buf], (use & 1) ^ 1)) {
          atomicCAS(status, 0, MU_DEV_TIMEOUT_MMA);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(buf * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase)) {
            atomicCAS(status, 0, MU_DEV_TIMEOUT_MMA);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * Cfg::STAGE_BYTES);
          const uint32_t sb = sa + Cfg::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t adesc = make_smem_desc(sa + k * 32, 16, 1024);
            const uint64_t bdesc = B_KMAJOR ? make_smem_desc(sb + k * 32, 16, 1024)
                                            : make_smem_desc(sb + k * 2048, 8192, 1024);
            umma_f16_g<CTAS>(tmem_d, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit_g<CTAS>(&empty_bar[stage]); // smem slot reusable once these MMAs retire
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok)
          umma_commit_g<CTAS>(&tfull_bar[buf]); // accumulator complete (both CTAs of a pair)
      }
    }
    __syncwarp();
  } else {
    // ---------------- epilogue (warps 2..9) ----------------
    // Two warps per TMEM lane quarter (warp & 3): they take alternate 64-column groups of the
    // tile, so every scheduler has two epilogue warps to hide each other's latencies.
    const int q = warp & 3; // TMEM lane quarter this warp may read
    const int half = (warp - 2) >> 2;
    const bool rnd = ep.round_each != 0;
    const float alpha = (rnd && ep.alpha != 1.0f) ? bf16_round(ep.alpha) : ep.alpha;
    const __nv_bfloat16 *bias = static_cast<const __nv_bfloat16 *>(ep.bias);
    const __nv_bfloat16 *resid = static_cast<const __nv_bfloat16 *>(ep.residual);
    __nv_bfloat16 *cout = static_cast<__nv_bfloat16 *>(ep.c);
    const bool split = ep.split_T > 0;
    const int HD = ep.split_H * ep.split_D;
    int it = 0;
    const uint64_t stream_policy = sh.b_evict_last > 1 ? l2_policy_evict_first() : 0ull;
    int gcount = 0; // staged 64-column groups issued by this warp (phase of its residual barrier)
    bool ok = true;
    auto release_accumulator = [&](int b) {
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (CTAS == 2 && !leader)
          mbar_arrive_cluster(&tempty_bar[b], 0);
        else
          mbar_arrive(&tempty_bar[b]);
      }
    };
    for (long long tile = tile0; tile < total_tiles && ok; tile += tile_step, ++it) {
      int nt, mt, bt;
      decode_tile(tile, tiles_m, tiles_n, panel, bt, mt, nt);
      mt = mt * CTAS + rank; // 128-row tile index
      const int buf_idx = it & 1;
      const uint32_t use = static_cast<uint32_t>(it >> 1);
      if (!mbar_wait(&tfull_bar[buf_idx], use & 1)) {
        atomicCAS(status, 0, MU_DEV_TIMEOUT_EPILOGUE);
        ok = false;
        break;
      }
      tc_fence_after();
      if (ep.tma_out) {
        // ---- staged epilogue: TMEM -> registers -> swizzled smem box -> TMA store ----
        const int m0 = mt * BM + q * 32; // first row of this warp's 32-row slab
        uint8_t *buf = out_stage + (warp - 2) * Cfg::OUT_BOX_BYTES;
        const bool has_res = ep.residual != nullptr;
        const bool has_alpha = ep.alpha != 1.0f;
        if (m0 < sh.M) {
#pragma unroll 1
          for (int g = half; g < BN / 64; g += 2) {
            const int n0 = nt * BN + g * 64;
            if (n0 >= sh.N)
              break; // warp-uniform
            // tensor-map coordinates, dimensions ordered by ascending stride
            int c0, c1, c2, c3, c4;
            if (ep.tma_mode == 2) { // [which][B][H][T][D]
              c0 = n0 % ep.split_D, c1 = m0 % ep.split_T, c2 = (n0 / ep.split_D) % ep.split_H;
              c3 = m0 / ep.split_T, c4 = n0 / HD;
            } else if (ep.tma_mode == 1) { // [B][T][H][D]: batch = (b, h)
              c0 = n0, c1 = bt % ep.batch_div, c2 = m0, c3 = bt / ep.batch_div, c4 = 0;
            } else { // [batch][M][N]
              c0 = n0, c1 = m0, c2 = bt, c3 = 0, c4 = 0;
            }
            if (lane == 0) {
              bulk_wait_read<0>(); // the previous store from this buffer has finished reading it
              if (has_res) {
                mbar_arrive_expect_tx(&res_bar[warp - 2], Cfg::OUT_BOX_BYTES);
                if (sh.b_evict_last > 1)
                  tma_load_5d_hint(buf, &tmR, &res_bar[warp - 2], c0, c1, c2, c3, c4, stream_policy);
                else
                  tma_load_5d(buf, &tmR, &res_bar[warp - 2], c0, c1, c2, c3, c4);
              }
            }
            __syncwarp();
            uint32_t r0[32], r1[32];
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                                   static_cast<uint32_t>(buf_idx * BN + g * 64);
            tmem_ld_32x32(taddr, r0);
            tmem_ld_32x32(taddr + 32, r1);
            tmem_ld_wait();
            if (has_res) {
              if (!mbar_wait(&res_bar[warp - 2], gcount & 1)) {
                atomicCAS(status, 0, MU_DEV_TIMEOUT_EPILOGUE);
                ok = false;
                break;
              }
            }
            uint8_t *row = buf + lane * 128;
            const __nv_bfloat16 *bp = bias ? bias + n0 : nullptr;
            const int l7 = lane & 7;
            switch (ep.act) {
            case ACT_RELU:
              epi_half<ACT_RELU>(r0, row, l7, 0, bp, has_res, alpha, has_alpha, rnd);
              epi_half<ACT_RELU>(r1, row, l7, 1, bp, has_res, alpha, has_alpha, rnd);
              break;
            case ACT_GELU:
              epi_half<ACT_GELU>(r0, row, l7, 0, bp, has_res, alpha, has_alpha, rnd);
              epi_half<ACT_GELU>(r1, row, l7, 1, bp, has_res, alpha, has_alpha, rnd);
              break;
            case ACT_SIGMOID:
              epi_half<ACT_SIGMOID>(r0, row, l7, 0, bp, has_res, alpha, has_alpha, rnd);
              epi_half<ACT_SIGMOID>(r1, row, l7, 1, bp, has_res, alpha, has_alpha, rnd);
              break;
            case ACT_TANH:
              epi_half<ACT_TANH>(r0, row, l7, 0, bp, has_res, alpha, has_alpha, rnd);
              epi_half<ACT_TANH>(r1, row, l7, 1, bp, has_res, alpha, has_alpha, rnd);
              break;
            default:
              epi_half<ACT_NONE>(r0, row, l7, 0, bp, has_res, alpha, has_alpha, rnd);
              epi_half<ACT_NONE>(r1, row, l7, 1, bp, has_res, alpha, has_alpha, rnd);
            }
            fence_proxy_async(); // generic-proxy writes → visible to the TMA store
            __syncwarp();
            if (lane == 0) {
              if (sh.b_evict_last > 1)
                tma_store_5d_hint(&tmC, buf, c0, c1, c2, c3, c4, stream_policy);
              else
                tma_store_5d(&tmC, buf, c0, c1, c2, c3, c4);
              bulk_commit();
            }
            if (ep.c_mirror) {
              // second copy of the box (plain [M,N] addressing), read back from the staging rows:
              // eight lanes cover one 128-byte row, a warp instruction four whole rows. The next
              // group's writes to this buffer come after a __syncwarp that follows these reads.
              __nv_bfloat16 *mc = static_cast<__nv_bfloat16 *>(ep.c_mirror);
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int idx = i * 32 + lane, r = idx >> 3, cc = idx & 7;
                const uint4 v = *reinterpret_cast<const uint4 *>(buf + r * 128 + ((cc ^ (r & 7)) << 4));
                const int m = m0 + r, n = n0 + cc * 8;
                if (m < sh.M && n < sh.N)
                  *reinterpret_cast<uint4 *>(mc + 1ll * m * ep.ldc + n) = v;
              }
            }
            ++gcount;
          }
        }
        release_accumulator(buf_idx);
        continue;
      }
      const int m = mt * BM + q * 32 + lane;
      const bool row_ok = m < sh.M;
      const long long batch_off =
          1ll * (bt / ep.batch_div) * ep.batch_hi + 1ll * (bt % ep.batch_div) * ep.batch_lo;
      long long row_off;
      if (split) {
        const int b = m / ep.split_T, t = m % ep.split_T;
        row_off = (1ll * b * ep.split_H * ep.split_T + t) * ep.split_D;
      } else {
        row_off = batch_off + 1ll * m * ep.ldc;
      }
#pragma unroll 1
      for (int chunk = half; chunk < BN / 32; chunk += 2) {
        const int n0 = nt * BN + chunk * 32;
        if (n0 >= sh.N)
          break; // warp-uniform
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                          static_cast<uint32_t>(buf_idx * BN + chunk * 32),
                      r);
        tmem_ld_wait();
        const bool full = (n0 + 32 <= sh.N) && ep.vec_ok;
        if (full) {
          long long off;
          if (split) {
            const int which = n0 / HD, rem = n0 % HD;
            const int h = rem / ep.split_D, d = rem % ep.split_D;
            off = which * ep.split_which_stride + row_off + 1ll * h * ep.split_T * ep.split_D + d;
          } else {
            off = row_off + n0;
          }
          uint32_t bw[16], rw[16];
          if (bias) {
            const uint4 *bp = reinterpret_cast<const uint4 *>(bias + n0);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 t = __ldg(bp + j);
              bw[4 * j] = t.x, bw[4 * j + 1] = t.y, bw[4 * j + 2] = t.z, bw[4 * j + 3] = t.w;
            }
          }
          if (resid && row_ok) {
            const uint4 *rp = reinterpret_cast<const uint4 *>(resid + off);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 t = rp[j];
              rw[4 * j] = t.x, rw[4 * j + 1] = t.y, rw[4 * j + 2] = t.z, rw[4 * j + 3] = t.w;
            }
          }
          uint32_t ow[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float b0 = bias ? bf16_lo(bw[j]) : 0.f, b1 = bias ? bf16_hi(bw[j]) : 0.f;
            const float r0 = (resid && row_ok) ? bf16_lo(rw[j]) : 0.f;
            const float r1 = (resid && row_ok) ? bf16_hi(rw[j]) : 0.f;
            const float v0 = epi_math(__uint_as_float(r[2 * j]), b0, r0, bias != nullptr,
                                      resid != nullptr, alpha, ep.act, rnd);
            const float v1 = epi_math(__uint_as_float(r[2 * j + 1]), b1, r1, bias != nullptr,
                                      resid != nullptr, alpha, ep.act, rnd);
            ow[j] = pack_bf16x2(v0, v1);
          }
          if (row_ok) {
            uint4 *op = reinterpret_cast<uint4 *>(cout + off);
#pragma unroll
            for (int j = 0; j < 4; ++j)
              op[j] = make_uint4(ow[4 * j], ow[4 * j + 1], ow[4 * j + 2], ow[4 * j + 3]);
          }
        } else if (row_ok) {
          for (int j = 0; j < 32; ++j) {
            const int n = n0 + j;
            if (n >= sh.N)
              break;
            long long off;
            if (split) {
              const int which = n / HD, rem = n % HD;
              const int h = rem / ep.split_D, d = rem % ep.split_D;
              off = which * ep.split_which_stride + row_off + 1ll * h * ep.split_T * ep.split_D + d;
            } else {
              off = row_off + n;
            }
            const float b = bias ? __bfloat162float(bias[n]) : 0.f;
            const float rs = resid ? __bfloat162float(resid[off]) : 0.f;
            // r[] must be indexed with a compile-time constant to stay in registers
            float acc = 0.f;
#pragma unroll
            for (int jj = 0; jj < 32; ++jj)
              acc = (jj == j) ? __uint_as_float(r[jj]) : acc;
            cout[off] = __float2bfloat16_rn(
                epi_math(acc, b, rs, bias != nullptr, resid != nullptr, alpha, ep.act, rnd));
          }
        }
      }
      release_accumulator(buf_idx);
    }
    if (lane == 0)
      bulk_wait<0>(); // every TMA store of this warp has completed before the CTA exits
  }

  tc_fence_before();
  // A pair leaves together: the leader's MMAs read the peer's shared memory and the peer signals
  // the leader's barriers, so neither may exit (or free TMEM) while the other still runs.
  if constexpr (CTAS == 2)
    cluster_sync_all();
  else
    __syncthreads();
  if (warp == 1)
    tmem_dealloc_g<CTAS>(tmem_base, Cfg::TMEM_COLS);
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void *p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &p, 12000, cudaEnableDefault,
                                         &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// rank-3 bf16 map, 128-byte swizzle. dims/strides in elements, inner stride 1.
static bool encode_map3(CUtensorMap *map, const void *base, unsigned long long d0,
                        unsigned long long d1, unsigned long long d2, unsigned long long s1,
                        unsigned long long s2, unsigned b0, unsigned b1) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn)
    return false;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {s1 * 2ull, s2 * 2ull};
  cuuint32_t box[3] = {b0, b1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(base), dims,
                  strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// rank-5 bf16 map, 128-byte swizzle; dims/strides in elements, ascending strides.
static bool encode_map5(CUtensorMap *map, const void *base, const unsigned long long (&d)[5],
                        const unsigned long long (&st)[4], const unsigned (&bx)[5]) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn)
    return false;
  cuuint64_t dims[5], strides[4];
  cuuint32_t box[5], estr[5] = {1, 1, 1, 1, 1};
  for (int i = 0; i < 5; ++i)
    dims[i] = d[i], box[i] = bx[i];
  for (int i = 0; i < 4; ++i)
    strides[i] = st[i] * 2ull;
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void *>(base), dims,
                  strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// Output / residual tensor maps for the staged epilogue. Returns false when the
// output addressing cannot be expressed (the kernel then stores directly).
static bool encode_out_maps(const Epilogue &ep, const GemmShape &sh, CUtensorMap *tmC,
                            CUtensorMap *tmR, int *mode) {
  auto al = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  if (!al(ep.c) || (ep.residual && !al(ep.residual)) || (ep.bias && !al(ep.bias)))
    return false;
  unsigned long long d[5], st[4];
  unsigned bx[5] = {64, 32, 1, 1, 1};
  const unsigned long long N = sh.N, M = sh.M;
  if (ep.split_T > 0) {
    const unsigned long long D = ep.split_D, T = ep.split_T, H = ep.split_H;
    if (D % 64 || T % 32 || M % T || N % (H * D) || ep.split_which_stride % 8 ||
        (N / (H * D) > 1 && ep.split_which_stride < M / T * H * T * D))
      return false;
    d[0] = D, d[1] = T, d[2] = H, d[3] = M / T, d[4] = N / (H * D);
    st[0] = D, st[1] = T * D, st[2] = H * T * D;
    st[3] = d[4] > 1 ? static_cast<unsigned long long>(ep.split_which_stride) : st[2] * d[3];
    *mode = 2;
  } else if (ep.batch_div > 1) {
    const unsigned long long H = ep.batch_div, lo = ep.batch_lo, ld = ep.ldc, hi = ep.batch_hi;
    if (sh.batch % ep.batch_div || lo % 8 || ld % 8 || hi % 8 || lo < N || ld < lo * H ||
        (sh.batch / ep.batch_div > 1 && hi < ld * M))
      return false;
    d[0] = N, d[1] = H, d[2] = M, d[3] = sh.batch / ep.batch_div, d[4] = 1;
    st[0] = lo, st[1] = ld, st[2] = d[3] > 1 ? hi : ld * M, st[3] = st[2] * d[3];
    bx[1] = 1, bx[2] = 32;
    *mode = 1;
  } else {
    const unsigned long long ld = ep.ldc, hi = ep.batch_hi;
    if (ld % 8 || ld < N || (sh.batch > 1 && (hi % 8 || hi < ld * M)))
      return false;
    d[0] = N, d[1] = M, d[2] = sh.batch, d[3] = 1, d[4] = 1;
    st[0] = ld, st[1] = sh.batch > 1 ? hi : ld * M, st[2] = st[1] * d[2], st[3] = st[2];
    *mode = 0;
  }
  if (!encode_map5(tmC, ep.c, d, st, bx))
    return false;
  if (ep.residual && !encode_map5(tmR, ep.residual, d, st, bx))
    return false;
  if (!ep.residual)
    *tmR = *tmC;
  return true;
}

static bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// -1: the launcher decides about the L2 hints; 0 none, 1 evict_last on B tiles, 2 that and evict_first on
// the residual and output streams (A/B timing).
static int g_b_hint = -1;
void set_gemm_b_hint(int v) { g_b_hint = v; }
// Bytes of L2 this process has set aside for evict_last lines (0: none). With a set-aside the hints
// hold a whole weight matrix of that size in L2 and more shapes profit.
static double g_l2_set_aside = 0;
void set_gemm_l2_set_aside(double bytes) { g_l2_set_aside = bytes; }

// Returns 0 ok, 1 shape/alignment not supported by this kernel, 2 launch/encode failure.
int launch_gemm_bf16_tcgen05(const GemmOperands &op, const GemmShape &sh, const Epilogue &ep,
                             int *status, int num_sms, cudaStream_t stream) {
  if (sh.M <= 0 || sh.N <= 0 || sh.K <= 0 || sh.batch <= 0)
    return 1;
  if (!aligned16(op.a) || !aligned16(op.b) || (op.lda % 8) || (op.ldb % 8) ||
      (op.a_batch % 8) || (op.b_batch % 8))
    return 1;
  GemmShape s2 = sh;
  // An operand shared by every batch (stride 0) or addressed as a column slab is
  // encoded with a single batch entry; its natural extent serves as the stride.
  const bool b_slab = op.b_col_per_batch > 0;
  if (b_slab && (op.b_kmajor || (op.b_col_per_batch % 8) || op.b_col_per_batch > 0x7fffffffll / sh.batch))
    return 1;
  s2.a_batched = (op.a_batch > 0 && sh.batch > 1) ? 1 : 0;
  s2.b_batched = (op.b_batch > 0 && sh.batch > 1 && !b_slab) ? 1 : 0;
  s2.b_col_per_batch = b_slab ? static_cast<int>(op.b_col_per_batch) : 0;
  const unsigned long long a_nb = s2.a_batched ? sh.batch : 1;
  const unsigned long long b_nb = s2.b_batched ? sh.batch : 1;
  const unsigned long long a_bs = s2.a_batched ? op.a_batch : 1ull * op.lda * sh.M;
  // Tile shape: 128 x {64,128,256} on single CTAs, 256 x {128,256} on CTA pairs. The persistent
  // grid runs ceil(tiles / slots) waves; a shape whose last wave is nearly empty loses up to a
  // whole wave (M = 8192, N = 2048 is 3.46 waves of 256 x 256 pair tiles but 6.92 of 256 x 128),
  // so the candidate with the smallest waves x tile area / relative tile speed wins. The speeds
  // are measured on the decoder's shapes at M = 8192 (CUDA events, idle GPU): 128-wide tiles run
  // at two thirds of the 256-wide ones whether paired or not (the epilogue and the pipeline
  // fill weigh twice as much per FLOP), single CTAs at 0.93 of a pair. In practice the narrow
  // tiles only win where N <= 128 or the wide ones would leave most SMs idle.
  int BN = sh.N > 128 ? 256 : (sh.N > 64 ? 128 : 64);
  int CT = 1;
  if (sh.force_bn > 0) {
    BN = sh.force_bn, CT = sh.force_ctas == 2 ? 2 : 1;
  } else if (sh.N > 64) {
    struct Cand { int bn, ct; double speed; };
    const Cand cands[4] = {{256, 2, 1.00}, {128, 2, 0.66}, {256, 1, 0.93}, {128, 1, 0.65}};
    double best = 0;
    for (const Cand &c : cands) {
      if (c.bn == 256 && sh.N <= 128) continue;
      if (c.ct == 2 && (sh.M < 1024 || num_sms < 2)) continue;
      const long long t = 1ll * ((sh.M + BM * c.ct - 1) / (BM * c.ct)) * ((sh.N + c.bn - 1) / c.bn) * sh.batch;
      const long long slots = c.ct == 2 ? num_sms / 2 : num_sms;
      if (c.ct == 2 && t < slots) continue; // too few pair tiles to fill the device
      const double waves = static_cast<double>((t + slots - 1) / slots);
      const double cost = waves * (BM * c.ct) * c.bn / c.speed / c.ct; // per-SM time units
      if (best == 0 || cost < best) best = cost, BN = c.bn, CT = c.ct;
    }
  }
  const bool pairs = CT == 2;
  const long long pair_tiles = 1ll * ((sh.M + 2 * BM - 1) / (2 * BM)) * ((sh.N + BN - 1) / BN) * sh.batch;
  // B wider than a third of L2 is cut into panels of about 24 MB (see decode_tile). Measured on the
  // 32000-column head at M = 65536: DRAM reads 3.80 / 3.13 / 3.89 GB with panels of 16 / 24 / 32 MB
  // (narrow panels re-read A more often, wide ones lose their weights to the logits streaming past).
  {
    const double b_bytes = 2.0 * sh.K * sh.N;
    const double tile_bytes = 2.0 * sh.K * BN;
    s2.panel_n = b_bytes > 48e6 ? static_cast<int>(24e6 / tile_bytes) : 0;
    if (b_bytes > 48e6 && s2.panel_n < 1)
      s2.panel_n = 1;
  }
  // L2 priorities. With a long K (fc2: K = 8192) every wave of tiles streams tens of MB of A past a B
  // that all of them share, and LRU drops B between waves: B tiles then ask for evict_last and the
  // single-use residual and output streams for evict_first. Measured at M = 65536, K = 8192, N = 2048:
  // DRAM reads 2610 -> 2077 MB, 1.498 -> 1.491 ms. With K = 2048 (fc1, the LM head) the same hints
  // save less traffic and cost 0.3-1 % time, so they stay off there.
  {
    const double b_bytes = 2.0 * sh.K * sh.N;
    const bool long_k = sh.K >= 4096 && b_bytes >= 8e6 && b_bytes <= 64e6;
    const bool wide_n = g_l2_set_aside > 0 && sh.N >= 8192 && b_bytes >= 8e6 && b_bytes <= g_l2_set_aside;
    const bool wanted = sh.M >= 4096 && !op.b_kmajor && (long_k || wide_n);
    s2.b_evict_last = g_b_hint >= 0 ? g_b_hint : (wanted ? 2 : 0);
  }
  CUtensorMap tmA, tmB;
  if (!encode_map3(&tmA, op.a, sh.K, sh.M, a_nb, op.lda, a_bs, BK, BM))
    return 2;
  bool okb;
  if (op.b_kmajor) {
    const unsigned long long b_bs = s2.b_batched ? op.b_batch : 1ull * op.ldb * sh.N;
    okb = encode_map3(&tmB, op.b, sh.K, sh.N, b_nb, op.ldb, b_bs, BK, BN / CT);
  } else {
    const unsigned long long cols = b_slab ? 1ull * op.b_col_per_batch * sh.batch : sh.N;
    const unsigned long long b_bs = s2.b_batched ? op.b_batch : 1ull * op.ldb * sh.K;
    okb = encode_map3(&tmB, op.b, cols, sh.K, b_nb, op.ldb, b_bs, 64, BK);
  }
  if (!okb)
    return 2;
  const long long tiles = 1ll * ((sh.M + BM - 1) / BM) * ((sh.N + BN - 1) / BN) * sh.batch;
  const int grid = static_cast<int>(tiles < num_sms ? tiles : num_sms);
  Epilogue ep2 = ep;
  CUtensorMap tmC, tmR;
  int mode = 0;
  ep2.tma_out = encode_out_maps(ep, sh, &tmC, &tmR, &mode) ? 1 : 0;
  ep2.tma_mode = mode;
  // the mirrored copy exists only in the staged epilogue of a plain [M,N] output
  if (ep.c_mirror && (!ep2.tma_out || mode != 0 || sh.batch != 1 || (sh.N % 8) ||
                      !aligned16(ep.c_mirror)))
    return 1;
  if (!ep2.tma_out)
    tmC = tmR = tmA; // placeholders, never dereferenced

#define MU_LAUNCH(BN_, KM_)                                                                      \
  do {                                                                                           \
    auto kern = gemm_bf16_tcgen05_kernel<BN_, KM_, 1>;                                           \
    static PerDeviceOnce attr_set;                                                               \
    if (attr_set.get() < 0) {                                                                             \
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,                \
                               GemmCfg<BN_>::SMEM_BYTES) != cudaSuccess)                         \
        return 2;                                                                                \
      attr_set.set(1);                                                                           \
    }                                                                                            \
    kern<<<grid, GEMM_THREADS, GemmCfg<BN_>::SMEM_BYTES, stream>>>(tmA, tmB, tmC, tmR, s2, ep2,     \
                                                                   status);                       \
  } while (0)

  // CTA pairs: clusters of two, as many as the device can hold at once (persistent).
#define MU_LAUNCH_PAIR(BN_, KM_)                                                                 \
  do {                                                                                           \
    auto kern = gemm_bf16_tcgen05_kernel<BN_, KM_, 2>;                                           \
    constexpr int smem = GemmCfg<BN_, 2>::SMEM_BYTES;                                            \
    static PerDeviceOnce cluster_cache;                                                          \
    int max_clusters = cluster_cache.get();                                                      \
    cudaLaunchConfig_t cfg = {};                                                                 \
    cudaLaunchAttribute at[1];                                                                   \
    at[0].id = cudaLaunchAttributeClusterDimension;                                              \
    at[0].val.clusterDim.x = 2, at[0].val.clusterDim.y = 1, at[0].val.clusterDim.z = 1;          \
    cfg.blockDim = dim3(GEMM_THREADS), cfg.dynamicSmemBytes = smem, cfg.stream = stream;         \
    cfg.attrs = at, cfg.numAttrs = 1;                                                            \
    if (max_clusters < 0) {                                                                      \
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) !=       \
          cudaSuccess)                                                                           \
        return 2;                                                                                \
      int dev = 0, dev_sms = 0; /* the whole device, whatever SM budget this call runs under */   \
      if (cudaGetDevice(&dev) != cudaSuccess ||                                                  \
          cudaDeviceGetAttribute(&dev_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)  \
        return 2;                                                                                \
      cfg.gridDim = dim3(dev_sms & ~1);                                                          \
      int n = 0;                                                                                 \
      if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0)               \
        return 2;                                                                                \
      max_clusters = n;                                                                          \
      cluster_cache.set(n);                                                                      \
    }                                                                                            \
    long long nc = pair_tiles < max_clusters ? pair_tiles : max_clusters;                        \
    if (nc > num_sms / 2)                                                                        \
      nc = num_sms / 2;                                                                          \
    cfg.gridDim = dim3(static_cast<unsigned>(2 * nc));                                           \
    if (cudaLaunchKernelEx(&cfg, kern, tmA, tmB, tmC, tmR, s2, ep2, status) != cudaSuccess)      \
      return 2;                                                                                  \
  } while (0)

  if (pairs) {
    if (BN == 256) {
      if (op.b_kmajor)
        MU_LAUNCH_PAIR(256, true);
      else
        MU_LAUNCH_PAIR(256, false);
    } else {
      if (op.b_kmajor)
        MU_LAUNCH_PAIR(128, true);
      else
        MU_LAUNCH_PAIR(128, false);
    }
    return cudaGetLastError() == cudaSuccess ? 0 : 2;
  }

  if (op.b_kmajor) {
    if (BN == 256)
      MU_LAUNCH(256, true);
    else if (BN == 128)
      MU_LAUNCH(128, true);
    else
      MU_LAUNCH(64, true);
  } else {
    if (BN == 256)
      MU_LAUNCH(256, false);
    else if (BN == 128)
      MU_LAUNCH(128, false);
    else
      MU_LAUNCH(64, false);
  }
#undef MU_LAUNCH
#undef MU_LAUNCH_PAIR
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

} // namespace mu
