// Fused attention core for sm_100a (bf16): S = scale·Q·K', causal mask, online
// softmax, O = P·V — scores and probabilities never touch HBM.
//
// Replaces the scale-mul → mask build → masked_fill → softmax → matmul chain of
// MultiHeadAttention::forward_impl (src/nn/attention.hpp:64-99), which the
// reference runs as five full passes over a [B·H·T, B·H·T] matrix (two of them
// on the host). Only the row's own head block is ever touched here.
//
// Persistent: one CTA per SM walks (head, 128-query tile) works, heavy and light query
// tiles paired so that every CTA sees the same number of key tiles; the rings run on
// across works, so the next work's loads and first Q·K' overlap this work's epilogue.
// 320 threads:
//   warp 0    TMA producer: Q per work, K and V tiles of 128 keys through two rings.
//   warp 1    tcgen05.mma issuer: S_j = Q·K_j' (M=128,N=128) into a double-
//             buffered TMEM S tile, O_j = P_j·V_j (M=128,N=D) into a double-
//             buffered TMEM O tile.
//   warps 2-9 two threads per query row (TMEM lane = row, each owns half of the
//             columns; two warps per scheduler): rounding/scale/mask,
//             running max and sum, P_j → swizzled smem (A operand of P·V);
//             O accumulates in TMEM over the key tiles of a work and is rescaled in
//             place only when the row maximum has grown by more than 2^8; the final
//             O/l is staged to smem and written with TMA (token-major, heads merged:
//             the [B,T,H·D] layout out_proj consumes).
// K addressing: LITERAL reads K's [N,D] buffer as a row-major [D,N] matrix
// (what the reference computes, see include/munet_b200.h), MATH is Q·Kᵀ.
// Numerics follow the reference's bf16 pipeline where it is cheap to: scores are
// rounded to bf16, multiplied by the bf16-rounded scale and rounded again before
// the softmax; P is rounded to bf16 before P·V; fp32 accumulation elsewhere.
#include "common.h"
#include "ptx.cuh"
#include <cuda.h>
#include <type_traits>

namespace mu {

constexpr int ATT_PARTS = 2;   // softmax warps per TMEM lane quarter (each owns 1/PARTS of the columns)
constexpr int ATT_THREADS = 64 + 128 * ATT_PARTS; // producer warp, MMA warp, softmax warps
constexpr int BQ = 128, BKV = 128;

template <int D> struct AttCfg {
  static constexpr int Q_BYTES = BQ * D * 2;
  static constexpr int K_BYTES = BKV * D * 2;
  static constexpr int V_BYTES = BKV * D * 2;
  static constexpr int P_BYTES = BQ * BKV * 2; // one of two buffers
  static constexpr int STAGES = D == 128 ? 2 : 4;
  static constexpr int KV_STAGE = K_BYTES + V_BYTES;
  // row maxima [tile parity][part][row] as bf16; the partial row sums [part][row] as fp32 reuse it
  static constexpr int XCHG_BYTES = ATT_PARTS * BQ * 4;
  static constexpr int SMEM_BYTES =
      Q_BYTES + STAGES * KV_STAGE + 2 * P_BYTES + XCHG_BYTES + 512 /*barriers*/;
  static constexpr int TMEM_COLS = 512; // S0 S1 at 0/128, O0 O1 at 256/256+D
};

struct AttParams {
  int T, H, BH;
  int causal;
  float scale;   // 1/sqrt(D) as float
  int n_qtiles;
  int chunk_heads; // heads whose K and V are worked on together (sized to stay in L2)
  int chunk_rot;   // rotation of the CTA deal from one chunk to the next
  // Two-query-tile kernel only: every output tile is also written, with ordinary 16-byte stores,
  // to mirror[(b*T + t) * out_ld + h*D + d] (null = off). The pointer may map another GPU's
  // memory: a tensor-parallel rank hands the output of its heads to its peer from inside the
  // kernel.
  __nv_bfloat16 *mirror;
  long long out_ld; // row stride of the output in elements (>= H*D)
};

template <int D, bool LITERAL>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap tmQ,
                         const __grid_constant__ CUtensorMap tmK,
                         const __grid_constant__ CUtensorMap tmV,
                         const __grid_constant__ CUtensorMap tmO, AttParams prm, int *status) {
  using Cfg = AttCfg<D>;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int DB = D / 64; // 64-element boxes along the head dim
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t *smem = smem_raw;
  if (smem_u32(smem_raw) & 1023u) { // swizzled TMA boxes need 1024-byte alignment
    if (threadIdx.x == 0)
      atomicCAS(status, 0, MU_DEV_BAD_INDEX);
    return;
  }
  uint8_t *sQ = smem;
  uint8_t *sKV = sQ + Cfg::Q_BYTES;
  uint8_t *sP = sKV + STAGES * Cfg::KV_STAGE;
  uint8_t *xchg = sP + 2 * Cfg::P_BYTES;
  uint64_t *bars = reinterpret_cast<uint64_t *>(xchg + Cfg::XCHG_BYTES);
  uint64_t *q_full = bars;
  // K and V have their own full/empty rings over the same stage memory: a K buffer is free as
  // soon as its Q·K' has run, long before the P·V that frees the V buffer of the same tile, so
  // the next K tiles are requested a whole softmax tile earlier than with a joint barrier.
  uint64_t *k_full = q_full + 1;
  uint64_t *k_empty = k_full + STAGES;
  uint64_t *v_full = k_empty + STAGES;
  uint64_t *v_empty = v_full + STAGES;
  uint64_t *s_full = v_empty + STAGES;
  uint64_t *s_empty = s_full + 2;
  uint64_t *p_full = s_empty + 2;
  // O accumulates in TMEM over the key tiles of a work (one buffer per work parity):
  //   o_done[tile parity]  a P·V has completed (P buffer reusable, O readable / rescalable)
  //   o_free[work parity]  the softmax warps have read the finished O of that buffer
  uint64_t *o_done = p_full + 2;
  uint64_t *o_free = o_done + 2;
  uint64_t *xbar = o_free + 2; // [quarter][tile parity]: paired softmax warps
  uint64_t *xend = xbar + 8;    // [quarter][0: row sums, 1: output staged]
  uint64_t *q_empty = xend + 8;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(q_empty + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Persistent CTA: every role walks the same static sequence of works (one head, one tile of 128
  // queries), produced by `next_work`. Under the causal mask a query tile qt sees qt + 1 key
  // tiles, so works differ in size by up to n_qtiles x. Heads are taken in chunks of `chunk_heads`
  // (their K and V stay in L2 while the chunk is worked on); inside a chunk the works are ordered
  // by falling size — all heads' last query tile first — and dealt to the CTAs in a serpentine
  // (pass 0: CTA 0..n-1, pass 1: n-1..0, ...), which pairs every large work with a small one;
  // from chunk to chunk the deal is rotated so that the leftovers of a partial last pass fall on
  // different CTAs. At 128 heads of 8 tiles that is 32 key tiles on the busiest of 148 CTAs where
  // head-by-head pairs of (heavy, light) tiles gave 36; larger batches end within a tile of even.
  // Pipeline counters (key tiles, works) run on across works so loads and Q.K' of the next work
  // overlap the epilogue of the current one.
  struct Work {
    int bh, q0, nk;
  };
  struct WorkIter {
    int chunk, pass;
  };
  const int n_cta = static_cast<int>(gridDim.x);
  auto next_work = [&](WorkIter &it, Work &wk) -> bool {
    for (;;) {
      const int h0 = it.chunk * prm.chunk_heads;
      if (h0 >= prm.BH)
        return false;
      const int hb = min(prm.chunk_heads, prm.BH - h0);
      const long long n_works = 1ll * hb * prm.n_qtiles;
      if (1ll * it.pass * n_cta >= n_works) {
        ++it.chunk, it.pass = 0;
        continue;
      }
      const int c = static_cast<int>((blockIdx.x + 1ll * it.chunk * prm.chunk_rot) % n_cta);
      const int slot = (it.pass & 1) ? n_cta - 1 - c : c;
      const long long p = 1ll * it.pass * n_cta + slot;
      ++it.pass;
      if (p >= n_works)
        continue; // this CTA sits out the partial last pass of the chunk
      const int qt = prm.n_qtiles - 1 - static_cast<int>(p / hb);
      wk.bh = h0 + static_cast<int>(p % hb);
      wk.q0 = qt * BQ;
      const int kv_len = prm.causal ? min(prm.T, wk.q0 + BQ) : prm.T;
      wk.nk = (kv_len + BKV - 1) / BKV;
      return true;
    }
  };

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&s_full[b], 1);
      mbar_init(&s_empty[b], 4 * ATT_PARTS);
      mbar_init(&p_full[b], 4 * ATT_PARTS);
      mbar_init(&o_done[b], 1);
      mbar_init(&o_free[b], 4 * ATT_PARTS);
    }
    for (int i = 0; i < 8; ++i) {
      mbar_init(&xbar[i], ATT_PARTS);
      mbar_init(&xend[i], ATT_PARTS);
    }
    fence_barrier_init();
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
    prefetch_tmap(&tmO);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base, tmem_O = tmem_base + 256;
  // Head size 64 leaves 128 tensor-memory columns free: the probabilities go there (two buffers of
  // 64 packed columns) and P.V takes its A operand from tensor memory instead of shared memory.
  constexpr bool P_TMEM = (D == 64);
  const uint32_t tmem_P = tmem_base + 384;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      bool ok = true;
      uint32_t kt = 0, w = 0; // key tiles and works issued so far
      WorkIter wit = {0, 0};
      for (Work wk; ok && next_work(wit, wk);) {
          // Q is single-buffered: the last Q·K' of the previous work must have read it
          if (!mbar_wait(q_empty, (w & 1) ^ 1)) {
            atomicCAS(status, 0, MU_DEV_TIMEOUT_PRODUCER);
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(q_full, Cfg::Q_BYTES);
#pragma unroll
          for (int db = 0; db < DB; ++db)
            tma_load_3d(sQ + db * (BQ * 128), &tmQ, q_full, db * 64, wk.q0, wk.bh);
          ++w;
          for (int j = 0; j < wk.nk; ++j, ++kt) {
            const int stage = kt % STAGES;
            const uint32_t par = ((kt / STAGES) & 1) ^ 1;
            if (!mbar_wait(&k_empty[stage], par)) {
              atomicCAS(status, 0, MU_DEV_TIMEOUT_PRODUCER);
              ok = false;
              break;
            }
            uint8_t *sK = sKV + stage * Cfg::KV_STAGE;
            uint8_t *sV = sK + Cfg::K_BYTES;
            mbar_arrive_expect_tx(&k_full[stage], Cfg::K_BYTES);
            const int k0 = j * BKV;
            if (LITERAL) {
              // K' tile = rows d, columns bh*T + k0.. of the [D, N] view: [dbox][nbox][64 x 128 B]
#pragma unroll
              for (int db = 0; db < DB; ++db)
#pragma unroll
                for (int nb = 0; nb < 2; ++nb)
                  tma_load_3d(sK + (db * 2 + nb) * 8192, &tmK, &k_full[stage],
                              wk.bh * prm.T + k0 + nb * 64, db * 64, 0);
            } else {
#pragma unroll
              for (int db = 0; db < DB; ++db)
                tma_load_3d(sK + db * (BKV * 128), &tmK, &k_full[stage], db * 64, k0, wk.bh);
            }
            if (!mbar_wait(&v_empty[stage], par)) {
              atomicCAS(status, 0, MU_DEV_TIMEOUT_PRODUCER);
              ok = false;
              break;
            }
            mbar_arrive_expect_tx(&v_full[stage], Cfg::V_BYTES);
            // V tile as MN-major B operand: [keybox][dbox][64 keys x 128 B]
#pragma unroll
            for (int kb = 0; kb < 2; ++kb)
#pragma unroll
              for (int db = 0; db < DB; ++db)
                tma_load_3d(sV + (kb * DB + db) * 8192, &tmV, &v_full[stage], db * 64,
                            k0 + kb * 64, wk.bh);
          }
        }
      if (!ok)
        for (int i = 0; i < 64; ++i)
          __nanosleep(1000);
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc(1u, 0u, LITERAL ? 1u : 0u, BQ, BKV);
      constexpr uint32_t idesc_pv = make_idesc(1u, 0u, 1u, BQ, D);
      const uint32_t q_addr = smem_u32(sQ);
      bool ok = true;
      uint32_t t = 0, w = 0; // key tiles and works issued so far (they index every ring)
      // P·V of tile number i (global count), the j-th of work number wi: needs its V tile and the
      // probabilities; the first one of a work overwrites that work's O buffer, which the
      // softmax warps must have drained (two works ago).
      auto issue_pv = [&](uint32_t i, int j, uint32_t wi) -> bool {
        const int b = i & 1;
        const uint32_t par = (i >> 1) & 1;
        const int ob = wi & 1;
        if (!mbar_wait(&v_full[i % STAGES], (i / STAGES) & 1) || !mbar_wait(&p_full[b], par))
          return false;
        if (j == 0 && !mbar_wait(&o_free[ob], ((wi >> 1) & 1) ^ 1))
          return false;
        tc_fence_after();
        const uint32_t p_addr = smem_u32(sP + b * Cfg::P_BYTES);
        const uint32_t v_addr = smem_u32(sKV + (i % STAGES) * Cfg::KV_STAGE + Cfg::K_BYTES);
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k) {
          const uint64_t ad = make_smem_desc(p_addr + (k / 4) * (BQ * 128) + (k % 4) * 32, 16, 1024);
          const uint64_t bd = make_smem_desc(v_addr + (k / 4) * (DB * 8192) + (k % 4) * 2048, 8192, 1024);
          if constexpr (P_TMEM)
            umma_f16_ts(tmem_O + ob * D, tmem_P + b * (BKV / 2) + k * 8, bd, idesc_pv, (j | k) != 0 ? 1u : 0u);
          else
            umma_f16(tmem_O + ob * D, ad, bd, idesc_pv, (j | k) != 0 ? 1u : 0u);
        }
        umma_commit(&o_done[b]);
        umma_commit(&v_empty[i % STAGES]);
        return true;
      };
      WorkIter wit = {0, 0};
      for (Work wk; ok && next_work(wit, wk);) {
          if (!mbar_wait(q_full, w & 1)) {
            atomicCAS(status, 0, MU_DEV_TIMEOUT_MMA);
            ok = false;
            break;
          }
          ++w;
          for (int j = 0; j < wk.nk && ok; ++j, ++t) {
            const int stage = t % STAGES, b = t & 1;
            if (!mbar_wait(&k_full[stage], (t / STAGES) & 1) ||
                !mbar_wait(&s_empty[b], ((t >> 1) & 1) ^ 1)) {
              atomicCAS(status, 0, MU_DEV_TIMEOUT_MMA);
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t k_addr = smem_u32(sKV + stage * Cfg::KV_STAGE);
#pragma unroll
            for (int k = 0; k < D / 16; ++k) {
              const uint64_t ad = make_smem_desc(q_addr + (k / 4) * (BQ * 128) + (k % 4) * 32, 16, 1024);
              const uint64_t bd =
                  LITERAL ? make_smem_desc(k_addr + (k / 4) * (2 * 8192) + (k % 4) * 2048, 8192, 1024)
                          : make_smem_desc(k_addr + (k / 4) * (BKV * 128) + (k % 4) * 32, 16, 1024);
              umma_f16(tmem_S + b * BKV, ad, bd, idesc_qk, k != 0 ? 1u : 0u);
            }
            umma_commit(&s_full[b]);
            umma_commit(&k_empty[stage]);
            if (j == wk.nk - 1)
              umma_commit(q_empty); // the producer may fetch the next work's Q
            if (j > 0 && !issue_pv(t - 1, j - 1, w - 1)) {
              atomicCAS(status, 0, MU_DEV_TIMEOUT_MMA);
              ok = false;
            }
          }
          if (ok && !issue_pv(t - 1, wk.nk - 1, w - 1)) {
            atomicCAS(status, 0, MU_DEV_TIMEOUT_MMA);
            ok = false;
          }
        }
    }
    __syncwarp();
  } else {
    // ------------- softmax / correction / output (warps 2..9, two per row quarter) -------
    // Warps w and w+4 share the TMEM lane quarter q = w & 3 (rows q*32..q*32+31); `half`
    // selects which 64 score columns and which D/2 output columns a thread owns. Two warps
    // per scheduler hide each other's dependent-issue latency. The pair agrees on the row
    // maximum through shared memory and a (bounded) mbarrier; row sums stay partial until the end.
    const int q = warp & 3;
    const int half = (warp - 2) >> 2; // which 1/PARTS of the columns
    const int row = q * 32 + lane;       // row inside the query tile = TMEM lane
    const uint32_t lane_sel = static_cast<uint32_t>(q * 32) << 16;
    const float scale_b = bf16_round(prm.scale);
    constexpr float L2E = 1.4426950408889634f;
    constexpr int SC = BKV / ATT_PARTS; // score columns per thread
    constexpr int DH = D / ATT_PARTS;   // output columns per thread
    uint16_t *xm = reinterpret_cast<uint16_t *>(xchg); // [tile parity][half][row] partial maxima (bf16)
    float *xl = reinterpret_cast<float *>(xchg);       // [half][row] partial row sums (end only)
    float o_acc[DH];
    bool ok = true;
    bool store_pending = false; // this thread issued the previous work's output store
    uint32_t t = 0, w = 0;      // key tiles and works consumed so far

    auto pair_sync = [&](uint64_t *bar, uint32_t parity) -> bool {
      __syncwarp();
      if (lane == 0)
        mbar_arrive(bar);
      return mbar_wait(bar, parity);
    };

    // Multiply this thread's part of the work's O accumulator (TMEM) by `a` — the online-softmax
    // correction. It is only called when the running maximum has grown by more than 2^8 since
    // the exponent reference was set (see below), and never while a P·V is in flight.
    auto rescale_o = [&](int ob, float a) {
      tc_fence_after();
      if constexpr (DH % 32 == 0) {
#pragma unroll
        for (int c = 0; c < DH / 32; ++c) {
          uint32_t r[32];
          const uint32_t addr = tmem_O + lane_sel + ob * D + half * DH + c * 32;
          tmem_ld_32x32(addr, r);
          tmem_ld_wait();
#pragma unroll
          for (int k = 0; k < 32; ++k)
            r[k] = __float_as_uint(__uint_as_float(r[k]) * a);
          tmem_st_32x32(addr, r);
        }
      } else {
        static_assert(DH % 32 == 0 || DH == 16, "output columns per thread");
        uint32_t r16[16];
        const uint32_t addr = tmem_O + lane_sel + ob * D + half * DH;
        tmem_ld_32x16(addr, r16);
        tmem_ld_wait();
#pragma unroll
        for (int k = 0; k < 16; ++k)
          r16[k] = __float_as_uint(__uint_as_float(r16[k]) * a);
        tmem_st_32x16(addr, r16);
      }
      tmem_st_wait();
      tc_fence_before();
    };
    // The finished O of a work: TMEM -> registers.
    auto load_o = [&](int ob) {
      tc_fence_after();
      if constexpr (DH % 32 == 0) {
#pragma unroll
        for (int c = 0; c < DH / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(tmem_O + lane_sel + ob * D + half * DH + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int k = 0; k < 32; ++k)
            o_acc[c * 32 + k] = __uint_as_float(r[k]);
        }
      } else {
        uint32_t r16[16];
        tmem_ld_32x16(tmem_O + lane_sel + ob * D + half * DH, r16);
        tmem_ld_wait();
#pragma unroll
        for (int k = 0; k < 16; ++k)
          o_acc[k] = __uint_as_float(r16[k]);
      }
      tc_fence_before();
    };

    WorkIter wit = {0, 0};
    for (Work wk; ok && next_work(wit, wk);) {
    const int q0 = wk.q0, nk = wk.nk, bh = wk.bh;
    const int qrow = q0 + row; // position in the sequence
    // m_ref is the maximum the exponents are taken against. It follows the running maximum
    // only when that has moved by more than 2^8: probabilities then stay below 256 (exact enough
    // in bf16, harmless in the fp32 accumulators) and O in TMEM almost never needs rescaling.
    float m_ref = -INFINITY, l_run = 0.f;
    const int ob = w & 1; // this work's O buffer
    for (int j = 0; j < nk && ok; ++j, ++t) {
      const int b = t & 1;
      if (!mbar_wait(&s_full[b], (t >> 1) & 1)) {
        atomicCAS(status, 0, MU_DEV_TIMEOUT_EPILOGUE);
        ok = false;
        break;
      }
      tc_fence_after();
      const int k0 = j * BKV;
      // keys this row may see inside the tile: [0, lim)
      int lim = prm.T - k0;
      if (prm.causal)
        lim = min(lim, qrow - k0 + 1);
      const bool need_mask = (k0 + BKV > prm.T) || (prm.causal && k0 + BKV > q0); // warp-uniform
      const uint32_t s_addr = tmem_S + lane_sel + b * BKV + half * SC;
      // pass 1: first rounding (fp32 accumulator -> bf16, packed pairs kept in registers), mask,
      // and the maximum over this thread's columns on the packed values. Rounding and the
      // (positive) scale are monotone, so the maximum of the transformed scores is the transform
      // of the maximum.
      uint32_t sp[SC / 2];
      uint32_t mxa[4] = {0xFF80FF80u, 0xFF80FF80u, 0xFF80FF80u, 0xFF80FF80u}; // four short max chains
      {
        uint32_t r[SC / 32][32];
#pragma unroll
        for (int c = 0; c < SC / 32; ++c)
          tmem_ld_32x32(s_addr + c * 32, r[c]);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < SC / 32; ++c)
#pragma unroll
          for (int k = 0; k < 32; k += 2) {
            uint32_t u = pack_bf16x2(__uint_as_float(r[c][k]), __uint_as_float(r[c][k + 1]));
            if (need_mask) {
              const int col = half * SC + c * 32 + k;
              if (col >= lim)
                u = (u & 0xFFFF0000u) | 0x0000FF80u;
              if (col + 1 >= lim)
                u = (u & 0x0000FFFFu) | 0xFF800000u;
            }
            sp[c * 16 + k / 2] = u;
            mxa[(k >> 1) & 3] = bf16x2_max(mxa[(k >> 1) & 3], u);
          }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0)
        mbar_arrive(&s_empty[b]); // the scores now live in registers
      const uint32_t mx2 = bf16x2_max(bf16x2_max(mxa[0], mxa[1]), bf16x2_max(mxa[2], mxa[3]));
      const float raw_mx = fmaxf(bf16_lo(mx2), bf16_hi(mx2));
      const float mine = bf16_round(raw_mx * scale_b); // exactly a bf16 value (or -inf)
      xm[(b * ATT_PARTS + half) * BQ + row] = static_cast<uint16_t>(__float_as_uint(mine) >> 16);
      if (store_pending) {
        // The previous work's output was staged in the P buffers; its store must have read them
        // before anyone of this row quarter (all behind the barrier below) writes P again.
        bulk_wait_read<0>();
        store_pending = false;
      }
      if (!pair_sync(&xbar[q * 2 + b], (t >> 1) & 1)) {
        atomicCAS(status, 0, MU_DEV_TIMEOUT_EPILOGUE);
        ok = false;
        break;
      }
      float mx = m_ref;
#pragma unroll
      for (int pt = 0; pt < ATT_PARTS; ++pt)
        mx = fmaxf(mx, __uint_as_float(static_cast<uint32_t>(xm[(b * ATT_PARTS + pt) * BQ + row]) << 16));
      // rows past the end of the sequence see no key at all: keep them finite
      const float m_new = (mx == -INFINITY) ? 0.f : mx;
      if (j == 0) {
        m_ref = m_new; // nothing accumulated yet
      } else {
        // Both warps of a pair see the same rows and the same maxima, so they take the same branch.
        const bool grow = (m_new - m_ref) * L2E > 8.0f;
        if (__any_sync(0xffffffffu, grow)) {
          // the previous P·V must have landed in O before it is scaled
          if (!mbar_wait(&o_done[(t - 1) & 1], ((t - 1) >> 1) & 1)) {
            atomicCAS(status, 0, MU_DEV_TIMEOUT_EPILOGUE);
            ok = false;
            break;
          }
          const float a = ex2_approx((m_ref - m_new) * L2E);
          rescale_o(ob, a);
          l_run *= a;
          m_ref = m_new;
        }
      }
      const float mL = m_ref * L2E;
      // P buffer b was last read by the P·V of tile t-2
      if (!mbar_wait(&o_done[b], ((t >> 1) & 1) ^ 1)) {
        atomicCAS(status, 0, MU_DEV_TIMEOUT_EPILOGUE);
        ok = false;
        break;
      }
      // pass 2: second rounding (times the bf16 scale, one packed multiply), probabilities ->
      // bf16 -> swizzled smem (K-major A operand of P·V). Masked columns hold -inf: exp2 gives 0.
      uint8_t *prow = sP + b * Cfg::P_BYTES + row * 128;
      const uint32_t scale2 = (__float_as_uint(scale_b) >> 16) * 0x00010001u;
      float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
      for (int c = 0; c < SC / 32; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int k = 0; k < 16; ++k) {
          const uint32_t u = bf16x2_mul(sp[c * 16 + k], scale2);
          const float p0 = ex2_approx(fmaf(bf16_lo(u), L2E, -mL));
          const float p1 = ex2_approx(fmaf(bf16_hi(u), L2E, -mL));
          sum0 += p0;
          sum1 += p1;
          pk[k] = pack_bf16x2(p0, p1);
        }
        if constexpr (P_TMEM) {
          tmem_st_32x16(tmem_P + lane_sel + b * (BKV / 2) + half * (SC / 2) + c * 16, pk);
          continue;
        }
        // 32 columns = four 16-byte chunks of one 64-column box of the P tile
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          const int col16 = (half * SC) / 8 + c * 4 + ch; // 16-byte chunk index inside the row
          const int cc = col16 & 7;
          *reinterpret_cast<uint4 *>(prow + (col16 >> 3) * (BQ * 128) + ((cc ^ (lane & 7)) << 4)) =
              make_uint4(pk[4 * ch], pk[4 * ch + 1], pk[4 * ch + 2], pk[4 * ch + 3]);
        }
      }
      if constexpr (P_TMEM)
        tmem_st_wait();
      tc_fence_before();
      if constexpr (!P_TMEM)
        fence_proxy_async();
      __syncwarp();
      if (lane == 0)
        mbar_arrive(&p_full[b]);
      l_run += sum0 + sum1;
    }
    // the last P·V of the work has completed: drain O and hand the buffer back
    if (ok && !mbar_wait(&o_done[(t - 1) & 1], ((t - 1) >> 1) & 1)) {
      atomicCAS(status, 0, MU_DEV_TIMEOUT_EPILOGUE);
      ok = false;
    }
    if (ok) {
      load_o(ob);
      __syncwarp();
      if (lane == 0)
        mbar_arrive(&o_free[ob]);
    }
    if (ok) {
      // full row sum = the pair's partial sums (every P·V has completed: xchg is idle)
      xl[half * BQ + row] = l_run;
      ok = pair_sync(&xend[q * 2 + 0], w & 1);
      float l_all = 0.f;
#pragma unroll
      for (int pt = 0; pt < ATT_PARTS; ++pt)
        l_all += xl[pt * BQ + row];
      if (!ok)
        l_all = 1.f;
      // normalise and stage this thread's D/2 columns in the (now idle) P buffer
      const float inv = l_all > 0.f ? 1.0f / l_all : 0.f;
      uint8_t *orow = sP + row * 128;
#pragma unroll
      for (int i = 0; i < DH / 8; ++i) {
        const int gc = (half * DH) / 8 + i;
        const int box = gc >> 3, cc = gc & 7;
        uint32_t ow[4];
#pragma unroll
        for (int k = 0; k < 4; ++k)
          ow[k] = pack_bf16x2(o_acc[i * 8 + 2 * k] * inv, o_acc[i * 8 + 2 * k + 1] * inv);
        *reinterpret_cast<uint4 *>(orow + box * (BQ * 128) + ((cc ^ (lane & 7)) << 4)) =
            make_uint4(ow[0], ow[1], ow[2], ow[3]);
      }
      fence_proxy_async();
      if (ok)
        ok = pair_sync(&xend[q * 2 + 1], w & 1);
      if (!ok)
        atomicCAS(status, 0, MU_DEV_TIMEOUT_EPILOGUE);
      if (ok && half == 0 && lane == 0 && q0 + q * 32 < prm.T) {
        const int bb = bh / prm.H, hh = bh % prm.H;
#pragma unroll
        for (int db = 0; db < DB; ++db)
          tma_store_5d(&tmO, sP + db * (BQ * 128) + q * 32 * 128, db * 64, hh, q0 + q * 32, bb, 0);
        bulk_commit();
        store_pending = true;
      }
    }
    ++w;
    } // works
    if (store_pending)
      bulk_wait<0>(); // shared memory must outlive the last store
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1)
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

// ---------------------------------------------------------------------------
// Two query tiles per CTA (the main kernel for D = 64 and 128)
// ---------------------------------------------------------------------------
// The kernel above keeps one query tile per CTA in flight and two threads per query row; its
// softmax warps are a chain of dependent steps per key tile (tensor-memory load, row-maximum
// exchange through shared memory, exponentials, probabilities to swizzled shared memory, proxy
// fence) that the tensor pipe waits on: 24 % busy. This kernel changes the three things that
// chain is made of:
//   * a work is one head with TWO adjacent query tiles, A and B, which share every K and V
//     tile; warps 2-5 run the softmax of A, warps 6-9 that of B, one thread per query row (its
//     TMEM lane), so the row maximum and the row sum never leave the thread;
//   * while the softmax of A runs, the tensor pipe works on B (P_B·V, Q_B·K' of the next tile)
//     and the other way round;
//   * the probabilities are written back to tensor memory over the score tile they came from
//     (64 packed columns) and P·V takes its A operand from tensor memory: no shared-memory
//     round trip, no proxy fence. MMAs of one CTA run in issue order, so Q·K' of the next key
//     tile, issued after P·V, cannot overwrite probabilities that are still being read.
// Tensor memory: S_A | S_B (128 columns each) | O_A | O_B (D columns each).
// Shared memory: Q_A, Q_B, a K ring and a V ring, one output staging tile.
template <int D> struct Att2Cfg {
  static constexpr int Q_BYTES = BQ * D * 2; // one query tile
  static constexpr int K_BYTES = BKV * D * 2;
  static constexpr int V_BYTES = BKV * D * 2;
  static constexpr int KS = D == 128 ? 2 : 4; // stages of the K ring
  static constexpr int VS = D == 128 ? 2 : 4; // stages of the V ring
  static constexpr int STG_BYTES = BQ * D * 2; // output staging, shared by A and B in turn
  static constexpr int SMEM_BYTES = 2 * Q_BYTES + KS * K_BYTES + VS * V_BYTES + STG_BYTES + 1024;
  static constexpr int TMEM_COLS = 512;
};

// MIRROR: the second copy of the output (AttParams::mirror) is compiled in; a separate
// instantiation so that the plain kernel keeps its register allocation.
template <int D, bool LITERAL, bool MIRROR>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attention2_tcgen05_kernel(const __grid_constant__ CUtensorMap tmQ,
                          const __grid_constant__ CUtensorMap tmK,
                          const __grid_constant__ CUtensorMap tmV,
                          const __grid_constant__ CUtensorMap tmO, AttParams prm, int *status) {
  using Cfg = Att2Cfg<D>;
  constexpr int KS = Cfg::KS, VS = Cfg::VS;
  constexpr int DB = D / 64;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t *smem = smem_raw;
  if (smem_u32(smem_raw) & 1023u) {
    if (threadIdx.x == 0)
      atomicCAS(status, 0, MU_DEV_BAD_INDEX);
    return;
  }
  uint8_t *sQ = smem;                         // [2][Q_BYTES]
  uint8_t *sK = sQ + 2 * Cfg::Q_BYTES;        // [KS][K_BYTES]
  uint8_t *sV = sK + KS * Cfg::K_BYTES;       // [VS][V_BYTES]
  uint8_t *sStg = sV + VS * Cfg::V_BYTES;     // [STG_BYTES]
  uint64_t *bars = reinterpret_cast<uint64_t *>(sStg + Cfg::STG_BYTES);
  uint64_t *q_full = bars;            // [2]
  uint64_t *q_empty = q_full + 2;     // [2]
  uint64_t *k_full = q_empty + 2;     // [KS]
  uint64_t *k_empty = k_full + KS;    // [KS]
  uint64_t *v_full = k_empty + KS;    // [VS]
  uint64_t *v_empty = v_full + VS;    // [VS]
  uint64_t *s_full = v_empty + VS;    // [2] scores of A / B complete (and every MMA before them)
  uint64_t *p_full = s_full + 2;      // [2] probabilities of A / B are in tensor memory
  uint64_t *o_full = p_full + 2;      // [2] last P·V of the work has completed
  uint64_t *o_free = o_full + 2;      // [2] the softmax warps have read O of the work
  uint64_t *stg_done = o_free + 2;    // [1] an output tile has left the staging buffer
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(stg_done + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_cta = static_cast<int>(gridDim.x);
  const int n_pairs = (prm.n_qtiles + 1) / 2;
  const int nkv = (prm.T + BKV - 1) / BKV;

  // A work = (head, pair of query tiles 2*pr, 2*pr+1). Same deal as above: heads in chunks that
  // fit L2, pairs by falling size, serpentine over the CTAs, rotated from chunk to chunk.
  struct Work {
    int bh, qa, nk_a, nk_b; // first row of tile A, key tiles of A and of B (0: no tile B)
  };
  struct WorkIter {
    int chunk, pass;
  };
  auto next_work = [&](WorkIter &it, Work &wk) -> bool {
    for (;;) {
      const int h0 = it.chunk * prm.chunk_heads;
      if (h0 >= prm.BH)
        return false;
      const int hb = min(prm.chunk_heads, prm.BH - h0);
      const long long n_works = 1ll * hb * n_pairs;
      if (1ll * it.pass * n_cta >= n_works) {
        ++it.chunk, it.pass = 0;
        continue;
      }
      const int c = static_cast<int>((blockIdx.x + 1ll * it.chunk * prm.chunk_rot) % n_cta);
      const int slot = (it.pass & 1) ? n_cta - 1 - c : c;
      const long long p = 1ll * it.pass * n_cta + slot;
      ++it.pass;
      if (p >= n_works)
        continue;
      const int pr = n_pairs - 1 - static_cast<int>(p / hb);
      wk.bh = h0 + static_cast<int>(p % hb);
      wk.qa = 2 * pr * BQ;
      const bool has_b = 2 * pr + 1 < prm.n_qtiles;
      wk.nk_a = prm.causal ? min(nkv, 2 * pr + 1) : nkv;
      wk.nk_b = has_b ? (prm.causal ? min(nkv, 2 * pr + 2) : nkv) : 0;
      return true;
    }
  };

  if (threadIdx.x == 0) {
    for (int x = 0; x < 2; ++x) {
      mbar_init(&q_full[x], 1);
      mbar_init(&q_empty[x], 1);
      mbar_init(&s_full[x], 1);
      mbar_init(&p_full[x], 4);
      mbar_init(&o_full[x], 1);
      mbar_init(&o_free[x], 4);
    }
    for (int s = 0; s < KS; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
    }
    for (int s = 0; s < VS; ++s) {
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    mbar_init(stg_done, 4);
    fence_barrier_init();
    prefetch_tmap(&tmQ);
    prefetch_tmap(&tmK);
    prefetch_tmap(&tmV);
    prefetch_tmap(&tmO);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base, tmem_O = tmem_base + 256;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      bool ok = true;
      uint32_t kt = 0, vt = 0;     // K / V tiles issued so far
      uint32_t wq[2] = {0, 0};     // works that had a tile A / B so far
      WorkIter wit = {0, 0};
      for (Work wk; ok && next_work(wit, wk);) {
        for (int x = 0; x < 2 && ok; ++x) {
          if (x == 1 && wk.nk_b == 0)
            break;
          // Q_x is single-buffered: the last Q·K' of the previous work must have read it
          if (!mbar_wait(&q_empty[x], (wq[x] & 1) ^ 1)) {
            atomicCAS(status, 0, MU_DEV_TIMEOUT_PRODUCER);
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&q_full[x], Cfg::Q_BYTES);
#pragma unroll
          for (int db = 0; db < DB; ++db)
            tma_load_3d(sQ + x * Cfg::Q_BYTES + db * (BQ * 128), &tmQ, &q_full[x], db * 64,
                        wk.qa + x * BQ, wk.bh);
          ++wq[x];
        }
        const int nk = max(wk.nk_a, wk.nk_b);
        for (int j = 0; j < nk && ok; ++j) {
          const int k0 = j * BKV;
          {
            const int stage = kt % KS;
            if (!mbar_wait(&k_empty[stage], ((kt / KS) & 1) ^ 1)) {
              atomicCAS(status, 0, MU_DEV_TIMEOUT_PRODUCER);
              ok = false;
              break;
            }
            uint8_t *dst = sK + stage * Cfg::K_BYTES;
            mbar_arrive_expect_tx(&k_full[stage], Cfg::K_BYTES);
            if (LITERAL) {
#pragma unroll
              for (int db = 0; db < DB; ++db)
#pragma unroll
                for (int nb = 0; nb < 2; ++nb)
                  tma_load_3d(dst + (db * 2 + nb) * 8192, &tmK, &k_full[stage],
                              wk.bh * prm.T + k0 + nb * 64, db * 64, 0);
            } else {
#pragma unroll
              for (int db = 0; db < DB; ++db)
                tma_load_3d(dst + db * (BKV * 128), &tmK, &k_full[stage], db * 64, k0, wk.bh);
            }
            ++kt;
          }
          {
            const int stage = vt % VS;
            if (!mbar_wait(&v_empty[stage], ((vt / VS) & 1) ^ 1)) {
              atomicCAS(status, 0, MU_DEV_TIMEOUT_PRODUCER);
              ok = false;
              break;
            }
            uint8_t *dst = sV + stage * Cfg::V_BYTES;
            mbar_arrive_expect_tx(&v_full[stage], Cfg::V_BYTES);
#pragma unroll
            for (int kb = 0; kb < 2; ++kb)
#pragma unroll
              for (int db = 0; db < DB; ++db)
                tma_load_3d(dst + (kb * DB + db) * 8192, &tmV, &v_full[stage], db * 64, k0 + kb * 64,
                            wk.bh);
            ++vt;
          }
        }
      }
      if (!ok)
        for (int i = 0; i < 64; ++i)
          __nanosleep(1000);
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc(1u, 0u, LITERAL ? 1u : 0u, BQ, BKV);
      constexpr uint32_t idesc_pv = make_idesc(1u, 0u, 1u, BQ, D);
      bool ok = true;
      uint32_t kq = 0, vq = 0;      // K / V tiles consumed so far
      uint32_t wq[2] = {0, 0};      // works with a tile A / B so far
      uint32_t pt[2] = {0, 0};      // probability tiles consumed so far, per query tile
      auto fail = [&]() {
        atomicCAS(status, 0, MU_DEV_TIMEOUT_MMA);
        ok = false;
      };
      // Operand descriptors are built once; a k-step only adds a constant to the 14-bit start
      // address field (units of 16 bytes; shared memory is far too small for a carry out of it).
      uint64_t q_desc[2], k_desc[KS], v_desc[VS];
#pragma unroll
      for (int x = 0; x < 2; ++x)
        q_desc[x] = make_smem_desc(smem_u32(sQ + x * Cfg::Q_BYTES), 16, 1024);
#pragma unroll
      for (int s = 0; s < KS; ++s)
        k_desc[s] = LITERAL ? make_smem_desc(smem_u32(sK + s * Cfg::K_BYTES), 8192, 1024)
                            : make_smem_desc(smem_u32(sK + s * Cfg::K_BYTES), 16, 1024);
#pragma unroll
      for (int s = 0; s < VS; ++s)
        v_desc[s] = make_smem_desc(smem_u32(sV + s * Cfg::V_BYTES), 8192, 1024);
      auto pick = [](const uint64_t *d, int n, int i) { // d[i] without indexing local memory
        uint64_t r = d[0];
#pragma unroll
        for (int s = 1; s < n; ++s)
          r = (i == s) ? d[s] : r;
        return r;
      };
      // S_x = Q_x · K'(stage)
      auto issue_qk = [&](int x, int stage) {
        const uint64_t qd = x ? q_desc[1] : q_desc[0];
        const uint64_t kd = pick(k_desc, KS, stage);
        const uint32_t d_addr = tmem_S + x * BKV;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint64_t ad = qd + static_cast<uint64_t>(((k / 4) * (BQ * 128) + (k % 4) * 32) >> 4);
          const uint64_t bd = kd + static_cast<uint64_t>(
                                       (LITERAL ? (k / 4) * (2 * 8192) + (k % 4) * 2048
                                                : (k / 4) * (BKV * 128) + (k % 4) * 32) >> 4);
          umma_f16(d_addr, ad, bd, idesc_qk, k != 0 ? 1u : 0u);
        }
        umma_commit(&s_full[x]);
      };
      // O_x (+)= P_x · V(stage), P_x in tensor memory over the first 64 columns of S_x
      auto issue_pv = [&](int x, int stage, bool accumulate) {
        const uint64_t vd = pick(v_desc, VS, stage);
        const uint32_t d_addr = tmem_O + x * D, a_addr = tmem_S + x * BKV;
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k) {
          const uint64_t bd = vd + static_cast<uint64_t>(((k / 4) * (DB * 8192) + (k % 4) * 2048) >> 4);
          umma_f16_ts(d_addr, a_addr + k * 8, bd, idesc_pv, (accumulate || k != 0) ? 1u : 0u);
        }
      };
      WorkIter wit = {0, 0};
      for (Work wk; ok && next_work(wit, wk);) {
        const int nk_x[2] = {wk.nk_a, wk.nk_b};
        const int nk = max(wk.nk_a, wk.nk_b);
        for (int x = 0; x < 2 && ok; ++x)
          if (nk_x[x] > 0 && !mbar_wait(&q_full[x], wq[x] & 1))
            fail();
        if (!ok)
          break;
        // first key tile: both score tiles
        if (!mbar_wait(&k_full[kq % KS], (kq / KS) & 1)) {
          fail();
          break;
        }
        tc_fence_after();
        for (int x = 0; x < 2; ++x)
          if (nk_x[x] > 0) {
            issue_qk(x, kq % KS);
            if (nk_x[x] == 1)
              umma_commit(&q_empty[x]);
          }
        umma_commit(&k_empty[kq % KS]);
        ++kq;
        for (int j = 0; j < nk && ok; ++j) {
          const int vstage = vq % VS;
          if (!mbar_wait(&v_full[vstage], (vq / VS) & 1)) {
            fail();
            break;
          }
          bool k_ready = false; // K of tile j+1 has been waited for
          for (int x = 0; x < 2 && ok; ++x) {
            if (j >= nk_x[x])
              continue;
            // probabilities of (x, j); the first P·V of a work overwrites O_x, which the
            // softmax warps must have read (previous work)
            if (!mbar_wait(&p_full[x], pt[x] & 1) ||
                (j == 0 && !mbar_wait(&o_free[x], (wq[x] & 1) ^ 1))) {
              fail();
              break;
            }
            ++pt[x];
            tc_fence_after();
            issue_pv(x, vstage, j > 0);
            if (j == nk_x[x] - 1)
              umma_commit(&o_full[x]);
            if (j + 1 < nk_x[x]) {
              if (!k_ready) {
                if (!mbar_wait(&k_full[kq % KS], (kq / KS) & 1)) {
                  fail();
                  break;
                }
                tc_fence_after();
                k_ready = true;
              }
              issue_qk(x, kq % KS);
              if (j + 1 == nk_x[x] - 1)
                umma_commit(&q_empty[x]);
            }
          }
          if (!ok)
            break;
          umma_commit(&v_empty[vstage]);
          ++vq;
          if (j + 1 < nk) {
            umma_commit(&k_empty[kq % KS]);
            ++kq;
          }
        }
        for (int x = 0; x < 2; ++x)
          if (nk_x[x] > 0)
            ++wq[x];
      }
    }
    __syncwarp();
  } else {
    // ---------------- softmax and output: warps 2-5 tile A, warps 6-9 tile B ----------------
    const int x = (warp - 2) >> 2;     // which query tile of the pair
    const int q = warp & 3;            // TMEM lane quarter this warp may access
    const int row = q * 32 + lane;     // row inside the query tile = TMEM lane
    const uint32_t lane_sel = static_cast<uint32_t>(q * 32) << 16;
    const uint32_t s_addr = tmem_S + lane_sel + x * BKV;
    const uint32_t o_addr = tmem_O + lane_sel + x * D;
    const float scale_b = bf16_round(prm.scale);
    const uint32_t scale2 = (__float_as_uint(scale_b) >> 16) * 0x00010001u;
    constexpr float L2E = 1.4426950408889634f;
    bool ok = true;
    uint32_t st = 0, wx = 0; // score tiles / works of this query tile so far
    uint32_t n_epi = 0;      // output tiles that went through the staging buffer before this one

    WorkIter wit = {0, 0};
    for (Work wk; ok && next_work(wit, wk);) {
      const int nk = x == 0 ? wk.nk_a : wk.nk_b;
      // the staging buffer is used in the order A, B of each work
      const uint32_t my_epi = n_epi + (x == 1 ? 1u : 0u);
      n_epi += wk.nk_b > 0 ? 2u : 1u;
      if (nk == 0)
        continue;
      const int q0 = wk.qa + x * BQ;
      const int qrow = q0 + row;
      float m_ref = -INFINITY, l_run = 0.f;
      for (int j = 0; j < nk && ok; ++j, ++st) {
        if (!mbar_wait(&s_full[x], st & 1)) {
          atomicCAS(status, 0, MU_DEV_TIMEOUT_EPILOGUE);
          ok = false;
          break;
        }
        tc_fence_after();
        const int k0 = j * BKV;
        int lim = prm.T - k0; // keys this row may see inside the tile: [0, lim)
        if (prm.causal)
          lim = min(lim, qrow - k0 + 1);
        const bool need_mask = (k0 + BKV > prm.T) || (prm.causal && k0 + BKV > q0); // warp-uniform
        // pass 1: first rounding (fp32 accumulator -> bf16 pairs kept in registers), mask, row maximum
        uint32_t sp[BKV / 2];
        uint32_t mxa[4] = {0xFF80FF80u, 0xFF80FF80u, 0xFF80FF80u, 0xFF80FF80u};
        // Two copies of the loop: only the tiles on the diagonal (and a ragged last tile) pay
        // for the per-column comparisons.
        auto pass1 = [&](auto masked) {
          constexpr bool MASKED = decltype(masked)::value;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t r[2][32];
            tmem_ld_32x32(s_addr + h * 64, r[0]);
            tmem_ld_32x32(s_addr + h * 64 + 32, r[1]);
            tmem_ld_wait();
#pragma unroll
            for (int c = 0; c < 2; ++c)
#pragma unroll
              for (int k = 0; k < 32; k += 2) {
                uint32_t u = pack_bf16x2(__uint_as_float(r[c][k]), __uint_as_float(r[c][k + 1]));
                if constexpr (MASKED) {
                  const int col = h * 64 + c * 32 + k;
                  if (col >= lim)
                    u = (u & 0xFFFF0000u) | 0x0000FF80u;
                  if (col + 1 >= lim)
                    u = (u & 0x0000FFFFu) | 0xFF800000u;
                }
                sp[h * 32 + c * 16 + k / 2] = u;
                mxa[(k >> 1) & 3] = bf16x2_max(mxa[(k >> 1) & 3], u);
              }
          }
        };
        if (need_mask)
          pass1(std::true_type{});
        else
          pass1(std::false_type{});
        const uint32_t mx2 = bf16x2_max(bf16x2_max(mxa[0], mxa[1]), bf16x2_max(mxa[2], mxa[3]));
        const float raw_mx = fmaxf(bf16_lo(mx2), bf16_hi(mx2));
        const float mine = bf16_round(raw_mx * scale_b); // exactly a bf16 value (or -inf)
        const float mx = fmaxf(m_ref, mine);
        const float m_new = (mx == -INFINITY) ? 0.f : mx; // rows past the end of the sequence
        if (j == 0) {
          m_ref = m_new;
        } else {
          // m_ref follows the running maximum only when that has moved by more than 2^8, so O in
          // tensor memory almost never needs rescaling. s_full of this tile was committed after
          // the previous P·V of this query tile, so O is at rest here.
          const bool grow = (m_new - m_ref) * L2E > 8.0f;
          if (__any_sync(0xffffffffu, grow)) {
            const float a = grow ? ex2_approx((m_ref - m_new) * L2E) : 1.0f;
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
              uint32_t r[32];
              tmem_ld_32x32(o_addr + c * 32, r);
              tmem_ld_wait();
#pragma unroll
              for (int k = 0; k < 32; ++k)
                r[k] = __float_as_uint(__uint_as_float(r[k]) * a);
              tmem_st_32x32(o_addr + c * 32, r);
            }
            tmem_st_wait();
            l_run *= a;
            if (grow)
              m_ref = m_new;
          }
        }
        const float mL = m_ref * L2E;
        // pass 2: second rounding (times the bf16 scale), probabilities -> bf16 pairs -> tensor
        // memory over the first 64 columns of the score tile. Masked columns hold -inf: exp2 gives 0.
        // the exponent arguments and the row sum run two columns per instruction (packed fp32)
        const uint64_t l2e2 = f32x2_pack(L2E, L2E), nml2 = f32x2_pack(-mL, -mL);
        uint64_t sum2[2] = {f32x2_pack(0.f, 0.f), f32x2_pack(0.f, 0.f)};
#pragma unroll
        for (int c = 0; c < BKV / 32; ++c) {
          uint32_t pk[16];
#pragma unroll
          for (int k = 0; k < 16; ++k) {
            const uint32_t u = bf16x2_mul(sp[c * 16 + k], scale2);
            float x0, x1;
            f32x2_unpack(f32x2_fma(f32x2_pack(bf16_lo(u), bf16_hi(u)), l2e2, nml2), x0, x1);
            const float p0 = ex2_approx(x0), p1 = ex2_approx(x1);
            sum2[k & 1] = f32x2_add(sum2[k & 1], f32x2_pack(p0, p1));
            pk[k] = pack_bf16x2(p0, p1);
          }
          tmem_st_32x16(s_addr + c * 16, pk);
        }
        float sum0, sum1;
        {
          float a0, a1, b0, b1;
          f32x2_unpack(sum2[0], a0, a1);
          f32x2_unpack(sum2[1], b0, b1);
          sum0 = a0 + b0, sum1 = a1 + b1;
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0)
          mbar_arrive(&p_full[x]);
        l_run += sum0 + sum1;
      }
      // ---- output: O / l -> bf16 -> staging tile -> TMA store (token-major, heads merged) ----
      if (ok && !mbar_wait(&o_full[x], wx & 1)) {
        atomicCAS(status, 0, MU_DEV_TIMEOUT_EPILOGUE);
        ok = false;
      }
      // the tile staged before this one must have left the buffer
      if (ok && my_epi > 0 && !mbar_wait(stg_done, (my_epi - 1) & 1)) {
        atomicCAS(status, 0, MU_DEV_TIMEOUT_EPILOGUE);
        ok = false;
      }
      if (ok) {
        tc_fence_after();
        const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
        uint8_t *orow = sStg + row * 128;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(o_addr + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int gc = c * 4 + i; // 16-byte chunk of the row
            const int box = gc >> 3, cc = gc & 7;
            uint32_t ow[4];
#pragma unroll
            for (int k = 0; k < 4; ++k)
              ow[k] = pack_bf16x2(__uint_as_float(r[i * 8 + 2 * k]) * inv,
                                  __uint_as_float(r[i * 8 + 2 * k + 1]) * inv);
            *reinterpret_cast<uint4 *>(orow + box * (BQ * 128) + ((cc ^ (lane & 7)) << 4)) =
                make_uint4(ow[0], ow[1], ow[2], ow[3]);
          }
        }
        tc_fence_before();
        fence_proxy_async();
        __syncwarp();
        const int bb = wk.bh / prm.H, hh = wk.bh % prm.H;
        if (lane == 0) {
          mbar_arrive(&o_free[x]); // O_x may be overwritten by the next work
          if (q0 + q * 32 < prm.T) {
#pragma unroll
            for (int db = 0; db < DB; ++db)
              tma_store_5d(&tmO, sStg + db * (BQ * 128) + q * 32 * 128, db * 64, hh, q0 + q * 32, bb, 0);
            bulk_commit();
          }
        }
        if (MIRROR && prm.mirror) {
          // second copy of this warp's 32 rows, read back from the staging tile: eight lanes
          // cover one 128-byte row segment, a warp instruction four of them
#pragma unroll
          for (int db = 0; db < DB; ++db)
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int idx = i * 32 + lane, r = idx >> 3, cc = idx & 7;
              const int t = q0 + q * 32 + r;
              const uint4 val = *reinterpret_cast<const uint4 *>(sStg + db * (BQ * 128) + (q * 32 + r) * 128 +
                                                                 ((cc ^ (r & 7)) << 4));
              if (t < prm.T)
                *reinterpret_cast<uint4 *>(prm.mirror + (1ll * bb * prm.T + t) * prm.out_ld + hh * D +
                                           db * 64 + cc * 8) = val;
            }
        }
        __syncwarp();
        if (lane == 0) {
          bulk_wait_read<0>();
          mbar_arrive(stg_done);
        }
        __syncwarp();
      }
      ++wx;
    }
    if (lane == 0)
      bulk_wait<0>(); // every store of this warp has completed before the CTA exits
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1)
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn att_encode_fn() {
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

static bool att_map(CUtensorMap *map, const void *base, int rank, const unsigned long long *d,
                    const unsigned long long *st, const unsigned *bx) {
  EncodeTiledFn fn = att_encode_fn();
  if (!fn)
    return false;
  cuuint64_t dims[5], strides[4];
  cuuint32_t box[5], estr[5] = {1, 1, 1, 1, 1};
  for (int i = 0; i < rank; ++i)
    dims[i] = d[i], box[i] = bx[i];
  for (int i = 0; i + 1 < rank; ++i)
    strides[i] = st[i] * 2ull;
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void *>(base), dims, strides,
            box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// 0: the two-query-tile kernel (default); 1: the one-tile kernel above. Set through
// mu_debug_attention_variant for A/B timing; both give results within the same tolerance.
static int g_attention_variant = 0;
void set_attention_variant(int v) { g_attention_variant = v; }

// Returns 0 ok, 1 shape/alignment outside this kernel's envelope, 2 launch failure.
// out_ld: row stride of the [B*T, H*D] output in elements (0 = dense); mirror: optional second
// destination with the same layout (two-query-tile kernel only).
int launch_attention_tcgen05_ex(const void *q, const void *k, const void *v, void *out, long long out_ld,
                                void *mirror, int B, int H, int T, int D, int causal, int literal,
                                int *status, cudaStream_t stream) {
  auto al = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  if ((D != 64 && D != 128) || T <= 0 || B <= 0 || H <= 0)
    return 1;
  if (!al(q) || !al(k) || !al(v) || !al(out) || !al(mirror))
    return 1;
  if (out_ld == 0)
    out_ld = 1ll * H * D;
  if (out_ld < 1ll * H * D || (out_ld % 8))
    return 1;
  if (mirror && g_attention_variant == 1)
    return 1;
  if (literal && (T % 8))
    return 1; // column offset bh*T must stay 16-byte aligned
  const unsigned long long BH = 1ull * B * H, uT = T, uD = D, Ntot = BH * uT;
  if (Ntot > 0x7fffffffull)
    return 1;
  CUtensorMap tmQ, tmK, tmV, tmO;
  {
    const unsigned long long d[3] = {uD, uT, BH}, st[2] = {uD, uT * uD};
    const unsigned bq[3] = {64, BQ, 1}, bv[3] = {64, 64, 1};
    if (!att_map(&tmQ, q, 3, d, st, bq) || !att_map(&tmV, v, 3, d, st, bv))
      return 2;
    if (!literal) {
      const unsigned bk[3] = {64, BKV, 1};
      if (!att_map(&tmK, k, 3, d, st, bk))
        return 2;
    }
  }
  if (literal) {
    const unsigned long long d[3] = {Ntot, uD, 1}, st[2] = {Ntot, Ntot * uD};
    const unsigned bk[3] = {64, 64, 1};
    if (!att_map(&tmK, k, 3, d, st, bk))
      return 2;
  }
  {
    // out[b][t][h][d], dimensions by ascending stride: d, h, t, b
    const unsigned long long d[5] = {uD, static_cast<unsigned long long>(H), uT,
                                     static_cast<unsigned long long>(B), 1};
    const unsigned long long ld = static_cast<unsigned long long>(out_ld);
    const unsigned long long st[4] = {uD, ld, uT * ld, uT * ld * B};
    const unsigned bx[5] = {64, 1, 32, 1, 1};
    if (!att_map(&tmO, out, 5, d, st, bx))
      return 2;
  }
  AttParams prm;
  prm.T = T, prm.H = H, prm.BH = static_cast<int>(BH), prm.causal = causal;
  prm.scale = 1.0f / sqrtf(static_cast<float>(D));
  prm.n_qtiles = (T + BQ - 1) / BQ;
  prm.mirror = static_cast<__nv_bfloat16 *>(mirror), prm.out_ld = out_ld;
  {
    // K and V of one head are 4*T*D bytes; a chunk of heads is kept to about 64 MB, half of L2
    const unsigned long long per_head = 4ull * uT * uD;
    unsigned long long g = (64ull << 20) / per_head;
    prm.chunk_heads = static_cast<int>(g < 1 ? 1 : (g > BH ? BH : g));
    prm.chunk_rot = 53;
  }
  // one persistent CTA per SM (the kernel's shared memory allows no more), fewer for small jobs
  int dev = 0, num_sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || num_sms <= 0)
    return 2;
  const bool two_tiles = g_attention_variant != 1;
  const unsigned long long n_works = BH * (two_tiles ? (prm.n_qtiles + 1) / 2 : prm.n_qtiles);
  dim3 grid(static_cast<unsigned>(n_works < static_cast<unsigned long long>(num_sms) ? n_works : num_sms));

#define MU_ATT2_LAUNCH_M(D_, L_, M_)                                                             \
  do {                                                                                           \
    auto kern = attention2_tcgen05_kernel<D_, L_, M_>;                                           \
    static PerDeviceOnce attr_set;                                                               \
    if (attr_set.get() < 0) {                                                                    \
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,                \
                               Att2Cfg<D_>::SMEM_BYTES) != cudaSuccess)                          \
        return 2;                                                                                \
      attr_set.set(1);                                                                           \
    }                                                                                            \
    kern<<<grid, ATT_THREADS, Att2Cfg<D_>::SMEM_BYTES, stream>>>(tmQ, tmK, tmV, tmO, prm, status); \
  } while (0)
#define MU_ATT2_LAUNCH(D_, L_) MU_ATT2_LAUNCH_M(D_, L_, false)

  if (two_tiles && mirror) { // tensor-parallel path: true Q·K' only (literal addressing is not sharded)
    if (literal)
      return 1;
    if (D == 128)
      MU_ATT2_LAUNCH_M(128, false, true);
    else
      MU_ATT2_LAUNCH_M(64, false, true);
    return cudaGetLastError() == cudaSuccess ? 0 : 2;
  }
  if (two_tiles) {
    if (D == 128) {
      if (literal)
        MU_ATT2_LAUNCH(128, true);
      else
        MU_ATT2_LAUNCH(128, false);
    } else {
      if (literal)
        MU_ATT2_LAUNCH(64, true);
      else
        MU_ATT2_LAUNCH(64, false);
    }
#undef MU_ATT2_LAUNCH
#undef MU_ATT2_LAUNCH_M
    return cudaGetLastError() == cudaSuccess ? 0 : 2;
  }

#define MU_ATT_LAUNCH(D_, L_)                                                                    \
  do {                                                                                           \
    auto kern = attention_tcgen05_kernel<D_, L_>;                                                \
    static PerDeviceOnce attr_set;                                                               \
    if (attr_set.get() < 0) {                                                                             \
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,                \
                               AttCfg<D_>::SMEM_BYTES) != cudaSuccess)                           \
        return 2;                                                                                \
      attr_set.set(1);                                                                           \
    }                                                                                            \
    kern<<<grid, ATT_THREADS, AttCfg<D_>::SMEM_BYTES, stream>>>(tmQ, tmK, tmV, tmO, prm, status); \
  } while (0)

  if (D == 128) {
    if (literal)
      MU_ATT_LAUNCH(128, true);
    else
      MU_ATT_LAUNCH(128, false);
  } else {
    if (literal)
      MU_ATT_LAUNCH(64, true);
    else
      MU_ATT_LAUNCH(64, false);
  }
#undef MU_ATT_LAUNCH
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int launch_attention_tcgen05(const void *q, const void *k, const void *v, void *out, int B, int H,
                             int T, int D, int causal, int literal, int *status,
                             cudaStream_t stream) {
  return launch_attention_tcgen05_ex(q, k, v, out, 0, nullptr, B, H, T, D, causal, literal, status, stream);
}

} // namespace mu
