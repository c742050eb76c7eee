// Internal shared definitions for the kernels and their host launchers.
#pragma once
#include <atomic>
#include <cstdint>
#include <cuda_runtime.h>

namespace mu {

// dtype codes follow the MuNet DataType enum order (src/types.hpp:16).
enum DType : int { F32 = 0, F16 = 1, BF16 = 2, I32 = 3 };
enum Act : int { ACT_NONE = 0, ACT_RELU = 1, ACT_GELU = 2, ACT_SIGMOID = 3, ACT_TANH = 4 };

// Where an output element (batch, m, n) of a GEMM goes, and what happens to
// the accumulator on the way. The same addressing is used for the residual.
struct Epilogue {
  void *c = nullptr;              // output base
  const void *bias = nullptr;     // [N], same dtype as c, or null
  const void *residual = nullptr; // same addressing as c, or null
  float alpha = 1.0f;             // accumulator scale (1 = none)
  int act = ACT_NONE;
  int round_each = 1; // bf16 only: round to bf16 after every op like the reference's
                      // per-op typed loops (src/core/ops/common.hpp:46-85)
  long long ldc = 0;  // row stride in elements
  // batch b lives at (b / batch_div) * batch_hi + (b % batch_div) * batch_lo
  long long batch_hi = 0, batch_lo = 0;
  int batch_div = 1;
  // Head-split store (QKV projection → head-major [which][B·H][T][D]):
  // enabled when split_T > 0. Row m = b·T + t, column n = which·(H·D) + h·D + d.
  int split_T = 0, split_H = 0, split_D = 0;
  long long split_which_stride = 0;
  int vec_ok = 0; // host-verified: 16-byte aligned rows/pointers → 128-bit stores allowed
  int tma_out = 0; // tcgen05 kernel: output (and residual) go through staged TMA boxes
  int tma_mode = 0; // coordinate scheme of the output tensor map: 0 plain, 1 merge-heads, 2 split-heads
  // tcgen05 kernel, plain [M,N] output only: a second copy of every output tile is written here
  // with ordinary 16-byte stores (whole 128-byte rows). The pointer may map another GPU's
  // memory: this is how a tensor-parallel rank hands its partial sums to its peer while the
  // GEMM is still running. Same row stride as c.
  void *c_mirror = nullptr;
};

struct GemmShape {
  int M = 0, N = 0, K = 0, batch = 1;
  // tcgen05 kernel only: how the batch index reaches the operands' tensor maps.
  int a_batched = 1;        // third TMA coordinate of A = batch index (else 0)
  int b_batched = 1;        // third TMA coordinate of B = batch index (else 0)
  int b_col_per_batch = 0;  // added to B's N coordinate per batch (B = column slab of a wide matrix)
  // Tile order: panels of `panel_n` column tiles are swept over all row tiles before the next
  // panel starts, so a panel of B stays in L2 while A streams past it (0 = one panel).
  int panel_n = 0;
  // > 0: use this tile width (64, 128, 256) and CTA count (1, 2) instead of the automatic choice
  int force_bn = 0, force_ctas = 0;
  // tcgen05 kernel: 1 = B tiles are loaded with the L2 evict_last priority (B is re-used by every wave
  // of tiles while A, the residual and the output stream past it); 2 = that, and the residual loads and
  // output stores carry evict_first
  int b_evict_last = 0;
};

// Operand addressing in elements. A is row-major [M,K]. B is row-major [K,N]
// (b_kmajor = 0, how MuNet stores Linear weights) or row-major [N,K]
// (b_kmajor = 1, "B transposed"). A batch stride of 0 shares the operand.
struct GemmOperands {
  const void *a = nullptr;
  long long lda = 0, a_batch = 0;
  const void *b = nullptr;
  long long ldb = 0, b_batch = 0;
  int b_kmajor = 0;
  // B of batch i is the column slab [i*b_col_per_batch, ...) of one wide row-major
  // [K, ldb] matrix (b_kmajor = 0 only). Used for the reference's literal K addressing.
  long long b_col_per_batch = 0;
};

struct SimtArgs {
  const void *a, *b;
  long long lda, ldb, a_batch, b_batch;
  int b_kmajor;
  int is_bf16;
  GemmShape sh;
  Epilogue ep;
};

// float32 NCHW convolution, weight [oC,iC,k,k], square stride s / padding p.
struct ConvArgs {
  const float *x, *w, *bias;
  float *y;
  int B, iC, iH, iW, oC, oH, oW, k, s, p;
  int relu, pool; // pool: 0 none, 2 = MaxPool2d(2,2,0) fused after the activation
};

// Per-device, thread-safe "done once" flags for settings that CUDA keeps per device (a kernel's
// dynamic shared-memory limit, the number of co-resident clusters). Index = current device.
struct PerDeviceOnce {
  static constexpr int MAX_DEV = 64;
  std::atomic<int> v[MAX_DEV];
  PerDeviceOnce() {
    for (auto &x : v)
      x.store(-1);
  }
  // value cached for the current device, or -1
  int get() const {
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= MAX_DEV)
      return -1;
    return v[d].load(std::memory_order_acquire);
  }
  void set(int value) {
    int d = 0;
    if (cudaGetDevice(&d) == cudaSuccess && d >= 0 && d < MAX_DEV)
      v[d].store(value, std::memory_order_release);
  }
};

} // namespace mu
