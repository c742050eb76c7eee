// Pair arithmetic of the Linear epilogue chain  y = act(alpha*x + bias) + residual  with the
// reference's per-op bf16 rounding (every op of the typed fallback rounds its result:
// src/backend/cpu_backend.hpp typed paths; GELU = x*sigmoid(1.702x), src/nn/activations.hpp:31-38).
// Shared by the GEMM epilogue and the standalone elementwise kernel so both give the same bits.
#pragma once
#include "common.h"
#include "ptx.cuh"

namespace mu {

// The same chain on a PAIR of adjacent columns with the activation fixed at compile
// time (hot path). Rounding two values costs one packed convert plus two bit ops,
// which halves the load on the conversion (XU) pipe.
__device__ __forceinline__ void round2(float &a, float &b) {
  const uint32_t u = pack_bf16x2(a, b);
  a = bf16_lo(u);
  b = bf16_hi(u);
}
__device__ __forceinline__ float fast_sigmoid(float t) {
  return __fdividef(1.0f, 1.0f + __expf(-t));
}

// ROUND_IN = false when x0/x1 already are bf16 values (an elementwise pass over stored data).
template <int ACT, bool ROUND_IN = true>
__device__ __forceinline__ uint32_t epi_pair(float x0, float x1, float b0, float b1, float r0,
                                             float r1, float alpha, bool has_alpha, bool has_bias,
                                             bool has_res, bool rnd) {
  if (rnd) {
    if (ROUND_IN)
      round2(x0, x1);
    if (has_alpha) {
      x0 *= alpha, x1 *= alpha;
      round2(x0, x1);
    }
    if (has_bias) {
      x0 += b0, x1 += b1;
      round2(x0, x1);
    }
    if (ACT == ACT_RELU) {
      x0 = fmaxf(x0, 0.0f), x1 = fmaxf(x1, 0.0f);
    } else if (ACT == ACT_GELU) {
      float t0 = x0 * 1.703125f, t1 = x1 * 1.703125f; // bf16(1.702)
      round2(t0, t1);
      float s0 = fast_sigmoid(t0), s1 = fast_sigmoid(t1);
      round2(s0, s1);
      x0 *= s0, x1 *= s1;
      if (has_res)
        round2(x0, x1);
    } else if (ACT == ACT_SIGMOID) {
      x0 = fast_sigmoid(x0), x1 = fast_sigmoid(x1);
      if (has_res)
        round2(x0, x1);
    } else if (ACT == ACT_TANH) {
      float t0 = x0 * 2.0f, t1 = x1 * 2.0f;
      round2(t0, t1);
      float s0 = fast_sigmoid(t0), s1 = fast_sigmoid(t1);
      round2(s0, s1);
      x0 = s0 * 2.0f - 1.0f, x1 = s1 * 2.0f - 1.0f;
      if (has_res)
        round2(x0, x1);
    }
    if (has_res)
      x0 += r0, x1 += r1;
  } else {
    if (has_alpha)
      x0 *= alpha, x1 *= alpha;
    x0 += b0, x1 += b1;
    if (ACT == ACT_RELU) {
      x0 = fmaxf(x0, 0.0f), x1 = fmaxf(x1, 0.0f);
    } else if (ACT == ACT_GELU) {
      x0 *= fast_sigmoid(1.702f * x0), x1 *= fast_sigmoid(1.702f * x1);
    } else if (ACT == ACT_SIGMOID) {
      x0 = fast_sigmoid(x0), x1 = fast_sigmoid(x1);
    } else if (ACT == ACT_TANH) {
      x0 = 2.0f * fast_sigmoid(2.0f * x0) - 1.0f, x1 = 2.0f * fast_sigmoid(2.0f * x1) - 1.0f;
    }
    x0 += r0, x1 += r1;
  }
  return pack_bf16x2(x0, x1); // the final rounding to the stored bf16
}

} // namespace mu
