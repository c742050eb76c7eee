// Large float32 convolutions on the tensor cores with the 3xTF32 GEMM of gemm_tf32x3.cu: as an
// implicit GEMM where the geometry allows it (stride 1, "same" padding, input channels a multiple
// of 32, rows that tile into 128-pixel boxes), through a materialised im2col matrix otherwise.
//
// BackendSpatialCapability::conv2d (src/core/backend.hpp:294-296; CPU loop
// src/backend/cpu_backend.hpp:768-796) is a direct NCHW convolution with float accumulation in
// (ic, kh, kw) order. conv.cu keeps that order bit for bit on the CUDA cores; from 2^31
// multiply-adds on, the layer runs here instead, with float32-class accuracy (inside the 1e-4
// tolerance of the float32 configs) rather than the reference's exact rounding:
//   1. im2col_split_kernel   x [B,iC,H,W] -> A_hi, A_lo [B*oH*oW, Kp], columns in the weight's
//                            own (ic, kh, kw) order, Kp = K rounded up to 4 (zero filled);
//   2. split of the weight   w [oC, K] -> B_hi, B_lo [oC, Kp] (already K-major: no transpose);
//   3. gemm_tf32x3_presplit  C [B*oH*oW, oC] = A * B' + bias, ReLU fused;
//   4. nhwc_to_nchw_kernel   back to the reference's NCHW layout, MaxPool2d(2,2,0) folded in.
// Implicit form: step 1 becomes nchw_to_nhwc_split_kernel (x -> NHWC hi / lo, 2x the input instead
// of 2 * k*k x), step 2 orders the weight [oC][kh][kw][iC], and the GEMM's producer fetches each
// k-block as a shifted 4-D box of the NHWC input (conv_tf32x3_implicit): for the 64->128 layer on
// 16x16 images that is 100 MB of scratch traffic where im2col wrote and re-read 604 MB.
#include "common.h"
#include "ptx.cuh"

namespace mu {

int gemm_tf32x3_presplit(const float *, const float *, const float *, const float *, float *, long long,
                         const float *, const float *, float, int, int, int, int, int *, int, cudaStream_t);
int conv_tf32x3_implicit(const float *, const float *, const float *, const float *, float *, const float *,
                         int, int, int, int, int, int, int, int, int *, int, cudaStream_t);
bool conv_tf32x3_implicit_ok(int, int, int, int, int, int, int);

__device__ __forceinline__ float conv_to_tf32(float x) {
  uint32_t u;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
  return __uint_as_float(u);
}

__global__ void __launch_bounds__(256)
im2col_split_kernel(const float *__restrict__ x, float *__restrict__ hi, float *__restrict__ lo, long long M,
                    int Kp, int K, int iC, int iH, int iW, int oH, int oW, int k, int s, int p) {
  const long long n = M * Kp;
  for (long long i = 1ll * blockIdx.x * blockDim.x + threadIdx.x; i < n; i += 1ll * gridDim.x * blockDim.x) {
    const int kk = static_cast<int>(i % Kp);
    const long long m = i / Kp;
    float v = 0.f;
    if (kk < K) {
      const int kw = kk % k, kh = (kk / k) % k, ic = kk / (k * k);
      const int ow = static_cast<int>(m % oW), oh = static_cast<int>((m / oW) % oH);
      const long long b = m / (1ll * oW * oH);
      const int ih = oh * s - p + kh, iw = ow * s - p + kw;
      if (ih >= 0 && ih < iH && iw >= 0 && iw < iW)
        v = __ldg(x + ((b * iC + ic) * iH + ih) * iW + iw);
    }
    const float h = conv_to_tf32(v);
    hi[i] = h;
    lo[i] = v - h;
  }
}

__global__ void __launch_bounds__(256)
weight_split_kernel(const float *__restrict__ w, float *__restrict__ hi, float *__restrict__ lo, int oC,
                    int K, int Kp) {
  const long long n = 1ll * oC * Kp;
  for (long long i = 1ll * blockIdx.x * blockDim.x + threadIdx.x; i < n; i += 1ll * gridDim.x * blockDim.x) {
    const int kk = static_cast<int>(i % Kp);
    const float v = kk < K ? w[(i / Kp) * K + kk] : 0.f;
    const float h = conv_to_tf32(v);
    hi[i] = h;
    lo[i] = v - h;
  }
}

// x [B, C, HW] -> hi, lo [B, HW, C] (NHWC), 32 x 32 tiles through shared memory.
__global__ void __launch_bounds__(256)
nchw_to_nhwc_split_kernel(const float *__restrict__ x, float *__restrict__ hi, float *__restrict__ lo, int C,
                          int HW) {
  __shared__ float tile[32][33];
  const int b = blockIdx.z, c0 = blockIdx.y * 32, s0 = blockIdx.x * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5; // 32 x 8
  for (int r = ty; r < 32; r += 8) {
    const int c = c0 + r, sp = s0 + tx;
    tile[r][tx] = (c < C && sp < HW) ? __ldg(x + (1ll * b * C + c) * HW + sp) : 0.f;
  }
  __syncthreads();
  for (int r = ty; r < 32; r += 8) {
    const int sp = s0 + r, c = c0 + tx;
    if (sp < HW && c < C) {
      const float v = tile[tx][r];
      const float h = conv_to_tf32(v);
      const long long at = (1ll * b * HW + sp) * C + c;
      hi[at] = h;
      lo[at] = v - h;
    }
  }
}

// w [oC][iC][k*k] -> hi, lo [oC][k*k][iC]
__global__ void __launch_bounds__(256)
weight_reorder_split_kernel(const float *__restrict__ w, float *__restrict__ hi, float *__restrict__ lo, int oC,
                            int iC, int kk) {
  const long long n = 1ll * oC * iC * kk;
  for (long long i = 1ll * blockIdx.x * blockDim.x + threadIdx.x; i < n; i += 1ll * gridDim.x * blockDim.x) {
    const int c = static_cast<int>(i % iC), tap = static_cast<int>((i / iC) % kk);
    const long long o = i / (1ll * iC * kk);
    const float v = w[(o * iC + c) * kk + tap];
    const float h = conv_to_tf32(v);
    hi[i] = h;
    lo[i] = v - h;
  }
}

// in [B, oH, oW, C] -> out [B, C, pH, pW]; pool == 2 takes the maximum of each 2x2 window
// (stride 2, no padding: nn::MaxPool2d(2,2,0) after a ReLU), pool == 0 copies. Tiles of
// 32 channels x 32 output positions go through shared memory so both sides are coalesced.
__global__ void __launch_bounds__(256)
nhwc_to_nchw_kernel(const float *__restrict__ in, float *__restrict__ out, int C, int oH, int oW, int pH,
                    int pW, int pool) {
  __shared__ float tile[32][33];
  const int b = blockIdx.z, c0 = blockIdx.y * 32, s0 = blockIdx.x * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5; // 32 x 8
  const int P = pH * pW;
  for (int r = ty; r < 32; r += 8) {
    const int sp = s0 + r, c = c0 + tx;
    float v = 0.f;
    if (sp < P && c < C) {
      const int ph = sp / pW, pw = sp % pW;
      if (pool == 2) {
        const float *q = in + ((1ll * b * oH + 2 * ph) * oW + 2 * pw) * C + c;
        v = fmaxf(fmaxf(q[0], q[C]), fmaxf(q[1ll * oW * C], q[1ll * oW * C + C]));
      } else {
        v = in[((1ll * b * oH + ph) * oW + pw) * C + c];
      }
    }
    tile[r][tx] = v;
  }
  __syncthreads();
  for (int r = ty; r < 32; r += 8) {
    const int c = c0 + r, sp = s0 + tx;
    if (c < C && sp < P)
      out[(1ll * b * C + c) * P + sp] = tile[tx][r];
  }
}

// bytes of scratch for one layer (256-byte aligned parts): A_hi, A_lo, B_hi, B_lo, C
size_t conv2d_tf32x3_scratch_bytes(const ConvArgs &a) {
  auto up = [](size_t v) { return (v + 255) & ~static_cast<size_t>(255); };
  const size_t M = static_cast<size_t>(a.B) * a.oH * a.oW, K = static_cast<size_t>(a.iC) * a.k * a.k;
  const size_t Kp = (K + 3) / 4 * 4;
  return 2 * up(M * Kp * 4) + 2 * up(static_cast<size_t>(a.oC) * Kp * 4) + up(M * a.oC * 4);
}

// Returns 0 ok, 1 outside the envelope (caller uses the direct kernel), 2 failure.
int launch_conv2d_tf32x3(const ConvArgs &a, void *scratch, int *status, int num_sms, cudaStream_t st) {
  if (a.oC % 4 || !scratch || (a.pool == 2 && !a.relu))
    return 1;
  auto up = [](size_t v) { return (v + 255) & ~static_cast<size_t>(255); };
  const long long M = 1ll * a.B * a.oH * a.oW;
  const int K = a.iC * a.k * a.k, Kp = (K + 3) / 4 * 4;
  if (M > 0x7fffffffll)
    return 1;
  const int pH = a.pool == 2 ? a.oH / 2 : a.oH, pW = a.pool == 2 ? a.oW / 2 : a.oW;
  if (pH <= 0 || pW <= 0 || a.B > 65535)
    return 1;
  uint8_t *s = static_cast<uint8_t *>(scratch);
  if (a.s == 1 && a.oH == a.iH && a.oW == a.iW &&
      conv_tf32x3_implicit_ok(a.B, a.iH, a.iW, a.iC, a.oC, a.k, a.p)) {
    // implicit GEMM: scratch = x_hi, x_lo (NHWC), w_hi, w_lo ([oC][k][k][iC]), C (NHWC); it fits in
    // what the im2col layout reserves (2 * M * iC <= 2 * M * Kp)
    const size_t xb = up(static_cast<size_t>(M) * a.iC * 4), wb = up(static_cast<size_t>(a.oC) * K * 4);
    float *xh = reinterpret_cast<float *>(s), *xl = reinterpret_cast<float *>(s + xb);
    float *wh = reinterpret_cast<float *>(s + 2 * xb), *wl = reinterpret_cast<float *>(s + 2 * xb + wb);
    float *cn = reinterpret_cast<float *>(s + 2 * xb + 2 * wb);
    const int HW = a.iH * a.iW;
    nchw_to_nhwc_split_kernel<<<dim3((HW + 31) / 32, (a.iC + 31) / 32, a.B), 256, 0, st>>>(a.x, xh, xl, a.iC, HW);
    weight_reorder_split_kernel<<<static_cast<unsigned>(num_sms > 0 ? num_sms * 4 : 256), 256, 0, st>>>(
        a.w, wh, wl, a.oC, a.iC, a.k * a.k);
    const int irc = conv_tf32x3_implicit(xh, xl, wh, wl, cn, a.bias, a.relu, a.B, a.iH, a.iW, a.iC, a.oC, a.k,
                                         a.p, status, num_sms, st);
    if (irc == 0) {
      dim3 grid((pH * pW + 31) / 32, (a.oC + 31) / 32, a.B);
      nhwc_to_nchw_kernel<<<grid, 256, 0, st>>>(cn, a.y, a.oC, a.oH, a.oW, pH, pW, a.pool);
      return cudaGetLastError() == cudaSuccess ? 0 : 2;
    }
    return irc == 1 ? 1 : 2;
  }
  float *ah = reinterpret_cast<float *>(s);
  float *al = reinterpret_cast<float *>(s + up(static_cast<size_t>(M) * Kp * 4));
  float *bh = reinterpret_cast<float *>(s + 2 * up(static_cast<size_t>(M) * Kp * 4));
  float *bl = bh + up(static_cast<size_t>(a.oC) * Kp * 4) / 4;
  float *cb = bl + up(static_cast<size_t>(a.oC) * Kp * 4) / 4;
  const unsigned eb = static_cast<unsigned>(num_sms > 0 ? num_sms * 16 : 1024);
  im2col_split_kernel<<<eb, 256, 0, st>>>(a.x, ah, al, M, Kp, K, a.iC, a.iH, a.iW, a.oH, a.oW, a.k, a.s, a.p);
  weight_split_kernel<<<eb, 256, 0, st>>>(a.w, bh, bl, a.oC, K, Kp);
  const int rc = gemm_tf32x3_presplit(ah, al, bh, bl, cb, a.oC, a.bias, nullptr, 1.0f, a.relu ? ACT_RELU : ACT_NONE,
                                      static_cast<int>(M), a.oC, Kp, status, num_sms, st);
  if (rc)
    return rc;
  dim3 grid((pH * pW + 31) / 32, (a.oC + 31) / 32, a.B);
  nhwc_to_nchw_kernel<<<grid, 256, 0, st>>>(cb, a.y, a.oC, a.oH, a.oW, pH, pW, a.pool);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

} // namespace mu
