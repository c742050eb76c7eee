// float32 Conv2d (NCHW, weight [oC,iC,k,k], square stride/padding) with fused
// bias, ReLU and 2x2/stride-2 max-pool epilogue; standalone MaxPool2d and
// GlobalAvgPool2d.
//
// Reference: Backend::conv2d / max_pool2d (src/core/backend.hpp:294-300; CPU
// kernels src/backend/cpu_backend.hpp:768-796, 833-855) and nn::GlobalAvgPool2d
// (src/nn/pooling.hpp:8-26, a [B·C,HW]·[HW,1] matmul against the float 1/HW).
//
// Results are bit-identical to the reference CPU kernels: every output starts at
// its bias and adds separately rounded products in (ic, kh, kw) order — no fused
// multiply-add, no reassociation; padding contributes exact zeros. ReLU and max
// are exact, so Conv→ReLU→MaxPool fused here equals the three reference ops.
//
// Tiling: one block = one image x OC_T output channels x a TH x TW output tile;
// input patch (with halo) and the weight slice of IC_T input channels are staged
// in shared memory; a thread owns one output pixel and OC_T/(256/(TH*TW)) channels.
#include "common.h"
#include <cfloat>

namespace mu {

constexpr int CONV_THREADS = 256;
constexpr int OC_T = 32;
constexpr int IC_T = 8;


template <int TH, int TW>
__global__ void __launch_bounds__(CONV_THREADS) conv2d_kernel(ConvArgs a) {
  constexpr int NPIX = TH * TW;
  constexpr int GROUPS = CONV_THREADS / NPIX; // channel sub-groups per block
  constexpr int OC_PER = OC_T / GROUPS;
  extern __shared__ __align__(16) float sm[];
  const int PH = (TH - 1) * a.s + a.k, PW = (TW - 1) * a.s + a.k; // input patch
  float *s_in = sm;                       // [IC_T][PH][PW]
  // weights after the patch, on a 16-byte boundary: [IC_T][k*k][OC_T]
  float *s_w = sm + ((IC_T * PH * PW + 3) & ~3);
  const int tiles_w = (a.oW + TW - 1) / TW;
  const int tile_y = (blockIdx.x / tiles_w) * TH, tile_x = (blockIdx.x % tiles_w) * TW;
  const int oc0 = blockIdx.y * OC_T;
  const int b = blockIdx.z;
  const int pix = threadIdx.x % NPIX, grp = threadIdx.x / NPIX;
  const int py = pix / TW, px = pix % TW;
  const int oy = tile_y + py, ox = tile_x + px;
  const int kk = a.k * a.k;

  float acc[OC_PER];
#pragma unroll
  for (int i = 0; i < OC_PER; ++i) {
    const int oc = oc0 + grp * OC_PER + i;
    acc[i] = (a.bias && oc < a.oC) ? a.bias[oc] : 0.0f;
  }
  const int in_y0 = tile_y * a.s - a.p, in_x0 = tile_x * a.s - a.p;
  for (int ic0 = 0; ic0 < a.iC; ic0 += IC_T) {
    const int nic = min(IC_T, a.iC - ic0);
    __syncthreads();
    for (int e = threadIdx.x; e < nic * PH * PW; e += CONV_THREADS) {
      const int ic = e / (PH * PW), r = (e / PW) % PH, c = e % PW;
      const int iy = in_y0 + r, ix = in_x0 + c;
      float v = 0.0f;
      if (iy >= 0 && iy < a.iH && ix >= 0 && ix < a.iW)
        v = a.x[((1ll * b * a.iC + ic0 + ic) * a.iH + iy) * a.iW + ix];
      s_in[e] = v;
    }
    for (int e = threadIdx.x; e < nic * kk * OC_T; e += CONV_THREADS) {
      const int oc = e % OC_T, t = (e / OC_T) % kk, ic = e / (OC_T * kk);
      float v = 0.0f;
      if (oc0 + oc < a.oC)
        v = a.w[((1ll * (oc0 + oc) * a.iC + ic0 + ic)) * kk + t];
      s_w[e] = v;
    }
    __syncthreads();
    for (int ic = 0; ic < nic; ++ic) {
      for (int kh = 0; kh < a.k; ++kh) {
        for (int kw = 0; kw < a.k; ++kw) {
          const float xv = s_in[(ic * PH + py * a.s + kh) * PW + px * a.s + kw];
          const float4 *wp = reinterpret_cast<const float4 *>(
              s_w + (ic * kk + kh * a.k + kw) * OC_T + grp * OC_PER);
#pragma unroll
          for (int i = 0; i < OC_PER / 4; ++i) {
            const float4 w4 = wp[i]; // same address across the warp: one broadcast read
            acc[4 * i + 0] = __fadd_rn(acc[4 * i + 0], __fmul_rn(xv, w4.x));
            acc[4 * i + 1] = __fadd_rn(acc[4 * i + 1], __fmul_rn(xv, w4.y));
            acc[4 * i + 2] = __fadd_rn(acc[4 * i + 2], __fmul_rn(xv, w4.z));
            acc[4 * i + 3] = __fadd_rn(acc[4 * i + 3], __fmul_rn(xv, w4.w));
          }
        }
      }
    }
  }
  const bool in_range = oy < a.oH && ox < a.oW;
#pragma unroll
  for (int i = 0; i < OC_PER; ++i) {
    const int oc = oc0 + grp * OC_PER + i;
    float v = acc[i];
    if (a.relu)
      v = v > 0.0f ? v : 0.0f;
    if (a.pool == 2) {
      // MaxPool2d(2,2,0): the window's four pixels sit in lanes l, l^1, l^TW, l^TW^1.
      // Pixels outside the feature map must not win: the reference never reads them.
      float m = in_range ? v : -FLT_MAX;
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, TW));
      const int qy = oy >> 1, qx = ox >> 1, qH = a.oH >> 1, qW = a.oW >> 1;
      if (!(py & 1) && !(px & 1) && qy < qH && qx < qW && oc < a.oC)
        a.y[((1ll * b * a.oC + oc) * qH + qy) * qW + qx] = fmaxf(m, -1e9f);
    } else if (in_range && oc < a.oC) {
      a.y[((1ll * b * a.oC + oc) * a.oH + oy) * a.oW + ox] = v;
    }
  }
}

// MaxPool2d, any k/s/p: cpu_backend.hpp:833-855 (initial value -1e9f).
__global__ void max_pool2d_kernel(const float *__restrict__ x, float *__restrict__ y, long long total,
                                  int C, int iH, int iW, int oH, int oW, int k, int s, int p) {
  const long long idx = 1ll * blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total)
    return;
  const int ow = idx % oW, oh = (idx / oW) % oH;
  const long long bc = idx / (1ll * oW * oH);
  float m = -1e9f;
  for (int kh = 0; kh < k; ++kh)
    for (int kw = 0; kw < k; ++kw) {
      const int ih = oh * s - p + kh, iw = ow * s - p + kw;
      if (ih >= 0 && ih < iH && iw >= 0 && iw < iW)
        m = fmaxf(m, x[(bc * iH + ih) * iW + iw]);
    }
  y[idx] = m;
}

// GlobalAvgPool2d: out[b,c] = sum_i x[i] * (1/HW), float, ascending i, separately
// rounded multiply and add (the reference's matmul against a constant column).
__global__ void global_avg_pool_kernel(const float *__restrict__ x, float *__restrict__ y,
                                       long long rows, int HW) {
  const long long r = 1ll * blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows)
    return;
  const float scale = 1.0f / static_cast<float>(HW);
  const float *xr = x + r * HW;
  float s = 0.0f;
  for (int i = 0; i < HW; ++i)
    s = __fadd_rn(s, __fmul_rn(xr[i], scale));
  y[r] = s;
}

// Returns 0 ok, 1 unsupported arguments, 2 launch failure.
int launch_conv2d(const ConvArgs &a, cudaStream_t st) {
  if (a.B <= 0 || a.oC <= 0 || a.oH <= 0 || a.oW <= 0)
    return 0;
  if (a.k <= 0 || a.s <= 0 || a.p < 0)
    return 1;
  if (a.pool != 0 && a.pool != 2)
    return 1;
  const bool small = a.oH <= 8 && a.oW <= 8;
  const int TH = small ? 8 : 16, TW = small ? 8 : 16;
  const int PH = (TH - 1) * a.s + a.k, PW = (TW - 1) * a.s + a.k;
  const size_t smem = sizeof(float) * (((static_cast<size_t>(IC_T) * PH * PW + 3) & ~size_t(3)) +
                                       static_cast<size_t>(IC_T) * a.k * a.k * OC_T);
  if (smem > 200 * 1024)
    return 1;
  dim3 grid(((a.oH + TH - 1) / TH) * ((a.oW + TW - 1) / TW), (a.oC + OC_T - 1) / OC_T, a.B);
  if (grid.y > 65535 || grid.z > 65535)
    return 1;
  if (small) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(conv2d_kernel<8, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    conv2d_kernel<8, 8><<<grid, CONV_THREADS, smem, st>>>(a);
  } else {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(conv2d_kernel<16, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    conv2d_kernel<16, 16><<<grid, CONV_THREADS, smem, st>>>(a);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int launch_max_pool2d(const float *x, float *y, int B, int C, int iH, int iW, int k, int s, int p,
                      cudaStream_t st) {
  if (k <= 0 || s <= 0 || p < 0)
    return 1;
  const int oH = (iH + 2 * p - k) / s + 1, oW = (iW + 2 * p - k) / s + 1;
  const long long total = 1ll * B * C * oH * oW;
  if (total <= 0)
    return 0;
  max_pool2d_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, st>>>(x, y, total, C, iH, iW,
                                                                                oH, oW, k, s, p);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

int launch_global_avg_pool(const float *x, float *y, long long rows, int HW, cudaStream_t st) {
  if (rows <= 0)
    return 0;
  global_avg_pool_kernel<<<static_cast<unsigned>((rows + 127) / 128), 128, 0, st>>>(x, y, rows, HW);
  return cudaGetLastError() == cudaSuccess ? 0 : 2;
}

} // namespace mu
