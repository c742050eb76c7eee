// extern "C" entry points of the spatial ops (declared in include/munet_b200.h):
// BackendSpatialCapability::conv2d / max_pool2d (src/core/backend.hpp:294-300) and
// nn::GlobalAvgPool2d (src/nn/pooling.hpp:8-26). float32 only: the CNN config of
// the reference is float32 and its dispatch forces half-precision convolutions to
// the CPU (src/core/op_dispatch.cpp:424-426).
#include "../../include/munet_b200.h"
#include "common.h"

namespace mu {
int launch_conv2d(const ConvArgs &, cudaStream_t);
size_t conv2d_tf32x3_scratch_bytes(const ConvArgs &);
int launch_conv2d_tf32x3(const ConvArgs &, void *, int *, int, cudaStream_t);
int launch_max_pool2d(const float *, float *, int, int, int, int, int, int, int, cudaStream_t);
int launch_global_avg_pool(const float *, float *, long long, int, cudaStream_t);
} // namespace mu

extern "C" {

// Error text goes through the context of the other entry points.
int mu_set_error(mu_ctx *ctx, int code, const char *msg);
int *mu_ctx_status_ptr(mu_ctx *ctx);
int mu_ctx_simt_forced(const mu_ctx *ctx);
int mu_ctx_select_device(mu_ctx *ctx);

int mu_conv2d(mu_ctx *ctx, const void *x, const void *w, const void *bias, void *y, int B, int iC,
              int iH, int iW, int oC, int k, int stride, int pad, int relu, int pool, int dtype,
              void *stream) {
  if (!ctx)
    return MU_ERR_INVALID;
  if (dtype != MU_F32)
    return mu_set_error(ctx, MU_ERR_UNSUPPORTED, "conv2d: only float32 is implemented");
  if (B < 0 || iC <= 0 || iH <= 0 || iW <= 0 || oC <= 0 || k <= 0 || stride <= 0 || pad < 0)
    return mu_set_error(ctx, MU_ERR_INVALID, "conv2d: bad dimensions");
  if (pool != 0 && pool != 2)
    return mu_set_error(ctx, MU_ERR_INVALID, "conv2d: fused pool must be 0 or 2 (MaxPool2d(2,2,0))");
  const int oH = (iH + 2 * pad - k) / stride + 1, oW = (iW + 2 * pad - k) / stride + 1;
  if (oH <= 0 || oW <= 0)
    return mu_set_error(ctx, MU_ERR_INVALID, "conv2d: kernel larger than the padded input");
  if (B == 0)
    return MU_OK;
  if (!x || !w || !y)
    return mu_set_error(ctx, MU_ERR_INVALID, "conv2d: null pointer");
  mu::ConvArgs a;
  a.x = static_cast<const float *>(x), a.w = static_cast<const float *>(w);
  a.bias = static_cast<const float *>(bias), a.y = static_cast<float *>(y);
  a.B = B, a.iC = iC, a.iH = iH, a.iW = iW, a.oC = oC, a.oH = oH, a.oW = oW;
  a.k = k, a.s = stride, a.p = pad, a.relu = relu ? 1 : 0, a.pool = pool;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // From 2^31 multiply-adds on: im2col + 3xTF32 tensor-core GEMM (float32-class accuracy); below,
  // and whenever that path declines, the direct kernel with the reference's accumulation order.
  const double macs = 1.0 * B * oH * oW * oC * iC * k * k;
  if (macs >= 2147483648.0 && !mu_ctx_simt_forced(ctx) && mu_ctx_select_device(ctx) == MU_OK) {
    void *scratch = nullptr;
    if (cudaMallocAsync(&scratch, mu::conv2d_tf32x3_scratch_bytes(a), st) == cudaSuccess) {
      const int trc = mu::launch_conv2d_tf32x3(a, scratch, mu_ctx_status_ptr(ctx), mu_ctx_num_sms(ctx), st);
      cudaFreeAsync(scratch, st);
      if (trc == 0)
        return MU_OK;
      if (trc == 2)
        return mu_set_error(ctx, MU_ERR_CUDA, cudaGetErrorString(cudaGetLastError()));
    } else {
      cudaGetLastError();
    }
  }
  const int rc = mu::launch_conv2d(a, st);
  if (rc == 1)
    return mu_set_error(ctx, MU_ERR_UNSUPPORTED, "conv2d: shape outside the kernel's envelope");
  if (rc)
    return mu_set_error(ctx, MU_ERR_CUDA, cudaGetErrorString(cudaGetLastError()));
  return MU_OK;
}

int mu_max_pool2d(mu_ctx *ctx, const void *x, void *y, int B, int C, int H, int W, int k, int stride,
                  int pad, int dtype, void *stream) {
  if (!ctx)
    return MU_ERR_INVALID;
  if (dtype != MU_F32)
    return mu_set_error(ctx, MU_ERR_UNSUPPORTED, "max_pool2d: only float32 is implemented");
  if (B < 0 || C <= 0 || H <= 0 || W <= 0 || k <= 0 || stride <= 0 || pad < 0)
    return mu_set_error(ctx, MU_ERR_INVALID, "max_pool2d: bad dimensions");
  if (B == 0)
    return MU_OK;
  if (!x || !y)
    return mu_set_error(ctx, MU_ERR_INVALID, "max_pool2d: null pointer");
  const int rc = mu::launch_max_pool2d(static_cast<const float *>(x), static_cast<float *>(y), B, C, H,
                                       W, k, stride, pad, static_cast<cudaStream_t>(stream));
  return rc ? mu_set_error(ctx, MU_ERR_CUDA, cudaGetErrorString(cudaGetLastError())) : MU_OK;
}

int mu_global_avg_pool(mu_ctx *ctx, const void *x, void *y, int B, int C, int H, int W, int dtype,
                       void *stream) {
  if (!ctx)
    return MU_ERR_INVALID;
  if (dtype != MU_F32)
    return mu_set_error(ctx, MU_ERR_UNSUPPORTED, "global_avg_pool: only float32 is implemented");
  if (B < 0 || C <= 0 || H <= 0 || W <= 0)
    return mu_set_error(ctx, MU_ERR_INVALID, "GlobalAvgPool2d expects NCHW input");
  if (B == 0)
    return MU_OK;
  if (!x || !y)
    return mu_set_error(ctx, MU_ERR_INVALID, "global_avg_pool: null pointer");
  const int rc = mu::launch_global_avg_pool(static_cast<const float *>(x), static_cast<float *>(y),
                                            1ll * B * C, H * W, static_cast<cudaStream_t>(stream));
  return rc ? mu_set_error(ctx, MU_ERR_CUDA, cudaGetErrorString(cudaGetLastError())) : MU_OK;
}

} // extern "C"
