// Broadcasting binary elementwise ops (add, sub, mul, div) over up to 6 dims:
// BackendElementwiseCapability::add/sub/mul/div with a BroadcastInfo
// (src/core/backend.hpp:214-221; CPU kernels src/backend/cpu_backend.hpp:238-330,
// typed fallback src/core/ops/common.hpp:46-85). out[i] = a[off_a(i)] op b[off_b(i)],
// offsets from per-dimension element strides (0 = broadcast).
// float32: one correctly rounded float op, as the reference CPU kernels compute it.
// bfloat16: evaluated in fp32 and rounded once to bf16 (the reference evaluates in
// double and rounds double→float→bf16; products of two bf16 are exact in fp32).
#include "../../include/munet_b200.h"
#include "common.h"
#include "ptx.cuh"

namespace mu {

struct BinaryArgs {
  const void *a, *b;
  void *out;
  long long total;
  int ndim, op;
  int shape[6];
  long long sa[6], sb[6];
  int contiguous; // both operands dense with the output shape
};

__device__ __forceinline__ float apply_op(float x, float y, int op) {
  switch (op) {
  case 0: return __fadd_rn(x, y);
  case 1: return __fsub_rn(x, y);
  case 2: return __fmul_rn(x, y);
  default: return __fdiv_rn(x, y);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) binary_broadcast_kernel(BinaryArgs g) {
  const long long stride = 1ll * gridDim.x * blockDim.x;
  for (long long i = 1ll * blockIdx.x * blockDim.x + threadIdx.x; i < g.total; i += stride) {
    long long oa = i, ob = i;
    if (!g.contiguous) {
      oa = ob = 0;
      long long rem = i;
      for (int d = g.ndim - 1; d >= 0; --d) {
        const long long c = rem % g.shape[d];
        rem /= g.shape[d];
        oa += c * g.sa[d];
        ob += c * g.sb[d];
      }
    }
    if (sizeof(T) == 4) {
      const float *a = static_cast<const float *>(g.a), *b = static_cast<const float *>(g.b);
      static_cast<float *>(g.out)[i] = apply_op(a[oa], b[ob], g.op);
    } else {
      const __nv_bfloat16 *a = static_cast<const __nv_bfloat16 *>(g.a);
      const __nv_bfloat16 *b = static_cast<const __nv_bfloat16 *>(g.b);
      static_cast<__nv_bfloat16 *>(g.out)[i] =
          __float2bfloat16_rn(apply_op(__bfloat162float(a[oa]), __bfloat162float(b[ob]), g.op));
    }
  }
}

} // namespace mu

extern "C" {
int mu_set_error(mu_ctx *ctx, int code, const char *msg);
int mu_ctx_num_sms(const mu_ctx *ctx);

int mu_binary_broadcast(mu_ctx *ctx, int op, const void *a, const void *b, void *out, int ndim,
                        const int *out_shape, const long long *strides_a,
                        const long long *strides_b, int dtype, void *stream) {
  if (!ctx)
    return MU_ERR_INVALID;
  if (op < MU_OP_ADD || op > MU_OP_DIV)
    return mu_set_error(ctx, MU_ERR_INVALID, "binary: unknown op");
  if (dtype != MU_F32 && dtype != MU_BF16)
    return mu_set_error(ctx, MU_ERR_UNSUPPORTED, "binary: dtype not implemented (float32, bfloat16)");
  if (ndim < 0 || ndim > 6 || (ndim > 0 && (!out_shape || !strides_a || !strides_b)))
    return mu_set_error(ctx, MU_ERR_INVALID, "binary: 0..6 dimensions with shape and strides");
  mu::BinaryArgs g;
  g.a = a, g.b = b, g.out = out, g.ndim = ndim, g.op = op, g.total = 1;
  long long dense = 1;
  bool contiguous = true;
  for (int d = ndim - 1; d >= 0; --d) {
    if (out_shape[d] < 0)
      return mu_set_error(ctx, MU_ERR_INVALID, "binary: negative dimension");
    g.shape[d] = out_shape[d], g.sa[d] = strides_a[d], g.sb[d] = strides_b[d];
    if (out_shape[d] != 1 && (strides_a[d] != dense || strides_b[d] != dense))
      contiguous = false;
    dense *= out_shape[d];
    g.total *= out_shape[d];
  }
  g.contiguous = contiguous ? 1 : 0;
  if (g.total == 0)
    return MU_OK;
  if (!a || !b || !out)
    return mu_set_error(ctx, MU_ERR_INVALID, "binary: null pointer");
  long long blocks = (g.total + 255) / 256;
  const long long cap = 1ll * mu_ctx_num_sms(ctx) * 32;
  if (blocks > cap)
    blocks = cap;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == MU_F32)
    mu::binary_broadcast_kernel<float><<<static_cast<unsigned>(blocks), 256, 0, st>>>(g);
  else
    mu::binary_broadcast_kernel<__nv_bfloat16><<<static_cast<unsigned>(blocks), 256, 0, st>>>(g);
  if (cudaGetLastError() != cudaSuccess)
    return mu_set_error(ctx, MU_ERR_CUDA, "binary: launch failed");
  return MU_OK;
}
}
