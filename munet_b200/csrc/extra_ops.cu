// Forward entry points of the Backend surface that the five benchmark models do not use but
// UNet-style and RMSNorm models do (src/core/backend.hpp:207-345):
//   unary exp/log/sqrt/rsqrt/sin/cos   src/backend/cpu_backend.hpp:533-586
//   broadcast_row                      cpu_backend.hpp:1051-1060
//   concat along one dimension         cpu_backend.hpp:416-452
//   upsample2d (nearest, integer scale) cpu_backend.hpp:889-902
//   batch_norm, eval branch            cpu_backend.hpp:920-968   y = g*(x-mean)*(1/sqrt(var+eps)) + b
//   sum / mean_last_dim / sum_to_shape cpu_backend.hpp:1040-1049, 1124-1137, 1084-1122
//   fill_uniform                       cpu_backend.hpp:1021-1038 (own counter-based generator)
// plus the two module formulas built from them:
//   LeakyReLU  relu(x) + (x - relu(x))*slope          src/nn/activations.hpp:76-88
//   RMSNorm    x * rsqrt(mean(x*x) + eps) * weight    src/nn/normalization.hpp:39-67
// float32 follows the reference's float operation order with correctly rounded single ops;
// bfloat16 evaluates in fp32 and rounds once (the reference rounds after every op).
#include "../../include/munet_b200.h"
#include "common.h"
#include "ptx.cuh"

namespace mu {

template <typename T> __device__ __forceinline__ float ldf(const T *p, long long i);
template <> __device__ __forceinline__ float ldf<float>(const float *p, long long i) { return p[i]; }
template <> __device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16 *p, long long i) {
  return __bfloat162float(p[i]);
}
__device__ __forceinline__ void stf(float *p, long long i, float v) { p[i] = v; }
__device__ __forceinline__ void stf(__nv_bfloat16 *p, long long i, float v) { p[i] = __float2bfloat16_rn(v); }

#define MU_GRID_STRIDE(i, n)                                                                       \
  for (long long i = 1ll * blockIdx.x * blockDim.x + threadIdx.x, _s = 1ll * gridDim.x * blockDim.x; \
       i < (n); i += _s)

// 16 bytes of T: what one thread moves per load / store in the memory-bound kernels below
// (4 floats or 8 bfloat16). The host picks the vector form when the pointers are 16-byte
// aligned; a tail shorter than one pack is finished element by element by the same launch.
template <typename T> struct alignas(16) Pack {
  static constexpr int N = 16 / sizeof(T);
  T v[N];
};
template <typename T> __device__ __forceinline__ float pack_get(const Pack<T> &p, int k);
template <> __device__ __forceinline__ float pack_get<float>(const Pack<float> &p, int k) { return p.v[k]; }
template <> __device__ __forceinline__ float pack_get<__nv_bfloat16>(const Pack<__nv_bfloat16> &p, int k) {
  return __bfloat162float(p.v[k]);
}
__device__ __forceinline__ void pack_set(Pack<float> &p, int k, float v) { p.v[k] = v; }
__device__ __forceinline__ void pack_set(Pack<__nv_bfloat16> &p, int k, float v) { p.v[k] = __float2bfloat16_rn(v); }
static bool al16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

__device__ __forceinline__ float unary_math(float v, int op, float slope) {
  switch (op) {
  case MU_UN_EXP: return expf(v);
  case MU_UN_LOG: return logf(v);
  case MU_UN_SQRT: return __fsqrt_rn(v);
  case MU_UN_RSQRT: return __fdiv_rn(1.0f, __fsqrt_rn(v));
  case MU_UN_SIN: return sinf(v);
  case MU_UN_COS: return cosf(v);
  default: { // leaky relu, in the reference's own op order
    const float p = v > 0.f ? v : 0.f;
    return __fadd_rn(p, __fmul_rn(__fsub_rn(v, p), slope));
  }
  }
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(256) unary_kernel(const T *x, T *y, long long n, int op, float slope) {
  long long done = 0;
  if (VEC) {
    constexpr int N = Pack<T>::N;
    const long long n_vec = n / N;
    MU_GRID_STRIDE(i, n_vec) {
      const Pack<T> in = reinterpret_cast<const Pack<T> *>(x)[i];
      Pack<T> out;
#pragma unroll
      for (int k = 0; k < N; ++k)
        pack_set(out, k, unary_math(pack_get(in, k), op, slope));
      reinterpret_cast<Pack<T> *>(y)[i] = out;
    }
    done = n_vec * N;
  }
  MU_GRID_STRIDE(j, n - done) stf(y, done + j, unary_math(ldf(x, done + j), op, slope));
}

// out[r, :] = row: with the row a whole number of packs, every thread stores 16 bytes and reads
// its pack of the (cache-resident) row once per store.
template <typename T, bool VEC>
__global__ void __launch_bounds__(256) broadcast_row_kernel(const T *row, T *out, long long rows, int cols) {
  if (VEC) {
    constexpr int N = Pack<T>::N;
    const int cv = cols / N;
    const long long n_vec = rows * cv;
    MU_GRID_STRIDE(i, n_vec)
      reinterpret_cast<Pack<T> *>(out)[i] = reinterpret_cast<const Pack<T> *>(row)[i % cv];
  } else {
    const long long n = rows * cols;
    MU_GRID_STRIDE(i, n) out[i] = row[i % cols];
  }
}

struct ConcatArgs {
  const void *in[8];
  long long span[8];  // elements one outer step takes in input j (dim_j * inner)
  long long start[8]; // element offset of input j inside one outer step of the output
  int n;
  long long out_span, outer;
};
template <typename T> __global__ void __launch_bounds__(256) concat_kernel(ConcatArgs g, T *out) {
  const long long n = g.outer * g.out_span;
  MU_GRID_STRIDE(i, n) {
    const long long o = i / g.out_span, r = i % g.out_span;
    int j = 0;
#pragma unroll
    for (int k = 1; k < 8; ++k)
      if (k < g.n && r >= g.start[k])
        j = k;
    out[i] = static_cast<const T *>(g.in[j])[o * g.span[j] + (r - g.start[j])];
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
upsample2d_kernel(const T *x, T *y, long long BC, int iH, int iW, int scale) {
  const int oH = iH * scale, oW = iW * scale;
  const long long n = BC * oH * oW;
  MU_GRID_STRIDE(i, n) {
    const int ow = static_cast<int>(i % oW), oh = static_cast<int>((i / oW) % oH);
    const long long bc = i / (1ll * oW * oH);
    y[i] = x[(bc * iH + oh / scale) * iW + ow / scale];
  }
}

// VEC: H*W is a whole number of packs, so the elements of a pack share their channel.
template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
batch_norm_eval_kernel(const T *x, const T *g, const T *b, const float *mean, const float *var, T *y,
                       long long n, int C, int spatial, float eps) {
  constexpr int N = VEC ? Pack<T>::N : 1;
  MU_GRID_STRIDE(i, n / N) {
    const int c = static_cast<int>((i * N / spatial) % C);
    const float inv_std = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var[c], eps)));
    const float gc = ldf(g, c), bc = ldf(b, c), mc = mean[c];
    if (VEC) {
      const Pack<T> in = reinterpret_cast<const Pack<T> *>(x)[i];
      Pack<T> out;
#pragma unroll
      for (int k = 0; k < N; ++k)
        pack_set(out, k, __fadd_rn(__fmul_rn(__fmul_rn(gc, __fsub_rn(pack_get(in, k), mc)), inv_std), bc));
      reinterpret_cast<Pack<T> *>(y)[i] = out;
    } else {
      stf(y, i, __fadd_rn(__fmul_rn(__fmul_rn(gc, __fsub_rn(ldf(x, i), mc)), inv_std), bc));
    }
  }
}

// One warp per row; accumulation in double like the reference's mean (cpu_backend.hpp:1124-1137).
// VEC: rows are a whole number of 16-byte packs and 16-byte aligned, so a lane moves a pack at a time.
template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
rms_norm_kernel(const T *x, const T *w, T *y, long long rows, int cols, float eps) {
  const int lane = threadIdx.x & 31;
  const long long row = 1ll * blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows)
    return;
  const T *xr = x + row * cols;
  constexpr int N = VEC ? Pack<T>::N : 1;
  double s = 0.0;
  for (int c = lane * N; c < cols; c += 32 * N) {
    if (VEC) {
      const Pack<T> p = *reinterpret_cast<const Pack<T> *>(xr + c);
#pragma unroll
      for (int k = 0; k < N; ++k) {
        const float v = pack_get(p, k);
        s += static_cast<double>(__fmul_rn(v, v));
      }
    } else {
      const float v = ldf(xr, c);
      s += static_cast<double>(__fmul_rn(v, v));
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    s += __shfl_xor_sync(0xffffffffu, s, o);
  const float m = static_cast<float>(s / static_cast<double>(cols));
  const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(m, eps)));
  for (int c = lane * N; c < cols; c += 32 * N) {
    if (VEC) {
      const Pack<T> p = *reinterpret_cast<const Pack<T> *>(xr + c);
      const Pack<T> g = *reinterpret_cast<const Pack<T> *>(w + c);
      Pack<T> o;
#pragma unroll
      for (int k = 0; k < N; ++k)
        pack_set(o, k, __fmul_rn(__fmul_rn(pack_get(p, k), r), pack_get(g, k)));
      *reinterpret_cast<Pack<T> *>(y + row * cols + c) = o;
    } else {
      stf(y + row * cols, c, __fmul_rn(__fmul_rn(ldf(xr, c), r), ldf(w, c)));
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
mean_last_dim_kernel(const T *x, T *out, long long outer, int dim, int mean) {
  const int lane = threadIdx.x & 31;
  const long long row = 1ll * blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= outer)
    return;
  double s = 0.0;
  for (int c = lane; c < dim; c += 32)
    s += static_cast<double>(ldf(x, row * dim + c));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0)
    stf(out, row, static_cast<float>(mean ? s / static_cast<double>(dim) : s));
}

// Whole-tensor sum: one block, double accumulation (deterministic; the reference adds
// sequentially in float, which this matches to float rounding on well-scaled data).
template <typename T> __global__ void __launch_bounds__(1024) sum_all_kernel(const T *x, T *out, long long n) {
  __shared__ double part[32];
  double s = 0.0;
  for (long long i = threadIdx.x; i < n; i += blockDim.x)
    s += static_cast<double>(ldf(x, i));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0)
    part[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    s = threadIdx.x < (blockDim.x >> 5) ? part[threadIdx.x] : 0.0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      s += __shfl_xor_sync(0xffffffffu, s, o);
    if (threadIdx.x == 0)
      stf(out, 0, static_cast<float>(s));
  }
}

struct ReduceArgs {
  int ndim;
  int in_shape[6];
  long long in_stride[6];
  int reduced[6]; // 1 where the output has extent 1 or no such dimension
  long long out_total, red_total;
};
// One thread per output element walks every input element that folds onto it.
template <typename T> __global__ void __launch_bounds__(256) sum_to_shape_kernel(ReduceArgs g, const T *x, T *out) {
  MU_GRID_STRIDE(o, g.out_total) {
    long long base = 0, rem = o;
    for (int d = g.ndim - 1; d >= 0; --d)
      if (!g.reduced[d]) {
        base += (rem % g.in_shape[d]) * g.in_stride[d];
        rem /= g.in_shape[d];
      }
    double s = 0.0;
    for (long long r = 0; r < g.red_total; ++r) {
      long long off = base, rr = r;
      for (int d = g.ndim - 1; d >= 0; --d)
        if (g.reduced[d]) {
          off += (rr % g.in_shape[d]) * g.in_stride[d];
          rr /= g.in_shape[d];
        }
      s += static_cast<double>(ldf(x, off));
    }
    stf(out, o, static_cast<float>(s));
  }
}

// Counter-based generator (a 64-bit mix of seed and index): the same (seed, index) gives the same
// value on any launch geometry. The reference's fill is mt19937 per thread chunk and depends on
// the host's thread count, so no bit parity exists to keep; range and moments are the contract.
template <typename T>
__global__ void __launch_bounds__(256)
fill_uniform_kernel(T *out, long long n, float low, float high, unsigned long long seed) {
  MU_GRID_STRIDE(i, n) {
    unsigned long long z = seed + 0x9E3779B97F4A7C15ull * static_cast<unsigned long long>(i + 1);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    const float u = static_cast<float>(z >> 40) * (1.0f / 16777216.0f); // [0, 1)
    stf(out, i, fmaf(u, high - low, low));
  }
}

static unsigned blocks_for(long long n, int num_sms) {
  long long b = (n + 255) / 256;
  const long long cap = 1ll * (num_sms > 0 ? num_sms : 1) * 32;
  if (b > cap)
    b = cap;
  return static_cast<unsigned>(b < 1 ? 1 : b);
}

} // namespace mu

extern "C" {
int mu_set_error(mu_ctx *ctx, int code, const char *msg);
int mu_ctx_select_device(mu_ctx *ctx);

#define MU_X_BEGIN(name)                                                                           \
  if (!ctx)                                                                                        \
    return MU_ERR_INVALID;                                                                         \
  if (dtype != MU_F32 && dtype != MU_BF16)                                                         \
    return mu_set_error(ctx, MU_ERR_UNSUPPORTED, name ": dtype not implemented (float32, bfloat16)"); \
  if (mu_ctx_select_device(ctx) != MU_OK)                                                          \
    return mu_set_error(ctx, MU_ERR_CUDA, name ": cannot select device");                          \
  cudaStream_t st = static_cast<cudaStream_t>(stream);                                             \
  const int sms = mu_ctx_num_sms(ctx);                                                             \
  (void)sms;
#define MU_X_END(name)                                                                             \
  if (cudaGetLastError() != cudaSuccess)                                                           \
    return mu_set_error(ctx, MU_ERR_CUDA, name ": launch failed");                                 \
  return MU_OK;
// launch KERNEL<T, VEC> for the dtype, vector form when `vec_ok`; `work` = threads' worth of items
#define MU_X_LAUNCH(KERNEL, vec_ok, work, ...)                                                     \
  do {                                                                                             \
    const unsigned nb = mu::blocks_for((work), sms);                                               \
    if (dtype == MU_F32) {                                                                         \
      typedef float T;                                                                             \
      if (vec_ok) KERNEL<T, true><<<nb, 256, 0, st>>>(__VA_ARGS__);                                \
      else KERNEL<T, false><<<nb, 256, 0, st>>>(__VA_ARGS__);                                      \
    } else {                                                                                       \
      typedef __nv_bfloat16 T;                                                                     \
      if (vec_ok) KERNEL<T, true><<<nb, 256, 0, st>>>(__VA_ARGS__);                                \
      else KERNEL<T, false><<<nb, 256, 0, st>>>(__VA_ARGS__);                                      \
    }                                                                                              \
  } while (0)
#define TP(p) static_cast<const T *>(p)
#define TPW(p) static_cast<T *>(p)
#define F32P(p) static_cast<const float *>(p)
#define BF16P(p) static_cast<const __nv_bfloat16 *>(p)

int mu_unary(mu_ctx *ctx, int op, const void *x, void *y, long long n, int dtype, void *stream) {
  MU_X_BEGIN("unary")
  if (op < MU_UN_EXP || op > MU_UN_COS)
    return mu_set_error(ctx, MU_ERR_INVALID, "unary: unknown op");
  if (n < 0)
    return mu_set_error(ctx, MU_ERR_INVALID, "unary: negative size");
  if (n == 0)
    return MU_OK;
  if (!x || !y)
    return mu_set_error(ctx, MU_ERR_INVALID, "unary: null pointer");
  const bool vec = mu::al16(x) && mu::al16(y) && n >= 64;
  const int per = dtype == MU_F32 ? 4 : 8;
  MU_X_LAUNCH(mu::unary_kernel, vec, vec ? n / per + per : n, TP(x), TPW(y), n, op, 0.f);
  MU_X_END("unary")
}

int mu_leaky_relu(mu_ctx *ctx, const void *x, void *y, long long n, float slope, int dtype, void *stream) {
  MU_X_BEGIN("LeakyReLU")
  if (n < 0)
    return mu_set_error(ctx, MU_ERR_INVALID, "LeakyReLU: negative size");
  if (n == 0)
    return MU_OK;
  if (!x || !y)
    return mu_set_error(ctx, MU_ERR_INVALID, "LeakyReLU: null pointer");
  // the slope tensor of the reference has the activation's dtype: round it the same way
  const float sl = dtype == MU_F32 ? slope : __bfloat162float(__float2bfloat16_rn(slope));
  const bool vec = mu::al16(x) && mu::al16(y) && n >= 64;
  const int per = dtype == MU_F32 ? 4 : 8;
  MU_X_LAUNCH(mu::unary_kernel, vec, vec ? n / per + per : n, TP(x), TPW(y), n, -1, sl);
  MU_X_END("LeakyReLU")
}

int mu_broadcast_row(mu_ctx *ctx, const void *row, void *out, long long rows, int cols, int dtype,
                     void *stream) {
  MU_X_BEGIN("broadcast_row")
  if (rows < 0 || cols < 0)
    return mu_set_error(ctx, MU_ERR_INVALID, "broadcast_row: negative size");
  if (rows == 0 || cols == 0)
    return MU_OK;
  if (!row || !out)
    return mu_set_error(ctx, MU_ERR_INVALID, "broadcast_row: null pointer");
  const int per = dtype == MU_F32 ? 4 : 8;
  const bool vec = mu::al16(row) && mu::al16(out) && cols % per == 0;
  MU_X_LAUNCH(mu::broadcast_row_kernel, vec, vec ? rows * cols / per : rows * cols, TP(row), TPW(out), rows, cols);
  MU_X_END("broadcast_row")
}

int mu_concat(mu_ctx *ctx, const void *const *inputs, const int *dim_sizes, int n_inputs, void *out,
              long long outer, long long inner, int dtype, void *stream) {
  MU_X_BEGIN("concat")
  if (n_inputs <= 0 || !inputs || !dim_sizes)
    return mu_set_error(ctx, MU_ERR_INVALID, "concat: expects at least one input");
  if (outer < 0 || inner < 0)
    return mu_set_error(ctx, MU_ERR_INVALID, "concat: negative size");
  long long out_dim = 0;
  for (int j = 0; j < n_inputs; ++j) {
    if (dim_sizes[j] < 0)
      return mu_set_error(ctx, MU_ERR_INVALID, "concat: negative dimension");
    out_dim += dim_sizes[j];
  }
  if (outer == 0 || inner == 0 || out_dim == 0)
    return MU_OK;
  if (!out)
    return mu_set_error(ctx, MU_ERR_INVALID, "concat: null output");
  if (n_inputs > 8)
    return mu_set_error(ctx, MU_ERR_UNSUPPORTED, "concat: more than 8 inputs");
  mu::ConcatArgs g;
  g.n = n_inputs;
  g.outer = outer;
  long long span = 0;
  for (int k = 0; k < 8; ++k) {
    g.in[k] = nullptr, g.span[k] = 0, g.start[k] = span;
    if (k < n_inputs) {
      if (!inputs[k] && dim_sizes[k] > 0)
        return mu_set_error(ctx, MU_ERR_INVALID, "concat: null input");
      g.in[k] = inputs[k];
      g.span[k] = dim_sizes[k] * inner;
      span += g.span[k];
    }
  }
  g.out_span = span;
  if (dtype == MU_F32)
    mu::concat_kernel<float><<<mu::blocks_for(outer * span, sms), 256, 0, st>>>(g, static_cast<float *>(out));
  else
    mu::concat_kernel<__nv_bfloat16><<<mu::blocks_for(outer * span, sms), 256, 0, st>>>(
        g, static_cast<__nv_bfloat16 *>(out));
  MU_X_END("concat")
}

int mu_upsample2d(mu_ctx *ctx, const void *x, void *y, int B, int C, int H, int W, int scale, int dtype,
                  void *stream) {
  MU_X_BEGIN("upsample2d")
  if (B < 0 || C < 0 || H < 0 || W < 0 || scale <= 0)
    return mu_set_error(ctx, MU_ERR_INVALID, "upsample2d: bad geometry");
  const long long n = 1ll * B * C * H * W * scale * scale;
  if (n == 0)
    return MU_OK;
  if (!x || !y)
    return mu_set_error(ctx, MU_ERR_INVALID, "upsample2d: null pointer");
  if (dtype == MU_F32)
    mu::upsample2d_kernel<float><<<mu::blocks_for(n, sms), 256, 0, st>>>(F32P(x), static_cast<float *>(y),
                                                                         1ll * B * C, H, W, scale);
  else
    mu::upsample2d_kernel<__nv_bfloat16><<<mu::blocks_for(n, sms), 256, 0, st>>>(
        BF16P(x), static_cast<__nv_bfloat16 *>(y), 1ll * B * C, H, W, scale);
  MU_X_END("upsample2d")
}

int mu_batch_norm_eval(mu_ctx *ctx, const void *x, const void *gamma, const void *beta,
                       const float *running_mean, const float *running_var, void *y, int B, int C,
                       int H, int W, float eps, int dtype, void *stream) {
  MU_X_BEGIN("batch_norm")
  if (B < 0 || C <= 0 || H < 0 || W < 0)
    return mu_set_error(ctx, MU_ERR_INVALID, "batch_norm: bad geometry");
  const long long n = 1ll * B * C * H * W;
  if (n == 0)
    return MU_OK;
  if (!x || !gamma || !beta || !running_mean || !running_var || !y)
    return mu_set_error(ctx, MU_ERR_INVALID, "batch_norm: null pointer");
  const int per = dtype == MU_F32 ? 4 : 8;
  const bool vec = mu::al16(x) && mu::al16(y) && (H * W) % per == 0;
  MU_X_LAUNCH(mu::batch_norm_eval_kernel, vec, vec ? n / per : n, TP(x), TP(gamma), TP(beta), running_mean,
              running_var, TPW(y), n, C, H * W, eps);
  MU_X_END("batch_norm")
}

int mu_rms_norm(mu_ctx *ctx, const void *x, const void *weight, void *y, long long rows, int cols,
                float eps, int dtype, void *stream) {
  MU_X_BEGIN("RMSNorm")
  if (rows < 0 || cols <= 0)
    return mu_set_error(ctx, MU_ERR_INVALID, "RMSNorm expects normalized_shape > 0");
  if (rows == 0)
    return MU_OK;
  if (!x || !weight || !y)
    return mu_set_error(ctx, MU_ERR_INVALID, "RMSNorm: null pointer");
  const unsigned nb = static_cast<unsigned>((rows + 7) / 8);
  const int per = dtype == MU_F32 ? 4 : 8;
  const bool vec = mu::al16(x) && mu::al16(weight) && mu::al16(y) && cols % per == 0;
  if (dtype == MU_F32) {
    if (vec) mu::rms_norm_kernel<float, true><<<nb, 256, 0, st>>>(F32P(x), F32P(weight), static_cast<float *>(y), rows, cols, eps);
    else mu::rms_norm_kernel<float, false><<<nb, 256, 0, st>>>(F32P(x), F32P(weight), static_cast<float *>(y), rows, cols, eps);
  } else {
    if (vec) mu::rms_norm_kernel<__nv_bfloat16, true><<<nb, 256, 0, st>>>(BF16P(x), BF16P(weight), static_cast<__nv_bfloat16 *>(y), rows, cols, eps);
    else mu::rms_norm_kernel<__nv_bfloat16, false><<<nb, 256, 0, st>>>(BF16P(x), BF16P(weight), static_cast<__nv_bfloat16 *>(y), rows, cols, eps);
  }
  MU_X_END("RMSNorm")
}

int mu_sum(mu_ctx *ctx, const void *x, void *out, long long n, int dtype, void *stream) {
  MU_X_BEGIN("sum")
  if (n < 0)
    return mu_set_error(ctx, MU_ERR_INVALID, "sum: negative size");
  if (!out || (n > 0 && !x))
    return mu_set_error(ctx, MU_ERR_INVALID, "sum: null pointer");
  if (dtype == MU_F32)
    mu::sum_all_kernel<float><<<1, 1024, 0, st>>>(F32P(x), static_cast<float *>(out), n);
  else
    mu::sum_all_kernel<__nv_bfloat16><<<1, 1024, 0, st>>>(BF16P(x), static_cast<__nv_bfloat16 *>(out), n);
  MU_X_END("sum")
}

int mu_mean_last_dim(mu_ctx *ctx, const void *x, void *out, long long outer, int dim, int dtype,
                     void *stream) {
  MU_X_BEGIN("mean_last_dim")
  if (outer < 0 || dim <= 0)
    return mu_set_error(ctx, MU_ERR_INVALID, "mean_last_dim: bad shape");
  if (outer == 0)
    return MU_OK;
  if (!x || !out)
    return mu_set_error(ctx, MU_ERR_INVALID, "mean_last_dim: null pointer");
  const unsigned nb = static_cast<unsigned>((outer + 7) / 8);
  if (dtype == MU_F32)
    mu::mean_last_dim_kernel<float><<<nb, 256, 0, st>>>(F32P(x), static_cast<float *>(out), outer, dim, 1);
  else
    mu::mean_last_dim_kernel<__nv_bfloat16><<<nb, 256, 0, st>>>(BF16P(x), static_cast<__nv_bfloat16 *>(out),
                                                               outer, dim, 1);
  MU_X_END("mean_last_dim")
}

int mu_sum_to_shape(mu_ctx *ctx, const void *x, void *out, const int *in_shape, int in_ndim,
                    const int *out_shape, int out_ndim, int dtype, void *stream) {
  MU_X_BEGIN("sum_to_shape")
  if (in_ndim < 0 || in_ndim > 6 || out_ndim < 0 || out_ndim > in_ndim ||
      (in_ndim > 0 && !in_shape) || (out_ndim > 0 && !out_shape))
    return mu_set_error(ctx, MU_ERR_INVALID, "sum_to_shape: 0..6 dimensions, output rank <= input rank");
  mu::ReduceArgs g;
  g.ndim = in_ndim, g.out_total = 1, g.red_total = 1;
  long long stride = 1;
  for (int d = in_ndim - 1; d >= 0; --d) {
    if (in_shape[d] < 0)
      return mu_set_error(ctx, MU_ERR_INVALID, "sum_to_shape: negative dimension");
    g.in_shape[d] = in_shape[d], g.in_stride[d] = stride;
    stride *= in_shape[d];
    const int od = d - (in_ndim - out_ndim);
    const bool kept = od >= 0 && out_shape[od] != 1;
    if (kept && out_shape[od] != in_shape[d])
      return mu_set_error(ctx, MU_ERR_INVALID, "sum_to_shape: output extent must be 1 or the input's");
    g.reduced[d] = kept ? 0 : 1;
    (kept ? g.out_total : g.red_total) *= in_shape[d];
  }
  if (g.out_total == 0)
    return MU_OK;
  if (!out || (g.red_total > 0 && !x))
    return mu_set_error(ctx, MU_ERR_INVALID, "sum_to_shape: null pointer");
  if (dtype == MU_F32)
    mu::sum_to_shape_kernel<float><<<mu::blocks_for(g.out_total, sms), 256, 0, st>>>(g, F32P(x), static_cast<float *>(out));
  else
    mu::sum_to_shape_kernel<__nv_bfloat16><<<mu::blocks_for(g.out_total, sms), 256, 0, st>>>(
        g, BF16P(x), static_cast<__nv_bfloat16 *>(out));
  MU_X_END("sum_to_shape")
}

int mu_fill_uniform(mu_ctx *ctx, void *out, long long n, float low, float high,
                    unsigned long long seed, int dtype, void *stream) {
  MU_X_BEGIN("fill_uniform")
  if (n < 0)
    return mu_set_error(ctx, MU_ERR_INVALID, "fill_uniform: negative size");
  if (n == 0)
    return MU_OK;
  if (!out)
    return mu_set_error(ctx, MU_ERR_INVALID, "fill_uniform: null pointer");
  if (dtype == MU_F32)
    mu::fill_uniform_kernel<float><<<mu::blocks_for(n, sms), 256, 0, st>>>(static_cast<float *>(out), n, low, high, seed);
  else
    mu::fill_uniform_kernel<__nv_bfloat16><<<mu::blocks_for(n, sms), 256, 0, st>>>(
        static_cast<__nv_bfloat16 *>(out), n, low, high, seed);
  MU_X_END("fill_uniform")
}
}
