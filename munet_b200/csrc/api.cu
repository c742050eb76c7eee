// extern "C" boundary of libmunet_b200.so (declared in include/munet_b200.h).
// Validates arguments, picks the kernel for each call and turns every failure
// into a status code + message; nothing here throws or exits.
#include "../../include/munet_b200.h"
#include "common.h"
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <new>

namespace mu {
int launch_gemm_bf16_tcgen05(const GemmOperands &, const GemmShape &, const Epilogue &, int *status,
                             int num_sms, cudaStream_t);
int launch_gemm_simt(const SimtArgs &, cudaStream_t);
int launch_layer_norm(const void *, const void *, const void *, void *, long long, int, float, int, int *, int,
                      cudaStream_t);
int launch_softmax(const void *, void *, long long, int, float, int, int, int, cudaStream_t);
int launch_softmax_bf16_rows(const void *, void *, long long, int, float, int, int, int *, int,
                             cudaStream_t);
int launch_embedding(const int *, const void *, const void *, void *, long long, int, int, int, int,
                     int *, cudaStream_t);
int launch_eltwise(const void *, const void *, const void *, void *, long long, int, int, int, int,
                   cudaStream_t);
int launch_argmax(const void *, int *, long long, int, int, cudaStream_t);
size_t gemm_tf32x3_scratch_bytes(int, int, int);
int launch_gemm_tf32x3(const float *, long long, const float *, long long, int, float *, long long,
                       const float *, const float *, float, int, int, int, int, void *, int *, int,
                       cudaStream_t);
int launch_attention_tcgen05(const void *, const void *, const void *, void *, int, int, int, int,
                             int, int, int *, cudaStream_t);
int launch_attention_tcgen05_ex(const void *, const void *, const void *, void *, long long, void *, int, int,
                                int, int, int, int, int *, cudaStream_t);
void set_attention_variant(int);
void set_gemm_b_hint(int);
void set_gemm_l2_set_aside(double);
} // namespace mu

struct mu_ctx {
  int device = 0;
  int num_sms = 0;
  int force_simt = 0;
  int sm_budget = 0; // > 0: persistent GEMM grids use at most this many SMs
  int gemm_bn = 0, gemm_ctas = 0; // > 0: tile shape forced by mu_ctx_set_gemm_tile
  int *d_status = nullptr;
  char err[512] = {0};
};

namespace {

int fail(mu_ctx *ctx, int code, const char *fmt, ...) {
  if (ctx) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(ctx->err, sizeof(ctx->err), fmt, ap);
    va_end(ap);
  }
  return code;
}

int cuda_fail(mu_ctx *ctx, const char *what, cudaError_t e) {
  return fail(ctx, MU_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

bool set_device(mu_ctx *ctx) {
  int cur = -1;
  if (cudaGetDevice(&cur) != cudaSuccess)
    return false;
  if (cur != ctx->device && cudaSetDevice(ctx->device) != cudaSuccess)
    return false;
  return true;
}

size_t esize(int dtype) { return dtype == MU_F32 || dtype == MU_I32 ? 4 : 2; }
bool al16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

bool epilogue_vec_ok(const mu::Epilogue &ep) {
  if (!al16(ep.c) || (ep.bias && !al16(ep.bias)) || (ep.residual && !al16(ep.residual)))
    return false;
  if (ep.split_T > 0)
    return ep.split_D % 32 == 0 && ep.split_which_stride % 8 == 0;
  return ep.ldc % 8 == 0 && ep.batch_hi % 8 == 0 && ep.batch_lo % 8 == 0;
}

// One GEMM: tcgen05 when dtype/alignment allow it, CUDA-core kernel otherwise.
int run_gemm(mu_ctx *ctx, const mu::GemmOperands &op, const mu::GemmShape &sh, mu::Epilogue ep,
             int dtype, cudaStream_t st, const char *who) {
  if (dtype != MU_F32 && dtype != MU_BF16)
    return fail(ctx, MU_ERR_UNSUPPORTED, "%s: dtype %d not implemented (float32, bfloat16)", who,
                dtype);
  if (sh.M == 0 || sh.N == 0 || sh.batch == 0)
    return MU_OK;
  if (!set_device(ctx))
    return fail(ctx, MU_ERR_CUDA, "%s: cannot select device %d", who, ctx->device);
  if (dtype == MU_BF16 && !ctx->force_simt && sh.K > 0) {
    ep.vec_ok = epilogue_vec_ok(ep) ? 1 : 0;
    mu::GemmShape shf = sh;
    shf.force_bn = ctx->gemm_bn, shf.force_ctas = ctx->gemm_ctas;
    const int sms = (ctx->sm_budget > 0 && ctx->sm_budget < ctx->num_sms) ? ctx->sm_budget : ctx->num_sms;
    int rc = mu::launch_gemm_bf16_tcgen05(op, shf, ep, ctx->d_status, sms, st);
    if (rc == 0)
      return MU_OK;
    if (rc == 2)
      return cuda_fail(ctx, who, cudaGetLastError());
    // rc == 1: shape or alignment outside the TMA kernel's envelope
  }
  if (ep.c_mirror)
    return fail(ctx, MU_ERR_UNSUPPORTED, "%s: a mirrored output needs the bfloat16 tensor-core kernel "
                "(plain [M,N] output, N a multiple of 8, 16-byte aligned rows)", who);
  // Large float32 products: tensor cores with every operand split in two TF32 parts (float32-class
  // accuracy, not the reference's accumulation order). Below 2^31 multiply-adds the CUDA-core
  // kernel keeps the reference's result bit for bit.
  if (dtype == MU_F32 && !ctx->force_simt && sh.batch == 1 && ep.split_T == 0 && ep.batch_div <= 1 &&
      1.0 * sh.M * sh.N * sh.K >= 2147483648.0 && sh.K % 4 == 0 && ep.ldc % 4 == 0) {
    // The split copies live in a stream-ordered allocation (pool-backed, legal inside a stream
    // capture): concurrent calls on different streams never share scratch.
    const size_t need = mu::gemm_tf32x3_scratch_bytes(sh.M, sh.N, sh.K);
    void *scratch = nullptr;
    if (cudaMallocAsync(&scratch, need, st) == cudaSuccess) {
      int rc = mu::launch_gemm_tf32x3(static_cast<const float *>(op.a), op.lda,
                                      static_cast<const float *>(op.b), op.ldb, op.b_kmajor,
                                      static_cast<float *>(ep.c), ep.ldc,
                                      static_cast<const float *>(ep.bias),
                                      static_cast<const float *>(ep.residual), ep.alpha, ep.act, sh.M,
                                      sh.N, sh.K, scratch, ctx->d_status, ctx->num_sms, st);
      cudaFreeAsync(scratch, st);
      if (rc == 0)
        return MU_OK;
      if (rc == 2)
        return cuda_fail(ctx, who, cudaGetLastError());
    } else {
      cudaGetLastError(); // out of memory: the CUDA-core kernel needs no scratch
    }
  }
  mu::SimtArgs g;
  g.a = op.a, g.b = op.b, g.lda = op.lda, g.ldb = op.ldb;
  g.a_batch = op.a_batch, g.b_batch = op.b_batch, g.b_kmajor = op.b_kmajor;
  g.is_bf16 = dtype == MU_BF16;
  g.sh = sh, g.ep = ep;
  int rc = mu::launch_gemm_simt(g, st);
  if (rc == 1)
    return fail(ctx, MU_ERR_INVALID, "%s: shape M=%d N=%d K=%d batch=%d out of range", who, sh.M,
                sh.N, sh.K, sh.batch);
  if (rc != 0)
    return cuda_fail(ctx, who, cudaGetLastError());
  return MU_OK;
}

#define MU_REQUIRE(cond, ...)                                                                    \
  do {                                                                                           \
    if (!(cond))                                                                                 \
      return fail(ctx, MU_ERR_INVALID, __VA_ARGS__);                                             \
  } while (0)

} // namespace

extern "C" {

int mu_abi_version(void) { return MU_ABI_VERSION; }

int mu_ctx_create(int device, mu_ctx **out) {
  if (!out)
    return MU_ERR_INVALID;
  *out = nullptr;
  mu_ctx *ctx = new (std::nothrow) mu_ctx();
  if (!ctx)
    return MU_ERR_NOMEM;
  ctx->device = device;
  cudaError_t e = cudaSetDevice(device);
  cudaDeviceProp prop;
  if (e == cudaSuccess)
    e = cudaGetDeviceProperties(&prop, device);
  if (e == cudaSuccess && prop.major != 10) {
    // Built for sm_100a only; there is no other code path.
    fprintf(stderr, "munet_b200: device %d is sm_%d%d, this library only runs on sm_100\n", device,
            prop.major, prop.minor);
    delete ctx;
    return MU_ERR_UNSUPPORTED;
  }
  if (e == cudaSuccess)
    e = cudaMalloc(&ctx->d_status, sizeof(int));
  if (e == cudaSuccess)
    e = cudaMemset(ctx->d_status, 0, sizeof(int));
  if (e != cudaSuccess) {
    fprintf(stderr, "munet_b200: context creation failed: %s\n", cudaGetErrorString(e));
    delete ctx;
    return MU_ERR_CUDA;
  }
  ctx->num_sms = prop.multiProcessorCount;
  {
    // Stream-ordered scratch (3xTF32 operand copies) is reused from the device's default pool:
    // keep freed blocks cached instead of returning them to the driver at every synchronisation.
    cudaMemPool_t pool = nullptr;
    if (cudaDeviceGetDefaultMemPool(&pool, device) == cudaSuccess && pool) {
      unsigned long long keep = ~0ull;
      cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
    }
    cudaGetLastError();
  }
  *out = ctx;
  return MU_OK;
}

void mu_timer_release(mu_ctx *ctx); // memory_ops.cu

void mu_ctx_destroy(mu_ctx *ctx) {
  if (!ctx)
    return;
  mu_timer_release(ctx);
  if (ctx->d_status)
    cudaFree(ctx->d_status);
  delete ctx;
}

const char *mu_last_error(const mu_ctx *ctx) { return ctx ? ctx->err : "null context"; }
// used by the entry points that live in other translation units
int mu_set_error(mu_ctx *ctx, int code, const char *msg) { return fail(ctx, code, "%s", msg); }
int mu_ctx_num_sms(const mu_ctx *ctx) { return ctx ? ctx->num_sms : 0; }
int mu_ctx_select_device(mu_ctx *ctx) { return (ctx && set_device(ctx)) ? MU_OK : MU_ERR_CUDA; }
// accessors for the entry points that live in other translation units
int *mu_ctx_status_ptr(mu_ctx *ctx) { return ctx ? ctx->d_status : nullptr; }
int mu_ctx_simt_forced(const mu_ctx *ctx) { return ctx ? ctx->force_simt : 0; }
int mu_ctx_set_sm_budget(mu_ctx *ctx, int n) {
  if (!ctx || n < 0)
    return MU_ERR_INVALID;
  ctx->sm_budget = n;
  return MU_OK;
}
int mu_ctx_set_gemm_tile(mu_ctx *ctx, int bn, int ctas) {
  if (!ctx)
    return MU_ERR_INVALID;
  const bool ok = (bn == 0 && ctas == 0) || ((bn == 64 || bn == 128 || bn == 256) && (ctas == 1 || ctas == 2) &&
                                             !(ctas == 2 && bn == 64));
  if (!ok)
    return fail(ctx, MU_ERR_INVALID, "gemm tile: width 64/128/256 on 1 CTA, 128/256 on 2; 0,0 = automatic");
  ctx->gemm_bn = bn, ctx->gemm_ctas = ctas;
  return MU_OK;
}
// Not part of the declared ABI: selects the fused attention kernel (0 two query tiles per CTA,
// 1 one tile per CTA) for timing one against the other. Process-wide.
void mu_debug_attention_variant(int v) { mu::set_attention_variant(v); }
// Not part of the declared ABI: L2 hints of the tensor-core GEMM: 0 none, 1 evict_last on the B tiles,
// 2 that and evict_first on the residual and output streams; -1 leaves the choice to the launcher.
// Process-wide, for timing one against the other.
void mu_debug_gemm_b_hint(int v) { mu::set_gemm_b_hint(v); }
int mu_ctx_set_l2_set_aside(mu_ctx *ctx, size_t bytes) {
  if (!ctx)
    return MU_ERR_INVALID;
  if (!set_device(ctx))
    return fail(ctx, MU_ERR_CUDA, "l2 set-aside: cannot select device %d", ctx->device);
  const cudaError_t e = cudaDeviceSetLimit(cudaLimitPersistingL2CacheSize, bytes);
  if (e != cudaSuccess)
    return cuda_fail(ctx, "l2 set-aside", e);
  mu::set_gemm_l2_set_aside(static_cast<double>(bytes));
  return MU_OK;
}
int mu_ctx_force_simt(mu_ctx *ctx, int on) {
  if (!ctx)
    return MU_ERR_INVALID;
  ctx->force_simt = on;
  return MU_OK;
}

int mu_alloc(mu_ctx *ctx, size_t bytes, void **ptr) {
  if (!ctx || !ptr)
    return MU_ERR_INVALID;
  *ptr = nullptr;
  if (bytes == 0)
    return MU_OK;
  if (!set_device(ctx))
    return fail(ctx, MU_ERR_CUDA, "mu_alloc: cannot select device");
  cudaError_t e = cudaMalloc(ptr, bytes);
  if (e == cudaErrorMemoryAllocation) {
    cudaGetLastError();
    return fail(ctx, MU_ERR_NOMEM, "mu_alloc: out of device memory (%zu bytes)", bytes);
  }
  if (e != cudaSuccess)
    return cuda_fail(ctx, "mu_alloc", e);
  return MU_OK;
}

int mu_free(mu_ctx *ctx, void *ptr) {
  if (!ctx)
    return MU_ERR_INVALID;
  if (!ptr)
    return MU_OK;
  cudaError_t e = cudaFree(ptr);
  return e == cudaSuccess ? MU_OK : cuda_fail(ctx, "mu_free", e);
}

int mu_copy(mu_ctx *ctx, void *dst, const void *src, size_t bytes, int kind, void *stream) {
  if (!ctx)
    return MU_ERR_INVALID;
  if (bytes == 0)
    return MU_OK;
  MU_REQUIRE(dst && src, "mu_copy: null pointer");
  cudaMemcpyKind k;
  if (kind == MU_COPY_H2D)
    k = cudaMemcpyHostToDevice;
  else if (kind == MU_COPY_D2H)
    k = cudaMemcpyDeviceToHost;
  else if (kind == MU_COPY_D2D)
    k = cudaMemcpyDeviceToDevice;
  else
    return fail(ctx, MU_ERR_INVALID, "mu_copy: unknown kind %d", kind);
  if (!set_device(ctx))
    return fail(ctx, MU_ERR_CUDA, "mu_copy: cannot select device");
  cudaError_t e = cudaMemcpyAsync(dst, src, bytes, k, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? MU_OK : cuda_fail(ctx, "mu_copy", e);
}

int mu_synchronize(mu_ctx *ctx) {
  if (!ctx)
    return MU_ERR_INVALID;
  if (!set_device(ctx))
    return fail(ctx, MU_ERR_CUDA, "mu_synchronize: cannot select device");
  cudaError_t e = cudaDeviceSynchronize();
  return e == cudaSuccess ? MU_OK : cuda_fail(ctx, "mu_synchronize", e);
}

int mu_check(mu_ctx *ctx, void *stream) {
  if (!ctx)
    return MU_ERR_INVALID;
  if (!set_device(ctx))
    return fail(ctx, MU_ERR_CUDA, "mu_check: cannot select device");
  cudaError_t e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess)
    return cuda_fail(ctx, "mu_check", e);
  int st = 0;
  e = cudaMemcpy(&st, ctx->d_status, sizeof(int), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess)
    return cuda_fail(ctx, "mu_check", e);
  if (st == 0)
    return MU_OK;
  cudaMemset(ctx->d_status, 0, sizeof(int));
  if (st == 110)
    return fail(ctx, MU_ERR_INDEX, "Embedding index out of range");
  return fail(ctx, MU_ERR_TIMEOUT, "device-side bounded wait ran out (code %d)", st);
}

int mu_matmul(mu_ctx *ctx, const void *a, const void *b, void *c, int M, int K, int N, int transA,
              int transB, int dtype, void *stream) {
  if (!ctx)
    return MU_ERR_INVALID;
  MU_REQUIRE(M >= 0 && K >= 0 && N >= 0, "matmul: negative dimension");
  if (transA)
    return fail(ctx, MU_ERR_UNSUPPORTED, "matmul: transA is a training-only path");
  if (M == 0 || N == 0)
    return MU_OK;
  MU_REQUIRE(a && b && c, "matmul: null pointer");
  mu::GemmOperands op;
  op.a = a, op.lda = K, op.b = b, op.ldb = transB ? K : N, op.b_kmajor = transB ? 1 : 0;
  mu::GemmShape sh{M, N, K, 1};
  mu::Epilogue ep;
  ep.c = c, ep.ldc = N, ep.round_each = 1;
  return run_gemm(ctx, op, sh, ep, dtype, static_cast<cudaStream_t>(stream), "matmul");
}

int mu_batched_matmul(mu_ctx *ctx, const void *a, const void *b, void *c, int batch, int M, int K,
                      int N, int transA, int transB, long long stride_a, long long stride_b,
                      long long stride_out, int dtype, void *stream) {
  if (!ctx)
    return MU_ERR_INVALID;
  MU_REQUIRE(batch >= 0 && M >= 0 && K >= 0 && N >= 0, "batched_matmul: negative dimension");
  if (transA)
    return fail(ctx, MU_ERR_UNSUPPORTED, "batched_matmul: transA is a training-only path");
  if (batch == 0 || M == 0 || N == 0)
    return MU_OK;
  MU_REQUIRE(a && b && c, "batched_matmul: null pointer");
  mu::Epilogue ep;
  ep.c = c, ep.ldc = N, ep.round_each = 1;
  if (stride_b == 0 && stride_a == 1ll * M * K && stride_out == 1ll * M * N &&
      1ll * batch * M < 2147483647ll) {
    // broadcast weights over a dense batch (how a 3-D Linear input arrives,
    // src/core/ops/matmul.cpp:300-326): fold the batch into M.
    mu::GemmOperands op;
  op.a = a, op.lda = K, op.b = b, op.ldb = transB ? K : N, op.b_kmajor = transB ? 1 : 0;
    mu::GemmShape sh{batch * M, N, K, 1};
    return run_gemm(ctx, op, sh, ep, dtype, static_cast<cudaStream_t>(stream), "batched_matmul");
  }
  mu::GemmOperands op;
  op.a = a, op.lda = K, op.a_batch = stride_a, op.b = b, op.ldb = transB ? K : N;
  op.b_batch = stride_b, op.b_kmajor = transB ? 1 : 0;
  mu::GemmShape sh{M, N, K, batch};
  ep.batch_hi = stride_out, ep.batch_div = 1;
  return run_gemm(ctx, op, sh, ep, dtype, static_cast<cudaStream_t>(stream), "batched_matmul");
}

int mu_linear(mu_ctx *ctx, const void *x, const void *w, const void *bias, const void *residual,
              void *y, int M, int K, int N, int act, int dtype, void *stream) {
  if (!ctx)
    return MU_ERR_INVALID;
  MU_REQUIRE(M >= 0 && K >= 0 && N >= 0, "linear: negative dimension");
  MU_REQUIRE(act >= MU_ACT_NONE && act <= MU_ACT_TANH, "linear: unknown activation %d", act);
  if (M == 0 || N == 0)
    return MU_OK;
  MU_REQUIRE(x && w && y, "linear: null pointer");
  mu::GemmOperands op;
  op.a = x, op.lda = K, op.b = w, op.ldb = N;
  mu::GemmShape sh{M, N, K, 1};
  mu::Epilogue ep;
  ep.c = y, ep.bias = bias, ep.residual = residual, ep.act = act, ep.ldc = N, ep.round_each = 1;
  return run_gemm(ctx, op, sh, ep, dtype, static_cast<cudaStream_t>(stream), "linear");
}

// Used by the executor, not part of the declared ABI: mu_linear whose output tiles are also
// written to `y_mirror` (same [M,N] layout; may be a peer GPU's memory) from inside the epilogue.
int mu_linear_mirrored(mu_ctx *ctx, const void *x, const void *w, const void *bias, const void *residual,
                       void *y, void *y_mirror, int M, int K, int N, int act, int dtype, void *stream) {
  if (!ctx)
    return MU_ERR_INVALID;
  MU_REQUIRE(M >= 0 && K >= 0 && N >= 0, "linear: negative dimension");
  MU_REQUIRE(act >= MU_ACT_NONE && act <= MU_ACT_TANH, "linear: unknown activation %d", act);
  if (M == 0 || N == 0)
    return MU_OK;
  MU_REQUIRE(x && w && y && y_mirror, "linear: null pointer");
  mu::GemmOperands op;
  op.a = x, op.lda = K, op.b = w, op.ldb = N;
  mu::GemmShape sh{M, N, K, 1};
  mu::Epilogue ep;
  ep.c = y, ep.bias = bias, ep.residual = residual, ep.act = act, ep.ldc = N, ep.round_each = 1;
  ep.c_mirror = y_mirror;
  return run_gemm(ctx, op, sh, ep, dtype, static_cast<cudaStream_t>(stream), "linear");
}

// x[B*T, K_in] · w[K_in, 3*H*D] (+ bias[3*H*D]) written head-major: q, k, v each [B*H*T, D].
// H is the number of heads this call produces (all of them, or one rank's share under
// tensor parallelism), so the output width H*D may differ from K_in.
int mu_linear_qkv_heads(mu_ctx *ctx, const void *x, const void *w_qkv, const void *bias_qkv, void *q,
                        void *k, void *v, int B, int T, int K_in, int H, int D, int dtype,
                        void *stream) {
  if (!ctx)
    return MU_ERR_INVALID;
  MU_REQUIRE(B >= 0 && T >= 0 && K_in > 0 && H > 0 && D > 0, "linear_qkv: bad dimensions");
  if (B == 0 || T == 0)
    return MU_OK;
  MU_REQUIRE(x && w_qkv && q && k && v, "linear_qkv: null pointer");
  const int E = H * D; // output width of each of q, k, v
  const long long per = 1ll * B * T * E;
  const size_t es = esize(dtype);
  // q, k, v are addressed from q with one stride; they may be separate buffers
  const long long dk = (static_cast<const char *>(k) - static_cast<const char *>(q));
  const long long dv = (static_cast<const char *>(v) - static_cast<const char *>(q));
  mu::GemmOperands op;
  op.a = x, op.lda = K_in, op.b = w_qkv, op.ldb = 3ll * E;
  mu::Epilogue ep;
  ep.bias = bias_qkv, ep.round_each = 1;
  ep.split_T = T, ep.split_H = H, ep.split_D = D;
  if (dk == static_cast<long long>(per * es) && dv == 2 * dk) {
    mu::GemmShape sh{B * T, 3 * E, K_in, 1};
    ep.c = q, ep.split_which_stride = per;
    return run_gemm(ctx, op, sh, ep, dtype, static_cast<cudaStream_t>(stream), "linear_qkv");
  }
  // separate destinations: three GEMMs over column slices of the fused weight
  void *outs[3] = {q, k, v};
  for (int i = 0; i < 3; ++i) {
    mu::GemmOperands opi = op;
    opi.b = static_cast<const char *>(w_qkv) + 1ll * i * E * es;
    mu::Epilogue epi = ep;
    epi.c = outs[i];
    epi.bias = bias_qkv ? static_cast<const char *>(bias_qkv) + 1ll * i * E * es : nullptr;
    epi.split_which_stride = 0;
    mu::GemmShape sh{B * T, E, K_in, 1};
    int rc = run_gemm(ctx, opi, sh, epi, dtype, static_cast<cudaStream_t>(stream), "linear_qkv");
    if (rc)
      return rc;
  }
  return MU_OK;
}

int mu_linear_qkv(mu_ctx *ctx, const void *x, const void *w_qkv, const void *bias_qkv, void *q,
                  void *k, void *v, int B, int T, int E, int H, int dtype, void *stream) {
  if (!ctx)
    return MU_ERR_INVALID;
  MU_REQUIRE(E > 0 && H > 0 && E % H == 0, "linear_qkv: bad dimensions");
  return mu_linear_qkv_heads(ctx, x, w_qkv, bias_qkv, q, k, v, B, T, E, H, E / H, dtype, stream);
}

// Bytes of the [B*H, T, T] score matrix of the composed path, or false when the product (or
// B*H*T, which the kernels index with 32-bit tile coordinates) does not fit: the factors are
// bounded by division so that nothing wraps.
static bool score_bytes(int B, int H, int T, int dtype, size_t *out) {
  const unsigned long long es = esize(dtype), uB = B, uH = H, uT = T;
  const unsigned long long cap = 1ull << 46; // 64 TiB: far beyond any device, far below 2^64
  if (uB * uH > 0x7fffffffull || uB * uH * uT > 0x7fffffffull)
    return false;
  if (uT > cap / uT || uB * uH > cap / (uT * uT) / es)
    return false;
  *out = static_cast<size_t>(uB * uH * uT * uT * es);
  return true;
}

size_t mu_attention_workspace_bytes_composed(int B, int H, int T, int D, int dtype) {
  (void)D;
  size_t n = 0;
  if (B <= 0 || H <= 0 || T <= 0 || !score_bytes(B, H, T, dtype, &n))
    return 0;
  return n;
}

size_t mu_attention_workspace_bytes(int B, int H, int T, int D, int dtype) {
  if (B <= 0 || H <= 0 || T <= 0)
    return 0;
  // the fused bf16 kernel (head size 64 or 128, T a multiple of 8) needs none
  if (dtype == MU_BF16 && (D == 64 || D == 128) && T % 8 == 0)
    return 0;
  // composed path: one [B*H, T, T] score/probability buffer (softmax runs in place)
  return mu_attention_workspace_bytes_composed(B, H, T, D, dtype);
}

// Used by the executor, not part of the declared ABI: the fused attention kernel writing its
// [B*T, H*D] output with row stride `out_ld` (a column slab of a wider tensor) and, from inside the
// kernel, a second copy to `out_mirror` (same layout; may be a peer GPU's memory). bfloat16 and
// head sizes 64 / 128 only: there is no composed path behind it.
int mu_attention_mirrored(mu_ctx *ctx, const void *q, const void *k, const void *v, void *out, long long out_ld,
                          void *out_mirror, int B, int H, int T, int D, int causal, int kmode, int dtype,
                          void *stream) {
  if (!ctx)
    return MU_ERR_INVALID;
  MU_REQUIRE(B > 0 && H > 0 && T > 0 && D > 0 && q && k && v && out, "attention: bad arguments");
  MU_REQUIRE(kmode == MU_K_LITERAL || kmode == MU_K_MATH, "attention: unknown kmode %d", kmode);
  if (dtype != MU_BF16 || ctx->force_simt)
    return fail(ctx, MU_ERR_UNSUPPORTED, "attention with a mirrored output needs the bfloat16 tensor-core kernel");
  if (!set_device(ctx))
    return fail(ctx, MU_ERR_CUDA, "attention: cannot select device %d", ctx->device);
  const int rc = mu::launch_attention_tcgen05_ex(q, k, v, out, out_ld, out_mirror, B, H, T, D, causal,
                                                 kmode == MU_K_LITERAL ? 1 : 0, ctx->d_status,
                                                 static_cast<cudaStream_t>(stream));
  if (rc == 2)
    return cuda_fail(ctx, "attention", cudaGetLastError());
  if (rc)
    return fail(ctx, MU_ERR_UNSUPPORTED, "attention with a mirrored output: head size %d, T %d or the "
                "alignment is outside the fused kernel's envelope", D, T);
  return MU_OK;
}

int mu_attention(mu_ctx *ctx, const void *q, const void *k, const void *v, void *out, int B, int H,
                 int T, int D, int causal, int kmode, int dtype, void *workspace,
                 size_t workspace_bytes, void *stream) {
  if (!ctx)
    return MU_ERR_INVALID;
  MU_REQUIRE(B >= 0 && H > 0 && T >= 0 && D > 0, "attention: bad dimensions");
  MU_REQUIRE(kmode == MU_K_LITERAL || kmode == MU_K_MATH, "attention: unknown kmode %d", kmode);
  if (dtype != MU_F32 && dtype != MU_BF16)
    return fail(ctx, MU_ERR_UNSUPPORTED, "attention: dtype %d not implemented", dtype);
  if (B == 0 || T == 0)
    return MU_OK;
  MU_REQUIRE(q && k && v && out, "attention: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (!set_device(ctx))
    return fail(ctx, MU_ERR_CUDA, "attention: cannot select device %d", ctx->device);
  if (dtype == MU_BF16 && !ctx->force_simt) {
    // fused tcgen05 kernel: scores and probabilities stay on chip, no workspace
    int rc = mu::launch_attention_tcgen05(q, k, v, out, B, H, T, D, causal,
                                          kmode == MU_K_LITERAL ? 1 : 0, ctx->d_status, st);
    if (rc == 0)
      return MU_OK;
    if (rc == 2)
      return cuda_fail(ctx, "attention", cudaGetLastError());
  }
  // composed path (any head size, float32): batched GEMM → softmax → batched GEMM
  size_t need = 0;
  if (!score_bytes(B, H, T, dtype, &need))
    return fail(ctx, MU_ERR_SIZE, "attention: B=%d H=%d T=%d is beyond what the kernels can index", B,
                H, T);
  MU_REQUIRE(workspace && workspace_bytes >= need,
             "attention: workspace too small (%zu < %zu bytes)", workspace_bytes, need);
  const int BH = B * H;
  const long long Ntot = 1ll * BH * T;
  const int E = H * D;
  // S = scale * Q·K'   (scale is a separately rounded multiply in the reference)
  {
    mu::GemmOperands op;
    op.a = q, op.lda = D, op.a_batch = 1ll * T * D;
    op.b = k;
    if (kmode == MU_K_LITERAL) {
      // K's [N,D] buffer read as row-major [D,N]; head block bh = columns bh*T..
      op.b_kmajor = 0, op.ldb = Ntot, op.b_batch = T, op.b_col_per_batch = T;
    } else {
      op.b_kmajor = 1, op.ldb = D, op.b_batch = 1ll * T * D;
    }
    mu::GemmShape sh{T, T, D, BH};
    mu::Epilogue ep;
    ep.c = workspace, ep.ldc = T, ep.batch_hi = 1ll * T * T, ep.batch_div = 1;
    ep.alpha = 1.0f / sqrtf(static_cast<float>(D));
    ep.round_each = 1;
    int rc = run_gemm(ctx, op, sh, ep, dtype, st, "attention(scores)");
    if (rc)
      return rc;
  }
  int rc = mu::launch_softmax(workspace, workspace, Ntot, T, 1.0f, causal ? T : 0, 0, dtype, st);
  if (rc)
    return cuda_fail(ctx, "attention(softmax)", cudaGetLastError());
  {
    mu::GemmOperands op;
    op.a = workspace, op.lda = T, op.a_batch = 1ll * T * T;
    op.b = v, op.b_kmajor = 0, op.ldb = D, op.b_batch = 1ll * T * D;
    mu::GemmShape sh{T, D, T, BH};
    mu::Epilogue ep;
    ep.c = out, ep.ldc = E, ep.batch_div = H, ep.batch_hi = 1ll * T * E, ep.batch_lo = D;
    ep.round_each = 1;
    return run_gemm(ctx, op, sh, ep, dtype, st, "attention(context)");
  }
}

int mu_layer_norm(mu_ctx *ctx, const void *x, const void *gamma, const void *beta, void *y,
                  long long rows, int cols, float eps, int dtype, void *stream) {
  if (!ctx)
    return MU_ERR_INVALID;
  MU_REQUIRE(rows >= 0 && cols > 0, "LayerNorm: input must have at least 1 dim");
  if (rows == 0)
    return MU_OK;
  MU_REQUIRE(x && gamma && beta && y, "LayerNorm: null pointer");
  if (!set_device(ctx))
    return fail(ctx, MU_ERR_CUDA, "LayerNorm: cannot select device");
  int rc = mu::launch_layer_norm(x, gamma, beta, y, rows, cols, eps, dtype, ctx->d_status, ctx->num_sms,
                                 static_cast<cudaStream_t>(stream));
  if (rc == 1)
    return fail(ctx, MU_ERR_UNSUPPORTED, "LayerNorm: dtype %d not implemented", dtype);
  return rc ? cuda_fail(ctx, "LayerNorm", cudaGetLastError()) : MU_OK;
}

int mu_softmax(mu_ctx *ctx, const void *x, void *y, long long rows, int cols, int dtype,
               void *stream) {
  if (!ctx)
    return MU_ERR_INVALID;
  MU_REQUIRE(rows >= 0 && cols > 0, "Softmax expects non-empty shape");
  if (rows == 0)
    return MU_OK;
  MU_REQUIRE(x && y, "Softmax: null pointer");
  if (!set_device(ctx))
    return fail(ctx, MU_ERR_CUDA, "Softmax: cannot select device");
  int rc = 1;
  if (dtype == MU_BF16) // model widths: persistent kernel on a shared-memory ring
    rc = mu::launch_softmax_bf16_rows(x, y, rows, cols, 1.0f, 0, 0, ctx->d_status, ctx->num_sms,
                                      static_cast<cudaStream_t>(stream));
  if (rc == 1)
    rc = mu::launch_softmax(x, y, rows, cols, 1.0f, 0, 0, dtype, static_cast<cudaStream_t>(stream));
  if (rc == 1)
    return fail(ctx, MU_ERR_UNSUPPORTED, "Softmax: dtype %d not implemented", dtype);
  return rc ? cuda_fail(ctx, "Softmax", cudaGetLastError()) : MU_OK;
}

int mu_embedding(mu_ctx *ctx, const int32_t *ids, const void *table, const void *pos, void *out,
                 int B, int T, int V, int D, int dtype, void *stream) {
  if (!ctx)
    return MU_ERR_INVALID;
  MU_REQUIRE(V > 0 && D > 0, "Embedding expects positive num_embeddings and embedding_dim");
  MU_REQUIRE(B >= 0 && T >= 0, "Embedding: negative dimension");
  if (B == 0 || T == 0)
    return MU_OK;
  MU_REQUIRE(ids && table && out, "Embedding: null pointer");
  if (!set_device(ctx))
    return fail(ctx, MU_ERR_CUDA, "Embedding: cannot select device");
  int rc = mu::launch_embedding(ids, table, pos, out, 1ll * B * T, T, V, D, dtype, ctx->d_status,
                                static_cast<cudaStream_t>(stream));
  if (rc == 1)
    return fail(ctx, MU_ERR_UNSUPPORTED, "Embedding: dtype %d not implemented", dtype);
  return rc ? cuda_fail(ctx, "Embedding", cudaGetLastError()) : MU_OK;
}

int mu_eltwise(mu_ctx *ctx, const void *x, const void *bias, const void *residual, void *y,
               long long n, int cols, int act, int dtype, void *stream) {
  if (!ctx)
    return MU_ERR_INVALID;
  MU_REQUIRE(n >= 0, "eltwise: negative size");
  MU_REQUIRE(act >= MU_ACT_NONE && act <= MU_ACT_TANH, "eltwise: unknown activation %d", act);
  if (n == 0)
    return MU_OK;
  MU_REQUIRE(x && y, "eltwise: null pointer");
  MU_REQUIRE(!bias || cols > 0, "eltwise: bias needs cols > 0");
  if (!set_device(ctx))
    return fail(ctx, MU_ERR_CUDA, "eltwise: cannot select device");
  int rc = mu::launch_eltwise(x, bias, residual, y, n, cols, act, dtype, ctx->num_sms,
                              static_cast<cudaStream_t>(stream));
  if (rc == 1)
    return fail(ctx, MU_ERR_UNSUPPORTED, "eltwise: dtype %d not implemented", dtype);
  return rc ? cuda_fail(ctx, "eltwise", cudaGetLastError()) : MU_OK;
}

int mu_argmax(mu_ctx *ctx, const void *x, int32_t *idx, long long rows, int cols, int dtype,
              void *stream) {
  if (!ctx)
    return MU_ERR_INVALID;
  MU_REQUIRE(rows >= 0 && cols > 0, "argmax: bad shape");
  if (rows == 0)
    return MU_OK;
  MU_REQUIRE(x && idx, "argmax: null pointer");
  if (!set_device(ctx))
    return fail(ctx, MU_ERR_CUDA, "argmax: cannot select device");
  int rc = mu::launch_argmax(x, idx, rows, cols, dtype, static_cast<cudaStream_t>(stream));
  if (rc == 1)
    return fail(ctx, MU_ERR_UNSUPPORTED, "argmax: dtype %d not implemented", dtype);
  return rc ? cuda_fail(ctx, "argmax", cudaGetLastError()) : MU_OK;
}

} // extern "C"
