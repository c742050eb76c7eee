/* TEST INFRASTRUCTURE ONLY — a CPU restatement of the MuNet forward-inference
 * arithmetic, used by tests/, __graft_entry__.smoke() and bench.py's CPU leg as
 * the parity checker.  The product library never links or calls this file.
 *
 * Parity status: PINNED.  Every function here is checked bit-for-bit against
 * the unmodified reference CPU core (oracle/_ref/libmunet_ref.so, built by
 * oracle/Makefile) in tests/test_oracle_vs_ref.py, and against the
 * known-answer values the reference's own tests hold (tests/test_oracle_kat.py).
 *
 * Paths are given relative to the reference checkout.
 *
 * dtype codes follow src/types.hpp:16 — 0 float32, 2 bfloat16 (3 int32 for ids).
 *
 * Two arithmetic regimes exist in the reference and both are restated:
 *   float32  — CPUBackend kernels: float multiply/add, sequential reduction
 *              (src/backend/cpu_backend.hpp), LayerNorm/softmax in double.
 *   bfloat16 — "typed fallback" loops: every scalar is widened to double, the
 *              op is evaluated in double and the result is rounded
 *              double→float→bf16 (RNE, src/types.hpp:311-317) after EVERY op
 *              (src/core/ops/common.hpp:46-85,128-165).
 *
 * Loops are parallelised with OpenMP over independent outputs only; each
 * output's reduction order is the reference's, so results do not depend on
 * the thread count.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

enum { DT_F32 = 0, DT_BF16 = 2 };
enum { ACT_NONE = 0, ACT_RELU = 1, ACT_GELU = 2, ACT_SIGMOID = 3, ACT_TANH = 4 };
enum { K_LITERAL = 0, K_MATH = 1 };

/* ---- bf16 <-> float, src/types.hpp:311-324 ---- */
static inline uint16_t f2bf(float v) {
  uint32_t bits;
  memcpy(&bits, &v, 4);
  uint32_t lsb = (bits >> 16) & 1u;
  bits += 0x7fffu + lsb;
  return (uint16_t)(bits >> 16);
}
static inline float bf2f(uint16_t v) {
  uint32_t bits = (uint32_t)v << 16;
  float out;
  memcpy(&out, &bits, 4);
  return out;
}
/* write_scalar_to_buffer(BFloat16, double): double → float → bf16 */
static inline uint16_t d2bf(double v) { return f2bf((float)v); }
static inline double bf2d(uint16_t v) { return (double)bf2f(v); }

/* ---- diagnostic variants (NOT the parity reference) ----
 * orc_set_variant(0), the default, is the pinned restatement of the reference. The bits below
 * swap one piece of its bfloat16 arithmetic for what a tensor-core kernel does instead, so that
 * how far two valid evaluation orders of the same bf16 pipeline drift apart can be measured on
 * the CPU, without any kernel in the loop:
 *   1  contractions (matmul, Q.K', P.V) accumulate in float instead of double
 *   2  attention rounds the UNNORMALISED probabilities exp(s - max) to bf16 before P.V and
 *      divides the float result by the float row sum (online-softmax order) instead of
 *      rounding the normalised probabilities (the reference's order)
 * Tests that compare a kernel with the checker always run variant 0. */
static int g_variant = 0;
void orc_set_variant(int flags) { g_variant = flags; }
int orc_get_variant(void) { return g_variant; }

uint16_t orc_float_to_bf16(float v) { return f2bf(v); }
float orc_bf16_to_float(uint16_t v) { return bf2f(v); }

/* ---- matmul: C[M,N] = A[M,K]·B[K,N] ----
 * float32: src/backend/cpu_backend.hpp:361-373 (float sum, k sequential)
 * bfloat16: src/core/ops/common.hpp:128-165 (double sum, one rounding) */
static void matmul_f32(const float *a, const float *b, float *c, int M, int K,
                       int N) {
#pragma omp parallel for schedule(static)
  for (int m = 0; m < M; ++m) {
    float *row = c + (size_t)m * N;
    for (int n = 0; n < N; ++n)
      row[n] = 0.0f;
    for (int k = 0; k < K; ++k) {
      const float av = a[(size_t)m * K + k];
      const float *br = b + (size_t)k * N;
      for (int n = 0; n < N; ++n)
        row[n] = row[n] + av * br[n];
    }
  }
}

static void matmul_bf16_facc(const uint16_t *a, const uint16_t *b, uint16_t *c,
                             int M, int K, int N) {
#pragma omp parallel
  {
    float *acc = (float *)malloc(sizeof(float) * (size_t)N);
#pragma omp for schedule(static)
    for (int m = 0; m < M; ++m) {
      for (int n = 0; n < N; ++n)
        acc[n] = 0.0f;
      for (int k = 0; k < K; ++k) {
        const float av = bf2f(a[(size_t)m * K + k]);
        const uint16_t *br = b + (size_t)k * N;
        for (int n = 0; n < N; ++n)
          acc[n] = acc[n] + av * bf2f(br[n]);
      }
      for (int n = 0; n < N; ++n)
        c[(size_t)m * N + n] = f2bf(acc[n]);
    }
    free(acc);
  }
}

static void matmul_bf16(const uint16_t *a, const uint16_t *b, uint16_t *c,
                        int M, int K, int N) {
  if (g_variant & 1) {
    matmul_bf16_facc(a, b, c, M, K, N);
    return;
  }
  double *bd = (double *)malloc(sizeof(double) * (size_t)K * N);
  for (size_t i = 0; i < (size_t)K * N; ++i)
    bd[i] = bf2d(b[i]);
#pragma omp parallel
  {
    double *acc = (double *)malloc(sizeof(double) * (size_t)N);
#pragma omp for schedule(static)
    for (int m = 0; m < M; ++m) {
      for (int n = 0; n < N; ++n)
        acc[n] = 0.0;
      for (int k = 0; k < K; ++k) {
        const double av = bf2d(a[(size_t)m * K + k]);
        const double *br = bd + (size_t)k * N;
        for (int n = 0; n < N; ++n)
          acc[n] = acc[n] + av * br[n];
      }
      for (int n = 0; n < N; ++n)
        c[(size_t)m * N + n] = d2bf(acc[n]);
    }
    free(acc);
  }
  free(bd);
}

int orc_matmul(const void *a, const void *b, void *c, int M, int K, int N,
               int dtype) {
  if (dtype == DT_F32)
    matmul_f32((const float *)a, (const float *)b, (float *)c, M, K, N);
  else if (dtype == DT_BF16)
    matmul_bf16((const uint16_t *)a, (const uint16_t *)b, (uint16_t *)c, M, K, N);
  else
    return 1;
  return 0;
}

/* ---- activations as the reference's module compositions ----
 * ReLU  src/backend/cpu_backend.hpp:493-500 / std::max(v,0.0)
 * Sigmoid cpu_backend.hpp:513-520 (float expf) / 1/(1+exp(-v)) in double
 * GELU  = x * sigmoid(x * c), c = 1.702 stored in the tensor dtype
 *         (src/nn/activations.hpp:31-38) — three separately rounded ops
 * Tanh  = sigmoid(x*2)*2 - 1 (src/nn/activations.hpp:20-29) */
static inline float sigmoid_f32(float x) { return 1.0f / (1.0f + expf(-x)); }
static inline uint16_t sigmoid_bf16(uint16_t x) {
  return d2bf(1.0 / (1.0 + exp(-bf2d(x))));
}
static inline uint16_t mul_bf16(uint16_t a, uint16_t b) {
  return d2bf(bf2d(a) * bf2d(b));
}
static inline uint16_t add_bf16(uint16_t a, uint16_t b) {
  return d2bf(bf2d(a) + bf2d(b));
}
static inline uint16_t sub_bf16(uint16_t a, uint16_t b) {
  return d2bf(bf2d(a) - bf2d(b));
}

static inline float act_f32(float x, int act) {
  switch (act) {
  case ACT_RELU:
    return x > 0 ? x : 0;
  case ACT_GELU: {
    const float c = 1.702f;
    float t = x * c;
    return x * sigmoid_f32(t);
  }
  case ACT_SIGMOID:
    return sigmoid_f32(x);
  case ACT_TANH: {
    float t = x * 2.0f;
    return sigmoid_f32(t) * 2.0f - 1.0f;
  }
  default:
    return x;
  }
}

static inline uint16_t act_bf16(uint16_t x, int act) {
  switch (act) {
  case ACT_RELU: {
    double v = bf2d(x);
    return d2bf(v > 0.0 ? v : 0.0);
  }
  case ACT_GELU: {
    const uint16_t c = f2bf(1.702f);
    return mul_bf16(x, sigmoid_bf16(mul_bf16(x, c)));
  }
  case ACT_SIGMOID:
    return sigmoid_bf16(x);
  case ACT_TANH: {
    const uint16_t two = f2bf(2.0f), one = f2bf(1.0f);
    return sub_bf16(mul_bf16(sigmoid_bf16(mul_bf16(x, two)), two), one);
  }
  default:
    return x;
  }
}

int orc_activation(const void *x, void *y, long n, int dtype, int act) {
  if (dtype == DT_F32) {
    const float *xp = (const float *)x;
    float *yp = (float *)y;
#pragma omp parallel for schedule(static)
    for (long i = 0; i < n; ++i)
      yp[i] = act_f32(xp[i], act);
  } else if (dtype == DT_BF16) {
    const uint16_t *xp = (const uint16_t *)x;
    uint16_t *yp = (uint16_t *)y;
#pragma omp parallel for schedule(static)
    for (long i = 0; i < n; ++i)
      yp[i] = act_bf16(xp[i], act);
  } else
    return 1;
  return 0;
}

/* residual add, same shape: cpu_backend.hpp:246-254 / typed binary fallback */
int orc_add(const void *a, const void *b, void *y, long n, int dtype) {
  if (dtype == DT_F32) {
    const float *ap = (const float *)a, *bp = (const float *)b;
    float *yp = (float *)y;
#pragma omp parallel for schedule(static)
    for (long i = 0; i < n; ++i)
      yp[i] = ap[i] + bp[i];
  } else if (dtype == DT_BF16) {
    const uint16_t *ap = (const uint16_t *)a, *bp = (const uint16_t *)b;
    uint16_t *yp = (uint16_t *)y;
#pragma omp parallel for schedule(static)
    for (long i = 0; i < n; ++i)
      yp[i] = add_bf16(ap[i], bp[i]);
  } else
    return 1;
  return 0;
}

/* ---- nn::Linear (+ activation module): y = act(x·W + b), W is [K,N]
 * src/nn/linear.hpp:28-34; the bias add is a second, separately rounded op. */
int orc_linear(const void *x, const void *w, const void *b, void *y, int M,
               int K, int N, int dtype, int act) {
  if (orc_matmul(x, w, y, M, K, N, dtype))
    return 1;
  if (dtype == DT_F32) {
    float *yp = (float *)y;
    const float *bp = (const float *)b;
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m)
      for (int n = 0; n < N; ++n) {
        float v = yp[(size_t)m * N + n];
        if (bp)
          v = v + bp[n];
        yp[(size_t)m * N + n] = act_f32(v, act);
      }
  } else {
    uint16_t *yp = (uint16_t *)y;
    const uint16_t *bp = (const uint16_t *)b;
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m)
      for (int n = 0; n < N; ++n) {
        uint16_t v = yp[(size_t)m * N + n];
        if (bp)
          v = add_bf16(v, bp[n]);
        yp[(size_t)m * N + n] = act_bf16(v, act);
      }
  }
  return 0;
}

/* ---- LayerNorm: src/core/ops/normalization.cpp:172-206 (all dtypes in double,
 * biased variance, eps inside the sqrt, eps is a float widened to double) ---- */
int orc_layer_norm(const void *x, const void *g, const void *b, void *y,
                   int rows, int cols, float eps, int dtype) {
  if (dtype != DT_F32 && dtype != DT_BF16)
    return 1;
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r) {
    double mean = 0.0;
    for (int c = 0; c < cols; ++c) {
      size_t i = (size_t)r * cols + c;
      mean += dtype == DT_F32 ? (double)((const float *)x)[i]
                              : bf2d(((const uint16_t *)x)[i]);
    }
    mean /= cols;
    double var = 0.0;
    for (int c = 0; c < cols; ++c) {
      size_t i = (size_t)r * cols + c;
      double xv = dtype == DT_F32 ? (double)((const float *)x)[i]
                                  : bf2d(((const uint16_t *)x)[i]);
      double d = xv - mean;
      var += d * d;
    }
    var /= cols;
    const double inv = 1.0 / sqrt(var + eps);
    for (int c = 0; c < cols; ++c) {
      size_t i = (size_t)r * cols + c;
      if (dtype == DT_F32) {
        double xv = ((const float *)x)[i];
        double xhat = (xv - mean) * inv;
        ((float *)y)[i] = (float)(xhat * (double)((const float *)g)[c] +
                                  (double)((const float *)b)[c]);
      } else {
        double xv = bf2d(((const uint16_t *)x)[i]);
        double xhat = (xv - mean) * inv;
        ((uint16_t *)y)[i] = d2bf(xhat * bf2d(((const uint16_t *)g)[c]) +
                                  bf2d(((const uint16_t *)b)[c]));
      }
    }
  }
  return 0;
}

/* ---- row softmax over the last dim ----
 * float32: cpu_backend.hpp:587-611 (float max, double exp/sum, float result)
 * bfloat16: src/core/ops/activations.cpp:211-243 (all double) */
int orc_softmax(const void *x, void *y, int rows, int cols, int dtype) {
  if (dtype != DT_F32 && dtype != DT_BF16)
    return 1;
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r) {
    if (dtype == DT_F32) {
      const float *in = (const float *)x + (size_t)r * cols;
      float *out = (float *)y + (size_t)r * cols;
      float mx = in[0];
      for (int i = 1; i < cols; ++i)
        if (in[i] > mx)
          mx = in[i];
      double s = 0.0;
      for (int i = 0; i < cols; ++i)
        s += exp((double)in[i] - (double)mx);
      for (int i = 0; i < cols; ++i)
        out[i] = (float)(exp((double)in[i] - (double)mx) / s);
    } else {
      const uint16_t *in = (const uint16_t *)x + (size_t)r * cols;
      uint16_t *out = (uint16_t *)y + (size_t)r * cols;
      double mx = bf2d(in[0]);
      for (int i = 1; i < cols; ++i) {
        double v = bf2d(in[i]);
        mx = mx < v ? v : mx;
      }
      double s = 0.0;
      for (int i = 0; i < cols; ++i)
        s += exp(bf2d(in[i]) - mx);
      for (int i = 0; i < cols; ++i)
        out[i] = d2bf(exp(bf2d(in[i]) - mx) / s);
    }
  }
  return 0;
}

/* ---- attention core on head-major q,k,v [BH·T, D] → ctx [BH·T, D] ----
 * Block-wise restatement of src/nn/attention.hpp:64-94.  The reference forms
 * the full [N,N] score matrix (N = BH·T), fills every entry outside the row's
 * own head block (and, if causal, every later position) with -1e9 and runs a
 * full-row softmax.  Those entries become exp(-1e9 - max) == 0.0 exactly, and
 * adding 0.0 terms changes neither the softmax sum nor the P·V sum, so only
 * the unmasked entries of each row are evaluated here, in the same order.
 *
 * kmode K_LITERAL reproduces what the reference computes: `k.transpose(0,1)`
 * only swaps shape/strides (src/tensor.cpp:420-426) and matmul ignores strides
 * (src/core/ops/matmul.cpp:331-392), so the score is
 *     S[i,j] = sum_d Q[i,d] * Kbuf[d*N + j]
 * i.e. K's [N,D] buffer read as a row-major [D,N] matrix.
 * kmode K_MATH is the textbook S[i,j] = sum_d Q[i,d] * K[j,d].
 * Scale 1/sqrt(D) is a float stored in the tensor dtype and applied as a
 * separate multiply before masking. */
int orc_attention_core(const void *q, const void *k, const void *v, void *ctx,
                       int BH, int T, int D, int causal, int dtype, int kmode) {
  if (dtype != DT_F32 && dtype != DT_BF16)
    return 1;
  const long N = (long)BH * T;
  const float scale_f = 1.0f / sqrtf((float)D);
  const uint16_t scale_b = f2bf(scale_f);
#pragma omp parallel
  {
    double *p = (double *)malloc(sizeof(double) * (size_t)T);
    float *sf = (float *)malloc(sizeof(float) * (size_t)T);
    double *acc = (double *)malloc(sizeof(double) * (size_t)D);
#pragma omp for schedule(dynamic, 16)
    for (long i = 0; i < N; ++i) {
      const long blk = i / T;
      const int ti = (int)(i % T);
      const int cnt = causal ? ti + 1 : T; /* unmasked columns blk*T .. +cnt-1 */
      const long j0 = blk * T;
      if (dtype == DT_F32) {
        const float *Q = (const float *)q, *K = (const float *)k,
                    *V = (const float *)v;
        float mx = 0;
        for (int jj = 0; jj < cnt; ++jj) {
          const long j = j0 + jj;
          float s = 0.0f;
          for (int d = 0; d < D; ++d) {
            float kv = kmode == K_LITERAL ? K[(size_t)d * N + j]
                                          : K[(size_t)j * D + d];
            s += Q[(size_t)i * D + d] * kv;
          }
          s = s * scale_f;
          sf[jj] = s;
          if (jj == 0 || s > mx)
            mx = s;
        }
        /* masked entries hold -1e9f; they only matter for the max if every
         * unmasked score is below it, which the fill value rules out */
        double sum = 0.0;
        for (int jj = 0; jj < cnt; ++jj)
          sum += exp((double)sf[jj] - (double)mx);
        for (int jj = 0; jj < cnt; ++jj)
          sf[jj] = (float)(exp((double)sf[jj] - (double)mx) / sum);
        float *out = (float *)ctx + (size_t)i * D;
        for (int d = 0; d < D; ++d) {
          float s = 0.0f;
          for (int jj = 0; jj < cnt; ++jj)
            s += sf[jj] * V[(size_t)(j0 + jj) * D + d];
          out[d] = s;
        }
      } else {
        const uint16_t *Q = (const uint16_t *)q, *K = (const uint16_t *)k,
                       *V = (const uint16_t *)v;
        double mx = 0;
        for (int jj = 0; jj < cnt; ++jj) {
          const long j = j0 + jj;
          double s = 0.0;
          for (int d = 0; d < D; ++d) {
            uint16_t kv = kmode == K_LITERAL ? K[(size_t)d * N + j]
                                             : K[(size_t)j * D + d];
            s += bf2d(Q[(size_t)i * D + d]) * bf2d(kv);
          }
          if (g_variant & 1) { /* diagnostic: float accumulation of Q.K' */
            float sfl = 0.0f;
            for (int d = 0; d < D; ++d) {
              uint16_t kv = kmode == K_LITERAL ? K[(size_t)d * N + j]
                                               : K[(size_t)j * D + d];
              sfl += bf2f(Q[(size_t)i * D + d]) * bf2f(kv);
            }
            s = (double)sfl;
          }
          uint16_t sb = mul_bf16(d2bf(s), scale_b);
          p[jj] = bf2d(sb);
          if (jj == 0 || p[jj] > mx)
            mx = p[jj];
        }
        double sum = 0.0;
        for (int jj = 0; jj < cnt; ++jj)
          sum += exp(p[jj] - mx);
        uint16_t *out = (uint16_t *)ctx + (size_t)i * D;
        if (g_variant & 2) { /* diagnostic: unnormalised P rounded, divide at the end */
          float lsum = 0.0f;
          for (int jj = 0; jj < cnt; ++jj) {
            const float e = (float)exp(p[jj] - mx);
            lsum += e;
            p[jj] = bf2d(f2bf(e));
          }
          for (int d = 0; d < D; ++d)
            acc[d] = 0.0;
          for (int jj = 0; jj < cnt; ++jj) {
            const double pv = p[jj];
            const uint16_t *vr = V + (size_t)(j0 + jj) * D;
            for (int d = 0; d < D; ++d)
              acc[d] = (g_variant & 1) ? (double)((float)acc[d] + (float)pv * bf2f(vr[d]))
                                       : acc[d] + pv * bf2d(vr[d]);
          }
          for (int d = 0; d < D; ++d)
            out[d] = f2bf((float)acc[d] * (1.0f / lsum));
          continue;
        }
        for (int jj = 0; jj < cnt; ++jj)
          p[jj] = bf2d(d2bf(exp(p[jj] - mx) / sum));
        for (int d = 0; d < D; ++d)
          acc[d] = 0.0;
        for (int jj = 0; jj < cnt; ++jj) {
          const double pv = p[jj];
          const uint16_t *vr = V + (size_t)(j0 + jj) * D;
          for (int d = 0; d < D; ++d)
            acc[d] = (g_variant & 1) ? (double)((float)acc[d] + (float)pv * bf2f(vr[d]))
                                     : acc[d] + pv * bf2d(vr[d]);
        }
        for (int d = 0; d < D; ++d)
          out[d] = d2bf(acc[d]);
      }
    }
    free(p);
    free(sf);
    free(acc);
  }
  return 0;
}

static size_t esize(int dtype) { return dtype == DT_F32 ? 4 : 2; }

/* [B,T,H,D] token-major  <->  [B,H,T,D] head-major (permute(0,2,1,3) +
 * contiguous, src/nn/attention.hpp:51-62,96-99) */
static void split_heads(const void *in, void *out, int B, int T, int H, int D,
                        int dtype, int inverse) {
  const size_t es = esize(dtype);
  for (int b = 0; b < B; ++b)
    for (int t = 0; t < T; ++t)
      for (int h = 0; h < H; ++h) {
        size_t tok = (((size_t)b * T + t) * H + h) * D;
        size_t hm = (((size_t)b * H + h) * T + t) * D;
        if (!inverse)
          memcpy((char *)out + hm * es, (const char *)in + tok * es, D * es);
        else
          memcpy((char *)out + tok * es, (const char *)in + hm * es, D * es);
      }
}

/* ---- nn::MultiHeadAttention::forward_impl, src/nn/attention.hpp:34-103 ----
 * params: q.w q.b k.w k.b v.w v.b o.w o.b ; x,y are [B,T,E] */
int orc_mha(const void *x, const void *const *params, void *y, int B, int T,
            int E, int H, int causal, int dtype, int kmode) {
  if (dtype != DT_F32 && dtype != DT_BF16)
    return 1;
  const int D = E / H, M = B * T;
  const size_t bytes = (size_t)M * E * esize(dtype);
  void *t0 = malloc(bytes), *qh = malloc(bytes), *kh = malloc(bytes),
       *vh = malloc(bytes), *ch = malloc(bytes);
  orc_linear(x, params[0], params[1], t0, M, E, E, dtype, ACT_NONE);
  split_heads(t0, qh, B, T, H, D, dtype, 0);
  orc_linear(x, params[2], params[3], t0, M, E, E, dtype, ACT_NONE);
  split_heads(t0, kh, B, T, H, D, dtype, 0);
  orc_linear(x, params[4], params[5], t0, M, E, E, dtype, ACT_NONE);
  split_heads(t0, vh, B, T, H, D, dtype, 0);
  orc_attention_core(qh, kh, vh, ch, B * H, T, D, causal, dtype, kmode);
  split_heads(ch, t0, B, T, H, D, dtype, 1);
  orc_linear(t0, params[6], params[7], y, M, E, E, dtype, ACT_NONE);
  free(t0);
  free(qh);
  free(kh);
  free(vh);
  free(ch);
  return 0;
}

/* ---- nn::Embedding index path, src/nn/linear.hpp:92-131 ----
 * returns 2 on an out-of-range id (the reference throws) */
int orc_embedding(const int32_t *ids, const void *table, void *out, int B,
                  int T, int V, int D, int dtype) {
  const size_t es = esize(dtype);
  for (long i = 0; i < (long)B * T; ++i) {
    int tok = ids[i];
    if (tok < 0 || tok >= V)
      return 2;
    memcpy((char *)out + (size_t)i * D * es,
           (const char *)table + (size_t)tok * D * es, D * es);
  }
  return 0;
}

/* ---- conv2d NCHW, weight [oC,iC,k,k]: cpu_backend.hpp:768-796 (float32) ---- */
int orc_conv2d(const float *x, const float *w, const float *b, float *y, int B,
               int iC, int iH, int iW, int oC, int k, int s, int p) {
  const int oH = (iH + 2 * p - k) / s + 1, oW = (iW + 2 * p - k) / s + 1;
  const long total = (long)B * oC * oH * oW;
#pragma omp parallel for schedule(static)
  for (long idx = 0; idx < total; ++idx) {
    int ow = idx % oW, oh = (idx / oW) % oH, oc = (idx / ((long)oW * oH)) % oC;
    int bb = idx / ((long)oW * oH * oC);
    float val = b ? b[oc] : 0.0f;
    for (int ic = 0; ic < iC; ++ic)
      for (int kh = 0; kh < k; ++kh)
        for (int kw = 0; kw < k; ++kw) {
          int ih = oh * s - p + kh, iw = ow * s - p + kw;
          if (ih >= 0 && ih < iH && iw >= 0 && iw < iW)
            val += x[(((size_t)bb * iC + ic) * iH + ih) * iW + iw] *
                   w[(((size_t)oc * iC + ic) * k + kh) * k + kw];
        }
    y[idx] = val;
  }
  return 0;
}

/* ---- max_pool2d: cpu_backend.hpp:833-855 (initial value -1e9f) ---- */
int orc_max_pool2d(const float *x, float *y, int B, int C, int iH, int iW,
                   int k, int s, int p) {
  const int oH = (iH + 2 * p - k) / s + 1, oW = (iW + 2 * p - k) / s + 1;
  const long total = (long)B * C * oH * oW;
#pragma omp parallel for schedule(static)
  for (long idx = 0; idx < total; ++idx) {
    int ow = idx % oW, oh = (idx / oW) % oH, c = (idx / ((long)oW * oH)) % C;
    int bb = idx / ((long)oW * oH * C);
    float mx = -1e9f;
    for (int kh = 0; kh < k; ++kh)
      for (int kw = 0; kw < k; ++kw) {
        int ih = oh * s - p + kh, iw = ow * s - p + kw;
        if (ih >= 0 && ih < iH && iw >= 0 && iw < iW) {
          float v = x[(((size_t)bb * C + c) * iH + ih) * iW + iw];
          mx = mx < v ? v : mx;
        }
      }
    y[idx] = mx;
  }
  return 0;
}

/* ---- GlobalAvgPool2d: a [B·C,HW]·[HW,1] matmul against a column filled with
 * the float 1/HW (src/nn/pooling.hpp:8-26) ---- */
int orc_global_avg_pool(const float *x, float *y, int B, int C, int H, int W) {
  const int HW = H * W;
  const float scale = 1.0f / (float)HW;
#pragma omp parallel for schedule(static)
  for (long r = 0; r < (long)B * C; ++r) {
    float s = 0.0f;
    for (int i = 0; i < HW; ++i)
      s += x[(size_t)r * HW + i] * scale;
    y[r] = s;
  }
  return 0;
}

/* ---- first-max-index argmax over the last dim (np.argmax rule; the reference
 * has no argmax op, its demos call np.argmax on the logits) ---- */
int orc_argmax(const void *x, int32_t *idx, long rows, int cols, int dtype) {
#pragma omp parallel for schedule(static)
  for (long r = 0; r < rows; ++r) {
    int best = 0;
    float bv = dtype == DT_F32 ? ((const float *)x)[(size_t)r * cols]
                               : bf2f(((const uint16_t *)x)[(size_t)r * cols]);
    for (int c = 1; c < cols; ++c) {
      float v = dtype == DT_F32
                    ? ((const float *)x)[(size_t)r * cols + c]
                    : bf2f(((const uint16_t *)x)[(size_t)r * cols + c]);
      if (v > bv) {
        bv = v;
        best = c;
      }
    }
    idx[r] = best;
  }
  return 0;
}

/* ---- Backend::all_reduce semantic: per element, sum over participants in
 * double, one rounding (src/core/all_reduce_runtime.hpp:85-105) ---- */
int orc_all_reduce_sum(const void *const *bufs, int world, void *out, long n,
                       int dtype) {
  for (long i = 0; i < n; ++i) {
    double s = 0.0;
    for (int r = 0; r < world; ++r)
      s += dtype == DT_F32 ? (double)((const float *)bufs[r])[i]
                           : bf2d(((const uint16_t *)bufs[r])[i]);
    if (dtype == DT_F32)
      ((float *)out)[i] = (float)s;
    else
      ((uint16_t *)out)[i] = d2bf(s);
  }
  return 0;
}

/* ---- GPT-style decoder forward (topology of the reference demo model,
 * demos/multigpu/gpt3_multi_gpu_demo.py:89-172), parameter order:
 *   [0] tok_embed[V,d] [1] pos_embed[T,d]
 *   per layer (16): ln1.w ln1.b q.w q.b k.w k.b v.w v.b o.w o.b ln2.w ln2.b
 *                   fc1.w fc1.b fc2.w fc2.b
 *   then ln_f.w ln_f.b head.w head.b
 * stop_after_layers < 0 → logits [B,T,V]; else hidden [B,T,d] after that many
 * layers. */
int orc_gpt_forward(const int32_t *ids, const void *const *params, void *out,
                    int B, int T, int V, int d, int H, int L, int dtype,
                    int stop_after_layers, int kmode) {
  if (dtype != DT_F32 && dtype != DT_BF16)
    return 1;
  const size_t es = esize(dtype);
  const int M = B * T;
  void *h = malloc((size_t)M * d * es), *t1 = malloc((size_t)M * d * es),
       *t2 = malloc((size_t)M * d * es), *f = malloc((size_t)M * 4 * d * es);
  int rc = orc_embedding(ids, params[0], h, B, T, V, d, dtype);
  if (rc) {
    free(h); free(t1); free(t2); free(f);
    return rc;
  }
  /* h = tok + pos (broadcast over batch) */
  for (int b = 0; b < B; ++b)
    orc_add((char *)h + (size_t)b * T * d * es, params[1],
            (char *)h + (size_t)b * T * d * es, (long)T * d, dtype);
  const int nl = stop_after_layers >= 0 ? stop_after_layers : L;
  for (int l = 0; l < nl; ++l) {
    const void *const *p = params + 2 + 16 * l;
    orc_layer_norm(h, p[0], p[1], t1, M, d, 1e-5f, dtype);
    orc_mha(t1, p + 2, t2, B, T, d, H, 1, dtype, kmode);
    orc_add(h, t2, h, (long)M * d, dtype);
    orc_layer_norm(h, p[10], p[11], t1, M, d, 1e-5f, dtype);
    orc_linear(t1, p[12], p[13], f, M, d, 4 * d, dtype, ACT_GELU);
    orc_linear(f, p[14], p[15], t2, M, 4 * d, d, dtype, ACT_NONE);
    orc_add(h, t2, h, (long)M * d, dtype);
  }
  if (stop_after_layers >= 0) {
    memcpy(out, h, (size_t)M * d * es);
  } else {
    const void *const *p = params + 2 + 16 * L;
    orc_layer_norm(h, p[0], p[1], t1, M, d, 1e-5f, dtype);
    orc_linear(t1, p[2], p[3], out, M, d, V, dtype, ACT_NONE);
  }
  free(h); free(t1); free(t2); free(f);
  return 0;
}

/* ------------------------------------------------------------------------
 * Remaining forward entry points (UNet-style and RMSNorm models).
 * float32 follows the CPU backend's float kernels, bfloat16 the typed fallback
 * (evaluate in double, round double -> float -> bf16 after EVERY op).
 * ---------------------------------------------------------------------- */

/* op: 0 exp, 1 log, 2 sqrt, 3 rsqrt, 4 sin, 5 cos.
 * float32: src/backend/cpu_backend.hpp:533-586; typed: src/core/ops/activations.cpp:66-190. */
int orc_unary(const void *x, void *y, long n, int dtype, int op) {
  if (dtype == DT_F32) {
    const float *a = x;
    float *o = y;
    for (long i = 0; i < n; ++i) {
      float v = a[i];
      o[i] = op == 0 ? expf(v) : op == 1 ? logf(v) : op == 2 ? sqrtf(v)
           : op == 3 ? 1.0f / sqrtf(v) : op == 4 ? sinf(v) : cosf(v);
    }
    return 0;
  }
  if (dtype != DT_BF16)
    return 1;
  const uint16_t *a = x;
  uint16_t *o = y;
  for (long i = 0; i < n; ++i) {
    double v = bf2d(a[i]);
    o[i] = d2bf(op == 0 ? exp(v) : op == 1 ? log(v) : op == 2 ? sqrt(v)
              : op == 3 ? 1.0 / sqrt(v) : op == 4 ? sin(v) : cos(v));
  }
  return 0;
}

/* nn::LeakyReLU, src/nn/activations.hpp:76-88: relu(x) + (x - relu(x)) * slope, the slope
 * held in a one-element tensor of the activation's dtype. */
int orc_leaky_relu(const void *x, void *y, long n, float slope, int dtype) {
  if (dtype == DT_F32) {
    const float *a = x;
    float *o = y;
    for (long i = 0; i < n; ++i) {
      float r = a[i] > 0 ? a[i] : 0;
      float d = a[i] - r;
      float m = d * slope;
      o[i] = r + m;
    }
    return 0;
  }
  if (dtype != DT_BF16)
    return 1;
  const uint16_t *a = x, sl = f2bf(slope);
  uint16_t *o = y;
  for (long i = 0; i < n; ++i) {
    double v = bf2d(a[i]);
    uint16_t r = d2bf(v > 0.0 ? v : 0.0);
    o[i] = add_bf16(r, mul_bf16(sub_bf16(a[i], r), sl));
  }
  return 0;
}

/* nn::RMSNorm, src/nn/normalization.hpp:53-62:
 * variance = mean(x*x, -1); normed = x * rsqrt(variance + eps); out = normed * weight.
 * mean accumulates in double (src/backend/cpu_backend.hpp:1124-1137; typed path
 * src/core/ops/shape.cpp:112-150). */
int orc_rms_norm(const void *x, const void *w, void *y, int rows, int cols, float eps, int dtype) {
  if (dtype == DT_F32) {
    const float *a = x, *g = w;
    float *o = y;
    for (int r = 0; r < rows; ++r) {
      double tot = 0.0;
      for (int c = 0; c < cols; ++c) {
        float sq = a[(size_t)r * cols + c] * a[(size_t)r * cols + c];
        tot += sq;
      }
      float var = (float)(tot / (double)cols);
      float ve = var + eps;
      float rs = 1.0f / sqrtf(ve);
      for (int c = 0; c < cols; ++c) {
        float nm = a[(size_t)r * cols + c] * rs;
        o[(size_t)r * cols + c] = nm * g[c];
      }
    }
    return 0;
  }
  if (dtype != DT_BF16)
    return 1;
  const uint16_t *a = x, *g = w, e = f2bf(eps);
  uint16_t *o = y;
  for (int r = 0; r < rows; ++r) {
    double tot = 0.0;
    for (int c = 0; c < cols; ++c)
      tot += bf2d(mul_bf16(a[(size_t)r * cols + c], a[(size_t)r * cols + c]));
    uint16_t var = d2bf(tot * (1.0 / (double)cols));
    uint16_t ve = add_bf16(var, e);
    uint16_t rs = d2bf(1.0 / sqrt(bf2d(ve)));
    for (int c = 0; c < cols; ++c)
      o[(size_t)r * cols + c] = mul_bf16(mul_bf16(a[(size_t)r * cols + c], rs), g[c]);
  }
  return 0;
}

/* batch_norm, eval branch (src/backend/cpu_backend.hpp:957-967): float arithmetic
 * y = g*(x-mean)*(1/sqrt(var+eps)) + b; bf16 inputs are widened to float and the result is
 * rounded once (src/core/ops/normalization.cpp:32-60). Statistics are float32. */
int orc_batch_norm_eval(const void *x, const void *g, const void *b, const float *mean,
                        const float *var, void *y, int B, int C, int H, int W, float eps,
                        int dtype) {
  if (dtype != DT_F32 && dtype != DT_BF16)
    return 1;
  const size_t spatial = (size_t)H * W, n = (size_t)B * C * spatial;
  for (size_t i = 0; i < n; ++i) {
    int c = (int)((i / spatial) % C);
    float xv, gv, bv;
    if (dtype == DT_F32) {
      xv = ((const float *)x)[i], gv = ((const float *)g)[c], bv = ((const float *)b)[c];
    } else {
      xv = bf2f(((const uint16_t *)x)[i]), gv = bf2f(((const uint16_t *)g)[c]),
      bv = bf2f(((const uint16_t *)b)[c]);
    }
    float inv_std = 1.0f / sqrtf(var[c] + eps);
    float d = xv - mean[c];
    float t = gv * d;
    float u = t * inv_std;
    float r = u + bv;
    if (dtype == DT_F32)
      ((float *)y)[i] = r;
    else
      ((uint16_t *)y)[i] = f2bf(r);
  }
  return 0;
}

/* sum of every element: float32 adds sequentially in float (src/backend/cpu_backend.hpp:1040-1049),
 * the typed path accumulates in double (src/core/ops/shape.cpp:56-66). */
int orc_sum(const void *x, void *out, long n, int dtype) {
  if (dtype == DT_F32) {
    float tot = 0.0f;
    for (long i = 0; i < n; ++i)
      tot += ((const float *)x)[i];
    *(float *)out = tot;
    return 0;
  }
  if (dtype != DT_BF16)
    return 1;
  double tot = 0.0;
  for (long i = 0; i < n; ++i)
    tot += bf2d(((const uint16_t *)x)[i]);
  *(uint16_t *)out = d2bf(tot);
  return 0;
}

/* mean over the last dimension, double accumulation in both paths
 * (src/backend/cpu_backend.hpp:1124-1137; src/core/ops/shape.cpp:112-155). */
int orc_mean_last_dim(const void *x, void *out, int outer, int dim, int dtype) {
  if (dtype != DT_F32 && dtype != DT_BF16)
    return 1;
  for (int r = 0; r < outer; ++r) {
    double tot = 0.0;
    for (int c = 0; c < dim; ++c)
      tot += dtype == DT_F32 ? (double)((const float *)x)[(size_t)r * dim + c]
                             : bf2d(((const uint16_t *)x)[(size_t)r * dim + c]);
    if (dtype == DT_F32)
      ((float *)out)[r] = (float)(tot / (double)dim);
    else
      ((uint16_t *)out)[r] = d2bf(tot * (1.0 / (double)dim));
  }
  return 0;
}
