// TEST INFRASTRUCTURE ONLY — never linked into the product library.
//
// A thin extern "C" driver over the UNMODIFIED MuNet CPU core.  The build
// recipe (oracle/Makefile, target `ref`) compiles this file together with the
// reference's own translation units, taken where they lie in the reference
// checkout (include path = its `src/`), into oracle/_ref/libmunet_ref.so.
// Nothing from the reference is copied into this repository: this file only
// *calls* the reference API (Tensor, nn::*, inference::Engine).
//
// Every entry point takes plain host pointers.  `dtype` follows the reference
// enum order (src/types.hpp:16): 0 = float32, 1 = float16, 2 = bfloat16,
// 3 = int32.  16-bit buffers are raw uint16 bit patterns.
// Return value: 0 on success, 1 on a C++ exception (text in ref_last_error()).

#include "inference.hpp"
#include "nn.hpp"
#include "tensor.hpp"
#include "core/all_reduce_runtime.hpp"

#include <cstring>
#include <memory>
#include <string>
#include <thread>
#include <vector>

using namespace munet;

namespace {

thread_local std::string g_err;

const Device kCpu{DeviceType::CPU, 0};

DataType dt(int code) { return static_cast<DataType>(code); }

Tensor from_host(const void *p, Shape shape, int dtype) {
  Tensor t(shape, kCpu, dt(dtype), false);
  if (t.bytes())
    std::memcpy(t.data(), p, t.bytes());
  return t;
}

void to_host(const Tensor &t, void *dst) {
  Tensor c = t.is_contiguous() ? t : t.contiguous();
  if (c.bytes())
    std::memcpy(dst, c.data(), c.bytes());
}

void set_param(Tensor &param, const void *src) {
  if (param.bytes())
    std::memcpy(param.data(), src, param.bytes());
  param.set_requires_grad(false);
}

std::shared_ptr<nn::Linear> make_linear(int in, int out, const void *w,
                                        const void *b, int dtype) {
  TensorOptions opt(kCpu, dt(dtype), false);
  auto lin = std::make_shared<nn::Linear>(in, out, b != nullptr, opt);
  set_param(lin->weight, w);
  if (b)
    set_param(lin->bias, b);
  lin->eval();
  return lin;
}

std::shared_ptr<nn::LayerNorm> make_ln(int d, const void *g, const void *b,
                                       float eps, int dtype) {
  TensorOptions opt(kCpu, dt(dtype), false);
  auto ln = std::make_shared<nn::LayerNorm>(d, eps, opt);
  set_param(ln->weight, g);
  set_param(ln->bias, b);
  ln->eval();
  return ln;
}

// params: q.w q.b k.w k.b v.w v.b o.w o.b
std::shared_ptr<nn::MultiHeadAttention>
make_mha(int E, int H, bool causal, const void *const *p, int dtype) {
  TensorOptions opt(kCpu, dt(dtype), false);
  auto mha = std::make_shared<nn::MultiHeadAttention>(E, H, causal, opt);
  auto named = mha->named_parameters("");
  const char *names[8] = {"q_proj.weight", "q_proj.bias",   "k_proj.weight",
                          "k_proj.bias",   "v_proj.weight", "v_proj.bias",
                          "out_proj.weight", "out_proj.bias"};
  for (int i = 0; i < 8; ++i) {
    Tensor t = named.at(names[i]);
    std::memcpy(t.data(), p[i], t.bytes());
  }
  for (auto &[name, t] : named) {
    Tensor tt = t;
    tt.set_requires_grad(false);
  }
  mha->eval();
  return mha;
}

Tensor apply_act(Tensor y, int act) {
  if (act == 1)
    return nn::ReLU().forward(y);
  if (act == 2)
    return nn::GELU().forward(y);
  if (act == 3)
    return nn::Sigmoid().forward(y);
  if (act == 4)
    return nn::Tanh().forward(y);
  return y;
}

template <typename Fn> int guarded(Fn &&fn) {
  try {
    inference::detail::InferenceModeGuard guard;
    fn();
    return 0;
  } catch (const std::exception &e) {
    g_err = e.what();
    return 1;
  } catch (...) {
    g_err = "unknown exception";
    return 1;
  }
}

} // namespace

extern "C" {

const char *ref_last_error() { return g_err.c_str(); }

int ref_hardware_concurrency() {
  return static_cast<int>(std::thread::hardware_concurrency());
}

// y[M,N] = act(x[M,K] · w[K,N] + b[N]) through nn::Linear (+ activation module).
int ref_linear(const void *x, const void *w, const void *b, void *y, int M,
               int K, int N, int dtype, int act) {
  return guarded([&] {
    auto lin = make_linear(K, N, w, b, dtype);
    Tensor out = apply_act(lin->forward(from_host(x, {M, K}, dtype)), act);
    to_host(out, y);
  });
}

// Raw 2-D matmul C[M,N] = A[M,K]·B[K,N] through Tensor::matmul.
int ref_matmul(const void *a, const void *b, void *c, int M, int K, int N,
               int dtype) {
  return guarded([&] {
    Tensor out =
        from_host(a, {M, K}, dtype).matmul(from_host(b, {K, N}, dtype));
    to_host(out, c);
  });
}

// Elementwise activation module over n elements (act: 1 relu, 2 gelu,
// 3 sigmoid, 4 tanh).
int ref_activation(const void *x, void *y, long n, int dtype, int act) {
  return guarded([&] {
    Tensor out = apply_act(from_host(x, {static_cast<int>(n)}, dtype), act);
    to_host(out, y);
  });
}

// Tensor::to(DataType) (src/tensor.cpp:249-284): the conversion the reference applies to every
// parameter when a float32 model is moved to another dtype.
int ref_convert(const void *x, void *y, long n, int from_dtype, int to_dtype) {
  return guarded([&] {
    Tensor out = from_host(x, {static_cast<int>(n)}, from_dtype).to(dt(to_dtype));
    to_host(out, y);
  });
}

// out = a + b, same shape (the residual add).
int ref_add(const void *a, const void *b, void *y, long n, int dtype) {
  return guarded([&] {
    Tensor out = from_host(a, {static_cast<int>(n)}, dtype) +
                 from_host(b, {static_cast<int>(n)}, dtype);
    to_host(out, y);
  });
}

int ref_layer_norm(const void *x, const void *g, const void *b, void *y,
                   int rows, int cols, float eps, int dtype) {
  return guarded([&] {
    auto ln = make_ln(cols, g, b, eps, dtype);
    to_host(ln->forward(from_host(x, {rows, cols}, dtype)), y);
  });
}

int ref_softmax(const void *x, void *y, int rows, int cols, int dtype) {
  return guarded([&] {
    to_host(from_host(x, {rows, cols}, dtype).softmax(-1), y);
  });
}

// nn::MultiHeadAttention on x[B,T,E]; params = q.w q.b k.w k.b v.w v.b o.w o.b.
// Materialises the [B·H·T, B·H·T] score matrix, so keep B·H·T small.
int ref_mha(const void *x, const void *const *params, void *y, int B, int T,
            int E, int H, int causal, int dtype) {
  return guarded([&] {
    auto mha = make_mha(E, H, causal != 0, params, dtype);
    to_host(mha->forward(from_host(x, {B, T, E}, dtype)), y);
  });
}

// Unary math through the Tensor API (op: 0 exp, 1 log, 2 sqrt, 3 rsqrt, 4 sin, 5 cos).
int ref_unary(const void *x, void *y, long n, int dtype, int op) {
  return guarded([&] {
    Tensor t = from_host(x, {static_cast<int>(n)}, dtype);
    Tensor out = op == 0 ? t.exp() : op == 1 ? t.log() : op == 2 ? t.sqrt()
               : op == 3 ? t.rsqrt() : op == 4 ? t.sin() : t.cos();
    to_host(out, y);
  });
}

int ref_leaky_relu(const void *x, void *y, long n, float slope, int dtype) {
  return guarded([&] {
    to_host(nn::LeakyReLU(slope).forward(from_host(x, {static_cast<int>(n)}, dtype)), y);
  });
}

int ref_rms_norm(const void *x, const void *w, void *y, int rows, int cols, float eps, int dtype) {
  return guarded([&] {
    TensorOptions opt(kCpu, dt(dtype), false);
    nn::RMSNorm m(cols, eps, opt);
    set_param(m.weight, w);
    m.eval();
    to_host(m.forward(from_host(x, {rows, cols}, dtype)), y);
  });
}

// nn::BatchNorm2d in eval mode with the given running statistics (float32).
int ref_batch_norm_eval(const void *x, const void *g, const void *b, const float *mean,
                        const float *var, void *y, int B, int C, int H, int W, float eps,
                        int dtype) {
  return guarded([&] {
    TensorOptions opt(kCpu, dt(dtype), false);
    nn::BatchNorm2d m(C, eps, 0.1f, opt);
    set_param(m.weight, g);
    set_param(m.bias, b);
    if (m.running_mean.dtype() != DataType::Float32 || m.running_var.dtype() != DataType::Float32)
      throw std::runtime_error("driver expects float32 running statistics");
    std::memcpy(m.running_mean.data(), mean, sizeof(float) * C);
    std::memcpy(m.running_var.data(), var, sizeof(float) * C);
    m.eval();
    to_host(m.forward(from_host(x, {B, C, H, W}, dtype)), y);
  });
}

int ref_upsample2d(const void *x, void *y, int B, int C, int H, int W, int scale, int dtype) {
  return guarded([&] { to_host(from_host(x, {B, C, H, W}, dtype).upsample2d(scale), y); });
}

// Tensor::cat of n inputs shaped [outer, dim_j, inner] along dimension 1.
int ref_concat(const void *const *inputs, const int *dims, int n, void *out, int outer, int inner,
               int dtype) {
  return guarded([&] {
    std::vector<Tensor> ts;
    for (int j = 0; j < n; ++j)
      ts.push_back(from_host(inputs[j], {outer, dims[j], inner}, dtype));
    to_host(Tensor::cat(ts, 1), out);
  });
}

int ref_sum(const void *x, void *out, long n, int dtype) {
  return guarded([&] { to_host(from_host(x, {static_cast<int>(n)}, dtype).sum(), out); });
}

int ref_mean_last_dim(const void *x, void *out, int outer, int dim, int dtype) {
  return guarded([&] { to_host(from_host(x, {outer, dim}, dtype).mean(-1, false), out); });
}

// nn::Embedding index path: ids[B,T] int32 → out[B,T,D] in the table's dtype.
int ref_embedding(const int32_t *ids, const void *table, void *out, int B,
                  int T, int V, int D, int dtype) {
  return guarded([&] {
    TensorOptions opt(kCpu, dt(dtype), false);
    nn::Embedding emb(V, D, opt);
    set_param(emb.weight, table);
    emb.eval();
    to_host(emb.forward(from_host(ids, {B, T}, 3)), out);
  });
}

int ref_conv2d(const void *x, const void *w, const void *b, void *y, int B,
               int iC, int iH, int iW, int oC, int k, int stride, int pad,
               int dtype) {
  return guarded([&] {
    TensorOptions opt(kCpu, dt(dtype), false);
    nn::Conv2d conv(iC, oC, k, stride, pad, opt);
    set_param(conv.weight, w);
    set_param(conv.bias, b);
    conv.eval();
    to_host(conv.forward(from_host(x, {B, iC, iH, iW}, dtype)), y);
  });
}

int ref_max_pool2d(const void *x, void *y, int B, int C, int H, int W, int k,
                   int stride, int pad, int dtype) {
  return guarded([&] {
    nn::MaxPool2d pool(k, stride, pad);
    to_host(pool.forward(from_host(x, {B, C, H, W}, dtype)), y);
  });
}

int ref_global_avg_pool(const void *x, void *y, int B, int C, int H, int W,
                        int dtype) {
  return guarded([&] {
    nn::GlobalAvgPool2d gap;
    to_host(gap.forward(from_host(x, {B, C, H, W}, dtype)), y);
  });
}

// GPT-style decoder forward with the topology of the reference's demo model
// (demos/multigpu/gpt3_multi_gpu_demo.py:89-172), built from nn:: modules:
//   h = tok_embed(ids) + pos_embed(arange(T))
//   per layer: h = h + attn(ln1(h)); h = h + fc2(gelu(fc1(ln2(h))))
//   logits = head(ln_f(h))
// params (all in `dtype`):
//   [0] tok_embed[V,d]  [1] pos_embed[T,d]
//   per layer l (16 each, base 2+16l): ln1.w ln1.b q.w q.b k.w k.b v.w v.b
//        o.w o.b ln2.w ln2.b fc1.w fc1.b fc2.w fc2.b
//   then ln_f.w ln_f.b head.w head.b
// stop_after_layers < 0 → full model incl. head (logits[B,T,V]); otherwise the
// hidden state [B,T,d] after that many layers is returned instead.
int ref_gpt_forward(const int32_t *ids, const void *const *params, void *out,
                    int B, int T, int V, int d, int H, int L, int dtype,
                    int stop_after_layers) {
  return guarded([&] {
    TensorOptions opt(kCpu, dt(dtype), false);
    nn::Embedding tok(V, d, opt), pos(T, d, opt);
    set_param(tok.weight, params[0]);
    set_param(pos.weight, params[1]);
    std::vector<int32_t> ar(T);
    for (int t = 0; t < T; ++t)
      ar[t] = t;
    Tensor h = tok.forward(from_host(ids, {B, T}, 3)) +
               pos.forward(from_host(ar.data(), {1, T}, 3));
    int nl = stop_after_layers >= 0 ? stop_after_layers : L;
    for (int l = 0; l < nl; ++l) {
      const void *const *p = params + 2 + 16 * l;
      auto ln1 = make_ln(d, p[0], p[1], 1e-5f, dtype);
      auto attn = make_mha(d, H, true, p + 2, dtype);
      auto ln2 = make_ln(d, p[10], p[11], 1e-5f, dtype);
      auto fc1 = make_linear(d, 4 * d, p[12], p[13], dtype);
      auto fc2 = make_linear(4 * d, d, p[14], p[15], dtype);
      h = h + attn->forward(ln1->forward(h));
      Tensor f = fc2->forward(nn::GELU().forward(fc1->forward(ln2->forward(h))));
      h = h + f;
    }
    if (stop_after_layers >= 0) {
      to_host(h, out);
      return;
    }
    const void *const *p = params + 2 + 16 * L;
    auto lnf = make_ln(d, p[0], p[1], 1e-5f, dtype);
    auto head = make_linear(d, V, p[2], p[3], dtype);
    to_host(head->forward(lnf->forward(h)), out);
  });
}

// inference::Engine over a deploy artifact: load(path) → compile(x) → run(x).
// The output is converted to float32 for the caller. out_shape gets up to 8 dims.
int ref_engine_run_npz(const char *path, const void *x, const int *shape,
                       int ndim, int in_dtype, float *out, long out_capacity,
                       int *out_shape, int *out_ndim) {
  return guarded([&] {
    inference::Engine engine;
    engine.load(std::string(path));
    Shape s(shape, shape + ndim);
    Tensor in = from_host(x, s, in_dtype);
    engine.compile(in);
    Tensor y = engine.run(in);
    Tensor yf = y.dtype() == DataType::Float32 ? y : y.to(DataType::Float32);
    if (static_cast<long>(yf.size()) > out_capacity)
      throw std::runtime_error("output buffer too small");
    *out_ndim = static_cast<int>(yf.shape().size());
    for (int i = 0; i < *out_ndim && i < 8; ++i)
      out_shape[i] = yf.shape()[i];
    to_host(yf, out);
  });
}

// Loader-only check: returns 0 when load_serialized accepts the artifact.
int ref_load_npz(const char *path) {
  return guarded([&] { (void)inference::load_serialized(std::string(path)); });
}

// Backend::all_reduce semantic: the reference's own reduction routine
// (src/core/all_reduce_runtime.hpp:85-133) over `world` participant buffers.
int ref_all_reduce_sum(const void *const *bufs, int world, void *out, long n,
                       int dtype) {
  return guarded([&] {
    const size_t bytes = static_cast<size_t>(n) * dtype_size(dt(dtype));
    std::vector<std::vector<uint8_t>> payloads(world);
    for (int r = 0; r < world; ++r) {
      const uint8_t *p = static_cast<const uint8_t *>(bufs[r]);
      payloads[r].assign(p, p + bytes);
    }
    std::vector<uint8_t> result;
    detail::reduce_sum_bytes(payloads, dt(dtype), static_cast<size_t>(n),
                             result);
    std::memcpy(out, result.data(), bytes);
  });
}

} // extern "C"
