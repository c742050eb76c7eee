// B200Backend — a MuNet `Backend` (src/core/backend.hpp:347-759) whose capabilities
// forward to the C ABI of libmunet_b200.so. This header is compiled against the
// MuNet headers (include path = its `src/`); it contains no kernels.
//
// Advertised (query_support): Matmul, ElementwiseBinary (add/sub/mul/div with
// broadcasting), BroadcastRow, UnaryActivation (relu, sigmoid, exp, log, sqrt, rsqrt, sin,
// cos), Softmax, Concat, Reduction, RandomFill for float32 and bfloat16; Convolution,
// Pooling (max-pool, nearest upsample) and BatchNorm (inference branch) for float32.
// Loss and OptimizerStep are not advertised, so MuNet's dispatcher keeps them on its CPU
// path exactly as it does for any partial backend (src/core/op_dispatch.cpp:670-718).
// Backward entry points and batch_norm(training=true) are training-only and throw.
// memset and to_contiguous run on the device; all_reduce sums over NCCL when a communicator
// is attached and otherwise joins the reference's in-process rendezvous;
// get_last_kernel_time_us reports the event time of the last compute call.
//
// Errors follow the reference convention: std::runtime_error with the C ABI's
// message (src/backend/cuda_backend.cu:15-31). copy() is complete on return
// because callers read host memory right after it (src/tensor.cpp:342-351).
#pragma once

#include "core/all_reduce_runtime.hpp"
#include "core/backend.hpp"
#include "munet_b200.h"
#include "storage.hpp"

#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

namespace munet {

class B200Backend : public Backend,
                    public BackendAllocationTransferCapability,
                    public BackendElementwiseCapability,
                    public BackendBlasCapability,
                    public BackendSpatialCapability,
                    public BackendReductionCapability,
                    public BackendShapeCapability,
                    public BackendNormalizationCapability,
                    public BackendRandomCapability {
public:
  explicit B200Backend(int index) {
    const int rc = mu_ctx_create(index, &ctx_);
    if (rc != MU_OK)
      throw std::runtime_error("B200Backend: cannot create a context on device " +
                               std::to_string(index) + " (status " + std::to_string(rc) + ")");
  }
  ~B200Backend() override { mu_ctx_destroy(ctx_); }
  const char *name() const override { return "b200"; }

  BackendAllocationTransferCapability *allocation_transfer_capability() override { return this; }
  const BackendAllocationTransferCapability *allocation_transfer_capability() const override { return this; }
  BackendElementwiseCapability *elementwise_capability() override { return this; }
  const BackendElementwiseCapability *elementwise_capability() const override { return this; }
  BackendBlasCapability *blas_capability() override { return this; }
  const BackendBlasCapability *blas_capability() const override { return this; }
  BackendSpatialCapability *spatial_capability() override { return this; }
  const BackendSpatialCapability *spatial_capability() const override { return this; }
  BackendReductionCapability *reduction_capability() override { return this; }
  const BackendReductionCapability *reduction_capability() const override { return this; }
  BackendShapeCapability *shape_capability() override { return this; }
  const BackendShapeCapability *shape_capability() const override { return this; }
  BackendNormalizationCapability *normalization_capability() override { return this; }
  const BackendNormalizationCapability *normalization_capability() const override { return this; }
  BackendRandomCapability *random_capability() override { return this; }
  const BackendRandomCapability *random_capability() const override { return this; }

  BackendSupport query_support(BackendFeature feature, DataType dtype,
                               const Shape *shape) const override {
    BackendSupport s = Backend::query_support(feature, dtype, shape);
    const bool f32 = dtype == DataType::Float32, bf16 = dtype == DataType::BFloat16;
    switch (feature) {
    case BackendFeature::Matmul:
    case BackendFeature::UnaryActivation:
    case BackendFeature::Softmax:
    case BackendFeature::ElementwiseBinary:
    case BackendFeature::BroadcastRow:
    case BackendFeature::Concat:
    case BackendFeature::Reduction:
    case BackendFeature::RandomFill:
      s.available = f32 || bf16;
      break;
    case BackendFeature::Convolution:
    case BackendFeature::Pooling:
    case BackendFeature::BatchNorm:
      s.available = f32;
      break;
    default:
      s.available = false; // CPU fallback decided by MuNet's dispatcher
    }
    return s;
  }

  // ---- allocation / transfer ------------------------------------------------
  void *allocate(size_t bytes) override {
    void *p = nullptr;
    check(mu_alloc(ctx_, bytes, &p));
    return p;
  }
  void deallocate(void *ptr) override { check(mu_free(ctx_, ptr)); }
  void memset(void *ptr, int value, size_t bytes) override {
    check(mu_memset(ctx_, ptr, value, bytes, nullptr));
  }
  void copy(const void *src, void *dst, size_t bytes, Device src_dev, Device dst_dev) override {
    const bool s_host = src_dev.type == DeviceType::CPU, d_host = dst_dev.type == DeviceType::CPU;
    if (s_host && d_host) { std::memcpy(dst, src, bytes); return; }
    const int kind = s_host ? MU_COPY_H2D : (d_host ? MU_COPY_D2H : MU_COPY_D2D);
    check(mu_copy(ctx_, dst, src, bytes, kind, nullptr));
    check(mu_check(ctx_, nullptr));
  }
  void synchronize() override { check(mu_synchronize(ctx_)); check(mu_check(ctx_, nullptr)); }
  // Backend::all_reduce = elementwise sum over the participants. With a communicator attached
  // (one process per GPU, set_comm) the sum runs in NCCL on the device, under a host deadline
  // like the reference's (MUNET_ALLREDUCE_TIMEOUT_MS). Without one the participants are threads
  // of this process, each with its own backend: that is the reference's own rendezvous
  // (src/core/all_reduce_runtime.hpp:107-240), staged through the host exactly as its CUDA
  // backend does (src/backend/cuda_backend.cu:963-966).
  void all_reduce(Storage &buffer, size_t num_elements) override {
    if (comm_) {
      if (num_elements * dtype_size(buffer.dtype()) > buffer.size_bytes())
        throw std::runtime_error("all_reduce: num_elements exceeds storage size");
      check(mu_all_reduce_sum(ctx_, comm_, buffer.data(), static_cast<long long>(num_elements),
                              code(buffer), nullptr));
      check(mu_comm_wait(ctx_, comm_, nullptr, 0));
      return;
    }
    detail::all_reduce_via_host(buffer, num_elements, *this, buffer.device(), true);
  }
  // The communicator stays owned by the caller and must outlive this backend's use of it.
  void set_comm(mu_comm *comm) { comm_ = comm; }
  double get_last_kernel_time_us() override { return mu_timer_last_us(ctx_); }
  bool reports_gpu_kernel_time() const override { return true; }
  void to_contiguous(const Storage &src, Storage &dst, const Shape &shape, const Strides &strides,
                     size_t offset) override {
    // strided gather on the device, any element size (head split / merge permutes of the
    // reference's own MultiHeadAttention go through here)
    if (shape.size() > 6 || shape.size() != strides.size())
      throw std::runtime_error("B200Backend: to_contiguous supports at most 6 dimensions");
    int sh[6];
    long long st[6];
    for (size_t d = 0; d < shape.size(); ++d) sh[d] = shape[d], st[d] = strides[d];
    timed([&] {
      check(mu_to_contiguous(ctx_, src.data(), dst.data(), static_cast<int>(shape.size()), sh, st,
                             static_cast<long long>(offset), static_cast<int>(dtype_size(src.dtype())),
                             nullptr));
    });
  }

  // ---- BLAS --------------------------------------------------------------------
  void matmul(const Storage &a, const Storage &b, Storage &out, int M, int K, int N, bool transA,
              bool transB) override {
    timed([&] {
      check(mu_matmul(ctx_, a.data(), b.data(), out.data(), M, K, N, transA, transB, code(a), nullptr));
    });
  }
  void batched_matmul(const Storage &a, const Storage &b, Storage &out, int batch, int M, int K,
                      int N, bool transA, bool transB, int64_t sa, int64_t sb, int64_t so) override {
    timed([&] {
      check(mu_batched_matmul(ctx_, a.data(), b.data(), out.data(), batch, M, K, N, transA, transB, sa,
                              sb, so, code(a), nullptr));
    });
  }

  // ---- elementwise ---------------------------------------------------------------
  void relu(const Storage &in, Storage &out, size_t n) override { unary(in, out, n, MU_ACT_RELU); }
  void sigmoid(const Storage &in, Storage &out, size_t n) override { unary(in, out, n, MU_ACT_SIGMOID); }
  void softmax(const Storage &in, Storage &out, int rows, int cols) override {
    timed([&] { check(mu_softmax(ctx_, in.data(), out.data(), rows, cols, code(in), nullptr)); });
  }
  void add(const Storage &a, const Storage &b, Storage &o, const BroadcastInfo &i) override { binary(MU_OP_ADD, a, b, o, i); }
  void sub(const Storage &a, const Storage &b, Storage &o, const BroadcastInfo &i) override { binary(MU_OP_SUB, a, b, o, i); }
  void mul(const Storage &a, const Storage &b, Storage &o, const BroadcastInfo &i) override { binary(MU_OP_MUL, a, b, o, i); }
  void div(const Storage &a, const Storage &b, Storage &o, const BroadcastInfo &i) override { binary(MU_OP_DIV, a, b, o, i); }
  void broadcast_row(const Storage &src, Storage &dst, int rows, int cols) override {
    check(mu_broadcast_row(ctx_, src.data(), dst.data(), rows, cols, code(src), nullptr));
  }
  void exp(const Storage &in, Storage &out, size_t n) override { math(MU_UN_EXP, in, out, n); }
  void log(const Storage &in, Storage &out, size_t n) override { math(MU_UN_LOG, in, out, n); }
  void sqrt(const Storage &in, Storage &out, size_t n) override { math(MU_UN_SQRT, in, out, n); }
  void rsqrt(const Storage &in, Storage &out, size_t n) override { math(MU_UN_RSQRT, in, out, n); }
  void sin(const Storage &in, Storage &out, size_t n) override { math(MU_UN_SIN, in, out, n); }
  void cos(const Storage &in, Storage &out, size_t n) override { math(MU_UN_COS, in, out, n); }
  void relu_backward(const Storage &, const Storage &, Storage &, size_t) override { training_only("relu_backward"); }
  void sigmoid_backward(const Storage &, const Storage &, Storage &, size_t) override { training_only("sigmoid_backward"); }
  void softmax_backward(const Storage &, const Storage &, Storage &, int, int) override { training_only("softmax_backward"); }

  // ---- spatial ---------------------------------------------------------------------
  void conv2d(const Storage &in, const Storage &weight, const Storage *bias, Storage &out, int B,
              int iC, int iH, int iW, int oC, int kH, int kW, int s, int p) override {
    if (kH != kW) throw std::runtime_error("B200Backend: conv2d needs a square kernel");
    timed([&] {
      check(mu_conv2d(ctx_, in.data(), weight.data(), bias ? bias->data() : nullptr, out.data(), B, iC,
                      iH, iW, oC, kH, s, p, 0, 0, code(in), nullptr));
    });
  }
  void max_pool2d(const Storage &in, Storage &out, int B, int C, int iH, int iW, int k, int s,
                  int p) override {
    check(mu_max_pool2d(ctx_, in.data(), out.data(), B, C, iH, iW, k, s, p, code(in), nullptr));
  }
  void upsample2d(const Storage &in, Storage &out, int B, int C, int iH, int iW, int scale) override {
    check(mu_upsample2d(ctx_, in.data(), out.data(), B, C, iH, iW, scale, code(in), nullptr));
  }
  void conv2d_backward(const Storage &, const Storage &, const Storage &, Storage &, Storage &,
                       Storage *, int, int, int, int, int, int, int, int, int) override { training_only("conv2d_backward"); }
  void max_pool2d_backward(const Storage &, const Storage &, Storage &, int, int, int, int, int, int,
                           int) override { training_only("max_pool2d_backward"); }
  void upsample2d_backward(const Storage &, Storage &, int, int, int, int, int) override { training_only("upsample2d_backward"); }

  // ---- reductions -------------------------------------------------------------------
  void sum_to_shape(const Storage &in, Storage &out, const Shape &in_shape, const Shape &out_shape) override {
    check(mu_sum_to_shape(ctx_, in.data(), out.data(), in_shape.data(), static_cast<int>(in_shape.size()),
                          out_shape.data(), static_cast<int>(out_shape.size()), code(in), nullptr));
  }
  void sum(const Storage &in, Storage &out, size_t n) override {
    check(mu_sum(ctx_, in.data(), out.data(), static_cast<long long>(n), code(in), nullptr));
  }
  void mean_last_dim(const Storage &in, Storage &out, int outer, int dim) override {
    check(mu_mean_last_dim(ctx_, in.data(), out.data(), outer, dim, code(in), nullptr));
  }

  // ---- shape ------------------------------------------------------------------------
  void concat(const std::vector<Storage *> &inputs, Storage &out, int dim,
              const std::vector<Shape> &shapes) override {
    if (inputs.empty() || shapes.size() != inputs.size())
      throw std::runtime_error("B200Backend: concat expects one shape per input");
    long long outer = 1, inner = 1;
    for (int i = 0; i < dim; ++i) outer *= shapes[0][i];
    for (size_t i = dim + 1; i < shapes[0].size(); ++i) inner *= shapes[0][i];
    std::vector<const void *> ptrs;
    std::vector<int> dims;
    for (size_t j = 0; j < inputs.size(); ++j) {
      ptrs.push_back(inputs[j]->data());
      dims.push_back(shapes[j][dim]);
    }
    check(mu_concat(ctx_, ptrs.data(), dims.data(), static_cast<int>(ptrs.size()), out.data(), outer,
                    inner, code(out), nullptr));
  }
  void concat_backward(const Storage &, std::vector<Storage *> &, int, const std::vector<Shape> &) override {
    training_only("concat_backward");
  }

  // ---- normalization ------------------------------------------------------------------
  void batch_norm(const Storage &in, const Storage &scale, const Storage &bias, Storage &running_mean,
                  Storage &running_var, Storage &, Storage &, Storage &out, int B, int C, int H, int W,
                  float, float eps, bool training) override {
    if (training) training_only("batch_norm(training=true)");
    if (running_mean.dtype() != DataType::Float32 || running_var.dtype() != DataType::Float32)
      throw std::runtime_error("B200Backend: batch_norm expects float32 running statistics");
    check(mu_batch_norm_eval(ctx_, in.data(), scale.data(), bias.data(),
                             static_cast<const float *>(running_mean.data()),
                             static_cast<const float *>(running_var.data()), out.data(), B, C, H, W, eps,
                             code(in), nullptr));
  }
  void batch_norm_backward(const Storage &, const Storage &, const Storage &, const Storage &,
                           const Storage &, Storage &, Storage &, Storage &, int, int, int, int,
                           float) override { training_only("batch_norm_backward"); }

  // ---- random -------------------------------------------------------------------------
  void fill_uniform(Storage &out, float low, float high, size_t n) override {
    check(mu_fill_uniform(ctx_, out.data(), static_cast<long long>(n), low, high, ++fill_calls_ * 0x9E3779B9ull,
                          code(out), nullptr));
  }

private:
  mu_ctx *ctx_ = nullptr;
  mu_comm *comm_ = nullptr;
  // every compute call sits between the context's event pair, like the reference's CUDA backend
  // brackets each kernel (src/backend/cuda_backend.cu:952-961)
  template <typename Fn> void timed(Fn &&fn) {
    mu_timer_begin(ctx_, nullptr);
    fn();
    mu_timer_end(ctx_, nullptr);
  }
  unsigned long long fill_calls_ = 41; // seeds successive fills differently, reproducibly per process
  void math(int op, const Storage &in, Storage &out, size_t n) {
    timed([&] { check(mu_unary(ctx_, op, in.data(), out.data(), static_cast<long long>(n), code(in), nullptr)); });
  }
  static int code(const Storage &s) { return static_cast<int>(s.dtype()); } // same enum order
  void check(int rc) const {
    if (rc != MU_OK) throw std::runtime_error(std::string("B200Backend: ") + mu_last_error(ctx_));
  }
  void unary(const Storage &in, Storage &out, size_t n, int act) {
    timed([&] {
      check(mu_eltwise(ctx_, in.data(), nullptr, nullptr, out.data(), static_cast<long long>(n), 1, act,
                       code(in), nullptr));
    });
  }
  void binary(int op, const Storage &a, const Storage &b, Storage &out, const BroadcastInfo &info) {
    const int nd = static_cast<int>(info.out_shape.size());
    if (nd > 6) throw std::runtime_error("B200Backend: broadcasting supports at most 6 dimensions");
    int shape[6];
    long long sa[6], sb[6];
    for (int d = 0; d < nd; ++d) {
      shape[d] = info.out_shape[d];
      sa[d] = info.strides_a[d];
      sb[d] = info.strides_b[d];
    }
    timed([&] {
      check(mu_binary_broadcast(ctx_, op, a.data(), b.data(), out.data(), nd, shape, sa, sb, code(a),
                                nullptr));
    });
  }
  [[noreturn]] static void training_only(const char *op) {
    throw std::runtime_error(std::string("B200Backend: '") + op + "' is a training-only entry point");
  }
};

} // namespace munet
