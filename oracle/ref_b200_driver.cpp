// TEST INFRASTRUCTURE ONLY — the drop-in proof.
//
// Compiled together with the UNMODIFIED MuNet core (same objects as
// libmunet_ref.so) and munet_b200/host/b200_backend.hpp into
// oracle/_ref/libmunet_ref_b200.so, linked against libmunet_b200.so. It registers
// B200Backend as MuNet's DeviceType::CUDA backend (what a maintainer does in
// BackendManager, src/backend/backend_manager.cpp:87-100) and lets the reference's
// own inference::Engine drive the B200 kernels through MuNet's own op front-ends
// and dispatcher. Nothing of the reference is copied; this file only calls it.
#include "b200_backend.hpp"
#include "inference.hpp"
#include "nn.hpp"
#include "tensor.hpp"
#include "backend/plugin_loader.hpp"

#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

using namespace munet;

namespace {
thread_local std::string g_err;
template <typename Fn> int guarded(Fn &&fn) {
  try {
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

const char *refb200_last_error() { return g_err.c_str(); }

// BackendManager::register_backend(DeviceType::CUDA, B200Backend factory)
int refb200_register() {
  return guarded([] {
    BackendManager::register_backend(
        DeviceType::CUDA, [](Device d) { return std::make_shared<B200Backend>(d.index); });
  });
}

// What MuNet's plugin discovery (src/backend/plugin_loader.cpp:101-176) reports for
// device "cuda" with the environment the caller set (MUNET_BACKEND_PLUGIN_DIR):
// returns 1 if an active plugin exists; writes "name|reason_code|detail".
int refb200_plugin_status(char *out, size_t cap) {
  int active = 0;
  guarded([&] {
    std::string s;
    for (const auto &st : plugin::plugins_for_device("cuda")) {
      if (st.active) active = 1;
      s += st.name + "|" + st.reason_code + "|" + st.detail + ";";
    }
    if (out && cap) {
      std::strncpy(out, s.c_str(), cap - 1);
      out[cap - 1] = 0;
    }
  });
  return active;
}

// inference::Engine{device = cuda:<index>} over a deploy artifact: load → compile → run.
// The model's parameters and every intermediate live in B200Backend allocations; ops
// the backend advertises run as B200 kernels, the rest take MuNet's CPU fallback.
int refb200_engine_run_npz(const char *path, int device_index, int dtype, const void *x,
                           const int *shape, int ndim, float *out, long out_capacity,
                           int *out_shape, int *out_ndim) {
  return guarded([&] {
    inference::EngineConfig cfg;
    cfg.device = Device{DeviceType::CUDA, device_index};
    inference::Engine engine(cfg);
    auto module = inference::load_serialized(std::string(path));
    if (dtype != 0) module->to(static_cast<DataType>(dtype));
    engine.load(module);
    Shape s(shape, shape + ndim);
    Tensor in(s, Device{DeviceType::CPU, 0}, DataType::Float32, false);
    std::memcpy(in.data(), x, in.bytes());
    if (dtype != 0) in = in.to(static_cast<DataType>(dtype));
    engine.compile(in);
    Tensor y = engine.run(in);
    Tensor yc = y.to(Device{DeviceType::CPU, 0});
    Tensor yf = yc.dtype() == DataType::Float32 ? yc : yc.to(DataType::Float32);
    if (static_cast<long>(yf.size()) > out_capacity) throw std::runtime_error("output buffer too small");
    *out_ndim = static_cast<int>(yf.shape().size());
    for (int i = 0; i < *out_ndim && i < 8; ++i) out_shape[i] = yf.shape()[i];
    Tensor c = yf.is_contiguous() ? yf : yf.contiguous();
    std::memcpy(out, c.data(), c.bytes());
  });
}

// The reference's own nn::MultiHeadAttention module (src/nn/attention.hpp:34-103) on
// DeviceType::CUDA: its three projections, the head split / merge permutes (to_contiguous),
// the stride-ignoring score matmul, scale, softmax and P.V all reach the B200 kernels through
// the adapter; the mask build and masked_fill take MuNet's CPU path, as on its own CUDA backend.
// params: q.w q.b k.w k.b v.w v.b o.w o.b in `dtype`; x and y are host buffers in `dtype`.
// *kernel_us receives Backend::get_last_kernel_time_us() after the forward.
int refb200_mha_forward(const void *x, const void *const *params, void *y, int B, int T, int E,
                        int H, int causal, int dtype, int device_index, double *kernel_us) {
  return guarded([&] {
    const Device cpu{DeviceType::CPU, 0}, dev{DeviceType::CUDA, device_index};
    const DataType dt = static_cast<DataType>(dtype);
    TensorOptions opt(cpu, dt, false);
    auto mha = std::make_shared<nn::MultiHeadAttention>(E, H, causal != 0, opt);
    auto named = mha->named_parameters("");
    const char *names[8] = {"q_proj.weight", "q_proj.bias", "k_proj.weight", "k_proj.bias",
                            "v_proj.weight", "v_proj.bias", "out_proj.weight", "out_proj.bias"};
    for (int i = 0; i < 8; ++i) {
      Tensor t = named.at(names[i]);
      std::memcpy(t.data(), params[i], t.bytes());
      t.set_requires_grad(false);
    }
    mha->to(dev);
    mha->eval();
    Tensor in({B, T, E}, cpu, dt, false);
    std::memcpy(in.data(), x, in.bytes());
    inference::detail::InferenceModeGuard guard;
    Tensor out = mha->forward(in.to(dev));
    if (kernel_us) *kernel_us = BackendManager::get(dev)->get_last_kernel_time_us();
    Tensor oc = out.to(cpu);
    Tensor c = oc.is_contiguous() ? oc : oc.contiguous();
    std::memcpy(y, c.data(), c.bytes());
  });
}

// Backend::all_reduce through the adapter without a communicator: `world` threads of this
// process, each with its own device buffer, meet in the reference's in-process rendezvous
// (tests/test_backend_manager.cpp:1371-1397 does the same on its CPU backend).
// bufs[i] are host arrays of n elements; every one receives the sum.
int refb200_all_reduce_threads(void *const *bufs, int world, long n, int dtype, int device_index) {
  return guarded([&] {
    setenv("MUNET_ALLREDUCE_WORLD_SIZE", std::to_string(world).c_str(), 1);
    const Device cpu{DeviceType::CPU, 0}, dev{DeviceType::CUDA, device_index};
    const DataType dt = static_cast<DataType>(dtype);
    auto backend = BackendManager::get(dev);
    std::vector<Tensor> ts;
    for (int i = 0; i < world; ++i) {
      Tensor h({static_cast<int>(n)}, cpu, dt, false);
      std::memcpy(h.data(), bufs[i], h.bytes());
      ts.push_back(h.to(dev));
    }
    std::vector<std::string> errs(world);
    std::vector<std::thread> th;
    for (int i = 0; i < world; ++i)
      th.emplace_back([&, i] {
        try {
          backend->all_reduce(*ts[i].impl_->storage, static_cast<size_t>(n));
        } catch (const std::exception &e) {
          errs[i] = e.what();
        }
      });
    for (auto &t : th) t.join();
    unsetenv("MUNET_ALLREDUCE_WORLD_SIZE");
    for (auto &e : errs)
      if (!e.empty()) throw std::runtime_error(e);
    for (int i = 0; i < world; ++i) {
      Tensor h = ts[i].to(cpu);
      std::memcpy(bufs[i], h.data(), h.bytes());
    }
  });
}

} // extern "C"
