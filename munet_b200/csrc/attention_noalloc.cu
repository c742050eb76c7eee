// mu_attention_static_scratch: the attention core for callers that are not
// allowed to allocate device memory.
//
// Who needs this: code that runs while the CUDA allocator is off limits — a host
// thread that must not take the allocator's device-wide lock or trigger an
// implicit synchronisation (a latency-critical serving loop, a callback running
// inside another library), a process whose memory budget was fixed up front by
// an operator, or an embedding host that hands this library raw pointers and
// owns every byte itself. Every other attention entry point of this library
// either needs a caller-provided workspace or an engine-owned arena, both of
// which somebody had to cudaMalloc.
//
// How: the [B*H, T, T] score / probability matrix of the composed path
// (batched GEMM -> row softmax -> batched GEMM) lives in a fixed array that is
// part of the library image, so it exists as soon as the library is loaded on a
// device and is never allocated or freed. The price is a hard size limit and
// that all calls share the one array.
#include "../../include/munet_b200.h"
#include "common.h"
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <mutex>

namespace mu {
int launch_gemm_bf16_tcgen05(const GemmOperands &, const GemmShape &, const Epilogue &, int *status,
                             int num_sms, cudaStream_t);
int launch_gemm_simt(const SimtArgs &, cudaStream_t);
int launch_softmax(const void *, void *, long long, int, float, int, int, int, cudaStream_t);
} // namespace mu

namespace {

// The scratch itself. In host code these names are only handles for the runtime's
// symbol lookup; the device address is obtained once per device below.
static __device__ __align__(256) unsigned char g_scores[MU_ATTENTION_STATIC_SCRATCH_BYTES];
static __device__ __align__(256) int g_status[64];

constexpr int kMaxDevices = 64;
struct PerDevice {
  bool ready = false;
  void *scores = nullptr;
  int *status = nullptr;
  int num_sms = 0;
};
PerDevice g_dev[kMaxDevices];
std::mutex g_mu;

int fail(char *err, size_t err_len, int code, const char *fmt, ...) {
  if (err && err_len) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(err, err_len, fmt, ap);
    va_end(ap);
  }
  return code;
}

bool al16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// One GEMM of the composed path: tensor-core kernel when the operands can be
// addressed by TMA, CUDA-core kernel otherwise. Neither allocates.
int gemm(const PerDevice &pd, const mu::GemmOperands &op, const mu::GemmShape &sh, mu::Epilogue ep,
         int dtype, cudaStream_t st) {
  if (dtype == MU_BF16) {
    ep.vec_ok = al16(ep.c) && ep.ldc % 8 == 0 && ep.batch_hi % 8 == 0 && ep.batch_lo % 8 == 0;
    const int rc = mu::launch_gemm_bf16_tcgen05(op, sh, ep, pd.status, pd.num_sms, st);
    if (rc != 1)
      return rc;
  }
  mu::SimtArgs g;
  g.a = op.a, g.b = op.b, g.lda = op.lda, g.ldb = op.ldb;
  g.a_batch = op.a_batch, g.b_batch = op.b_batch, g.b_kmajor = op.b_kmajor;
  g.is_bf16 = dtype == MU_BF16;
  g.sh = sh, g.ep = ep;
  return mu::launch_gemm_simt(g, st);
}

} // namespace

extern "C" int mu_attention_static_scratch(int device, const void *q, const void *k, const void *v,
                                           void *out, int B, int H, int T, int D, int causal,
                                           int kmode, int dtype, void *stream, int sync_and_check,
                                           char *err, size_t err_len) {
  if (err && err_len)
    err[0] = 0;
  if (device < 0 || device >= kMaxDevices)
    return fail(err, err_len, MU_ERR_INVALID, "attention: device index %d out of range", device);
  if (B < 0 || H <= 0 || T < 0 || D <= 0)
    return fail(err, err_len, MU_ERR_INVALID, "attention: bad dimensions");
  if (kmode != MU_K_LITERAL && kmode != MU_K_MATH)
    return fail(err, err_len, MU_ERR_INVALID, "attention: unknown kmode %d", kmode);
  if (dtype != MU_F32 && dtype != MU_BF16)
    return fail(err, err_len, MU_ERR_UNSUPPORTED, "attention: dtype %d not implemented", dtype);
  if (B == 0 || T == 0)
    return MU_OK;
  if (!q || !k || !v || !out)
    return fail(err, err_len, MU_ERR_INVALID, "attention: null pointer");
  const size_t es = dtype == MU_F32 ? 4 : 2;
  // B*H*T*T*es can wrap in 64 bits (e.g. B = H = 32768, T = 65536, fp32 is 2^64): divide the
  // limit down factor by factor instead of multiplying the sizes up.
  const unsigned long long cap = MU_ATTENTION_STATIC_SCRATCH_BYTES / es;
  const unsigned long long uB = B, uH = H, uT = T;
  if (uT > cap / uT || uH > cap / (uT * uT) || uB > cap / (uT * uT * uH))
    return fail(err, err_len, MU_ERR_SIZE,
                "attention: B*H*T*T*%zu bytes of scores (B=%d H=%d T=%d) exceed the built-in scratch "
                "of %u bytes; use mu_attention with a caller-provided workspace",
                es, B, H, T, MU_ATTENTION_STATIC_SCRATCH_BYTES);

  // The launches below need `device` current; the caller's current device is put back on
  // every way out.
  struct DeviceGuard {
    int prev = -1;
    bool switched = false;
    ~DeviceGuard() {
      if (switched)
        cudaSetDevice(prev);
    }
  } guard;
  if (cudaGetDevice(&guard.prev) != cudaSuccess)
    return fail(err, err_len, MU_ERR_CUDA, "attention: cannot query the current device");
  if (guard.prev != device) {
    if (cudaSetDevice(device) != cudaSuccess)
      return fail(err, err_len, MU_ERR_CUDA, "attention: cannot select device %d", device);
    guard.switched = true;
  }

  PerDevice pd;
  {
    // First call on a device: look up where this device keeps the arrays. The
    // lookup must run with that device current and outside any stream capture.
    std::lock_guard<std::mutex> lock(g_mu);
    PerDevice &slot = g_dev[device];
    if (!slot.ready) {
      void *ps = nullptr, *pst = nullptr;
      cudaError_t e = cudaGetSymbolAddress(&ps, g_scores);
      if (e == cudaSuccess)
        e = cudaGetSymbolAddress(&pst, g_status);
      int sms = 0;
      if (e == cudaSuccess)
        e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
      if (e != cudaSuccess)
        return fail(err, err_len, MU_ERR_CUDA, "attention: scratch set-up failed: %s",
                    cudaGetErrorString(e));
      slot.scores = ps;
      slot.status = static_cast<int *>(pst);
      slot.num_sms = sms;
      slot.ready = true;
    }
    pd = slot;
  }

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // the status word keeps whatever the previous call left: it has to start at zero
  if (cudaMemsetAsync(pd.status, 0, sizeof(int), st) != cudaSuccess)
    return fail(err, err_len, MU_ERR_CUDA, "attention: status clear failed");

  const int BH = B * H;
  const long long Ntot = 1ll * BH * T;
  const int E = H * D;
  int rc;
  {
    mu::GemmOperands op;
    op.a = q, op.lda = D, op.a_batch = 1ll * T * D;
    op.b = k;
    if (kmode == MU_K_LITERAL) {
      op.b_kmajor = 0, op.ldb = Ntot, op.b_batch = T, op.b_col_per_batch = T;
    } else {
      op.b_kmajor = 1, op.ldb = D, op.b_batch = 1ll * T * D;
    }
    mu::GemmShape sh;
    sh.M = T, sh.N = T, sh.K = D, sh.batch = BH;
    mu::Epilogue ep;
    ep.c = pd.scores, ep.ldc = T, ep.batch_hi = 1ll * T * T, ep.batch_div = 1;
    ep.alpha = 1.0f / sqrtf(static_cast<float>(D));
    ep.round_each = 1;
    rc = gemm(pd, op, sh, ep, dtype, st);
  }
  if (rc == 0)
    rc = mu::launch_softmax(pd.scores, pd.scores, Ntot, T, 1.0f, causal ? T : 0, 0, dtype, st);
  if (rc == 0) {
    mu::GemmOperands op;
    op.a = pd.scores, op.lda = T, op.a_batch = 1ll * T * T;
    op.b = v, op.b_kmajor = 0, op.ldb = D, op.b_batch = 1ll * T * D;
    mu::GemmShape sh;
    sh.M = T, sh.N = D, sh.K = T, sh.batch = BH;
    mu::Epilogue ep;
    ep.c = out, ep.ldc = E, ep.batch_div = H, ep.batch_hi = 1ll * T * E, ep.batch_lo = D;
    ep.round_each = 1;
    rc = gemm(pd, op, sh, ep, dtype, st);
  }
  if (rc == 1)
    return fail(err, err_len, MU_ERR_INVALID,
                "attention: B=%d H=%d T=%d D=%d is outside what the kernels of the composed path "
                "address (nothing was launched for the rejected step)", B, H, T, D);
  if (rc != 0)
    return fail(err, err_len, MU_ERR_CUDA, "attention: launch failed: %s",
                cudaGetErrorString(cudaGetLastError()));
  if (sync_and_check) {
    cudaError_t e = cudaStreamSynchronize(st);
    int word = 0;
    if (e == cudaSuccess)
      e = cudaMemcpy(&word, pd.status, sizeof(int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess)
      return fail(err, err_len, MU_ERR_CUDA, "attention: %s", cudaGetErrorString(e));
    if (word != 0)
      return fail(err, err_len, MU_ERR_TIMEOUT, "attention: device-side bounded wait ran out (%d)",
                  word);
  }
  return MU_OK;
}
