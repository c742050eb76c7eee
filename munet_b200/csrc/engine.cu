// Compiled inference executor (host C++ over the C ABI of the kernels).
//
// Stands in for munet::inference::Engine (src/inference.hpp:292-801) running a
// module tree (src/core/module.hpp, src/nn/*.hpp). Where the reference's
// compile() only records a shape contract and run() re-walks the modules
// eagerly, allocating every intermediate (src/inference.hpp:446-610), this
// engine lowers the module tree ONCE per input shape into a flat op list with
//   * a fusion pass: Linear+bias+activation(+residual) → one GEMM epilogue,
//     q/k/v projections → one GEMM that writes head-major, residual adds and
//     head split/merge permutes folded into GEMM epilogues, token+position
//     embedding → one gather;
//   * a buffer plan: liveness intervals over the op list → one device arena
//     (no allocation at run time, vs. one Backend::allocate per op,
//     src/storage.hpp:10-21);
//   * a CUDA graph of the whole forward, replayed by run().
// Module semantics (parameter names, layouts, eval-mode behaviour) follow the
// reference's nn:: classes; citations sit next to each lowering rule.
#include "../../include/munet_b200.h"
#include "engine_io.h"
#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <cuda_runtime.h>
#include <map>
#include <set>
#include <memory>
#include <string>
#include <vector>

using mu::Json;
using mu::NamedTensor;

extern "C" int mu_ctx_simt_forced(const mu_ctx *ctx); // api.cu
extern "C" { // peer_reduce.cu
size_t mu_peer_flags_bytes(void);
int mu_peer_arm(mu_ctx *, void *, unsigned, void *);
int mu_peer_step(mu_ctx *, void *, void *);
int mu_peer_signal(mu_ctx *, void *, void *, unsigned, unsigned, void *);
int mu_peer_wait_done(mu_ctx *, void *, unsigned, unsigned, void *);
int mu_linear_mirrored(mu_ctx *, const void *, const void *, const void *, const void *, void *, void *, int,
                       int, int, int, int, void *); // api.cu
int mu_peer_reduce(mu_ctx *, const void *, const void *, const void *, const void *, void *, long long, int,
                   void *, void *, unsigned, unsigned, unsigned, void *);
int mu_peer_wait_ready(mu_ctx *, void *, unsigned, unsigned, void *);
int mu_peer_signal_done(mu_ctx *, void *, void *, unsigned, unsigned, void *);
int mu_attention_mirrored(mu_ctx *, const void *, const void *, const void *, void *, long long, void *, int,
                          int, int, int, int, int, int, void *); // api.cu
}

namespace {

enum OpKind {
  OP_EMBED, OP_LN, OP_LINEAR, OP_QKV, OP_ATTN, OP_ELTWISE, OP_ARGMAX, OP_CONV, OP_MAXPOOL, OP_GAP,
  OP_ALLREDUCE, OP_BATCHNORM, OP_UPSAMPLE, OP_LEAKY, OP_RMSNORM,
  // tensor-parallel exchange over peer memory (peer_reduce.cu): start of a forward, "the peer has
  // read my earlier partials", "my partial is complete", the fused sum + bias + residual, and a
  // kernel-less op that only joins the second stream back into the main one
  OP_PEER_STEP, OP_PEER_WAIT, OP_PEER_SIGNAL, OP_PEER_REDUCE, OP_JOIN,
  // gathered attention (tp_exchange 3): "what the peer pushed for this exchange has arrived" and
  // "I have consumed it" (the reduce kernel of the other exchanges says the latter itself)
  OP_PEER_WAITRDY, OP_PEER_SIGDONE
};

struct Tensor {
  size_t bytes = 0;
  int first = -1, last = -1; // op indices of definition and last use
  size_t offset = 0;
  int alias_of = -1;
  bool external = false; // engine input: lives in its own buffer
};

struct Op {
  OpKind kind;
  int in = -1, res = -1, out = -1, out2 = -1, out3 = -1, ws = -1;
  int w = -1, b = -1, w2 = -1, b2 = -1;
  int M = 0, K = 0, N = 0, act = 0;
  int B = 0, T = 0, H = 0, D = 0, V = 0, causal = 0;
  int iC = 0, iH = 0, iW = 0, oC = 0, ksz = 0, stride = 1, pad = 0, relu = 0, pool = 0; // spatial ops
  float eps = 1e-5f;
  long long n = 0;
  size_t ws_bytes = 0;
  // Row chunk of a tensor-parallel row-parallel layer: the op works on rows [row0, row0 + M) of
  // its tensors. `side` ops run on the engine's second stream (the all-reduce of one chunk under
  // the GEMM of the next); `rec_ev` is recorded after the op, `wait_ev` awaited before it.
  long long row0 = 0;
  int side = 0, wait_ev = -1, rec_ev = -1;
  int budget = 0; // GEMM leaves a few SMs to the exchange kernel running beside it
  int xidx = 0;   // peer exchange: number of this exchange within one forward
  int pin = -1;   // pushed exchange: the buffer of this rank that the PEER's GEMM writes (the GEMM of
                  // this rank writes the same offset of the peer's arena)
};

struct Weight {
  size_t offset = 0, bytes = 0;
};

struct Val {
  int tid = -1;
  std::vector<int> shape;
  int dtype = MU_F32;
  long long numel() const {
    long long n = 1;
    for (int s : shape)
      n *= s;
    return n;
  }
};

// Rows [r0,r1) x columns [c0,c1) of a parameter viewed as [prod(leading dims), last dim]
// (negative = whole extent): the tensor-parallel shard of a weight or bias.
struct Slice { long long r0 = -1, r1 = -1, c0 = -1, c1 = -1; };

size_t esize(int dt) { return (dt == MU_F32 || dt == MU_I32) ? 4 : 2; }
size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

uint16_t f2bf(float v) { // RNE exactly like the reference (src/types.hpp:311-317)
  uint32_t bits;
  memcpy(&bits, &v, 4);
  bits += 0x7fffu + ((bits >> 16) & 1u);
  return static_cast<uint16_t>(bits >> 16);
}

} // namespace

// Everything that depends on the concrete input shape: the lowered op list, the arena behind it
// and the captured graph. An engine keeps one of these per shape it has met under a wildcard
// contract; the weights are staged once and shared by all of them.
struct PlanState {
  std::vector<Tensor> tensors;
  std::vector<Op> ops;
  void *arena = nullptr;
  void *input_buf = nullptr;
  size_t arena_bytes = 0, input_bytes = 0;
  std::vector<int> in_shape, out_shape;
  int in_dtype = MU_F32, out_dtype = MU_F32;
  int out_tid = -1, argmax_tid = -1;
  cudaGraphExec_t gexec = nullptr;
  cudaGraph_t graph = nullptr;
  long long n_launches = 0;
  int n_events = 0;
  std::vector<cudaEvent_t> events;
  unsigned long long last_used = 0;
};

struct mu_engine {
  mu_ctx *ctx = nullptr;
  int dtype = MU_F32; // compute dtype of floating tensors
  int kmode = MU_K_LITERAL;
  int use_graph = 1;
  int want_argmax = 0;
  // Megatron-style tensor parallelism over `comm` (decoder blocks only): this rank computes
  // heads / MLP columns [tp_rank/tp_size) and all-reduces the row-parallel partial sums.
  int tp_rank = 0, tp_size = 1;
  mu_comm *comm = nullptr;
  Json config;
  std::map<std::string, NamedTensor> params;
  bool loaded = false, compiled = false;

  std::vector<Tensor> tensors;
  std::vector<Op> ops;
  std::vector<Weight> weights;
  std::map<std::string, int> weight_ids;
  std::vector<uint8_t> weight_stage; // host staging of converted weights
  struct DevCopy { size_t dst, dst_pitch; const void *src; size_t src_pitch, width, rows; };
  std::vector<DevCopy> dev_copies;   // weights whose source already lives on the device
  std::vector<bool> dev_weight;      // per weight: filled by device copies
  void *weight_slab = nullptr;
  void *arena = nullptr;
  void *input_buf = nullptr;
  size_t arena_bytes = 0, weight_bytes = 0, input_bytes = 0;
  size_t weights_uploaded = 0; // how many entries of `weights` already live in the slab
  std::vector<int> in_shape, out_shape;
  int in_dtype = MU_F32, out_dtype = MU_F32;
  int out_tid = -1, argmax_tid = -1;
  cudaGraphExec_t gexec = nullptr;
  cudaGraph_t graph = nullptr;
  cudaStream_t cap_stream = nullptr;
  long long n_launches = 0;
  char err[768] = {0};
  // Shape contract of compile(): extents the input must have, -1 = any
  // (detail::ShapeContract, src/inference.hpp:128-176). Plans of other shapes that satisfy it
  // wait in `parked`; the members above are the active plan.
  std::vector<int> contract;
  std::vector<PlanState> parked;
  int plan_cache_entries = 8;
  unsigned long long use_clock = 0;

  void park_active() {
    PlanState p;
    p.tensors.swap(tensors), p.ops.swap(ops);
    p.arena = arena, p.input_buf = input_buf, arena = nullptr, input_buf = nullptr;
    p.arena_bytes = arena_bytes, p.input_bytes = input_bytes;
    p.in_shape.swap(in_shape), p.out_shape.swap(out_shape);
    p.in_dtype = in_dtype, p.out_dtype = out_dtype, p.out_tid = out_tid, p.argmax_tid = argmax_tid;
    p.gexec = gexec, p.graph = graph, gexec = nullptr, graph = nullptr;
    p.n_launches = n_launches, p.n_events = n_events, n_events = 0;
    p.events.swap(events);
    p.last_used = use_clock;
    out_tid = argmax_tid = -1;
    parked.push_back(std::move(p));
  }
  void activate(size_t i) {
    PlanState p = std::move(parked[i]);
    parked.erase(parked.begin() + static_cast<long>(i));
    tensors.swap(p.tensors), ops.swap(p.ops);
    arena = p.arena, input_buf = p.input_buf, arena_bytes = p.arena_bytes, input_bytes = p.input_bytes;
    in_shape.swap(p.in_shape), out_shape.swap(p.out_shape);
    in_dtype = p.in_dtype, out_dtype = p.out_dtype, out_tid = p.out_tid, argmax_tid = p.argmax_tid;
    gexec = p.gexec, graph = p.graph, n_launches = p.n_launches, n_events = p.n_events;
    events.swap(p.events);
  }
  void free_plan(PlanState &p) {
    if (p.gexec) cudaGraphExecDestroy(p.gexec);
    if (p.graph) cudaGraphDestroy(p.graph);
    for (auto &ev : p.events) cudaEventDestroy(ev);
    if (p.arena) mu_free(ctx, p.arena);
    if (p.input_buf) mu_free(ctx, p.input_buf);
  }
  // the active plan only (weights stay)
  void release_active_plan() {
    if (gexec) cudaGraphExecDestroy(gexec), gexec = nullptr;
    if (graph) cudaGraphDestroy(graph), graph = nullptr;
    for (auto &ev : events) cudaEventDestroy(ev);
    events.clear(), n_events = 0;
    if (arena) mu_free(ctx, arena), arena = nullptr;
    if (input_buf) mu_free(ctx, input_buf), input_buf = nullptr;
    tensors.clear(), ops.clear();
    out_tid = argmax_tid = -1;
  }
  int build_plan(const std::vector<int> &shape, int input_dtype);

  int fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(err, sizeof(err), fmt, ap);
    va_end(ap);
    return code;
  }

  // every plan, but not the weights: compile() with a new contract starts from here
  void release_plans() {
    release_active_plan();
    for (auto &p : parked) free_plan(p);
    parked.clear();
    contract.clear();
    compiled = false;
  }
  void release_compiled() {
    release_plans();
    if (peer_flags_local) mu_free(ctx, peer_flags_local), peer_flags_local = nullptr;
    peer_flags_remote = peer_arena = nullptr;
    if (cap_stream) cudaStreamDestroy(cap_stream), cap_stream = nullptr;
    if (side_stream) cudaStreamDestroy(side_stream), side_stream = nullptr;
    if (weight_slab) mu_free(ctx, weight_slab), weight_slab = nullptr;
    weights.clear(), weight_ids.clear();
    weight_stage.clear(), dev_copies.clear(), dev_weight.clear();
    weight_bytes = 0, weights_uploaded = 0;
  }

  // ---- lowering helpers ----------------------------------------------------
  int new_tensor(size_t bytes) {
    Tensor t;
    t.bytes = bytes;
    tensors.push_back(t);
    return static_cast<int>(tensors.size()) - 1;
  }
  int root(int tid) const {
    while (tensors[tid].alias_of >= 0)
      tid = tensors[tid].alias_of;
    return tid;
  }
  void touch(int tid, int op_index) {
    if (tid < 0) return;
    Tensor &t = tensors[root(tid)];
    if (t.first < 0) t.first = op_index;
    t.last = std::max(t.last, op_index);
  }
  int push(const Op &op) {
    const int idx = static_cast<int>(ops.size());
    ops.push_back(op);
    for (int t : {op.in, op.res, op.out, op.out2, op.out3, op.ws, op.pin})
      touch(t, idx);
    return idx;
  }

  // Looks a tensor up by its dotted path and remembers that the module tree asked for it.
  mutable std::set<std::string> used_params;
  const NamedTensor *find_param(const std::string &name) const {
    auto it = params.find(name);
    if (it == params.end()) return nullptr;
    used_params.insert(name);
    return &it->second;
  }

  // Stage a parameter (converted to the compute dtype) into the weight slab.
  // `parts` are concatenated along the last axis (fused q/k/v weights); `sl` selects the
  // same sub-block of every part.
  int stage_weight(const std::vector<std::string> &parts, std::string *why, Slice sl = Slice()) {
    std::string key;
    for (auto &p : parts) key += p + "|";
    key += std::to_string(sl.r0) + "," + std::to_string(sl.r1) + "," + std::to_string(sl.c0) + "," +
           std::to_string(sl.c1);
    auto it = weight_ids.find(key);
    if (it != weight_ids.end()) return it->second;
    struct Part { const NamedTensor *t; long long R, C, r0, r1, c0, c1; };
    std::vector<Part> ps;
    long long rows = -1, cols_total = 0;
    bool any_dev = false;
    for (auto &p : parts) {
      const NamedTensor *t = find_param(p);
      if (!t) { *why = "missing tensor '" + p + "'"; return -1; }
      if (t->dtype != MU_F32 && t->dtype != dtype) {
        *why = "tensor '" + p + "' has dtype " + std::to_string(t->dtype) +
               ", expected float32 or the compute dtype";
        return -1;
      }
      Part q;
      q.t = t;
      q.C = t->shape.empty() ? 1 : t->shape.back();
      q.R = q.C > 0 ? t->numel() / q.C : 0;
      q.r0 = sl.r0 < 0 ? 0 : sl.r0, q.r1 = sl.r1 < 0 ? q.R : sl.r1;
      q.c0 = sl.c0 < 0 ? 0 : sl.c0, q.c1 = sl.c1 < 0 ? q.C : sl.c1;
      if (q.r0 > q.r1 || q.r1 > q.R || q.c0 > q.c1 || q.c1 > q.C) {
        *why = "slice out of range for '" + p + "'";
        return -1;
      }
      if (rows >= 0 && q.r1 - q.r0 != rows) { *why = "concat shape mismatch at '" + p + "'"; return -1; }
      rows = q.r1 - q.r0;
      cols_total += q.c1 - q.c0;
      any_dev = any_dev || t->on_device;
      ps.push_back(q);
    }
    const size_t es = esize(dtype);
    Weight w;
    w.bytes = static_cast<size_t>(rows) * cols_total * es;
    w.offset = align_up(weight_bytes, 256);
    weight_bytes = w.offset + w.bytes;
    long long col0 = 0;
    if (any_dev) {
      // device-resident sources: strided device-to-device copies into the slab
      for (auto &q : ps) {
        if (!q.t->on_device || q.t->dtype != dtype) {
          *why = "device-resident tensors must all be on the device and already have the compute dtype";
          return -1;
        }
        const char *src = static_cast<const char *>(q.t->data) + (q.r0 * q.C + q.c0) * es;
        dev_copies.push_back({w.offset + static_cast<size_t>(col0) * es,
                              static_cast<size_t>(cols_total) * es, src,
                              static_cast<size_t>(q.C) * es,
                              static_cast<size_t>(q.c1 - q.c0) * es, static_cast<size_t>(rows)});
        col0 += q.c1 - q.c0;
      }
      dev_weight.push_back(true);
    } else {
      dev_weight.push_back(false);
      if (weight_stage.size() < weight_bytes) weight_stage.resize(weight_bytes);
      uint8_t *dst = weight_stage.data() + w.offset;
      for (auto &q : ps) {
        const long long c = q.c1 - q.c0;
        for (long long r = 0; r < rows; ++r) {
          uint8_t *d = dst + (static_cast<size_t>(r) * cols_total + col0) * es;
          const long long src_index = (q.r0 + r) * q.C + q.c0;
          if (q.t->dtype == dtype) {
            memcpy(d, static_cast<const uint8_t *>(q.t->data) + static_cast<size_t>(src_index) * es, c * es);
          } else { // float32 → bfloat16, Tensor::to(DataType) semantics (src/tensor.cpp:249-284)
            const float *src = static_cast<const float *>(q.t->data) + src_index;
            uint16_t *o = reinterpret_cast<uint16_t *>(d);
            for (long long i = 0; i < c; ++i) o[i] = f2bf(src[i]);
          }
        }
        col0 += c;
      }
    }
    weights.push_back(w);
    const int id = static_cast<int>(weights.size()) - 1;
    weight_ids[key] = id;
    return id;
  }

  // next/next2: the following siblings inside a Sequential (fusion look-ahead);
  // *fused_count = how many of them this node absorbed.
  int lower(const Json &node, const std::string &prefix, Val &v, const Json *next, bool *fused_next,
            const Json *next2 = nullptr, int *fused_count = nullptr);
  // par: 0 replicated, 1 column-parallel (this rank's slice of the outputs), 2 row-parallel
  // (this rank's slice of the inputs; partial sums are all-reduced, then bias/residual),
  // 3 replicated weights, token rows split: this rank computes its half of the rows and the
  // epilogue also writes them into the peer's copy of the output (two ranks, peer exchange)
  int lower_linear(const std::string &prefix, int K, int N, bool bias, int act, int res_tid, Val &v,
                   int par = 0);
  int lower_mha(const std::string &prefix, int E, int H, bool causal, int res_tid, Val &v,
                bool shard = false);
  int lower_block(const std::string &prefix, int d, int H, Val &v);
  int plan_and_allocate();
  int launch_all(cudaStream_t st);
  int n_events = 0, tp_overlap = 1, tp_comm_sms = 20;
  // tp_exchange 1: partial sums of the row-parallel layers meet through peer memory
  // (peer_reduce.cu) instead of NCCL; needs mu_engine_attach_peer after compile.
  // tp_exchange 2: the same counters, but the row-parallel GEMM itself writes every output tile
  // into the peer's memory as well (Epilogue::c_mirror), so the transfer runs under the GEMM and
  // the reduce kernel reads local memory only. Two receive buffers, used by alternate exchanges,
  // stay reserved for the whole plan (the peer writes them whenever it is ahead).
  // tp_exchange 3: as 2, and the attention sub-block exchanges the attention OUTPUT instead of
  // out_proj's partial sums: the attention kernel writes the columns of this rank's heads into
  // both ranks' [tokens, E] buffer, out_proj then runs unsharded on every rank with bias and
  // residual in its epilogue. Half the bytes cross the link and no reduce kernel follows.
  int tp_exchange = 0, peer_exchanges = 0;
  int peer_in[2] = {-1, -1};
  // The peer reads this rank's partial sums straight out of the arena, so a partial must stay
  // untouched until the peer has signalled that it is done with it — which this rank only waits
  // for before its next row-parallel GEMM. The partial's lifetime in the buffer plan is therefore
  // stretched to that wait (or to the end of the forward), not just to its last local reader.
  int peer_last_partial = -1;
  unsigned peer_ctas = 0;
  void *peer_flags_local = nullptr, *peer_flags_remote = nullptr, *peer_arena = nullptr;
  int capture_graph();
  std::vector<cudaEvent_t> events;
  cudaStream_t side_stream = nullptr;
  // rows [row0, ...) of a [rows, cols] tensor (nullptr stays nullptr)
  void *rows(int tid, long long row0, int cols) const {
    void *p = tptr(tid);
    return p ? static_cast<char *>(p) + static_cast<size_t>(row0) * cols * esize(dtype) : nullptr;
  }
  int launch_op(const Op &op, cudaStream_t st);
  void op_work(const Op &op, double *flops, double *bytes) const;
  void *tptr(int tid) const {
    if (tid < 0) return nullptr;
    const Tensor &t = tensors[root(tid)];
    return t.external ? input_buf : static_cast<char *>(arena) + t.offset;
  }
  void *wptr(int wid) const {
    return wid < 0 ? nullptr : static_cast<char *>(weight_slab) + weights[wid].offset;
  }
};

namespace {

int act_code(const std::string &type) {
  if (type == "ReLU") return MU_ACT_RELU;
  if (type == "GELU") return MU_ACT_GELU;
  if (type == "Sigmoid") return MU_ACT_SIGMOID;
  if (type == "Tanh") return MU_ACT_TANH;
  return -1;
}

} // namespace

// nn::Linear (src/nn/linear.hpp:9-37): weight [in,out], optional bias [out];
// the following activation module and a residual add ride in the GEMM epilogue.
int mu_engine::lower_linear(const std::string &prefix, int K, int N, bool bias, int act,
                            int res_tid, Val &v, int par) {
  if (tp_size <= 1) par = 0;
  if (par && (N % tp_size || K % tp_size))
    return fail(MU_ERR_INVALID, "Linear '%s': %dx%d does not divide over %d tensor-parallel ranks",
                prefix.c_str(), K, N, tp_size);
  const int Kl = par == 2 ? K / tp_size : K, Nl = par == 1 ? N / tp_size : N;
  if (v.shape.empty() || v.shape.back() != Kl)
    return fail(MU_ERR_INVALID, "Linear '%s': input last dim %d != in_features %d", prefix.c_str(),
                v.shape.empty() ? -1 : v.shape.back(), Kl);
  std::string why;
  Slice wsl, bsl;
  if (par == 1) wsl.c0 = bsl.c0 = 1ll * tp_rank * Nl, wsl.c1 = bsl.c1 = 1ll * (tp_rank + 1) * Nl;
  if (par == 2) wsl.r0 = 1ll * tp_rank * Kl, wsl.r1 = 1ll * (tp_rank + 1) * Kl;
  Op op;
  op.kind = OP_LINEAR;
  op.w = stage_weight({prefix + "weight"}, &why, wsl);
  if (op.w < 0) return fail(MU_ERR_INVALID, "Linear '%s': %s", prefix.c_str(), why.c_str());
  int bias_id = -1;
  if (bias) {
    bias_id = stage_weight({prefix + "bias"}, &why, bsl);
    if (bias_id < 0) return fail(MU_ERR_INVALID, "Linear '%s': %s", prefix.c_str(), why.c_str());
  }
  op.M = static_cast<int>(v.numel() / Kl), op.K = Kl, op.N = Nl, op.act = act;
  op.in = v.tid;
  if (par == 2) {
    // partial = x_local · W[rows of this rank]; sum over ranks; then the bias (once) and the
    // residual, like the unsharded layer
    if (act != MU_ACT_NONE) return fail(MU_ERR_INVALID, "row-parallel Linear cannot carry an activation");
    op.out = new_tensor(static_cast<size_t>(op.M) * Nl * esize(dtype));
    int e_out;
    if (res_tid >= 0) {
      e_out = new_tensor(0);
      tensors[e_out].alias_of = root(res_tid);
    } else {
      e_out = op.out;
    }
    // Rows are cut into chunks so that the exchange of chunk i (second stream) runs under the
    // GEMM of chunk i+1; what consumes a chunk waits for its exchange.
    const int Mtot = op.M;
    int chunks = (tp_overlap && Mtot >= 4096) ? 4 : 1;
    const int rows_per = ((Mtot + chunks - 1) / chunks + 255) / 256 * 256;
    chunks = (Mtot + rows_per - 1) / rows_per;
    std::vector<int> done_ev(chunks, -1);
    if (tp_exchange >= 2) {
      // receive buffers are handed out by a count of their own: some exchanges use none
      const int x = peer_exchanges, slot = x & 1;
      const size_t bytes = static_cast<size_t>(Mtot) * Nl * esize(dtype);
      if (peer_in[slot] < 0) {
        peer_in[slot] = new_tensor(bytes);
        touch(peer_in[slot], 0); // reserved from the first op on
      } else if (tensors[peer_in[slot]].bytes != bytes) {
        return fail(MU_ERR_UNSUPPORTED, "Linear '%s': the pushed exchange needs row-parallel outputs of one size",
                    prefix.c_str());
      }
      // the peer's receive buffer `slot` was last read by its reduce of exchange x - 2
      Op w;
      w.kind = OP_PEER_WAIT, w.xidx = std::max(0, x - 1);
      push(w);
      Op g = op;
      g.pin = peer_in[slot];
      push(g);
      Op sg;
      sg.kind = OP_PEER_SIGNAL, sg.xidx = x;
      push(sg);
      Op r;
      r.kind = OP_PEER_REDUCE, r.in = op.out, r.pin = peer_in[slot], r.b = bias_id, r.N = Nl, r.res = res_tid;
      r.out = e_out, r.n = 1ll * Mtot * Nl, r.xidx = x;
      push(r);
      ++peer_exchanges;
      v.tid = e_out;
      v.shape.back() = Nl;
      return MU_OK;
    }
    if (tp_exchange) {
      // peer-memory exchange: GEMM chunk -> "partial complete" to the peer -> fused
      // (mine + peer's) + bias + residual on the second stream
      for (int c = 0; c < chunks; ++c) {
        if (c == 0) {
          Op w;
          w.kind = OP_PEER_WAIT, w.xidx = peer_exchanges, w.in = peer_last_partial;
          push(w);
          peer_last_partial = op.out;
        }
        Op g = op;
        g.row0 = 1ll * c * rows_per, g.M = std::min(rows_per, Mtot - c * rows_per);
        g.budget = chunks > 1 ? 1 : 0;
        push(g);
        Op sg;
        sg.kind = OP_PEER_SIGNAL, sg.xidx = peer_exchanges;
        Op r;
        r.kind = OP_PEER_REDUCE, r.in = op.out, r.b = bias_id, r.N = Nl, r.res = res_tid, r.out = e_out;
        r.row0 = g.row0, r.n = 1ll * g.M * Nl, r.xidx = peer_exchanges;
        if (chunks > 1) {
          sg.rec_ev = n_events++;
          r.side = 1, r.wait_ev = sg.rec_ev, r.rec_ev = n_events++;
          done_ev[c] = r.rec_ev;
        }
        push(sg);
        push(r);
        ++peer_exchanges;
      }
      for (int c = 0; c < chunks && chunks > 1; ++c) {
        Op j;
        j.kind = OP_JOIN, j.wait_ev = done_ev[c], j.in = e_out; // keeps the result live across the join
        push(j);
      }
      v.tid = e_out;
      v.shape.back() = Nl;
      return MU_OK;
    }
    for (int c = 0; c < chunks; ++c) {
      Op g = op;
      g.row0 = 1ll * c * rows_per, g.M = std::min(rows_per, Mtot - c * rows_per);
      Op ar;
      ar.kind = OP_ALLREDUCE, ar.in = op.out, ar.out = op.out, ar.row0 = g.row0, ar.N = Nl;
      ar.n = 1ll * g.M * Nl;
      if (chunks > 1) {
        g.rec_ev = n_events++;
        g.budget = 1;
        ar.side = 1, ar.wait_ev = g.rec_ev, ar.rec_ev = n_events++;
        done_ev[c] = ar.rec_ev;
      }
      push(g);
      push(ar);
    }
    for (int c = 0; c < chunks; ++c) {
      Op e;
      e.kind = OP_ELTWISE, e.in = op.out, e.b = bias_id, e.N = Nl, e.res = res_tid, e.out = e_out;
      e.row0 = 1ll * c * rows_per;
      e.n = 1ll * std::min(rows_per, Mtot - c * rows_per) * Nl;
      e.wait_ev = done_ev[c];
      push(e);
    }
    v.tid = e_out;
    v.shape.back() = Nl;
    return MU_OK;
  }
  op.b = bias_id;
  op.res = res_tid;
  if (res_tid >= 0) {
    // x + f(x): the epilogue reads and writes the same element, so the residual
    // stream is updated in place.
    op.out = new_tensor(0);
    tensors[op.out].alias_of = root(res_tid);
  } else {
    op.out = new_tensor(static_cast<size_t>(op.M) * Nl * esize(dtype));
  }
  if (par == 3 && tp_size == 2 && op.M % 2 == 0) {
    const int half = op.M / 2;
    op.row0 = 1ll * tp_rank * half, op.M = half;
    op.pin = op.out; // the same rows of the peer's copy
  }
  push(op);
  v.tid = op.out;
  v.shape.back() = Nl;
  return MU_OK;
}

// nn::MultiHeadAttention::forward_impl (src/nn/attention.hpp:34-103).
int mu_engine::lower_mha(const std::string &prefix, int E, int H, bool causal, int res_tid, Val &v,
                         bool shard) {
  if (v.shape.size() != 3)
    return fail(MU_ERR_INVALID, "MultiHeadAttention expects input shape [B,T,E]");
  if (v.shape[2] != E)
    return fail(MU_ERR_INVALID, "MultiHeadAttention expects last dim == embed_dim");
  if (H <= 0 || E % H)
    return fail(MU_ERR_INVALID, "MultiHeadAttention: embed_dim must be divisible by num_heads");
  const int B = v.shape[0], T = v.shape[1], D = E / H;
  const bool tp = tp_size > 1 && shard;
  if (tp && H % tp_size)
    return fail(MU_ERR_INVALID, "MultiHeadAttention: %d heads do not divide over %d ranks", H, tp_size);
  const int Hfull = H;
  if (tp) H = H / tp_size; // this rank's heads [tp_rank*H, (tp_rank+1)*H)
  const int El = H * D;
  const size_t per = static_cast<size_t>(B) * T * El * esize(dtype);
  std::string why;
  Slice sl;
  if (tp) sl.c0 = 1ll * tp_rank * El, sl.c1 = 1ll * (tp_rank + 1) * El;
  (void)Hfull;
  Op q;
  q.kind = OP_QKV;
  q.w = stage_weight({prefix + "q_proj.weight", prefix + "k_proj.weight", prefix + "v_proj.weight"}, &why, sl);
  if (q.w >= 0)
    q.b = stage_weight({prefix + "q_proj.bias", prefix + "k_proj.bias", prefix + "v_proj.bias"}, &why, sl);
  if (q.w < 0 || q.b < 0)
    return fail(MU_ERR_INVALID, "MultiHeadAttention '%s': %s", prefix.c_str(), why.c_str());
  q.B = B, q.T = T, q.K = E, q.H = H, q.D = D;
  q.in = v.tid;
  q.out = new_tensor(3 * per); // q | k | v, head-major, contiguous
  push(q);
  Op a;
  a.kind = OP_ATTN;
  a.in = q.out;
  a.B = B, a.T = T, a.H = H, a.D = D, a.causal = causal;
  // a context forced onto the CUDA-core kernels runs the composed path for every shape
  a.ws_bytes = mu_ctx_simt_forced(ctx) ? mu_attention_workspace_bytes_composed(B, H, T, D, dtype)
                                       : mu_attention_workspace_bytes(B, H, T, D, dtype);
  a.ws = new_tensor(a.ws_bytes);
  if (tp && tp_exchange >= 3) {
    // gathered attention: this rank's heads are columns [tp_rank*El, +El) of a [tokens, E] buffer
    // that exists on both ranks; the kernel writes them here and into the peer's copy
    const int x = peer_exchanges, slot = x & 1;
    const size_t bytes = static_cast<size_t>(B) * T * E * esize(dtype);
    if (peer_in[slot] < 0) {
      peer_in[slot] = new_tensor(bytes);
      touch(peer_in[slot], 0); // reserved from the first op on
    } else if (tensors[peer_in[slot]].bytes != bytes) {
      return fail(MU_ERR_UNSUPPORTED, "MultiHeadAttention '%s': the gathered exchange needs buffers of one size",
                  prefix.c_str());
    }
    Op w;
    w.kind = OP_PEER_WAIT, w.xidx = std::max(0, x - 1); // the peer has consumed exchange x - 2
    push(w);
    a.out = peer_in[slot], a.pin = peer_in[slot];
    a.N = E, a.K = tp_rank * El; // row stride and first column of this rank's heads
    push(a);
    Op sg;
    sg.kind = OP_PEER_SIGNAL, sg.xidx = x;
    push(sg);
    Op wr;
    wr.kind = OP_PEER_WAITRDY, wr.xidx = x;
    push(wr);
    ++peer_exchanges;
    v.tid = peer_in[slot];
    v.shape = {B * T, E};
    const bool split_rows = tp_exchange == 4 && (B * T) % 2 == 0 && res_tid >= 0;
    int rc = lower_linear(prefix + "out_proj.", E, E, true, MU_ACT_NONE, res_tid, v, split_rows ? 3 : 0);
    Op sd;
    sd.kind = OP_PEER_SIGDONE, sd.xidx = x, sd.in = peer_in[slot];
    push(sd);
    if (split_rows && rc == MU_OK) {
      // out_proj ran on this rank's half of the token rows and wrote them into both copies of
      // the residual stream; the other half arrives from the peer. That stream is live on both
      // ranks from the embedding to the last layer, at the same arena offset, and the peer can
      // only write it between this rank's attention kernel (its READY) and this wait, when
      // nothing here reads those rows.
      const int x1 = peer_exchanges;
      Op s1, w1, d1;
      s1.kind = OP_PEER_SIGNAL, s1.xidx = x1, s1.in = v.tid;
      w1.kind = OP_PEER_WAITRDY, w1.xidx = x1, w1.in = v.tid;
      d1.kind = OP_PEER_SIGDONE, d1.xidx = x1, d1.in = v.tid;
      push(s1);
      push(w1);
      push(d1);
      ++peer_exchanges;
    }
    v.shape = {B, T, E};
    return rc;
  }
  a.out = new_tensor(per);
  push(a);
  v.tid = a.out;
  v.shape = {B * T, El};
  int rc = lower_linear(prefix + "out_proj.", E, E, true, MU_ACT_NONE, res_tid, v, tp ? 2 : 0);
  v.shape = {B, T, E};
  return rc;
}

// Pre-norm decoder block (demos/multigpu/gpt3_multi_gpu_demo.py:89-113):
//   x = x + attn(ln1(x)); x = x + ff(ln2(x)), ff = Linear(d,4d) → GELU → Linear(4d,d)
int mu_engine::lower_block(const std::string &prefix, int d, int H, Val &v) {
  std::string why;
  for (int half = 0; half < 2; ++half) {
    const std::string ln = prefix + (half ? "ln2." : "ln1.");
    Op n;
    n.kind = OP_LN;
    n.w = stage_weight({ln + "weight"}, &why);
    if (n.w >= 0) n.b = stage_weight({ln + "bias"}, &why);
    if (n.w < 0 || n.b < 0) return fail(MU_ERR_INVALID, "LayerNorm '%s': %s", ln.c_str(), why.c_str());
    n.M = static_cast<int>(v.numel() / d), n.N = d;
    n.in = v.tid;
    n.out = new_tensor(static_cast<size_t>(v.numel()) * esize(dtype));
    push(n);
    Val h = v;
    h.tid = n.out;
    int rc;
    if (half == 0) {
      rc = lower_mha(prefix + "attn.", d, H, true, v.tid, h, true);
    } else {
      rc = lower_linear(prefix + "ff.0.", d, 4 * d, true, MU_ACT_GELU, -1, h, 1);
      if (rc == MU_OK) rc = lower_linear(prefix + "ff.2.", 4 * d, d, true, MU_ACT_NONE, v.tid, h, 2);
    }
    if (rc) return rc;
    v.tid = h.tid;
  }
  return MU_OK;
}

int mu_engine::lower(const Json &node, const std::string &prefix, Val &v, const Json *next,
                     bool *fused_next, const Json *next2, int *fused_count) {
  if (fused_next) *fused_next = false;
  if (fused_count) *fused_count = 0;
  if (!node.is_object()) return fail(MU_ERR_INVALID, "Serialized module config root must be a JSON object");
  const Json *ty = node.get("type");
  if (!ty || !ty->is_string()) return fail(MU_ERR_INVALID, "module config is missing 'type'");
  const std::string &type = ty->str;
  auto req_int = [&](const char *k, int *out) {
    const Json *j = node.get(k);
    if (!j || !j->is_number()) return false;
    *out = static_cast<int>(j->num);
    return true;
  };
  auto req_bool = [&](const char *k, bool *out) {
    const Json *j = node.get(k);
    if (!j || j->kind != Json::BOOL) return false;
    *out = j->b;
    return true;
  };
  std::string why;

  if (type == "Sequential") { // src/nn/sequential.hpp:8-28, children named by index
    const Json *layers = node.get("layers");
    if (!layers || !layers->is_array()) return fail(MU_ERR_INVALID, "Sequential: missing 'layers'");
    for (size_t i = 0; i < layers->arr.size(); ++i) {
      const Json *nx = i + 1 < layers->arr.size() ? &layers->arr[i + 1] : nullptr;
      const Json *nx2 = i + 2 < layers->arr.size() ? &layers->arr[i + 2] : nullptr;
      bool fused = false;
      int count = 0;
      int rc = lower(layers->arr[i], prefix + std::to_string(i) + ".", v, nx, &fused, nx2, &count);
      if (rc) return rc;
      if (count > 0) i += count;
      else if (fused) ++i;
    }
    return MU_OK;
  }
  if (type == "Linear") {
    int K, N;
    bool bias;
    if (!req_int("in_features", &K) || !req_int("out_features", &N) || !req_bool("bias", &bias))
      return fail(MU_ERR_INVALID, "Linear: missing in_features/out_features/bias");
    int act = MU_ACT_NONE;
    if (next && next->is_object() && next->get("type") && next->get("type")->is_string()) {
      const int a = act_code(next->get("type")->str);
      if (a > 0) { act = a; if (fused_next) *fused_next = true; }
    }
    return lower_linear(prefix, K, N, bias, act, -1, v);
  }
  if (act_code(type) > 0) {
    Op op;
    op.kind = OP_ELTWISE, op.act = act_code(type), op.n = v.numel();
    op.in = v.tid, op.out = new_tensor(static_cast<size_t>(op.n) * esize(dtype));
    push(op);
    v.tid = op.out;
    return MU_OK;
  }
  if (type == "LeakyReLU") { // src/nn/activations.hpp:76-88
    const Json *sl = node.get("negative_slope");
    if (!sl || !sl->is_number()) return fail(MU_ERR_INVALID, "LeakyReLU: missing negative_slope");
    Op op;
    op.kind = OP_LEAKY, op.eps = static_cast<float>(sl->num), op.n = v.numel();
    op.in = v.tid, op.out = new_tensor(static_cast<size_t>(op.n) * esize(dtype));
    push(op);
    v.tid = op.out;
    return MU_OK;
  }
  if (type == "RMSNorm") { // src/nn/normalization.hpp:39-67
    int d;
    const Json *eps = node.get("eps");
    if (!req_int("normalized_shape", &d) || !eps || !eps->is_number())
      return fail(MU_ERR_INVALID, "RMSNorm: missing normalized_shape/eps");
    if (d <= 0) return fail(MU_ERR_INVALID, "RMSNorm expects normalized_shape > 0");
    if (v.shape.empty() || v.shape.back() != d)
      return fail(MU_ERR_INVALID, "RMSNorm expects last dim to match normalized_shape");
    Op n;
    n.kind = OP_RMSNORM, n.eps = static_cast<float>(eps->num);
    n.w = stage_weight({prefix + "weight"}, &why);
    if (n.w < 0) return fail(MU_ERR_INVALID, "RMSNorm: %s", why.c_str());
    n.M = static_cast<int>(v.numel() / d), n.N = d, n.in = v.tid;
    n.out = new_tensor(static_cast<size_t>(v.numel()) * esize(dtype));
    push(n);
    v.tid = n.out;
    return MU_OK;
  }
  if (type == "BatchNorm2d") { // src/nn/normalization.hpp:69-108, eval: running statistics
    int c;
    const Json *eps = node.get("eps");
    if (!req_int("num_features", &c) || !eps || !eps->is_number())
      return fail(MU_ERR_INVALID, "BatchNorm2d: missing num_features/eps");
    if (v.shape.size() != 4 || v.shape[1] != c)
      return fail(MU_ERR_INVALID, "BatchNorm2d expects NCHW input with C == num_features");
    if (dtype != MU_F32) return fail(MU_ERR_UNSUPPORTED, "BatchNorm2d: only float32 is implemented");
    Op n;
    n.kind = OP_BATCHNORM, n.eps = static_cast<float>(eps->num);
    n.w = stage_weight({prefix + "weight"}, &why);
    if (n.w >= 0) n.b = stage_weight({prefix + "bias"}, &why);
    if (n.b >= 0) n.w2 = stage_weight({prefix + "running_mean"}, &why);
    if (n.w2 >= 0) n.b2 = stage_weight({prefix + "running_var"}, &why);
    if (n.w < 0 || n.b < 0 || n.w2 < 0 || n.b2 < 0) return fail(MU_ERR_INVALID, "BatchNorm2d: %s", why.c_str());
    n.B = v.shape[0], n.iC = c, n.iH = v.shape[2], n.iW = v.shape[3], n.in = v.tid;
    n.out = new_tensor(static_cast<size_t>(v.numel()) * 4);
    push(n);
    v.tid = n.out;
    return MU_OK;
  }
  if (type == "Upsample") { // src/nn/pooling.hpp:37-43, nearest neighbour
    int sc;
    if (!req_int("scale_factor", &sc) || sc <= 0) return fail(MU_ERR_INVALID, "Upsample: missing scale_factor");
    if (v.shape.size() != 4) return fail(MU_ERR_INVALID, "Upsample expects NCHW input");
    Op u;
    u.kind = OP_UPSAMPLE, u.B = v.shape[0], u.iC = v.shape[1], u.iH = v.shape[2], u.iW = v.shape[3];
    u.stride = sc, u.in = v.tid;
    u.out = new_tensor(static_cast<size_t>(v.numel()) * sc * sc * esize(dtype));
    push(u);
    v.tid = u.out, v.shape = {u.B, u.iC, u.iH * sc, u.iW * sc};
    return MU_OK;
  }
  if (type == "Conv2d") { // src/nn/linear.hpp:39-64; ReLU and MaxPool2d(2,2,0) that follow are fused
    int iC, oC, k, s, p;
    if (!req_int("in_channels", &iC) || !req_int("out_channels", &oC) || !req_int("kernel_size", &k) ||
        !req_int("stride", &s) || !req_int("padding", &p))
      return fail(MU_ERR_INVALID, "Conv2d: missing in_channels/out_channels/kernel_size/stride/padding");
    if (v.shape.size() != 4 || v.shape[1] != iC)
      return fail(MU_ERR_INVALID, "Conv2d expects NCHW input with %d channels", iC);
    if (dtype != MU_F32)
      return fail(MU_ERR_UNSUPPORTED, "Conv2d: only float32 is implemented");
    if (k <= 0 || s <= 0 || p < 0)
      return fail(MU_ERR_INVALID, "Conv2d: bad kernel_size/stride/padding");
    Op c;
    c.kind = OP_CONV;
    c.w = stage_weight({prefix + "weight"}, &why);
    if (c.w >= 0) c.b = stage_weight({prefix + "bias"}, &why);
    if (c.w < 0 || c.b < 0) return fail(MU_ERR_INVALID, "Conv2d '%s': %s", prefix.c_str(), why.c_str());
    c.B = v.shape[0], c.iC = iC, c.iH = v.shape[2], c.iW = v.shape[3], c.oC = oC;
    c.ksz = k, c.stride = s, c.pad = p;
    int oH = (c.iH + 2 * p - k) / s + 1, oW = (c.iW + 2 * p - k) / s + 1;
    if (oH <= 0 || oW <= 0) return fail(MU_ERR_INVALID, "Conv2d: kernel larger than the padded input");
    // look ahead inside the enclosing Sequential: ReLU, then MaxPool2d(2,2,0)
    int consumed = 0;
    if (next && next->is_object() && next->get("type") && next->get("type")->is_string() &&
        next->get("type")->str == "ReLU") {
      c.relu = 1;
      consumed = 1;
      const Json *n2 = next2;
      if (n2 && n2->is_object() && n2->get("type") && n2->get("type")->is_string() &&
          n2->get("type")->str == "MaxPool2d") {
        const Json *pk = n2->get("kernel_size"), *ps = n2->get("stride"), *pp = n2->get("padding");
        if (pk && ps && pp && pk->is_number() && ps->is_number() && pp->is_number() &&
            static_cast<int>(pk->num) == 2 && static_cast<int>(ps->num) == 2 &&
            static_cast<int>(pp->num) == 0 && oH >= 2 && oW >= 2) {
          c.pool = 2;
          consumed = 2;
          oH /= 2, oW /= 2;
        }
      }
    }
    c.in = v.tid;
    c.out = new_tensor(static_cast<size_t>(c.B) * oC * oH * oW * 4);
    push(c);
    v.tid = c.out, v.shape = {c.B, oC, oH, oW};
    if (fused_count) *fused_count = consumed;
    if (fused_next) *fused_next = consumed > 0;
    return MU_OK;
  }
  if (type == "MaxPool2d") { // src/nn/pooling.hpp:28-36
    int k, s, p;
    if (!req_int("kernel_size", &k) || !req_int("stride", &s) || !req_int("padding", &p))
      return fail(MU_ERR_INVALID, "MaxPool2d: missing kernel_size/stride/padding");
    if (v.shape.size() != 4) return fail(MU_ERR_INVALID, "MaxPool2d expects NCHW input");
    if (dtype != MU_F32) return fail(MU_ERR_UNSUPPORTED, "MaxPool2d: only float32 is implemented");
    if (k <= 0 || s <= 0 || p < 0) return fail(MU_ERR_INVALID, "MaxPool2d: bad kernel_size/stride/padding");
    Op m;
    m.kind = OP_MAXPOOL, m.B = v.shape[0], m.iC = v.shape[1], m.iH = v.shape[2], m.iW = v.shape[3];
    m.ksz = k, m.stride = s, m.pad = p;
    const int oH = (m.iH + 2 * p - k) / s + 1, oW = (m.iW + 2 * p - k) / s + 1;
    if (oH <= 0 || oW <= 0) return fail(MU_ERR_INVALID, "MaxPool2d: window larger than the input");
    m.in = v.tid;
    m.out = new_tensor(static_cast<size_t>(m.B) * m.iC * oH * oW * 4);
    push(m);
    v.tid = m.out, v.shape = {m.B, m.iC, oH, oW};
    return MU_OK;
  }
  if (type == "GlobalAvgPool2d") { // src/nn/pooling.hpp:8-26 → [B,C,1,1]
    if (v.shape.size() != 4) return fail(MU_ERR_INVALID, "GlobalAvgPool2d expects NCHW input");
    if (dtype != MU_F32) return fail(MU_ERR_UNSUPPORTED, "GlobalAvgPool2d: only float32 is implemented");
    Op g;
    g.kind = OP_GAP, g.B = v.shape[0], g.iC = v.shape[1], g.iH = v.shape[2], g.iW = v.shape[3];
    g.in = v.tid;
    g.out = new_tensor(static_cast<size_t>(g.B) * g.iC * 4);
    push(g);
    v.tid = g.out, v.shape = {g.B, g.iC, 1, 1};
    return MU_OK;
  }
  if (type == "Dropout") return MU_OK; // eval mode: identity (src/nn/activations.hpp:47-50)
  if (type == "Flatten") {             // src/nn/linear.hpp:66-73
    if (v.shape.empty()) return fail(MU_ERR_INVALID, "Flatten: empty shape");
    const int b0 = v.shape[0];
    v.shape = {b0, static_cast<int>(v.numel() / std::max(b0, 1))};
    return MU_OK;
  }
  if (type == "LayerNorm") { // src/nn/normalization.hpp:8-37
    int d;
    const Json *eps = node.get("eps");
    if (!req_int("normalized_shape", &d) || !eps || !eps->is_number())
      return fail(MU_ERR_INVALID, "LayerNorm: missing normalized_shape/eps");
    if (v.shape.empty() || v.shape.back() != d)
      return fail(MU_ERR_INVALID, "LayerNorm expects last dim to match normalized_shape");
    Op n;
    n.kind = OP_LN, n.eps = static_cast<float>(eps->num);
    n.w = stage_weight({prefix + "weight"}, &why);
    if (n.w >= 0) n.b = stage_weight({prefix + "bias"}, &why);
    if (n.w < 0 || n.b < 0) return fail(MU_ERR_INVALID, "LayerNorm: %s", why.c_str());
    n.M = static_cast<int>(v.numel() / d), n.N = d, n.in = v.tid;
    n.out = new_tensor(static_cast<size_t>(v.numel()) * esize(dtype));
    push(n);
    v.tid = n.out;
    return MU_OK;
  }
  if (type == "Embedding") { // index path, src/nn/linear.hpp:92-131
    int V, D;
    if (!req_int("num_embeddings", &V) || !req_int("embedding_dim", &D))
      return fail(MU_ERR_INVALID, "Embedding: missing num_embeddings/embedding_dim");
    if (V <= 0 || D <= 0)
      return fail(MU_ERR_INVALID, "Embedding expects positive num_embeddings and embedding_dim");
    if (v.shape.size() != 2 || v.dtype != MU_I32)
      return fail(MU_ERR_INVALID, "Embedding expects [B,T] int32 indices");
    Op e;
    e.kind = OP_EMBED, e.B = v.shape[0], e.T = v.shape[1], e.V = V, e.D = D;
    e.w = stage_weight({prefix + "weight"}, &why);
    if (e.w < 0) return fail(MU_ERR_INVALID, "Embedding: %s", why.c_str());
    e.in = v.tid;
    e.out = new_tensor(static_cast<size_t>(e.B) * e.T * D * esize(dtype));
    push(e);
    v.tid = e.out, v.shape = {e.B, e.T, D}, v.dtype = dtype;
    return MU_OK;
  }
  if (type == "MultiHeadAttention") {
    int E, H;
    bool causal;
    if (!req_int("embed_dim", &E) || !req_int("num_heads", &H) || !req_bool("causal", &causal))
      return fail(MU_ERR_INVALID, "MultiHeadAttention: missing embed_dim/num_heads/causal");
    return lower_mha(prefix, E, H, causal, -1, v);
  }
  // ---- extension node types (a superset of the reference's deploy format, which has
  // no residual container and therefore cannot express a decoder) ----
  if (type == "TransformerBlock") {
    int d, H;
    if (!req_int("d_model", &d) || !req_int("n_heads", &H))
      return fail(MU_ERR_INVALID, "TransformerBlock: missing d_model/n_heads");
    if (v.shape.size() != 3 || v.shape[2] != d)
      return fail(MU_ERR_INVALID, "TransformerBlock expects [B,T,d_model]");
    return lower_block(prefix, d, H, v);
  }
  if (type == "GPTDecoder") { // SimpleGPT, demos/multigpu/gpt3_multi_gpu_demo.py:116-172
    int V, C, d, H, L;
    if (!req_int("vocab", &V) || !req_int("ctx_len", &C) || !req_int("d_model", &d) ||
        !req_int("n_heads", &H) || !req_int("n_layers", &L))
      return fail(MU_ERR_INVALID, "GPTDecoder: missing vocab/ctx_len/d_model/n_heads/n_layers");
    if (v.shape.size() != 2 || v.dtype != MU_I32)
      return fail(MU_ERR_INVALID, "GPTDecoder expects [B,T] int32 token ids");
    const int B = v.shape[0], T = v.shape[1];
    if (T > C) return fail(MU_ERR_INVALID, "GPTDecoder: sequence length %d exceeds ctx_len %d", T, C);
    Op e;
    e.kind = OP_EMBED, e.B = B, e.T = T, e.V = V, e.D = d;
    e.w = stage_weight({prefix + "token_embed.weight"}, &why);
    if (e.w >= 0) e.w2 = stage_weight({prefix + "pos_embed.weight"}, &why);
    if (e.w < 0 || e.w2 < 0) return fail(MU_ERR_INVALID, "GPTDecoder: %s", why.c_str());
    e.in = v.tid;
    e.out = new_tensor(static_cast<size_t>(B) * T * d * esize(dtype));
    push(e);
    v.tid = e.out, v.shape = {B, T, d}, v.dtype = dtype;
    for (int l = 0; l < L; ++l) {
      int rc = lower_block(prefix + "blocks." + std::to_string(l) + ".", d, H, v);
      if (rc) return rc;
    }
    Op n;
    n.kind = OP_LN;
    n.w = stage_weight({prefix + "ln_f.weight"}, &why);
    if (n.w >= 0) n.b = stage_weight({prefix + "ln_f.bias"}, &why);
    if (n.w < 0 || n.b < 0) return fail(MU_ERR_INVALID, "GPTDecoder: %s", why.c_str());
    n.M = B * T, n.N = d, n.in = v.tid;
    n.out = new_tensor(static_cast<size_t>(B) * T * d * esize(dtype));
    push(n);
    v.tid = n.out;
    // under tensor parallelism the LM head is column-parallel: each rank owns a vocabulary slab
    return lower_linear(prefix + "head.", d, V, true, MU_ACT_NONE, -1, v, 1);
  }
  return fail(MU_ERR_UNSUPPORTED, "Unsupported serialized module type for C++ reconstruction: %s",
              type.c_str());
}

// Liveness-based arena plan: tensors that are never live at the same op may
// share bytes. Largest-first first-fit over the already placed tensors.
int mu_engine::plan_and_allocate() {
  std::vector<int> order;
  for (size_t i = 0; i < tensors.size(); ++i)
    if (tensors[i].alias_of < 0 && !tensors[i].external && tensors[i].bytes > 0) order.push_back(static_cast<int>(i));
  std::sort(order.begin(), order.end(), [&](int a, int b) { return tensors[a].bytes > tensors[b].bytes; });
  std::vector<int> placed;
  arena_bytes = 0;
  for (int id : order) {
    Tensor &t = tensors[id];
    std::vector<std::pair<size_t, size_t>> busy;
    for (int p : placed) {
      const Tensor &o = tensors[p];
      if (o.first <= t.last && t.first <= o.last) busy.push_back({o.offset, o.offset + o.bytes});
    }
    std::sort(busy.begin(), busy.end());
    size_t off = 0;
    for (auto &iv : busy) {
      if (off + t.bytes <= iv.first) break;
      off = std::max(off, align_up(iv.second, 1024));
    }
    t.offset = off;
    arena_bytes = std::max(arena_bytes, off + t.bytes);
    placed.push_back(id);
  }
  int rc = mu_alloc(ctx, std::max<size_t>(arena_bytes, 16), &arena);
  if (rc) return fail(rc, "arena allocation of %zu bytes failed: %s", arena_bytes, mu_last_error(ctx));
  rc = mu_alloc(ctx, std::max<size_t>(input_bytes, 16), &input_buf);
  if (rc) return fail(rc, "input buffer allocation failed: %s", mu_last_error(ctx));
  // the warm-up forward of compile() reads this buffer before any run(): all-zero
  // ids / activations are valid inputs for every op
  if (cudaMemset(input_buf, 0, std::max<size_t>(input_bytes, 16)) != cudaSuccess)
    return fail(MU_ERR_CUDA, "input buffer clear failed");
  if (weight_slab) {
    // a further plan of an engine whose weights are already on the device: the module tree is
    // the same, so lowering must have found every parameter in the slab
    if (weights.size() != weights_uploaded)
      return fail(MU_ERR_INVALID, "Engine: this input shape needs parameters the first plan did not stage");
    return MU_OK;
  }
  rc = mu_alloc(ctx, std::max<size_t>(weight_bytes, 16), &weight_slab);
  if (rc) return fail(rc, "weight slab allocation of %zu bytes failed: %s", weight_bytes, mu_last_error(ctx));
  // upload weights: host-staged ones in one copy per contiguous run, device ones D2D
  for (size_t i = 0; i < weights.size(); ++i) {
    const Weight &w = weights[i];
    if (dev_weight[i] || w.bytes == 0) continue;
    if (cudaMemcpy(static_cast<char *>(weight_slab) + w.offset, weight_stage.data() + w.offset,
                   w.bytes, cudaMemcpyHostToDevice) != cudaSuccess)
      return fail(MU_ERR_CUDA, "weight upload failed: %s", cudaGetErrorString(cudaGetLastError()));
  }
  for (auto &d : dev_copies)
    if (cudaMemcpy2D(static_cast<char *>(weight_slab) + d.dst, d.dst_pitch, d.src, d.src_pitch, d.width,
                     d.rows, cudaMemcpyDeviceToDevice) != cudaSuccess)
      return fail(MU_ERR_CUDA, "weight copy failed: %s", cudaGetErrorString(cudaGetLastError()));
  std::vector<uint8_t>().swap(weight_stage);
  dev_copies.clear();
  weights_uploaded = weights.size();
  return MU_OK;
}

int mu_engine::launch_all(cudaStream_t st) {
  n_launches = 0;
  if (n_events > 0 && events.empty()) {
    events.resize(n_events);
    for (auto &ev : events)
      if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess)
        return fail(MU_ERR_CUDA, "event creation failed");
    if (cudaStreamCreateWithFlags(&side_stream, cudaStreamNonBlocking) != cudaSuccess)
      return fail(MU_ERR_CUDA, "stream creation failed");
  }
  for (const Op &op : ops) {
    // the second stream only ever runs work that waits on an event of `st`, and `st` waits on
    // every event the second stream records: both a plain run and a stream capture stay joined
    cudaStream_t s = op.side ? side_stream : st;
    if (op.wait_ev >= 0 && cudaStreamWaitEvent(s, events[op.wait_ev], 0) != cudaSuccess)
      return fail(MU_ERR_CUDA, "stream wait failed");
    // a chunked GEMM leaves a few SMs free: the all-reduce of the previous chunk runs beside it
    const bool chunked_gemm = op.kind == OP_LINEAR && op.budget;
    if (chunked_gemm) mu_ctx_set_sm_budget(ctx, std::max(2, mu_ctx_num_sms(ctx) - tp_comm_sms));
    int rc = launch_op(op, s);
    if (chunked_gemm) mu_ctx_set_sm_budget(ctx, 0);
    if (rc) return rc;
    if (op.rec_ev >= 0 && cudaEventRecord(events[op.rec_ev], s) != cudaSuccess)
      return fail(MU_ERR_CUDA, "event record failed");
  }
  return MU_OK;
}

int mu_engine::launch_op(const Op &op, cudaStream_t st) {
  {
    int rc = MU_OK;
    switch (op.kind) {
    case OP_EMBED:
      rc = mu_embedding(ctx, static_cast<const int32_t *>(tptr(op.in)), wptr(op.w), wptr(op.w2),
                        tptr(op.out), op.B, op.T, op.V, op.D, dtype, st);
      n_launches += 1;
      break;
    case OP_LN:
      rc = mu_layer_norm(ctx, tptr(op.in), wptr(op.w), wptr(op.b), tptr(op.out), op.M, op.N, op.eps,
                         dtype, st);
      n_launches += 1;
      break;
    case OP_LINEAR:
      if (op.pin >= 0) {
        if (!peer_arena)
          return fail(MU_ERR_INVALID, "Engine: the peer exchange needs mu_engine_attach_peer after compile");
        char *mirror = static_cast<char *>(peer_arena) +
                       (static_cast<char *>(rows(op.pin, op.row0, op.N)) - static_cast<char *>(arena));
        rc = mu_linear_mirrored(ctx, rows(op.in, op.row0, op.K), wptr(op.w), wptr(op.b),
                                rows(op.res, op.row0, op.N), rows(op.out, op.row0, op.N), mirror, op.M, op.K,
                                op.N, op.act, dtype, st);
        n_launches += 1;
        break;
      }
      rc = mu_linear(ctx, rows(op.in, op.row0, op.K), wptr(op.w), wptr(op.b), rows(op.res, op.row0, op.N),
                     rows(op.out, op.row0, op.N), op.M, op.K, op.N, op.act, dtype, st);
      n_launches += 1;
      break;
    case OP_QKV: {
      char *base = static_cast<char *>(tptr(op.out));
      const size_t per = static_cast<size_t>(op.B) * op.T * op.H * op.D * esize(dtype);
      rc = mu_linear_qkv_heads(ctx, tptr(op.in), wptr(op.w), wptr(op.b), base, base + per, base + 2 * per,
                               op.B, op.T, op.K, op.H, op.D, dtype, st);
      n_launches += 1;
      break;
    }
    case OP_ATTN: {
      char *base = static_cast<char *>(tptr(op.in));
      const size_t per = static_cast<size_t>(op.B) * op.T * op.H * op.D * esize(dtype);
      if (op.pin >= 0) {
        if (!peer_arena)
          return fail(MU_ERR_INVALID, "Engine: the peer exchange needs mu_engine_attach_peer after compile");
        char *mine = static_cast<char *>(tptr(op.pin)) + static_cast<size_t>(op.K) * esize(dtype);
        char *theirs = static_cast<char *>(peer_arena) + (mine - static_cast<char *>(arena));
        rc = mu_attention_mirrored(ctx, base, base + per, base + 2 * per, mine, op.N, theirs, op.B, op.H, op.T,
                                   op.D, op.causal, kmode, dtype, st);
        n_launches += 1;
        break;
      }
      rc = mu_attention(ctx, base, base + per, base + 2 * per, tptr(op.out), op.B, op.H, op.T, op.D,
                        op.causal, kmode, dtype, tptr(op.ws), op.ws_bytes, st);
      n_launches += op.ws_bytes ? 3 : 1; // composed path: scores, softmax, context; fused: one kernel
      break;
    }
    case OP_ELTWISE:
      rc = mu_eltwise(ctx, rows(op.in, op.row0, op.N), wptr(op.b), rows(op.res, op.row0, op.N),
                      rows(op.out, op.row0, op.N), op.n, op.b >= 0 ? op.N : 1, op.act, dtype, st);
      n_launches += 1;
      break;
    case OP_ALLREDUCE:
      rc = mu_all_reduce_sum(ctx, comm, rows(op.in, op.row0, op.N), op.n, dtype, st);
      n_launches += 1;
      break;
    case OP_ARGMAX:
      rc = mu_argmax(ctx, tptr(op.in), static_cast<int32_t *>(tptr(op.out)), op.M, op.N, dtype, st);
      n_launches += 1;
      break;
    case OP_CONV:
      rc = mu_conv2d(ctx, tptr(op.in), wptr(op.w), wptr(op.b), tptr(op.out), op.B, op.iC, op.iH, op.iW,
                     op.oC, op.ksz, op.stride, op.pad, op.relu, op.pool, dtype, st);
      n_launches += 1;
      break;
    case OP_MAXPOOL:
      rc = mu_max_pool2d(ctx, tptr(op.in), tptr(op.out), op.B, op.iC, op.iH, op.iW, op.ksz, op.stride,
                         op.pad, dtype, st);
      n_launches += 1;
      break;
    case OP_GAP:
      rc = mu_global_avg_pool(ctx, tptr(op.in), tptr(op.out), op.B, op.iC, op.iH, op.iW, dtype, st);
      n_launches += 1;
      break;
    case OP_LEAKY:
      rc = mu_leaky_relu(ctx, tptr(op.in), tptr(op.out), op.n, op.eps, dtype, st);
      n_launches += 1;
      break;
    case OP_RMSNORM:
      rc = mu_rms_norm(ctx, tptr(op.in), wptr(op.w), tptr(op.out), op.M, op.N, op.eps, dtype, st);
      n_launches += 1;
      break;
    case OP_BATCHNORM:
      rc = mu_batch_norm_eval(ctx, tptr(op.in), wptr(op.w), wptr(op.b), static_cast<const float *>(wptr(op.w2)),
                              static_cast<const float *>(wptr(op.b2)), tptr(op.out), op.B, op.iC, op.iH,
                              op.iW, op.eps, dtype, st);
      n_launches += 1;
      break;
    case OP_UPSAMPLE:
      rc = mu_upsample2d(ctx, tptr(op.in), tptr(op.out), op.B, op.iC, op.iH, op.iW, op.stride, dtype, st);
      n_launches += 1;
      break;
    case OP_JOIN:
      break;
    case OP_PEER_STEP:
    case OP_PEER_WAIT:
    case OP_PEER_SIGNAL:
    case OP_PEER_WAITRDY:
    case OP_PEER_SIGDONE:
    case OP_PEER_REDUCE: {
      if (!peer_arena || !peer_flags_remote)
        return fail(MU_ERR_INVALID, "Engine: the peer exchange needs mu_engine_attach_peer after compile");
      const unsigned per = static_cast<unsigned>(peer_exchanges), idx = static_cast<unsigned>(op.xidx);
      if (op.kind == OP_PEER_STEP) rc = mu_peer_step(ctx, peer_flags_local, st);
      else if (op.kind == OP_PEER_WAIT) rc = mu_peer_wait_done(ctx, peer_flags_local, per, idx, st);
      else if (op.kind == OP_PEER_SIGNAL) rc = mu_peer_signal(ctx, peer_flags_local, peer_flags_remote, per, idx, st);
      else if (op.kind == OP_PEER_WAITRDY) rc = mu_peer_wait_ready(ctx, peer_flags_local, per, idx, st);
      else if (op.kind == OP_PEER_SIGDONE) rc = mu_peer_signal_done(ctx, peer_flags_local, peer_flags_remote, per, idx, st);
      else {
        // both ranks planned the same arena: the peer's partial sits at the same offset in its arena
        const char *a = static_cast<const char *>(rows(op.in, op.row0, op.N));
        const char *a_peer = op.pin >= 0 ? static_cast<const char *>(tptr(op.pin)) // pushed by the peer
                                         : static_cast<const char *>(peer_arena) + (a - static_cast<const char *>(arena));
        rc = mu_peer_reduce(ctx, a, a_peer, wptr(op.b), rows(op.res, op.row0, op.N), rows(op.out, op.row0, op.N),
                            op.n, op.N, peer_flags_local, peer_flags_remote, per, idx, peer_ctas, st);
      }
      n_launches += 1;
      if (rc) return fail(rc, "peer exchange launch failed");
      break;
    }
    default:
      rc = MU_ERR_UNSUPPORTED;
    }
    if (rc) return fail(rc, "op launch failed: %s", mu_last_error(ctx));
  }
  return MU_OK;
}

// Algorithmic work of one op: FLOPs for contractions (attention counted
// causal-useful: only the unmasked half of the score square), bytes that must
// be read plus bytes that must be written once for the HBM-bound ops.
void mu_engine::op_work(const Op &op, double *flops, double *bytes) const {
  const double es = static_cast<double>(esize(dtype));
  *flops = 0, *bytes = 0;
  switch (op.kind) {
  case OP_LINEAR:
    *flops = 2.0 * op.M * op.K * op.N;
    *bytes = es * (1.0 * op.M * op.K + 1.0 * op.K * op.N + 1.0 * op.M * op.N * (op.res >= 0 ? 2 : 1));
    break;
  case OP_QKV:
    *flops = 2.0 * op.B * op.T * op.K * 3.0 * op.H * op.D;
    *bytes = es * (1.0 * op.B * op.T * (op.K + 3.0 * op.H * op.D) + 3.0 * op.K * op.H * op.D);
    break;
  case OP_ATTN: {
    const double sq = 1.0 * op.B * op.H * op.T * op.T * op.D;
    *flops = op.causal ? 2.0 * sq : 4.0 * sq; // QK' + PV, halved when causal
    *bytes = es * 4.0 * op.B * op.H * op.T * op.D;
    break;
  }
  case OP_LN:
    *bytes = es * 2.0 * op.M * op.N;
    break;
  case OP_EMBED:
    *bytes = es * 2.0 * op.B * op.T * op.D + 4.0 * op.B * op.T;
    break;
  case OP_ELTWISE:
    *bytes = es * op.n * (op.res >= 0 ? 3 : 2);
    break;
  case OP_ARGMAX:
    *bytes = es * op.M * op.N + 4.0 * op.M;
    break;
  case OP_ALLREDUCE:
    *bytes = es * op.n; // bytes each rank contributes
    break;
  case OP_PEER_REDUCE:
    *bytes = es * op.n; // bytes read from the peer over NVLink
    break;
  case OP_CONV: {
    const double oH = (op.iH + 2 * op.pad - op.ksz) / op.stride + 1, oW = (op.iW + 2 * op.pad - op.ksz) / op.stride + 1;
    *flops = 2.0 * op.B * op.oC * oH * oW * op.iC * op.ksz * op.ksz;
    *bytes = 4.0 * (1.0 * op.B * op.iC * op.iH * op.iW + 1.0 * op.oC * op.iC * op.ksz * op.ksz +
                    1.0 * op.B * op.oC * oH * oW / (op.pool == 2 ? 4 : 1));
    break;
  }
  case OP_MAXPOOL:
  case OP_GAP:
    *bytes = 4.0 * op.B * op.iC * op.iH * op.iW;
    break;
  case OP_LEAKY:
    *bytes = es * 2.0 * op.n;
    break;
  case OP_RMSNORM:
    *bytes = es * 2.0 * op.M * op.N;
    break;
  case OP_BATCHNORM:
    *bytes = es * 2.0 * op.B * op.iC * op.iH * op.iW;
    break;
  case OP_UPSAMPLE:
    *bytes = es * (1.0 + op.stride * op.stride) * op.B * op.iC * op.iH * op.iW;
    break;
  default:
    break;
  }
}

extern "C" {

// Eager (graph-free) forward with a CUDA-event pair around every op, `reps`
// times; reports per-op mean milliseconds, kind and algorithmic work.
// kinds: 0 embed, 1 layer_norm, 2 linear, 3 qkv linear, 4 attention, 5 eltwise, 6 argmax,
// 7 conv2d, 8 max_pool2d, 9 global_avg_pool.
int mu_engine_profile(mu_engine *e, int reps, int capacity, int *n_ops, int *kinds, float *ms,
                      double *flops, double *bytes, void *stream) {
  if (!e || !e->compiled || reps <= 0) return MU_ERR_INVALID;
  const int n = static_cast<int>(e->ops.size());
  if (n_ops) *n_ops = n;
  if (capacity < n) return e->fail(MU_ERR_SIZE, "profile: capacity %d < %d ops", capacity, n);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  std::vector<cudaEvent_t> ev(2 * static_cast<size_t>(n));
  for (auto &x : ev)
    if (cudaEventCreate(&x) != cudaSuccess) return e->fail(MU_ERR_CUDA, "event creation failed");
  std::vector<double> acc(n, 0.0);
  int rc = MU_OK;
  for (int r = 0; r < reps && rc == MU_OK; ++r) {
    for (int i = 0; i < n && rc == MU_OK; ++i) {
      cudaEventRecord(ev[2 * i], st);
      rc = e->launch_op(e->ops[i], st);
      cudaEventRecord(ev[2 * i + 1], st);
    }
    if (rc == MU_OK) rc = mu_check(e->ctx, st);
    if (rc) break;
    for (int i = 0; i < n; ++i) {
      float t = 0;
      cudaEventElapsedTime(&t, ev[2 * i], ev[2 * i + 1]);
      acc[i] += t;
    }
  }
  for (auto &x : ev) cudaEventDestroy(x);
  if (rc) return rc;
  for (int i = 0; i < n; ++i) {
    kinds[i] = static_cast<int>(e->ops[i].kind);
    ms[i] = static_cast<float>(acc[i] / reps);
    e->op_work(e->ops[i], &flops[i], &bytes[i]);
  }
  return MU_OK;
}

// GEMM geometry of every op of the active plan, four ints per op: M, K, N and 1 when a residual
// is added in the epilogue (zeros for ops that are not linears). Lets a caller group the timings
// of mu_engine_profile by problem shape.
int mu_engine_op_dims(const mu_engine *e, int capacity, int *dims) {
  if (!e || !e->compiled || !dims) return MU_ERR_INVALID;
  const int n = static_cast<int>(e->ops.size());
  if (capacity < n) return MU_ERR_SIZE;
  for (int i = 0; i < n; ++i) {
    const Op &op = e->ops[i];
    int *d = dims + 4 * i;
    d[0] = d[1] = d[2] = d[3] = 0;
    if (op.kind == OP_LINEAR) d[0] = op.M, d[1] = op.K, d[2] = op.N, d[3] = op.res >= 0 ? 1 : 0;
    else if (op.kind == OP_QKV) d[0] = op.B * op.T, d[1] = op.K, d[2] = 3 * op.H * op.D;
  }
  return MU_OK;
}

int mu_engine_create(mu_ctx *ctx, mu_engine **out) {
  if (!ctx || !out) return MU_ERR_INVALID;
  mu_engine *e = new (std::nothrow) mu_engine();
  if (!e) return MU_ERR_NOMEM;
  e->ctx = ctx;
  *out = e;
  return MU_OK;
}

void mu_engine_destroy(mu_engine *e) {
  if (!e) return;
  e->release_compiled();
  delete e;
}

const char *mu_engine_last_error(const mu_engine *e) { return e ? e->err : "null engine"; }

int mu_engine_set_option(mu_engine *e, const char *name, int value) {
  if (!e || !name) return MU_ERR_INVALID;
  const std::string n(name);
  if (n == "kmode") {
    if (value != MU_K_LITERAL && value != MU_K_MATH) return e->fail(MU_ERR_INVALID, "kmode must be 0 or 1");
    e->kmode = value;
  } else if (n == "use_graph") e->use_graph = value;
  else if (n == "argmax") e->want_argmax = value;
  else if (n == "tp_rank") e->tp_rank = value;
  else if (n == "tp_size") e->tp_size = value;
  else if (n == "tp_overlap") e->tp_overlap = value;
  else if (n == "tp_comm_sms") e->tp_comm_sms = value;
  else if (n == "plan_cache_entries") e->plan_cache_entries = value;
  else if (n == "tp_exchange") e->tp_exchange = value;
  else return e->fail(MU_ERR_INVALID, "unknown option '%s'", name);
  return MU_OK;
}

static int finish_load(mu_engine *e, int compute_dtype) {
  if (compute_dtype != MU_F32 && compute_dtype != MU_BF16)
    return e->fail(MU_ERR_UNSUPPORTED, "compute dtype %d not implemented (float32, bfloat16)", compute_dtype);
  e->dtype = compute_dtype;
  e->loaded = true;
  return MU_OK;
}

int mu_engine_load(mu_engine *e, const char *path, int compute_dtype) {
  if (!e || !path) return MU_ERR_INVALID;
  e->release_compiled();
  e->params.clear();
  e->loaded = false;
  std::string why;
  if (!mu::load_artifact(path, &e->config, &e->params, &why))
    return e->fail(MU_ERR_INVALID, "%s", why.c_str());
  return finish_load(e, compute_dtype);
}

int mu_engine_load_memory(mu_engine *e, const char *config_json, int n_tensors,
                          const char *const *names, const void *const *data, const int *dtypes,
                          const int *ndims, const long long *shapes, int on_device,
                          int compute_dtype) {
  if (!e || !config_json || n_tensors < 0) return MU_ERR_INVALID;
  e->release_compiled();
  e->params.clear();
  e->loaded = false;
  std::string why;
  if (!mu::parse_json(config_json, &e->config, &why))
    return e->fail(MU_ERR_INVALID, "config JSON: %s", why.c_str());
  size_t s = 0;
  for (int i = 0; i < n_tensors; ++i) {
    NamedTensor t;
    t.dtype = dtypes[i];
    for (int d = 0; d < ndims[i]; ++d) t.shape.push_back(shapes[s++]);
    t.data = data[i];
    t.on_device = on_device != 0;
    e->params[names[i]] = std::move(t);
  }
  return finish_load(e, compute_dtype);
}

// Communicator for the tensor-parallel all-reduces (options "tp_size"/"tp_rank" select the shard).
int mu_engine_set_comm(mu_engine *e, mu_comm *comm) {
  if (!e) return MU_ERR_INVALID;
  e->comm = comm;
  return MU_OK;
}

// Lower, plan and capture the forward for one concrete input shape into the active plan
// (which must be empty). The weights are staged and uploaded by the first plan only.
int mu_engine::build_plan(const std::vector<int> &shape, int input_dtype) {
  Val v;
  v.shape = shape;
  v.dtype = input_dtype;
  in_shape = v.shape, in_dtype = input_dtype;
  input_bytes = static_cast<size_t>(v.numel()) * esize(input_dtype);
  v.tid = new_tensor(input_bytes);
  tensors[v.tid].external = true;
  const bool first = weight_slab == nullptr;
  used_params.clear();
  peer_exchanges = 0;
  peer_in[0] = peer_in[1] = -1;
  if (tp_exchange && tp_size > 1) {
    if (tp_size != 2) return fail(MU_ERR_UNSUPPORTED, "Engine: the peer-memory exchange is built for two ranks");
    if (dtype != MU_BF16) return fail(MU_ERR_UNSUPPORTED, "Engine: the peer-memory exchange is built for bfloat16");
    Op stp;
    stp.kind = OP_PEER_STEP;
    push(stp);
    // nothing of this forward may overwrite arena bytes the peer could still be reading from the
    // previous forward's last exchange
    Op w;
    w.kind = OP_PEER_WAIT, w.xidx = 0;
    push(w);
    peer_last_partial = -1;
  }
  int rc = lower(config, "", v, nullptr, nullptr);
  if (rc) return rc;
  // Every serialized tensor must belong to a module of the tree, as in the reference's loader
  // (src/inference_serialization.cpp:1043-1051). BatchNorm2d's momentum-only state and Dropout
  // have no tensors, so anything left over is a mismatch between config and payload.
  if (first)
    for (const auto &kv : params)
      if (!used_params.count(kv.first))
        return fail(MU_ERR_INVALID,
                    "Serialized tensor '%s' does not match any named parameter/buffer in the "
                    "reconstructed module", kv.first.c_str());
  out_tid = v.tid, out_shape = v.shape, out_dtype = v.dtype;
  if (want_argmax) {
    Op a;
    a.kind = OP_ARGMAX, a.N = v.shape.back(), a.M = static_cast<int>(v.numel() / a.N);
    a.in = v.tid, a.out = new_tensor(static_cast<size_t>(a.M) * 4);
    push(a);
    argmax_tid = a.out;
  }
  // the outputs stay live to the end of the plan
  const int last = static_cast<int>(ops.size());
  touch(out_tid, last);
  if (argmax_tid >= 0) touch(argmax_tid, last);
  if (peer_last_partial >= 0) touch(peer_last_partial, last);
  for (int t : peer_in) touch(t, last);
  rc = plan_and_allocate();
  if (rc) return rc;
  if (tp_exchange && tp_size > 1) {
    // the peer's arena and counters are not known yet: mu_engine_attach_peer warms up and captures
    rc = mu_alloc(ctx, mu_peer_flags_bytes(), &peer_flags_local);
    if (rc) return fail(rc, "peer counter allocation failed: %s", mu_last_error(ctx));
    if (cudaMemset(peer_flags_local, 0, mu_peer_flags_bytes()) != cudaSuccess)
      return fail(MU_ERR_CUDA, "peer counter clear failed");
    return MU_OK;
  }
  return capture_graph();
}

// Warm-up forward (sets per-kernel attributes), then capture and instantiate the graph of the
// active plan. Under a peer exchange both ranks run this at the same time (the warm-up forward is
// a real exchange).
int mu_engine::capture_graph() {
  if (!use_graph) return MU_OK;
  int rc;
  {
    if (!cap_stream && cudaStreamCreateWithFlags(&cap_stream, cudaStreamNonBlocking) != cudaSuccess)
      return fail(MU_ERR_CUDA, "stream creation failed");
    // warm-up launch outside capture (sets per-kernel attributes), then capture
    rc = launch_all(cap_stream);
    if (rc) return rc;
    rc = mu_check(ctx, cap_stream);
    if (rc) return fail(rc, "warm-up forward failed: %s", mu_last_error(ctx));
    if (cudaStreamBeginCapture(cap_stream, cudaStreamCaptureModeThreadLocal) != cudaSuccess)
      return fail(MU_ERR_CUDA, "graph capture could not start");
    rc = launch_all(cap_stream);
    cudaError_t ce = cudaStreamEndCapture(cap_stream, &graph);
    if (rc) return rc;
    if (ce != cudaSuccess) return fail(MU_ERR_CUDA, "graph capture failed: %s", cudaGetErrorString(ce));
    ce = cudaGraphInstantiate(&gexec, graph, 0);
    if (ce != cudaSuccess) return fail(MU_ERR_CUDA, "graph instantiate failed: %s", cudaGetErrorString(ce));
  }
  return MU_OK;
}

// Why `actual` breaks the contract, in the reference's words (ShapeContract::mismatch_reason,
// src/inference.hpp:162-176); nullptr when it fits.
static const char *contract_mismatch(const std::vector<int> &contract, const int *actual, int ndim,
                                     int *index) {
  if (static_cast<int>(contract.size()) != ndim) return "rank mismatch";
  for (int i = 0; i < ndim; ++i)
    if (contract[i] != -1 && contract[i] != actual[i]) {
      *index = i;
      return "dim mismatch at index";
    }
  return nullptr;
}

int mu_engine_compile_contract(mu_engine *e, const int *example_shape, int ndim,
                               const int *expected_shape, int input_dtype) {
  if (!e || !example_shape || ndim <= 0) return MU_ERR_INVALID;
  if (!e->loaded) return e->fail(MU_ERR_INVALID, "Engine: no module loaded");
  if (e->tp_size < 1 || e->tp_rank < 0 || e->tp_rank >= e->tp_size)
    return e->fail(MU_ERR_INVALID, "Engine: bad tensor-parallel rank %d of %d", e->tp_rank, e->tp_size);
  if (e->tp_size > 1 && (!e->comm || mu_comm_world(e->comm) != e->tp_size))
    return e->fail(MU_ERR_INVALID, "Engine: tp_size %d needs a communicator of that size", e->tp_size);
  if (e->tp_size > 1 && e->kmode == MU_K_LITERAL)
    // literal K addressing reinterprets the WHOLE head-major K buffer ([B*H*T, D] read as
    // [D, B*H*T]), so a score mixes rows of every head: it does not commute with sharding heads
    return e->fail(MU_ERR_UNSUPPORTED,
                   "Engine: tensor parallelism needs kmode = MU_K_MATH (literal K addressing reads "
                   "across all heads and cannot be sharded by head)");
  if (e->tp_size > 1 && e->want_argmax)
    return e->fail(MU_ERR_UNSUPPORTED, "Engine: argmax over a vocabulary-sharded head is not implemented");
  for (int i = 0; i < ndim; ++i)
    if (example_shape[i] <= 0)
      return e->fail(MU_ERR_INVALID, "Engine: compile needs a concrete positive input shape");
  if (input_dtype != MU_I32 && input_dtype != e->dtype)
    return e->fail(MU_ERR_INVALID, "Engine: input dtype %d does not match compute dtype %d", input_dtype, e->dtype);
  std::vector<int> contract(example_shape, example_shape + ndim);
  if (expected_shape) {
    contract.assign(expected_shape, expected_shape + ndim);
    for (int i = 0; i < ndim; ++i)
      if (contract[i] != -1 && contract[i] <= 0)
        return e->fail(MU_ERR_INVALID, "Engine: expected input shape holds positive extents or -1");
    int idx = 0;
    if (const char *why = contract_mismatch(contract, example_shape, ndim, &idx))
      return e->fail(MU_ERR_INVALID, "Engine compile input shape mismatch: %s %d", why, idx);
  }
  // The weights staged by an earlier compile() stay in their slab (the sources they were read
  // from may be gone by now); only the plans are rebuilt. Options that change which slices of
  // the parameters a rank holds ("tp_size", "tp_rank") therefore belong before the first compile.
  e->release_plans();
  e->contract = contract;
  int rc = e->build_plan(std::vector<int>(example_shape, example_shape + ndim), input_dtype);
  if (rc) {
    e->contract.clear();
    return rc;
  }
  e->compiled = true;
  return MU_OK;
}

int mu_engine_compile(mu_engine *e, const int *input_shape, int ndim, int input_dtype) {
  return mu_engine_compile_contract(e, input_shape, ndim, nullptr, input_dtype);
}

// Make the plan of `shape` the active one: the active plan itself, a parked one, or a new one
// (lowered, planned and captured now; the least recently used plan is dropped beyond
// "plan_cache_entries"). The shape must satisfy the compile-time contract.
int mu_engine_select_shape(mu_engine *e, const int *shape, int ndim) {
  if (!e || !shape || ndim <= 0) return MU_ERR_INVALID;
  if (!e->compiled) return e->fail(MU_ERR_INVALID, "Engine: run() called before compile()");
  int idx = 0;
  if (const char *why = contract_mismatch(e->contract, shape, ndim, &idx)) {
    if (why[0] == 'r') return e->fail(MU_ERR_INVALID, "Engine run input shape mismatch: %s", why);
    return e->fail(MU_ERR_INVALID, "Engine run input shape mismatch: %s %d", why, idx);
  }
  for (int i = 0; i < ndim; ++i)
    if (shape[i] <= 0) return e->fail(MU_ERR_INVALID, "Engine: input extents must be positive");
  const std::vector<int> want(shape, shape + ndim);
  ++e->use_clock;
  if (want == e->in_shape) return MU_OK;
  if (e->peer_flags_local)
    return e->fail(MU_ERR_UNSUPPORTED, "Engine: one plan per engine under the peer-memory exchange");
  const int in_dtype = e->in_dtype;
  e->park_active();
  for (size_t i = 0; i < e->parked.size(); ++i)
    if (e->parked[i].in_shape == want) {
      e->activate(i);
      return MU_OK;
    }
  // room for one more: drop the least recently used plans
  while (static_cast<int>(e->parked.size()) + 1 > std::max(1, e->plan_cache_entries)) {
    size_t lru = 0;
    for (size_t i = 1; i < e->parked.size(); ++i)
      if (e->parked[i].last_used < e->parked[lru].last_used) lru = i;
    e->free_plan(e->parked[lru]);
    e->parked.erase(e->parked.begin() + static_cast<long>(lru));
  }
  int rc = e->build_plan(want, in_dtype);
  if (rc) {
    // fall back to a plan that works so that the engine stays usable
    e->release_active_plan();
    if (!e->parked.empty()) e->activate(e->parked.size() - 1);
    else e->compiled = false;
    return rc;
  }
  return MU_OK;
}

int mu_engine_plan_count(const mu_engine *e) {
  return (e && e->compiled) ? static_cast<int>(e->parked.size()) + 1 : 0;
}

// Peer-memory exchange (option "tp_exchange" = 1, two ranks): after compile each rank exports its
// arena and its counters (mu_engine_peer_info + mu_ipc_export), the host hands the handles to the
// other rank, which opens them (mu_ipc_open) and attaches the mappings here. Attaching runs the
// warm-up forward and captures the graph, so both ranks must call it at the same time.
int mu_engine_peer_info(const mu_engine *e, void **arena, void **counters) {
  if (!e || !e->compiled || !e->peer_flags_local || !arena || !counters) return MU_ERR_INVALID;
  *arena = e->arena, *counters = e->peer_flags_local;
  return MU_OK;
}

int mu_engine_attach_peer(mu_engine *e, void *peer_arena, void *peer_counters) {
  if (!e || !peer_arena || !peer_counters) return MU_ERR_INVALID;
  if (!e->compiled || !e->peer_flags_local)
    return e->fail(MU_ERR_INVALID, "Engine: attach_peer needs a compiled engine with tp_exchange = 1 or 2");
  e->peer_arena = peer_arena, e->peer_flags_remote = peer_counters;
  const int sms = mu_ctx_num_sms(e->ctx);
  // four CTAs of 512 threads per SM: with eight loads each in flight, 20 SMs keep ~5 MB on the wire
  e->peer_ctas = static_cast<unsigned>(4 * (e->tp_overlap ? std::max(1, e->tp_comm_sms) : sms));
  int rc = mu_peer_arm(e->ctx, e->peer_flags_local, e->peer_ctas, nullptr);
  if (rc == MU_OK) rc = mu_check(e->ctx, nullptr);
  if (rc) return e->fail(rc, "peer counter set-up failed: %s", mu_last_error(e->ctx));
  return e->capture_graph();
}

int mu_engine_output_shape(const mu_engine *e, int *shape, int *ndim, int *dtype) {
  if (!e || !e->compiled || !shape || !ndim) return MU_ERR_INVALID;
  *ndim = static_cast<int>(e->out_shape.size());
  for (size_t i = 0; i < e->out_shape.size() && i < 8; ++i) shape[i] = e->out_shape[i];
  if (dtype) *dtype = e->out_dtype;
  return MU_OK;
}

int mu_engine_stats(const mu_engine *e, long long *arena_bytes, long long *weight_bytes,
                    long long *n_ops, long long *n_launches, long long *unplanned_bytes) {
  if (!e || !e->compiled) return MU_ERR_INVALID;
  if (arena_bytes) *arena_bytes = static_cast<long long>(e->arena_bytes);
  if (weight_bytes) *weight_bytes = static_cast<long long>(e->weight_bytes);
  if (n_ops) *n_ops = static_cast<long long>(e->ops.size());
  if (n_launches) *n_launches = e->n_launches;
  if (unplanned_bytes) {
    long long s = 0;
    for (auto &t : e->tensors)
      if (t.alias_of < 0 && !t.external) s += static_cast<long long>(t.bytes);
    *unplanned_bytes = s;
  }
  return MU_OK;
}

// Engine::run (src/inference.hpp:541-610): strict input contract, forward, output.
// input/output may be host or device pointers; argmax_out (optional) receives
// int32 indices over the last dim when the "argmax" option is set.
int mu_engine_run(mu_engine *e, const void *input, int input_on_host, void *output,
                  int output_on_host, int32_t *argmax_out, int argmax_on_host, void *stream) {
  if (!e) return MU_ERR_INVALID;
  if (!e->compiled) return e->fail(MU_ERR_INVALID, "Engine: run() called before compile()");
  if (!input) return e->fail(MU_ERR_INVALID, "Engine: null input");
  if (e->peer_flags_local && !e->peer_arena)
    return e->fail(MU_ERR_INVALID, "Engine: the peer exchange needs mu_engine_attach_peer before run()");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int rc = mu_copy(e->ctx, e->input_buf, input, e->input_bytes,
                   input_on_host ? MU_COPY_H2D : MU_COPY_D2D, st);
  if (rc) return e->fail(rc, "input copy failed: %s", mu_last_error(e->ctx));
  if (e->gexec) {
    cudaError_t ce = cudaGraphLaunch(e->gexec, st);
    if (ce != cudaSuccess) return e->fail(MU_ERR_CUDA, "graph launch failed: %s", cudaGetErrorString(ce));
  } else {
    rc = e->launch_all(st);
    if (rc) return rc;
  }
  if (output) {
    size_t bytes = esize(e->out_dtype);
    for (int s : e->out_shape) bytes *= s;
    rc = mu_copy(e->ctx, output, e->tptr(e->out_tid), bytes, output_on_host ? MU_COPY_D2H : MU_COPY_D2D, st);
    if (rc) return e->fail(rc, "output copy failed: %s", mu_last_error(e->ctx));
  }
  if (argmax_out && e->argmax_tid >= 0) {
    size_t rows = 1;
    for (size_t i = 0; i + 1 < e->out_shape.size(); ++i) rows *= e->out_shape[i];
    rc = mu_copy(e->ctx, argmax_out, e->tptr(e->argmax_tid), rows * 4,
                 argmax_on_host ? MU_COPY_D2H : MU_COPY_D2D, st);
    if (rc) return e->fail(rc, "argmax copy failed: %s", mu_last_error(e->ctx));
  }
  if (output_on_host || (argmax_out && argmax_on_host)) {
    rc = mu_check(e->ctx, st);
    if (rc) return e->fail(rc, "%s", mu_last_error(e->ctx));
  }
  return MU_OK;
}

// Device address of the planned output (valid until the next compile); lets a
// caller consume logits in place instead of copying 4 GB around.
void *mu_engine_output_ptr(const mu_engine *e) { return (e && e->compiled) ? e->tptr(e->out_tid) : nullptr; }
void *mu_engine_argmax_ptr(const mu_engine *e) {
  return (e && e->compiled && e->argmax_tid >= 0) ? e->tptr(e->argmax_tid) : nullptr;
}

} // extern "C"
