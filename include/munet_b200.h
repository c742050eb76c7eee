/* munet_b200 — C ABI of the B200 (sm_100a) forward-inference kernels.
 *
 * This is the thin boundary a MuNet device backend binds to: plain pointers and
 * sizes, no C++ or torch types.  Every function returns an int status
 * (MU_OK == 0), never throws and never exits; mu_last_error(ctx) gives the text
 * of the last failure on that context.  All compute entry points are
 * asynchronous on the `stream` argument (a cudaStream_t passed as void*, NULL =
 * the legacy default stream).  Device-side faults that cannot be known at
 * launch time (a bounded wait that ran out, an out-of-range embedding id) are
 * latched in a per-context status word and reported by mu_check().
 *
 * Threading: a context may be used from any host thread, by one thread at a time
 * (its error text and its SM budget are per-context state); kernels of different
 * contexts and of different streams of one context run concurrently. An engine
 * belongs to the context it was created on and is driven by one thread at a time.
 *
 * Citations name the interface of the reference (bryan-pakulski/MuNet, paths
 * relative to its checkout) that each entry point stands in for.
 *
 * dtype codes follow the reference DataType enum order (src/types.hpp:16).
 */
#ifndef MUNET_B200_H
#define MUNET_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MU_ABI_VERSION 1

enum mu_status {
  MU_OK = 0,
  MU_ERR_INVALID = 1,     /* bad argument (null pointer, negative size, …) */
  MU_ERR_UNSUPPORTED = 2, /* dtype / mode this build does not implement */
  MU_ERR_CUDA = 3,        /* a CUDA runtime / driver call failed */
  MU_ERR_TIMEOUT = 4,     /* a bounded device-side wait ran out */
  MU_ERR_INDEX = 5,       /* embedding id out of range */
  MU_ERR_NOMEM = 6,
  MU_ERR_SIZE = 7         /* size beyond a documented maximum */
};

enum mu_dtype { MU_F32 = 0, MU_F16 = 1, MU_BF16 = 2, MU_I32 = 3 };

/* Activation modules (src/nn/activations.hpp): GELU is x*sigmoid(1.702x),
 * Tanh is sigmoid(2x)*2-1, exactly as the reference composes them. */
enum mu_act { MU_ACT_NONE = 0, MU_ACT_RELU = 1, MU_ACT_GELU = 2, MU_ACT_SIGMOID = 3, MU_ACT_TANH = 4 };

/* How attention scores address K (src/nn/attention.hpp:64).
 * MU_K_LITERAL reproduces the reference bit-for-bit in structure: its
 * `k.transpose(0,1)` is a stride-only view and its matmul ignores strides, so
 * scores are sum_d Q[i,d] * Kbuf[d*N + j] with N = B*H*T.
 * MU_K_MATH is the textbook Q·K^T. */
enum mu_kmode { MU_K_LITERAL = 0, MU_K_MATH = 1 };

enum mu_copy_kind { MU_COPY_H2D = 1, MU_COPY_D2H = 2, MU_COPY_D2D = 3 };

typedef struct mu_ctx mu_ctx;

/* ---- context, memory, synchronisation -------------------------------------
 * Replaces Backend construction per (type,index) (src/backend/backend_manager.cpp:102-123)
 * and Backend::allocate / deallocate / copy / synchronize
 * (src/core/backend.hpp:207-232; CUDA reference src/backend/cuda_backend.cu:842-961). */
int mu_abi_version(void);
int mu_ctx_create(int device, mu_ctx **out);
void mu_ctx_destroy(mu_ctx *ctx);
const char *mu_last_error(const mu_ctx *ctx);
int mu_ctx_num_sms(const mu_ctx *ctx);
/* force every matmul onto the CUDA-core kernel (debug / A-B checks); 0 restores */
int mu_ctx_force_simt(mu_ctx *ctx, int on);
/* Persistent GEMM kernels launch one CTA per SM; n > 0 limits them to n SMs so that a kernel
 * running beside them (a collective on another stream) finds free SMs. 0 = all SMs. */
int mu_ctx_set_sm_budget(mu_ctx *ctx, int n);
/* Tuning knob: the bf16 tensor-core GEMM picks its tile (128 x 64/128/256 on one CTA, 256 x 128/256
 * on a CTA pair) from the problem size and the SM count; bn > 0 fixes the tile width and `ctas`
 * (1 or 2) the CTA count for every later GEMM of this context. 0, 0 restores the automatic choice.
 * Results do not depend on the tile shape (same accumulation order per output element). */
int mu_ctx_set_gemm_tile(mu_ctx *ctx, int bn, int ctas);
/* L2 set-aside for weights. `bytes` of the L2 of the context's device are reserved for cache lines
 * loaded with the evict_last priority (cudaLimitPersistingL2CacheSize of the calling process's CUDA
 * context: it ends with the process and changes nothing on the GPU for anyone else); the bf16
 * tensor-core GEMM then keeps a weight matrix that fits (fc1 / fc2 of the decoder: 33.5 MB) in L2
 * while activations and outputs stream past it, instead of re-fetching part of it for every wave
 * of tiles. Measured on the 24-layer decoder at 65 536 tokens with 40 MB: DRAM traffic of the GEMMs
 * 1.18 -> 1.03 of the algorithmic bytes, step time unchanged (the GEMMs gain what LayerNorm loses
 * to the smaller remaining L2). 0 turns it off (the default: the limit is process-wide, so the
 * application decides). Results do not change. */
int mu_ctx_set_l2_set_aside(mu_ctx *ctx, size_t bytes);
int mu_alloc(mu_ctx *ctx, size_t bytes, void **ptr);
int mu_free(mu_ctx *ctx, void *ptr);
int mu_copy(mu_ctx *ctx, void *dst, const void *src, size_t bytes, int kind, void *stream);
/* Backend::memset (src/core/backend.hpp:209; CUDA reference src/backend/cuda_backend.cu:946-950):
 * every byte of [ptr, ptr+bytes) becomes (unsigned char)value, asynchronous on `stream`. */
int mu_memset(mu_ctx *ctx, void *ptr, int value, size_t bytes, void *stream);
/* Backend::to_contiguous (src/core/backend.hpp:224-226; CPU kernel
 * src/backend/cpu_backend.hpp:1139-1156): dst[row-major index] = src[offset + sum idx_d *
 * strides_d] for a view of up to 6 dimensions; strides and offset in elements, elem_size in
 * bytes (1, 2, 4 or 8 — whatever the dtype). Views whose last dimension is contiguous (the
 * head split / merge permutes of attention) move 16 bytes per thread. */
int mu_to_contiguous(mu_ctx *ctx, const void *src, void *dst, int ndim, const int *shape,
                     const long long *strides, long long offset, int elem_size, void *stream);
/* Backend::get_last_kernel_time_us (src/core/backend.hpp:231; the CUDA reference brackets each
 * kernel with an event pair, src/backend/cuda_backend.cu:952-961): mu_timer_begin / mu_timer_end
 * record the context's event pair on `stream` around whatever the caller enqueues in between;
 * mu_timer_last_us waits for the closing event and returns the device time in microseconds
 * (0 when no bracket has been closed). */
int mu_timer_begin(mu_ctx *ctx, void *stream);
int mu_timer_end(mu_ctx *ctx, void *stream);
double mu_timer_last_us(mu_ctx *ctx);
int mu_synchronize(mu_ctx *ctx);
/* Synchronise `stream`, then report and clear the latched device status. */
int mu_check(mu_ctx *ctx, void *stream);

/* ---- BLAS capability -------------------------------------------------------
 * BackendBlasCapability::matmul / batched_matmul (src/core/backend.hpp:250-260):
 * C[M,N] = op(A)·op(B), row-major. transA is a training-only path
 * (autograd) and returns MU_ERR_UNSUPPORTED. stride_b == 0 broadcasts B. */
int mu_matmul(mu_ctx *ctx, const void *a, const void *b, void *c, int M, int K, int N,
              int transA, int transB, int dtype, void *stream);
int mu_batched_matmul(mu_ctx *ctx, const void *a, const void *b, void *c, int batch, int M, int K,
                      int N, int transA, int transB, long long stride_a, long long stride_b,
                      long long stride_out, int dtype, void *stream);

/* ---- fused Linear ----------------------------------------------------------
 * nn::Linear::forward_impl (src/nn/linear.hpp:28-34) = matmul + broadcast add,
 * fused with the activation module that follows it in a Sequential and with the
 * residual add of a decoder block (demos/multigpu/gpt3_multi_gpu_demo.py:106-113):
 *   y[M,N] = act(x[M,K]·w[K,N] + bias[N]) + residual[M,N]
 * bias and residual may be NULL. w is [in_features, out_features] row-major. */
int mu_linear(mu_ctx *ctx, const void *x, const void *w, const void *bias, const void *residual,
              void *y, int M, int K, int N, int act, int dtype, void *stream);

/* Fused q/k/v projections of nn::MultiHeadAttention (src/nn/attention.hpp:46-62):
 * x[B*T,E]·w[E,3E] + bias[3E] with w = [q_proj.weight | k_proj.weight | v_proj.weight]
 * concatenated on the output axis; the result is written head-major, i.e. what
 * reshape[B,T,H,D].permute(0,2,1,3).contiguous() produces: q,k,v each [B*H*T, D]. */
int mu_linear_qkv(mu_ctx *ctx, const void *x, const void *w_qkv, const void *bias_qkv, void *q,
                  void *k, void *v, int B, int T, int E, int H, int dtype, void *stream);

/* Same with the input width separate from the produced heads: w is [K_in, 3*H*D]. Used
 * for a tensor-parallel shard that computes H = num_heads / tp_size of the heads. */
int mu_linear_qkv_heads(mu_ctx *ctx, const void *x, const void *w_qkv, const void *bias_qkv, void *q,
                        void *k, void *v, int B, int T, int K_in, int H, int D, int dtype,
                        void *stream);

/* ---- attention core --------------------------------------------------------
 * The scale / mask / softmax / P·V part of MultiHeadAttention::forward_impl
 * (src/nn/attention.hpp:64-99) on head-major q,k,v [B*H*T, D]; `out` is the merged
 * token-major context [B*T, H*D] that feeds out_proj. Block-diagonal masking is
 * implicit (each head attends to itself only). workspace: mu_attention_workspace_bytes. */
size_t mu_attention_workspace_bytes(int B, int H, int T, int D, int dtype);
/* mu_attention_workspace_bytes returns 0 where the fused kernel applies (bfloat16, D 64 or 128,
 * T a multiple of 8). A context switched to the CUDA-core kernels (mu_ctx_force_simt) takes the
 * composed GEMM -> softmax -> GEMM path for every shape and always needs the [B*H,T,T] score
 * buffer: this returns that size (0 if it would not fit in 2^46 bytes or B*H*T exceeds 2^31-1,
 * which mu_attention rejects with MU_ERR_SIZE). */
size_t mu_attention_workspace_bytes_composed(int B, int H, int T, int D, int dtype);
int mu_attention(mu_ctx *ctx, const void *q, const void *k, const void *v, void *out, int B, int H,
                 int T, int D, int causal, int kmode, int dtype, void *workspace,
                 size_t workspace_bytes, void *stream);

/* ---- attention core without any allocation ---------------------------------
 * No counterpart in the reference. For callers that may not allocate device
 * memory at all (a latency-critical loop that must stay off the allocator's
 * lock, a process with a memory budget fixed up front, a host that owns every
 * byte and only lends pointers): the same computation as mu_attention's composed
 * path, with the [B*H,T,T] score matrix kept in an array that is part of the
 * library image (MU_ATTENTION_STATIC_SCRATCH_BYTES on every device that loads the
 * library, until process exit). It takes no context and calls no cudaMalloc,
 * cudaFree or allocating library routine.
 *  - B*H*T*T*sizeof(dtype) beyond the array is rejected with MU_ERR_SIZE (checked without
 *    overflow, before anything is launched).
 *  - The launches need `device` current; the caller's current device is restored on return.
 *  - The first call on a device looks the array up (cudaGetSymbolAddress with
 *    that device current); make that first call before any stream capture.
 *  - All calls share the array: two calls whose kernels overlap on the GPU
 *    (different streams, or concurrent host threads) race. Serialise them.
 *  - sync_and_check != 0 synchronises `stream` and reports a latched device fault;
 *    with 0 the call is asynchronous and such a fault goes unreported.
 *  - err/err_len: optional buffer that receives the failure text. */
#define MU_ATTENTION_STATIC_SCRATCH_BYTES 67108864u
int mu_attention_static_scratch(int device, const void *q, const void *k, const void *v, void *out,
                                int B, int H, int T, int D, int causal, int kmode, int dtype,
                                void *stream, int sync_and_check, char *err, size_t err_len);

/* ---- normalisation / softmax ----------------------------------------------
 * ops::layer_norm (src/core/ops/normalization.cpp:125-224; host-only in the
 * reference) and Backend::softmax over the last dim (src/core/backend.hpp:243). */
int mu_layer_norm(mu_ctx *ctx, const void *x, const void *gamma, const void *beta, void *y,
                  long long rows, int cols, float eps, int dtype, void *stream);
int mu_softmax(mu_ctx *ctx, const void *x, void *y, long long rows, int cols, int dtype,
               void *stream);

/* ---- spatial ops (float32, NCHW) -------------------------------------------
 * BackendSpatialCapability::conv2d / max_pool2d (src/core/backend.hpp:294-300; CPU
 * kernels src/backend/cpu_backend.hpp:768-796,833-855) and nn::GlobalAvgPool2d
 * (src/nn/pooling.hpp:8-26). weight is [oC,iC,k,k]; stride/pad are square; bias may
 * be NULL. mu_conv2d can fuse the ReLU module and a MaxPool2d(2,2,0) that follow it
 * in a Sequential (relu != 0, pool == 2): y is then [B,oC,oH/2,oW/2].
 * Layers below 2^31 multiply-adds (and every layer on a context with mu_ctx_force_simt) are
 * bit-identical to the reference CPU kernel (same summation order, no fused multiply-add);
 * larger ones run as im2col + 3xTF32 on the tensor cores: float32-class accuracy (within the
 * 1e-4 relative bound), not identical bits. The same split applies to float32 mu_matmul /
 * mu_linear at 2^31 multiply-adds. */
int mu_conv2d(mu_ctx *ctx, const void *x, const void *w, const void *bias, void *y, int B, int iC,
              int iH, int iW, int oC, int k, int stride, int pad, int relu, int pool, int dtype,
              void *stream);
int mu_max_pool2d(mu_ctx *ctx, const void *x, void *y, int B, int C, int H, int W, int k, int stride,
                  int pad, int dtype, void *stream);
int mu_global_avg_pool(mu_ctx *ctx, const void *x, void *y, int B, int C, int H, int W, int dtype,
                       void *stream);

/* ---- embedding -------------------------------------------------------------
 * nn::Embedding index path (src/nn/linear.hpp:92-131): out[b,t,:] = table[ids[b,t],:]
 * (+ pos[t,:] when pos != NULL — the token + position sum of the decoder).
 * An id outside [0,V) latches MU_ERR_INDEX (the reference throws). */
int mu_embedding(mu_ctx *ctx, const int32_t *ids, const void *table, const void *pos, void *out,
                 int B, int T, int V, int D, int dtype, void *stream);

/* ---- elementwise chain -----------------------------------------------------
 * Backend::add / relu / sigmoid and the activation modules built from them
 * (src/core/backend.hpp:233-242, src/nn/activations.hpp):
 *   y = act(x + bias[i % cols]) + residual ; bias / residual may be NULL. */
int mu_eltwise(mu_ctx *ctx, const void *x, const void *bias, const void *residual, void *y,
               long long n, int cols, int act, int dtype, void *stream);

/* Broadcasting binary ops: BackendElementwiseCapability::add / sub / mul / div with a
 * BroadcastInfo (src/core/backend.hpp:214-221, src/types.hpp:420-425): up to 6 output
 * dims, per-dimension element strides of each operand (0 = broadcast along that dim).
 * float32 results are bit-identical to the reference CPU kernels. */
enum mu_binary_op { MU_OP_ADD = 0, MU_OP_SUB = 1, MU_OP_MUL = 2, MU_OP_DIV = 3 };
int mu_binary_broadcast(mu_ctx *ctx, int op, const void *a, const void *b, void *out, int ndim,
                        const int *out_shape, const long long *strides_a,
                        const long long *strides_b, int dtype, void *stream);

/* ---- remaining forward entry points of the Backend surface --------------------
 * float32 and bfloat16 (bfloat16 evaluates in fp32 and rounds once). Shapes of extent 0 are
 * accepted and do nothing. */

/* BackendElementwiseCapability::exp / log / sqrt / rsqrt / sin / cos
 * (src/core/backend.hpp:228-233; CPU kernels src/backend/cpu_backend.hpp:533-586). */
enum mu_unary_op { MU_UN_EXP = 0, MU_UN_LOG = 1, MU_UN_SQRT = 2, MU_UN_RSQRT = 3, MU_UN_SIN = 4,
                   MU_UN_COS = 5 };
int mu_unary(mu_ctx *ctx, int op, const void *x, void *y, long long n, int dtype, void *stream);

/* nn::LeakyReLU (src/nn/activations.hpp:76-88): relu(x) + (x - relu(x)) * slope, one pass. */
int mu_leaky_relu(mu_ctx *ctx, const void *x, void *y, long long n, float slope, int dtype,
                  void *stream);

/* BackendElementwiseCapability::broadcast_row (src/core/backend.hpp:217-218;
 * cpu_backend.hpp:1051-1060): out[r, :] = row for r in [0, rows). */
int mu_broadcast_row(mu_ctx *ctx, const void *row, void *out, long long rows, int cols, int dtype,
                     void *stream);

/* BackendShapeCapability::concat (src/core/backend.hpp:257-258; cpu_backend.hpp:416-452).
 * `outer` = product of the dimensions before the concatenation axis, `inner` = product of
 * those after it, dim_sizes[j] = extent of input j along the axis. At most 8 inputs. */
int mu_concat(mu_ctx *ctx, const void *const *inputs, const int *dim_sizes, int n_inputs, void *out,
              long long outer, long long inner, int dtype, void *stream);

/* BackendSpatialCapability::upsample2d (src/core/backend.hpp:300-301; cpu_backend.hpp:889-902):
 * nearest neighbour, integer scale, NCHW. */
int mu_upsample2d(mu_ctx *ctx, const void *x, void *y, int B, int C, int H, int W, int scale,
                  int dtype, void *stream);

/* BackendNormalizationCapability::batch_norm with training=false (src/core/backend.hpp:308-312;
 * cpu_backend.hpp:957-967): y = gamma[c]*(x - mean[c])*(1/sqrt(var[c] + eps)) + beta[c].
 * The running statistics are float32 whatever `dtype` is (the reference keeps them in the
 * accumulation type, src/nn/normalization.hpp:84-98). The training branch is not built. */
int mu_batch_norm_eval(mu_ctx *ctx, const void *x, const void *gamma, const void *beta,
                       const float *running_mean, const float *running_var, void *y, int B, int C,
                       int H, int W, float eps, int dtype, void *stream);

/* nn::RMSNorm (src/nn/normalization.hpp:39-67): x * rsqrt(mean(x*x, last dim) + eps) * weight. */
int mu_rms_norm(mu_ctx *ctx, const void *x, const void *weight, void *y, long long rows, int cols,
                float eps, int dtype, void *stream);

/* BackendReductionCapability (src/core/backend.hpp:239-247; cpu_backend.hpp:1040-1049,
 * 1124-1137, 1084-1122): sum of every element into out[0]; mean over the last dimension;
 * sum onto a broadcast-compatible smaller shape (output extents are 1 or the input's, aligned
 * at the trailing dimensions). Accumulation is in double. */
int mu_sum(mu_ctx *ctx, const void *x, void *out, long long n, int dtype, void *stream);
int mu_mean_last_dim(mu_ctx *ctx, const void *x, void *out, long long outer, int dim, int dtype,
                     void *stream);
int mu_sum_to_shape(mu_ctx *ctx, const void *x, void *out, const int *in_shape, int in_ndim,
                    const int *out_shape, int out_ndim, int dtype, void *stream);

/* BackendRandomCapability::fill_uniform (src/core/backend.hpp:341-344). The reference's CPU
 * fill depends on the host's thread count (cpu_backend.hpp:1021-1038), so there are no bits to
 * match: values are a pure function of (seed, index), uniform in [low, high). */
int mu_fill_uniform(mu_ctx *ctx, void *out, long long n, float low, float high,
                    unsigned long long seed, int dtype, void *stream);

/* ---- argmax ---------------------------------------------------------------
 * The reference has no argmax op; its demos take np.argmax of the logits
 * (demos/transformers/decoder_block_demo.py:112). First maximum wins. */
int mu_argmax(mu_ctx *ctx, const void *x, int32_t *idx, long long rows, int cols, int dtype,
              void *stream);

/* ---- all-reduce ------------------------------------------------------------
 * Backend::all_reduce (src/core/backend.hpp:199,473-477): elementwise SUM over the
 * participants (src/core/all_reduce_runtime.hpp:85-133). The reference stages every
 * buffer through host memory inside one process; here each process owns one GPU and the
 * sum runs in NCCL over NVLink. The 128-byte id from mu_comm_unique_id (rank 0) is
 * handed to the other ranks by the host (e.g. torch.distributed broadcast). A NULL comm
 * or a world of 1 makes mu_all_reduce_sum a no-op. mu_comm_check is a non-blocking host
 * check for a failed peer. */
typedef struct mu_comm mu_comm;
int mu_comm_unique_id(void *out, size_t capacity);
int mu_comm_create(mu_ctx *ctx, const void *unique_id, int rank, int world, mu_comm **out);
void mu_comm_destroy(mu_comm *comm);
int mu_comm_rank(const mu_comm *comm);
int mu_comm_world(const mu_comm *comm);
int mu_all_reduce_sum(mu_ctx *ctx, mu_comm *comm, void *buffer, long long n, int dtype,
                      void *stream);
int mu_comm_check(mu_ctx *ctx, mu_comm *comm);
/* Host deadline for the collectives enqueued on `stream`: returns MU_OK once the stream has
 * drained, or after timeout_ms (<= 0: MUNET_ALLREDUCE_TIMEOUT_MS, default 10000, the reference's
 * variable and default) aborts the communicator and returns MU_ERR_TIMEOUT with the reference's
 * message "all_reduce: timeout waiting for participants" (src/core/all_reduce_runtime.hpp:205-225:
 * a participant that never arrives). mu_comm_abort is ncclCommAbort: the communicator is unusable
 * afterwards and every later call on it fails. */
int mu_comm_wait(mu_ctx *ctx, mu_comm *comm, void *stream, int timeout_ms);
int mu_comm_abort(mu_comm *comm);

/* ---- compiled inference executor -------------------------------------------
 * Stands in for munet::inference::Engine (src/inference.hpp:292-801) and
 * load_serialized (src/inference_serialization.cpp:1086-1089).
 *   mu_engine_load         Engine::load(path): parse + validate a deploy artifact
 *                          (.npz of .npy members, JSON module tree in __config__).
 *   mu_engine_load_memory  Engine::load(module): same module tree given as JSON text
 *                          plus named tensors already in memory (host or device).
 *   mu_engine_compile      Engine::compile(example): fixes the input shape contract,
 *                          lowers the module tree to a fused op list, plans one arena,
 *                          uploads weights and captures a CUDA graph.
 *   mu_engine_run          Engine::run(input): strict shape contract, one graph launch.
 * Module types: the reference's Sequential, Linear, ReLU, Sigmoid, Tanh, GELU, Dropout,
 * Flatten, LayerNorm, Embedding, MultiHeadAttention, plus the extension containers
 * TransformerBlock{d_model,n_heads} and GPTDecoder{vocab,ctx_len,d_model,n_heads,n_layers}
 * (the reference format has no residual container, so it cannot express a decoder).
 * compute_dtype: MU_F32 or MU_BF16; float32 tensors are converted on load like
 * Module::to(DataType) (src/core/module.hpp:177-194). */
typedef struct mu_engine mu_engine;
int mu_engine_create(mu_ctx *ctx, mu_engine **out);
void mu_engine_destroy(mu_engine *engine);
const char *mu_engine_last_error(const mu_engine *engine);
/* options: "kmode" (mu_kmode), "use_graph" (0/1), "argmax" (0/1: also produce int32 argmax),
 * "plan_cache_entries" (plans kept under a wildcard contract), "tp_size" / "tp_rank" / "tp_overlap" /
 * "tp_exchange" (tensor parallelism, below). Set them before the first compile. */
int mu_engine_set_option(mu_engine *engine, const char *name, int value);
int mu_engine_load(mu_engine *engine, const char *artifact_path, int compute_dtype);
/* shapes: all tensors' dims concatenated, ndims[i] of them per tensor */
int mu_engine_load_memory(mu_engine *engine, const char *config_json, int n_tensors,
                          const char *const *names, const void *const *data, const int *dtypes,
                          const int *ndims, const long long *shapes, int on_device,
                          int compute_dtype);
/* Tensor parallelism (no counterpart in the reference, which has none): options "tp_size" and
 * "tp_rank" plus a communicator of that size shard every decoder block Megatron-style —
 * q/k/v and fc1 by output columns (heads), out_proj and fc2 by input rows with an all-reduce
 * of the partial sums, the LM head by vocabulary columns (output = this rank's slab).
 * Option "tp_overlap" (default 1) cuts the row-parallel layers into four row chunks and runs
 * the all-reduce of one chunk on a second stream under the GEMM of the next. */
int mu_engine_set_comm(mu_engine *engine, mu_comm *comm);
/* Option "tp_exchange" = 1 (two ranks, bfloat16): the partial sums of the row-parallel layers
 * meet through peer memory instead of NCCL. Each rank's exchange kernel reads the other rank's
 * partial straight over NVLink (plain peer loads; no TMA, multicast or multimem) and writes
 * sum + bias + residual in one pass; two counters per rank, written by the peer, order the
 * GEMMs and the reads, and every device-side wait on them is bounded (MU_ERR_TIMEOUT from
 * mu_check / mu_engine_run when the peer never arrives). Set-up, after mu_engine_compile on both
 * ranks: mu_engine_peer_info -> mu_ipc_export (a 64-byte handle each for the arena and the
 * counters) -> hand the handles to the other process -> mu_ipc_open -> mu_engine_attach_peer.
 * Attaching runs one forward and captures the graph: both ranks call it at the same time. The
 * communicator is still required at compile (it defines rank and size). */
size_t mu_peer_flags_bytes(void);
int mu_ipc_export(mu_ctx *ctx, const void *device_ptr, void *handle_out, size_t capacity);
int mu_ipc_open(mu_ctx *ctx, const void *handle, void **peer_ptr);
int mu_ipc_close(mu_ctx *ctx, void *peer_ptr);
int mu_engine_peer_info(const mu_engine *engine, void **arena, void **counters);
int mu_engine_attach_peer(mu_engine *engine, void *peer_arena, void *peer_counters);
int mu_engine_compile(mu_engine *engine, const int *input_shape, int ndim, int input_dtype);
/* Engine::compile(example, expected_input_shape) with -1 wildcards (detail::ShapeContract,
 * src/inference.hpp:128-176; tests/test_inference.cpp:402-438): expected_shape[i] == -1 lets
 * dimension i vary from run to run (NULL = the example's exact shape). The plan for the example
 * shape is built now; mu_engine_select_shape makes the plan of another shape that fits the
 * contract the active one, building it on first sight (weights are shared, each plan has its own
 * arena and graph; option "plan_cache_entries", default 8, bounds how many are kept, least
 * recently used first out). A shape that breaks the contract is refused with the reference's
 * words ("rank mismatch" / "dim mismatch at index i"). mu_engine_run always runs the active plan. */
int mu_engine_compile_contract(mu_engine *engine, const int *example_shape, int ndim,
                               const int *expected_shape, int input_dtype);
int mu_engine_select_shape(mu_engine *engine, const int *shape, int ndim);
int mu_engine_plan_count(const mu_engine *engine);
int mu_engine_output_shape(const mu_engine *engine, int *shape, int *ndim, int *dtype);
int mu_engine_stats(const mu_engine *engine, long long *arena_bytes, long long *weight_bytes,
                    long long *n_ops, long long *n_launches, long long *unplanned_bytes);
int mu_engine_run(mu_engine *engine, const void *input, int input_on_host, void *output,
                  int output_on_host, int32_t *argmax_out, int argmax_on_host, void *stream);
/* Per-op timing of an eager forward (CUDA events around every op, mean of `reps`),
 * with each op's algorithmic FLOPs / bytes: the engine-level counterpart of the
 * reference's Profiler rows (src/core/util/profiler.hpp:31-185).
 * kinds: 0 embed, 1 layer_norm, 2 linear, 3 qkv linear, 4 attention, 5 eltwise, 6 argmax. */
int mu_engine_profile(mu_engine *engine, int reps, int capacity, int *n_ops, int *kinds, float *ms,
                      double *flops, double *bytes, void *stream);
/* M, K, N and a residual flag (four ints per op, zeros for ops that are not linears) of the
 * active plan's ops, in the order mu_engine_profile reports them. */
int mu_engine_op_dims(const mu_engine *engine, int capacity, int *dims);
void *mu_engine_output_ptr(const mu_engine *engine);
/* Host-only: parse + validate a deploy artifact exactly as mu_engine_load does
 * (parse_and_validate_artifact, src/inference_serialization.cpp:919-1033) and
 * write a JSON summary {"config": <module tree>, "tensors": {name: {dtype, shape}}}.
 * Needs no device. Returns MU_OK, MU_ERR_INVALID (text in err) or MU_ERR_SIZE. */
int mu_artifact_inspect(const char *path, char *json_out, size_t json_cap, char *err,
                        size_t err_len);
void *mu_engine_argmax_ptr(const mu_engine *engine);

#ifdef __cplusplus
}
#endif
#endif /* MUNET_B200_H */
