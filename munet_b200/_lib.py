"""ctypes binding of the C ABI in include/munet_b200.h.

``Context`` wraps one ``mu_ctx`` (one device).  Its methods take any object with
a ``data_ptr()`` (torch tensors) or raw integer device addresses; torch is used
only by callers for device memory and streams, never for compute.
"""
from __future__ import annotations

import ctypes as C
import os

F32, F16, BF16, I32 = 0, 1, 2, 3
ACT = {"none": 0, "relu": 1, "gelu": 2, "sigmoid": 3, "tanh": 4, None: 0}
K_LITERAL, K_MATH = 0, 1
COPY_H2D, COPY_D2H, COPY_D2D = 1, 2, 3

_HERE = os.path.dirname(os.path.abspath(__file__))


class MuNetError(RuntimeError):
    """A non-zero status from the native library (message = mu_last_error)."""

    def __init__(self, code: int, message: str):
        super().__init__(f"[munet_b200 status {code}] {message}")
        self.code = code


def lib_path() -> str:
    return os.path.join(_HERE, "lib", "libmunet_b200.so")


_lib = None

_vp, _i, _ll, _sz, _f = C.c_void_p, C.c_int, C.c_longlong, C.c_size_t, C.c_float

# name -> (restype, argtypes); mirrors include/munet_b200.h one to one
SIGNATURES = {
    "mu_abi_version": (_i, []),
    "mu_ctx_create": (_i, [_i, C.POINTER(_vp)]),
    "mu_ctx_destroy": (None, [_vp]),
    "mu_last_error": (C.c_char_p, [_vp]),
    "mu_ctx_num_sms": (_i, [_vp]),
    "mu_ctx_force_simt": (_i, [_vp, _i]),
    "mu_ctx_set_sm_budget": (_i, [_vp, _i]),
    "mu_ctx_set_gemm_tile": (_i, [_vp, _i, _i]),
    "mu_ctx_set_l2_set_aside": (_i, [_vp, _sz]),
    "mu_alloc": (_i, [_vp, _sz, C.POINTER(_vp)]),
    "mu_free": (_i, [_vp, _vp]),
    "mu_copy": (_i, [_vp, _vp, _vp, _sz, _i, _vp]),
    "mu_memset": (_i, [_vp, _vp, _i, _sz, _vp]),
    "mu_to_contiguous": (_i, [_vp, _vp, _vp, _i, C.POINTER(_i), C.POINTER(_ll), _ll, _i, _vp]),
    "mu_timer_begin": (_i, [_vp, _vp]),
    "mu_timer_end": (_i, [_vp, _vp]),
    "mu_timer_last_us": (C.c_double, [_vp]),
    "mu_synchronize": (_i, [_vp]),
    "mu_check": (_i, [_vp, _vp]),
    "mu_matmul": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]),
    "mu_batched_matmul": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _ll, _ll, _ll, _i, _vp]),
    "mu_linear": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "mu_linear_qkv": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "mu_linear_qkv_heads": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]),
    "mu_attention_workspace_bytes": (_sz, [_i, _i, _i, _i, _i]),
    "mu_attention_workspace_bytes_composed": (_sz, [_i, _i, _i, _i, _i]),
    "mu_attention": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _sz, _vp]),
    "mu_attention_static_scratch": (_i, [_i, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _i,
                                         C.c_char_p, _sz]),
    "mu_conv2d": (_i, [_vp, _vp, _vp, _vp, _vp] + [_i] * 11 + [_vp]),
    "mu_max_pool2d": (_i, [_vp, _vp, _vp] + [_i] * 8 + [_vp]),
    "mu_global_avg_pool": (_i, [_vp, _vp, _vp] + [_i] * 5 + [_vp]),
    "mu_layer_norm": (_i, [_vp, _vp, _vp, _vp, _vp, _ll, _i, _f, _i, _vp]),
    "mu_softmax": (_i, [_vp, _vp, _vp, _ll, _i, _i, _vp]),
    "mu_embedding": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]),
    "mu_eltwise": (_i, [_vp, _vp, _vp, _vp, _vp, _ll, _i, _i, _i, _vp]),
    "mu_argmax": (_i, [_vp, _vp, _vp, _ll, _i, _i, _vp]),
    "mu_unary": (_i, [_vp, _i, _vp, _vp, _ll, _i, _vp]),
    "mu_leaky_relu": (_i, [_vp, _vp, _vp, _ll, C.c_float, _i, _vp]),
    "mu_broadcast_row": (_i, [_vp, _vp, _vp, _ll, _i, _i, _vp]),
    "mu_concat": (_i, [_vp, C.POINTER(_vp), C.POINTER(_i), _i, _vp, _ll, _ll, _i, _vp]),
    "mu_upsample2d": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]),
    "mu_batch_norm_eval": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, C.c_float, _i, _vp]),
    "mu_rms_norm": (_i, [_vp, _vp, _vp, _vp, _ll, _i, C.c_float, _i, _vp]),
    "mu_sum": (_i, [_vp, _vp, _vp, _ll, _i, _vp]),
    "mu_mean_last_dim": (_i, [_vp, _vp, _vp, _ll, _i, _i, _vp]),
    "mu_sum_to_shape": (_i, [_vp, _vp, _vp, C.POINTER(_i), _i, C.POINTER(_i), _i, _i, _vp]),
    "mu_fill_uniform": (_i, [_vp, _vp, _ll, C.c_float, C.c_float, C.c_ulonglong, _i, _vp]),
    "mu_binary_broadcast": (_i, [_vp, _i, _vp, _vp, _vp, _i, C.POINTER(_i), C.POINTER(_ll),
                                 C.POINTER(_ll), _i, _vp]),
    "mu_comm_unique_id": (_i, [_vp, _sz]),
    "mu_comm_create": (_i, [_vp, _vp, _i, _i, C.POINTER(_vp)]),
    "mu_comm_destroy": (None, [_vp]),
    "mu_comm_rank": (_i, [_vp]),
    "mu_comm_world": (_i, [_vp]),
    "mu_all_reduce_sum": (_i, [_vp, _vp, _vp, _ll, _i, _vp]),
    "mu_comm_check": (_i, [_vp, _vp]),
    "mu_comm_wait": (_i, [_vp, _vp, _vp, _i]),
    "mu_comm_abort": (_i, [_vp]),
    "mu_engine_create": (_i, [_vp, C.POINTER(_vp)]),
    "mu_engine_destroy": (None, [_vp]),
    "mu_engine_last_error": (C.c_char_p, [_vp]),
    "mu_engine_set_option": (_i, [_vp, C.c_char_p, _i]),
    "mu_engine_load": (_i, [_vp, C.c_char_p, _i]),
    "mu_engine_load_memory": (_i, [_vp, C.c_char_p, _i, C.POINTER(C.c_char_p), C.POINTER(_vp),
                                   C.POINTER(_i), C.POINTER(_i), C.POINTER(_ll), _i, _i]),
    "mu_engine_set_comm": (_i, [_vp, _vp]),
    "mu_engine_compile": (_i, [_vp, C.POINTER(_i), _i, _i]),
    "mu_engine_compile_contract": (_i, [_vp, C.POINTER(_i), _i, C.POINTER(_i), _i]),
    "mu_engine_select_shape": (_i, [_vp, C.POINTER(_i), _i]),
    "mu_engine_plan_count": (_i, [_vp]),
    "mu_peer_flags_bytes": (_sz, []),
    "mu_ipc_export": (_i, [_vp, _vp, _vp, _sz]),
    "mu_ipc_open": (_i, [_vp, _vp, C.POINTER(_vp)]),
    "mu_ipc_close": (_i, [_vp, _vp]),
    "mu_engine_peer_info": (_i, [_vp, C.POINTER(_vp), C.POINTER(_vp)]),
    "mu_engine_attach_peer": (_i, [_vp, _vp, _vp]),
    "mu_engine_op_dims": (_i, [_vp, _i, C.POINTER(_i)]),
    "mu_engine_output_shape": (_i, [_vp, C.POINTER(_i), C.POINTER(_i), C.POINTER(_i)]),
    "mu_engine_stats": (_i, [_vp] + [C.POINTER(_ll)] * 5),
    "mu_engine_run": (_i, [_vp, _vp, _i, _vp, _i, _vp, _i, _vp]),
    "mu_engine_profile": (_i, [_vp, _i, _i, C.POINTER(_i), C.POINTER(_i), C.POINTER(_f),
                               C.POINTER(C.c_double), C.POINTER(C.c_double), _vp]),
    "mu_engine_output_ptr": (_vp, [_vp]),
    "mu_artifact_inspect": (_i, [C.c_char_p, C.c_char_p, _sz, C.c_char_p, _sz]),
    "mu_engine_argmax_ptr": (_vp, [_vp]),
}


def lib() -> C.CDLL:
    """Load libmunet_b200.so (built in-tree by ``python -m munet_b200.build``)."""
    global _lib
    if _lib is None:
        path = lib_path()
        if not os.path.exists(path):
            raise ImportError(
                f"{path} is missing: build the CUDA extension first "
                "(python -m munet_b200.build). There is no fallback implementation.")
        handle = C.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError here = ABI mismatch, fail loudly
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def _ptr(t):
    if t is None:
        return None
    if isinstance(t, int):
        return t
    return t.data_ptr()


def _stream(stream):
    if stream is None:
        try:
            import torch
            return torch.cuda.current_stream().cuda_stream
        except Exception:
            return None
    if isinstance(stream, int):
        return stream
    return stream.cuda_stream


class Context:
    """One device context of the native backend."""

    def __init__(self, device: int = 0):
        self._lib = lib()
        h = _vp()
        rc = self._lib.mu_ctx_create(device, C.byref(h))
        if rc != 0:
            raise MuNetError(rc, f"mu_ctx_create(device={device}) failed")
        self._h = h
        self.device = device

    def close(self):
        if getattr(self, "_h", None):
            self._lib.mu_ctx_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _rc(self, rc: int):
        if rc != 0:
            raise MuNetError(rc, self._lib.mu_last_error(self._h).decode())

    @property
    def num_sms(self) -> int:
        return self._lib.mu_ctx_num_sms(self._h)

    def force_simt(self, on: bool):
        self._rc(self._lib.mu_ctx_force_simt(self._h, int(on)))

    def set_sm_budget(self, n: int):
        """Limit persistent GEMM grids to ``n`` SMs (0 = all): room for a kernel running beside them."""
        self._rc(self._lib.mu_ctx_set_sm_budget(self._h, int(n)))

    def set_gemm_tile(self, bn: int = 0, ctas: int = 0):
        """Fix the bf16 GEMM tile (width 64/128/256, 1 or 2 CTAs); 0, 0 = automatic."""
        self._rc(self._lib.mu_ctx_set_gemm_tile(self._h, int(bn), int(ctas)))

    def set_l2_set_aside(self, nbytes: int):
        """Reserve ``nbytes`` of L2 for the GEMMs' weight tiles (a limit of this process's CUDA
        context; 0 = off)."""
        self._rc(self._lib.mu_ctx_set_l2_set_aside(self._h, int(nbytes)))

    def check(self, stream=None):
        """Synchronise the stream and raise if a kernel latched a device-side error."""
        self._rc(self._lib.mu_check(self._h, _stream(stream)))

    def synchronize(self):
        self._rc(self._lib.mu_synchronize(self._h))

    def memset(self, ptr, value: int, nbytes: int, stream=None):
        self._rc(self._lib.mu_memset(self._h, _ptr(ptr), int(value), int(nbytes), _stream(stream)))

    def to_contiguous(self, src, dst, shape, strides, offset: int, elem_size: int, stream=None):
        """Row-major copy of a strided view (strides / offset in elements, at most 6 dims)."""
        n = len(shape)
        self._rc(self._lib.mu_to_contiguous(
            self._h, _ptr(src), _ptr(dst), n, (C.c_int * max(n, 1))(*shape),
            (C.c_longlong * max(n, 1))(*strides), int(offset), int(elem_size), _stream(stream)))

    def timer_begin(self, stream=None):
        self._rc(self._lib.mu_timer_begin(self._h, _stream(stream)))

    def timer_end(self, stream=None):
        self._rc(self._lib.mu_timer_end(self._h, _stream(stream)))

    def timer_last_us(self) -> float:
        return float(self._lib.mu_timer_last_us(self._h))

    # -- BLAS ----------------------------------------------------------------
    def matmul(self, a, b, c, M, K, N, dtype, transA=False, transB=False, stream=None):
        self._rc(self._lib.mu_matmul(self._h, _ptr(a), _ptr(b), _ptr(c), M, K, N, int(transA),
                                     int(transB), dtype, _stream(stream)))

    def batched_matmul(self, a, b, c, batch, M, K, N, stride_a, stride_b, stride_out, dtype,
                       transA=False, transB=False, stream=None):
        self._rc(self._lib.mu_batched_matmul(self._h, _ptr(a), _ptr(b), _ptr(c), batch, M, K, N,
                                             int(transA), int(transB), stride_a, stride_b,
                                             stride_out, dtype, _stream(stream)))

    def linear(self, x, w, bias, y, M, K, N, dtype, act="none", residual=None, stream=None):
        self._rc(self._lib.mu_linear(self._h, _ptr(x), _ptr(w), _ptr(bias), _ptr(residual), _ptr(y),
                                     M, K, N, ACT[act], dtype, _stream(stream)))

    def linear_qkv(self, x, w_qkv, bias_qkv, q, k, v, B, T, E, H, dtype, stream=None):
        self._rc(self._lib.mu_linear_qkv(self._h, _ptr(x), _ptr(w_qkv), _ptr(bias_qkv), _ptr(q),
                                         _ptr(k), _ptr(v), B, T, E, H, dtype, _stream(stream)))

    def attention_workspace_bytes(self, B, H, T, D, dtype) -> int:
        return int(self._lib.mu_attention_workspace_bytes(B, H, T, D, dtype))

    def attention(self, q, k, v, out, B, H, T, D, causal, kmode, dtype, workspace, workspace_bytes,
                  stream=None):
        self._rc(self._lib.mu_attention(self._h, _ptr(q), _ptr(k), _ptr(v), _ptr(out), B, H, T, D,
                                        int(causal), kmode, dtype, _ptr(workspace),
                                        workspace_bytes, _stream(stream)))

    # -- rows / elementwise ----------------------------------------------------
    def layer_norm(self, x, gamma, beta, y, rows, cols, dtype, eps=1e-5, stream=None):
        self._rc(self._lib.mu_layer_norm(self._h, _ptr(x), _ptr(gamma), _ptr(beta), _ptr(y), rows,
                                         cols, eps, dtype, _stream(stream)))

    def softmax(self, x, y, rows, cols, dtype, stream=None):
        self._rc(self._lib.mu_softmax(self._h, _ptr(x), _ptr(y), rows, cols, dtype, _stream(stream)))

    def embedding(self, ids, table, pos, out, B, T, V, D, dtype, stream=None):
        self._rc(self._lib.mu_embedding(self._h, _ptr(ids), _ptr(table), _ptr(pos), _ptr(out), B, T,
                                        V, D, dtype, _stream(stream)))

    def eltwise(self, x, y, n, dtype, act="none", bias=None, cols=1, residual=None, stream=None):
        self._rc(self._lib.mu_eltwise(self._h, _ptr(x), _ptr(bias), _ptr(residual), _ptr(y), n, cols,
                                      ACT[act], dtype, _stream(stream)))

    # -- spatial -----------------------------------------------------------------
    def conv2d(self, x, w, bias, y, B, iC, iH, iW, oC, k, stride, pad, dtype, relu=False, pool=0,
               stream=None):
        self._rc(self._lib.mu_conv2d(self._h, _ptr(x), _ptr(w), _ptr(bias), _ptr(y), B, iC, iH, iW, oC,
                                     k, stride, pad, int(relu), pool, dtype, _stream(stream)))

    def max_pool2d(self, x, y, B, Cc, H, W, k, stride, pad, dtype, stream=None):
        self._rc(self._lib.mu_max_pool2d(self._h, _ptr(x), _ptr(y), B, Cc, H, W, k, stride, pad, dtype,
                                         _stream(stream)))

    def global_avg_pool(self, x, y, B, Cc, H, W, dtype, stream=None):
        self._rc(self._lib.mu_global_avg_pool(self._h, _ptr(x), _ptr(y), B, Cc, H, W, dtype,
                                              _stream(stream)))

    def binary(self, op, a, b, out, out_shape, strides_a, strides_b, dtype, stream=None):
        """op in add/sub/mul/div; strides in elements, 0 = broadcast along that dim."""
        n = len(out_shape)
        code = {"add": 0, "sub": 1, "mul": 2, "div": 3}[op]
        self._rc(self._lib.mu_binary_broadcast(
            self._h, code, _ptr(a), _ptr(b), _ptr(out), n, (C.c_int * max(n, 1))(*out_shape),
            (C.c_longlong * max(n, 1))(*strides_a), (C.c_longlong * max(n, 1))(*strides_b), dtype,
            _stream(stream)))

    # -- remaining forward entry points ---------------------------------------------
    UNARY = {"exp": 0, "log": 1, "sqrt": 2, "rsqrt": 3, "sin": 4, "cos": 5}

    def unary(self, op, x, y, n, dtype, stream=None):
        self._rc(self._lib.mu_unary(self._h, self.UNARY[op], _ptr(x), _ptr(y), n, dtype, _stream(stream)))

    def leaky_relu(self, x, y, n, slope, dtype, stream=None):
        self._rc(self._lib.mu_leaky_relu(self._h, _ptr(x), _ptr(y), n, slope, dtype, _stream(stream)))

    def broadcast_row(self, row, out, rows, cols, dtype, stream=None):
        self._rc(self._lib.mu_broadcast_row(self._h, _ptr(row), _ptr(out), rows, cols, dtype,
                                            _stream(stream)))

    def concat(self, inputs, dim_sizes, out, outer, inner, dtype, stream=None):
        n = len(inputs)
        ptrs = (_vp * max(n, 1))(*[_ptr(t) for t in inputs])
        self._rc(self._lib.mu_concat(self._h, ptrs, (C.c_int * max(n, 1))(*dim_sizes), n, _ptr(out),
                                     outer, inner, dtype, _stream(stream)))

    def upsample2d(self, x, y, B, Cc, H, W, scale, dtype, stream=None):
        self._rc(self._lib.mu_upsample2d(self._h, _ptr(x), _ptr(y), B, Cc, H, W, scale, dtype,
                                         _stream(stream)))

    def batch_norm_eval(self, x, gamma, beta, mean, var, y, B, Cc, H, W, eps, dtype, stream=None):
        self._rc(self._lib.mu_batch_norm_eval(self._h, _ptr(x), _ptr(gamma), _ptr(beta), _ptr(mean),
                                              _ptr(var), _ptr(y), B, Cc, H, W, eps, dtype,
                                              _stream(stream)))

    def rms_norm(self, x, w, y, rows, cols, dtype, eps=1e-5, stream=None):
        self._rc(self._lib.mu_rms_norm(self._h, _ptr(x), _ptr(w), _ptr(y), rows, cols, eps, dtype,
                                       _stream(stream)))

    def sum(self, x, out, n, dtype, stream=None):
        self._rc(self._lib.mu_sum(self._h, _ptr(x), _ptr(out), n, dtype, _stream(stream)))

    def mean_last_dim(self, x, out, outer, dim, dtype, stream=None):
        self._rc(self._lib.mu_mean_last_dim(self._h, _ptr(x), _ptr(out), outer, dim, dtype,
                                            _stream(stream)))

    def sum_to_shape(self, x, out, in_shape, out_shape, dtype, stream=None):
        ni, no = len(in_shape), len(out_shape)
        self._rc(self._lib.mu_sum_to_shape(self._h, _ptr(x), _ptr(out), (C.c_int * max(ni, 1))(*in_shape),
                                           ni, (C.c_int * max(no, 1))(*out_shape), no, dtype,
                                           _stream(stream)))

    def fill_uniform(self, out, n, low, high, seed, dtype, stream=None):
        self._rc(self._lib.mu_fill_uniform(self._h, _ptr(out), n, low, high, seed, dtype,
                                           _stream(stream)))

    def argmax(self, x, idx, rows, cols, dtype, stream=None):
        self._rc(self._lib.mu_argmax(self._h, _ptr(x), _ptr(idx), rows, cols, dtype, _stream(stream)))

    def all_reduce_sum(self, comm, buf, n, dtype, stream=None):
        self._rc(self._lib.mu_all_reduce_sum(self._h, comm._h if comm else None, _ptr(buf), n, dtype,
                                             _stream(stream)))


class Comm:
    """One NCCL communicator (one process per GPU). ``unique_id`` is the 128-byte id made by
    ``Comm.new_unique_id()`` on one rank and handed to the others by the host."""

    def __init__(self, ctx: "Context", unique_id: bytes, rank: int, world: int):
        self._lib = lib()
        self.ctx = ctx
        h = _vp()
        buf = C.create_string_buffer(bytes(unique_id), 128)
        rc = self._lib.mu_comm_create(ctx._h, buf, rank, world, C.byref(h))
        if rc != 0:
            raise MuNetError(rc, self._lib.mu_last_error(ctx._h).decode())
        self._h = h
        self.rank, self.world = rank, world

    @staticmethod
    def new_unique_id() -> bytes:
        buf = C.create_string_buffer(128)
        rc = lib().mu_comm_unique_id(buf, 128)
        if rc != 0:
            raise MuNetError(rc, "mu_comm_unique_id failed (is libnccl.so.2 loadable?)")
        return buf.raw

    @classmethod
    def from_torch_distributed(cls, ctx: "Context"):
        """Build the communicator over the default torch.distributed group (id exchanged there)."""
        import torch
        import torch.distributed as dist
        rank, world = dist.get_rank(), dist.get_world_size()
        ids = [cls.new_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        return cls(ctx, ids[0], rank, world)

    def check(self):
        rc = self._lib.mu_comm_check(self.ctx._h, self._h)
        if rc != 0:
            raise MuNetError(rc, self._lib.mu_last_error(self.ctx._h).decode())

    def wait(self, stream=None, timeout_ms: int = 0):
        """Host deadline for the collectives enqueued on ``stream`` (0 = MUNET_ALLREDUCE_TIMEOUT_MS
        or 10 s): raises MuNetError(MU_ERR_TIMEOUT) and aborts the communicator when a participant
        never arrives."""
        rc = self._lib.mu_comm_wait(self.ctx._h, self._h, _stream(stream), int(timeout_ms))
        if rc != 0:
            raise MuNetError(rc, self._lib.mu_last_error(self.ctx._h).decode())

    def abort(self):
        self._lib.mu_comm_abort(self._h)

    def close(self):
        if getattr(self, "_h", None):
            self._lib.mu_comm_destroy(self._h)
            self._h = None
