"""TEST INFRASTRUCTURE ONLY: numpy bindings for the two CPU parity checkers.

* ``port``  – ``oracle/liboracle.so``: our C restatement (``oracle/oracle.c``).
* ``ref``   – ``oracle/_ref/libmunet_ref.so``: the unmodified reference CPU core
  behind ``oracle/ref_driver.cpp`` (built only where the reference checkout is
  present; the prebuilt library is what travels to a GPU machine).

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline / reference
legs of ``bench.py`` may import this package.  The product package must never do so.

16-bit tensors are numpy ``uint16`` bit patterns; helpers ``to_bf16`` /
``from_bf16`` convert with the reference's rounding (src/types.hpp:311-324).
dtype codes: 0 float32, 2 bfloat16 (reference enum order, src/types.hpp:16).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
PORT_PATH = os.path.join(_HERE, "liboracle.so")
REF_PATH = os.path.join(_HERE, "_ref", "libmunet_ref.so")

F32, BF16, I32 = 0, 2, 3
ACT = {"none": 0, "relu": 1, "gelu": 2, "sigmoid": 3, "tanh": 4}
K_LITERAL, K_MATH = 0, 1


def reference_checkout() -> str | None:
    """Where the reference's sources are: $MUNET_REF, else a directory named ``reference`` beside
    this repository; None when neither exists (the prebuilt oracle/_ref is then used as it is)."""
    cand = os.environ.get("MUNET_REF") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
    return cand if os.path.isdir(os.path.join(cand, "src")) else None


def build(ref: bool = True) -> None:
    """Compile the checkers (C port always; the reference core when its checkout exists)."""
    subprocess.check_call(["make", "-s", "-C", _HERE, "port"])
    src = reference_checkout() if ref else None
    if src:
        subprocess.check_call(["make", "-s", "-C", _HERE, "ref", "-j8", "REF=" + src])
        lib_dir = os.path.join(_HERE, "..", "munet_b200", "lib", "libmunet_b200.so")
        if os.path.exists(lib_dir):  # drop-in proof: reference core + our Backend adapter
            subprocess.check_call(["make", "-s", "-C", _HERE, "refb200", "-j8", "REF=" + src])


def to_bf16(a) -> np.ndarray:
    """float32 → bf16 bits, RNE via the +0x7fff+lsb trick (src/types.hpp:311-317)."""
    b = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    lsb = (b >> np.uint32(16)) & np.uint32(1)
    return ((b + np.uint32(0x7FFF) + lsb) >> np.uint32(16)).astype(np.uint16)


def from_bf16(a) -> np.ndarray:
    return (np.ascontiguousarray(a, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def np_dtype(code: int):
    return {F32: np.float32, BF16: np.uint16, I32: np.int32}[code]


def as_float(a: np.ndarray, code: int) -> np.ndarray:
    return a.astype(np.float32) if code == F32 else from_bf16(a)


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, code):
    return None if a is None else np.ascontiguousarray(a, dtype=np_dtype(code))


class _Lib:
    """Shared shape of both checkers; ``prefix`` selects ``orc_`` or ``ref_`` symbols."""

    def __init__(self, path: str, prefix: str):
        if not os.path.exists(path):
            raise FileNotFoundError(f"{path} is not built (run `make -C oracle`)")
        self.lib = C.CDLL(path)
        self.prefix = prefix
        self.is_ref = prefix == "ref_"
        if self.is_ref:
            self.lib.ref_last_error.restype = C.c_char_p

    def _call(self, name, *args):
        fn = getattr(self.lib, self.prefix + name)
        fn.restype = C.c_int
        rc = fn(*args)
        if rc != 0:
            msg = self.lib.ref_last_error().decode() if self.is_ref else f"status {rc}"
            raise RuntimeError(f"{self.prefix}{name} failed: {msg}")

    # -- ops ---------------------------------------------------------------
    def linear(self, x, w, b, dtype, act="none"):
        x, w, b = _c(x, dtype), _c(w, dtype), _c(b, dtype)
        M, K = x.shape
        N = w.shape[1]
        y = np.empty((M, N), np_dtype(dtype))
        self._call("linear", _p(x), _p(w), _p(b), _p(y), M, K, N, dtype, ACT[act])
        return y

    def matmul(self, a, b, dtype):
        a, b = _c(a, dtype), _c(b, dtype)
        M, K = a.shape
        N = b.shape[1]
        y = np.empty((M, N), np_dtype(dtype))
        self._call("matmul", _p(a), _p(b), _p(y), M, K, N, dtype)
        return y

    def activation(self, x, dtype, act):
        x = _c(x, dtype)
        y = np.empty_like(x)
        self._call("activation", _p(x), _p(y), C.c_long(x.size), dtype, ACT[act])
        return y

    def add(self, a, b, dtype):
        a, b = _c(a, dtype), _c(b, dtype)
        y = np.empty_like(a)
        self._call("add", _p(a), _p(b), _p(y), C.c_long(a.size), dtype)
        return y

    def layer_norm(self, x, g, b, dtype, eps=1e-5):
        x, g, b = _c(x, dtype), _c(g, dtype), _c(b, dtype)
        cols = x.shape[-1]
        rows = x.size // cols
        y = np.empty_like(x)
        self._call("layer_norm", _p(x), _p(g), _p(b), _p(y), rows, cols, C.c_float(eps), dtype)
        return y

    def softmax(self, x, dtype):
        x = _c(x, dtype)
        cols = x.shape[-1]
        y = np.empty_like(x)
        self._call("softmax", _p(x), _p(y), x.size // cols, cols, dtype)
        return y

    def mha(self, x, params, H, causal, dtype, kmode=K_LITERAL):
        x = _c(x, dtype)
        B, T, E = x.shape
        ps = [_c(p, dtype) for p in params]
        arr = (C.c_void_p * 8)(*[p.ctypes.data for p in ps])
        y = np.empty_like(x)
        extra = () if self.is_ref else (kmode,)
        if self.is_ref and kmode != K_LITERAL:
            raise ValueError("the reference only computes literal K addressing")
        self._call("mha", _p(x), arr, _p(y), B, T, E, H, int(causal), dtype, *extra)
        return y

    def embedding(self, ids, table, dtype):
        ids = _c(ids, I32)
        table = _c(table, dtype)
        B, T = ids.shape
        V, D = table.shape
        y = np.empty((B, T, D), np_dtype(dtype))
        self._call("embedding", _p(ids), _p(table), _p(y), B, T, V, D, dtype)
        return y

    def conv2d(self, x, w, b, stride=1, pad=0):
        x, w, b = _c(x, F32), _c(w, F32), _c(b, F32)
        B, iC, iH, iW = x.shape
        oC, _, k, _ = w.shape
        oH = (iH + 2 * pad - k) // stride + 1
        oW = (iW + 2 * pad - k) // stride + 1
        y = np.empty((B, oC, oH, oW), np.float32)
        extra = (F32,) if self.is_ref else ()
        self._call("conv2d", _p(x), _p(w), _p(b), _p(y), B, iC, iH, iW, oC, k, stride, pad, *extra)
        return y

    def max_pool2d(self, x, k=2, stride=2, pad=0):
        x = _c(x, F32)
        B, Cc, H, W = x.shape
        oH = (H + 2 * pad - k) // stride + 1
        oW = (W + 2 * pad - k) // stride + 1
        y = np.empty((B, Cc, oH, oW), np.float32)
        extra = (F32,) if self.is_ref else ()
        self._call("max_pool2d", _p(x), _p(y), B, Cc, H, W, k, stride, pad, *extra)
        return y

    def global_avg_pool(self, x):
        x = _c(x, F32)
        B, Cc, H, W = x.shape
        y = np.empty((B, Cc, 1, 1), np.float32)
        extra = (F32,) if self.is_ref else ()
        self._call("global_avg_pool", _p(x), _p(y), B, Cc, H, W, *extra)
        return y

    # -- remaining forward entry points ------------------------------------------
    UNARY = {"exp": 0, "log": 1, "sqrt": 2, "rsqrt": 3, "sin": 4, "cos": 5}

    def unary(self, x, dtype, op):
        x = _c(x, dtype)
        y = np.empty_like(x)
        self._call("unary", _p(x), _p(y), C.c_long(x.size), dtype, self.UNARY[op])
        return y

    def leaky_relu(self, x, slope, dtype):
        x = _c(x, dtype)
        y = np.empty_like(x)
        self._call("leaky_relu", _p(x), _p(y), C.c_long(x.size), C.c_float(slope), dtype)
        return y

    def rms_norm(self, x, w, dtype, eps=1e-5):
        x, w = _c(x, dtype), _c(w, dtype)
        cols = x.shape[-1]
        y = np.empty_like(x)
        self._call("rms_norm", _p(x), _p(w), _p(y), x.size // cols, cols, C.c_float(eps), dtype)
        return y

    def batch_norm_eval(self, x, g, b, mean, var, dtype, eps=1e-5):
        x, g, b = _c(x, dtype), _c(g, dtype), _c(b, dtype)
        mean, var = _c(mean, F32), _c(var, F32)
        B, Cc, H, W = x.shape
        y = np.empty_like(x)
        self._call("batch_norm_eval", _p(x), _p(g), _p(b), _p(mean), _p(var), _p(y), B, Cc, H, W,
                   C.c_float(eps), dtype)
        return y

    def sum(self, x, dtype):
        x = _c(x, dtype)
        y = np.empty((1,), np_dtype(dtype))
        self._call("sum", _p(x), _p(y), C.c_long(x.size), dtype)
        return y

    def mean_last_dim(self, x, dtype):
        x = _c(x, dtype)
        dim = x.shape[-1]
        y = np.empty(x.shape[:-1], np_dtype(dtype))
        self._call("mean_last_dim", _p(x), _p(y), x.size // dim, dim, dtype)
        return y

    def upsample2d(self, x, scale, dtype):
        """Reference only (data movement: numpy's repeat is the CPU checker)."""
        x = _c(x, dtype)
        B, Cc, H, W = x.shape
        y = np.empty((B, Cc, H * scale, W * scale), np_dtype(dtype))
        self._call("upsample2d", _p(x), _p(y), B, Cc, H, W, scale, dtype)
        return y

    def concat(self, xs, dtype):
        """Reference only: inputs shaped [outer, dim_j, inner], joined along axis 1."""
        xs = [_c(x, dtype) for x in xs]
        outer, _, inner = xs[0].shape
        dims = [x.shape[1] for x in xs]
        y = np.empty((outer, sum(dims), inner), np_dtype(dtype))
        arr = (C.c_void_p * len(xs))(*[x.ctypes.data for x in xs])
        self._call("concat", arr, (C.c_int * len(xs))(*dims), len(xs), _p(y), outer, inner, dtype)
        return y

    def gpt_forward(self, ids, params, V, d, H, L, dtype, stop_after_layers=-1, kmode=K_LITERAL):
        ids = _c(ids, I32)
        B, T = ids.shape
        ps = [_c(p, dtype) for p in params]
        assert len(ps) == 2 + 16 * L + 4
        arr = (C.c_void_p * len(ps))(*[p.ctypes.data for p in ps])
        last = V if stop_after_layers < 0 else d
        y = np.empty((B, T, last), np_dtype(dtype))
        extra = () if self.is_ref else (kmode,)
        self._call("gpt_forward", _p(ids), arr, _p(y), B, T, V, d, H, L, dtype,
                   stop_after_layers, *extra)
        return y

    def all_reduce_sum(self, bufs, dtype):
        bs = [_c(b, dtype) for b in bufs]
        arr = (C.c_void_p * len(bs))(*[b.ctypes.data for b in bs])
        y = np.empty_like(bs[0])
        self._call("all_reduce_sum", arr, len(bs), _p(y), C.c_long(bs[0].size), dtype)
        return y


class Port(_Lib):
    def __init__(self):
        super().__init__(PORT_PATH, "orc_")

    def attention_core(self, q, k, v, BH, T, D, causal, dtype, kmode=K_LITERAL):
        q, k, v = _c(q, dtype), _c(k, dtype), _c(v, dtype)
        y = np.empty_like(q)
        self._call("attention_core", _p(q), _p(k), _p(v), _p(y), BH, T, D, int(causal), dtype, kmode)
        return y

    def set_variant(self, flags: int):
        """Diagnostic arithmetic variants of the C restatement (0 = the pinned reference
        behaviour; 1 = float accumulation in contractions; 2 = unnormalised-P rounding in
        attention). Only drift measurements use non-zero values; parity tests never do."""
        self.lib.orc_set_variant(int(flags))

    def argmax(self, x, dtype):
        x = _c(x, dtype)
        cols = x.shape[-1]
        rows = x.size // cols
        idx = np.empty(x.shape[:-1], np.int32)
        self._call("argmax", _p(x), _p(idx), C.c_long(rows), cols, dtype)
        return idx


class Ref(_Lib):
    def __init__(self):
        super().__init__(REF_PATH, "ref_")

    def convert(self, x, from_dtype, to_dtype):
        """Tensor::to(DataType) of the reference on a flat host array."""
        x = _c(x, from_dtype)
        y = np.empty(x.shape, np_dtype(to_dtype))
        self._call("convert", _p(x), _p(y), C.c_long(x.size), from_dtype, to_dtype)
        return y

    def hardware_concurrency(self) -> int:
        return int(self.lib.ref_hardware_concurrency())

    def engine_run_npz(self, path, x, in_dtype=F32, out_capacity=1 << 24):
        x = _c(x, in_dtype)
        shape = (C.c_int * x.ndim)(*x.shape)
        out = np.empty(out_capacity, np.float32)
        oshape = (C.c_int * 8)()
        ond = C.c_int(0)
        self._call("engine_run_npz", path.encode(), _p(x), shape, x.ndim, in_dtype,
                   _p(out), C.c_long(out_capacity), oshape, C.byref(ond))
        shp = tuple(oshape[i] for i in range(ond.value))
        return out[: int(np.prod(shp))].reshape(shp).copy()

    def load_npz_ok(self, path) -> tuple[bool, str]:
        fn = self.lib.ref_load_npz
        fn.restype = C.c_int
        rc = fn(path.encode())
        return rc == 0, ("" if rc == 0 else self.lib.ref_last_error().decode())


_port = None
_ref = None


def port() -> Port:
    global _port
    if _port is None:
        _port = Port()
    return _port


def ref() -> Ref:
    global _ref
    if _ref is None:
        _ref = Ref()
    return _ref


def have_ref() -> bool:
    return os.path.exists(REF_PATH)


REF_B200_PATH = os.path.join(_HERE, "_ref", "libmunet_ref_b200.so")


def have_ref_b200() -> bool:
    return os.path.exists(REF_B200_PATH)


class RefB200:
    """The unmodified reference core with munet_b200's Backend adapter registered as its
    CUDA backend (oracle/ref_b200_driver.cpp): MuNet's own Engine drives the B200 kernels."""

    def __init__(self):
        self.lib = C.CDLL(REF_B200_PATH)
        self.lib.refb200_last_error.restype = C.c_char_p

    def register(self):
        if self.lib.refb200_register() != 0:
            raise RuntimeError(self.lib.refb200_last_error().decode())

    def plugin_status(self):
        buf = C.create_string_buffer(4096)
        active = self.lib.refb200_plugin_status(buf, 4096)
        return bool(active), buf.value.decode()

    def engine_run_npz(self, path, x, dtype=F32, device_index=0, out_capacity=1 << 22):
        x = np.ascontiguousarray(x, dtype=np.float32)
        shape = (C.c_int * x.ndim)(*x.shape)
        out = np.empty(out_capacity, np.float32)
        oshape, ond = (C.c_int * 8)(), C.c_int(0)
        rc = self.lib.refb200_engine_run_npz(path.encode(), device_index, dtype, _p(x), shape, x.ndim,
                                             _p(out), C.c_long(out_capacity), oshape, C.byref(ond))
        if rc != 0:
            raise RuntimeError(self.lib.refb200_last_error().decode())
        shp = tuple(oshape[i] for i in range(ond.value))
        return out[: int(np.prod(shp))].reshape(shp).copy()

    def mha_forward(self, x, params, H, causal, dtype, device_index=0):
        """nn::MultiHeadAttention of the reference on the B200 backend; returns (y, last kernel us)."""
        x = _c(x, dtype)
        B, T, E = x.shape
        ps = [_c(p, dtype) for p in params]
        arr = (C.c_void_p * 8)(*[p.ctypes.data for p in ps])
        y = np.empty_like(x)
        us = C.c_double(0.0)
        rc = self.lib.refb200_mha_forward(_p(x), arr, _p(y), B, T, E, H, int(causal), dtype, device_index,
                                          C.byref(us))
        if rc != 0:
            raise RuntimeError(self.lib.refb200_last_error().decode())
        return y, us.value

    def all_reduce_threads(self, bufs, dtype, device_index=0):
        """Backend::all_reduce from len(bufs) threads of this process; returns what each one holds."""
        bs = [np.array(_c(b, dtype)) for b in bufs]
        arr = (C.c_void_p * len(bs))(*[b.ctypes.data for b in bs])
        rc = self.lib.refb200_all_reduce_threads(arr, len(bs), C.c_long(bs[0].size), dtype, device_index)
        if rc != 0:
            raise RuntimeError(self.lib.refb200_last_error().decode())
        return bs
