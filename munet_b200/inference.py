"""Host-side mirror of the reference's inference interface
(``munet::inference::Engine``, src/inference.hpp:292-801; Python binding
src/bindings.cpp:1272-1334): ``load`` → ``compile`` → ``run`` / ``run_batch``,
plus ``save_deploy`` which writes the reference's deploy-artifact format
(src/bindings.cpp:2031-2079, documentation/guides/serialization.md).

All compute happens in the native executor (csrc/engine.cu); this module only
marshals pointers.  Inputs/outputs are numpy arrays (host) or torch CUDA tensors.
"""
from __future__ import annotations

import ctypes as C
import json

import numpy as np

from ._lib import BF16, F32, I32, Context, MuNetError, _stream, lib

_NP = {F32: np.float32, BF16: np.uint16, I32: np.int32}


def gpt_decoder_config(vocab: int, ctx_len: int, d_model: int, n_heads: int, n_layers: int) -> dict:
    """Module tree of the reference's decoder demo (demos/multigpu/gpt3_multi_gpu_demo.py:116-172)
    as an extension node of the deploy format."""
    return {"type": "GPTDecoder", "vocab": vocab, "ctx_len": ctx_len, "d_model": d_model,
            "n_heads": n_heads, "n_layers": n_layers}


def gpt_param_names(n_layers: int) -> list[str]:
    """Parameter names in the flat order the CPU checker uses (oracle.gpt_forward)."""
    names = ["token_embed.weight", "pos_embed.weight"]
    for l in range(n_layers):
        p = f"blocks.{l}."
        names += [p + "ln1.weight", p + "ln1.bias"]
        for proj in ("q_proj", "k_proj", "v_proj", "out_proj"):
            names += [p + f"attn.{proj}.weight", p + f"attn.{proj}.bias"]
        names += [p + "ln2.weight", p + "ln2.bias", p + "ff.0.weight", p + "ff.0.bias",
                  p + "ff.2.weight", p + "ff.2.bias"]
    return names + ["ln_f.weight", "ln_f.bias", "head.weight", "head.bias"]


def gpt_param_shapes(vocab: int, ctx_len: int, d_model: int, n_layers: int) -> dict:
    """name → shape for every parameter of the decoder (Linear weights are [in, out])."""
    d = d_model
    shapes = {}
    for name in gpt_param_names(n_layers):
        leaf = name.split(".")[-1]
        if name == "token_embed.weight":
            s = (vocab, d)
        elif name == "pos_embed.weight":
            s = (ctx_len, d)
        elif ".ln" in name or name.startswith("ln_f"):
            s = (d,)
        elif ".ff.0." in name:
            s = (d, 4 * d) if leaf == "weight" else (4 * d,)
        elif ".ff.2." in name:
            s = (4 * d, d) if leaf == "weight" else (d,)
        elif name.startswith("head."):
            s = (d, vocab) if leaf == "weight" else (vocab,)
        else:
            s = (d, d) if leaf == "weight" else (d,)
        shapes[name] = s
    return shapes


def save_deploy(path: str, config: dict, tensors: dict[str, np.ndarray], producer: str = "munet"):
    """Write a MuNet deploy artifact: uncompressed .npz, metadata members as 0-d arrays,
    float32 / float16 / int32 payload, ``__tensor_names__`` = sorted payload keys."""
    payload = {}
    for k, v in tensors.items():
        v = np.ascontiguousarray(v)
        if v.dtype not in (np.float32, np.float16, np.int32):
            raise ValueError(f"{k}: deploy artifacts hold float32/float16/int32 tensors only")
        payload[k] = v
    meta = {
        "__format_name__": np.array("munet_model"),
        "__format_revision__": np.array(1, dtype=np.int64),
        "__format_version__": np.array("munet_model_v1"),
        "__producer__": np.array(producer),
        "__artifact_kind__": np.array("deploy_model"),
        "__artifact_scope__": np.array("runtime_only"),
        "__default_load_mode__": np.array("eval"),
        "__contains_training_state__": np.array(False),
        "__recommended_loader__": np.array("load_for_inference"),
        "__compile_contract_policy__": np.array("external"),
        "__config__": np.array(json.dumps(config)),
        "__tensor_names__": np.array(json.dumps(sorted(payload))),
    }
    with open(path, "wb") as f:
        np.savez(f, **meta, **payload)


def inspect_artifact(path: str) -> dict:
    """Validate a deploy artifact on the host (no GPU) and return its module tree and
    tensor table; raises MuNetError with the loader's message when it is rejected."""
    cap = 1 << 22
    out, err = C.create_string_buffer(cap), C.create_string_buffer(1024)
    rc = lib().mu_artifact_inspect(path.encode(), out, cap, err, 1024)
    if rc:
        raise MuNetError(rc, err.value.decode())
    return json.loads(out.value.decode())


class Engine:
    """``load`` → ``compile`` → ``run``; one instance per device context."""

    def __init__(self, ctx: Context | None = None, device: int = 0, compute_dtype: int = F32,
                 kmode: int = 0, use_graph: bool = True, argmax: bool = False, comm=None):
        self._lib = lib()
        self.ctx = ctx or Context(device)
        self.compute_dtype = compute_dtype
        h = C.c_void_p()
        rc = self._lib.mu_engine_create(self.ctx._h, C.byref(h))
        if rc:
            raise MuNetError(rc, "mu_engine_create failed")
        self._h = h
        self._keep = None
        self.argmax = argmax
        self._opt("kmode", kmode)
        self._opt("use_graph", int(use_graph))
        self._opt("argmax", int(argmax))
        self.comm = comm
        if comm is not None and comm.world > 1:  # tensor-parallel shard of the decoder blocks
            self._opt("tp_size", comm.world)
            self._opt("tp_rank", comm.rank)
            self._rc(self._lib.mu_engine_set_comm(self._h, comm._h))
        self.input_shape = None
        self.output_shape = None

    def _rc(self, rc):
        if rc:
            raise MuNetError(rc, self._lib.mu_engine_last_error(self._h).decode())

    def _opt(self, name, value):
        self._rc(self._lib.mu_engine_set_option(self._h, name.encode(), int(value)))

    def close(self):
        if getattr(self, "_h", None):
            self._lib.mu_engine_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- load ------------------------------------------------------------------
    def load(self, source, tensors=None, tensor_dtype: int | None = None):
        """``load(path)`` reads a deploy artifact; ``load(config_dict, tensors)`` takes the
        module tree and named tensors (numpy float32 / uint16-bf16, or torch CUDA tensors)."""
        if isinstance(source, str):
            self._rc(self._lib.mu_engine_load(self._h, source.encode(), self.compute_dtype))
            return self
        names = list(tensors)
        n = len(names)
        on_device = any(hasattr(tensors[k], "data_ptr") for k in names)
        ptrs, dts, nds, shp, keep = [], [], [], [], []
        for k in names:
            t = tensors[k]
            if hasattr(t, "data_ptr"):
                if not on_device:
                    raise ValueError("mixing host and device tensors in one load is not supported")
                tt = t.contiguous()
                keep.append(tt)
                ptrs.append(tt.data_ptr())
                dts.append(_torch_code(tt.dtype))
                shape = tuple(tt.shape)
            else:
                a = np.ascontiguousarray(t)
                keep.append(a)
                ptrs.append(a.ctypes.data)
                dts.append(tensor_dtype if (tensor_dtype is not None and a.dtype == np.uint16)
                           else {np.dtype(np.float32): F32, np.dtype(np.uint16): BF16,
                                 np.dtype(np.int32): I32, np.dtype(np.float16): 1}[a.dtype])
                shape = a.shape
            nds.append(len(shape))
            shp += list(shape)
        self._keep = keep
        self._rc(self._lib.mu_engine_load_memory(
            self._h, json.dumps(source).encode(), n,
            (C.c_char_p * n)(*[k.encode() for k in names]), (C.c_void_p * n)(*ptrs),
            (C.c_int * n)(*dts), (C.c_int * n)(*nds), (C.c_longlong * max(len(shp), 1))(*shp),
            int(on_device), self.compute_dtype))
        return self

    # -- compile ---------------------------------------------------------------
    def compile(self, input_shape, input_dtype: int | None = None):
        shape = tuple(int(s) for s in input_shape)
        dt = self.compute_dtype if input_dtype is None else input_dtype
        self._rc(self._lib.mu_engine_compile(self._h, (C.c_int * len(shape))(*shape), len(shape), dt))
        self._keep = None  # weights now live in the engine's slab
        self.input_shape, self.input_dtype = shape, dt
        out = (C.c_int * 8)()
        nd, odt = C.c_int(), C.c_int()
        self._rc(self._lib.mu_engine_output_shape(self._h, out, C.byref(nd), C.byref(odt)))
        self.output_shape = tuple(out[i] for i in range(nd.value))
        self.output_dtype = odt.value
        return self

    def stats(self) -> dict:
        v = [C.c_longlong() for _ in range(5)]
        self._rc(self._lib.mu_engine_stats(self._h, *[C.byref(x) for x in v]))
        keys = ["arena_bytes", "weight_bytes", "n_ops", "n_launches", "unplanned_bytes"]
        return {k: x.value for k, x in zip(keys, v)}

    # -- run -------------------------------------------------------------------
    def run(self, x, out=None, stream=None):
        """Host numpy in → host numpy out (copies inside), or CUDA tensor in → result stays in
        the engine's arena (returned as raw device pointer via ``output_ptr``) unless ``out``."""
        if self.input_shape is None:
            raise MuNetError(1, "Engine: run() called before compile()")
        host_in = isinstance(x, np.ndarray)
        if tuple(x.shape) != self.input_shape:
            raise MuNetError(1, f"Engine: input shape {tuple(x.shape)} does not match compiled "
                                f"contract {self.input_shape}")
        if host_in:
            x = np.ascontiguousarray(x, dtype=_NP[self.input_dtype])
            xin = x.ctypes.data
            if out is None:
                out = np.empty(self.output_shape, _NP[self.output_dtype])
            am = np.empty(self.output_shape[:-1], np.int32) if self.argmax else None
            self._rc(self._lib.mu_engine_run(self._h, xin, 1, out.ctypes.data, 1,
                                             None if am is None else am.ctypes.data, 1,
                                             _stream(stream)))
            return (out, am) if self.argmax else out
        self._rc(self._lib.mu_engine_run(self._h, x.data_ptr(), 0,
                                         None if out is None else out.data_ptr(), 0, None, 0,
                                         _stream(stream)))
        return out

    OP_KINDS = ["embed", "layer_norm", "linear", "qkv_linear", "attention", "eltwise", "argmax",
                "conv2d", "max_pool2d", "global_avg_pool", "all_reduce", "batch_norm", "upsample",
                "leaky_relu", "rms_norm"]

    def profile(self, reps: int = 1, stream=None) -> list[dict]:
        """Eager forward with CUDA events around every op: per-op ms + algorithmic work."""
        cap = self.stats()["n_ops"]
        n = C.c_int()
        kinds = (C.c_int * cap)()
        ms = (C.c_float * cap)()
        fl = (C.c_double * cap)()
        by = (C.c_double * cap)()
        self._rc(self._lib.mu_engine_profile(self._h, reps, cap, C.byref(n), kinds, ms, fl, by,
                                             _stream(stream)))
        return [{"kind": self.OP_KINDS[kinds[i]], "ms": ms[i], "flops": fl[i], "bytes": by[i]}
                for i in range(n.value)]

    def run_batch(self, inputs, stream=None):
        """Engine::run_batch (src/inference.hpp:612-627): independent inputs, one run each."""
        return [self.run(x, stream=stream) for x in inputs]

    @property
    def output_ptr(self) -> int:
        return int(self._lib.mu_engine_output_ptr(self._h) or 0)

    @property
    def argmax_ptr(self) -> int:
        return int(self._lib.mu_engine_argmax_ptr(self._h) or 0)


def _torch_code(dt) -> int:
    import torch
    return {torch.float32: F32, torch.bfloat16: BF16, torch.int32: I32, torch.float16: 1}[dt]
