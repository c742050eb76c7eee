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


class PreparedInputCache:
    """Device copies of host inputs, keyed by the identity and version of the host object:
    the reference's ``detail::PreparedInputCache`` (src/inference.hpp:186-289). Same policy:
    at most ``max_entries`` entries and ``max_bytes`` bytes, a value larger than ``max_bytes`` is
    not cached, storing under an identity that is already present replaces it, and room is made
    by evicting the oldest entries first. ``store`` returns the number of evictions."""

    def __init__(self, max_entries: int = 8, max_bytes: int = 64 * 1024 * 1024):
        self.configure(max_entries, max_bytes)

    def configure(self, max_entries: int, max_bytes: int):
        self.max_entries, self.max_bytes = int(max_entries), int(max_bytes)
        self.reset()

    def reset(self):
        self._entries = []  # [identity, version, value, nbytes], oldest first
        self.current_bytes = 0

    def find(self, identity, version):
        for ident, ver, value, _ in self._entries:
            if ident == identity and ver == version:
                return value
        return None

    def store(self, identity, version, value, nbytes: int) -> int:
        if value is None or self.max_entries == 0 or self.max_bytes == 0 or nbytes > self.max_bytes:
            return 0
        for i, e in enumerate(self._entries):
            if e[0] == identity:
                self.current_bytes -= e[3]
                del self._entries[i]
                break
        evictions = 0
        while self._entries and (len(self._entries) >= self.max_entries
                                 or self.current_bytes + nbytes > self.max_bytes):
            self.current_bytes -= self._entries[0][3]
            del self._entries[0]
            evictions += 1
        self._entries.append([identity, version, value, nbytes])
        self.current_bytes += nbytes
        return evictions

    def __len__(self):
        return len(self._entries)


def _input_identity(x):
    """(identity, version) of a host input, or None when changes to it cannot be noticed.
    torch CPU tensors carry a version counter (bumped by in-place ops, like the reference's
    ``Tensor::version``); a numpy array only qualifies when it is read-only."""
    if hasattr(x, "_version") and hasattr(x, "data_ptr"):
        return (id(x), x.data_ptr()), int(x._version)
    if isinstance(x, np.ndarray) and not x.flags.writeable:
        return (id(x), x.ctypes.data), 0
    return None


class Engine:
    """``load`` → ``compile`` → ``run``; one instance per device context."""

    def __init__(self, ctx: Context | None = None, device: int = 0, compute_dtype: int = F32,
                 kmode: int = 0, use_graph: bool = True, argmax: bool = False, comm=None,
                 tp_overlap: bool | None = None, tp_exchange: str = "nccl"):
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
            if tp_exchange not in ("nccl", "peer", "push", "gather", "rows"):
                raise ValueError("tp_exchange is 'nccl', 'peer', 'push', 'gather' or 'rows'")
            # row chunks with the exchange of one under the GEMM of the next pay off for the NCCL
            # path (measured 105.5 against 108.6 ms on the 24-layer decoder) but not for the
            # peer-memory one, whose kernel wants every SM for its NVLink loads (93.6 against 96.4)
            if tp_overlap is None or tp_exchange in ("push", "gather", "rows"):  # the pushed exchanges are never chunked
                tp_overlap = tp_exchange == "nccl"
            self._opt("tp_overlap", int(tp_overlap))
            # "peer": the reduce kernel loads the other rank's partial over NVLink; "push": the
            # row-parallel GEMM writes its tiles into the other rank's memory while it runs;
            # "gather": as "push" for the MLP, and the attention kernel writes its heads' output
            # into both ranks' buffer so that out_proj runs unsharded (no partial sums to add);
            # "rows": as "gather", but each rank runs out_proj on its half of the token rows only
            # and its epilogue writes them into both ranks' residual stream
            self._opt("tp_exchange", {"nccl": 0, "peer": 1, "push": 2, "gather": 3, "rows": 4}[tp_exchange])
            self._rc(self._lib.mu_engine_set_comm(self._h, comm._h))
        self.tp_exchange = tp_exchange if (comm is not None and comm.world > 1) else "nccl"
        self._peer_maps = []
        self.input_shape = None
        self.output_shape = None
        # host-side bookkeeping with the reference's names (EngineStats, src/inference.hpp:43-68)
        self._cache = PreparedInputCache()
        self._estats = {"runs": 0, "load_to_device_ms": 0.0, "compile_ms": 0.0, "last_run_ms": 0.0,
                        "last_prepare_input_ms": 0.0, "last_forward_ms": 0.0,
                        "compiled_input_shape": [], "compiled_output_shape": [],
                        "prepared_input_cache_hits": 0, "prepared_input_cache_misses": 0,
                        "prepared_input_cache_evictions": 0}
        self._observer = None
        # EngineConfig flags of the reference (src/inference.hpp:30-41)
        self._strict_shape_check = True
        self._lean_mode = False
        self._capture_profiler_memory = False
        self._contract = None  # expected input shape, -1 = any extent

    # -- reference-style configuration and bookkeeping ------------------------------
    def set_strict_shape_check(self, enabled: bool):
        """Engine::set_strict_shape_check (src/inference.hpp:317-319). With the check off the
        reference forwards whatever arrives; here an input of another shape (same rank) gets a
        plan of its own on first sight."""
        self._strict_shape_check = bool(enabled)

    def set_lean_mode(self, enabled: bool):
        """Engine::set_lean_mode (src/inference.hpp:330-335): drop the diagnostic bookkeeping —
        memory capture is switched off with it, and the load event no longer reports parameter
        counts."""
        self._lean_mode = bool(enabled)
        if enabled:
            self._capture_profiler_memory = False

    def set_capture_profiler_memory(self, enabled: bool):
        """Engine::set_capture_profiler_memory (src/inference.hpp:323-328): record the device
        memory behind the engine after load, compile and every run; leaves lean mode."""
        self._capture_profiler_memory = bool(enabled)
        if enabled:
            self._lean_mode = False

    @property
    def lean_mode(self) -> bool:
        return self._lean_mode

    @property
    def capture_profiler_memory(self) -> bool:
        return self._capture_profiler_memory

    def _refresh_memory_stats(self):
        if self._capture_profiler_memory and self.input_shape is not None:
            st = self.stats()
            self._estats["current_memory_bytes"] = st["arena_bytes"] + st["weight_bytes"]
            self._estats["peak_memory_bytes"] = max(self._estats.get("peak_memory_bytes", 0),
                                                    self._estats["current_memory_bytes"])

    def set_observer(self, observer):
        """``observer(event: dict)`` is called for load/compile/run completion and errors
        (EngineEvent, src/inference.hpp:70-92)."""
        self._observer = observer

    def _emit(self, kind, duration_ms=0.0, message=""):
        if self._observer is not None:
            self._observer({"type": kind, "device": ("cuda", self.ctx.device), "run_index": self._estats["runs"],
                            "duration_ms": duration_ms, "input_shape": list(self.input_shape or ()),
                            "output_shape": list(self.output_shape or ()), "message": message})

    def set_prepared_input_cache_entries(self, entries: int):
        self._cache.configure(entries, self._cache.max_bytes)

    def set_prepared_input_cache_max_bytes(self, nbytes: int):
        self._cache.configure(self._cache.max_entries, nbytes)

    def clear_prepared_input_cache(self):
        self._cache.reset()

    @property
    def engine_stats(self) -> dict:
        """EngineStats of the reference plus the executor's plan figures (``stats()``)."""
        d = dict(self._estats)
        d["prepared_input_cache_entries"] = len(self._cache)
        d["prepared_input_cache_bytes"] = self._cache.current_bytes
        return d

    def _prepared(self, x):
        """Device copy of a host input through the cache; None when the input cannot be keyed."""
        key = _input_identity(x)
        if key is None:
            return None
        hit = self._cache.find(*key)
        if hit is not None:
            self._estats["prepared_input_cache_hits"] += 1
            return hit
        self._estats["prepared_input_cache_misses"] += 1
        import torch
        self._check_contract(tuple(x.shape))
        # the same conversion the uncached path applies: an int64 id tensor or a float64 array
        # must not reach the engine as raw bytes
        t = _as_host_tensor(x, self.input_dtype)
        dev = t.to(torch.device("cuda", self.ctx.device))
        self._estats["prepared_input_cache_evictions"] += self._cache.store(
            key[0], key[1], dev, dev.numel() * dev.element_size())
        return dev

    def prepare_batch(self, inputs):
        """Engine::prepare_batch (src/inference.hpp:368-382): move the inputs to the device ahead
        of the runs; ``run`` on the same (unchanged) host object then skips the copy."""
        if self.input_shape is None:
            raise MuNetError(1, "Engine: prepare_batch() called before compile()")
        for x in inputs:
            self._prepared(x)

    def _rc(self, rc):
        if rc:
            raise MuNetError(rc, self._lib.mu_engine_last_error(self._h).decode())

    def _check_contract(self, shape):
        """The compile-time contract (exact extents or -1 wildcards) against ``shape``, with the
        reference's reasons (ShapeContract::mismatch_reason, src/inference.hpp:162-176)."""
        c = self._contract if self._strict_shape_check else (-1,) * len(self._contract)
        reason = None
        if len(shape) != len(c):
            reason = "rank mismatch"
        else:
            for i, (want, got) in enumerate(zip(c, shape)):
                if want != -1 and want != got:
                    reason = f"dim mismatch at index {i}"
                    break
        if reason:
            self._emit("error", message="run failed: shape contract")
            raise MuNetError(1, f"Engine run input shape mismatch: {reason} (input shape "
                                f"{tuple(shape)} does not match compiled contract {tuple(self._contract)})")

    def _select(self, shape):
        """Make the plan of ``shape`` the active one (built on first sight)."""
        if tuple(shape) == self.input_shape:
            return
        if not self._strict_shape_check and any(w != -1 and w != g for w, g in zip(self._contract, shape)):
            # outside the compiled contract but allowed: widen the engine's contract to the rank
            n = len(shape)
            self._rc(self._lib.mu_engine_compile_contract(
                self._h, (C.c_int * n)(*shape), n, (C.c_int * n)(*([-1] * n)), self.input_dtype))
            self._contract = (-1,) * n
        else:
            self._rc(self._lib.mu_engine_select_shape(self._h, (C.c_int * len(shape))(*shape), len(shape)))
        self.input_shape = tuple(shape)
        self._read_output_shape()

    def select_shape(self, shape):
        """Make the plan for ``shape`` (which must satisfy the compile-time contract) the active
        one ahead of a run, so that building it is not part of the first run's time."""
        if self.input_shape is None:
            raise MuNetError(1, "Engine: select_shape() called before compile()")
        shape = tuple(int(s) for s in shape)
        self._check_contract(shape)
        self._select(shape)

    def _read_output_shape(self):
        out = (C.c_int * 8)()
        nd, odt = C.c_int(), C.c_int()
        self._rc(self._lib.mu_engine_output_shape(self._h, out, C.byref(nd), C.byref(odt)))
        self.output_shape = tuple(out[i] for i in range(nd.value))
        self.output_dtype = odt.value

    @property
    def plan_count(self) -> int:
        """Plans (one per concrete input shape met so far) the engine holds."""
        return int(self._lib.mu_engine_plan_count(self._h))

    def _opt(self, name, value):
        self._rc(self._lib.mu_engine_set_option(self._h, name.encode(), int(value)))

    def close(self):
        if getattr(self, "_h", None):
            self._lib.mu_engine_destroy(self._h)
            self._h = None
            for p in getattr(self, "_peer_maps", []):
                self._lib.mu_ipc_close(self.ctx._h, p)
            self._peer_maps = []

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- load ------------------------------------------------------------------
    def load(self, source, tensors=None, tensor_dtype: int | None = None):
        """``load(path)`` reads a deploy artifact; ``load(config_dict, tensors)`` takes the
        module tree and named tensors (numpy float32 / uint16-bf16, or torch CUDA tensors)."""
        import time
        t0 = time.perf_counter()
        if isinstance(source, str):
            try:
                self._rc(self._lib.mu_engine_load(self._h, source.encode(), self.compute_dtype))
            except MuNetError as e:
                self._emit("error", message=f"load failed: {e}")
                raise
            self._estats["load_to_device_ms"] = (time.perf_counter() - t0) * 1e3
            self._emit("load_completed", self._estats["load_to_device_ms"], self._load_message(None))
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
        self._estats["load_to_device_ms"] = (time.perf_counter() - t0) * 1e3
        self._emit("load_completed", self._estats["load_to_device_ms"], self._load_message(n))
        return self

    def _load_message(self, n_tensors):
        """The reference's load event text (src/inference.hpp:426-438); the tensor census is part
        of the diagnostics that lean mode leaves out."""
        msg = f"Module loaded on cuda:{self.ctx.device}; gradients will remain disabled during compile/run"
        if not self._lean_mode and n_tensors is not None:
            msg += f" ({n_tensors} parameter/buffer tensor(s) staged)"
        return msg

    # -- compile ---------------------------------------------------------------
    def compile(self, input_shape, input_dtype: int | None = None, expected_input_shape=None,
                expected_output_shape=None):
        """Engine::compile (src/inference.hpp:446-539). ``expected_input_shape`` may hold -1 for
        extents that vary between runs (tests/test_inference.cpp:402-438); every concrete shape
        met later gets its own plan, the weights are shared. ``expected_output_shape`` is checked
        against the example's output like the reference does."""
        import time
        t0 = time.perf_counter()
        shape = tuple(int(s) for s in input_shape)
        dt = self.compute_dtype if input_dtype is None else input_dtype
        n = len(shape)
        exp = None if expected_input_shape is None else tuple(int(s) for s in expected_input_shape)
        try:
            if exp is not None and len(exp) != n:
                raise MuNetError(1, "Engine compile input shape mismatch: rank mismatch")
            self._rc(self._lib.mu_engine_compile_contract(
                self._h, (C.c_int * n)(*shape), n, None if exp is None else (C.c_int * n)(*exp), dt))
        except MuNetError as e:
            self._emit("error", message=f"compile failed: {e}")
            raise
        self._keep = None  # weights now live in the engine's slab
        self.input_shape, self.input_dtype = shape, dt
        self._contract = exp if exp is not None else shape
        self._read_output_shape()
        if expected_output_shape is not None:
            eo = tuple(int(s) for s in expected_output_shape)
            bad = len(eo) != len(self.output_shape) or any(
                w != -1 and w != g for w, g in zip(eo, self.output_shape))
            if bad:
                self._emit("error", message="compile failed: output shape contract")
                raise MuNetError(1, f"Engine compile output shape mismatch: expected {eo}, "
                                    f"got {self.output_shape}")
        self._cache.reset()
        self._estats.update(compile_ms=(time.perf_counter() - t0) * 1e3,
                            compiled_input_shape=list(shape), compiled_output_shape=list(self.output_shape))
        self._refresh_memory_stats()
        self._emit("compile_completed", self._estats["compile_ms"])
        return self

    def peer_handles(self) -> list:
        """CUDA IPC handles (64 bytes each) of this rank's arena and exchange counters, to be
        handed to the other rank of a two-rank peer-memory exchange (tp_exchange="peer")."""
        arena, counters = C.c_void_p(), C.c_void_p()
        self._rc(self._lib.mu_engine_peer_info(self._h, C.byref(arena), C.byref(counters)))
        out = []
        for ptr in (arena, counters):
            buf = C.create_string_buffer(64)
            self.ctx._rc(self._lib.mu_ipc_export(self.ctx._h, ptr, buf, 64))
            out.append(buf.raw)
        return out

    def attach_peer(self, their_handles):
        """Map the other rank's arena and counters and attach them. Runs one forward (a real
        exchange) and captures the graph: both ranks call this at the same time."""
        maps = []
        for raw in their_handles:
            p = C.c_void_p()
            self.ctx._rc(self._lib.mu_ipc_open(self.ctx._h, C.create_string_buffer(raw, 64), C.byref(p)))
            maps.append(p)
        self._peer_maps = maps
        self._rc(self._lib.mu_engine_attach_peer(self._h, maps[0], maps[1]))
        return self

    def attach_peer_via_torch_distributed(self):
        """peer_handles() traded over the default torch.distributed group, then attach_peer()."""
        import torch.distributed as dist
        everyone = [None] * dist.get_world_size()
        dist.all_gather_object(everyone, self.peer_handles())
        dist.barrier()
        return self.attach_peer(everyone[1 - dist.get_rank()])

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
        import time
        t0 = time.perf_counter()
        self._estats["last_prepare_input_ms"] = 0.0
        host_in = isinstance(x, np.ndarray) or (hasattr(x, "is_cuda") and not x.is_cuda)
        self._check_contract(tuple(x.shape))
        self._select(tuple(x.shape))
        if host_in and len(self._cache) and _input_identity(x) is not None \
                and self._cache.find(*_input_identity(x)) is not None:
            dev = self._prepared(x)  # prepared earlier and unchanged since: no host copy
            self._estats["last_prepare_input_ms"] = (time.perf_counter() - t0) * 1e3
            if out is None:
                out = np.empty(self.output_shape, _NP[self.output_dtype])
            am = np.empty(self.output_shape[:-1], np.int32) if self.argmax else None
            self._rc(self._lib.mu_engine_run(self._h, dev.data_ptr(), 0, out.ctypes.data, 1,
                                             None if am is None else am.ctypes.data, 1, _stream(stream)))
            self._ran(t0)
            return (out, am) if self.argmax else out
        if host_in:
            x = _as_host_tensor(x, self.input_dtype)  # kept alive until the call returns
            xin = x.data_ptr()
            if out is None:
                out = np.empty(self.output_shape, _NP[self.output_dtype])
            am = np.empty(self.output_shape[:-1], np.int32) if self.argmax else None
            self._rc(self._lib.mu_engine_run(self._h, xin, 1, out.ctypes.data, 1,
                                             None if am is None else am.ctypes.data, 1,
                                             _stream(stream)))
            self._ran(t0)
            return (out, am) if self.argmax else out
        # a device tensor is consumed as raw bytes: its dtype must be the compiled input dtype
        if _torch_code(x.dtype) != self.input_dtype:
            self._emit("error", message="run failed: input dtype")
            raise MuNetError(1, f"Engine: CUDA input has dtype {x.dtype}, the engine was compiled for "
                                f"dtype code {self.input_dtype}; convert it before run()")
        if not x.is_contiguous():
            x = x.contiguous()
        self._rc(self._lib.mu_engine_run(self._h, x.data_ptr(), 0,
                                         None if out is None else out.data_ptr(), 0, None, 0,
                                         _stream(stream)))
        self._ran(t0)
        return out

    def _ran(self, t0):
        import time
        ms = (time.perf_counter() - t0) * 1e3
        self._estats["runs"] += 1
        self._estats["last_run_ms"] = ms
        self._estats["last_forward_ms"] = ms - self._estats["last_prepare_input_ms"]
        self._refresh_memory_stats()
        self._emit("run_completed", ms)

    OP_KINDS = ["embed", "layer_norm", "linear", "qkv_linear", "attention", "eltwise", "argmax",
                "conv2d", "max_pool2d", "global_avg_pool", "all_reduce", "batch_norm", "upsample",
                "leaky_relu", "rms_norm", "peer_step", "peer_wait", "peer_signal", "peer_reduce", "join",
                "peer_wait_ready", "peer_signal_done"]

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
        dims = (C.c_int * (4 * cap))()
        self._rc(self._lib.mu_engine_op_dims(self._h, cap, dims))
        return [{"kind": self.OP_KINDS[kinds[i]], "ms": ms[i], "flops": fl[i], "bytes": by[i],
                 "mkn": (dims[4 * i], dims[4 * i + 1], dims[4 * i + 2]), "residual": bool(dims[4 * i + 3])}
                for i in range(n.value)]

    def run_batch(self, inputs, stream=None):
        """Engine::run_batch (src/inference.hpp:612-627): independent inputs, one run each."""
        outputs = []
        self.run_batch_into(inputs, outputs, stream=stream)
        return outputs

    def run_batch_into(self, inputs, outputs: list, stream=None):
        """Engine::run_batch_into: ``outputs`` is cleared and receives one result per input."""
        outputs.clear()
        for x in inputs:
            outputs.append(self.run(x, stream=stream))

    @property
    def output_ptr(self) -> int:
        return int(self._lib.mu_engine_output_ptr(self._h) or 0)

    @property
    def argmax_ptr(self) -> int:
        return int(self._lib.mu_engine_argmax_ptr(self._h) or 0)


def _torch_code(dt) -> int:
    import torch
    return {torch.float32: F32, torch.bfloat16: BF16, torch.int32: I32, torch.float16: 1}.get(dt, -1)


def _as_host_tensor(x, code: int):
    """A contiguous torch CPU tensor holding ``x`` in the engine's input dtype. 16-bit patterns
    (numpy uint16, torch int16) given for a bfloat16 input are taken as bf16 bits, as everywhere
    else in this package; any other dtype is converted by value (int64 ids -> int32, float64 ->
    float32, ...), which is what the reference's prepare_input does with Tensor::to."""
    import torch
    want = _torch_dtype(code)
    if isinstance(x, np.ndarray):
        if code == BF16 and x.dtype == np.uint16:
            return torch.from_numpy(np.ascontiguousarray(x).view(np.int16)).view(torch.bfloat16)
        t = torch.from_numpy(np.ascontiguousarray(x))
    else:
        t = x
    if code == BF16 and t.dtype == torch.int16:
        return t.contiguous().view(torch.bfloat16)
    return t.contiguous().to(want)


def _torch_dtype(code: int):
    import torch
    return {F32: torch.float32, BF16: torch.bfloat16, I32: torch.int32, 1: torch.float16}[code]
