"""ONNX -> MuNet deploy artifact for single-stream ("native sequential") graphs.

Stands in for ``munet.inference.compile_onnx`` / ``report_onnx_unsupported_ops`` /
``onnx_native_conversion_map`` of the reference
(python/munet_nn/_helpers/onnx_integration.py:166-169, 234-426, 864-926): a graph with one input and
one output whose nodes form a chain is lowered node by node to MuNet layers; anything else is
refused with the list of operators that block the conversion. The result is the (config, tensors)
pair that ``munet_b200.inference.Engine.load`` and ``save_deploy`` take, i.e. a deploy artifact
the reference's own loader reads as well.

The ``onnx`` package is not needed: an ONNX file is a protobuf ``ModelProto`` and the few
messages that matter here (ModelProto, GraphProto, NodeProto, AttributeProto, TensorProto,
ValueInfoProto) are decoded straight from the wire format with the field numbers of the public
``onnx.proto``.

Operators lowered: Gemm (transA = 0, alpha = beta = 1), MatMul with a constant right-hand side,
Conv (2-D, one group, unit dilation, square kernel / stride, symmetric padding), MaxPool (2-D,
square, symmetric), Relu, LeakyRelu, Sigmoid, Tanh, Gelu, Flatten (axis 1), GlobalAveragePool, and
(beyond the reference's list) BatchNormalization in its inference form; Identity passes through;
Constant nodes feed later nodes.
"""
from __future__ import annotations

import struct
from collections import Counter

import numpy as np

__all__ = ["read_onnx", "compile_onnx", "report_onnx_unsupported_ops", "onnx_native_conversion_map"]


# --------------------------------------------------------------------------------------------
# protobuf wire format
# --------------------------------------------------------------------------------------------
def _varint(buf: bytes, pos: int):
    val = shift = 0
    while True:
        if pos >= len(buf):
            raise ValueError("ONNX file truncated inside a varint")
        b = buf[pos]
        pos += 1
        val |= (b & 0x7F) << shift
        if not b & 0x80:
            return val, pos
        shift += 7
        if shift > 63:
            raise ValueError("ONNX file: varint longer than 64 bits")


def _fields(buf: bytes):
    """Yield (field number, wire type, value) of one message; length-delimited values are bytes."""
    pos, n = 0, len(buf)
    while pos < n:
        key, pos = _varint(buf, pos)
        num, wt = key >> 3, key & 7
        if wt == 0:
            val, pos = _varint(buf, pos)
        elif wt == 1:
            if pos + 8 > n:
                raise ValueError("ONNX file truncated inside a 64-bit field")
            val, pos = buf[pos:pos + 8], pos + 8
        elif wt == 2:
            ln, pos = _varint(buf, pos)
            if ln > n - pos:
                raise ValueError("ONNX file truncated inside a length-delimited field")
            val, pos = buf[pos:pos + ln], pos + ln
        elif wt == 5:
            if pos + 4 > n:
                raise ValueError("ONNX file truncated inside a 32-bit field")
            val, pos = buf[pos:pos + 4], pos + 4
        else:
            raise ValueError(f"ONNX file: unsupported wire type {wt}")
        yield num, wt, val


def _sint64(v: int) -> int:  # int64 fields are plain two's complement varints
    return v - (1 << 64) if v >= (1 << 63) else v


def _packed_varints(val, wt):
    if wt == 0:
        return [_sint64(val)]
    out, pos = [], 0
    while pos < len(val):
        v, pos = _varint(val, pos)
        out.append(_sint64(v))
    return out


def _packed_floats(val, wt):
    if wt == 5:
        return [struct.unpack("<f", val)[0]]
    return list(struct.unpack("<%df" % (len(val) // 4), val))


# --------------------------------------------------------------------------------------------
# ONNX messages (field numbers of onnx.proto)
# --------------------------------------------------------------------------------------------
_TENSOR_DTYPES = {1: np.float32, 2: np.uint8, 3: np.int8, 5: np.int16, 6: np.int32, 7: np.int64,
                  9: np.bool_, 10: np.float16, 11: np.float64}


def _tensor(buf: bytes):
    dims, dtype, name, raw = [], 0, "", None
    floats, int32s, int64s, doubles = [], [], [], []
    for num, wt, val in _fields(buf):
        if num == 1:
            dims += _packed_varints(val, wt)
        elif num == 2:
            dtype = val
        elif num == 4:
            floats += _packed_floats(val, wt)
        elif num == 5:
            int32s += _packed_varints(val, wt)
        elif num == 7:
            int64s += _packed_varints(val, wt)
        elif num == 8:
            name = val.decode()
        elif num == 9:
            raw = val
        elif num == 10:
            doubles += (list(struct.unpack("<%dd" % (len(val) // 8), val)) if wt == 2
                        else [struct.unpack("<d", val)[0]])
        elif num == 13 or (num == 14 and val == 1):
            raise ValueError(f"ONNX tensor '{name}': external data is not supported")
    if dtype not in _TENSOR_DTYPES:
        raise ValueError(f"ONNX tensor '{name}': data type {dtype} is not supported")
    np_dt = np.dtype(_TENSOR_DTYPES[dtype])
    count = int(np.prod(dims)) if dims else 1
    if raw is not None:
        if len(raw) != count * np_dt.itemsize:
            raise ValueError(f"ONNX tensor '{name}': raw_data holds {len(raw)} bytes, "
                             f"shape {dims} needs {count * np_dt.itemsize}")
        arr = np.frombuffer(raw, dtype=np_dt.newbyteorder("<")).astype(np_dt)
    elif dtype == 1:
        arr = np.asarray(floats, dtype=np.float32)
    elif dtype == 11:
        arr = np.asarray(doubles, dtype=np.float64)
    elif dtype == 7:
        arr = np.asarray(int64s, dtype=np.int64)
    elif dtype == 10:  # float16 travels as its bit pattern in int32_data
        arr = np.asarray(int32s, dtype=np.uint16).view(np.float16)
    else:
        arr = np.asarray(int32s).astype(np_dt)
    if arr.size != count:
        raise ValueError(f"ONNX tensor '{name}': {arr.size} values for shape {dims}")
    return name, arr.reshape(dims)


def _attribute(buf: bytes):
    name, out = "", {}
    for num, wt, val in _fields(buf):
        if num == 1:
            name = val.decode()
        elif num == 2:
            out["f"] = struct.unpack("<f", val)[0]
        elif num == 3:
            out["i"] = _sint64(val)
        elif num == 4:
            out["s"] = val
        elif num == 5:
            out["t"] = _tensor(val)[1]
        elif num == 7:
            out.setdefault("floats", []).extend(_packed_floats(val, wt))
        elif num == 8:
            out.setdefault("ints", []).extend(_packed_varints(val, wt))
        elif num == 20:
            out["type"] = val
    # AttributeProto.type names the member that carries the value (a zero or an empty list may
    # be left off the wire); files without it are read by whichever member is present
    by_type = {1: ("f", 0.0), 2: ("i", 0), 3: ("s", b""), 4: ("t", None), 6: ("floats", []), 7: ("ints", [])}
    if out.get("type") in by_type:
        key, default = by_type[out["type"]]
        return name, out.get(key, default)
    for key in ("f", "i", "s", "t", "floats", "ints"):
        if key in out:
            return name, out[key]
    return name, None


def _node(buf: bytes):
    node = {"input": [], "output": [], "name": "", "op_type": "", "attrs": {}}
    for num, _, val in _fields(buf):
        if num == 1:
            node["input"].append(val.decode())
        elif num == 2:
            node["output"].append(val.decode())
        elif num == 3:
            node["name"] = val.decode()
        elif num == 4:
            node["op_type"] = val.decode()
        elif num == 5:
            k, v = _attribute(val)
            node["attrs"][k] = v
    return node


def _value_name(buf: bytes) -> str:
    for num, _, val in _fields(buf):
        if num == 1:
            return val.decode()
    return ""


def read_onnx(source) -> dict:
    """Decode an ONNX ``ModelProto`` (a path or its bytes) into plain Python: ``nodes`` (dicts with
    input / output / op_type / attrs), ``initializers`` (name -> ndarray), ``inputs`` and ``outputs``
    (names; initializers listed as inputs, as old exporters do, are left out of ``inputs``)."""
    if isinstance(source, (bytes, bytearray, memoryview)):
        buf = bytes(source)
    else:
        with open(source, "rb") as f:
            buf = f.read()
    graph = None
    ir_version = 0
    for num, wt, val in _fields(buf):
        if num == 1 and wt == 0:
            ir_version = val
        elif num == 7 and wt == 2:
            graph = val
    if graph is None:
        raise ValueError("not an ONNX model: no graph")
    model = {"ir_version": ir_version, "nodes": [], "initializers": {}, "inputs": [], "outputs": []}
    for num, wt, val in _fields(graph):
        if wt != 2:
            continue
        if num == 1:
            model["nodes"].append(_node(val))
        elif num == 5:
            k, arr = _tensor(val)
            model["initializers"][k] = arr
        elif num == 11:
            model["inputs"].append(_value_name(val))
        elif num == 12:
            model["outputs"].append(_value_name(val))
    model["inputs"] = [n for n in model["inputs"] if n not in model["initializers"]]
    return model


# --------------------------------------------------------------------------------------------
# lowering
# --------------------------------------------------------------------------------------------
_LOWERED = {
    "Gemm": "nn.Linear", "MatMul": "nn.Linear", "Conv": "nn.Conv2d", "MaxPool": "nn.MaxPool2d",
    "Relu": "nn.ReLU", "LeakyRelu": "nn.LeakyReLU", "Sigmoid": "nn.Sigmoid", "Tanh": "nn.Tanh",
    "Gelu": "nn.GELU", "Flatten": "nn.Flatten", "GlobalAveragePool": "nn.GlobalAvgPool2d",
    "BatchNormalization": "nn.BatchNorm2d",
}
_PASS_THROUGH = {"Identity": "pass_through", "Constant": "constant"}


def onnx_native_conversion_map() -> dict:
    """Operator -> {"status", "munet"}: what the native lowering does with each ONNX operator
    (python/munet_nn/_helpers/onnx_integration.py:166-169 is the reference's table; operators its
    table assigns to the development-only graph interpreter are not listed here)."""
    out = {op: {"status": "lowered", "munet": layer} for op, layer in _LOWERED.items()}
    out.update({op: {"status": "pass_through", "munet": kind} for op, kind in _PASS_THROUGH.items()})
    return out


def _conversion_failures(model: dict) -> dict:
    counts = Counter(n["op_type"] for n in model["nodes"])
    bad = [op for op in sorted(counts) if op not in _LOWERED and op not in _PASS_THROUGH]
    return {"op_counts": dict(sorted(counts.items())), "unsupported_unique": bad,
            "unsupported_total": int(sum(counts[op] for op in bad))}


def report_onnx_unsupported_ops(source) -> list:
    """Sorted unique operators of the model that block the native conversion."""
    return _conversion_failures(read_onnx(source))["unsupported_unique"]


class _NotSequential(ValueError):
    pass


def _lower(model: dict):
    if len(model["inputs"]) != 1 or len(model["outputs"]) != 1:
        raise _NotSequential("the graph needs exactly one input and one output")
    consts = dict(model["initializers"])
    stream = model["inputs"][0]
    layers, tensors = [], {}

    def emit(cfg, **params):
        idx = len(layers)
        layers.append(cfg)
        for key, arr in params.items():
            if arr is not None:
                tensors[f"{idx}.{key}"] = np.ascontiguousarray(arr, dtype=np.float32)

    for node in model["nodes"]:
        op, attrs = node["op_type"], node["attrs"]
        if op == "Constant":
            if "value" in attrs and isinstance(attrs["value"], np.ndarray) and node["output"]:
                consts[node["output"][0]] = attrs["value"]
            continue
        if len(node["output"]) != 1:
            raise _NotSequential(f"op={op} has output arity={len(node['output'])}")
        if not node["input"] or node["input"][0] != stream:
            raise _NotSequential(f"op={op} is not a single-stream transform")

        def precondition(ok, what):
            if not ok:
                raise _NotSequential(f"op={op} failed lowering preconditions: {what}")

        if op == "Identity":
            pass
        elif op == "Gemm":
            w = consts.get(node["input"][1]) if len(node["input"]) > 1 else None
            precondition(w is not None and w.ndim == 2, "constant 2-D weight")
            precondition(attrs.get("transA", 0) == 0 and attrs.get("alpha", 1.0) == 1.0 and
                         attrs.get("beta", 1.0) == 1.0, "transA = 0, alpha = beta = 1")
            if attrs.get("transB", 0):
                w = w.T  # MuNet stores Linear weights [in, out]
            b = None
            if len(node["input"]) >= 3 and node["input"][2]:
                b = consts.get(node["input"][2])
                precondition(b is not None and b.size == w.shape[1], "constant bias of out_features values")
                b = b.reshape(w.shape[1])
            emit({"type": "Linear", "in_features": int(w.shape[0]), "out_features": int(w.shape[1]),
                  "bias": b is not None}, weight=w, bias=b)
        elif op == "MatMul":
            w = consts.get(node["input"][1]) if len(node["input"]) > 1 else None
            precondition(w is not None and w.ndim == 2, "constant 2-D right-hand side")
            emit({"type": "Linear", "in_features": int(w.shape[0]), "out_features": int(w.shape[1]),
                  "bias": False}, weight=w)
        elif op == "Conv":
            w = consts.get(node["input"][1]) if len(node["input"]) > 1 else None
            precondition(w is not None and w.ndim == 4 and w.shape[2] == w.shape[3], "constant square 2-D kernel")
            st = attrs.get("strides", [1, 1])
            pd = attrs.get("pads", [0, 0, 0, 0])
            precondition(attrs.get("group", 1) == 1 and all(d == 1 for d in attrs.get("dilations", [1, 1])),
                         "one group, unit dilation")
            precondition(len(st) == 2 and st[0] == st[1] and len(pd) == 4 and len(set(pd)) == 1,
                         "square stride, symmetric padding")
            precondition(attrs.get("auto_pad", b"NOTSET") in (b"NOTSET", b""), "explicit padding")
            b = np.zeros(w.shape[0], dtype=np.float32)  # nn::Conv2d always carries a bias
            if len(node["input"]) >= 3 and node["input"][2]:
                b = consts.get(node["input"][2])
                precondition(b is not None and b.size == w.shape[0], "constant bias of out_channels values")
                b = b.reshape(w.shape[0])
            emit({"type": "Conv2d", "in_channels": int(w.shape[1]), "out_channels": int(w.shape[0]),
                  "kernel_size": int(w.shape[2]), "stride": int(st[0]), "padding": int(pd[0])},
                 weight=w, bias=b)
        elif op == "MaxPool":
            ks = attrs.get("kernel_shape")
            precondition(ks is not None and len(ks) == 2 and ks[0] == ks[1], "square 2-D window")
            st = attrs.get("strides", ks)
            pd = attrs.get("pads", [0, 0, 0, 0])
            precondition(st[0] == st[1] and pd[0] == pd[2] and pd[1] == pd[3] and pd[0] == pd[1],
                         "square stride, symmetric padding")
            emit({"type": "MaxPool2d", "kernel_size": int(ks[0]), "stride": int(st[0]), "padding": int(pd[0])})
        elif op == "BatchNormalization":
            # inference form: y = (x - mean) / sqrt(var + eps) * scale + B over the channel axis
            ins = [consts.get(n) for n in node["input"][1:5]] if len(node["input"]) >= 5 else []
            precondition(len(ins) == 4 and all(t is not None and t.ndim == 1 and t.size == ins[0].size for t in ins),
                         "constant scale, B, mean and var of one length")
            precondition(attrs.get("training_mode", 0) == 0, "inference mode")
            emit({"type": "BatchNorm2d", "num_features": int(ins[0].size),
                  "eps": float(attrs.get("epsilon", 1e-5)), "momentum": float(attrs.get("momentum", 0.9))},
                 weight=ins[0], bias=ins[1], running_mean=ins[2], running_var=ins[3])
        elif op == "LeakyRelu":
            emit({"type": "LeakyReLU", "negative_slope": float(attrs.get("alpha", 0.01))})
        elif op == "Flatten":
            precondition(attrs.get("axis", 1) == 1, "axis 1")
            emit({"type": "Flatten"})
        elif op in ("Relu", "Sigmoid", "Tanh", "Gelu", "GlobalAveragePool"):
            emit({"type": {"Relu": "ReLU", "Sigmoid": "Sigmoid", "Tanh": "Tanh", "Gelu": "GELU",
                           "GlobalAveragePool": "GlobalAvgPool2d"}[op]})
        else:
            raise _NotSequential(f"unsupported op={op}")
        stream = node["output"][0]
    if stream != model["outputs"][0] or not layers:
        raise _NotSequential("the output stream does not end at the graph output")
    return {"type": "Sequential", "layers": layers}, tensors


def compile_onnx(source, output_path=None):
    """Strict conversion of an ONNX model to (config, tensors) for ``Engine.load``; with
    ``output_path`` the deploy artifact is written as well. Raises ``ValueError`` naming the
    operators that block the conversion (same wording as the reference) or the reason why the graph
    is not a single-stream chain. There is no interpreter to fall back to."""
    model = read_onnx(source)
    fail = _conversion_failures(model)
    if fail["unsupported_total"] > 0:
        raise ValueError("compile_onnx: conversion failed. "
                         f"model='{source if isinstance(source, str) else '<bytes>'}', "
                         f"unsupported_unique={fail['unsupported_unique']}, "
                         f"unsupported_total={fail['unsupported_total']}, "
                         f"op_counts={fail['op_counts']}")
    try:
        config, tensors = _lower(model)
    except _NotSequential as e:
        raise ValueError(f"compile_onnx: native sequential lowering skipped: {e}") from None
    if output_path is not None:
        from .inference import save_deploy
        save_deploy(output_path, config, tensors)
    return config, tensors
