"""ONNX -> deploy artifact (munet_b200/onnx_import.py).

Known answers are the ones of the reference's own ONNX tests (tests/test_python.py:1239-1361: a
Gemm + Relu model and a Conv + LeakyRelu + GlobalAveragePool model with their expected outputs).
The artifacts written by compile_onnx are run by the unmodified reference engine on the CPU, and
on a GPU by this package's engine."""
import os

import numpy as np
import pytest

import oracle
from munet_b200 import onnx_import as oi
from tests import onnx_fixture as ox

W = np.array([[1.0, 0.0], [0.0, 2.0], [1.0, 1.0]], dtype=np.float32)
B = np.array([0.5, -1.0], dtype=np.float32)
X = np.array([[1.0, 2.0, 3.0], [-1.0, 0.5, 2.0]], dtype=np.float32)


def gemm_relu(trans_b=0, raw=False, as_inputs=False):
    w = W.T.copy() if trans_b else W
    return ox.model([ox.node("Gemm", ["x", "W", "B"], ["z"], transB=trans_b), ox.node("Relu", ["z"], ["y"])],
                    [ox.value_info("x", [None, 3])], [ox.value_info("y", [None, 2])],
                    [ox.tensor("W", w, raw=raw), ox.tensor("B", B, raw=raw)],
                    list_initializers_as_inputs=as_inputs)


def conv_lrelu_gap():
    return ox.model([ox.node("Conv", ["x", "W", "B"], ["z"]), ox.node("LeakyRelu", ["z"], ["a"], alpha=0.1),
                     ox.node("GlobalAveragePool", ["a"], ["y"])],
                    [ox.value_info("x", [1, 1, 2, 2])], [ox.value_info("y", [1, 1, 1, 1])],
                    [ox.tensor("W", np.array([[[[1.0]]]], dtype=np.float32)),
                     ox.tensor("B", np.array([0.0], dtype=np.float32))])


@pytest.mark.parametrize("trans_b,raw,as_inputs", [(0, False, False), (1, False, False), (0, True, True)])
def test_gemm_relu_lowers_to_linear_relu(trans_b, raw, as_inputs):
    cfg, tensors = oi.compile_onnx(gemm_relu(trans_b, raw, as_inputs))
    assert cfg == {"type": "Sequential", "layers": [
        {"type": "Linear", "in_features": 3, "out_features": 2, "bias": True}, {"type": "ReLU"}]}
    assert np.array_equal(tensors["0.weight"], W) and np.array_equal(tensors["0.bias"], B)


def test_reader_sees_nodes_attributes_and_initializers():
    m = oi.read_onnx(ox.model(
        [ox.node("MaxPool", ["x"], ["p"], kernel_shape=[2, 2], strides=[2, 2], pads=[0, 0, 0, 0]),
         ox.node("Constant", [], ["c"], value=np.arange(6, dtype=np.float32).reshape(2, 3)),
         ox.node("LeakyRelu", ["p"], ["y"], alpha=0.25)],
        [ox.value_info("x", [1, 1, 4, 4])], [ox.value_info("y", [1, 1, 2, 2])],
        [ox.tensor("idx", np.array([3, -1, 2 ** 40], dtype=np.int64))]))
    assert [n["op_type"] for n in m["nodes"]] == ["MaxPool", "Constant", "LeakyRelu"]
    assert m["nodes"][0]["attrs"] == {"kernel_shape": [2, 2], "strides": [2, 2], "pads": [0, 0, 0, 0]}
    assert m["nodes"][2]["attrs"]["alpha"] == np.float32(0.25)
    assert np.array_equal(m["nodes"][1]["attrs"]["value"], np.arange(6, dtype=np.float32).reshape(2, 3))
    assert m["initializers"]["idx"].tolist() == [3, -1, 2 ** 40]
    assert m["inputs"] == ["x"] and m["outputs"] == ["y"] and m["ir_version"] == 7


def test_constant_node_feeds_a_matmul():
    data = ox.model([ox.node("Constant", [], ["w"], value=W), ox.node("MatMul", ["x", "w"], ["y"])],
                    [ox.value_info("x", [None, 3])], [ox.value_info("y", [None, 2])], [])
    cfg, tensors = oi.compile_onnx(data)
    assert cfg["layers"] == [{"type": "Linear", "in_features": 3, "out_features": 2, "bias": False}]
    assert np.array_equal(tensors["0.weight"], W) and "0.bias" not in tensors


def test_conv_without_bias_gets_the_zero_bias_the_module_needs():
    w = np.arange(2 * 1 * 3 * 3, dtype=np.float32).reshape(2, 1, 3, 3)
    data = ox.model([ox.node("Conv", ["x", "w"], ["y"], kernel_shape=[3, 3], pads=[1, 1, 1, 1], strides=[2, 2])],
                    [ox.value_info("x", [1, 1, 8, 8])], [ox.value_info("y", [1, 2, 4, 4])], [ox.tensor("w", w)])
    cfg, tensors = oi.compile_onnx(data)
    assert cfg["layers"] == [{"type": "Conv2d", "in_channels": 1, "out_channels": 2, "kernel_size": 3,
                              "stride": 2, "padding": 1}]
    assert np.array_equal(tensors["0.weight"], w) and np.array_equal(tensors["0.bias"], np.zeros(2, np.float32))
    lopsided = ox.model([ox.node("Conv", ["x", "w"], ["y"], pads=[0, 1, 0, 1])],
                        [ox.value_info("x", [1, 1, 8, 8])], [ox.value_info("y", [1, 2, 6, 8])], [ox.tensor("w", w)])
    with pytest.raises(ValueError, match="symmetric padding"):
        oi.compile_onnx(lopsided)


def _conv_bn_relu():
    rng = np.random.default_rng(8)
    w = (rng.standard_normal((3, 2, 3, 3)) * 0.4).astype(np.float32)
    scale, shift, mean = (rng.standard_normal(3).astype(np.float32) for _ in range(3))
    var = (rng.random(3) + 0.5).astype(np.float32)
    data = ox.model([ox.node("Conv", ["x", "w"], ["c"], kernel_shape=[3, 3], pads=[1, 1, 1, 1]),
                     ox.node("BatchNormalization", ["c", "s", "b", "m", "v"], ["n"], epsilon=1e-3),
                     ox.node("Relu", ["n"], ["y"])],
                    [ox.value_info("x", [2, 2, 6, 6])], [ox.value_info("y", [2, 3, 6, 6])],
                    [ox.tensor("w", w), ox.tensor("s", scale), ox.tensor("b", shift), ox.tensor("m", mean),
                     ox.tensor("v", var)])
    x = rng.standard_normal((2, 2, 6, 6)).astype(np.float32)
    xp = np.pad(x, ((0, 0), (0, 0), (1, 1), (1, 1))).astype(np.float64)
    conv = np.zeros((2, 3, 6, 6))
    for kh in range(3):
        for kw in range(3):
            conv += np.einsum("bihw,oi->bohw", xp[:, :, kh:kh + 6, kw:kw + 6], w[:, :, kh, kw])
    c = lambda t: t[None, :, None, None].astype(np.float64)
    want = np.maximum((conv - c(mean)) / np.sqrt(c(var) + 1e-3) * c(scale) + c(shift), 0.0)
    return data, x, want


def test_batch_normalization_lowers_to_batchnorm2d(tmp_path):
    data, x, want = _conv_bn_relu()
    cfg, tensors = oi.compile_onnx(data)
    assert [l["type"] for l in cfg["layers"]] == ["Conv2d", "BatchNorm2d", "ReLU"]
    assert cfg["layers"][1]["num_features"] == 3 and abs(cfg["layers"][1]["eps"] - 1e-3) < 1e-9
    assert sorted(k for k in tensors if k.startswith("1.")) == ["1.bias", "1.running_mean", "1.running_var",
                                                                "1.weight"]
    if oracle.have_ref():  # the reference's own engine agrees with the formula
        path = str(tmp_path / "conv_bn_relu.npz")
        oi.compile_onnx(data, output_path=path)
        assert np.allclose(oracle.ref().engine_run_npz(path, x), want, rtol=1e-4, atol=1e-5)


def test_unsupported_ops_are_reported_like_the_reference():
    data = ox.model([ox.node("Relu", ["x"], ["a"]), ox.node("NonMaxSuppression", ["a"], ["b"]),
                     ox.node("Loop", ["b"], ["y"])],
                    [ox.value_info("x", [1, 4])], [ox.value_info("y", [1, 4])], [])
    assert oi.report_onnx_unsupported_ops(data) == ["Loop", "NonMaxSuppression"]
    with pytest.raises(ValueError, match=r"compile_onnx: conversion failed\. .*unsupported_unique=\['Loop', "
                                         r"'NonMaxSuppression'\], unsupported_total=2, op_counts="):
        oi.compile_onnx(data)
    assert oi.report_onnx_unsupported_ops(gemm_relu()) == []


def test_graphs_that_are_not_one_chain_are_refused():
    two_streams = ox.model([ox.node("Relu", ["x"], ["a"]), ox.node("Sigmoid", ["x"], ["y"])],
                           [ox.value_info("x", [1, 4])], [ox.value_info("y", [1, 4])], [])
    with pytest.raises(ValueError, match="not a single-stream transform"):
        oi.compile_onnx(two_streams)
    scaled = ox.model([ox.node("Gemm", ["x", "W"], ["y"], alpha=2.0)],
                      [ox.value_info("x", [None, 3])], [ox.value_info("y", [None, 2])], [ox.tensor("W", W)])
    with pytest.raises(ValueError, match="failed lowering preconditions"):
        oi.compile_onnx(scaled)
    dangling = ox.model([ox.node("Relu", ["x"], ["a"])], [ox.value_info("x", [1, 4])],
                        [ox.value_info("y", [1, 4])], [])
    with pytest.raises(ValueError, match="does not end at the graph output"):
        oi.compile_onnx(dangling)


def test_truncated_files_are_rejected_not_misread():
    data = gemm_relu()
    for cut in (1, len(data) // 3, len(data) - 5):
        with pytest.raises(ValueError):
            oi.compile_onnx(data[:cut])
    with pytest.raises(ValueError, match="no graph"):
        oi.read_onnx(b"")


def test_conversion_map_names_every_lowered_operator():
    mp = oi.onnx_native_conversion_map()
    for op in ("Gemm", "MatMul", "Conv", "MaxPool", "Relu", "LeakyRelu", "Sigmoid", "Tanh", "Gelu", "Flatten",
               "GlobalAveragePool"):
        assert mp[op]["status"] == "lowered"
    assert mp["Identity"]["status"] == "pass_through"
    assert mp["Gemm"]["munet"] == "nn.Linear" and mp["GlobalAveragePool"]["munet"] == "nn.GlobalAvgPool2d"


@pytest.mark.skipif(not oracle.have_ref(), reason="the compiled reference core is not present")
def test_artifacts_run_on_the_unmodified_reference_engine(tmp_path):
    """compile_onnx(output_path=...) writes a deploy artifact; the reference's own Engine (CPU)
    loads it and returns the values the reference's ONNX tests expect."""
    p1 = str(tmp_path / "linear_relu.npz")
    oi.compile_onnx(gemm_relu(), output_path=p1)
    y = oracle.ref().engine_run_npz(p1, X)
    assert np.allclose(y, np.maximum(X @ W + B, 0.0), atol=1e-5)
    p2 = str(tmp_path / "conv_lrelu_gap.npz")
    oi.compile_onnx(conv_lrelu_gap(), output_path=p2)
    x = np.array([[[[-1.0, 3.0], [2.0, -4.0]]]], dtype=np.float32)
    y = oracle.ref().engine_run_npz(p2, x)
    assert np.allclose(y.reshape(-1), [(-0.1 + 3.0 + 2.0 - 0.4) / 4.0], atol=1e-5)


@pytest.mark.gpu
def test_imported_models_run_on_the_b200_engine():
    import munet_b200 as mb
    from munet_b200.inference import Engine
    eng = Engine(compute_dtype=mb.F32)
    eng.load(*oi.compile_onnx(gemm_relu(trans_b=1)))
    eng.compile(X.shape)
    assert np.allclose(eng.run(X), np.maximum(X @ W + B, 0.0), atol=1e-5)
    eng.close()
    x = np.array([[[[-1.0, 3.0], [2.0, -4.0]]]], dtype=np.float32)
    eng = Engine(compute_dtype=mb.F32)
    eng.load(*oi.compile_onnx(conv_lrelu_gap()))
    eng.compile(x.shape)
    assert np.allclose(np.asarray(eng.run(x)).reshape(-1), [(-0.1 + 3.0 + 2.0 - 0.4) / 4.0], atol=1e-5)
    eng.close()
    # a small CNN chain: Conv -> Relu -> MaxPool -> Flatten -> Gemm against a numpy evaluation
    rng = np.random.default_rng(3)
    cw = rng.standard_normal((4, 2, 3, 3)).astype(np.float32) * 0.3
    cb = rng.standard_normal(4).astype(np.float32)
    fw = rng.standard_normal((4 * 4 * 4, 5)).astype(np.float32) * 0.1
    data = ox.model([ox.node("Conv", ["x", "cw", "cb"], ["c"], kernel_shape=[3, 3], pads=[1, 1, 1, 1], strides=[1, 1]),
                     ox.node("Relu", ["c"], ["r"]),
                     ox.node("MaxPool", ["r"], ["p"], kernel_shape=[2, 2], strides=[2, 2]),
                     ox.node("Flatten", ["p"], ["f"], axis=1), ox.node("MatMul", ["f", "fw"], ["y"])],
                    [ox.value_info("x", [3, 2, 8, 8])], [ox.value_info("y", [3, 5])],
                    [ox.tensor("cw", cw, raw=True), ox.tensor("cb", cb), ox.tensor("fw", fw, raw=True)])
    xin = rng.standard_normal((3, 2, 8, 8)).astype(np.float32)
    eng = Engine(compute_dtype=mb.F32)
    eng.load(*oi.compile_onnx(data))
    eng.compile(xin.shape)
    got = np.asarray(eng.run(xin))
    xp = np.pad(xin, ((0, 0), (0, 0), (1, 1), (1, 1)))
    conv = np.zeros((3, 4, 8, 8), dtype=np.float64)
    for kh in range(3):
        for kw in range(3):
            conv += np.einsum("bihw,oi->bohw", xp[:, :, kh:kh + 8, kw:kw + 8].astype(np.float64), cw[:, :, kh, kw])
    conv = np.maximum(conv + cb[None, :, None, None], 0.0)
    pooled = conv.reshape(3, 4, 4, 2, 4, 2).max(axis=(3, 5))
    want = pooled.reshape(3, -1) @ fw
    assert np.allclose(got, want, rtol=1e-4, atol=1e-4)
    eng.close()
    data, xin, want = _conv_bn_relu()
    eng = Engine(compute_dtype=mb.F32)
    eng.load(*oi.compile_onnx(data))
    eng.compile(xin.shape)
    assert np.allclose(np.asarray(eng.run(xin)), want, rtol=1e-4, atol=1e-5)
    eng.close()
