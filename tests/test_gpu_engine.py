"""GPU parity of the compiled executor against the CPU checker: decoder forward
(bf16 2e-2, fp32 1e-4), MLP artifacts (fp32 logits bit-exact, argmax bit-exact),
the reference's own known-answer artifacts, shape-contract and error behaviour."""
import numpy as np
import pytest

import oracle
from oracle import BF16, F32, I32
from tests.test_oracle_vs_ref import gpt_params
from tests.util import assert_close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    import munet_b200 as mb
    c = mb.Context(0)
    yield c
    c.close()


def make_engine(ctx, dtype, **kw):
    from munet_b200.inference import Engine
    return Engine(ctx=ctx, compute_dtype=dtype, **kw)


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("kmode", [oracle.K_LITERAL, oracle.K_MATH])
@pytest.mark.parametrize("B,T,V,d,H,L", [(2, 32, 96, 64, 2, 2), (3, 24, 50, 48, 3, 1)])
def test_gpt_decoder_matches_checker(ctx, dtype, kmode, B, T, V, d, H, L):
    from munet_b200.inference import gpt_decoder_config, gpt_param_names
    rng = np.random.default_rng(B * T + d)
    ps = gpt_params(rng, V, T, d, L, dtype, std=0.08)
    ids = rng.integers(0, V, (B, T)).astype(np.int32)
    want = oracle.port().gpt_forward(ids, ps, V, d, H, L, dtype, kmode=kmode)
    eng = make_engine(ctx, dtype, kmode=kmode, argmax=True)
    eng.load(gpt_decoder_config(V, T, d, H, L), dict(zip(gpt_param_names(L), ps)), tensor_dtype=dtype)
    eng.compile((B, T), I32)
    got, am = eng.run(ids)
    assert got.shape == (B, T, V)
    assert_close(got, want, dtype, what="decoder logits")
    # argmax is computed on the device from the device logits: first-max rule
    assert np.array_equal(am, oracle.port().argmax(got, dtype))
    agree = float((am == oracle.port().argmax(want, dtype)).mean())
    assert agree >= (0.999 if dtype == F32 else 0.9), f"argmax agreement {agree}"
    st = eng.stats()
    assert st["arena_bytes"] < st["unplanned_bytes"]  # the buffer plan reuses memory
    eng.close()


def mlp_artifact(tmp_path, rng, sizes, acts, name="mlp.npz", producer="munet"):
    from munet_b200.inference import save_deploy
    layers, tensors, idx = [], {}, 0
    for i in range(len(sizes) - 1):
        layers.append({"type": "Linear", "in_features": sizes[i], "out_features": sizes[i + 1], "bias": True})
        tensors[f"{idx}.weight"] = (rng.standard_normal((sizes[i], sizes[i + 1])) *
                                    np.sqrt(2.0 / sizes[i])).astype(np.float32)
        tensors[f"{idx}.bias"] = np.zeros(sizes[i + 1], np.float32)
        idx += 1
        if i < len(acts) and acts[i]:
            layers.append({"type": acts[i]})
            idx += 1
    path = str(tmp_path / name)
    save_deploy(path, {"type": "Sequential", "layers": layers}, tensors, producer=producer)
    return path, tensors


def mlp_oracle(x, tensors, acts):
    h, idx = x, 0
    for i in range(len(acts) + 1):
        a = acts[i] if i < len(acts) and acts[i] else None
        h = oracle.port().linear(h, tensors[f"{idx}.weight"], tensors[f"{idx}.bias"], F32,
                                 {"ReLU": "relu", "GELU": "gelu", None: "none"}[a])
        idx += 2 if a else 1
    return h


@pytest.mark.parametrize("kmode,V,d,H,L,B,T", [(oracle.K_LITERAL, 1024, 1024, 8, 2, 4, 512),
                                               (oracle.K_MATH, 512, 512, 8, 2, 8, 256)])
def test_repeated_forwards_are_bit_identical(ctx, kmode, V, d, H, L, B, T):
    """No kernel on the path uses atomics or an order that depends on timing: the same input gives
    the same bits every time, also with other traffic going through L2 and HBM in between (a race
    in a barrier hand-over of the GEMM or attention pipelines would show up here)."""
    import torch
    from munet_b200.inference import gpt_decoder_config, gpt_param_names
    rng = np.random.default_rng(21)
    ps = gpt_params(rng, V, T, d, L, BF16, std=0.03)
    ids = rng.integers(0, V, (B, T)).astype(np.int32)
    eng = make_engine(ctx, BF16, kmode=kmode)
    eng.load(gpt_decoder_config(V, T, d, H, L), dict(zip(gpt_param_names(L), ps)), tensor_dtype=BF16)
    eng.compile((B, T), I32)
    first = eng.run(ids).copy()
    junk = torch.empty(192 << 20, device="cuda", dtype=torch.uint8)
    for it in range(40):
        if it % 3 == 0:
            junk.add_(1)
        assert np.array_equal(eng.run(ids), first), f"forward {it} differs from the first"
    eng.close()


def test_mlp_config_fp32_bit_exact(ctx, tmp_path):
    """784→512→ReLU→512→ReLU→10, batch 256: logits and argmax identical to the reference."""
    rng = np.random.default_rng(1001)
    path, tensors = mlp_artifact(tmp_path, rng, [784, 512, 512, 10], ["ReLU", "ReLU"])
    x = np.random.default_rng(2001).random((256, 784), dtype=np.float32)
    want = mlp_oracle(x, tensors, ["ReLU", "ReLU"])
    eng = make_engine(ctx, F32, argmax=True).load(path).compile((256, 784))
    got, am = eng.run(x)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    assert np.array_equal(am, oracle.port().argmax(want, F32))
    if oracle.have_ref():
        ref = oracle.ref().engine_run_npz(path, x)
        assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))
    eng.close()


def test_reference_known_answers(ctx, tmp_path):
    """Artifacts with the values of the reference's own engine tests
    (tests/test_inference.cpp:887-919 and :990-1022)."""
    from munet_b200.inference import save_deploy
    p1 = str(tmp_path / "kat1.npz")
    save_deploy(p1, {"type": "Sequential", "layers": [
        {"type": "Linear", "in_features": 2, "out_features": 2, "bias": True}, {"type": "ReLU"}]},
        {"0.weight": np.array([[1, -1], [0.5, 2]], np.float32), "0.bias": np.array([0.25, -0.75], np.float32)})
    eng = make_engine(ctx, F32).load(p1).compile((1, 2))
    assert np.array_equal(eng.run(np.array([[2, 3]], np.float32)), np.array([[3.75, 3.25]], np.float32))
    eng.close()
    p2 = str(tmp_path / "kat2.npz")
    save_deploy(p2, {"type": "Linear", "in_features": 2, "out_features": 2, "bias": True},
                {"weight": np.array([[2, 0], [0, 3]], np.float32), "bias": np.array([1, -2], np.float32)},
                producer="munet_nn")
    eng = make_engine(ctx, F32).load(p2).compile((1, 2))
    assert np.array_equal(eng.run(np.array([[4, 5]], np.float32)), np.array([[9, 13]], np.float32))
    eng.close()
    # Dropout is the identity in eval mode (tests/test_inference.cpp:921-939,1024-1060)
    p3 = str(tmp_path / "kat3.npz")
    save_deploy(p3, {"type": "Sequential", "layers": [
        {"type": "Dropout", "p": 0.9}, {"type": "Linear", "in_features": 2, "out_features": 2, "bias": True}]},
        {"1.weight": np.eye(2, dtype=np.float32), "1.bias": np.zeros(2, np.float32)})
    eng = make_engine(ctx, F32).load(p3).compile((1, 2))
    assert np.array_equal(eng.run(np.array([[7, 11]], np.float32)), np.array([[7, 11]], np.float32))
    eng.close()


def test_contract_and_errors(ctx, tmp_path):
    import munet_b200 as mb
    from munet_b200.inference import save_deploy
    rng = np.random.default_rng(0)
    path, _ = mlp_artifact(tmp_path, rng, [8, 4], [])
    eng = make_engine(ctx, F32).load(path)
    with pytest.raises(mb.MuNetError, match="before compile"):
        eng.run(np.zeros((2, 8), np.float32))
    eng.compile((2, 8))
    with pytest.raises(mb.MuNetError, match="shape"):  # strict shape contract (tests/test_inference.cpp:402-438)
        eng.run(np.zeros((3, 8), np.float32))
    eng.close()
    bad = str(tmp_path / "custom.npz")  # unknown node type must be rejected (tests/test_inference.cpp:974-988)
    save_deploy(bad, {"type": "__custom__"}, {})
    eng = make_engine(ctx, F32).load(bad)
    with pytest.raises(mb.MuNetError, match="Unsupported serialized module type"):
        eng.compile((1, 2))
    eng.close()
    with pytest.raises(mb.MuNetError, match="Unable to open"):
        make_engine(ctx, F32).load(str(tmp_path / "missing.npz"))
    # a payload tensor no module of the tree claims (src/inference_serialization.cpp:1043-1051)
    extra = str(tmp_path / "extra.npz")
    save_deploy(extra, {"type": "Linear", "in_features": 2, "out_features": 2, "bias": False},
                {"weight": np.eye(2, dtype=np.float32), "bias": np.zeros(2, np.float32)})
    eng = make_engine(ctx, F32).load(extra)
    with pytest.raises(mb.MuNetError, match="'bias' does not match any named parameter"):
        eng.compile((1, 2))
    eng.close()


def test_prepared_inputs_stats_and_observer(ctx, tmp_path):
    """Engine::prepare_batch / run_batch_into / EngineStats / observer (src/inference.hpp:43-92,
    368-382, 612-637): a prepared, unchanged host input is served from its device copy, an input
    changed in place is not, and the counters and events say so."""
    import torch
    import munet_b200 as mb
    rng = np.random.default_rng(3)
    path, tensors = mlp_artifact(tmp_path, rng, [8, 16, 4], ["ReLU"])
    events = []
    eng = make_engine(ctx, F32)
    eng.set_observer(events.append)
    eng.load(path).compile((5, 8))
    xs = [torch.from_numpy(rng.standard_normal((5, 8)).astype(np.float32)) for _ in range(3)]
    want = [mlp_oracle(x.numpy(), tensors, ["ReLU"]) for x in xs]
    eng.prepare_batch(xs)
    st = eng.engine_stats
    assert st["prepared_input_cache_entries"] == 3 and st["prepared_input_cache_misses"] == 3
    assert st["prepared_input_cache_bytes"] == 3 * 5 * 8 * 4
    outs = []
    eng.run_batch_into(xs, outs)
    for o, w in zip(outs, want):
        assert np.array_equal(o, w)
    st = eng.engine_stats
    assert st["prepared_input_cache_hits"] == 3 and st["runs"] == 3
    assert st["compiled_input_shape"] == [5, 8] and st["compiled_output_shape"] == [5, 4]
    xs[0].mul_(2.0)  # in-place change: the cached copy is stale and must not be used
    assert np.array_equal(eng.run(xs[0]), mlp_oracle(xs[0].numpy(), tensors, ["ReLU"]))
    assert eng.engine_stats["prepared_input_cache_hits"] == 3
    eng.set_prepared_input_cache_entries(1)  # reconfiguring drops the entries
    eng.prepare_batch(xs)
    st = eng.engine_stats
    assert st["prepared_input_cache_entries"] == 1 and st["prepared_input_cache_evictions"] == 2
    kinds = [e["type"] for e in events]
    assert kinds[:2] == ["load_completed", "compile_completed"] and kinds.count("run_completed") == 4
    with pytest.raises(mb.MuNetError):
        eng.run(np.zeros((4, 8), np.float32))
    assert events[-1]["type"] == "error"
    eng.close()


def test_wildcard_shape_contract_builds_one_plan_per_shape(ctx, tmp_path):
    """Engine::compile(example, {-1, 8}) (tests/test_inference.cpp:402-438): the batch extent may
    vary from run to run, the feature extent may not. Every new concrete shape gets its own plan
    (arena + graph) over the shared weights; a shape seen before reuses its plan; the number of
    plans kept is bounded."""
    import munet_b200 as mb
    rng = np.random.default_rng(21)
    path, tensors = mlp_artifact(tmp_path, rng, [8, 16, 4], ["ReLU"])
    eng = make_engine(ctx, F32).load(path)
    with pytest.raises(mb.MuNetError, match="dim mismatch at index 1"):
        eng.compile((1, 8), expected_input_shape=(-1, 9))      # the example itself must fit
    with pytest.raises(mb.MuNetError, match="output shape mismatch"):
        eng.compile((1, 8), expected_input_shape=(-1, 8), expected_output_shape=(-1, 5))
    eng.compile((1, 8), expected_input_shape=(-1, 8), expected_output_shape=(-1, 4))
    assert eng.plan_count == 1
    for batch in (4, 1, 7, 4):
        x = rng.standard_normal((batch, 8)).astype(np.float32)
        got = eng.run(x)
        assert got.shape == (batch, 4)
        assert np.array_equal(got, mlp_oracle(x, tensors, ["ReLU"]))
    assert eng.plan_count == 3                                    # shapes 1, 4 and 7
    with pytest.raises(mb.MuNetError, match="dim mismatch at index 1"):
        eng.run(np.zeros((4, 9), np.float32))
    with pytest.raises(mb.MuNetError, match="rank mismatch"):
        eng.run(np.zeros((4, 8, 1), np.float32))
    eng._opt("plan_cache_entries", 2)
    for batch in (2, 3, 5):
        x = rng.standard_normal((batch, 8)).astype(np.float32)
        assert np.array_equal(eng.run(x), mlp_oracle(x, tensors, ["ReLU"]))
    assert eng.plan_count <= 2
    x = rng.standard_normal((1, 8)).astype(np.float32)            # an evicted shape is rebuilt
    assert np.array_equal(eng.run(x), mlp_oracle(x, tensors, ["ReLU"]))
    # strict_shape_check off: the reference forwards any shape (tests/test_inference.cpp:402-419)
    eng2 = make_engine(ctx, F32).load(path).compile((2, 8))
    with pytest.raises(mb.MuNetError, match="dim mismatch at index 0"):
        eng2.run(np.zeros((3, 8), np.float32))
    eng2.set_strict_shape_check(False)
    x = rng.standard_normal((3, 8)).astype(np.float32)
    assert np.array_equal(eng2.run(x), mlp_oracle(x, tensors, ["ReLU"]))
    eng.close()
    eng2.close()


def test_lean_mode_and_memory_capture(ctx, tmp_path):
    """Engine::set_lean_mode / set_capture_profiler_memory (src/inference.hpp:323-341): each one
    switches the other off; memory figures appear in the stats only while capture is on; the load
    event carries the tensor census only outside lean mode."""
    rng = np.random.default_rng(22)
    path, tensors = mlp_artifact(tmp_path, rng, [8, 4], [])
    events = []
    eng = make_engine(ctx, F32)
    eng.set_observer(events.append)
    eng.set_capture_profiler_memory(True)
    assert eng.capture_profiler_memory and not eng.lean_mode
    eng.load({"type": "Linear", "in_features": 8, "out_features": 4, "bias": True},
             {"weight": tensors["0.weight"], "bias": tensors["0.bias"]})
    assert "2 parameter/buffer tensor(s)" in events[-1]["message"]
    eng.compile((3, 8))
    x = rng.standard_normal((3, 8)).astype(np.float32)
    eng.run(x)
    st = eng.engine_stats
    assert st["current_memory_bytes"] > 0 and st["peak_memory_bytes"] >= st["current_memory_bytes"]
    eng.set_lean_mode(True)
    assert eng.lean_mode and not eng.capture_profiler_memory
    eng.load({"type": "Linear", "in_features": 8, "out_features": 4, "bias": True},
             {"weight": tensors["0.weight"], "bias": tensors["0.bias"]})
    assert "tensor(s)" not in events[-1]["message"] and "gradients will remain disabled" in events[-1]["message"]
    eng.compile((3, 8))
    want = oracle.port().linear(x, tensors["0.weight"], tensors["0.bias"], F32)
    assert np.array_equal(eng.run(x), want)
    eng.close()


def test_prepared_input_is_converted_like_a_plain_run(ctx):
    """prepare_batch + run must give what a plain run gives for inputs whose dtype is not the
    compiled one: torch.randint's int64 ids and a float64 array."""
    import torch
    import munet_b200 as mb
    from munet_b200.inference import gpt_decoder_config, gpt_param_names
    B, T, V, d, H, L = 2, 16, 50, 32, 2, 1
    rng = np.random.default_rng(23)
    ps = gpt_params(rng, V, T, d, L, F32, std=0.08)
    eng = make_engine(ctx, F32, kmode=oracle.K_MATH)
    eng.load(gpt_decoder_config(V, T, d, H, L), dict(zip(gpt_param_names(L), ps)))
    eng.compile((B, T), I32)
    ids64 = torch.randint(0, V, (B, T))                       # int64
    plain = eng.run(ids64.numpy().astype(np.int32))
    eng.prepare_batch([ids64])
    assert eng.engine_stats["prepared_input_cache_entries"] == 1
    assert np.array_equal(eng.run(ids64), plain)
    assert eng.engine_stats["prepared_input_cache_hits"] == 1
    with pytest.raises(mb.MuNetError, match="dtype"):          # a device tensor is taken as raw bytes
        eng.run(ids64.cuda())
    assert eng.run(ids64.to(torch.int32).cuda()) is None       # result stays in the arena
    eng.close()


@pytest.mark.parametrize("kmode", [oracle.K_LITERAL, oracle.K_MATH])
def test_float32_artifact_runs_in_bfloat16(ctx, tmp_path, kmode):
    """Module::to(BFloat16) on load (src/core/module.hpp:177-194, Tensor::to src/tensor.cpp:249-284):
    an artifact of float32 tensors loaded with compute_dtype = bfloat16 must behave like the
    checker fed with the same tensors rounded to bf16 by the reference's rule (RNE, +0x7fff+lsb)."""
    from munet_b200.inference import gpt_decoder_config, gpt_param_names, save_deploy
    B, T, V, d, H, L = 2, 32, 96, 64, 2, 2
    rng = np.random.default_rng(24)
    ps32 = gpt_params(rng, V, T, d, L, F32, std=0.08)
    # values that sit exactly between two bf16 numbers exercise round-to-nearest-even
    ps32[0].reshape(-1)[:4] = np.array([1.00390625, 1.01171875, -1.00390625, 3.0e-39], np.float32)
    names = gpt_param_names(L)
    path = str(tmp_path / "decoder_f32.npz")
    save_deploy(path, gpt_decoder_config(V, T, d, H, L), dict(zip(names, ps32)))
    ids = rng.integers(0, V, (B, T)).astype(np.int32)
    ids[0, 0] = 0  # the row with the tie values is looked up
    want = oracle.port().gpt_forward(ids, [oracle.to_bf16(p) for p in ps32], V, d, H, L, BF16, kmode=kmode)
    for source in ("artifact", "memory"):
        eng = make_engine(ctx, BF16, kmode=kmode)
        if source == "artifact":
            eng.load(path)
        else:
            eng.load(gpt_decoder_config(V, T, d, H, L), dict(zip(names, ps32)))
        eng.compile((B, T), I32)
        assert_close(eng.run(ids), want, BF16, what=f"fp32 {source} in bf16")
        eng.close()


def test_inference_baseline_report(tmp_path):
    """The replay of the reference's benchmark protocol (tools/inference_baseline.cpp:348-428)
    runs and prints a report with the reference's sections and keys."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for dtype, lean in (("float32", "0"), ("bfloat16", "1")):
        r = subprocess.run([sys.executable, "-m", "munet_b200.inference_baseline", "--dtype", dtype,
                            "--single-run-iters", "5", "--batch-run-iters", "2", "--warmup-runs", "1",
                            "--preallocate-batch-inputs", "1", "--lean-mode", lean],
                           cwd=root, capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, r.stderr
        rep = json.loads(r.stdout)
        for section in ("memory_policy", "shape_contract", "cold_load", "compile", "steady_single_run",
                        "steady_batch_run", "memory_bytes"):
            assert section in rep
        assert rep["lean_mode"] == (lean == "1") and rep["dtype"] == dtype
        assert rep["shape_contract"]["compiled_input_shape"] == [32, 256]
        assert rep["shape_contract"]["compiled_output_shape"] == [32, 128]
        assert rep["steady_single_run"]["avg_wall_ms"] > 0 and rep["steady_batch_run"]["avg_per_input_wall_ms"] > 0
        assert rep["memory_bytes"]["prepared_input_cache_hits"] >= 2 * 4  # prepared inputs were reused
