"""Golden vectors: outputs of the unmodified reference on small seeded inputs, committed as
tests/golden/reference_outputs.npz (made by tests/golden/make_golden.py). They need neither the
reference checkout nor its built library.

CPU: the checker restatement (oracle/oracle.c) reproduces every vector bit for bit.
GPU: the kernels, through the C ABI, match them (float32 bit for bit where the kernel keeps the
reference's operation order, otherwise within the config tolerance)."""
import os

import numpy as np
import pytest

import oracle
from oracle import BF16, F32

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_outputs.npz"))
DT = {"f32": F32, "bf16": BF16}


def same(a, b):
    assert a.shape == b.shape and a.dtype == b.dtype, (a.shape, b.shape, a.dtype, b.dtype)
    assert np.array_equal(a.view(np.uint8), b.view(np.uint8))


def gpt_ps(tag):
    keys = sorted(k for k in G.files if k.startswith(f"gpt.{tag}.p"))
    return [G[k] for k in keys]


@pytest.mark.parametrize("tag", ["f32", "bf16"])
def test_checker_reproduces_reference_vectors(tag):
    P, dt = oracle.port(), DT[tag]
    x, w, b = G[f"linear.{tag}.x"], G[f"linear.{tag}.w"], G[f"linear.{tag}.b"]
    for act in ("none", "relu", "gelu", "sigmoid", "tanh"):
        same(P.linear(x, w, b, dt, act), G[f"linear.{tag}.{act}.y"])
    same(P.add(G[f"add.{tag}.a"], G[f"add.{tag}.b"], dt), G[f"add.{tag}.y"])
    z, g, bb = G[f"norm.{tag}.x"], G[f"norm.{tag}.g"], G[f"norm.{tag}.b"]
    same(P.layer_norm(z, g, bb, dt), G[f"norm.{tag}.layer_norm"])
    same(P.softmax(z, dt), G[f"norm.{tag}.softmax"])
    same(P.rms_norm(z, g, dt), G[f"norm.{tag}.rms_norm"])
    same(P.leaky_relu(z.reshape(-1), 0.1, dt), G[f"norm.{tag}.leaky_relu"])
    ps = [G[f"mha.{tag}.p{i}"] for i in range(8)]
    for causal in (0, 1):
        same(P.mha(G[f"mha.{tag}.x"], ps, 4, bool(causal), dt), G[f"mha.{tag}.causal{causal}.y"])
    same(P.gpt_forward(G[f"gpt.{tag}.ids"], gpt_ps(tag), 50, 32, 2, 2, dt), G[f"gpt.{tag}.logits"])


def test_checker_reproduces_reference_spatial_vectors():
    P = oracle.port()
    y = P.conv2d(G["conv.x"], G["conv.w"], G["conv.b"], 1, 1)
    same(y, G["conv.y"])
    same(P.max_pool2d(np.maximum(y, 0)), G["conv.pool"])
    same(P.global_avg_pool(y), G["conv.gap"])
    same(P.batch_norm_eval(y, G["bn.g"], G["bn.b"], G["bn.mean"], G["bn.var"], F32), G["bn.y"])


@pytest.mark.gpu
@pytest.mark.parametrize("tag", ["f32", "bf16"])
def test_kernels_match_reference_vectors(tag):
    import munet_b200 as mb
    from munet_b200.inference import Engine, gpt_decoder_config, gpt_param_names
    from tests.util import assert_close, empty_dev, to_dev, to_host
    ctx, dt = mb.Context(0), DT[tag]
    x, w, b = G[f"linear.{tag}.x"], G[f"linear.{tag}.w"], G[f"linear.{tag}.b"]
    for act in ("none", "relu", "gelu", "sigmoid", "tanh"):
        y = empty_dev((19, 24), dt)
        ctx.linear(to_dev(x, dt), to_dev(w, dt), to_dev(b, dt), y, 19, 40, 24, dt, act=act)
        ctx.check()
        want = G[f"linear.{tag}.{act}.y"]
        if dt == F32 and act in ("none", "relu"):
            same(to_host(y), want)
        else:
            assert_close(to_host(y), want, dt, what=f"linear {act}")
    z, g, bb = G[f"norm.{tag}.x"], G[f"norm.{tag}.g"], G[f"norm.{tag}.b"]
    for name, call in (("layer_norm", lambda o: ctx.layer_norm(to_dev(z, dt), to_dev(g, dt), to_dev(bb, dt), o, 13, 72, dt)),
                       ("softmax", lambda o: ctx.softmax(to_dev(z, dt), o, 13, 72, dt)),
                       ("rms_norm", lambda o: ctx.rms_norm(to_dev(z, dt), to_dev(g, dt), o, 13, 72, dt))):
        o = empty_dev((13, 72), dt)
        call(o)
        ctx.check()
        assert_close(to_host(o), G[f"norm.{tag}.{name}"], dt, what=name)
    # the whole decoder through the executor, literal K addressing like the reference
    V, d, H, L, T = 50, 32, 2, 2, 9
    eng = Engine(ctx=ctx, compute_dtype=dt, kmode=mb.K_LITERAL)
    eng.load(gpt_decoder_config(V, T, d, H, L), dict(zip(gpt_param_names(L), gpt_ps(tag))), tensor_dtype=dt)
    eng.compile((2, T), mb.I32)
    assert_close(eng.run(G[f"gpt.{tag}.ids"]), G[f"gpt.{tag}.logits"], dt, what="decoder logits")
    eng.close()
    ctx.close()


@pytest.mark.gpu
def test_spatial_kernels_match_reference_vectors():
    import munet_b200 as mb
    from tests.util import empty_dev, to_dev, to_host
    ctx = mb.Context(0)
    y = empty_dev((2, 5, 9, 8), F32)
    ctx.conv2d(to_dev(G["conv.x"], F32), to_dev(G["conv.w"], F32), to_dev(G["conv.b"], F32), y, 2, 3, 9, 8, 5,
               3, 1, 1, F32)
    ctx.check()
    same(to_host(y), G["conv.y"])
    p = empty_dev((2, 5, 4, 4), F32)
    ctx.conv2d(to_dev(G["conv.x"], F32), to_dev(G["conv.w"], F32), to_dev(G["conv.b"], F32), p, 2, 3, 9, 8, 5,
               3, 1, 1, F32, relu=True, pool=2)
    ctx.check()
    same(to_host(p), G["conv.pool"])
    o = empty_dev((2, 5, 9, 8), F32)
    ctx.batch_norm_eval(y, to_dev(G["bn.g"], F32), to_dev(G["bn.b"], F32), to_dev(G["bn.mean"], F32),
                        to_dev(G["bn.var"], F32), o, 2, 5, 9, 8, 1e-5, F32)
    ctx.check()
    same(to_host(o), G["bn.y"])
    ctx.close()
