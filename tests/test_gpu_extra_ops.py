"""GPU: the remaining forward entry points of the Backend surface (unary math, LeakyReLU,
broadcast_row, concat, upsample2d, batch_norm eval, RMSNorm, reductions, fill_uniform) against
the CPU checker (arithmetic) or numpy (pure data movement)."""
import numpy as np
import pytest

import oracle
from oracle import BF16, F32
from tests.util import assert_close, empty_dev, rnd, to_dev, to_host

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    import munet_b200 as mb
    c = mb.Context(0)
    yield c
    c.close()


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("op", ["exp", "log", "sqrt", "rsqrt", "sin", "cos"])
def test_unary(ctx, dtype, op):
    rng = np.random.default_rng(21)
    for n in (1, 1000, 70001):
        x = rnd(rng, (n,), dtype, 2.0)
        if op in ("log", "sqrt", "rsqrt"):
            xf = np.abs(oracle.as_float(x, dtype)) + 0.01
            x = xf.astype(np.float32) if dtype == F32 else oracle.to_bf16(xf)
        y = empty_dev((n,), dtype)
        ctx.unary(op, to_dev(x, dtype), y, n, dtype)
        ctx.check()
        want = oracle.port().unary(x, dtype, op)
        if dtype == F32 and op in ("sqrt", "rsqrt"):  # correctly rounded on both sides
            assert np.array_equal(to_host(y), want)
        else:
            assert_close(to_host(y), want, dtype, what=op)


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_leaky_relu(ctx, dtype):
    rng = np.random.default_rng(22)
    x = rnd(rng, (5003,), dtype, 3.0)
    for slope in (0.01, 0.2):
        y = empty_dev(x.shape, dtype)
        ctx.leaky_relu(to_dev(x, dtype), y, x.size, slope, dtype)
        ctx.check()
        want = oracle.port().leaky_relu(x, slope, dtype)
        if dtype == F32:
            assert np.array_equal(to_host(y), want)
        else:
            assert_close(to_host(y), want, dtype, what="leaky_relu")


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_broadcast_row_concat_upsample(ctx, dtype):
    rng = np.random.default_rng(23)
    row = rnd(rng, (37,), dtype)
    out = empty_dev((11, 37), dtype)
    ctx.broadcast_row(to_dev(row, dtype), out, 11, 37, dtype)
    assert np.array_equal(to_host(out), np.broadcast_to(row, (11, 37)))

    for dims, outer, inner in (((3, 1, 5), 4, 6), ((2, 7), 1, 1), ((4, 0, 3, 1, 1, 2, 9, 5), 3, 10)):
        xs = [rnd(rng, (outer, d, inner), dtype) for d in dims]
        out = empty_dev((outer, sum(dims), inner), dtype)
        devs = [to_dev(x, dtype) for x in xs]
        ctx.concat(devs, list(dims), out, outer, inner, dtype)
        ctx.check()
        assert np.array_equal(to_host(out), np.concatenate(xs, axis=1))

    x = rnd(rng, (2, 3, 5, 7), dtype)
    for scale in (1, 2, 3):
        y = empty_dev((2, 3, 5 * scale, 7 * scale), dtype)
        ctx.upsample2d(to_dev(x, dtype), y, 2, 3, 5, 7, scale, dtype)
        ctx.check()
        assert np.array_equal(to_host(y), np.repeat(np.repeat(x, scale, axis=2), scale, axis=3))


def test_concat_limits(ctx):
    import munet_b200 as mb
    t = empty_dev((4,), F32)
    with pytest.raises(mb.MuNetError, match="more than 8"):
        ctx.concat([t] * 9, [1] * 9, t, 1, 1, F32)
    ctx.concat([t], [0], t, 3, 5, F32)  # nothing to copy


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_batch_norm_eval(ctx, dtype):
    rng = np.random.default_rng(24)
    B, Cc, H, W = 4, 6, 5, 7
    x = rnd(rng, (B, Cc, H, W), dtype, 2.0)
    g, b = rnd(rng, (Cc,), dtype), rnd(rng, (Cc,), dtype)
    mean = rng.standard_normal(Cc).astype(np.float32)
    var = (rng.random(Cc) + 0.1).astype(np.float32)
    y = empty_dev(x.shape, dtype)
    ctx.batch_norm_eval(to_dev(x, dtype), to_dev(g, dtype), to_dev(b, dtype), to_dev(mean, F32),
                        to_dev(var, F32), y, B, Cc, H, W, 1e-5, dtype)
    ctx.check()
    # float arithmetic in the reference's order, correctly rounded single ops: same bits
    assert np.array_equal(to_host(y), oracle.port().batch_norm_eval(x, g, b, mean, var, dtype))


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("rows,cols", [(19, 96), (1, 7), (300, 2048)])
def test_rms_norm(ctx, dtype, rows, cols):
    rng = np.random.default_rng(rows + cols)
    x, w = rnd(rng, (rows, cols), dtype, 2.0), rnd(rng, (cols,), dtype)
    y = empty_dev((rows, cols), dtype)
    ctx.rms_norm(to_dev(x, dtype), to_dev(w, dtype), y, rows, cols, dtype)
    ctx.check()
    assert_close(to_host(y), oracle.port().rms_norm(x, w, dtype), dtype, what="rms_norm")


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_reductions(ctx, dtype):
    rng = np.random.default_rng(25)
    x = rnd(rng, (23, 130), dtype)
    out = empty_dev((23,), dtype)
    ctx.mean_last_dim(to_dev(x, dtype), out, 23, 130, dtype)
    ctx.check()
    assert_close(to_host(out), oracle.port().mean_last_dim(x, dtype), dtype, what="mean_last_dim")
    s = empty_dev((1,), dtype)
    ctx.sum(to_dev(x, dtype), s, x.size, dtype)
    ctx.check()
    assert_close(to_host(s), oracle.port().sum(x.reshape(-1), dtype), dtype, what="sum")
    # sum_to_shape: numpy sum over the broadcast dimensions, in double
    xf = oracle.as_float(x, dtype).astype(np.float64).reshape(23, 10, 13)
    for out_shape, axes in (((10, 13), (0,)), ((23, 1, 13), (1,)), ((1,), (0, 1, 2)), ((13,), (0, 1)),
                            ((23, 10, 13), ())):
        want = xf.sum(axis=axes, keepdims=False).reshape(out_shape).astype(np.float32)
        want = want if dtype == F32 else oracle.to_bf16(want)
        o = empty_dev(out_shape, dtype)
        ctx.sum_to_shape(to_dev(x, dtype), o, [23, 10, 13], list(out_shape), dtype)
        ctx.check()
        assert_close(to_host(o), want, dtype, what=f"sum_to_shape {out_shape}")


def test_sum_to_shape_rejects_mismatch(ctx):
    import munet_b200 as mb
    t = empty_dev((24,), F32)
    with pytest.raises(mb.MuNetError, match="extent must be 1"):
        ctx.sum_to_shape(t, t, [4, 6], [4, 5], F32)


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_fill_uniform(ctx, dtype):
    n = 200000
    a, b = empty_dev((n,), dtype), empty_dev((n,), dtype)
    ctx.fill_uniform(a, n, -2.0, 3.0, 7, dtype)
    ctx.fill_uniform(b, n, -2.0, 3.0, 7, dtype)
    ctx.check()
    va = oracle.as_float(to_host(a), dtype)
    assert np.array_equal(to_host(a), to_host(b))          # a pure function of (seed, index)
    assert va.min() >= -2.0 and va.max() <= 3.0
    assert abs(va.mean() - 0.5) < 0.02 and abs(va.var() - 25.0 / 12.0) < 0.05
    ctx.fill_uniform(b, n, -2.0, 3.0, 8, dtype)
    assert not np.array_equal(to_host(a), to_host(b))


def test_engine_unet_style_block(tmp_path):
    """Conv2d → BatchNorm2d (running statistics) → LeakyReLU → Upsample → Conv2d through the
    executor, float32: identical bits to the same ops of the CPU checker, and to the reference's
    own Engine where its library is present."""
    import munet_b200 as mb
    from munet_b200.inference import Engine, save_deploy
    rng = np.random.default_rng(31)
    t = {
        "0.weight": (rng.standard_normal((8, 3, 3, 3)) * 0.3).astype(np.float32),
        "0.bias": rng.standard_normal(8).astype(np.float32) * 0.1,
        "1.weight": rng.standard_normal(8).astype(np.float32),
        "1.bias": rng.standard_normal(8).astype(np.float32),
        "1.running_mean": rng.standard_normal(8).astype(np.float32) * 0.2,
        "1.running_var": (rng.random(8) + 0.5).astype(np.float32),
        "4.weight": (rng.standard_normal((4, 8, 3, 3)) * 0.2).astype(np.float32),
        "4.bias": np.zeros(4, np.float32),
    }
    cfg = {"type": "Sequential", "layers": [
        {"type": "Conv2d", "in_channels": 3, "out_channels": 8, "kernel_size": 3, "stride": 1, "padding": 1},
        {"type": "BatchNorm2d", "num_features": 8, "eps": 1e-5, "momentum": 0.1},
        {"type": "LeakyReLU", "negative_slope": 0.2},
        {"type": "Upsample", "scale_factor": 2},
        {"type": "Conv2d", "in_channels": 8, "out_channels": 4, "kernel_size": 3, "stride": 1, "padding": 1}]}
    path = str(tmp_path / "unet_block.npz")
    save_deploy(path, cfg, t)
    x = rng.random((2, 3, 10, 12), dtype=np.float32)
    P = oracle.port()
    h = P.conv2d(x, t["0.weight"], t["0.bias"], 1, 1)
    h = P.batch_norm_eval(h, t["1.weight"], t["1.bias"], t["1.running_mean"], t["1.running_var"], F32)
    h = P.leaky_relu(h, 0.2, F32).reshape(h.shape)
    h = np.repeat(np.repeat(h, 2, axis=2), 2, axis=3)
    want = P.conv2d(h, t["4.weight"], t["4.bias"], 1, 1)
    eng = Engine(compute_dtype=F32).load(path).compile(x.shape)
    got = eng.run(x)
    assert got.shape == (2, 4, 20, 24)
    assert np.array_equal(got, want)
    if oracle.have_ref():
        assert np.array_equal(got, oracle.ref().engine_run_npz(path, x))
    eng.close()
    with pytest.raises(mb.MuNetError, match="num_features"):
        bad = dict(cfg, layers=[cfg["layers"][0], {"type": "BatchNorm2d", "num_features": 5, "eps": 1e-5}])
        Engine(compute_dtype=F32).load(bad, t).compile(x.shape)


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_engine_rms_norm_mlp(dtype):
    """Linear → RMSNorm → LeakyReLU → Linear in both compute dtypes."""
    from munet_b200.inference import Engine
    rng = np.random.default_rng(32)
    t32 = {"0.weight": (rng.standard_normal((48, 64)) * 0.2).astype(np.float32),
           "0.bias": (rng.standard_normal(64) * 0.1).astype(np.float32),
           "1.weight": rng.standard_normal(64).astype(np.float32),
           "3.weight": (rng.standard_normal((64, 24)) * 0.2).astype(np.float32),
           "3.bias": np.zeros(24, np.float32)}
    t = {k: (v if dtype == F32 else oracle.to_bf16(v)) for k, v in t32.items()}
    cfg = {"type": "Sequential", "layers": [
        {"type": "Linear", "in_features": 48, "out_features": 64, "bias": True},
        {"type": "RMSNorm", "normalized_shape": 64, "eps": 1e-5},
        {"type": "LeakyReLU", "negative_slope": 0.01},
        {"type": "Linear", "in_features": 64, "out_features": 24, "bias": True}]}
    x = rnd(rng, (33, 48), dtype)
    P = oracle.port()
    h = P.linear(x, t["0.weight"], t["0.bias"], dtype)
    h = P.rms_norm(h, t["1.weight"], dtype)
    h = P.leaky_relu(h, 0.01, dtype).reshape(h.shape)
    want = P.linear(h, t["3.weight"], t["3.bias"], dtype)
    eng = Engine(compute_dtype=dtype).load(cfg, t, tensor_dtype=dtype).compile(x.shape)
    got = eng.run(x)
    assert_close(got, want, dtype, what="rms-norm mlp")
    eng.close()
