"""GPU parity of the spatial ops and of the small CNN config (float32): every output
must be bit-identical to the CPU checker, which is itself bit-identical to the
reference CPU kernels (same summation order, no fused multiply-add)."""
import numpy as np
import pytest

import oracle
from oracle import F32
from tests.util import assert_close, empty_dev, to_dev, to_host

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    import munet_b200 as mb
    c = mb.Context(0)
    yield c
    c.close()


def same(a, b):
    assert a.shape == b.shape
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32)), f"max diff {np.abs(a - b).max()}"


@pytest.mark.parametrize("B,iC,H,W,oC,k,s,p", [
    (2, 3, 32, 32, 64, 3, 1, 1), (3, 64, 16, 16, 128, 3, 1, 1), (2, 128, 8, 8, 256, 3, 1, 1),
    (2, 5, 13, 11, 7, 3, 1, 0), (1, 4, 9, 9, 6, 3, 2, 1), (2, 3, 20, 20, 40, 5, 1, 2), (1, 1, 3, 3, 1, 2, 1, 0)])
def test_conv2d_bit_exact(ctx, B, iC, H, W, oC, k, s, p):
    rng = np.random.default_rng(B + iC + H + oC)
    x = rng.random((B, iC, H, W), dtype=np.float32)
    w = (rng.standard_normal((oC, iC, k, k)) * np.sqrt(2.0 / (iC * k * k))).astype(np.float32)
    b = (rng.standard_normal(oC) * 0.1).astype(np.float32)
    want = oracle.port().conv2d(x, w, b, s, p)
    y = empty_dev(want.shape, F32)
    ctx.conv2d(to_dev(x, F32), to_dev(w, F32), to_dev(b, F32), y, B, iC, H, W, oC, k, s, p, F32)
    ctx.check()
    same(to_host(y), want)
    # fused ReLU + MaxPool2d(2,2,0) equals the three separate reference ops
    if want.shape[2] >= 2 and want.shape[3] >= 2:
        want_p = oracle.port().max_pool2d(np.maximum(want, 0), 2, 2, 0)
        yp = empty_dev(want_p.shape, F32)
        ctx.conv2d(to_dev(x, F32), to_dev(w, F32), to_dev(b, F32), yp, B, iC, H, W, oC, k, s, p, F32,
                   relu=True, pool=2)
        ctx.check()
        same(to_host(yp), want_p)


@pytest.mark.parametrize("k,s,p", [(2, 2, 0), (3, 2, 1), (3, 1, 1)])
def test_max_pool_and_gap_bit_exact(ctx, k, s, p):
    rng = np.random.default_rng(k * 10 + s)
    x = rng.standard_normal((3, 5, 12, 10)).astype(np.float32)
    want = oracle.port().max_pool2d(x, k, s, p)
    y = empty_dev(want.shape, F32)
    ctx.max_pool2d(to_dev(x, F32), y, 3, 5, 12, 10, k, s, p, F32)
    ctx.check()
    same(to_host(y), want)
    g = empty_dev((3, 5, 1, 1), F32)
    ctx.global_avg_pool(to_dev(x, F32), g, 3, 5, 12, 10, F32)
    ctx.check()
    same(to_host(g), oracle.port().global_avg_pool(x))


def cnn_config_and_weights(rng):
    layers, tensors, idx = [], {}, 0
    for ic, oc, tail in ((3, 64, "pool"), (64, 128, "pool"), (128, 256, "gap")):
        layers.append({"type": "Conv2d", "in_channels": ic, "out_channels": oc, "kernel_size": 3,
                       "stride": 1, "padding": 1})
        tensors[f"{idx}.weight"] = (rng.standard_normal((oc, ic, 3, 3)) * np.sqrt(2.0 / (ic * 9))).astype(np.float32)
        tensors[f"{idx}.bias"] = np.zeros(oc, np.float32)
        layers.append({"type": "ReLU"})
        layers.append({"type": "MaxPool2d", "kernel_size": 2, "stride": 2, "padding": 0} if tail == "pool"
                      else {"type": "GlobalAvgPool2d"})
        idx += 3
    layers.append({"type": "Flatten"})
    layers.append({"type": "Linear", "in_features": 256, "out_features": 10, "bias": True})
    tensors[f"{idx + 1}.weight"] = (rng.standard_normal((256, 10)) * np.sqrt(2.0 / 256)).astype(np.float32)
    tensors[f"{idx + 1}.bias"] = np.zeros(10, np.float32)
    return {"type": "Sequential", "layers": layers}, tensors


def cnn_oracle(x, t):
    P = oracle.port()
    h = P.max_pool2d(np.maximum(P.conv2d(x, t["0.weight"], t["0.bias"], 1, 1), 0))
    h = P.max_pool2d(np.maximum(P.conv2d(h, t["3.weight"], t["3.bias"], 1, 1), 0))
    h = P.global_avg_pool(np.maximum(P.conv2d(h, t["6.weight"], t["6.bias"], 1, 1), 0))
    return P.linear(h.reshape(h.shape[0], -1), t["10.weight"], t["10.bias"], F32)


def test_small_cnn_config_bit_exact(ctx, tmp_path):
    """conv3x3(3→64)+ReLU+pool, conv3x3(64→128)+ReLU+pool, conv3x3(128→256)+ReLU+GAP, linear 256→10
    on [B,3,32,32] U[0,1): logits and argmax identical to the reference (B reduced for the CPU side)."""
    from munet_b200.inference import Engine, save_deploy
    rng = np.random.default_rng(1003)
    cfg, tensors = cnn_config_and_weights(rng)
    path = str(tmp_path / "cnn.npz")
    save_deploy(path, cfg, tensors)
    B = 16
    x = np.random.default_rng(2003).random((B, 3, 32, 32), dtype=np.float32)
    want = cnn_oracle(x, tensors)
    eng = Engine(ctx=ctx, compute_dtype=F32, argmax=True).load(path).compile((B, 3, 32, 32))
    got, am = eng.run(x)
    same(got, want)
    assert np.array_equal(am, oracle.port().argmax(want, F32))
    # 12 modules fuse to 6 ops: 3 conv blocks (ReLU and both max-pools folded in), GAP, linear, argmax
    assert eng.stats()["n_ops"] == 6
    if oracle.have_ref():
        same(got, oracle.ref().engine_run_npz(path, x))
    eng.close()


@pytest.mark.parametrize("B,iC,H,oC,relu,pool", [(256, 64, 16, 128, True, 2), (96, 128, 8, 256, True, 0),
                                                 (300, 3, 32, 64, False, 0), (70, 40, 18, 100, True, 2)])
def test_large_conv_on_tensor_cores_matches_direct_kernel(ctx, B, iC, H, oC, relu, pool):
    """From 2^31 multiply-adds on a convolution runs as im2col + 3xTF32 GEMM. The direct kernel
    (the reference's accumulation order, bit-exact against the CPU checker in the tests above) is
    the witness: float32-class agreement, 1e-5 against the config tolerance of 1e-4."""
    rng = np.random.default_rng(B + iC)
    x = rng.standard_normal((B, iC, H, H)).astype(np.float32)
    w = (rng.standard_normal((oC, iC, 3, 3)) * np.sqrt(2.0 / (iC * 9))).astype(np.float32)
    b = (rng.standard_normal(oC) * 0.1).astype(np.float32)
    oH = H // 2 if pool else H
    outs = []
    for simt in (True, False):
        y = empty_dev((B, oC, oH, oH), F32)
        ctx.force_simt(simt)
        ctx.conv2d(to_dev(x, F32), to_dev(w, F32), to_dev(b, F32), y, B, iC, H, H, oC, 3, 1, 1, F32,
                   relu=relu, pool=pool)
        ctx.check()
        outs.append(to_host(y))
    ctx.force_simt(False)
    direct, tensor = outs
    macs = B * H * H * oC * iC * 9
    if macs >= 2 ** 31:
        assert not np.array_equal(direct, tensor), "expected the tensor-core path"
    assert_close(tensor, direct, F32, rtol=1e-5, what="conv im2col+3xTF32 vs direct")
    # one image against the CPU checker ties both to the reference
    P = oracle.port()
    want = P.conv2d(x[:1], w, b, 1, 1)
    if relu:
        want = np.maximum(want, 0)
    if pool:
        want = P.max_pool2d(want)
    assert_close(tensor[:1], want, F32, rtol=1e-5, what="conv vs checker")


@pytest.mark.parametrize("B,iC,H,W,oC,k,relu,pool", [
    (64, 32, 32, 32, 64, 5, True, 0),     # 5x5 filter, four image rows per 128-pixel box
    (512, 128, 8, 8, 256, 3, True, 0),    # two whole images per box
    (256, 64, 4, 32, 128, 3, False, 0),   # one image = one box (4 rows of 32)
    (16, 32, 64, 64, 32, 3, True, 2),     # two rows per box, MaxPool folded into the layout pass
    (66, 64, 8, 8, 64, 3, True, 0),       # 66 images in boxes of two
    (65, 64, 8, 8, 64, 3, True, 0),       # an odd image count cannot be boxed: im2col path
])
def test_implicit_gemm_conv_geometries(ctx, B, iC, H, W, oC, k, relu, pool):
    """The implicit-GEMM convolution (shifted 4-D boxes of the NHWC input as k-blocks, zero fill as
    padding) over the ways 128 output pixels can be cut out of the images, against the direct
    kernel (bit-exact with the reference) on every output and the CPU checker on the first and
    last image."""
    rng = np.random.default_rng(B + iC + H + k)
    pad = (k - 1) // 2
    x = rng.standard_normal((B, iC, H, W)).astype(np.float32)
    w = (rng.standard_normal((oC, iC, k, k)) * np.sqrt(2.0 / (iC * k * k))).astype(np.float32)
    b = (rng.standard_normal(oC) * 0.1).astype(np.float32)
    oH, oW = (H // 2, W // 2) if pool else (H, W)
    outs = []
    for simt in (True, False):
        y = empty_dev((B, oC, oH, oW), F32)
        ctx.force_simt(simt)
        ctx.conv2d(to_dev(x, F32), to_dev(w, F32), to_dev(b, F32), y, B, iC, H, W, oC, k, 1, pad, F32,
                   relu=relu, pool=pool)
        ctx.check()
        outs.append(to_host(y))
    ctx.force_simt(False)
    direct, tensor = outs
    if B * H * W * oC * iC * k * k >= 2 ** 31:
        assert not np.array_equal(direct, tensor), "expected the tensor-core path"
    # float32-class agreement: two summation orders of up to 1152 float products differ by a few
    # 1e-6 relative; 3e-5 elementwise is a third of the 1e-4 tolerance of the float32 configs
    assert_close(tensor, direct, F32, rtol=3e-5, what="implicit-GEMM conv vs direct")
    P = oracle.port()
    for i in (0, B - 1):
        want = P.conv2d(x[i:i + 1], w, b, 1, pad)
        if relu:
            want = np.maximum(want, 0)
        if pool:
            want = P.max_pool2d(want)
        assert_close(tensor[i:i + 1], want, F32, rtol=3e-5, what="implicit-GEMM conv vs checker")
