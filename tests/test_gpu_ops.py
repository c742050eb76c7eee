"""GPU parity: every C-ABI entry point against the CPU checker (oracle/) on the
same seeded inputs.  float32 tolerance 1e-4, bfloat16 2e-2, relative as defined
in tests/util.close; float32 matmul/linear (none, relu) and argmax are bit-exact."""
import numpy as np
import pytest

import oracle
from oracle import BF16, F32, I32
from tests.util import assert_close, empty_dev, rnd, to_dev, to_host

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    import munet_b200 as mb
    c = mb.Context(0)
    yield c
    c.close()


def dev_linear(ctx, x, w, b, dtype, act="none", res=None, simt=False):
    M, K = x.shape
    N = w.shape[1]
    y = empty_dev((M, N), dtype)
    ctx.force_simt(simt)
    ctx.linear(to_dev(x, dtype), to_dev(w, dtype), None if b is None else to_dev(b, dtype), y,
               M, K, N, dtype, act=act, residual=None if res is None else to_dev(res, dtype))
    ctx.check()
    ctx.force_simt(False)
    return to_host(y)


@pytest.mark.parametrize("M,K,N", [(128, 64, 64), (128, 64, 256), (256, 512, 384), (1000, 328, 520),
                                   (77, 40, 24), (2048, 1024, 1024)])
@pytest.mark.parametrize("act", ["none", "gelu"])
def test_linear_bf16_tcgen05(ctx, M, K, N, act):
    rng = np.random.default_rng(M + K + N)
    x = rnd(rng, (M, K), BF16)
    w = rnd(rng, (K, N), BF16, 1.0 / np.sqrt(K))
    b = rnd(rng, (N,), BF16, 0.02)
    want = oracle.port().linear(x, w, b, BF16, act)
    got = dev_linear(ctx, x, w, b, BF16, act)
    assert_close(got, want, BF16, what="linear bf16")
    got_simt = dev_linear(ctx, x, w, b, BF16, act, simt=True)
    assert_close(got_simt, want, BF16, what="linear bf16 (cuda-core kernel)")


@pytest.mark.parametrize("M,K,N", [(1152, 256, 3840), (1100, 200, 3800), (2560, 128, 2048)])
@pytest.mark.parametrize("transB", [False, True])
def test_linear_bf16_cta_pairs(ctx, M, K, N, transB):
    """Shapes large enough for the CTA-pair (256 x 256 tile) kernel, ragged in M, N and K, with
    bias + GELU + residual; weights as [K,N] (Linear) and as [N,K] (matmul with transB)."""
    rng = np.random.default_rng(M + K + N)
    x = rnd(rng, (M, K), BF16)
    w = rnd(rng, (K, N), BF16, 1.0 / np.sqrt(K))
    b, r = rnd(rng, (N,), BF16, 0.05), rnd(rng, (M, N), BF16)
    P = oracle.port()
    if not transB:
        want = P.add(P.linear(x, w, b, BF16, "gelu"), r, BF16)
        assert_close(dev_linear(ctx, x, w, b, BF16, "gelu", res=r), want, BF16, what="pair linear")
    else:
        c = empty_dev((M, N), BF16)
        ctx.matmul(to_dev(x, BF16), to_dev(np.ascontiguousarray(w.T), BF16), c, M, K, N, BF16, transB=True)
        ctx.check()
        assert_close(to_host(c), P.matmul(x, w, BF16), BF16, what="pair matmul transB")


@pytest.mark.parametrize("budget", [2, 37, 100])
def test_linear_bf16_under_an_sm_budget(ctx, budget):
    """A persistent GEMM limited to a few SMs (what the executor does while a collective runs
    beside it) walks the same tiles with fewer CTAs: same bits as the unrestricted launch, for the
    CTA-pair kernel (odd budgets round down to whole pairs) and the single-CTA kernel."""
    rng = np.random.default_rng(budget)
    for M, K, N in ((2560, 128, 2048), (300, 256, 512)):
        x, w, b = rnd(rng, (M, K), BF16), rnd(rng, (K, N), BF16, 1.0 / np.sqrt(K)), rnd(rng, (N,), BF16, 0.05)
        full = dev_linear(ctx, x, w, b, BF16, "gelu")
        ctx.set_sm_budget(budget)
        try:
            limited = dev_linear(ctx, x, w, b, BF16, "gelu")
        finally:
            ctx.set_sm_budget(0)
        assert np.array_equal(full, limited)


def test_linear_bf16_l2_set_aside_changes_no_bits(ctx):
    """mu_ctx_set_l2_set_aside reserves L2 for the weight tiles and switches the loads of long-K and
    wide-N shapes to the evict_last / evict_first priorities: cache behaviour only, same results."""
    rng = np.random.default_rng(41)
    shapes = ((4096, 4096, 1024, "none", True), (4096, 1024, 8192, "gelu", False), (512, 4096, 1024, "none", False))
    base = []
    for M, K, N, act, res in shapes:
        x, w, b = rnd(rng, (M, K), BF16), rnd(rng, (K, N), BF16, 1.0 / np.sqrt(K)), rnd(rng, (N,), BF16, 0.05)
        r = rnd(rng, (M, N), BF16) if res else None
        base.append((x, w, b, r, act, dev_linear(ctx, x, w, b, BF16, act, res=r)))
    ctx.set_l2_set_aside(32 << 20)
    try:
        for x, w, b, r, act, want in base:
            assert np.array_equal(dev_linear(ctx, x, w, b, BF16, act, res=r), want)
    finally:
        ctx.set_l2_set_aside(0)


def test_linear_bf16_wide_weights_use_column_panels(ctx):
    """A weight matrix wider than the L2 budget (here 49 MB) is swept in panels of column tiles,
    the last one narrower. Every output tile must still be produced exactly once: compared with
    the CUDA-core kernel on the whole output and with the CPU checker on a few rows."""
    rng = np.random.default_rng(77)
    M, K, N = 1100, 2048, 12032
    x = rnd(rng, (M, K), BF16)
    w = rnd(rng, (K, N), BF16, 1.0 / np.sqrt(K))
    b = rnd(rng, (N,), BF16, 0.05)
    got = dev_linear(ctx, x, w, b, BF16)
    assert_close(got, dev_linear(ctx, x, w, b, BF16, simt=True), BF16, what="panels vs cuda-core kernel")
    rows = [0, 127, 128, 255, 256, 700, 1023, 1024, 1099]
    assert_close(got[rows], oracle.port().linear(x[rows], w, b, BF16), BF16, what="panels vs checker")


@pytest.mark.parametrize("act", ["none", "relu", "gelu", "sigmoid", "tanh"])
def test_linear_bf16_acts_residual(ctx, act):
    rng = np.random.default_rng(5)
    M, K, N = 300, 256, 512
    x, w = rnd(rng, (M, K), BF16), rnd(rng, (K, N), BF16, 1.0 / 16)
    b, r = rnd(rng, (N,), BF16, 0.1), rnd(rng, (M, N), BF16)
    want = oracle.port().add(oracle.port().linear(x, w, b, BF16, act), r, BF16)
    assert_close(dev_linear(ctx, x, w, b, BF16, act, res=r), want, BF16, what=f"linear+{act}+res")
    want_nb = oracle.port().linear(x, w, None, BF16, act)
    assert_close(dev_linear(ctx, x, w, None, BF16, act), want_nb, BF16, what="linear no bias")


@pytest.mark.parametrize("M,K,N", [(256, 784, 512), (256, 512, 10), (33, 17, 5), (1, 64, 3)])
@pytest.mark.parametrize("act", ["none", "relu"])
def test_linear_f32_bit_exact(ctx, M, K, N, act):
    rng = np.random.default_rng(M * 3 + N)
    x = rng.random((M, K), dtype=np.float32)
    w = rnd(rng, (K, N), F32, np.sqrt(2.0 / K))
    b = rnd(rng, (N,), F32, 0.1)
    want = oracle.port().linear(x, w, b, F32, act)
    got = dev_linear(ctx, x, w, b, F32, act)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), \
        f"max diff {np.abs(got - want).max()}"


@pytest.mark.parametrize("M,K,N,act,res", [(2048, 1024, 1024, "none", False), (1300, 1284, 1300, "gelu", True),
                                           (4100, 516, 1028, "relu", False)])
def test_linear_f32_tensor_core_split(ctx, M, K, N, act, res):
    """float32 products of 2^31 multiply-adds and more run on the tensor cores with every operand
    split into two TF32 parts. Both that result and the CUDA-core kernel's (the reference's float
    accumulation order) are compared with a float64 evaluation: the split product must be
    float32-class — within 3e-5 of the truth (the config tolerance is 1e-4). The tensor core adds
    into its accumulator with truncation, so the split product carries a small bias toward zero
    that the sequential float sum does not have; summing K in chunks keeps it below 1e-5 of the
    result's RMS whatever K is."""
    rng = np.random.default_rng(M + N)
    x = rnd(rng, (M, K), F32)
    w = rnd(rng, (K, N), F32, 1.0 / np.sqrt(K))
    b = rnd(rng, (N,), F32, 0.1)
    r = rnd(rng, (M, N), F32) if res else None
    t = x.astype(np.float64) @ w.astype(np.float64) + b
    if act == "gelu":
        t = t / (1.0 + np.exp(-1.702 * t))
    elif act == "relu":
        t = np.maximum(t, 0.0)
    if res:
        t = t + r
    simt = dev_linear(ctx, x, w, b, F32, act, res=r, simt=True)
    got = dev_linear(ctx, x, w, b, F32, act, res=r)
    assert not np.array_equal(got, simt), "expected the tensor-core path, got the CUDA-core bits"
    assert_close(got, t.astype(np.float32), F32, rtol=3e-5, what="3xTF32 linear vs float64")
    assert_close(simt, t.astype(np.float32), F32, rtol=3e-5, what="CUDA-core linear vs float64")
    rms = float(np.sqrt((t * t).mean()))
    assert abs(float(((got - t) * np.sign(t)).mean())) < 1e-5 * rms


@pytest.mark.parametrize("act", ["gelu", "sigmoid", "tanh"])
def test_linear_f32_acts(ctx, act):
    rng = np.random.default_rng(9)
    x, w, b = rnd(rng, (64, 96), F32), rnd(rng, (96, 80), F32, 0.1), rnd(rng, (80,), F32, 0.1)
    assert_close(dev_linear(ctx, x, w, b, F32, act), oracle.port().linear(x, w, b, F32, act), F32)


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("transB", [False, True])
def test_matmul_and_batched(ctx, dtype, transB):
    rng = np.random.default_rng(11)
    M, K, N, batch = 96, 128, 64, 5
    a = rnd(rng, (batch, M, K), dtype)
    b = rnd(rng, (batch, K, N), dtype, 1.0 / np.sqrt(K))
    want = np.stack([oracle.port().matmul(a[i], b[i], dtype) for i in range(batch)])
    bd = np.ascontiguousarray(np.swapaxes(b, 1, 2)) if transB else b
    c = empty_dev((batch, M, N), dtype)
    ctx.batched_matmul(to_dev(a, dtype), to_dev(bd, dtype), c, batch, M, K, N, M * K, K * N, M * N,
                       dtype, transB=transB)
    ctx.check()
    assert_close(to_host(c), want, dtype, what="batched_matmul")
    # broadcast weights (stride_b = 0): how a 3-D Linear input reaches the backend
    want0 = np.stack([oracle.port().matmul(a[i], b[0], dtype) for i in range(batch)])
    ctx.batched_matmul(to_dev(a, dtype), to_dev(bd[0], dtype), c, batch, M, K, N, M * K, 0, M * N,
                       dtype, transB=transB)
    ctx.check()
    assert_close(to_host(c), want0, dtype, what="batched_matmul broadcast")
    c2 = empty_dev((M, N), dtype)
    ctx.matmul(to_dev(a[1], dtype), to_dev(bd[1], dtype), c2, M, K, N, dtype, transB=transB)
    ctx.check()
    assert_close(to_host(c2), want[1], dtype, what="matmul")


def test_matmul_transA_is_rejected(ctx):
    import munet_b200 as mb
    t = empty_dev((4, 4), F32)
    with pytest.raises(mb.MuNetError):
        ctx.matmul(t, t, t, 4, 4, 4, F32, transA=True)


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("rows,cols", [(64, 512), (1000, 2048), (7, 200), (5, 33), (3, 4096),
                                       (1, 2048), (2371, 1024), (40003, 512), (20011, 2048)])
def test_layer_norm(ctx, dtype, rows, cols):
    rng = np.random.default_rng(rows + cols)
    x = rnd(rng, (rows, cols), dtype, 2.0)
    g, b = rnd(rng, (cols,), dtype), rnd(rng, (cols,), dtype)
    y = empty_dev((rows, cols), dtype)
    ctx.layer_norm(to_dev(x, dtype), to_dev(g, dtype), to_dev(b, dtype), y, rows, cols, dtype)
    ctx.check()
    assert_close(to_host(y), oracle.port().layer_norm(x, g, b, dtype), dtype, what="layer_norm")


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("rows,cols", [(64, 256), (100, 1024), (9, 33), (4, 5000), (3, 512),
                                       (20011, 2048), (40001, 256)])
def test_softmax(ctx, dtype, rows, cols):
    rng = np.random.default_rng(rows * cols)
    x = rnd(rng, (rows, cols), dtype, 3.0)
    y = empty_dev((rows, cols), dtype)
    ctx.softmax(to_dev(x, dtype), y, rows, cols, dtype)
    ctx.check()
    got, want = to_host(y), oracle.port().softmax(x, dtype)
    assert_close(got, want, dtype, what="softmax")
    assert np.allclose(oracle.as_float(got, dtype).sum(-1), 1.0, atol=2e-2 if dtype == BF16 else 1e-5)


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_embedding(ctx, dtype):
    import munet_b200 as mb
    rng = np.random.default_rng(3)
    B, T, V, D = 3, 17, 100, 64
    table, pos = rnd(rng, (V, D), dtype), rnd(rng, (T, D), dtype)
    ids = rng.integers(0, V, (B, T)).astype(np.int32)
    out = empty_dev((B, T, D), dtype)
    ctx.embedding(to_dev(ids, I32), to_dev(table, dtype), None, out, B, T, V, D, dtype)
    ctx.check()
    want = oracle.port().embedding(ids, table, dtype)
    assert np.array_equal(to_host(out), want)
    ctx.embedding(to_dev(ids, I32), to_dev(table, dtype), to_dev(pos, dtype), out, B, T, V, D, dtype)
    ctx.check()
    want_pos = np.stack([oracle.port().add(want[b], pos, dtype) for b in range(B)])
    assert np.array_equal(to_host(out), want_pos)
    bad = ids.copy()
    bad[1, 2] = V  # the reference throws "Embedding index out of range"
    ctx.embedding(to_dev(bad, I32), to_dev(table, dtype), None, out, B, T, V, D, dtype)
    with pytest.raises(mb.MuNetError, match="out of range"):
        ctx.check()
    ctx.check()  # status is cleared after being reported


@pytest.mark.parametrize("act", ["none", "relu", "gelu", "sigmoid", "tanh"])
@pytest.mark.parametrize("rows,cols", [(1, 8), (333, 512), (70001, 64)])
def test_eltwise_bf16_chain(ctx, act, rows, cols):
    """bias + activation + residual in one pass (vector path), against the same three ops of the
    CPU checker applied one after another with its per-op rounding."""
    rng = np.random.default_rng(rows + cols)
    x, r = rnd(rng, (rows, cols), BF16, 2.0), rnd(rng, (rows, cols), BF16)
    b = rnd(rng, (cols,), BF16)
    y = empty_dev((rows, cols), BF16)
    ctx.eltwise(to_dev(x, BF16), y, rows * cols, BF16, act=act, bias=to_dev(b, BF16), cols=cols,
                residual=to_dev(r, BF16))
    ctx.check()
    o = oracle.port()
    want = o.add(x, np.broadcast_to(b, x.shape).copy(), BF16)
    if act != "none":
        want = o.activation(want, BF16, act)
    want = o.add(want, r, BF16)
    assert_close(to_host(y), want, BF16, what=f"bias+{act}+residual")


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("act", ["relu", "gelu", "sigmoid", "tanh"])
def test_eltwise(ctx, dtype, act):
    rng = np.random.default_rng(4)
    for n in (4096, 1001):
        x = rnd(rng, (n,), dtype, 2.0)
        y = empty_dev((n,), dtype)
        ctx.eltwise(to_dev(x, dtype), y, n, dtype, act=act)
        ctx.check()
        assert_close(to_host(y), oracle.port().activation(x, dtype, act), dtype, what=act)
    a, b = rnd(rng, (64, 48), dtype), rnd(rng, (64, 48), dtype)
    y = empty_dev((64, 48), dtype)
    ctx.eltwise(to_dev(a, dtype), y, a.size, dtype, residual=to_dev(b, dtype))
    ctx.check()
    want = oracle.port().add(a, b, dtype)
    if dtype == F32:
        assert np.array_equal(to_host(y), want)
    else:
        assert_close(to_host(y), want, dtype)


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_argmax_first_max(ctx, dtype):
    rng = np.random.default_rng(6)
    x = rnd(rng, (50, 1000), dtype)
    xf = oracle.as_float(x, dtype).copy()
    xf[3, 10] = xf[3, 500] = 100.0  # tie: the first index wins
    x = xf if dtype == F32 else oracle.to_bf16(xf)
    idx = empty_dev((50,), I32)
    ctx.argmax(to_dev(x, dtype), idx, 50, 1000, dtype)
    ctx.check()
    want = oracle.port().argmax(x, dtype)
    assert np.array_equal(to_host(idx), want) and want[3] == 10


@pytest.mark.parametrize("rows,cols", [(37, 32000), (5, 8), (9, 1000), (300, 1032), (4, 1001)])
def test_argmax_bf16_ties(ctx, rows, cols):
    """bf16 logits quantised coarsely: most rows hold their maximum several times, and the
    smallest index must win on every one of them (vector path for widths divisible by 8)."""
    rng = np.random.default_rng(rows * 7 + cols)
    xf = np.round(rng.standard_normal((rows, cols)) * 4).astype(np.float32) / 4
    xf[0, :] = -np.inf          # nothing beats -inf: index 0
    if rows > 2:
        xf[1, :] = 0.0
        xf[1, cols // 2] = -0.0  # signed zeros compare equal
        xf[2, cols - 1] = 1000.0
    x = oracle.to_bf16(xf)
    idx = empty_dev((rows,), I32)
    ctx.argmax(to_dev(x, BF16), idx, rows, cols, BF16)
    ctx.check()
    want = np.argmax(oracle.as_float(x, BF16), axis=-1).astype(np.int32)
    assert np.array_equal(oracle.port().argmax(x, BF16), want)
    assert np.array_equal(to_host(idx), want)


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("kmode", [oracle.K_LITERAL, oracle.K_MATH])
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("B,H,T,D", [(2, 4, 64, 64), (1, 2, 256, 128), (2, 2, 24, 16), (1, 3, 10, 8),
                                     (1, 3, 384, 128), (1, 2, 696, 64), (2, 1, 640, 128)])
def test_attention_core(ctx, dtype, kmode, causal, B, H, T, D):
    rng = np.random.default_rng(B * 1000 + T + D)
    n = B * H * T
    q, k, v = (rnd(rng, (n, D), dtype) for _ in range(3))
    want_hm = oracle.port().attention_core(q, k, v, B * H, T, D, causal, dtype, kmode)
    # merge heads: [B,H,T,D] -> [B,T,H*D]
    want = np.ascontiguousarray(want_hm.reshape(B, H, T, D).transpose(0, 2, 1, 3)).reshape(B * T, H * D)
    out = empty_dev((B * T, H * D), dtype)
    nbytes = ctx.attention_workspace_bytes(B, H, T, D, dtype)
    import torch
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    ctx.attention(to_dev(q, dtype), to_dev(k, dtype), to_dev(v, dtype), out, B, H, T, D, causal,
                  kmode, dtype, ws, nbytes)
    ctx.check()
    # long causal rows average hundreds of values: outputs far below the tensor's RMS, where the
    # rounding of single probabilities to bf16 (ours unnormalised, the reference's normalised) shows
    assert_close(to_host(out), want, dtype, what="attention", worst_cap=2.0 if T >= 512 else 1.0)


@pytest.mark.parametrize("kmode", [oracle.K_LITERAL, oracle.K_MATH])
@pytest.mark.parametrize("causal", [True, False])
def test_attention_growing_maximum_rescales_accumulator(ctx, kmode, causal):
    """Keys whose magnitude grows along the sequence: the row maximum jumps by far more than 2^8
    from one 128-key tile to the next, which is the case where the output accumulator kept in
    tensor memory has to be rescaled in place (otherwise it is left alone)."""
    rng = np.random.default_rng(99)
    B, H, T, D = 1, 2, 512, 64
    n = B * H * T
    q = rnd(rng, (n, D), BF16)
    grow = (1.0 + 30.0 * (np.arange(n) % T) / T)[:, None]
    k = oracle.to_bf16(oracle.from_bf16(rnd(rng, (n, D), BF16)) * grow.astype(np.float32))
    v = rnd(rng, (n, D), BF16)
    want_hm = oracle.port().attention_core(q, k, v, B * H, T, D, causal, BF16, kmode)
    want = np.ascontiguousarray(want_hm.reshape(B, H, T, D).transpose(0, 2, 1, 3)).reshape(B * T, H * D)
    out = empty_dev((B * T, H * D), BF16)
    nbytes = ctx.attention_workspace_bytes(B, H, T, D, BF16)
    ws = empty_dev((max(nbytes, 16),), oracle.I32) if False else None
    import torch
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device="cuda")
    ctx.attention(to_dev(q, BF16), to_dev(k, BF16), to_dev(v, BF16), out, B, H, T, D, causal, kmode, BF16,
                  ws, nbytes)
    ctx.check()
    assert_close(to_host(out), want, BF16, what="attention with growing maxima")


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("B,T,E,H", [(2, 64, 256, 4), (1, 24, 48, 3)])
def test_linear_qkv_head_major(ctx, dtype, B, T, E, H):
    rng = np.random.default_rng(E)
    x = rnd(rng, (B * T, E), dtype)
    ws = [rnd(rng, (E, E), dtype, 1 / np.sqrt(E)) for _ in range(3)]
    bs = [rnd(rng, (E,), dtype, 0.1) for _ in range(3)]
    wqkv = np.ascontiguousarray(np.concatenate(ws, axis=1))
    bqkv = np.concatenate(bs)
    D = E // H
    qkv = empty_dev((3, B * H * T, D), dtype)
    ctx.linear_qkv(to_dev(x, dtype), to_dev(wqkv, dtype), to_dev(bqkv, dtype), qkv[0], qkv[1], qkv[2],
                   B, T, E, H, dtype)
    ctx.check()
    got = to_host(qkv)
    for i in range(3):
        y = oracle.port().linear(x, ws[i], bs[i], dtype)
        hm = np.ascontiguousarray(y.reshape(B, T, H, D).transpose(0, 2, 1, 3)).reshape(B * H * T, D)
        if dtype == F32:
            assert np.array_equal(got[i], hm)
        else:
            assert_close(got[i], hm, dtype, what="qkv")


def test_empty_inputs(ctx):
    t = empty_dev((8,), F32)
    ctx.linear(t, t, None, t, 0, 4, 4, F32)
    ctx.layer_norm(t, t, t, t, 0, 8, F32)
    ctx.softmax(t, t, 0, 8, F32)
    ctx.eltwise(t, t, 0, F32, act="relu")
    ctx.check()


@pytest.mark.parametrize("kmode", [oracle.K_LITERAL, oracle.K_MATH])
def test_attention_core_headline_geometry(ctx, kmode):
    """The attention shape of the 24-layer decoder config — 16 heads of 128, 1024 positions, causal,
    eight key tiles per row — for one sequence, in both K addressing modes, against the checker.
    Late rows average up to 1024 values, so single outputs lie far below the tensor's RMS where one
    bf16 rounding of a probability shows: the elementwise bound is relaxed by 2, the norm-wise
    error still has to meet 2e-2."""
    rng = np.random.default_rng(16 * 1024 + 128 + kmode)
    B, H, T, D = 1, 16, 1024, 128
    n = B * H * T
    q, k, v = (rnd(rng, (n, D), BF16) for _ in range(3))
    want_hm = oracle.port().attention_core(q, k, v, B * H, T, D, True, BF16, kmode)
    want = np.ascontiguousarray(want_hm.reshape(B, H, T, D).transpose(0, 2, 1, 3)).reshape(B * T, H * D)
    out = empty_dev((B * T, H * D), BF16)
    assert ctx.attention_workspace_bytes(B, H, T, D, BF16) == 0  # the fused kernel takes this shape
    import torch
    ws = torch.empty(16, dtype=torch.uint8, device="cuda")
    ctx.attention(to_dev(q, BF16), to_dev(k, BF16), to_dev(v, BF16), out, B, H, T, D, True, kmode, BF16, ws, 0)
    ctx.check()
    assert_close(to_host(out), want, BF16, what="attention 1x16x1024x128", worst_cap=2.0)


@pytest.mark.parametrize("n", [4096, 8192])
@pytest.mark.parametrize("dtype", [BF16, F32])
def test_linear_sweep_large_sizes_sampled_rows(ctx, n, dtype):
    """Y = GELU(X.W + b) with M = N = K = n at the two large sizes of the linear-operator sweep:
    the whole product runs on the GPU, and sampled rows (tile borders, first and last) are compared
    with the CPU checker's own chain for that dtype — double accumulation and per-op rounding for
    bfloat16, the sequential float sum for float32 (the tensor-core float32 path is float32-class,
    not bit-identical: 1e-4 relative)."""
    rng = np.random.default_rng(n + dtype)
    x = rnd(rng, (n, n), dtype, 1.0 / np.sqrt(n))  # X and W ~ N(0, 1/K), b ~ N(0, 0.02)
    w = rnd(rng, (n, n), dtype, 1.0 / np.sqrt(n))
    b = rnd(rng, (n,), dtype, 0.02)
    got = dev_linear(ctx, x, w, b, dtype, "gelu")
    rows = [0, 127, 128, 255, 256, n // 2 - 1, n // 2, n - 129, n - 128, n - 1]
    want = oracle.port().linear(x[rows], w, b, dtype, "gelu")
    assert_close(got[rows], want, dtype, what=f"linear sweep n={n}")
    assert np.isfinite(oracle.as_float(got, dtype)).all()


def test_memset_and_to_contiguous(ctx):
    """Backend::memset and Backend::to_contiguous on the device: byte fill; the head split permute
    [B,T,H,D] -> [B,H,T,D] for 2- and 4-byte elements (vector path), a transpose that breaks the
    inner contiguity (scalar path), a 6-D view with an offset, and 1- and 8-byte elements."""
    import torch
    t = torch.full((1000,), 7, dtype=torch.uint8, device="cuda")
    ctx.memset(t[8:], 0xAB, 900)
    ctx.check()
    h = t.cpu().numpy()
    assert (h[:8] == 7).all() and (h[8:908] == 0xAB).all() and (h[908:] == 7).all()

    rng = np.random.default_rng(12)
    B, T, H, D = 2, 24, 3, 16
    for np_dt, es in ((np.uint16, 2), (np.float32, 4), (np.uint8, 1), (np.float64, 8)):
        src = (rng.standard_normal((B, T, H, D)) * 50).astype(np_dt)
        view = src.transpose(0, 2, 1, 3)
        strides = [s // es for s in view.strides]
        d_src = torch.from_numpy(src.view(np.uint8).reshape(-1)).cuda()
        d_dst = torch.empty(src.nbytes, dtype=torch.uint8, device="cuda")
        ctx.to_contiguous(d_src, d_dst, list(view.shape), strides, 0, es)
        ctx.check()
        assert np.array_equal(d_dst.cpu().numpy().view(np_dt).reshape(view.shape), np.ascontiguousarray(view))
        tr = src.reshape(B * T, H * D).T  # inner stride != 1
        ctx.to_contiguous(d_src, d_dst, list(tr.shape), [s // es for s in tr.strides], 0, es)
        ctx.check()
        assert np.array_equal(d_dst.cpu().numpy().view(np_dt).reshape(tr.shape), np.ascontiguousarray(tr))
    base = rng.standard_normal(5000).astype(np.float32)
    shape, strides, off = [2, 3, 2, 2, 3, 4], [1200, 400, 100, 40, 8, 1], 17
    want = np.lib.stride_tricks.as_strided(base[off:], shape=shape, strides=[4 * s for s in strides])
    d_src = torch.from_numpy(base).cuda()
    d_dst = torch.empty(int(np.prod(shape)), dtype=torch.float32, device="cuda")
    ctx.to_contiguous(d_src, d_dst, shape, strides, off, 4)
    ctx.check()
    assert np.array_equal(d_dst.cpu().numpy().reshape(shape), np.ascontiguousarray(want))
    import munet_b200 as mb
    with pytest.raises(mb.MuNetError, match="at most 6"):
        ctx.to_contiguous(d_src, d_dst, [1] * 7, [1] * 7, 0, 4)


def test_kernel_timer_brackets_device_time(ctx):
    """get_last_kernel_time_us: the event pair around a GEMM reports a positive device time, and a
    larger GEMM takes longer than a small one."""
    rng = np.random.default_rng(2)
    times = []
    for n in (256, 4096):
        x, w = to_dev(rnd(rng, (n, n), BF16), BF16), to_dev(rnd(rng, (n, n), BF16, 0.02), BF16)
        y = empty_dev((n, n), BF16)
        ctx.linear(x, w, None, y, n, n, n, BF16)  # warm-up
        ctx.timer_begin()
        ctx.linear(x, w, None, y, n, n, n, BF16)
        ctx.timer_end()
        times.append(ctx.timer_last_us())
        ctx.check()
    assert 0.0 < times[0] < times[1]


@pytest.mark.parametrize("M,K,N", [(2304, 320, 1100), (8192, 256, 2048)])
def test_linear_bf16_every_tile_shape_gives_the_same_bits(ctx, M, K, N):
    """The GEMM picks its tile from the problem size (128 x 64/128/256 on one CTA, 256 x 128/256 on
    a CTA pair). Every shape sums each output element in the same order, so forcing each of them
    must reproduce the automatic choice bit for bit — ragged edges, bias, GELU and residual
    included — and that result must match the checker."""
    rng = np.random.default_rng(M + N)
    x, w = rnd(rng, (M, K), BF16), rnd(rng, (K, N), BF16, 1.0 / np.sqrt(K))
    b, r = rnd(rng, (N,), BF16, 0.05), rnd(rng, (M, N), BF16)
    auto = dev_linear(ctx, x, w, b, BF16, "gelu", res=r)
    rows = [0, 127, 128, 255, 256, M // 2, M - 129, M - 1]
    P = oracle.port()
    assert_close(auto[rows], P.add(P.linear(x[rows], w, b, BF16, "gelu"), r[rows], BF16), BF16, what="auto tile")
    try:
        for bn, ctas in ((64, 1), (128, 1), (256, 1), (128, 2), (256, 2)):
            ctx.set_gemm_tile(bn, ctas)
            got = dev_linear(ctx, x, w, b, BF16, "gelu", res=r)
            assert np.array_equal(got, auto), f"tile {bn} x {ctas} CTA differs from the automatic choice"
    finally:
        ctx.set_gemm_tile(0, 0)
    import munet_b200 as mb
    with pytest.raises(mb.MuNetError):
        ctx.set_gemm_tile(64, 2)
