"""GPU: the drop-in proof. The UNMODIFIED reference core (oracle/_ref) runs its own
inference::Engine on DeviceType::CUDA with munet_b200's Backend adapter registered, so
MuNet's own op front-ends and dispatcher call the B200 kernels through the C ABI."""
import os

import numpy as np
import pytest

import oracle
from oracle import BF16, F32
from tests.test_gpu_engine import mlp_artifact, mlp_oracle
from tests.util import assert_close

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not oracle.have_ref_b200(), reason="libmunet_ref_b200.so not built")]

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def ref_b200():
    r = oracle.RefB200()
    r.register()
    return r


def test_plugin_is_active_on_a_gpu_box(ref_b200, monkeypatch):
    monkeypatch.setenv("MUNET_BACKEND_PLUGIN_DIR", os.path.join(ROOT, "munet_b200", "lib"))
    active, report = ref_b200.plugin_status()
    assert active and "b200|ok|" in report, report


def test_reference_engine_runs_mlp_on_b200_backend_fp32(ref_b200, tmp_path):
    rng = np.random.default_rng(1001)
    path, tensors = mlp_artifact(tmp_path, rng, [784, 512, 512, 10], ["ReLU", "ReLU"])
    x = np.random.default_rng(2001).random((64, 784), dtype=np.float32)
    got = ref_b200.engine_run_npz(path, x, F32)
    want = mlp_oracle(x, tensors, ["ReLU", "ReLU"])
    # matmul and relu run on the B200 (bit-exact kernels), the bias add takes MuNet's CPU fallback
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_reference_engine_runs_mlp_on_b200_backend_bf16(ref_b200, tmp_path):
    rng = np.random.default_rng(7)
    path, tensors = mlp_artifact(tmp_path, rng, [256, 512, 128], ["GELU"])
    x = rng.standard_normal((128, 256)).astype(np.float32)
    got = ref_b200.engine_run_npz(path, x, BF16)
    bt = {k: oracle.to_bf16(v) for k, v in tensors.items()}
    h = oracle.port().linear(oracle.to_bf16(x), bt["0.weight"], bt["0.bias"], BF16, "gelu")
    want = oracle.from_bf16(oracle.port().linear(h, bt["2.weight"], bt["2.bias"], BF16))
    assert_close(got, want, F32, rtol=2e-2, what="reference Engine on B200Backend, bf16")


def test_reference_engine_runs_unet_style_block_on_b200_backend(ref_b200, tmp_path):
    """Conv2d → BatchNorm2d → LeakyReLU → Upsample → Conv2d → GlobalAvgPool2d → Flatten → RMSNorm
    through MuNet's own Engine with every op dispatched to the B200 backend (conv, batch-norm
    inference branch, relu/sub/mul/add of LeakyReLU, nearest upsample, the GAP matmul, mean,
    rsqrt): float32, compared with the same modules of the CPU checker."""
    from munet_b200.inference import save_deploy
    rng = np.random.default_rng(41)
    t = {
        "0.weight": (rng.standard_normal((8, 3, 3, 3)) * 0.3).astype(np.float32),
        "0.bias": (rng.standard_normal(8) * 0.1).astype(np.float32),
        "1.weight": rng.standard_normal(8).astype(np.float32),
        "1.bias": rng.standard_normal(8).astype(np.float32),
        "1.running_mean": (rng.standard_normal(8) * 0.2).astype(np.float32),
        "1.running_var": (rng.random(8) + 0.5).astype(np.float32),
        "4.weight": (rng.standard_normal((4, 8, 3, 3)) * 0.2).astype(np.float32),
        "4.bias": np.zeros(4, np.float32),
        "7.weight": rng.standard_normal(4).astype(np.float32),
    }
    cfg = {"type": "Sequential", "layers": [
        {"type": "Conv2d", "in_channels": 3, "out_channels": 8, "kernel_size": 3, "stride": 1, "padding": 1},
        {"type": "BatchNorm2d", "num_features": 8, "eps": 1e-5, "momentum": 0.1},
        {"type": "LeakyReLU", "negative_slope": 0.2},
        {"type": "Upsample", "scale_factor": 2},
        {"type": "Conv2d", "in_channels": 8, "out_channels": 4, "kernel_size": 3, "stride": 1, "padding": 1},
        {"type": "GlobalAvgPool2d"},
        {"type": "Flatten"},
        {"type": "RMSNorm", "normalized_shape": 4, "eps": 1e-5}]}
    path = str(tmp_path / "unet_block.npz")
    save_deploy(path, cfg, t)
    x = rng.random((2, 3, 10, 12), dtype=np.float32)
    P = oracle.port()
    h = P.conv2d(x, t["0.weight"], t["0.bias"], 1, 1)
    h = P.batch_norm_eval(h, t["1.weight"], t["1.bias"], t["1.running_mean"], t["1.running_var"], F32)
    h = P.leaky_relu(h, 0.2, F32).reshape(h.shape)
    h = np.repeat(np.repeat(h, 2, axis=2), 2, axis=3)
    h = P.conv2d(h, t["4.weight"], t["4.bias"], 1, 1)
    h = P.global_avg_pool(h).reshape(2, 4)
    want = P.rms_norm(h, t["7.weight"], F32)
    got = ref_b200.engine_run_npz(path, x, F32)
    assert got.shape == want.shape
    assert_close(got, want, F32, what="reference Engine on B200Backend, UNet-style block")


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("causal", [True, False])
def test_reference_mha_module_runs_on_b200_backend(ref_b200, dtype, causal):
    """The reference's own nn::MultiHeadAttention on the B200 backend: projections, the head split
    and merge permutes (device-side to_contiguous, 2- and 4-byte elements), the stride-ignoring
    score matmul (literal K addressing), scale, softmax and P.V — against the checker's module,
    which is pinned to the same module on the reference's CPU backend."""
    rng = np.random.default_rng(31 + dtype)
    B, T, E, H = 2, 24, 64, 4

    def r(shape, scale=1.0):
        a = (rng.standard_normal(shape) * scale).astype(np.float32)
        return a if dtype == F32 else oracle.to_bf16(a)
    params = []
    for _ in range(4):
        params += [r((E, E), 1.0 / np.sqrt(E)), r((E,), 0.05)]
    x = r((B, T, E))
    got, kernel_us = ref_b200.mha_forward(x, params, H, causal, dtype)
    want = oracle.port().mha(x, params, H, causal, dtype, kmode=oracle.K_LITERAL)
    assert_close(got, want, dtype, what="reference MultiHeadAttention on B200Backend")
    assert kernel_us > 0.0  # get_last_kernel_time_us reports the device time of the last op


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_all_reduce_through_the_adapter_matches_reduce_sum_bytes(ref_b200, dtype):
    """Tensor.all_reduce on the drop-in backend with two and three in-process participants (the
    reference's rendezvous, tests/test_backend_manager.cpp:1371-1397): every participant ends
    with the checker's sum (double accumulation, one rounding)."""
    rng = np.random.default_rng(33)
    for world in (2, 3):
        bufs = [(rng.standard_normal(257)).astype(np.float32) for _ in range(world)]
        if dtype == BF16:
            bufs = [oracle.to_bf16(b) for b in bufs]
        want = oracle.port().all_reduce_sum(bufs, dtype)
        for got in ref_b200.all_reduce_threads(bufs, dtype):
            assert np.array_equal(got, want)
    # the reference's known answer: [1,2] + [3,4] -> [4,6] on both
    a, b = ref_b200.all_reduce_threads([np.array([1, 2], np.float32), np.array([3, 4], np.float32)], F32)
    assert a.tolist() == [4.0, 6.0] and b.tolist() == [4.0, 6.0]
