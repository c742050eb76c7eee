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
