"""The allocation-free attention entry point against the regular one and against the CPU checker.

Collected last on purpose (file name): if it fails under ``-x`` every other test
has already run.  It goes through the C ABI only, needs no context object, and is
called twice in a row to show that what the first call left in the shared
built-in scratch does not leak into the second."""
import ctypes as C

import numpy as np
import pytest

import oracle
from oracle import BF16, F32
from tests.util import assert_close, empty_dev, rnd, to_dev, to_host

pytestmark = pytest.mark.gpu

SCRATCH_BYTES = 64 << 20


def call_static(lib, q, k, v, out, B, H, T, D, causal, kmode, dtype):
    import torch
    err = C.create_string_buffer(512)
    rc = lib.mu_attention_static_scratch(0, q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                                         B, H, T, D, int(causal), kmode, dtype,
                                         torch.cuda.current_stream().cuda_stream, 1, err, 512)
    return rc, err.value.decode()


@pytest.mark.parametrize("dtype,B,H,T,D", [(F32, 2, 2, 40, 16), (BF16, 2, 3, 64, 32), (BF16, 1, 2, 128, 64)])
@pytest.mark.parametrize("kmode", [oracle.K_LITERAL, oracle.K_MATH])
def test_static_scratch_matches_regular_entry_point(dtype, B, H, T, D, kmode):
    import torch
    import munet_b200 as mb
    lib = mb.lib()
    ctx = mb.Context(0)
    rng = np.random.default_rng(T + D)
    n = B * H * T
    outs = []
    for call in range(2):  # two calls in a row, different data, different causal flag
        causal = call == 0
        q, k, v = (to_dev(rnd(rng, (n, D), dtype), dtype) for _ in range(3))
        want = empty_dev((B * T, H * D), dtype)
        nbytes = max(ctx.attention_workspace_bytes(B, H, T, D, dtype), 16)
        ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        ctx.attention(q, k, v, want, B, H, T, D, causal, kmode, dtype, ws, nbytes)
        ctx.check()
        got = empty_dev((B * T, H * D), dtype)
        rc, msg = call_static(lib, q, k, v, got, B, H, T, D, causal, kmode, dtype)
        assert rc == 0, msg
        assert_close(to_host(got), to_host(want), dtype, what=f"static scratch call {call}")
        # and against the CPU checker, so that a fault shared by both entry points would show
        hm = oracle.port().attention_core(to_host(q), to_host(k), to_host(v), B * H, T, D, causal, dtype, kmode)
        ref = np.ascontiguousarray(hm.reshape(B, H, T, D).transpose(0, 2, 1, 3)).reshape(B * T, H * D)
        assert_close(to_host(got), ref, dtype, what=f"static scratch call {call} vs checker")
        outs.append(to_host(got))
    assert not np.array_equal(outs[0], outs[1])
    ctx.close()


def test_static_scratch_rejects_oversize():
    import munet_b200 as mb
    lib = mb.lib()
    t = empty_dev((16,), F32)
    B, H, T, D = 1, 1, 8192, 16  # 8192*8192*4 bytes = 256 MiB of scores
    assert B * H * T * T * 4 > SCRATCH_BYTES
    rc, msg = call_static(lib, t, t, t, t, B, H, T, D, True, 0, F32)
    assert rc == 7 and "exceed" in msg  # MU_ERR_SIZE, nothing was launched


def test_static_scratch_restores_the_callers_device():
    """The call selects the device it was asked for and puts the caller's current device back."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two visible devices")
    import munet_b200 as mb
    lib = mb.lib()
    rng = np.random.default_rng(5)
    B, H, T, D = 1, 2, 32, 16
    with torch.cuda.device(0):
        q, k, v = (to_dev(rnd(rng, (B * H * T, D), F32), F32) for _ in range(3))
        got = empty_dev((B * T, H * D), F32)
    torch.cuda.set_device(1)
    err = C.create_string_buffer(512)
    rc = lib.mu_attention_static_scratch(0, q.data_ptr(), k.data_ptr(), v.data_ptr(), got.data_ptr(),
                                         B, H, T, D, 1, 1, F32, None, 1, err, 512)
    assert rc == 0, err.value.decode()
    assert torch.cuda.current_device() == 1
    torch.cuda.set_device(0)
    hm = oracle.port().attention_core(to_host(q), to_host(k), to_host(v), B * H, T, D, True, F32, 1)
    ref = np.ascontiguousarray(hm.reshape(B, H, T, D).transpose(0, 2, 1, 3)).reshape(B * T, H * D)
    assert_close(to_host(got), ref, F32, what="static scratch from another current device")
