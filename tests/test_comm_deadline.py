"""GPU (one device): a participant that never joins an all-reduce. The reference waits
MUNET_ALLREDUCE_TIMEOUT_MS for every participant and then throws "all_reduce: timeout waiting for
participants" (src/core/all_reduce_runtime.hpp:205-225, tests/test_backend_manager.cpp:1399-1425).
Here the failure is made on the host: a stand-in for NCCL (tests/fake_nccl.cpp) whose collective
keeps the stream busy past the deadline — no kernel waits for anything. Runs in a child process
because the library binds NCCL once per process."""
import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = textwrap.dedent("""
    import ctypes, sys, time
    import torch
    import munet_b200 as mb
    fake = ctypes.CDLL(sys.argv[1])
    ctx = mb.Context(0)
    comm = mb.Comm(ctx, mb.Comm.new_unique_id(), 0, 2)      # "two ranks"; the other never shows up
    buf = torch.ones(1024, device="cuda")
    stream = torch.cuda.current_stream()
    ctx.all_reduce_sum(comm, buf, 1024, mb.F32)
    t0 = time.time()
    try:
        comm.wait(stream, timeout_ms=200)
    except mb.MuNetError as e:
        waited = time.time() - t0
        assert e.code == 4, e                               # MU_ERR_TIMEOUT
        assert "timeout waiting for participants" in str(e) and "200 ms" in str(e), e
        assert 0.15 < waited < 1.2, waited                  # gave up at the deadline, not at the end
    else:
        raise SystemExit("the deadline did not fire")
    assert fake.fake_nccl_reduces() == 1 and fake.fake_nccl_aborts() == 1   # ncclCommAbort ran
    for call in (lambda: ctx.all_reduce_sum(comm, buf, 1024, mb.F32), comm.check):
        try:
            call()
        except mb.MuNetError as e:
            assert "aborted" in str(e), e
        else:
            raise SystemExit("an aborted communicator was used again")
    torch.cuda.synchronize()                                # the stalled stream drains by itself
    assert float(buf.sum()) == 1024.0                       # the context is still usable
    y = torch.empty(8, 8, device="cuda")
    ctx.linear(torch.ones(8, 8, device="cuda"), torch.ones(8, 8, device="cuda"), None, y, 8, 8, 8, mb.F32)
    ctx.check()
    assert float(y.sum()) == 8 * 8 * 8
    # a collective that does finish in time passes the same deadline
    comm2 = mb.Comm(ctx, mb.Comm.new_unique_id(), 0, 2)
    ctx.all_reduce_sum(comm2, buf, 1024, mb.F32)
    comm2.wait(stream, timeout_ms=5000)
    comm2.close(); comm.close(); ctx.close()
    print("DEADLINE_OK")
""")


def test_missing_participant_hits_the_host_deadline(tmp_path):
    so = str(tmp_path / "libfake_nccl.so")
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    subprocess.check_call(["g++", "-O1", "-shared", "-fPIC", "-o", so, os.path.join(ROOT, "tests", "fake_nccl.cpp"),
                           f"-I{cuda}/include", f"-L{cuda}/lib64", "-lcudart", f"-Wl,-rpath,{cuda}/lib64"])
    env = dict(os.environ, MUNET_B200_NCCL_LIBRARY=so, FAKE_NCCL_STALL_MS="1500", PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-c", CHILD, so], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "DEADLINE_OK" in r.stdout, r.stdout + r.stderr
