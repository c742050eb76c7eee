"""Build the native libraries in-tree with nvcc for sm_100a.

    python -m munet_b200.build            # libmunet_b200.so (+ plugin probe)

The shared objects land in ``munet_b200/lib/`` next to the sources so that a
source snapshot carries them; nothing is installed into site-packages.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "lib")

NVCC_FLAGS = [
    "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC",
]

KERNEL_SOURCES = ["api.cu", "gemm_tcgen05.cu", "gemm_simt.cu", "rowwise.cu"]


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA extension cannot be built")
    return exe


def _stale(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    deps = list(sources)
    for d in (CSRC, os.path.join(HERE, "..", "include")):
        deps += [os.path.join(d, f) for f in os.listdir(d) if f.endswith((".h", ".cuh", ".hpp"))]
    return any(os.path.getmtime(s) > t for s in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(LIB, exist_ok=True)
    out = os.path.join(LIB, "libmunet_b200.so")
    srcs = [os.path.join(CSRC, s) for s in KERNEL_SOURCES if os.path.exists(os.path.join(CSRC, s))]
    extra = sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC)
                   if f.endswith(".cu") and os.path.join(CSRC, f) not in srcs)
    srcs += extra
    if force or _stale(out, srcs):
        objs = []
        procs = []
        objdir = os.path.join(LIB, "obj")
        os.makedirs(objdir, exist_ok=True)
        for s in srcs:
            o = os.path.join(objdir, os.path.basename(s)[:-3] + ".o")
            objs.append(o)
            if force or _stale(o, [s]):
                cmd = [nvcc(), *NVCC_FLAGS, "-c", s, "-o", o]
                if verbose:
                    cmd.insert(1, "-Xptxas")
                    cmd.insert(2, "-v")
                procs.append((s, subprocess.Popen(cmd)))
        for s, p in procs:
            if p.wait() != 0:
                raise RuntimeError(f"nvcc failed on {s}")
        subprocess.check_call([nvcc(), "-shared", "-o", out, *objs, "-Xcompiler", "-fPIC"])
    # MuNet plugin probe (plain C++, no CUDA link dependency)
    probe_src = os.path.join(CSRC, "plugin_probe.cpp")
    probe_out = os.path.join(LIB, "libmunet_backend_b200.so")
    if os.path.exists(probe_src) and (force or _stale(probe_out, [probe_src])):
        cxx = os.environ.get("CXX") or shutil.which("g++") or "g++"
        subprocess.check_call([cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-o", probe_out,
                               probe_src, "-ldl"])
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
