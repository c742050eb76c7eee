"""munet_b200 — B200 (sm_100a) forward-inference backend for MuNet models.

The compute lives in ``lib/libmunet_b200.so`` (hand-written CUDA, C ABI declared
in ``include/munet_b200.h``).  This package is the Python-side binding of that
ABI plus the host mirror of the reference's inference interface; importing it
never falls back to another implementation: if the native library is missing,
loading fails with an error that says how to build it.
"""
from ._lib import (  # noqa: F401
    ACT, BF16, F32, I32, K_LITERAL, K_MATH, Comm, Context, MuNetError, lib, lib_path,
)

__all__ = ["ACT", "BF16", "F32", "I32", "K_LITERAL", "K_MATH", "Comm", "Context", "MuNetError", "lib",
           "lib_path"]
