"""CPU-only: the backend plugin probe library exports the five symbols MuNet's loader
binds (src/backend/plugin_loader.cpp:101-176) with the values it checks, and MuNet's own
discovery code (compiled into oracle/_ref) finds and classifies it."""
import ctypes as C
import os

import pytest

import oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PLUGIN = os.path.join(ROOT, "munet_b200", "lib", "libmunet_backend_b200.so")


def test_probe_symbols_and_values():
    lib = C.CDLL(PLUGIN)
    lib.munet_backend_plugin_abi_version.restype = C.c_uint32
    lib.munet_backend_plugin_name.restype = C.c_char_p
    lib.munet_backend_plugin_device_type.restype = C.c_char_p
    lib.munet_backend_plugin_capability_flags.restype = C.c_uint64
    lib.munet_backend_plugin_probe.restype = C.c_char_p
    assert lib.munet_backend_plugin_abi_version() == 1
    assert lib.munet_backend_plugin_name() == b"b200"
    assert lib.munet_backend_plugin_device_type() == b"cuda"  # enables MuNet's CUDA slot
    assert lib.munet_backend_plugin_capability_flags() == 0x3F
    err = lib.munet_backend_plugin_probe()  # NULL = ok; otherwise a static reason string
    assert err is None or b"Missing runtime dependency" in err or b"ABI" in err


@pytest.mark.skipif(not oracle.have_ref_b200(), reason="oracle/_ref/libmunet_ref_b200.so not built")
def test_reference_loader_discovers_the_plugin(monkeypatch):
    monkeypatch.setenv("MUNET_BACKEND_PLUGIN_DIR", os.path.dirname(PLUGIN))
    active, report = oracle.RefB200().plugin_status()
    assert "b200|" in report
    # with a driver present the probe passes ("ok"); without one MuNet reports the missing dependency
    assert ("b200|ok|" in report) == active
    if not active:
        assert "b200|runtime_dependency_missing|" in report
