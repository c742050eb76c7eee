"""CPU-only: the C-ABI library loads and exports every symbol include/munet_b200.h
declares, and the ctypes table binds exactly that set. No compute is called."""
import ctypes as C
import os
import re

import munet_b200
from munet_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "munet_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mu_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_functions():
    names = declared_functions()
    assert "mu_linear" in names and "mu_engine_run" in names and len(names) >= 30


def test_library_exports_every_declared_symbol():
    handle = C.CDLL(munet_b200.lib_path())
    missing = [n for n in declared_functions() if not hasattr(handle, n)]
    assert not missing, f"declared but not exported: {missing}"


def test_ctypes_table_matches_header():
    assert sorted(_lib.SIGNATURES) == declared_functions()


def test_abi_version_and_no_fallback(tmp_path, monkeypatch):
    assert munet_b200.lib().mu_abi_version() == 1
    # a missing library must fail loudly, never fall back to another implementation
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "_HERE", str(tmp_path))
    try:
        _lib.lib()
    except ImportError as e:
        assert "no fallback" in str(e).lower()
    else:
        raise AssertionError("loading a missing library did not fail")
