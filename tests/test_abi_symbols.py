"""The shared library builds, loads and exports every symbol include/b200dsa.h declares
(no compute calls: this runs without a GPU)."""
import os
import re

from transarch_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200dsa.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200dsa_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_exports_header_symbols():
    build.build()
    lib = _lib.load()
    names = declared_symbols()
    assert "b200dsa_topk_select" in names
    for n in names:
        assert hasattr(lib, n), f"{n} declared in b200dsa.h but not exported"
    assert set(names) == set(_lib.SIGNATURES), "ctypes signatures and header disagree"
    assert lib.b200dsa_abi_version() >= 1


def test_argument_validation_rejects_without_launching():
    lib = _lib.load()
    # k out of range -> EINVAL before any CUDA call
    rc = lib.b200dsa_topk_select(1, 8, 1, 8, None, None, 0, 0, 1, None, 0, None, 0, 0, None, 0, 0, None, 1, None, 8, None)
    assert rc == -1
    assert b"topk_select" in lib.b200dsa_last_error()
