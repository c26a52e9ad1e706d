"""The C-ABI library builds for sm_100a, loads without a GPU, and exports exactly the entry points
that include/thrust_b200.h declares (no compute calls here)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "thrust_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\bint\s+(tb200_\w+)\s*\(", text)))


def test_header_declares_entry_points():
    syms = declared_symbols()
    for name in ("tb200_reduce", "tb200_inclusive_scan", "tb200_exclusive_scan", "tb200_sort_by_key", "tb200_copy_if",
                 "tb200_partition", "tb200_partition_copy", "tb200_unique_copy", "tb200_reduce_by_key", "tb200_merge_by_key",
                 "tb200_merge_sort_by_key"):
        assert name in syms


def test_library_exports_every_declared_symbol():
    from thrust_b200 import _lib, build
    build.build()
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared_symbols():
        assert hasattr(lib, name), "libthrust_b200.so does not export " + name
    assert set(declared_symbols()) == set(_lib.PROTOTYPES), "ctypes prototypes and header disagree"
    assert lib.tb200_sm_arch() == 100


def test_size_queries_need_no_gpu():
    """Workspace size queries are pure host arithmetic."""
    from thrust_b200 import _lib
    lib = _lib.load()
    need = ctypes.c_size_t(0)
    assert lib.tb200_reduce(None, 1 << 20, 4, 6, 0, None, None, None, ctypes.byref(need), None) == 0 and need.value >= 256
    assert lib.tb200_sort_by_key(None, None, None, None, 1 << 20, 5, 4, 0, 0, 32, None, ctypes.byref(need), None) == 0
    assert need.value > (1 << 20) // 8192 * 1024
    assert lib.tb200_reduce(None, 8, 8, 4, 0, None, None, None, ctypes.byref(need), None) == 801       # f32 -> i32 unsupported
    assert lib.tb200_sort_by_key(None, None, None, None, 8, 5, 3, 0, 0, 32, None, ctypes.byref(need), None) == 801    # 3-byte values
    assert lib.tb200_reduce(None, 8, 4, 6, 0, None, None, None, None, None) == 1                      # no size pointer


def test_missing_library_fails_loudly(monkeypatch):
    from thrust_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", os.path.join(ROOT, "thrust_b200", "no_such_library.so"))
    with pytest.raises(RuntimeError, match="no CPU or library fallback"):
        _lib.load()
