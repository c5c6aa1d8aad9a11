"""The C-ABI library loads without a GPU and exports exactly what include/fastmoe_b200.h
declares; argument validation answers before any CUDA call."""

import ctypes
import re
from pathlib import Path

import pytest

from fastmoe_b200 import _lib

HEADER = Path(__file__).resolve().parent.parent / "include" / "fastmoe_b200.h"


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(fmoe_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree():
    names = declared_functions()
    assert len(names) >= 15
    assert sorted(_lib.SIGNATURES) == names


def test_every_declared_symbol_is_exported():
    handle = _lib.lib()
    for name in declared_functions():
        assert hasattr(handle, name), f"{name} is declared but not exported"
    assert handle.fmoe_abi_version() == 2
    assert handle.fmoe_status_name(-3) == b"FMOE_ERR_WORKSPACE"


def test_size_queries_need_no_gpu():
    handle = _lib.lib()
    small = handle.fmoe_combine_plan_bytes(10, 5)
    big = handle.fmoe_combine_plan_bytes(65536, 8192)
    assert 0 < small < big and big % 256 == 0
    assert handle.fmoe_build_index_bytes(16384, 256, 8) >= 16384 // 32 * 256 * 4
    sizes = (ctypes.c_int64 * 3)(4, 0, 2)
    assert handle.fmoe_combine_host_arena_bytes(sizes, 3, 6, 5, 64, _lib.FMOE_BF16) > 6 * 64 * 2


def test_argument_errors_are_reported_without_launching():
    with pytest.raises(ValueError, match="bad dtype"):
        _lib.call("fmoe_combine_gather", None, None, 1, 1, 1, 1, 7, 0, None)
    with pytest.raises(ValueError, match="plan is null"):
        _lib.call("fmoe_combine_gather", None, None, 8, 1, 1, 8, _lib.FMOE_F32, 0, None)
    with pytest.raises(ValueError, match="K=9 exceeds E=8"):
        _lib.call("fmoe_route_topk", None, 0, 4, 8, 9, None, None, 0, None)
    with pytest.raises(ValueError, match="unknown key"):
        _lib.tune("no_such_knob", 1)
    assert b"unknown key" in _lib.lib().fmoe_last_error()
    # empty problems succeed without touching the device
    assert _lib.call("fmoe_combine_scatter", None, None, None, None, 0, None, 0, None, 0, 0, 0, 0, 0, 0, None, None) == 0
    assert _lib.call("fmoe_permute_fwd", None, 0, None, None, 0, 2, 8, _lib.FMOE_BF16, None) == 0
