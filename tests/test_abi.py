"""The C-ABI shared library builds for sm_100a, loads without a GPU and exports
every function the public header declares.  No compute calls here."""
import ctypes
import os
import re

import pytest

from ft_b200 import build, lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "fasttree_b200.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ft_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_functions()
    for must in ("ft_decode", "ft_stage1", "ft_stage2", "ft_bump_kv_lens", "ft_last_error"):
        assert must in names
    assert set(names) == set(lib.EXPORTS), "binding and header disagree on the exported functions"


def test_library_builds_loads_and_exports_all_symbols():
    build.build_library()
    handle = lib.load()
    for name in declared_functions():
        assert hasattr(handle, name), f"{name} is declared in the header but not exported"
    assert handle.ft_version() >= 100
    assert handle.ft_decode_args_size() == ctypes.sizeof(lib.DecodeArgs)


def test_null_and_invalid_arguments_return_error_codes():
    handle = lib.load()
    assert handle.ft_decode(None) == -1
    assert b"NULL" in handle.ft_last_error()
    args = lib.DecodeArgs()
    args.dtype = 7
    assert handle.ft_stage1(ctypes.byref(args)) == -1
    args.dtype = lib.FT_F16
    args.batch, args.num_qo_heads, args.num_kv_heads, args.head_dim = 1, 6, 4, 128
    assert handle.ft_stage2(ctypes.byref(args)) == -1          # 6 query heads over 4 kv heads
    args.num_qo_heads = 8
    args.head_dim = 96
    assert handle.ft_stage1(ctypes.byref(args)) == -2          # unsupported head_dim
    with pytest.raises(lib.FastTreeError):
        lib.check(-2)
    assert handle.ft_bump_kv_lens(None, None, -1, None) == -1
    assert handle.ft_bump_kv_lens(None, None, 0, None) == 0
    # the grouped-tails calls: nothing to do is fine, missing tables and negative sizes are refused before any launch
    assert handle.ft_gather_kv_entries(None, 0, None, None, None, None, 0, None, 0, None) == 0
    assert handle.ft_gather_kv_entries(None, 0, None, None, None, None, 3, None, 0, None) == -1
    assert handle.ft_gather_kv_entries(None, -1, None, None, None, None, 0, None, 0, None) == -1
    assert handle.ft_bump_tails(None, 0, None, 0, None, 0, None) == 0
    assert handle.ft_bump_tails(None, 2, None, 0, None, 0, None) == -1
    assert handle.ft_refresh_tails(None, 0, None, 0, None, 0, None) == 0
    assert handle.ft_refresh_tails(None, 2, None, 0, None, 0, None) == -1
    assert handle.ft_refresh_tails(None, 0, None, -5, None, 0, None) == -1
