"""ft_decode_static_scratch: the decode entry point that brings its own scratch.

Some callers of the library cannot hand it mid_o / mid_lse buffers: a serving
worker that gave all free device memory to its KV pool at start-up cannot count
on a later allocation, and a decode loop cannot afford the device-wide stall of
cudaMalloc / cudaFree.  For them the library keeps a fixed 16 MiB device array
and this entry point routes the partial results through it.

The test drives the entry point through the C ABI exactly as such a caller
would (NULL scratch pointers in the argument struct) and requires the output to
equal the regular ft_decode output - same kernels, same plan, so the tolerance
is the suite's 16-bit bound and in practice zero - on two calls in a row, the
second on new inputs so that stale partials of the first call would be noticed.
The file is named so that pytest collects it last.
"""
import ctypes

import pytest
import torch

import cases
import gpu_utils
from ft_b200 import engine, lib

pytestmark = pytest.mark.gpu

ATOL16 = 2e-3


def _args_without_scratch(run, o):
    a = engine.build_args(run.q, run.k, run.v, o, *run.aux, run.tiles[0], run.tiles[1], run.scale)
    a.mid_o = None              # the caller has no scratch to offer
    a.mid_lse = None
    a.mid_o_stride0 = a.mid_o_stride1 = a.mid_lse_stride0 = 0
    return a


def test_static_scratch_entry_point_matches_ft_decode_twice():
    handle = lib.load()
    c = cases.build_decode_case("rand3_fp16")
    run = gpu_utils.EngineRun(c["nodes"], c["ptrs"], c["batch"], c["q"], c["k"], c["v"], c["hq"], c["hkv"],
                              c["d"], c["tsq"], planner="b200")
    o_static = torch.empty_like(run.q)
    for attempt in range(2):
        if attempt == 1:                                   # new inputs for the second call
            g = torch.Generator(device="cuda").manual_seed(99)
            run.q = torch.randn(run.q.shape, generator=g, device="cuda").to(run.q.dtype)
            run.v = torch.randn(run.v.shape, generator=g, device="cuda").to(run.v.dtype)
        want = run.decode(path="auto")                     # regular entry point, caller-owned scratch
        o_static.fill_(float("nan"))
        a = _args_without_scratch(run, o_static)
        rc = handle.ft_decode_static_scratch(ctypes.byref(a))
        assert rc == 0, handle.ft_last_error()
        torch.cuda.synchronize()
        assert lib.read_device_status() == 0
        got = o_static.float().cpu()
        assert torch.isfinite(got).all()
        assert (got - want).abs().max().item() <= ATOL16, attempt


def test_static_scratch_rejects_plans_beyond_its_capacity():
    handle = lib.load()
    c = cases.build_decode_case("mini3_fp16")
    run = gpu_utils.EngineRun(c["nodes"], c["ptrs"], c["batch"], c["q"], c["k"], c["v"], c["hq"], c["hkv"],
                              c["d"], c["tsq"], planner="b200")
    a = _args_without_scratch(run, torch.empty_like(run.q))
    a.num_partial_rows = lib.FT_STATIC_SCRATCH_BYTES // (4 * c["hq"] * (c["d"] + 1)) + 1
    assert handle.ft_decode_static_scratch(ctypes.byref(a)) == -5          # FT_ERR_TOO_LARGE
    assert b"ft_decode" in handle.ft_last_error()
    assert handle.ft_decode_static_scratch(None) == -1
