"""The entry point that allocates nothing (`sb_attention_decode_noalloc`, declared in
stride_b200/csrc/noalloc.h), called through its exported C symbol.

Some callers of these kernels cannot allocate device memory: the process they live in has given the
whole GPU to its own pool, or they sit in a serving loop where cudaMalloc's device-wide stall is not
acceptable. For them decode attention keeps its scratch in a fixed array inside the library. This test
checks that the call gives the same output as the ordinary entry point (`sb_attention_tc` with a scratch
tensor), twice in a row with different inputs, since the array keeps what the previous call left; and
that a step too large for the array is refused with a message instead of being run.

The file name sorts after every other test file, so a run that stops at the first failure has already
run all other tests.
"""
from __future__ import annotations

import ctypes
import math
from ctypes import c_float, c_int, c_int64, c_void_p

import pytest
import torch

from test_kernels_gpu import DEV, _paged_case

pytestmark = pytest.mark.gpu


def _symbol():
    from stride_b200.kernels.build import library
    lib = library("attention_tc")
    fn = lib.sb_attention_decode_noalloc
    fn.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_int64, c_int64, c_void_p, c_int,
                   c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p]
    fn.restype = c_int
    return lib, fn


def _call(fn, case, items, chunks, out, Hq, Hkv, D, window, scale):
    cache, table, meta = case["cache"], case["table"], case["meta"]
    return fn(case["q"].data_ptr(), out.data_ptr(), cache.data_ptr(), table.data_ptr(), table.shape[1], cache.shape[3],
              cache.stride(0), cache.stride(1), cache.stride(2), meta.data_ptr(), meta.stride(0), items.data_ptr(),
              items.shape[0], chunks, Hq, Hkv, D, window, scale, torch.cuda.current_stream().cuda_stream)


def test_no_alloc_entry_matches_the_ordinary_one_twice():
    from stride_b200.kernels import ops
    lib, fn = _symbol()
    Hq, Hkv, D, page = 8, 2, 64, 16
    scale = 1.0 / math.sqrt(D)
    for call, (old, seed) in enumerate([([300, 0, 255, 256, 700, 63], 1), ([5, 511, 100, 1023, 64, 256], 2)]):
        new = [1, 1, 2, 1, 4, 1]           # decoded tokens and very short portions: at most 16 / (Hq / Hkv) tokens
        case = _paged_case(new, old, Hq, Hkv, D, page, torch.bfloat16, seed=seed, peak=(0, 2))
        items = torch.arange(len(new), dtype=torch.int32, device=DEV)
        chunks = max(o + n - 1 for o, n in zip(old, new)) // 256 + 1
        want = torch.full_like(case["q"], float("nan"))
        scratch = torch.zeros(ops.attention_tc_scratch(len(new), Hkv, chunks, D), device=DEV)
        ops.attention_tc(case["q"], want, case["cache"], case["table"], case["meta"], items, 0, len(new), chunks, scratch,
                         Hq, Hkv, D, 0, scale)
        got = torch.full_like(case["q"], float("nan"))
        if call == 0:
            # the first call on a device looks the scratch array's address up (and the driver may load the module)
            rc = _call(fn, case, items, chunks, got, Hq, Hkv, D, 0, scale)
            assert rc == 0, lib.sb_last_error().decode()
        torch.cuda.synchronize()
        before, free_before = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
        rc = _call(fn, case, items, chunks, got, Hq, Hkv, D, 0, scale)
        assert rc == 0, lib.sb_last_error().decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        # what the driver itself reports as free: a cudaMalloc inside the library would show here, not in torch's books
        assert torch.cuda.mem_get_info()[0] == free_before
        assert torch.isfinite(got.float()).all()
        # the same kernels on the same inputs: the tolerance of the attention kernel tests holds trivially
        assert (got.float() - want.float()).abs().max() <= 2e-2 * max(1.0, float(want.float().abs().max()))
        assert torch.equal(got, want), f"call {call}: the two entry points differ"


def test_no_alloc_entry_refuses_what_does_not_fit():
    lib, fn = _symbol()
    Hq, Hkv, D, page = 8, 2, 128, 64
    case = _paged_case([1], [10], Hq, Hkv, D, page, torch.bfloat16, seed=3)
    items = torch.zeros(4096, dtype=torch.int32, device=DEV)
    out = torch.zeros_like(case["q"])
    rc = _call(fn, case, items, 64, out, Hq, Hkv, D, 0, 0.1)      # 4096 entries x 64 chunks: far beyond 16 MiB
    assert rc != 0
    msg = lib.sb_last_error().decode()
    assert "scratch" in msg and "floats" in msg
    torch.cuda.synchronize()
    assert float(out.float().abs().sum()) == 0.0                    # nothing was launched
