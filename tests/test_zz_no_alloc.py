"""The allocation-free scan entry point against the regular one.

Some callers cannot allocate device memory where they need a prefix sum: a plugin inside an
application that owns every byte of device memory, or a serving loop that must never reach
the CUDA allocator (cudaMalloc stalls the device).  ``shmt_scan_static`` keeps its look-back
state in a fixed array inside the library instead of context scratch.
This file checks, through the C-ABI, that it returns exactly what ``shmt_scan`` returns —
integer prefix sums are bit-exact, so the tolerance is zero — on two calls in a row (the
array keeps the previous call's state, which the second call must clear), and that it
refuses inputs beyond its fixed limit.  Named to be collected last.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

LIMIT = 1 << 24


def _scan_static(lib, t, exclusive):
    code = {torch.int32: 0, torch.int64: 1}[t.dtype]
    return lib.shmt_scan_static(t.data_ptr(), code, t.numel(), int(exclusive),
                                torch.cuda.current_stream().cuda_stream)


def _scan_regular(lib, ctx, t, exclusive):
    code = {torch.int32: 0, torch.int64: 1}[t.dtype]
    return lib.shmt_scan(ctx, t.data_ptr(), code, t.numel(), int(exclusive),
                         torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("dtype", [torch.int32, torch.int64])
def test_static_scan_equals_regular_scan_twice_in_a_row(dtype):
    from shmtensor_b200 import _lib
    lib = _lib.lib
    torch.cuda.set_device(0)
    ctx = C.c_void_p()
    _lib.check(lib.shmt_ctx_create(0, C.byref(ctx)))
    try:
        g = torch.Generator(device="cuda").manual_seed(11)
        # second call is smaller than the first, so stale tile flags of the first would
        # break it if they were not cleared; the third is larger again
        for n, exclusive in ((3_000_001, False), (70_003, True), (5_000_000, False)):
            src = torch.randint(-1000, 1000, (n,), generator=g, device="cuda").to(dtype)
            a, b = src.clone(), src.clone()
            _lib.check(_scan_static(lib, a, exclusive))
            _lib.check(_scan_regular(lib, ctx, b, exclusive))
            # no bounded wait ran out (the check also waits for the stream)
            _lib.check(lib.shmt_scan_static_check(torch.cuda.current_stream().cuda_stream))
            assert torch.equal(a, b), f"n={n} exclusive={exclusive}"
            want = torch.cumsum(src.to(torch.int64), 0)
            if exclusive:
                want = want - src
            assert torch.equal(a, want.to(dtype))
    finally:
        lib.shmt_ctx_destroy(ctx)


def test_static_scan_limit_and_arguments():
    from shmtensor_b200 import _lib, capi
    lib = _lib.lib
    torch.cuda.set_device(0)
    big = torch.ones(LIMIT + 1, dtype=torch.int32, device="cuda")
    assert _scan_static(lib, big, False) == _lib.ERR_INVALID
    assert "exceed the fixed scratch" in _lib.last_error()
    assert (big == 1).all()                       # refused means untouched
    ok = big[:LIMIT]
    _lib.check(_scan_static(lib, ok, False))      # exactly at the limit
    torch.cuda.synchronize()
    assert ok[-1].item() == LIMIT and ok[12345].item() == 12346
    assert lib.shmt_scan_static(None, 0, 5, 0, None) == _lib.ERR_INVALID
    assert lib.shmt_scan_static(None, 7, 0, 0, None) == _lib.ERR_INVALID
    assert lib.shmt_scan_static(None, 0, 0, 0, None) == _lib.OK      # empty input: nothing to do
    t = torch.arange(1, 1001, dtype=torch.int64, device="cuda")
    capi.scan_static_(t)                          # the Python wrapper takes the same route
    assert t[-1].item() == 500500
