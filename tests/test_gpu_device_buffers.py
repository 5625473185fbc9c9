"""Device buffers that peers open through CUDA IPC (shmt_dev_alloc)."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_shared_buffers_are_whole_2mb_pages():
    """A peer maps an allocation whose size is not a multiple of 2 MB with small pages (random
    row reads from a buffer of several GB then run 10-20x slower), so the allocation behind
    shmt_dev_alloc is always whole 2 MB pages, whatever size was asked for."""
    from cuda.bindings import driver
    from shmtensor_b200._lib import check, lib
    torch.zeros(1, device="cuda")
    for want in (16, (2 << 20) - 512, (2 << 20), 3 * (2 << 20) + 512, 22_200_002 * 512 // 64):
        out = C.c_void_p()
        check(lib.shmt_dev_alloc(want, C.byref(out)))
        err, base, size = driver.cuMemGetAddressRange(out.value)
        assert int(err) == 0 and int(base) == out.value
        assert size >= want and size % (2 << 20) == 0
        # the handle of the rounded allocation can be taken (what share_device_buffer does)
        handle = (C.c_char * 64)()
        check(lib.shmt_ipc_get_handle(out.value, handle))
        check(lib.shmt_dev_free(out.value))
