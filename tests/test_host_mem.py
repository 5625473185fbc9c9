"""Shared-memory and mmap'ed-.npy tensors, on the CPU (reference: example/test_shm_tensor.py,
example/test_disk_tensor.py)."""
import os
import subprocess
import sys
import textwrap
import uuid
from pathlib import Path

import numpy as np
import pytest
import torch

from conftest import load_golden

ROOT = Path(__file__).resolve().parent.parent


def test_shared_mem_life_cycle():
    from shmtensor_b200 import capi
    name = f"shmt_test_{uuid.uuid4().hex[:8]}"
    assert not capi.file_exist(name)
    ptr, fd = capi.create_shared_mem(name, 48)
    try:
        assert capi.file_exist(name)
        a = capi.open_shared_tensor(ptr, torch.int16, (2, 3, 4))
        a[:] = 1000
        ptr2, fd2 = capi.open_shared_mem(name, 48)
        b = capi.open_shared_tensor(ptr2, torch.int16, [2, 3, 4])
        assert torch.equal(a, b) and b.dtype == torch.int16 and tuple(b.shape) == (2, 3, 4)
        b[0, 0, 0] = -5
        assert a[0, 0, 0] == -5
        del b
        os.close(fd2)
    finally:
        del a
        capi.release_shared_mem(name, 48, ptr, fd)
    assert not capi.file_exist(name)
    with pytest.raises(RuntimeError, match="fail to open"):
        capi.open_shared_mem(name, 48)


@pytest.mark.parametrize("dtype", ["float64", "float32", "float16", "int64", "int32", "int16",
                                   "int8", "uint8"])
def test_disk_tensor_round_trip(tmp_path, dtype):
    from shmtensor_b200 import DiskTensor
    g = load_golden("npy_shm.json")["npy"]
    rng = np.random.default_rng(g["seed"])
    arr = (rng.standard_normal(g["shape"]) * 50).astype(dtype)
    path = str(tmp_path / "a.npy")
    np.save(path, arr)
    t = DiskTensor(path)
    assert torch.equal(t.tensor_, torch.from_numpy(arr))
    assert t.shape == torch.Size(g["shape"]) and t.dtype == torch.from_numpy(arr).dtype
    t.tensor_[0, 0, 0] = 3  # MAP_SHARED: writes reach the file
    del t
    assert np.load(path)[0, 0, 0] == 3


def test_disk_tensor_rejects_what_the_reference_rejects(tmp_path):
    from shmtensor_b200 import capi
    p = str(tmp_path / "f.npy")
    np.save(p, np.asfortranarray(np.ones((3, 4))))
    with pytest.raises(RuntimeError, match="fortran"):
        capi.open_mmap_tensor(p, False)
    p2 = str(tmp_path / "c.npy")
    np.save(p2, np.ones(3, dtype=np.complex64))
    with pytest.raises(RuntimeError, match="dtype"):
        capi.open_mmap_tensor(p2, False)
    with pytest.raises(RuntimeError, match="Unable to open"):
        capi.open_mmap_tensor(str(tmp_path / "missing.npy"), False)
    (tmp_path / "junk.npy").write_bytes(b"not an npy file at all")
    with pytest.raises(RuntimeError, match="magic"):
        capi.open_mmap_tensor(str(tmp_path / "junk.npy"), False)


def test_npy_v2_header(tmp_path):
    from shmtensor_b200 import capi
    arr = np.arange(24, dtype=np.int32).reshape(4, 6)
    p = str(tmp_path / "v2.npy")
    with open(p, "wb") as f:
        np.lib.format.write_array(f, arr, version=(2, 0))
    t, size, ptr, fd = capi.open_mmap_tensor(p, False)
    assert torch.equal(t, torch.from_numpy(arr))
    del t
    capi.close_mmap_tensor(size, ptr, fd, False)


WORKER = textwrap.dedent("""
    import sys, torch, torch.distributed as dist
    sys.path.insert(0, {root!r})
    from shmtensor_b200 import ShmTensor
    dist.init_process_group(backend='gloo', init_method='env://')
    t = ShmTensor({name!r}, (2, 3, 4), dist.get_rank(), dist.get_world_size(), None, torch.int16)
    if dist.get_rank() == 0:
        t.tensor_[:] = 1000
    dist.barrier()
    assert (t.tensor_ == 1000).all(), t.tensor_
    assert t.shape == torch.Size([2, 3, 4]) and t.dtype == torch.int16
    dist.barrier()
    del t
    print('rank', dist.get_rank(), 'ok')
""")


def test_shm_tensor_two_ranks_gloo(tmp_path):
    """Rank 0 writes through the segment, rank 1 reads it (example/test_shm_tensor.py)."""
    name = f"shmt_test_{uuid.uuid4().hex[:8]}"
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(root=str(ROOT), name=name))
    port = 29500 + os.getpid() % 2000
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), OMP_NUM_THREADS="1")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=120)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)
    from shmtensor_b200 import capi
    assert not capi.file_exist(name)  # the creator unlinked it


def test_shm_tensor_refuses_a_taken_name():
    from shmtensor_b200 import ShmTensor, capi
    name = f"shmt_test_{uuid.uuid4().hex[:8]}"
    ptr, fd = capi.create_shared_mem(name, 16)
    try:
        with pytest.raises(Exception, match="already exist"):
            ShmTensor(name, (4,), 0, 1)
        with pytest.raises(Exception, match="Invalid shape"):
            ShmTensor(name + "x", (0,), 0, 1)
    finally:
        capi.release_shared_mem(name, 16, ptr, fd)
