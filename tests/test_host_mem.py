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


def test_exclusive_create_and_unlink():
    from shmtensor_b200 import capi
    from shmtensor_b200._lib import ERR_OS, ShmtError
    name = f"shmt_test_{uuid.uuid4().hex[:8]}"
    ptr, fd = capi.create_shared_mem(name, 4096, exclusive=True)
    try:
        with pytest.raises(ShmtError, match="already exists") as err:
            capi.create_shared_mem(name, 4096, exclusive=True)
        assert err.value.code == ERR_OS
        p2, fd2 = capi.create_shared_mem(name, 4096)      # the reference's create: opens what is there
        capi.open_shared_tensor(ptr, torch.int32, (4,))[:] = 7
        assert capi.open_shared_tensor(p2, torch.int32, (4,)).tolist() == [7, 7, 7, 7]
    finally:
        capi.release_shared_mem(name, 4096, ptr, fd)
    assert not capi.file_exist(name)
    capi.unlink_shared_mem(name)                          # absent name: not an error


def test_shm_tensor_overwrites_a_stale_segment_when_asked():
    from shmtensor_b200 import ShmTensor, capi
    name = f"shmt_test_{uuid.uuid4().hex[:8]}"
    ptr, fd = capi.create_shared_mem(name, 64)            # what a killed run leaves behind
    capi.open_shared_tensor(ptr, torch.int64, (8,))[:] = -5
    t = ShmTensor(name, (8,), 0, 1, None, torch.int64, overwrite_stale=True)
    assert (t.tensor_ == 0).all()                         # a new segment, not the old bytes
    t.tensor_[:] = 3
    assert capi.open_shared_tensor(ptr, torch.int64, (8,)).tolist() == [-5] * 8
    del t
    assert not capi.file_exist(name)
    import ctypes as C
    from shmtensor_b200._lib import lib                   # drop the stale mapping (name already gone)
    C.CDLL(None).munmap(C.c_void_p(ptr), C.c_size_t(64))
    os.close(fd)


def test_numa_placement_of_a_fresh_segment():
    from shmtensor_b200 import ShmTensor, capi
    assert capi.numa_nodes() >= 1
    name = f"shmt_test_{uuid.uuid4().hex[:8]}"
    t = ShmTensor(name, (1 << 20,), 0, 1, None, torch.float32, numa="interleave")
    t.tensor_[:] = 1.5
    assert float(t.tensor_.sum()) == 1.5 * (1 << 20)
    del t
    u = ShmTensor(name, (1 << 20,), 0, 1, None, torch.float32, numa=0)
    u.tensor_[:] = 2.0
    assert float(u.tensor_[-1]) == 2.0
    del u
    with pytest.raises(Exception, match="holds no memory"):
        ShmTensor(name, (1 << 20,), 0, 1, None, torch.float32, numa=977)
    capi.unlink_shared_mem(name)


def test_prefault_makes_a_fresh_segment_resident():
    from shmtensor_b200 import capi
    name = f"shmt_test_{uuid.uuid4().hex[:8]}"
    nbytes = 64 << 20
    ptr, fd = capi.create_shared_mem(name, nbytes, exclusive=True)
    try:
        capi.prefault(ptr, nbytes, 4)
        t = capi.open_shared_tensor(ptr, torch.uint8, (nbytes,))
        assert int(t.sum()) == 0                       # still all zeros, now present
        t[::4096] = 1
        assert int(t.sum()) == nbytes // 4096
    finally:
        capi.release_shared_mem(name, nbytes, ptr, fd)
    from shmtensor_b200._lib import ERR_INVALID, lib
    assert lib.shmt_host_prefault(None, 10, 1) == ERR_INVALID


def test_disk_tensor_read_only_and_bfloat16(tmp_path):
    from shmtensor_b200 import DiskTensor
    arr = np.arange(24, dtype=np.float32).reshape(2, 3, 4)
    path = str(tmp_path / "ro.npy")
    np.save(path, arr)
    os.chmod(path, 0o444)
    t = DiskTensor(path, read_only=True)                  # a file this process may not write
    assert torch.equal(t.tensor_, torch.from_numpy(arr))
    del t
    os.chmod(path, 0o644)
    # bfloat16 rows saved as opaque 2-byte items, the form numpy can carry them in
    rows = torch.randn(5, 8).to(torch.bfloat16)
    path2 = str(tmp_path / "bf16.npy")
    np.save(path2, rows.view(torch.int16).numpy().view("V2"))
    b = DiskTensor(path2)
    assert b.dtype == torch.bfloat16 and torch.equal(b.tensor_.view(torch.int16), rows.view(torch.int16))


TAKEN_WORKER = textwrap.dedent("""
    import sys, torch, torch.distributed as dist
    sys.path.insert(0, {root!r})
    from shmtensor_b200 import ShmTensor
    dist.init_process_group(backend='gloo', init_method='env://')
    try:
        ShmTensor({name!r}, (8,), dist.get_rank(), dist.get_world_size(), None, torch.int16)
    except Exception as exc:
        assert 'already exist' in str(exc), exc
        print('rank', dist.get_rank(), 'refused')
    else:
        raise SystemExit('a taken name was accepted')
    t = ShmTensor({name!r}, (8,), dist.get_rank(), dist.get_world_size(), None, torch.int16,
                  overwrite_stale=True)
    dist.barrier()
    del t
""")


def test_a_taken_name_fails_on_every_rank_instead_of_hanging(tmp_path):
    from shmtensor_b200 import capi
    name = f"shmt_test_{uuid.uuid4().hex[:8]}"
    ptr, fd = capi.create_shared_mem(name, 16)
    try:
        script = tmp_path / "worker.py"
        script.write_text(TAKEN_WORKER.format(root=str(ROOT), name=name))
        port = 31500 + os.getpid() % 2000
        procs = []
        for rank in range(2):
            env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1",
                       MASTER_PORT=str(port), OMP_NUM_THREADS="1")
            procs.append(subprocess.Popen([sys.executable, str(script)], env=env,
                                          stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
        outs = [p.communicate(timeout=120)[0] for p in procs]
        assert all(p.returncode == 0 for p in procs), "\n".join(outs)
        assert all("refused" in o for o in outs)
    finally:
        import ctypes as C
        C.CDLL(None).munmap(C.c_void_p(ptr), C.c_size_t(16))
        os.close(fd)
        capi.unlink_shared_mem(name)
