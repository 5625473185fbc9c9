"""The drop-in boundary: after ``install_dropin()`` the reference's import names resolve to this
package, and every function the reference's pybind module exports (src/pybind.cc:16-65) exists
with the same keyword names, so scripts written against ``ShmTensorLib`` / ``shmtensor`` run as
they are."""
import inspect

import numpy as np
import pytest
import torch

# name -> keyword names, as the reference's module defines them (src/pybind.cc:17-58)
REFERENCE_API = {
    "create_shared_mem": ["name", "size", "pin_memory"],
    "open_shared_mem": ["name", "size", "pin_memory"],
    "release_shared_mem": ["name", "size", "ptr", "fd", "pin_memory"],
    "open_shared_tensor": ["ptr", "dtype", "shape"],
    "file_exist": ["filename"],
    "open_mmap_tensor": ["filename", "pin_memory"],
    "close_mmap_tensor": ["size", "ptr", "fd", "pin_memory"],
    "thrust_scan": ["tensor"],
    "pin_memory": ["data"],
    "unpin_memory": ["data"],
    "uva_fetch": ["data", "indices"],
    "cache_fetch": ["uva_data", "gpu_data", "indices", "hashmap"],
    "cache_fetch_with_mask": ["uva_data", "gpu_data", "indices", "mask"],
    "uva_set": ["data", "indices", "update"],
    "cache_set": ["uva_data", "gpu_data", "indices", "update", "hashmap"],
    "cache_set_with_mask": ["uva_data", "gpu_data", "indices", "update", "mask"],
    "csr_sampling": ["indptr", "indices", "seeds", "num_picks", "replace"],
    "csr_cache_sampling": ["uva_indptr", "uva_indices", "gpu_indptr", "gpu_indices", "hashmap", "seeds",
                           "num_picks", "replace"],
    "create_subcsr": ["uva_indptr", "uva_indices", "seeds"],
    "tensor_relabel": ["tensors"],
}


def test_reference_names_and_keywords():
    import shmtensor_b200
    shmtensor_b200.install_dropin()
    import ShmTensorLib as capi
    import shmtensor
    assert shmtensor.capi is capi
    for cls in ("ShmTensor", "DiskTensor", "GPUSamplingDataloader"):
        assert hasattr(shmtensor, cls)
    for name, kwargs in REFERENCE_API.items():
        fn = getattr(capi, name)
        params = list(inspect.signature(fn).parameters)
        assert params[:len(kwargs)] == kwargs, (name, params)
        # anything beyond the reference's arguments is optional
        extra = list(inspect.signature(fn).parameters.values())[len(kwargs):]
        assert all(p.default is not inspect.Parameter.empty for p in extra), name
    m = capi.CUCOStaticHashmap
    assert list(inspect.signature(m.__init__).parameters)[1:] == ["keys", "values", "load_factor"]
    for method in ("query", "capacity", "memory_usage"):
        assert callable(getattr(m, method))
    # constructor arguments of the Python classes (python/shmtensor/shm_tensor.py:21, disk_tensor.py:10,
    # sampling.py:32-41)
    assert list(inspect.signature(shmtensor.ShmTensor.__init__).parameters)[1:8] == [
        "name", "shape", "local_rank", "local_world_size", "local_group", "dtype", "pin_memory"]
    assert list(inspect.signature(shmtensor.DiskTensor.__init__).parameters)[1:3] == ["filename", "pin_memory"]
    assert list(inspect.signature(shmtensor.GPUSamplingDataloader.__init__).parameters)[1:10] == [
        "indptr", "indices", "seeds", "batchsize", "num_picks", "replace", "use_ddp", "shuffle", "drop_last"]


@pytest.mark.gpu
def test_a_script_written_against_the_reference_runs_unchanged():
    """The flow of the reference's example scripts, through its own import names and keyword
    arguments: map over cached rows, fetch == data[query] for 1-D and 3-D tables, set -> fetch round
    trip, cached sampling + relabel, the scan, all by keyword."""
    import shmtensor_b200
    shmtensor_b200.install_dropin()
    import ShmTensorLib as capi
    from shmtensor import GPUSamplingDataloader

    for data in (torch.arange(100).float(), torch.randn(100, 20, 10)):
        capi.pin_memory(data=data)
        try:
            cached = torch.randperm(100)[:40].cuda()
            gpu_data = data[cached.cpu()].cuda()
            hashmap = capi.CUCOStaticHashmap(keys=cached, values=torch.arange(40).cuda(), load_factor=0.8)
            assert hashmap.capacity() == 50 and hashmap.memory_usage() > 0
            query = torch.randint(0, 100, (1000,)).cuda()
            out = capi.cache_fetch(uva_data=data, gpu_data=gpu_data, indices=query, hashmap=hashmap)
            assert torch.equal(out.cpu(), data[query.cpu()])
            mask = hashmap.query(query)
            out = capi.cache_fetch_with_mask(uva_data=data, gpu_data=gpu_data, indices=query, mask=mask)
            assert torch.equal(out.cpu(), data[query.cpu()])
            assert torch.equal(capi.uva_fetch(data=data, indices=query).cpu(), data[query.cpu()])
            ids = torch.randperm(100)[:30].cuda()
            update = torch.randn(30, *data.shape[1:]).cuda()
            capi.cache_set(uva_data=data, gpu_data=gpu_data, indices=ids, update=update, hashmap=hashmap)
            back = capi.cache_fetch(uva_data=data, gpu_data=gpu_data, indices=ids, hashmap=hashmap)
            assert torch.equal(back, update)
        finally:
            torch.cuda.synchronize()
            capi.unpin_memory(data=data)

    indptr = torch.tensor([0, 0, 4, 9, 15, 100, 101, 107])
    indices = torch.arange(107)
    seeds = torch.tensor([5, 0, 1, 2, 3, 4, 6]).int().cuda()
    sub_indptr, sub_indices = capi.csr_sampling(indptr=indptr.cuda(), indices=indices.cuda(), seeds=seeds,
                                                num_picks=5, replace=False)
    assert sub_indptr.tolist() == [0, 1, 1, 5, 10, 15, 20, 25] and sub_indices[0].item() == 100
    capi.pin_memory(indptr)
    capi.pin_memory(indices)
    try:
        cache_seeds = torch.tensor([5, 2, 1]).cuda()
        gpu_indptr, gpu_indices = capi.create_subcsr(uva_indptr=indptr, uva_indices=indices, seeds=cache_seeds)
        assert gpu_indptr.tolist() == [0, 1, 6, 10]
        hashmap = capi.CUCOStaticHashmap(cache_seeds, torch.arange(3).cuda(), 0.8)
        p, x = capi.csr_cache_sampling(uva_indptr=indptr, uva_indices=indices, gpu_indptr=gpu_indptr,
                                       gpu_indices=gpu_indices, hashmap=hashmap, seeds=seeds, num_picks=5,
                                       replace=False)
        assert p.tolist() == [0, 1, 1, 5, 10, 15, 20, 25] and x[1:5].tolist() == [0, 1, 2, 3]
    finally:
        torch.cuda.synchronize()
        capi.unpin_memory(indptr)
        capi.unpin_memory(indices)
    unique, (a, b) = capi.tensor_relabel(tensors=[torch.tensor([2, 0, 4, 1, 4]).cuda(), torch.tensor([3, 0, 8]).cuda()])
    assert unique.tolist() == [2, 0, 4, 1, 3, 8] and a.tolist() == [0, 1, 2, 3, 2] and b.tolist() == [4, 1, 5]
    t = torch.ones(1000, dtype=torch.int32).cuda()
    capi.thrust_scan(tensor=t)
    assert t[-1].item() == 1000
    # the dataloader under its reference name, with the reference's positional arguments
    rng = np.random.default_rng(0)
    deg = rng.integers(0, 30, size=2000)
    ip = torch.from_numpy(np.concatenate([[0], np.cumsum(deg)]))
    ix = torch.from_numpy(rng.integers(0, 2000, size=int(ip[-1])))
    dl = GPUSamplingDataloader(ip, ix, torch.arange(0, 512), 128, [10, 5], False, False, True, False)
    n = 0
    for frontier, output_nodes, blocks in dl:
        assert len(blocks) == 2 and output_nodes.numel() == 128
        n += 1
    assert n == len(dl) == 4
    del dl
