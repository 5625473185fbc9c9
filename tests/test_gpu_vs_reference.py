"""Our C-ABI path against the reference's OWN kernels, run side by side on the GPU.

``oracle/_ref/ShmTensorLib.so`` is the reference's source compiled unmodified (recipe:
``oracle/build_ref.py``; its cuCollections map is replaced by the stand-in under
``oracle/ref_shim``).  Skipped when that build is not present.  Bit-exact for hashmap, fetch,
set, relabel, sub-CSR and sampling offsets; sampled rows are compared where the algorithm
fixes them (deg <= fan-out) and checked for membership elsewhere.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    from oracle import build_ref
    try:
        mod = build_ref.load_reference()
    except Exception as exc:  # noqa: BLE001
        pytest.skip(f"reference build not loadable: {exc}")
    if mod is None:
        pytest.skip("oracle/_ref/ShmTensorLib.so has not been built")
    return mod


@pytest.fixture(scope="module")
def capi():
    from shmtensor_b200 import capi
    return capi


@pytest.mark.parametrize("kd,vd", [(torch.int32, torch.int32), (torch.int64, torch.int32),
                                   (torch.int32, torch.int64), (torch.int64, torch.int64)])
def test_hashmap_query(ref, capi, kd, vd):
    g = torch.Generator(device="cuda").manual_seed(1)
    keys = torch.unique(torch.randint(0, 1 << 30, (200_000,), generator=g, device="cuda")).to(kd)
    vals = torch.arange(keys.numel(), device="cuda").to(vd)
    a, b = ref.CUCOStaticHashmap(keys, vals, 0.5), capi.CUCOStaticHashmap(keys, vals, 0.5)
    assert a.capacity() == b.capacity()
    req = torch.randint(0, 1 << 30, (300_000,), generator=g, device="cuda")
    req[:100_000] = keys[:100_000].long()
    ra, rb = a.query(req), b.query(req)
    assert ra.dtype == rb.dtype and torch.equal(ra, rb)


@pytest.mark.parametrize("shape", [(5000,), (5000, 100), (300, 7, 9)])
def test_fetch_and_set(ref, capi, shape):
    g = torch.Generator().manual_seed(2)
    data_a = torch.randn(*shape, generator=g)
    data_b = data_a.clone()
    ref.pin_memory(data_a)
    capi.pin_memory(data_b)
    try:
        rows = shape[0]
        cached = torch.randperm(rows, generator=g)[: rows // 3]
        vals = torch.arange(cached.numel()).cuda()
        gpu_a, gpu_b = data_a[cached].cuda(), data_b[cached].cuda()
        ma = ref.CUCOStaticHashmap(cached.cuda(), vals, 0.8)
        mb = capi.CUCOStaticHashmap(cached.cuda(), vals, 0.8)
        q = torch.randint(0, rows, (4001,), generator=g).cuda()
        for fa, fb in ((ref.uva_fetch(data_a, q), capi.uva_fetch(data_b, q)),
                       (ref.cache_fetch(data_a, gpu_a, q, ma), capi.cache_fetch(data_b, gpu_b, q, mb)),
                       (ref.cache_fetch_with_mask(data_a, gpu_a, q, ma.query(q)),
                        capi.cache_fetch_with_mask(data_b, gpu_b, q, mb.query(q)))):
            assert fa.shape == fb.shape and fa.dtype == fb.dtype
            assert torch.equal(fa.view(torch.int32), fb.view(torch.int32))
        ids = torch.unique(torch.randint(0, rows, (700,), generator=g)).cuda()
        upd = torch.randn(ids.numel(), *shape[1:], generator=g).cuda()
        ref.cache_set(data_a, gpu_a, ids, upd, ma)
        capi.cache_set(data_b, gpu_b, ids, upd, mb)
        torch.cuda.synchronize()
        assert torch.equal(gpu_a, gpu_b) and torch.equal(data_a, data_b)
        ref.uva_set(data_a, ids, upd * 2)
        capi.uva_set(data_b, ids, upd * 2)
        ref.cache_set_with_mask(data_a, gpu_a, ids, upd * 3, ma.query(ids))
        capi.cache_set_with_mask(data_b, gpu_b, ids, upd * 3, mb.query(ids))
        torch.cuda.synchronize()
        assert torch.equal(gpu_a, gpu_b) and torch.equal(data_a, data_b)
    finally:
        ref.unpin_memory(data_a)
        capi.unpin_memory(data_b)


@pytest.mark.parametrize("dtype", [torch.int32, torch.int64])
@pytest.mark.parametrize("sizes,hi", [((10, 10), 15), ((1024, 9000), 20_000), ((50_000, 400_000), 2_400_000)])
def test_relabel(ref, capi, dtype, sizes, hi):
    g = torch.Generator(device="cuda").manual_seed(sum(sizes))
    ins = [torch.randint(0, hi, (s,), generator=g, device="cuda").to(dtype) for s in sizes]
    ua, ra = ref.tensor_relabel(ins)
    ub, rb = capi.tensor_relabel(ins)
    assert torch.equal(ua, ub) and len(ra) == len(rb)
    for x, y in zip(ra, rb):
        assert x.dtype == y.dtype and torch.equal(x, y)


def _graph(n_nodes, max_deg, seed):
    rng = np.random.default_rng(seed)
    deg = rng.integers(0, max_deg, size=n_nodes)
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    indices = np.arange(indptr[-1], dtype=np.int64)        # value == position
    return torch.from_numpy(indptr), torch.from_numpy(indices), deg


@pytest.mark.parametrize("replace", [False, True])
def test_sampling_and_subcsr(ref, capi, replace):
    indptr, indices, deg = _graph(8000, 40, 5)
    ia, xa = indptr.clone(), indices.clone()
    ref.pin_memory(ia), ref.pin_memory(xa)
    capi.pin_memory(indptr), capi.pin_memory(indices)
    try:
        g = torch.Generator().manual_seed(9)
        hot = torch.randperm(8000, generator=g)[:2500].cuda()
        gpa, gia = ref.create_subcsr(ia, xa, hot)
        gpb, gib = capi.create_subcsr(indptr, indices, hot)
        assert torch.equal(gpa, gpb) and torch.equal(gia, gib)
        vals = torch.arange(2500).cuda()
        ma, mb = ref.CUCOStaticHashmap(hot, vals, 0.8), capi.CUCOStaticHashmap(hot, vals, 0.8)
        seeds = torch.randint(0, 8000, (3000,), generator=g).int().cuda()
        k = 10
        for pa, sa, pb, sb in ((*ref.csr_sampling(ia, xa, seeds, k, replace), *capi.csr_sampling(indptr, indices, seeds, k, replace)),
                               (*ref.csr_cache_sampling(ia, xa, gpa, gia, ma, seeds, k, replace),
                                *capi.csr_cache_sampling(indptr, indices, gpb, gib, mb, seeds, k, replace))):
            assert pa.dtype == pb.dtype and torch.equal(pa, pb)          # offsets: bit-exact
            assert sa.numel() == sb.numel() and sa.dtype == sb.dtype
            p = pa.cpu().numpy()
            sa_n, sb_n = sa.cpu().numpy(), sb.cpu().numpy()
            d = deg[seeds.cpu().numpy()]
            lo = indptr.numpy()[seeds.cpu().numpy()]
            row_of = np.repeat(np.arange(seeds.numel()), np.diff(p))
            # both implementations only ever return positions of the right row
            for s in (sa_n, sb_n):
                assert ((s >= lo[row_of]) & (s < lo[row_of] + d[row_of])).all()
            if not replace:
                fixed = (d <= k)[row_of]                                   # copied rows: identical
                assert np.array_equal(sa_n[fixed], sb_n[fixed])
    finally:
        ref.unpin_memory(ia), ref.unpin_memory(xa)
        capi.unpin_memory(indptr), capi.unpin_memory(indices)
