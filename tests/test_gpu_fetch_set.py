"""Fused fetch / set kernels against the oracle (bit-exact, compared as raw bytes)."""
import numpy as np
import pytest
import torch

from conftest import load_golden
from oracle import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def capi():
    from shmtensor_b200 import capi
    return capi


def _bytes_equal(t: torch.Tensor, a: np.ndarray) -> bool:
    return np.array_equal(t.cpu().contiguous().view(torch.uint8).numpy().reshape(-1),
                          np.ascontiguousarray(a).view(np.uint8).reshape(-1))


def _pinned(capi, arr: np.ndarray) -> torch.Tensor:
    t = torch.from_numpy(arr.copy())
    capi.pin_memory(t)
    return t


def _cache(capi, data: torch.Tensor, cached_ids: np.ndarray, kd=torch.int64, vd=torch.int64, lf=0.8):
    ids = torch.from_numpy(cached_ids)
    gpu = data[ids].cuda()
    m = capi.CUCOStaticHashmap(ids.to(kd).cuda(), torch.arange(ids.numel(), dtype=vd, device="cuda"), lf)
    return gpu, m


def test_golden_shapes_one_dim_and_three_dim(capi):
    g = load_golden("fetch_set.json")
    rng = np.random.default_rng(g["multi_dim_seed"])
    for arr in (np.arange(100, dtype=np.float32),
                rng.standard_normal(g["multi_dim_shape"]).astype(np.float32)):
        data = _pinned(capi, arr)
        try:
            cached = np.array(g["cached_ids"])
            gpu, m = _cache(capi, data, cached)
            q = torch.tensor(g["query"], dtype=torch.int64, device="cuda")
            want = oracle.cache_fetch(arr, arr[cached], np.array(g["query"]),
                                      oracle.hashmap_build(cached, np.arange(cached.size)))
            for out in (capi.uva_fetch(data, q), capi.cache_fetch(data, gpu, q, m),
                        capi.cache_fetch_with_mask(data, gpu, q, m.query(q))):
                assert out.is_cuda and out.dtype == torch.float32
                assert tuple(out.shape) == (q.numel(), *arr.shape[1:])
                assert _bytes_equal(out, want)
        finally:
            capi.unpin_memory(data)


@pytest.mark.parametrize("dtype,width", [(np.float32, 100), (np.float32, 128), (np.float64, 3),
                                         (np.int8, 7), (np.uint8, 1), (np.int16, 33),
                                         (np.int64, 5), (np.int32, 1), (np.float16, 24)])
@pytest.mark.parametrize("idx_dtype", [torch.int32, torch.int64])
def test_dtype_and_width_sweep(capi, dtype, width, idx_dtype):
    """Row sizes that exercise every vector width (16/8/4/2/1 bytes) and ragged tails."""
    rng = np.random.default_rng(width)
    rows = 5000
    arr = rng.integers(-100, 100, size=(rows, width)).astype(dtype)
    data = _pinned(capi, arr)
    try:
        cached = rng.choice(rows, size=rows // 3, replace=False)
        gpu, m = _cache(capi, data, cached, kd=idx_dtype, vd=torch.int32)
        qn = rng.integers(0, rows, size=3001)
        q = torch.from_numpy(qn).to(idx_dtype).cuda()
        want = arr[qn]
        assert _bytes_equal(capi.cache_fetch(data, gpu, q, m), want)
        assert _bytes_equal(capi.uva_fetch(data, q), want)
        mask = m.query(q)
        assert mask.dtype == torch.int32
        assert _bytes_equal(capi.cache_fetch_with_mask(data, gpu, q, mask), want)
    finally:
        capi.unpin_memory(data)


def test_hits_really_come_from_the_gpu_copy(capi):
    """Make the cached copy differ from the host rows: hits must return the cached bytes."""
    rng = np.random.default_rng(1)
    arr = rng.standard_normal((2000, 100)).astype(np.float32)
    data = _pinned(capi, arr)
    try:
        cached = rng.choice(2000, size=700, replace=False)
        gpu, m = _cache(capi, data, cached)
        gpu += 1000.0
        qn = rng.integers(0, 2000, size=4096)
        q = torch.from_numpy(qn).cuda()
        table = oracle.hashmap_build(cached, np.arange(cached.size))
        want = oracle.cache_fetch(arr, gpu.cpu().numpy(), qn, table)
        assert _bytes_equal(capi.cache_fetch(data, gpu, q, m), want)
        # NaN payloads are bytes like any other
        gpu.view(torch.int32)[0, :] = 0x7FC00001
        want = oracle.cache_fetch(arr, gpu.cpu().numpy(), qn, table)
        assert _bytes_equal(capi.cache_fetch(data, gpu, q, m), want)
    finally:
        capi.unpin_memory(data)


@pytest.mark.parametrize("n", [0, 1, 31, 32, 33, 1000, 100_000])
def test_batch_sizes(capi, n):
    rng = np.random.default_rng(n + 1)
    arr = rng.standard_normal((10_000, 100)).astype(np.float32)
    data = _pinned(capi, arr)
    try:
        cached = rng.choice(10_000, size=9000, replace=False)
        gpu, m = _cache(capi, data, cached)
        qn = rng.integers(0, 10_000, size=n)
        q = torch.from_numpy(qn).cuda()
        out = capi.cache_fetch(data, gpu, q, m)
        assert tuple(out.shape) == (n, 100)
        assert _bytes_equal(out, arr[qn])
    finally:
        capi.unpin_memory(data)


def test_gpu_resident_table_and_unaligned_views(capi):
    """The 'uva' table may also live on the GPU; views at odd offsets pick a narrower vector."""
    arr = torch.arange(4000 * 25, dtype=torch.float32, device="cuda").reshape(4000, 25)
    q = torch.randint(0, 3999, (999,), device="cuda")
    assert torch.equal(capi.uva_fetch(arr, q), arr[q])
    view = arr.reshape(-1)[1:1 + 3999 * 25].reshape(3999, 25)  # base 4 bytes off a 16-byte boundary
    assert torch.equal(capi.uva_fetch(view, q), view[q])


def test_set_round_trips(capi):
    """example/test_cache_set.py: set then fetch returns the update, for uva / map / mask."""
    rng = np.random.default_rng(2)
    for arr in (rng.standard_normal(1000).astype(np.float32),
                rng.standard_normal((20_000, 128)).astype(np.float32)):
        data = _pinned(capi, arr)
        try:
            rows = arr.shape[0]
            cached = rng.choice(rows, size=int(rows * 0.7), replace=False)
            gpu, m = _cache(capi, data, cached)
            table = oracle.hashmap_build(cached, np.arange(cached.size))
            for size in (10, 100, rows // 2):
                ids_n = np.unique(rng.integers(0, rows, size=size))
                ids = torch.from_numpy(ids_n).cuda()
                upd_n = rng.standard_normal((ids_n.size, *arr.shape[1:])).astype(np.float32)
                upd = torch.from_numpy(upd_n).cuda()
                host_o, gpu_o = data.numpy().copy(), gpu.cpu().numpy()
                # map variant
                capi.cache_set(data, gpu, ids, upd, m)
                torch.cuda.synchronize()
                oracle.cache_set(host_o, gpu_o, ids_n, upd_n, table)
                assert _bytes_equal(gpu, gpu_o) and np.array_equal(data.numpy(), host_o)
                assert _bytes_equal(capi.cache_fetch(data, gpu, ids, m), upd_n)
                # mask variant
                upd2 = upd + 1
                capi.cache_set_with_mask(data, gpu, ids, upd2, m.query(ids))
                assert torch.equal(capi.cache_fetch_with_mask(data, gpu, ids, m.query(ids)), upd2)
                # uva variant writes the host table only
                capi.uva_set(data, ids, upd)
                torch.cuda.synchronize()
                assert np.array_equal(data.numpy()[ids_n], upd_n)
                assert torch.equal(capi.uva_fetch(data, ids), upd)
        finally:
            capi.unpin_memory(data)


def test_set_argument_errors(capi):
    data = torch.zeros(10, 4, device="cuda")
    ids = torch.tensor([1, 2], device="cuda")
    with pytest.raises(RuntimeError, match="dtype"):
        capi.uva_set(data, ids, torch.zeros(2, 4, dtype=torch.float64, device="cuda"))
    with pytest.raises(RuntimeError, match="one row per index"):
        capi.uva_set(data, ids, torch.zeros(3, 4, device="cuda"))
    with pytest.raises(RuntimeError, match="int32 or int64"):
        capi.uva_fetch(data, ids.float())
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        capi.uva_fetch(data, ids.cpu())


def test_insert_set_small_against_oracle(capi):
    rng = np.random.default_rng(9)
    keys_n = rng.choice(1 << 40, size=5000, replace=False).astype(np.int64)
    rows_n = rng.standard_normal((5000, 64)).astype(np.float32)
    keys, rows = torch.from_numpy(keys_n).cuda(), torch.from_numpy(rows_n).cuda()
    slots = torch.arange(5000, dtype=torch.int32, device="cuda")
    m = capi.CUCOStaticHashmap.empty(10_000, torch.int64, torch.int32)
    gpu = torch.zeros(5000, 64, device="cuda")
    capi.cache_insert_set(gpu, keys[:3000], slots[:3000], rows[:3000], m)
    # second call: 1000 known keys (overwrite in their old slots) + 2000 new ones
    order = torch.cat([torch.arange(2000, 3000), torch.arange(3000, 5000)]).cuda()
    newrows = rows[order] * 2
    # offer wrong slots for the known keys: the stored slot must win
    offered = slots[order].clone()
    offered[:1000] = 4999 - torch.arange(1000, dtype=torch.int32, device="cuda")
    capi.cache_insert_set(gpu, keys[order], offered, newrows, m)
    table, gpu_o = {}, np.zeros((5000, 64), np.float32)
    oracle.insert_set(table, gpu_o, keys_n[:3000], np.arange(3000), rows_n[:3000])
    oracle.insert_set(table, gpu_o, keys_n[order.cpu().numpy()], offered.cpu().numpy(),
                      (rows_n[order.cpu().numpy()] * 2))
    assert m.size() == 5000 == len(table)
    assert _bytes_equal(gpu, gpu_o)
    got = m.query(keys).cpu().numpy()
    assert np.array_equal(got, np.array([table[int(k)] for k in keys_n], dtype=np.int32))


def test_config5_insert_set_full_size(capi):
    """4,000,000 int64 keys over 2^40 with 256-d bf16 rows at load factor 0.5, then 1,000,000
    lookups (half absent): slots and rows bit-exact, checked by round trip."""
    g = torch.Generator(device="cuda").manual_seed(55)
    keys = torch.unique(torch.randint(0, 1 << 40, (4_100_000,), generator=g, device="cuda"))
    keys = keys[torch.randperm(keys.numel(), generator=g, device="cuda")][:4_000_000]
    n = keys.numel()
    rows = torch.randn(n, 256, generator=g, device="cuda").to(torch.bfloat16)
    slots = torch.arange(n, dtype=torch.int32, device="cuda")
    m = capi.CUCOStaticHashmap.empty(8_000_000, torch.int64, torch.int32)
    gpu = torch.zeros(n, 256, dtype=torch.bfloat16, device="cuda")
    capi.cache_insert_set(gpu, keys, slots, rows, m)
    assert m.size() == n and m.capacity() == 8_000_000
    assert torch.equal(gpu.view(torch.int16), rows.view(torch.int16))      # slot i holds row i
    present = torch.randint(0, n, (500_000,), generator=g, device="cuda")
    absent = torch.randint(1 << 40, 1 << 41, (500_000,), generator=g, device="cuda")
    req = torch.cat([keys[present], absent])
    perm = torch.randperm(req.numel(), generator=g, device="cuda")
    out = m.query(req[perm])
    want = torch.cat([slots[present], torch.full((500_000,), -1, dtype=torch.int32, device="cuda")])[perm]
    assert torch.equal(out, want)
    fetched = capi.cache_fetch(None, gpu, keys[present], m)                 # no host table: all hits
    assert torch.equal(fetched.view(torch.int16), rows[present].view(torch.int16))
    # overwrite through the reference-named entry point as well
    capi.cache_set(None, gpu, keys[present[:1000]], rows[present[:1000]] * 0, m)
    assert (capi.cache_fetch(None, gpu, keys[present[:1000]], m) == 0).all()


def test_config2_full_size_equals_index_select(capi):
    """2,400,000 x 100 float32 pinned host table, top 20 % cached behind an int64->int32 map at
    load factor 0.5, 500,000 queries: bit-exact with index_select on the host table."""
    g = torch.Generator().manual_seed(2)
    rows, dim, nq = 2_400_000, 100, 500_000
    data = torch.randn(rows, dim, generator=g)
    capi.pin_memory(data)
    try:
        score = torch.rand(rows, generator=g).pow(-0.6)
        hot = torch.argsort(score, descending=True)[: rows // 5]
        gpu = data[hot].cuda()
        m = capi.CUCOStaticHashmap(hot.cuda(), torch.arange(hot.numel(), dtype=torch.int32, device="cuda"), 0.5)
        assert m.capacity() == 960_000
        q = torch.cat([hot[torch.randint(0, hot.numel(), (400_000,), generator=g)],
                       torch.randint(0, rows, (100_000,), generator=g)])
        q = q[torch.randperm(nq, generator=g)]
        out = capi.cache_fetch(data, gpu, q.cuda(), m)
        want = torch.index_select(data, 0, q)
        assert torch.equal(out.cpu().view(torch.int32), want.view(torch.int32))
    finally:
        capi.unpin_memory(data)


def test_config1_gather_from_shared_memory_tensor(capi):
    """1,000,000 x 128 float32 table in POSIX shared memory (registered with CUDA), 200,000 int64
    ids drawn Zipf(1.0), duplicates allowed: the gathered [200000, 128] tensor is bit-exact with
    torch.index_select on the shared tensor."""
    import uuid
    name = f"shmt_test_{uuid.uuid4().hex[:8]}"
    rows, dim, nq = 1_000_000, 128, 200_000
    ptr, fd = capi.create_shared_mem(name, rows * dim * 4, pin_memory=True)
    try:
        table = capi.open_shared_tensor(ptr, torch.float32, (rows, dim))
        g = torch.Generator().manual_seed(1)
        for lo in range(0, rows, 250_000):
            table[lo:lo + 250_000].normal_(generator=g)
        rng = np.random.default_rng(1)
        w = 1.0 / np.arange(1, rows + 1, dtype=np.float64)
        cdf = np.cumsum(w) / w.sum()
        ranks = np.minimum(np.searchsorted(cdf, rng.random(nq)), rows - 1)
        ids = torch.from_numpy(rng.permutation(rows)[ranks].astype(np.int64))
        out = capi.uva_fetch(table, ids.cuda())
        want = torch.index_select(table, 0, ids)
        assert tuple(out.shape) == (nq, dim)
        assert torch.equal(out.cpu().view(torch.int32), want.view(torch.int32))
        del table, want
    finally:
        capi.release_shared_mem(name, rows * dim * 4, ptr, fd, pin_memory=True)
    assert not capi.file_exist(name)


def test_no_bounded_wait_ran_out(capi):
    """Every fetch above went through the bulk-copy kernel; none of its bounded waits gave up."""
    assert capi.device_fault() == 0


def test_cache_replace_keeps_fetch_exact(capi):
    """Evict a quarter of the cached rows, admit other ids into their slots, fetch again."""
    rng = np.random.default_rng(21)
    n_rows, width, n_cached = 40_000, 100, 8_000
    table_n = rng.standard_normal((n_rows, width)).astype(np.float32)
    table = torch.from_numpy(table_n.copy())
    capi.pin_memory(table)
    try:
        perm = rng.permutation(n_rows)
        cached, others = perm[:n_cached].copy(), perm[n_cached:]
        gpu_rows = torch.from_numpy(table_n[cached]).cuda()
        hmap = capi.CUCOStaticHashmap(torch.from_numpy(cached).cuda(),
                                      torch.arange(n_cached, dtype=torch.int32, device="cuda"), 0.5)
        evict, admit = cached[:2000], others[:2000]
        assert capi.cache_replace(table, gpu_rows, hmap, torch.from_numpy(evict).cuda(),
                                  torch.from_numpy(admit).cuda()) == 2000
        assert hmap.size() == n_cached
        ids = torch.from_numpy(rng.integers(0, n_rows, size=50_000)).cuda()
        out = capi.cache_fetch(table, gpu_rows, ids, hmap)
        assert torch.equal(out.cpu(), table[ids.cpu()])
        # the admitted ids are served from HBM now: poison the host copy and fetch them
        slots = hmap.query(torch.from_numpy(admit).cuda())
        assert (slots >= 0).all() and (hmap.query(torch.from_numpy(evict).cuda()) == -1).all()
        assert torch.equal(gpu_rows[slots.long()].cpu(), torch.from_numpy(table_n[admit]))
    finally:
        capi.unpin_memory(table)
