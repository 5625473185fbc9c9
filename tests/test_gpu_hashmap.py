"""Static hashmap on the GPU against the oracle (bit-exact)."""
import numpy as np
import pytest
import torch

from conftest import load_golden
from oracle import oracle

pytestmark = pytest.mark.gpu

DT = {"int32": torch.int32, "int64": torch.int64}


@pytest.fixture(scope="module")
def capi():
    from shmtensor_b200 import capi
    return capi


def test_golden_four_dtype_combos(capi):
    g = load_golden("hashmap.json")
    for kd, vd in g["dtype_combos"]:
        keys = torch.tensor(g["keys"], dtype=DT[kd], device="cuda")
        vals = torch.tensor(g["values"], dtype=DT[vd], device="cuda")
        m = capi.CUCOStaticHashmap(keys, vals, g["load_factor"])
        assert m.capacity() == g["capacity"]
        assert m.memory_usage() > 0 and m.size() == keys.numel()
        out = m.query(torch.tensor(g["requests"], dtype=torch.int64, device="cuda"))
        assert out.dtype == DT[vd]
        assert out.cpu().tolist() == g["answers"]
        assert torch.equal(m.query(keys), vals)


@pytest.mark.parametrize("n,lf", [(1, 0.5), (31, 0.8), (1000, 0.1), (100_000, 0.5), (100_000, 0.99),
                                  (50_000, 1.0)])
def test_random_keys_match_oracle(capi, n, lf):
    rng = np.random.default_rng(n)
    keys = rng.choice(1 << 40, size=n, replace=False).astype(np.int64)
    vals = rng.integers(0, 1 << 50, size=n).astype(np.int64)
    m = capi.CUCOStaticHashmap(torch.from_numpy(keys).cuda(), torch.from_numpy(vals).cuda(), lf)
    assert m.capacity() == oracle.hashmap_capacity(n, lf)
    req = np.concatenate([keys[rng.integers(0, n, size=n)], rng.integers(0, 1 << 40, size=n)])
    rng.shuffle(req)
    want = oracle.hashmap_query(oracle.hashmap_build(keys, vals), req)
    got = m.query(torch.from_numpy(req).cuda())
    assert np.array_equal(got.cpu().numpy(), want)


def test_requests_are_narrowed_to_the_key_dtype(capi):
    keys = torch.tensor([5, 7, -3], dtype=torch.int32, device="cuda")
    vals = torch.tensor([50, 70, 30], dtype=torch.int32, device="cuda")
    m = capi.CUCOStaticHashmap(keys, vals, 0.5)
    req = torch.tensor([5 + (1 << 32), 7, -3, 8, -1], dtype=torch.int64, device="cuda")
    assert m.query(req).cpu().tolist() == [50, 70, 30, -1, -1]
    # a 2-D request keeps its shape, like the reference's full_like
    assert m.query(req[:4].reshape(2, 2)).shape == (2, 2)


def test_empty_and_errors(capi):
    e = torch.empty(0, dtype=torch.int64, device="cuda")
    m = capi.CUCOStaticHashmap(e, e, 0.5)
    assert m.capacity() == 0
    assert m.query(torch.tensor([1, 2], device="cuda")).cpu().tolist() == [-1, -1]
    assert m.query(e).numel() == 0
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        capi.CUCOStaticHashmap(torch.zeros(2, dtype=torch.int64), e, 0.5)
    with pytest.raises(RuntimeError, match="int32 or int64"):
        capi.CUCOStaticHashmap(torch.zeros(2, device="cuda"), torch.zeros(2, dtype=torch.int64, device="cuda"), 0.5)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        m.query(torch.tensor([1]))


def test_insert_into_live_map_and_overflow(capi):
    m = capi.CUCOStaticHashmap.empty(1000)
    k1 = torch.arange(0, 600, device="cuda")
    m.insert(k1, k1 * 2)
    m.insert(k1[:100], k1[:100] * 3)          # assign
    assert m.size() == 600
    got = m.query(torch.arange(0, 700, device="cuda")).cpu()
    want = torch.cat([torch.arange(100) * 3, torch.arange(100, 600) * 2, torch.full((100,), -1)])
    assert torch.equal(got, want)
    from shmtensor_b200._lib import ShmtError, ERR_CAPACITY
    with pytest.raises(ShmtError) as err:      # more distinct keys than slots
        m.insert(torch.arange(10_000, 20_000, device="cuda"), torch.arange(10_000, device="cuda"))
    assert err.value.code == ERR_CAPACITY
    # the map is still usable and old keys are intact
    assert m.query(torch.tensor([5, 599], device="cuda")).cpu().tolist() == [15, 1198]


def test_overflow_is_reported_once_not_forever(capi):
    """An overflow belongs to the call that overflowed: once erase has made room, the next insert
    (and the fused insert+set) that fits must succeed."""
    from shmtensor_b200._lib import ShmtError, ERR_CAPACITY
    m = capi.CUCOStaticHashmap.empty(1000)
    base = torch.arange(0, 900, device="cuda")
    m.insert(base, base)
    with pytest.raises(ShmtError) as err:
        m.insert(torch.arange(10_000, 20_000, device="cuda"), torch.arange(10_000, device="cuda"))
    assert err.value.code == ERR_CAPACITY
    stored = m.query(torch.arange(10_000, 20_000, device="cuda"))
    m.erase(torch.arange(10_000, 20_000, device="cuda")[stored >= 0])
    m.erase(base[:500])
    assert m.size() == 400
    fresh = torch.arange(50_000, 50_300, device="cuda")
    m.insert(fresh, fresh + 1)                      # fits: must not raise
    assert torch.equal(m.query(fresh), fresh + 1) and m.size() == 700
    rows = torch.zeros(1000, 4, device="cuda")
    more = torch.arange(60_000, 60_100, device="cuda")
    capi.cache_insert_set(rows, more, torch.arange(100, device="cuda"), torch.ones(100, 4, device="cuda"), m)
    assert m.size() == 800 and rows[:100].eq(1).all()


def test_config5_map_full_size(capi):
    """4,000,000 unique int64 keys over 2^40 at load factor 0.5; 1,000,000 lookups, half absent."""
    g = torch.Generator(device="cuda").manual_seed(5)
    keys = torch.unique(torch.randint(0, 1 << 40, (4_100_000,), generator=g, device="cuda"))
    keys = keys[torch.randperm(keys.numel(), generator=g, device="cuda")][:4_000_000]
    slots = torch.arange(keys.numel(), dtype=torch.int32, device="cuda")
    m = capi.CUCOStaticHashmap(keys, slots, 0.5)
    assert m.capacity() == 8_000_000 and m.size() == 4_000_000
    present = keys[torch.randint(0, keys.numel(), (500_000,), generator=g, device="cuda")]
    absent = torch.randint(1 << 40, 1 << 41, (500_000,), generator=g, device="cuda")
    req = torch.cat([present, absent])
    perm = torch.randperm(req.numel(), generator=g, device="cuda")
    out = m.query(req[perm])
    # property check at full size: a hit returns a slot whose key is the request; absent -> -1
    hit = out >= 0
    assert hit.sum().item() == 500_000
    assert torch.equal(keys[out[hit].long()], req[perm][hit])
    assert (req[perm][~hit] >= (1 << 40)).all()
    # and every key maps to its own slot
    assert torch.equal(m.query(keys), slots)


@pytest.mark.parametrize("kd,vd", [("int64", "int64"), ("int32", "int32"), ("int64", "int32")])
def test_erase_against_oracle(capi, kd, vd):
    rng = np.random.default_rng(11)
    hi = 1 << (30 if kd == "int32" else 40)
    keys = rng.choice(hi, size=20_000, replace=False).astype(np.int64)
    vals = rng.integers(0, 1 << 30, size=keys.size).astype(np.int64)
    m = capi.CUCOStaticHashmap(torch.from_numpy(keys).cuda().to(DT[kd]),
                               torch.from_numpy(vals).cuda().to(DT[vd]), 0.5)
    table = oracle.hashmap_build(keys, vals)
    # erase a third of the keys, some absent ones and one key listed twice
    gone = np.concatenate([keys[::3], rng.integers(hi, 2 * hi - 1, size=500) if kd == "int64"
                           else np.array([], dtype=np.int64)])
    got = m.erase(torch.from_numpy(gone).cuda().to(DT[kd]))
    want = oracle.hashmap_erase(table, gone)
    assert got.dtype == DT[vd] and np.array_equal(got.cpu().numpy().astype(np.int64), want)
    assert m.size() == len(table)
    twice = torch.from_numpy(np.array([keys[1], keys[1]])).cuda().to(DT[kd])
    assert sorted(m.erase(twice).cpu().tolist()) == [-1, table.pop(int(keys[1]))]
    probe = np.concatenate([keys, gone])
    got = m.query(torch.from_numpy(probe).cuda()).cpu().numpy().astype(np.int64)
    assert np.array_equal(got, oracle.hashmap_query(table, probe))
    # reserved keys are no-ops
    assert m.erase(torch.tensor([-1, -2], device="cuda").to(DT[kd])).cpu().tolist() == [-1, -1]
    assert m.query(torch.tensor([-2], device="cuda")).cpu().tolist() == [-1]


def test_erased_slots_are_taken_again(capi):
    """Forty rounds of evicting half of the keys and admitting as many new ones into a map with
    two slots per key: without reuse of erased slots the table would fill up and overflow."""
    rng = np.random.default_rng(12)
    n = 50_000
    pool = rng.choice(1 << 40, size=n * 25, replace=False).astype(np.int64)
    live = pool[:n].copy()
    vals = np.arange(n, dtype=np.int64)
    m = capi.CUCOStaticHashmap(torch.from_numpy(live).cuda(), torch.from_numpy(vals).cuda(), 0.5)
    table = oracle.hashmap_build(live, vals)
    nxt = n
    for r in range(40):
        out_idx = rng.choice(n, size=n // 2, replace=False)
        freed = m.erase(torch.from_numpy(live[out_idx]).cuda())
        assert np.array_equal(freed.cpu().numpy(), oracle.hashmap_erase(table, live[out_idx]))
        fresh = pool[nxt:nxt + n // 2]
        nxt += n // 2
        m.insert(torch.from_numpy(fresh).cuda(), freed)          # new ids take the freed values
        table.update(oracle.hashmap_build(fresh, freed.cpu().numpy()))
        live[out_idx] = fresh
        assert m.size() == n
    probe = np.concatenate([live, pool[:n]])
    got = m.query(torch.from_numpy(probe).cuda()).cpu().numpy()
    assert np.array_equal(got, oracle.hashmap_query(table, probe))
    # duplicates inside one insert batch still land in one slot
    dup = torch.from_numpy(np.repeat(pool[-1000:], 4)).cuda()
    m.erase(torch.from_numpy(live[:2000]).cuda())
    m.insert(dup, torch.arange(dup.numel(), device="cuda"))
    assert m.size() == n - 2000 + 1000
