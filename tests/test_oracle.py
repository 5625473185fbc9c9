"""The oracle against the reference's known-answer vectors (CPU only)."""
import numpy as np
import pytest

from conftest import load_golden
from oracle import oracle


def test_relabel_golden_vector():
    g = load_golden("relabel.json")
    ins = [np.array(x, dtype=np.int64) for x in g["inputs"]]
    for fn in (oracle.tensor_relabel, oracle.tensor_relabel_literal):
        uniq, rel = fn(ins)
        assert uniq.tolist() == g["unique"]
        assert [r.tolist() for r in rel] == g["relabel"]


@pytest.mark.parametrize("seed", range(5))
def test_relabel_vectorised_equals_literal(seed):
    rng = np.random.default_rng(seed)
    ins = [rng.integers(0, 50, size=rng.integers(1, 80)).astype(np.int32) for _ in range(3)]
    u1, r1 = oracle.tensor_relabel(ins)
    u2, r2 = oracle.tensor_relabel_literal(ins)
    assert np.array_equal(u1, u2) and u1.dtype == np.int32
    for a, b in zip(r1, r2):
        assert np.array_equal(a, b)


def _graph(g):
    return (np.array(g["indptr"], dtype=np.int64), np.arange(g["n_indices"], dtype=np.int64),
            np.array(g["seeds"], dtype=np.int32))


def _check_expectations(exp, sub_indptr, sub_indices):
    assert sub_indptr.tolist() == exp["sub_indptr"]
    assert sub_indices.size == exp["sub_indptr"][-1]
    for b, e, vals in exp.get("exact", []):
        assert sub_indices[b:e].tolist() == vals
    for b, e, lo, hi, distinct in exp["ranged"]:
        seg = sub_indices[b:e]
        assert ((seg >= lo) & (seg < hi)).all()
        if distinct:
            assert np.unique(seg).size == seg.size


@pytest.mark.parametrize("cached", [False, True])
def test_sampling_golden(cached):
    g = load_golden("sampling.json")
    indptr, indices, seeds = _graph(g)
    kw = {}
    if cached:
        c = g["cache"]
        cs = np.array(c["cache_seeds"], dtype=np.int64)
        gp, gi = oracle.create_subcsr(indptr, indices, cs)
        assert gp.tolist() == c["gpu_indptr"] and gi.tolist() == c["gpu_indices"]
        kw = dict(table=oracle.hashmap_build(cs, np.arange(cs.size)), gpu_indptr=gp, gpu_indices=gi)
    rng = np.random.default_rng(0)
    for replace, key in ((True, "replace_true"), (False, "replace_false")):
        p, x = oracle.csr_sampling(indptr, indices, seeds, g["num_picks"], replace, rng, **kw)
        _check_expectations(g[key], p, x)
        oracle.check_sample(indptr, indices, seeds, g["num_picks"], replace, p, x,
                            positional=True, **kw)
        assert p.dtype == np.int64


def test_hashmap_golden():
    g = load_golden("hashmap.json")
    keys, vals = np.array(g["keys"]), np.array(g["values"])
    table = oracle.hashmap_build(keys, vals)
    assert oracle.hashmap_capacity(keys.size, g["load_factor"]) == g["capacity"]
    for kd, vd in g["dtype_combos"]:
        out = oracle.hashmap_query(table, np.array(g["requests"], dtype=np.int64), np.dtype(kd), np.dtype(vd))
        assert out.dtype == np.dtype(vd)
        assert out.tolist() == g["answers"]
    # requests are narrowed to the key dtype before the lookup
    wide = np.array([keys[0] + (1 << 32)], dtype=np.int64)
    assert oracle.hashmap_query(table, wide, np.int32)[0] == vals[0]
    assert oracle.hashmap_query(table, wide, np.int64)[0] == -1


def test_hashmap_erase_contract():
    table = oracle.hashmap_build(np.arange(10), np.arange(10) * 7)
    assert oracle.hashmap_erase(table, np.array([3, 99, 3, 0])).tolist() == [21, -1, -1, 0]
    assert oracle.hashmap_query(table, np.array([0, 3, 4])).tolist() == [-1, -1, 28]
    assert len(table) == 8


def test_fetch_set_round_trip():
    g = load_golden("fetch_set.json")
    rng = np.random.default_rng(g["multi_dim_seed"])
    for data in (np.arange(100, dtype=np.float32), rng.standard_normal(g["multi_dim_shape"]).astype(np.float32)):
        cached = np.array(g["cached_ids"])
        table = oracle.hashmap_build(cached, np.arange(cached.size))
        gpu = data[cached].copy()
        q = np.array(g["query"])
        out = oracle.cache_fetch(data, gpu, q, table)
        assert np.array_equal(out, data[q])
        assert np.array_equal(oracle.uva_fetch(data, q), data[q])
        ids = np.array(g["set_ids"])
        upd = (rng.standard_normal((ids.size, *data.shape[1:])) + 5).astype(np.float32)
        host, dev = data.copy(), gpu.copy()
        oracle.cache_set(host, dev, ids, upd, table)
        assert np.array_equal(oracle.cache_fetch(host, dev, ids, table), upd)
        hit = np.isin(ids, cached)
        assert np.array_equal(host[ids[hit]], data[ids[hit]])  # hits leave the host row alone


def test_insert_set_equals_build_then_set():
    rng = np.random.default_rng(3)
    keys = rng.choice(1 << 20, size=64, replace=False)
    rows = rng.standard_normal((64, 8)).astype(np.float32)
    a = np.zeros((64, 8), np.float32)
    t = {}
    oracle.insert_set(t, a, keys, np.arange(64), rows)
    b = np.zeros((64, 8), np.float32)
    t2 = oracle.hashmap_build(keys, np.arange(64))
    oracle.cache_set(np.zeros((1, 8), np.float32), b, keys, rows, t2)
    assert t == t2 and np.array_equal(a, b)


def test_scan():
    a = np.array([1, 2, 3, 2**31 - 1, 5], dtype=np.int32)
    assert oracle.scan_inclusive(a).tolist() == [1, 3, 6, -(2**31) + 5, -(2**31) + 10]
    assert oracle.scan_exclusive(np.array([3, 1, 4], dtype=np.int64)).tolist() == [0, 3, 4]


def test_cpu_baseline_library_matches_oracle():
    from oracle import build_oracle
    import ctypes as C
    lib = build_oracle.load_cpu()
    rng = np.random.default_rng(5)
    table = rng.standard_normal((1000, 25)).astype(np.float32)
    idx = rng.integers(0, 1000, size=333)
    out = np.empty((333, 25), np.float32)
    lib.oracle_gather(table.ctypes.data, idx.ctypes.data, 333, 100, out.ctypes.data)
    assert np.array_equal(out, oracle.uva_fetch(table, idx))
    ids = rng.integers(0, 40, size=500)
    uniq, rel = np.empty(500, np.int64), np.empty(500, np.int64)
    n = lib.oracle_relabel(ids.ctypes.data, 500, uniq.ctypes.data, rel.ctypes.data)
    wu, (wr,) = oracle.tensor_relabel([ids])
    assert np.array_equal(uniq[:n], wu) and np.array_equal(rel, wr)
    deg = rng.integers(0, 30, size=200)
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    indices = np.arange(indptr[-1], dtype=np.int32)
    seeds = rng.integers(0, 200, size=64)
    for replace in (0, 1):
        sp = np.empty(65, np.int64)
        so = np.empty(64 * 7, np.int32)
        nnz = lib.oracle_sample_hop(indptr.ctypes.data, indices.ctypes.data, 0, seeds.ctypes.data,
                                    64, 7, replace, 99, sp.ctypes.data, so.ctypes.data)
        oracle.check_sample(indptr, indices, seeds, 7, bool(replace), sp, so[:nnz], positional=True)


def test_bulk_sample_checker_agrees_with_the_per_seed_checker():
    """`check_sample_bulk` (whole-array form used at full size) accepts what `check_sample` accepts
    and rejects the same corruptions."""
    rng = np.random.default_rng(12)
    deg = rng.integers(0, 40, size=400)
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    indices = np.concatenate([rng.permutation(3000)[:d] for d in deg]).astype(np.int32)
    seeds = rng.integers(0, 400, size=500)
    for k, replace in ((5, False), (64, False), (7, True)):
        p, x = oracle.csr_sampling(indptr, indices, seeds, k, replace, np.random.default_rng(k))
        oracle.check_sample(indptr, indices, seeds, k, replace, p, x, positional=True)
        oracle.check_sample_bulk(indptr, indices, seeds, k, replace, p, x, distinct_rows=True)
        picked = np.flatnonzero(np.diff(p) > 0)
        big = [i for i in picked if deg[seeds[i]] > k] or list(picked)
        i = int(big[0])
        outside = x.copy()
        outside[p[i]] = 2999 if 2999 not in indices[indptr[seeds[i]]:indptr[seeds[i] + 1]] else 2998
        with pytest.raises(AssertionError):
            oracle.check_sample_bulk(indptr, indices, seeds, k, replace, p, outside, distinct_rows=True)
        if not replace and deg[seeds[i]] > k:
            twice = x.copy()
            twice[p[i] + 1] = twice[p[i]]
            with pytest.raises(AssertionError, match="twice"):
                oracle.check_sample_bulk(indptr, indices, seeds, k, replace, p, twice, distinct_rows=True)
        wrong_ptr = p.copy()
        wrong_ptr[-1] += 1
        with pytest.raises(AssertionError, match="sub_indptr"):
            oracle.check_sample_bulk(indptr, indices, seeds, k, replace, wrong_ptr, x)
