"""Fused sampling hop and sub-CSR builder against the oracle.

Offsets and rows with deg <= k are bit-exact; sampled rows are checked for membership,
distinct positions and (chi-square, p > 0.01) uniformity, as the reference's algorithm is only
defined up to its random stream.
"""
import numpy as np
import pytest
import torch
from scipy import stats

from conftest import load_golden
from oracle import oracle

pytestmark = pytest.mark.gpu

DT = {torch.int32: np.int32, torch.int64: np.int64}


@pytest.fixture(scope="module")
def capi():
    from shmtensor_b200 import capi
    capi.set_sampling_seed(1234)
    return capi


def _expect(exp, sub_indptr, sub_indices):
    assert sub_indptr.cpu().tolist() == exp["sub_indptr"]
    x = sub_indices.cpu().numpy()
    assert x.size == exp["sub_indptr"][-1]
    for b, e, vals in exp.get("exact", []):
        assert x[b:e].tolist() == vals
    for b, e, lo, hi, distinct in exp["ranged"]:
        assert ((x[b:e] >= lo) & (x[b:e] < hi)).all()
        if distinct:
            assert np.unique(x[b:e]).size == e - b


@pytest.mark.parametrize("ptr_dt,idx_dt", [(torch.int64, torch.int64), (torch.int32, torch.int32),
                                           (torch.int64, torch.int32)])
def test_golden_uncached(capi, ptr_dt, idx_dt):
    g = load_golden("sampling.json")
    indptr = torch.tensor(g["indptr"], dtype=ptr_dt, device="cuda")
    indices = torch.arange(g["n_indices"], dtype=idx_dt, device="cuda")
    seeds = torch.tensor(g["seeds"], dtype=torch.int32, device="cuda")
    for replace, key in ((True, "replace_true"), (False, "replace_false")):
        p, x = capi.csr_sampling(indptr, indices, seeds, g["num_picks"], replace)
        assert p.dtype == ptr_dt and x.dtype == idx_dt and p.is_cuda and x.is_cuda
        _expect(g[key], p, x)


def test_golden_cached_with_pinned_host_csr(capi):
    g = load_golden("sampling.json")
    indptr = torch.tensor(g["indptr"], dtype=torch.int64)
    indices = torch.arange(g["n_indices"], dtype=torch.int64)
    capi.pin_memory(indptr)
    capi.pin_memory(indices)
    try:
        c = g["cache"]
        cache_seeds = torch.tensor(c["cache_seeds"], dtype=torch.int64, device="cuda")
        gp, gi = capi.create_subcsr(indptr, indices, cache_seeds)
        assert gp.cpu().tolist() == c["gpu_indptr"] and gi.cpu().tolist() == c["gpu_indices"]
        m = capi.CUCOStaticHashmap(cache_seeds, torch.arange(3, device="cuda"), c["load_factor"])
        seeds = torch.tensor(g["seeds"], dtype=torch.int32, device="cuda")  # int32 seeds, int64 keys
        for replace, key in ((True, "replace_true"), (False, "replace_false")):
            p, x = capi.csr_cache_sampling(indptr, indices, gp, gi, m, seeds, g["num_picks"], replace)
            _expect(g[key], p, x)
    finally:
        capi.unpin_memory(indptr)
        capi.unpin_memory(indices)


def _random_graph(rng, n_nodes, max_deg, idx_dtype=np.int32):
    deg = rng.integers(0, max_deg, size=n_nodes)
    deg[rng.integers(0, n_nodes, size=n_nodes // 10)] = 0
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    indices = np.concatenate([rng.permutation(max(n_nodes, max_deg))[:d] for d in deg] or [[]]).astype(idx_dtype)
    return indptr, indices


@pytest.mark.parametrize("k", [1, 5, 8, 10, 15, 16, 25, 32, 40, 100])
@pytest.mark.parametrize("replace", [False, True])
def test_random_graph_legal_samples(capi, k, replace):
    rng = np.random.default_rng(k)
    indptr_n, indices_n = _random_graph(rng, 3000, 200)
    seeds_n = rng.integers(0, 3000, size=5000)
    indptr, indices = torch.from_numpy(indptr_n).cuda(), torch.from_numpy(indices_n).cuda()
    p, x = capi.csr_sampling(indptr, indices, torch.from_numpy(seeds_n).cuda(), k, replace)
    oracle.check_sample(indptr_n, indices_n, seeds_n, k, replace, p.cpu().numpy(), x.cpu().numpy(),
                        positional=True)


@pytest.mark.parametrize("n_seeds", [0, 1, 31, 33, 1024, 70_000])
def test_seed_counts_and_cached_rows(capi, n_seeds):
    rng = np.random.default_rng(n_seeds + 7)
    indptr_n, indices_n = _random_graph(rng, 20_000, 60)
    hot_n = rng.choice(20_000, size=4000, replace=False)
    indptr, indices = torch.from_numpy(indptr_n), torch.from_numpy(indices_n)
    capi.pin_memory(indptr)
    capi.pin_memory(indices)
    try:
        hot = torch.from_numpy(hot_n).cuda()
        gp, gi = capi.create_subcsr(indptr, indices, hot)
        wp, wi = oracle.create_subcsr(indptr_n, indices_n, hot_n)
        assert np.array_equal(gp.cpu().numpy(), wp) and np.array_equal(gi.cpu().numpy(), wi)
        m = capi.CUCOStaticHashmap(hot.int(), torch.arange(4000, dtype=torch.int32, device="cuda"), 0.8)
        table = oracle.hashmap_build(hot_n, np.arange(4000))
        seeds_n = rng.integers(0, 20_000, size=n_seeds)
        seeds = torch.from_numpy(seeds_n).cuda()
        for k, replace in ((10, False), (5, True)):
            p, x = capi.csr_cache_sampling(indptr, indices, gp, gi, m, seeds, k, replace)
            oracle.check_sample(indptr_n, indices_n, seeds_n, k, replace, p.cpu().numpy(),
                                x.cpu().numpy(), table=table, gpu_indptr=wp, gpu_indices=wi,
                                positional=True)
            p2, x2 = capi.csr_sampling(indptr, indices, seeds, k, replace)   # UVA only
            assert torch.equal(p, p2) and x2.numel() == x.numel()
    finally:
        capi.unpin_memory(indptr)
        capi.unpin_memory(indices)


@pytest.mark.parametrize("deg,k", [(20, 5), (40, 15), (17, 16), (100, 32), (300, 40), (1000, 10),
                                   # fan-outs above 32: positions drawn into a shared-memory set; rows shorter
                                   # than 2k draw what to leave out instead
                                   (10_000, 64), (1000, 100), (100, 64), (70, 40), (41, 40), (5000, 1024),
                                   (3000, 1500)])
def test_without_replacement_is_uniform(capi, deg, k):
    """Chi-square on how often each position of one row is picked (marginal k/deg), p > 0.01,
    plus: every sample is k distinct positions."""
    indptr = torch.tensor([0, deg], dtype=torch.int64, device="cuda")
    indices = torch.arange(deg, dtype=torch.int32, device="cuda")     # value == position
    reps = 40_000 if k <= 128 else 4_000
    seeds = torch.zeros(reps, dtype=torch.int64, device="cuda")
    p, x = capi.csr_sampling(indptr, indices, seeds, k, False)
    x = x.cpu().numpy().reshape(reps, k)
    assert ((x >= 0) & (x < deg)).all()
    assert (np.sort(x, axis=1)[:, 1:] != np.sort(x, axis=1)[:, :-1]).all(), "duplicate position"
    counts = np.bincount(x.reshape(-1), minlength=deg)
    chi2, pval = stats.chisquare(counts)
    assert pval > 0.01, (chi2, pval)
    # two calls draw different samples (the call counter advances) ...
    _, y = capi.csr_sampling(indptr, indices, seeds, k, False)
    assert not np.array_equal(np.sort(y.cpu().numpy().reshape(reps, k), 1), np.sort(x, 1))
    # ... and a pinned seed reproduces them
    capi.set_sampling_seed(99)
    _, a = capi.csr_sampling(indptr, indices, seeds, k, False)
    capi.set_sampling_seed(99)
    _, b = capi.csr_sampling(indptr, indices, seeds, k, False)
    assert torch.equal(a, b)


def test_large_fanout_subsets_are_uniform_not_only_their_marginals(capi):
    """Fan-out 33 of a 35-row goes through the shared-memory set in its leave-out form: the two
    positions left out must be a uniform pair, all C(35,2) = 595 of them equally likely; fan-out 33
    of a 70-row through its keep form: pairs of kept positions (0,1), (0,2) ... must occur at the
    rate k(k-1)/(deg(deg-1))."""
    indptr = torch.tensor([0, 35], dtype=torch.int64, device="cuda")
    indices = torch.arange(35, dtype=torch.int32, device="cuda")
    reps = 120_000
    _, x = capi.csr_sampling(indptr, indices, torch.zeros(reps, dtype=torch.int32, device="cuda"), 33, False)
    x = x.cpu().numpy().reshape(reps, 33)
    present = np.zeros((reps, 35), dtype=bool)
    present[np.arange(reps)[:, None], x] = True
    assert (present.sum(1) == 33).all()
    left = np.argwhere(~present)[:, 1].reshape(reps, 2)
    counts = np.bincount(left[:, 0] * 35 + left[:, 1], minlength=35 * 35)
    counts = counts[counts > 0]
    assert counts.size == 595 and stats.chisquare(counts)[1] > 0.01
    indptr = torch.tensor([0, 70], dtype=torch.int64, device="cuda")
    indices = torch.arange(70, dtype=torch.int32, device="cuda")
    _, y = capi.csr_sampling(indptr, indices, torch.zeros(reps, dtype=torch.int32, device="cuda"), 33, False)
    y = y.cpu().numpy().reshape(reps, 33)
    present = np.zeros((reps, 70), dtype=bool)
    present[np.arange(reps)[:, None], y] = True
    both = (present[:, :8, None] & present[:, None, :8]).sum(0)[np.triu_indices(8, 1)]
    expect = reps * 33 * 32 / (70 * 69)
    # 28 pair counts, each binomial: all within 5 standard deviations of the expectation
    assert (np.abs(both - expect) < 5 * np.sqrt(expect)).all(), (both, expect)


def test_large_fanout_on_a_cached_graph_and_fused_relabel(capi):
    """Fan-outs 40 and 64 over a partly cached power-law graph, hop by hop and through the fused
    mini-batch (which claims relabel slots inside the sampling kernel for every fan-out)."""
    rng = np.random.default_rng(21)
    deg = np.minimum((rng.pareto(1.0, size=4000) * 20).astype(np.int64), 3000)
    indptr_n = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    indices_n = np.concatenate([rng.choice(4000, size=d, replace=False) for d in deg]).astype(np.int32)
    indptr, indices = torch.from_numpy(indptr_n).cuda(), torch.from_numpy(indices_n).cuda()
    hot_n = np.argsort(-deg)[:800].copy()
    hot = torch.from_numpy(hot_n).cuda()
    gp, gi = capi.create_subcsr(indptr, indices, hot)
    hmap = capi.CUCOStaticHashmap(hot, torch.arange(800, device="cuda"), 0.5)
    seeds_n = rng.integers(0, 4000, size=600).astype(np.int32)
    seeds = torch.from_numpy(seeds_n).cuda()
    for k in (40, 64):
        p, x = capi.csr_cache_sampling(indptr, indices, gp, gi, hmap, seeds, k, False)
        oracle.check_sample_bulk(indptr_n, indices_n, seeds_n, k, False, p.cpu().numpy(), x.cpu().numpy(),
                                 distinct_rows=True)
        p, x = capi.csr_cache_sampling(indptr, indices, gp, gi, hmap, seeds, k, True)
        oracle.check_sample_bulk(indptr_n, indices_n, seeds_n, k, True, p.cpu().numpy(), x.cpu().numpy())
    capi.set_sampling_seed(77)
    _, hops = capi.sample_minibatch(indptr, indices, seeds, [40, 3], False, gp, gi, hmap)
    capi.set_sampling_seed(77)
    cur = seeds
    for (sp, sx, rel, nxt), k in zip(hops, (40, 3)):
        p, x = capi.csr_cache_sampling(indptr, indices, gp, gi, hmap, cur, k, False)
        want_next, (_, want_rel) = capi.tensor_relabel([cur, x])
        assert torch.equal(sp, p) and torch.equal(sx, x)
        assert torch.equal(nxt, want_next) and torch.equal(rel, want_rel)
        wu, (_, wx) = oracle.tensor_relabel([cur.cpu().numpy(), x.cpu().numpy()])
        assert np.array_equal(nxt.cpu().numpy(), wu) and np.array_equal(rel.cpu().numpy(), wx)
        cur = nxt


def test_pairs_are_uniform_without_replacement(capi):
    """Uniform k-subsets, not just uniform marginals: all C(6,2) pairs of a 6-row equally likely."""
    indptr = torch.tensor([0, 6], dtype=torch.int64, device="cuda")
    indices = torch.arange(6, dtype=torch.int64, device="cuda")
    reps = 60_000
    _, x = capi.csr_sampling(indptr, indices, torch.zeros(reps, dtype=torch.int32, device="cuda"), 2, False)
    x = np.sort(x.cpu().numpy().reshape(reps, 2), axis=1)
    counts = np.bincount(x[:, 0] * 6 + x[:, 1], minlength=36)
    counts = counts[counts > 0]
    assert counts.size == 15
    assert stats.chisquare(counts)[1] > 0.01


@pytest.mark.parametrize("deg,k", [(7, 5), (50, 20), (3, 40)])
def test_with_replacement_is_uniform(capi, deg, k):
    indptr = torch.tensor([0, deg], dtype=torch.int32, device="cuda")
    indices = torch.arange(deg, dtype=torch.int32, device="cuda")
    reps = 30_000
    p, x = capi.csr_sampling(indptr, indices, torch.zeros(reps, dtype=torch.int64, device="cuda"), k, True)
    assert p[-1].item() == reps * k
    counts = np.bincount(x.cpu().numpy(), minlength=deg)
    assert counts.size == deg and stats.chisquare(counts)[1] > 0.01


def test_high_degree_rows_and_power_law_graph(capi):
    """Degrees up to 10,000 (the cap of the headline workload), fan-outs 15/10/5."""
    rng = np.random.default_rng(3)
    deg = np.minimum((rng.pareto(1.1, size=5000) * 3).astype(np.int64), 10_000)
    deg[:3] = [10_000, 9_999, 16]
    indptr_n = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    indices_n = np.concatenate([rng.choice(2_400_000, size=d, replace=False) for d in deg]).astype(np.int32)
    indptr, indices = torch.from_numpy(indptr_n).cuda(), torch.from_numpy(indices_n).cuda()
    seeds_n = np.concatenate([[0, 1, 2], rng.integers(0, 5000, size=1021)])
    for k in (15, 10, 5):
        p, x = capi.csr_sampling(indptr, indices, torch.from_numpy(seeds_n).cuda(), k, False)
        oracle.check_sample(indptr_n, indices_n, seeds_n, k, False, p.cpu().numpy(), x.cpu().numpy(),
                            positional=True)


@pytest.mark.parametrize("ptr_dt,idx_dt", [(torch.int64, torch.int32), (torch.int32, torch.int32),
                                           (torch.int64, torch.int64)])
def test_edge_ids_name_the_sampled_edges(capi, ptr_dt, idx_dt):
    """Every edge id is the position of its neighbour in the full edge array and lies in the
    row of its seed, for host rows and for cached rows, and asking for edge ids changes nothing
    else about the hop."""
    rng = np.random.default_rng(17)
    deg = np.minimum((rng.pareto(1.2, size=6000) * 6).astype(np.int64), 900)
    indptr_n = np.concatenate([[0], np.cumsum(deg)]).astype(DT[ptr_dt])
    indices_n = rng.integers(0, 6000, size=int(indptr_n[-1])).astype(DT[idx_dt])
    indptr, indices = torch.from_numpy(indptr_n).cuda(), torch.from_numpy(indices_n).cuda()
    hot = torch.from_numpy(np.argsort(-deg)[:1500].copy()).cuda()
    gp, gi = capi.create_subcsr(indptr, indices, hot)
    base = capi.subcsr_edge_base(indptr, hot)
    assert torch.equal(base, indptr[hot])
    hmap = capi.CUCOStaticHashmap(hot, torch.arange(1500, device="cuda"), 0.5)
    seeds = torch.from_numpy(rng.integers(0, 6000, size=3000)).cuda()
    for k, replace in ((4, False), (15, False), (40, False), (6, True), (50, True)):
        for cached in (False, True):
            extra = dict(gpu_indptr=gp, gpu_indices=gi, gpu_edge_base=base, hashmap=hmap) if cached else {}
            capi.set_sampling_seed(3)
            p, x, e = capi.csr_sampling_with_eids(indptr, indices, seeds, k, replace, **extra)
            capi.set_sampling_seed(3)
            p0, x0 = (capi.csr_cache_sampling(indptr, indices, gp, gi, hmap, seeds, k, replace) if cached
                      else capi.csr_sampling(indptr, indices, seeds, k, replace))
            assert torch.equal(p, p0) and torch.equal(x, x0)
            assert e.dtype == ptr_dt and e.numel() == x.numel()
            assert torch.equal(indices[e.long()], x)
            owner = torch.repeat_interleave(seeds, (p[1:] - p[:-1]).long())
            assert bool(((e >= indptr[owner]) & (e < indptr[owner + 1])).all())
            if not replace:   # distinct positions: no edge twice for one seed occurrence
                occ = torch.repeat_interleave(torch.arange(seeds.numel(), device="cuda"), (p[1:] - p[:-1]).long())
                key = occ * (int(indptr_n[-1]) + 1) + e.long()
                assert torch.unique(key).numel() == key.numel()
    with pytest.raises(RuntimeError, match="needs gpu_edge_base"):
        capi.csr_sampling_with_eids(indptr, indices, seeds, 4, False, gpu_indptr=gp, gpu_indices=gi, hashmap=hmap)


def test_edge_ids_through_the_fused_minibatch(capi):
    rng = np.random.default_rng(23)
    deg = np.minimum((rng.pareto(1.2, size=5000) * 6).astype(np.int64), 700)
    indptr_n = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    indices_n = np.concatenate([rng.choice(5000, size=d, replace=False) for d in deg]).astype(np.int32)
    indptr, indices = torch.from_numpy(indptr_n).cuda(), torch.from_numpy(indices_n).cuda()
    hot = torch.from_numpy(np.argsort(-deg)[:1200].copy()).cuda()
    gp, gi = capi.create_subcsr(indptr, indices, hot)
    base = capi.subcsr_edge_base(indptr, hot)
    hmap = capi.CUCOStaticHashmap(hot, torch.arange(1200, device="cuda"), 0.5)
    seeds = torch.from_numpy(rng.integers(0, 5000, size=777).astype(np.int32)).cuda()
    for cached in (True, False):
        extra = (gp, gi, hmap, base) if cached else (None, None, None, None)
        capi.set_sampling_seed(41)
        _, plain = capi.sample_minibatch(indptr, indices, seeds, [4, 40, 9], False, *extra[:3])
        capi.set_sampling_seed(41)
        front, hops = capi.sample_minibatch(indptr, indices, seeds, [4, 40, 9], False, *extra, return_eids=True)
        cur = seeds
        for (sp, sx, rel, nxt, eid), (sp0, sx0, rel0, nxt0) in zip(hops, plain):
            assert torch.equal(sp, sp0) and torch.equal(sx, sx0) and torch.equal(rel, rel0) and torch.equal(nxt, nxt0)
            assert eid.dtype == indptr.dtype and eid.numel() == sx.numel()
            assert torch.equal(indices[eid], sx)
            owner = torch.repeat_interleave(cur.long(), (sp[1:] - sp[:-1]))
            assert bool(((eid >= indptr[owner]) & (eid < indptr[owner + 1])).all())
            cur = nxt
        assert torch.equal(front, hops[-1][3])
    with pytest.raises(RuntimeError, match="need gpu_edge_base"):
        capi.sample_minibatch(indptr, indices, seeds, [4], False, gp, gi, hmap, return_eids=True)


def test_sampling_errors(capi):
    indptr = torch.tensor([0, 2], device="cuda")
    indices = torch.tensor([0, 1], device="cuda")
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        capi.csr_sampling(indptr, indices, torch.tensor([0]), 2, False)
    with pytest.raises(RuntimeError, match="int32 or int64"):
        capi.csr_sampling(indptr.float(), indices, torch.tensor([0], device="cuda"), 2, False)


@pytest.mark.parametrize("ptr_dt", [torch.int64, torch.int32])
def test_row_offsets_at_an_odd_element_offset(capi, ptr_dt):
    """`indptr` handed over as a view that starts one element into its storage (a slice, or an .npy
    payload at an odd offset) is only element-aligned: the paired row-bound load must not be used
    on misaligned addresses, and results must equal those of an aligned copy."""
    rng = np.random.default_rng(5)
    deg = rng.integers(0, 40, size=3000)
    indptr_n = np.concatenate([[0], np.cumsum(deg)]).astype(DT[ptr_dt])
    indices_n = rng.integers(0, 3000, size=int(indptr_n[-1])).astype(np.int32)
    indices = torch.from_numpy(indices_n).cuda()
    padded = torch.empty(indptr_n.size + 1, dtype=ptr_dt, device="cuda")
    padded[1:] = torch.from_numpy(indptr_n).cuda()
    view = padded[1:]
    assert view.data_ptr() % (2 * view.element_size()) != 0 and view.is_contiguous()
    aligned = view.clone()
    seeds = torch.from_numpy(rng.integers(0, 3000, size=2000)).cuda()
    hot = torch.from_numpy(rng.choice(3000, size=700, replace=False)).cuda()
    gp, gi = capi.create_subcsr(aligned, indices, hot)
    gp_pad = torch.empty(gp.numel() + 1, dtype=gp.dtype, device="cuda")
    gp_pad[1:] = gp
    hmap = capi.CUCOStaticHashmap(hot, torch.arange(700, device="cuda"), 0.5)
    for k in (5, 64):
        capi.set_sampling_seed(99)
        p0, x0 = capi.csr_sampling(aligned, indices, seeds, k, False)
        q0, y0 = capi.csr_cache_sampling(aligned, indices, gp, gi, hmap, seeds, k, False)
        capi.set_sampling_seed(99)
        p1, x1 = capi.csr_sampling(view, indices, seeds, k, False)
        q1, y1 = capi.csr_cache_sampling(view, indices, gp_pad[1:], gi, hmap, seeds, k, False)
        assert torch.equal(p0, p1) and torch.equal(x0, x1)
        assert torch.equal(q0, q1) and torch.equal(y0, y1)
        oracle.check_sample(indptr_n, indices_n, seeds.cpu().numpy(), k, False, p1.cpu().numpy(),
                            x1.cpu().numpy())
