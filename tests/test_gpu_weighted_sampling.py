"""Weighted neighbour sampling (not in the reference, whose sampler is uniform): draws with
replacement follow the weights (chi-square, p > 0.01); draws without replacement have the
inclusion probabilities of sequential weighted sampling without replacement, computed exactly
by enumeration; rows with deg <= k are copied; cached rows behave like host rows."""
import itertools

import numpy as np
import pytest
import torch
from scipy import stats

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def capi():
    from shmtensor_b200 import capi
    capi.set_sampling_seed(4321)
    return capi


def _one_row(weights):
    deg = len(weights)
    indptr = torch.tensor([0, deg], dtype=torch.int64, device="cuda")
    indices = torch.arange(deg, dtype=torch.int32, device="cuda")
    return indptr, indices, torch.tensor(weights, dtype=torch.float32, device="cuda")


@pytest.mark.parametrize("k", [1, 7, 40])
def test_with_replacement_follows_the_weights(capi, k):
    rng = np.random.default_rng(k)
    w = rng.random(50) * 3 + 0.05
    w[7] = 25.0
    indptr, indices, weights = _one_row(w)
    reps = 200_000 // k
    p, x = capi.csr_weighted_sampling(indptr, indices, weights, torch.zeros(reps, dtype=torch.int64, device="cuda"),
                                      k, True)
    assert p[-1].item() == reps * k and x.numel() == reps * k
    counts = np.bincount(x.cpu().numpy(), minlength=50)
    assert stats.chisquare(counts, f_exp=w / w.sum() * counts.sum())[1] > 0.01


def test_a_single_pick_is_proportional_to_its_weight(capi):
    w = np.array([1.0, 2.0, 3.0, 4.0, 10.0, 0.5, 0.5, 1.0, 1.0, 7.0] * 5)   # deg 50 > 32: several chunks
    indptr, indices, weights = _one_row(w)
    reps = 150_000
    _, x = capi.csr_weighted_sampling(indptr, indices, weights, torch.zeros(reps, dtype=torch.int32, device="cuda"),
                                      1, False)
    counts = np.bincount(x.cpu().numpy(), minlength=50)
    assert stats.chisquare(counts, f_exp=w / w.sum() * reps)[1] > 0.01


def test_without_replacement_has_the_sequential_inclusion_probabilities(capi):
    w = np.array([5.0, 1.0, 1.0, 2.0, 0.5, 3.0, 1.0, 0.25, 4.0])
    k = 4
    # exact: P(set) summed over the orders in which sequential draws without replacement produce it
    incl = np.zeros(len(w))
    for seq in itertools.permutations(range(len(w)), k):
        prob, rest = 1.0, w.sum()
        for i in seq:
            prob *= w[i] / rest
            rest -= w[i]
        incl[list(seq)] += prob
    assert abs(incl.sum() - k) < 1e-9
    indptr, indices, weights = _one_row(w)
    reps = 200_000
    p, x = capi.csr_weighted_sampling(indptr, indices, weights, torch.zeros(reps, dtype=torch.int64, device="cuda"),
                                      k, False)
    x = x.cpu().numpy().reshape(reps, k)
    assert (np.sort(x, 1)[:, 1:] != np.sort(x, 1)[:, :-1]).all(), "an edge was picked twice"
    counts = np.bincount(x.reshape(-1), minlength=len(w))
    z = (counts - reps * incl) / np.sqrt(reps * incl * (1 - incl))
    assert (np.abs(z) < 4.5).all(), z


def test_weighted_hop_on_a_cached_graph_with_edge_ids(capi):
    rng = np.random.default_rng(5)
    deg = np.minimum((rng.pareto(1.2, size=3000) * 6).astype(np.int64), 500)
    indptr_n = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    indices_n = np.concatenate([rng.choice(3000, size=d, replace=False) for d in deg]).astype(np.int32)
    w_n = (rng.random(indices_n.size) + 0.01).astype(np.float32)
    indptr, indices, weights = (torch.from_numpy(a).cuda() for a in (indptr_n, indices_n, w_n))
    hot = torch.from_numpy(np.argsort(-deg)[:700].copy()).cuda()
    gp, gi = capi.create_subcsr(indptr, indices, hot)
    _, gw = capi.create_subcsr(indptr, weights.view(torch.int32), hot)
    gw = gw.view(torch.float32)
    base = capi.subcsr_edge_base(indptr, hot)
    hmap = capi.CUCOStaticHashmap(hot, torch.arange(700, device="cuda"), 0.5)
    seeds = torch.from_numpy(rng.integers(0, 3000, size=2500)).cuda()
    from oracle import oracle
    for k, replace in ((5, False), (32, False), (12, True), (48, True)):
        capi.set_sampling_seed(9)
        p, x, e = capi.csr_weighted_sampling(indptr, indices, weights, seeds, k, replace, gp, gi, gw, hmap, base,
                                             return_eids=True)
        capi.set_sampling_seed(9)
        p1, x1 = capi.csr_weighted_sampling(indptr, indices, weights, seeds, k, replace)   # uncached: same draws
        assert torch.equal(p, p1) and torch.equal(x, x1)
        oracle.check_sample_bulk(indptr_n, indices_n, seeds.cpu().numpy(), k, replace, p.cpu().numpy(),
                                 x.cpu().numpy(), distinct_rows=True)
        assert torch.equal(indices[e], x)
    from shmtensor_b200._lib import ShmtError
    with pytest.raises(ShmtError, match="limited to 32"):
        capi.csr_weighted_sampling(indptr, indices, weights, seeds, 33, False)
    with pytest.raises(RuntimeError, match="float32"):
        capi.csr_weighted_sampling(indptr, indices, weights.double(), seeds, 3, False)


def test_heavier_edges_win_more_often_on_long_rows(capi):
    """deg 2,000, fan-out 10: the 20 edges that carry half of the total weight take about half of
    the picks' first-order mass (a loose bound; the exact law is checked on the short row above)."""
    w = np.ones(2000)
    w[:20] = 99.0
    indptr, indices, weights = _one_row(w)
    reps = 20_000
    _, x = capi.csr_weighted_sampling(indptr, indices, weights, torch.zeros(reps, dtype=torch.int64, device="cuda"),
                                      10, False)
    x = x.cpu().numpy().reshape(reps, 10)
    assert (np.sort(x, 1)[:, 1:] != np.sort(x, 1)[:, :-1]).all()
    share = (x < 20).mean()
    assert 0.44 < share < 0.50, share   # sequential draws on the CPU give 0.471


@pytest.mark.parametrize("cached", [False, True])
def test_weighted_minibatch_equals_weighted_hops(capi, cached):
    """shmt_sample_minibatch_weighted: all hops in one native call, the same draws as one
    csr_weighted_sampling + tensor_relabel per hop."""
    rng = np.random.default_rng(11)
    n_nodes = 4000
    deg = np.minimum((rng.pareto(1.2, size=n_nodes) * 6).astype(np.int64), 400)
    indptr_n = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    indices_n = np.concatenate([rng.choice(n_nodes, size=d, replace=False) for d in deg]).astype(np.int32)
    w_n = (rng.random(indices_n.size) + 0.01).astype(np.float32)
    indptr, indices, weights = (torch.from_numpy(a).cuda() for a in (indptr_n, indices_n, w_n))
    gp = gi = gw = hmap = None
    if cached:
        hot = torch.from_numpy(np.argsort(-deg)[:900].copy()).cuda()
        gp, gi = capi.create_subcsr(indptr, indices, hot)
        gw = capi.create_subcsr(indptr, weights.view(torch.int32), hot)[1].view(torch.float32)
        hmap = capi.CUCOStaticHashmap(hot, torch.arange(900, device="cuda"), 0.5)
    for n_seeds, fanouts, replace in ((512, [4, 8, 3], False), (100, [32, 2], False), (300, [6, 40], True)):
        seeds = torch.from_numpy(rng.choice(n_nodes, size=n_seeds, replace=False)).int().cuda()
        capi.set_sampling_seed(31)
        want, cur = [], seeds
        for k in fanouts:
            p, x = capi.csr_weighted_sampling(indptr, indices, weights, cur, k, replace, gp, gi, gw, hmap)
            nxt, (_, rx) = capi.tensor_relabel([cur, x])
            want.append((p, x, rx, nxt))
            cur = nxt
        capi.set_sampling_seed(31)
        frontier, hops = capi.sample_minibatch(indptr, indices, seeds, fanouts, replace, gp, gi, hmap,
                                               weights=weights, gpu_weights=gw)
        assert torch.equal(frontier, cur) and len(hops) == len(fanouts)
        for (p, x, rx, nxt), (p2, x2, rx2, nxt2) in zip(want, hops):
            assert torch.equal(p, p2) and torch.equal(x, x2) and torch.equal(rx, rx2) and torch.equal(nxt, nxt2)
    from shmtensor_b200._lib import ShmtError
    with pytest.raises(ShmtError, match="at most 32"):
        capi.sample_minibatch(indptr, indices, seeds, [33], False, gp, gi, hmap, weights=weights, gpu_weights=gw)
    with pytest.raises(RuntimeError, match="cannot be combined"):
        capi.sample_minibatch(indptr, indices, seeds, [3], False, weights=weights, return_eids=True)
    capi.check_async()
