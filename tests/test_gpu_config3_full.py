"""Config 3 at full size: 2,400,000 nodes / 62,000,000 edges, top 20 % of the nodes cached,
1,024 seeds, hops over reversed([15, 10, 5]), relabel after every hop — the loop of the
reference's GPUSamplingDataloader.__next__ (python/shmtensor/sampling.py:117-147).

Every hop must be a legal outcome of the reference's sampler (offsets exact, rows with
deg <= k copied exactly, every other pick inside its row and no position twice) and every
relabel must equal the oracle's first-occurrence relabel bit for bit.
"""
import numpy as np
import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def graph():
    import bench
    from shmtensor_b200 import capi
    indptr_n, indices_n, deg = bench.make_graph()
    assert indptr_n.size == 2_400_001 and indices_n.size == 62_000_000
    indptr, indices = torch.from_numpy(indptr_n), torch.from_numpy(indices_n)
    capi.pin_memory(indptr)
    capi.pin_memory(indices)
    hot_n = np.argsort(-deg, kind="stable")[:480_000].copy()
    hot = torch.from_numpy(hot_n).cuda()
    gp, gi = capi.create_subcsr(indptr, indices, hot)
    hmap = capi.CUCOStaticHashmap(hot.int(), torch.arange(480_000, dtype=torch.int32, device="cuda"), 0.8)
    yield capi, indptr_n, indices_n, indptr, indices, hot_n, gp, gi, hmap
    torch.cuda.synchronize()
    capi.unpin_memory(indptr)
    capi.unpin_memory(indices)


def test_cached_adjacency_is_the_hot_rows(graph):
    capi, indptr_n, indices_n, indptr, indices, hot_n, gp, gi, hmap = graph
    deg = indptr_n[hot_n + 1] - indptr_n[hot_n]
    assert np.array_equal(gp.cpu().numpy(), np.concatenate([[0], np.cumsum(deg)]))
    # spot rows: the first, the last and 2,000 random cached rows hold the host rows
    rng = np.random.default_rng(1)
    gpn, gin = gp.cpu().numpy(), gi.cpu().numpy()
    for s in np.concatenate([[0, hot_n.size - 1], rng.integers(0, hot_n.size, size=2000)]):
        r = hot_n[s]
        assert np.array_equal(gin[gpn[s]:gpn[s + 1]], indices_n[indptr_n[r]:indptr_n[r + 1]])


@pytest.mark.parametrize("fused", [True, False])
def test_three_hops_with_relabel(graph, fused):
    capi, indptr_n, indices_n, indptr, indices, hot_n, gp, gi, hmap = graph
    rng = np.random.default_rng(11)
    capi.set_sampling_seed(31)
    fan = [5, 10, 15]                                  # reversed([15, 10, 5])
    for batch in range(2):
        seeds_n = rng.integers(0, 2_400_000, size=1024).astype(np.int32)
        seeds = torch.from_numpy(seeds_n).cuda()
        if fused:
            _, hops = capi.sample_minibatch(indptr, indices, seeds, fan, False, gp, gi, hmap)
        else:
            hops, cur = [], seeds
            for k in fan:
                sp, sx = capi.csr_cache_sampling(indptr, indices, gp, gi, hmap, cur, k, False)
                nxt, (_, rel) = capi.tensor_relabel([cur, sx])
                hops.append((sp, sx, rel, nxt))
                cur = nxt
        cur_n = seeds_n
        total = 0
        for (sp, sx, rel, nxt), k in zip(hops, fan):
            oracle.check_sample_bulk(indptr_n, indices_n, cur_n, k, False, sp.cpu().numpy(),
                                     sx.cpu().numpy(), distinct_rows=True)
            want_unique, (_, want_rel) = oracle.tensor_relabel([cur_n, sx.cpu().numpy()])
            assert np.array_equal(nxt.cpu().numpy(), want_unique)
            assert np.array_equal(rel.cpu().numpy(), want_rel)
            cur_n = want_unique
            total += sx.numel()
        assert total > 300_000 and cur_n.size > 100_000   # the size the config is quoted on


def test_uncached_sampling_gives_the_same_offsets(graph):
    """The cache changes where rows are read from, never what a hop returns."""
    capi, indptr_n, indices_n, indptr, indices, hot_n, gp, gi, hmap = graph
    seeds = torch.from_numpy(np.random.default_rng(3).integers(0, 2_400_000, size=50_000)).cuda()
    capi.set_sampling_seed(5)
    p0, x0 = capi.csr_cache_sampling(indptr, indices, gp, gi, hmap, seeds, 10, False)
    capi.set_sampling_seed(5)
    p1, x1 = capi.csr_sampling(indptr, indices, seeds, 10, False)
    assert torch.equal(p0, p1) and torch.equal(x0, x1)
