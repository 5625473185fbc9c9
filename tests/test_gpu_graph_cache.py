"""Turnover of the cached sub-graph: rows leave and enter the GPU cache in place, and sampling
through the cache stays what sampling the host CSR gives (the reference rebuilds the whole cached
CSR to change it, src/cache_graph_sampling.cu:455-492)."""
import numpy as np
import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu


def _graph(rng, n):
    deg = np.minimum((rng.pareto(1.1, size=n) * 5).astype(np.int64), 3000)
    deg[:5] = [0, 1, 8, 9, 3000]
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    indices = np.concatenate([rng.choice(n, size=d, replace=False) for d in deg]).astype(np.int32)
    return deg, indptr, indices


def _check_rows(gc, nodes_n, indptr_n, indices_n):
    v = gc.hashmap.query(torch.from_numpy(nodes_n).cuda())
    assert bool((v >= 0).all()) and bool((v % 2 == 0).all())
    b = gc.bounds[v].cpu().numpy()
    e = gc.bounds[v + 1].cpu().numpy()
    arena = gc.arena.cpu().numpy()
    assert np.array_equal(e - b, indptr_n[nodes_n + 1] - indptr_n[nodes_n])
    for i in np.random.default_rng(0).integers(0, nodes_n.size, size=min(400, nodes_n.size)):
        r = nodes_n[i]
        assert np.array_equal(arena[b[i]:e[i]], indices_n[indptr_n[r]:indptr_n[r + 1]])


def test_graph_cache_samples_like_the_host_graph_through_many_turnovers():
    from shmtensor_b200 import GraphCache, capi
    rng = np.random.default_rng(33)
    n = 20_000
    deg, indptr_n, indices_n = _graph(rng, n)
    indptr, indices = torch.from_numpy(indptr_n), torch.from_numpy(indices_n)
    capi.pin_memory(indptr)
    capi.pin_memory(indices)
    try:
        cached = np.concatenate([np.arange(5), rng.choice(np.arange(5, n), size=3995, replace=False)])
        gc = GraphCache(indptr, indices, torch.from_numpy(cached).cuda())
        _check_rows(gc, cached, indptr_n, indices_n)
        seeds_n = rng.integers(0, n, size=5000)
        seeds = torch.from_numpy(seeds_n).cuda()
        used_after_first_rounds = None
        for rnd in range(30):
            capi.set_sampling_seed(100 + rnd)
            p, x = capi.csr_cache_sampling(indptr, indices, gc.gpu_indptr, gc.gpu_indices, gc.hashmap, seeds, 10, False)
            capi.set_sampling_seed(100 + rnd)
            p0, x0 = capi.csr_sampling(indptr, indices, seeds, 10, False)       # no cache: same draws
            assert torch.equal(p, p0) and torch.equal(x, x0), rnd
            _, hops = capi.sample_minibatch(indptr, indices, seeds[:512].int(), [5, 10], False, gc.gpu_indptr,
                                            gc.gpu_indices, gc.hashmap)
            cur = seeds_n[:512].astype(np.int32)
            for (sp, sx, rel, nxt), k in zip(hops, (5, 10)):
                oracle.check_sample_bulk(indptr_n, indices_n, cur, k, False, sp.cpu().numpy(), sx.cpu().numpy(),
                                         distinct_rows=True)
                cur = nxt.cpu().numpy()
            # a third of the cached nodes leave, as many others enter (some listed twice)
            leave = rng.choice(cached, size=1300, replace=False)
            pool = np.setdiff1d(np.arange(n), cached)
            enter = rng.choice(pool, size=1300, replace=False)
            got = gc.replace(torch.from_numpy(np.concatenate([leave, leave[:7]])).cuda(), torch.from_numpy(enter).cuda())
            assert got == 1300 and gc.rows() == 4000
            cached = np.concatenate([np.setdiff1d(cached, leave), enter])
            assert bool((gc.hashmap.query(torch.from_numpy(leave).cuda()) == -1).all())
            _check_rows(gc, cached, indptr_n, indices_n)
            if rnd == 9:
                used_after_first_rounds = gc.arena_used()
        # freed blocks are taken again: the arena does not keep growing with the number of turnovers
        assert gc.arena_used() <= 1.5 * used_after_first_rounds
    finally:
        torch.cuda.synchronize()
        capi.unpin_memory(indptr)
        capi.unpin_memory(indices)


def test_graph_cache_refuses_what_does_not_fit():
    from shmtensor_b200 import GraphCache
    indptr = torch.tensor([0, 4, 8, 1008, 1012], dtype=torch.int64, device="cuda")
    indices = torch.arange(1012, dtype=torch.int32, device="cuda")
    gc = GraphCache(indptr, indices, torch.tensor([0, 1], device="cuda"), arena_elements=64)
    with pytest.raises(RuntimeError, match="arena is full"):
        gc.replace(torch.tensor([0], device="cuda"), torch.tensor([2], device="cuda"))   # a 1,000-neighbour row
    assert gc.replace(torch.tensor([1], device="cuda"), torch.tensor([3], device="cuda")) == 1
    v = gc.hashmap.query(torch.tensor([3], device="cuda"))
    assert gc.arena[gc.bounds[v]:gc.bounds[v + 1]].tolist() == [1008, 1009, 1010, 1011]


def test_dataloader_with_a_replaceable_cache():
    from shmtensor_b200 import GPUSamplingDataloader, capi
    rng = np.random.default_rng(2)
    deg, indptr_n, indices_n = _graph(rng, 8000)
    indptr, indices = torch.from_numpy(indptr_n), torch.from_numpy(indices_n)
    dl = GPUSamplingDataloader(indptr, indices, torch.arange(0, 2048), 512, [10, 5], shuffle=False)
    hotness = torch.from_numpy(deg.astype(np.float32))
    dl.create_cache(int(indices.nbytes * 0.3), hotness, replaceable=True)
    assert dl.has_cache and dl.graph_cache.rows() > 0
    is_cached = dl.hashmap.query(torch.arange(8000, device="cuda")) >= 0
    cached = is_cached.nonzero(as_tuple=True)[0]
    assert cached.numel() == dl.graph_cache.rows() >= 8      # the hottest rows are the longest: few fit
    n_swap = cached.numel() // 2
    # rows without neighbours or with few of them always fit into what the evicted rows free
    small = ((~is_cached) & torch.from_numpy(deg <= 8).cuda()).nonzero(as_tuple=True)[0][:n_swap]
    assert dl.replace_cache(cached[-n_swap:], small) == n_swap
    assert bool((dl.hashmap.query(small) >= 0).all()) and bool((dl.hashmap.query(cached[-n_swap:]) == -1).all())
    for frontier, output_nodes, blocks in dl:
        cur = output_nodes.cpu().numpy()
        for (sub_indptr, relabel_indices, n_src, n_dst) in reversed(blocks):
            assert sub_indptr.numel() == n_dst + 1 and int(relabel_indices.max()) < n_src
        assert frontier.numel() == blocks[0][2]
    del dl
