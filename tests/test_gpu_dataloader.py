"""Multi-hop mini-batches through GPUSamplingDataloader (reference: python/shmtensor/sampling.py)."""
import numpy as np
import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu


def _graph(n_nodes=20_000, seed=0):
    rng = np.random.default_rng(seed)
    deg = np.minimum((rng.pareto(1.3, size=n_nodes) * 4).astype(np.int64), 2000)
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    indices = rng.integers(0, n_nodes, size=int(indptr[-1])).astype(np.int64)
    return indptr, indices


@pytest.mark.parametrize("cached", [False, True])
def test_three_hop_batches_are_consistent(cached):
    from shmtensor_b200 import GPUSamplingDataloader
    indptr_n, indices_n = _graph()
    indptr, indices = torch.from_numpy(indptr_n), torch.from_numpy(indices_n)
    dl = GPUSamplingDataloader(indptr, indices, torch.arange(0, 4096), 1024, [15, 10, 5],
                               shuffle=False)
    if cached:
        hotness = torch.from_numpy(np.diff(indptr_n).astype(np.float32))
        dl.create_cache(int((indptr.nbytes + indices.nbytes) * 0.5), hotness)
        assert dl.has_cache and dl.hashmap.key_dtype == torch.int32
        assert dl.indptr.is_cuda and not dl.indices.is_cuda      # offsets on the GPU, cold rows on the host
    assert len(dl) == 4
    deg = np.diff(indptr_n)
    n_batches = 0
    for input_nodes, output_nodes, blocks in dl:
        assert len(blocks) == 3 and output_nodes.numel() == 1024
        assert torch.equal(output_nodes.cpu(), torch.arange(n_batches * 1024, (n_batches + 1) * 1024))
        n_batches += 1
        # hops are sampled over reversed(num_picks); blocks[-1] is the first one sampled
        n_dst_expected = 1024
        for (sub_indptr, rel, n_src, n_dst), k in zip(reversed(blocks), (5, 10, 15)):
            assert n_dst == n_dst_expected and sub_indptr.numel() == n_dst + 1
            assert rel.numel() == sub_indptr[-1].item() and n_src >= n_dst
            assert rel.min().item() >= 0 and rel.max().item() < n_src
            assert (np.diff(sub_indptr.cpu().numpy()) <= k).all()
            n_dst_expected = n_src
        assert input_nodes.numel() == n_dst_expected
        # seeds are unique, so every frontier starts with the previous one, in order
        assert torch.equal(input_nodes[:1024], output_nodes)
        first_ptr = blocks[-1][0].cpu().numpy()
        assert np.array_equal(np.diff(first_ptr), np.minimum(deg[output_nodes.cpu().numpy()], 5))
        assert torch.unique(input_nodes).numel() == input_nodes.numel()
    assert n_batches == 4


def test_relabel_contract_inside_the_loader():
    """One hop done by hand: frontier == oracle relabel of [seeds, sub_indices]."""
    from shmtensor_b200 import capi
    indptr_n, indices_n = _graph(seed=1)
    indptr, indices = torch.from_numpy(indptr_n).cuda(), torch.from_numpy(indices_n).cuda()
    seeds = torch.randperm(20_000, device="cuda")[:1024]
    p, x = capi.csr_sampling(indptr, indices, seeds, 10, False)
    uniq, (rs, rx) = capi.tensor_relabel([seeds, x])
    wu, (ws, wx) = oracle.tensor_relabel([seeds.cpu().numpy(), x.cpu().numpy()])
    assert np.array_equal(uniq.cpu().numpy(), wu)
    assert np.array_equal(rs.cpu().numpy(), ws) and np.array_equal(rx.cpu().numpy(), wx)
    assert torch.equal(rs, torch.arange(1024, device="cuda"))   # seeds are unique and come first
    assert torch.equal(uniq[rx], x)


def test_presampling_and_weight_size():
    from shmtensor_b200 import GPUSamplingDataloader
    indptr_n, indices_n = _graph(5000, seed=2)
    dl = GPUSamplingDataloader(torch.from_numpy(indptr_n), torch.from_numpy(indices_n),
                               torch.arange(2000), 500, [5, 5], shuffle=True, drop_last=True)
    s_hot, f_hot = dl.presampling()
    assert s_hot.shape == (5000,) and f_hot.shape == (5000,)
    assert s_hot.sum() >= 2000 and (f_hot >= s_hot).all()
    full, item = dl.compute_weight_size(f_hot)
    assert full == indptr_n.nbytes + indices_n.nbytes and item > 0


@pytest.mark.parametrize("cached", [False, True])
@pytest.mark.parametrize("idx_dtype", [torch.int32, torch.int64])
def test_fused_minibatch_equals_hop_by_hop(cached, idx_dtype):
    """shmt_sample_minibatch queues all hops without a host round trip; with the same Philox key
    and call counter it must return exactly what the per-hop calls return."""
    from shmtensor_b200 import capi
    indptr_n, indices_n = _graph(30_000, seed=3)
    indptr = torch.from_numpy(indptr_n)
    indices = torch.from_numpy(indices_n).to(idx_dtype)
    capi.pin_memory(indptr)
    capi.pin_memory(indices)
    try:
        gp = gi = hmap = None
        if cached:
            hot = torch.from_numpy(np.argsort(-np.diff(indptr_n))[:6000].copy()).cuda()
            gp, gi = capi.create_subcsr(indptr, indices, hot)
            hmap = capi.CUCOStaticHashmap(hot.int(), torch.arange(6000, dtype=torch.int32, device="cuda"), 0.8)
        # the last case's third relabel is sized for 8192 * 11 * 11 * 6 = 5.9 M ids: the fused path then
        # takes the large-tile compact kernel where the per-hop calls (sized by the real counts) do not
        for n_seeds, fanouts in ((1024, [5, 10, 15]), (1, [3]), (333, [40, 2]), (8192, [10, 10, 5])):
            seeds = torch.randperm(30_000, device="cuda")[:n_seeds].to(idx_dtype)
            capi.set_sampling_seed(4242)
            want, cur = [], seeds
            for k in fanouts:
                if cached:
                    p, x = capi.csr_cache_sampling(indptr, indices, gp, gi, hmap, cur, k, False)
                else:
                    p, x = capi.csr_sampling(indptr, indices, cur, k, False)
                nxt, (_, rx) = capi.tensor_relabel([cur, x])
                want.append((p, x, rx, nxt))
                cur = nxt
            capi.set_sampling_seed(4242)
            frontier, hops = capi.sample_minibatch(indptr, indices, seeds, fanouts, False, gp, gi, hmap)
            assert torch.equal(frontier, cur) and len(hops) == len(fanouts)
            for (p, x, rx, nxt), (p2, x2, rx2, nxt2) in zip(want, hops):
                assert torch.equal(p, p2) and torch.equal(x, x2)
                assert torch.equal(rx, rx2) and torch.equal(nxt, nxt2)
            # twice in a row: the relabel table must come back clean
            capi.set_sampling_seed(4242)
            frontier2, _ = capi.sample_minibatch(indptr, indices, seeds, fanouts, False, gp, gi, hmap)
            assert torch.equal(frontier2, frontier)
    finally:
        capi.unpin_memory(indptr)
        capi.unpin_memory(indices)


@pytest.mark.parametrize("fused", [True, False])
def test_blocks_with_edge_ids(fused):
    """`with_edge_ids`: every block carries, for each sampled neighbour, its position in `indices`,
    with and without a cache (the reference passes an empty edge-id tensor to its block builder)."""
    from shmtensor_b200 import GPUSamplingDataloader
    rng = np.random.default_rng(6)
    deg = np.minimum((rng.pareto(1.3, size=3000) * 5).astype(np.int64), 300)
    indptr_n = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    indices_n = rng.integers(0, 3000, size=int(indptr_n[-1])).astype(np.int64)
    indptr, indices = torch.from_numpy(indptr_n), torch.from_numpy(indices_n)
    dl = GPUSamplingDataloader(indptr, indices, torch.arange(0, 1024), 256, [6, 3], shuffle=False, fused=fused,
                               with_edge_ids=True)
    dl.create_cache(int(indices.nbytes * 0.4), torch.from_numpy(deg.astype(np.float32)))
    assert dl.has_cache and dl.gpu_edge_base is not None
    flat = torch.from_numpy(indices_n).cuda()
    n = 0
    for frontier, output_nodes, blocks in dl:
        # blocks[0] is the outermost hop; walk from the seeds outwards
        src = frontier
        for sub_indptr, relabel_indices, n_src, n_dst, eids in blocks:
            assert eids.numel() == relabel_indices.numel() == int(sub_indptr[-1])
            # an edge id names the neighbour the relabelled index stands for
            assert torch.equal(flat[eids], src[relabel_indices.long()].long())
            src = src[:n_dst]
        n += 1
    assert n == 4
    del dl


@pytest.mark.parametrize("fused", [True, False])
def test_loader_on_its_own_stream_yields_the_same_batches(fused):
    """own_stream=True: sampling runs on the loader's stream while the caller's stream works on the
    batch before; every batch equals the one the plain loader yields, and what the caller computes
    from a batch on its own stream sees finished tensors."""
    from shmtensor_b200 import GPUSamplingDataloader, capi
    indptr_n, indices_n = _graph(seed=5)
    hotness = torch.from_numpy(np.diff(indptr_n).astype(np.float32))
    feats = torch.randn(20_000, 64, device="cuda")
    runs = []
    for own in (False, True):
        # a loader registers its host arrays for the GPU: each gets arrays of its own
        indptr, indices = torch.from_numpy(indptr_n.copy()), torch.from_numpy(indices_n.copy())
        dl = GPUSamplingDataloader(indptr, indices, torch.arange(0, 8192), 1024, [15, 10, 5], shuffle=False,
                                   fused=fused, own_stream=own)
        dl.create_cache(int((indptr.nbytes + indices.nbytes) * 0.5), hotness)
        capi.set_sampling_seed(99)
        out = []
        for _ in range(2):  # two epochs: the second re-enters __iter__ with work still queued
            for input_nodes, output_nodes, blocks in dl:
                # consumer work queued on the caller's stream, not waited for before the next batch
                pooled = feats[input_nodes.long()].sum(0)
                for _ in range(20):
                    pooled = pooled + feats[input_nodes.long()].sum(0)
                out.append((input_nodes, [b[0] for b in blocks], [b[1] for b in blocks], pooled))
        torch.cuda.synchronize()
        runs.append(out)
    assert len(runs[0]) == len(runs[1]) == 16
    for a, b in zip(*runs):
        assert torch.equal(a[0], b[0]) and torch.equal(a[3], b[3])
        assert all(torch.equal(x, y) for x, y in zip(a[1], b[1]))
        assert all(torch.equal(x, y) for x, y in zip(a[2], b[2]))
    capi.check_async()


@pytest.mark.parametrize("cached", [False, True])
def test_loader_with_edge_weights(cached):
    """edge_weights: every hop picks in proportion to the weights; the fused loader and the
    call-per-hop loader yield the same batches, and an edge of weight ~0 next to heavy ones
    is (almost) never taken from a long row."""
    from shmtensor_b200 import GPUSamplingDataloader, capi
    indptr_n, indices_n = _graph(seed=8)
    rng = np.random.default_rng(8)
    w_n = (rng.random(indices_n.size) + 0.5).astype(np.float32)
    light = rng.random(indices_n.size) < 0.5
    w_n[light] = 1e-12
    hotness = torch.from_numpy(np.diff(indptr_n).astype(np.float32))
    runs = []
    for fused in (True, False):
        indptr, indices = torch.from_numpy(indptr_n.copy()), torch.from_numpy(indices_n.copy())
        dl = GPUSamplingDataloader(indptr, indices, torch.arange(0, 3072), 1024, [4, 6], shuffle=False, fused=fused,
                                   edge_weights=torch.from_numpy(w_n.copy()))
        if cached:
            dl.create_cache(int((indptr.nbytes + indices.nbytes) * 0.5), hotness)
            assert dl.has_cache and dl.gpu_weights is not None and dl.gpu_weights.numel() == dl.gpu_indices.numel()
        capi.set_sampling_seed(55)
        runs.append([(inp, [b[0] for b in blocks], [b[1] for b in blocks]) for inp, _, blocks in dl])
    torch.cuda.synchronize()
    assert len(runs[0]) == len(runs[1]) == 3
    for a, b in zip(*runs):
        assert torch.equal(a[0], b[0])
        assert all(torch.equal(x, y) for x, y in zip(a[1], b[1])) and all(torch.equal(x, y) for x, y in zip(a[2], b[2]))
    # first hop of one batch by hand: rows with at least 4 heavy edges among many yield heavy edges only
    seeds = torch.arange(0, 1024, device="cuda")
    p, x, e = capi.csr_weighted_sampling(torch.from_numpy(indptr_n).cuda(), torch.from_numpy(indices_n).cuda(),
                                         torch.from_numpy(w_n).cuda(), seeds, 4, False, return_eids=True)
    picked_light = light[e.cpu().numpy()]
    row_of = np.repeat(np.arange(1024), np.diff(p.cpu().numpy()))
    n_heavy = np.array([(~light[indptr_n[r]:indptr_n[r + 1]]).sum() for r in range(1024)])
    deg = np.diff(indptr_n)[:1024]
    strict = (n_heavy[row_of] >= 4) & (deg[row_of] > 4)
    assert strict.sum() > 100 and picked_light[strict].sum() == 0
    with pytest.raises(RuntimeError, match="fused=False"):
        GPUSamplingDataloader(torch.from_numpy(indptr_n.copy()), torch.from_numpy(indices_n.copy()), torch.arange(8), 4,
                              [2], with_edge_ids=True, edge_weights=torch.from_numpy(w_n.copy()))
