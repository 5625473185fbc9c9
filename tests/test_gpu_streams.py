"""Calls issued from different torch streams get different libshmt contexts, so mini-batches,
relabels and scans that overlap on the GPU do not share look-back state, result words or the
relabel table.  Two host threads, one stream each, run mini-batches at the same time; every
result must be a legal sample with the oracle's relabel, exactly as when run alone."""
import threading

import numpy as np
import pytest
import torch

from oracle import oracle

pytestmark = pytest.mark.gpu


def _graph(rng, n, mean_deg):
    deg = np.minimum((rng.pareto(1.3, size=n) * mean_deg / 3).astype(np.int64), 400)
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    indices = np.concatenate([rng.choice(n, size=d, replace=False) for d in deg]).astype(np.int32)
    return indptr, indices


def test_one_context_per_stream():
    from shmtensor_b200 import capi
    dev = torch.device("cuda", 0)
    a, b = torch.cuda.Stream(), torch.cuda.Stream()
    with torch.cuda.stream(a):
        ca = capi._ctx(dev)
    with torch.cuda.stream(b):
        cb = capi._ctx(dev)
        capi.reserve_minibatch(512, [5, 10, 15])
        assert capi.context_scratch_bytes() >= 16 * (512 * 6 * 11 * 16) // 1024
    assert ca != cb and capi._ctx(dev) not in (ca, cb)
    with torch.cuda.stream(a):
        assert capi._ctx(dev) == ca


def test_minibatches_on_two_streams_at_once():
    from shmtensor_b200 import capi
    rng = np.random.default_rng(8)
    indptr_n, indices_n = _graph(rng, 30_000, 30)
    indptr, indices = torch.from_numpy(indptr_n).cuda(), torch.from_numpy(indices_n).cuda()
    fan = [5, 10, 15]
    results, errors = {}, []

    def worker(tag, seed):
        try:
            stream = torch.cuda.Stream()
            r = np.random.default_rng(seed)
            out = []
            with torch.cuda.stream(stream):
                for _ in range(25):
                    seeds_n = r.integers(0, 30_000, size=700).astype(np.int32)
                    _, hops = capi.sample_minibatch(indptr, indices, torch.from_numpy(seeds_n).cuda(), fan, False)
                    scan = torch.ones(300_000, dtype=torch.int32, device="cuda")
                    capi.thrust_scan(scan)                       # same context, same stream, in between
                    uniq, (rel,) = capi.tensor_relabel([hops[-1][1]])
                    stream.synchronize()
                    out.append((seeds_n, [tuple(t.cpu().numpy() for t in h) for h in hops], scan[-1].item(),
                                uniq.cpu().numpy(), rel.cpu().numpy()))
            results[tag] = out
        except Exception as exc:  # noqa: BLE001
            errors.append((tag, exc))

    threads = [threading.Thread(target=worker, args=(t, 100 + t)) for t in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    for tag in range(2):
        for seeds_n, hops, scan_last, uniq, rel in results[tag]:
            cur = seeds_n
            for (sp, sx, r, nxt), k in zip(hops, fan):
                oracle.check_sample_bulk(indptr_n, indices_n, cur, k, False, sp, sx, distinct_rows=True)
                wu, (_, wx) = oracle.tensor_relabel([cur, sx])
                assert np.array_equal(nxt, wu) and np.array_equal(r, wx)
                cur = wu
            assert scan_last == 300_000
            wu, (wr,) = oracle.tensor_relabel([hops[-1][1]])
            assert np.array_equal(uniq, wu) and np.array_equal(rel, wr)
    assert capi.device_fault() == 0
