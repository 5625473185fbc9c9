"""Partitioned feature cache: host-side plan on two gloo ranks (CPU), fetch on one GPU."""
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent

WORKER = textwrap.dedent("""
    import sys, torch, torch.distributed as dist
    sys.path.insert(0, {root!r})
    from shmtensor_b200.partition import plan_partition, owner_of, OWNER_SHIFT
    dist.init_process_group(backend='gloo', init_method='env://')
    rank, world = dist.get_rank(), dist.get_world_size()
    g = torch.Generator().manual_seed(5)
    ids = torch.randperm(1_000_000, generator=g)[:50_000]
    owner, slot, counts = plan_partition(ids, world)
    # every rank computes the same plan
    digest = torch.stack([owner.sum(), slot.sum(), torch.tensor(counts).sum()])
    gathered = [torch.zeros_like(digest) for _ in range(world)]
    dist.all_gather(gathered, digest)
    assert all(torch.equal(t, digest) for t in gathered)
    assert sum(counts) == ids.numel() and min(counts) > 0.4 * ids.numel() / world
    # slots are dense per owner, in the order the ids appear
    mine = owner == rank
    assert torch.equal(slot[mine], torch.arange(counts[rank]))
    assert torch.equal(owner, owner_of(ids, world)) and int(slot.max()) < (1 << OWNER_SHIFT)
    # the directory value decodes back to (owner, slot)
    v = (owner << OWNER_SHIFT) | slot
    assert torch.equal(v >> OWNER_SHIFT, owner) and torch.equal(v & ((1 << OWNER_SHIFT) - 1), slot)
    # the shard sizes every rank expects match what each owner would allocate
    c = torch.tensor([counts[rank]])
    allc = [torch.zeros_like(c) for _ in range(world)]
    dist.all_gather(allc, c)
    assert [int(x) for x in allc] == counts
    dist.barrier()
    print('rank', rank, 'ok')
""")


def test_partition_plan_agrees_across_two_gloo_ranks(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(root=str(ROOT)))
    port = 31500 + os.getpid() % 2000
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), OMP_NUM_THREADS="1")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=180)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)


def test_owner_hash_spreads_degree_sorted_ids():
    from shmtensor_b200.partition import owner_of
    ids = torch.arange(0, 80_000)            # consecutive ids, the worst case for a modulo
    for world in (2, 4, 8):
        counts = torch.bincount(owner_of(ids, world), minlength=world)
        assert counts.min() > 0.9 * 80_000 / world


@pytest.mark.gpu
def test_partitioned_fetch_single_rank_is_bit_exact():
    from shmtensor_b200 import capi
    from shmtensor_b200.partition import PartitionedFeatureCache
    rng = np.random.default_rng(4)
    table_n = rng.standard_normal((50_000, 100)).astype(np.float32)
    table = torch.from_numpy(table_n.copy())
    capi.pin_memory(table)
    try:
        cached = torch.from_numpy(rng.choice(50_000, size=10_000, replace=False))
        pc = PartitionedFeatureCache(table, cached)
        assert pc.world == 1 and pc.counts == [10_000]
        q = torch.from_numpy(rng.integers(0, 50_000, size=20_001)).cuda()
        out = pc.fetch(q)
        assert torch.equal(out.cpu().view(torch.int32), table[q.cpu()].view(torch.int32))
        # hits come from the shard: change it and see the change
        pc.shard += 1.0
        out2 = pc.fetch(cached[:100].cuda())
        assert torch.equal(out2.cpu(), table[cached[:100]] + 1.0)
        assert capi.device_fault() == 0
        pc.close()
    finally:
        capi.unpin_memory(table)
