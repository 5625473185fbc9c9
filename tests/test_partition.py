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
    from shmtensor_b200.partition import plan_partition, plan_directory, owner_of, OWNER_SHIFT
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
    # with the 1000 hottest ids replicated: every rank resolves them to its own shard, the other
    # ids to the same (owner, slot) everywhere, and each rank's rows are dense in slot order
    values, mine, pcounts, rep = plan_directory(ids, world, rank, 1000)
    low = (1 << OWNER_SHIFT) - 1
    assert rep == 1000 and sum(pcounts) == ids.numel() - 1000
    assert bool(((values[:1000] >> OWNER_SHIFT) == rank).all())
    assert torch.equal(values[:1000] & low, pcounts[rank] + torch.arange(1000))
    assert torch.equal(mine[pcounts[rank]:], ids[:1000]) and mine.numel() == pcounts[rank] + 1000
    shared = values[1000:].clone()
    allv = [torch.zeros_like(shared) for _ in range(world)]
    dist.all_gather(allv, shared)
    assert all(torch.equal(t, shared) for t in allv)
    own = (shared >> OWNER_SHIFT) == rank
    assert torch.equal(ids[1000:][own], mine[:pcounts[rank]])
    assert torch.equal(shared[own] & low, torch.arange(pcounts[rank]))
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


def test_directory_plan_single_rank_and_default_replication():
    from shmtensor_b200.partition import OWNER_SHIFT, default_replication, plan_directory
    ids = torch.randperm(10_000)[:3000]
    values, mine, counts, rep = plan_directory(ids, 1, 0, 500)   # one rank: nothing to replicate
    assert rep == 0 and counts == [3000] and torch.equal(mine, ids)
    assert torch.equal(values, torch.arange(3000))
    assert default_replication(480_000, 1) == 0
    assert default_replication(480_000, 4) == 15_000 and default_replication(2000, 8) == 1024
    assert default_replication(500, 8) == 500
    from shmtensor_b200.partition import head_for_mass
    assert head_for_mass(torch.tensor([5.0, 3.0, 1.0, 1.0]), 0.5) == 1      # 5 of 10 is half
    assert head_for_mass(torch.tensor([5.0, 3.0, 1.0, 1.0]), 0.8) == 2
    assert head_for_mass(torch.tensor([5.0, 3.0, 1.0, 1.0]), 1.0) == 4
    assert head_for_mass(torch.tensor([]), 0.5) == 0 and head_for_mass(torch.ones(7), 0.0) == 0
    zipf = 1.0 / torch.arange(1, 480_001, dtype=torch.float64) ** 1.1
    assert head_for_mass(zipf, 0.5) < 200                                   # a skewed stream's head is tiny
    # more replicas than ids: everything is replicated
    values, mine, counts, rep = plan_directory(ids, 4, 2, 10_000)
    assert rep == 3000 and counts == [0, 0, 0, 0] and torch.equal(mine, ids)
    assert torch.equal(values, (2 << OWNER_SHIFT) | torch.arange(3000))


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
        # turnover in place: a fifth of the cached ids leave, other ids take their rows
        pc.shard.copy_(table[cached].cuda())
        others = torch.from_numpy(np.setdiff1d(np.arange(50_000), cached.numpy())[:2_000])
        # (ten of them listed twice: an id is evicted once, and the pairing stays deterministic)
        assert pc.replace(torch.cat([cached[:2_000], cached[:10]]), others) == 2_000 and pc.directory.size() == 10_000
        assert bool((pc.directory.query(cached[:2_000].cuda()) == -1).all())
        rows = pc.directory.query(others.cuda())
        assert bool((rows >= 0).all()) and torch.equal(pc.shard[rows].cpu(), table[others])
        assert torch.equal(pc.fetch(q).cpu().view(torch.int32), table[q.cpu()].view(torch.int32))
        pc.close()
    finally:
        capi.unpin_memory(table)


@pytest.mark.gpu
def test_two_ranks_emulated_on_one_gpu_with_replicated_hot_rows():
    """Both ranks' shards and directories built in one process on one GPU (nothing waits on
    another launch), fetched through the same entry point the multi-GPU cache uses."""
    import ctypes as C

    from shmtensor_b200 import capi
    from shmtensor_b200._lib import check, lib
    from shmtensor_b200.partition import OWNER_SHIFT, plan_directory
    rng = np.random.default_rng(9)
    table_n = rng.standard_normal((30_000, 64)).astype(np.float32)
    table = torch.from_numpy(table_n.copy())
    capi.pin_memory(table)
    try:
        cached = torch.from_numpy(rng.choice(30_000, size=8_000, replace=False))
        world, rep = 2, 500
        shards, dirs = [], []
        for r in range(world):
            values, mine, counts, got_rep = plan_directory(cached, world, r, rep)
            assert got_rep == rep and mine.numel() == counts[r] + rep
            shards.append(capi.uva_fetch(table, mine.cuda()) + float(r + 1))  # tagged: +1 / +2
            dirs.append(capi.CUCOStaticHashmap(cached.cuda(), values.cuda(), 0.5))
        bases = (C.c_void_p * world)(*[s.data_ptr() for s in shards])
        q_n = np.concatenate([cached.numpy()[rng.integers(0, 8_000, size=20_000)],
                              rng.integers(0, 30_000, size=5_000)])
        q = torch.from_numpy(q_n).cuda()
        for r in range(world):
            out = torch.empty((q.numel(), 64), dtype=torch.float32, device="cuda")
            check(lib.shmt_fetch_partitioned(dirs[r]._handle, bases, world, OWNER_SHIFT, table.data_ptr(),
                                             q.data_ptr(), 1, q.numel(), 256, out.data_ptr(),
                                             torch.cuda.current_stream().cuda_stream))
            # expected tag per row: 0 for misses, own tag for replicated ids, the owner's tag otherwise
            v = dirs[r].query(q).cpu()
            tag = torch.where(v >= 0, (v >> OWNER_SHIFT) + 1, torch.zeros_like(v)).to(torch.float32)
            assert torch.equal(out.cpu(), table[q.cpu()] + tag[:, None])
            is_rep = torch.isin(q.cpu(), cached[:rep])
            assert bool((tag[is_rep] == r + 1).all()) and bool(is_rep.any())
        assert capi.device_fault() == 0
    finally:
        capi.unpin_memory(table)
