#!/usr/bin/env python
"""Benchmark of the cached feature fetch (the hot path's headline metric).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (one step = one batch through the fused probe+gather kernel): a pinned host table of
2,400,000 x 100 float32 rows, N(0,1); the top 20 % of rows by a seeded power-law score are
cached in HBM behind a static hashmap (int64 keys -> int32 slots, load factor 0.5); each
batch is 500,000 int64 ids, rank-Zipf(1.1) over the score ranking mixed with uniform rows so
that about 80 % hit the cache; misses are read from the host table through UVA.  With N > 1
ranks (torchrun), the cached rows are hash-partitioned over the GPUs and remote hits are read
over NVLink by the same kernel; every rank runs its own batches (weak scaling).

Prints one JSON line (rank 0).  ``value`` times the kernel with ids already on the GPU;
``e2e`` times the public call with the ids starting in pinned host memory and a read-back of
the last fetched row.  ``--impl reference`` times the reference's CPU path for the same
fetch (``data[q]`` = torch.index_select on the host table, example/test_cache_fetch.py:138)
on the host cores.  Data is synthetic and seeded.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

ROWS, DIM, BATCH = 2_400_000, 100, 500_000
CACHE_FRACTION, LOAD_FACTOR, ZIPF_ALPHA, UNIFORM_SHARE = 0.20, 0.5, 1.1, 0.21
ROW_BYTES = DIM * 4
N_BATCHES = 8
METRIC, UNIT = "fetched feature GB/s", "GB/s"
NCU_DRAM_BYTES_PER_LAUNCH = 210_300_000  # 63.8 MB read + 146.5 MB written (ncu, headline batch)
WORKLOAD = ("1-GPU cached feature fetch: pinned 2,400,000x100 f32 host table, top 20% rows cached "
            "behind int64->int32 map (load 0.5), 500,000 int64 ids/batch Zipf(1.1), ~80% hits, misses via UVA")


# --------------------------------------------------------------------------- synthetic data
def make_scores(seed: int = 2024) -> np.ndarray:
    """Seeded power-law 'degree' score per row (Pareto tail, like node degrees)."""
    rng = np.random.default_rng(seed)
    return rng.pareto(1.1, size=ROWS) + rng.random(ROWS) * 1e-6


def make_batches(ranking: np.ndarray, n_batches: int, seed: int) -> list:
    """Query batches: rank-Zipf(ZIPF_ALPHA) over the score ranking, mixed with uniform rows."""
    rng = np.random.default_rng(seed)
    w = 1.0 / np.arange(1, ROWS + 1, dtype=np.float64) ** ZIPF_ALPHA
    cdf = np.cumsum(w)
    cdf /= cdf[-1]
    out = []
    n_uniform = int(BATCH * UNIFORM_SHARE)
    for _ in range(n_batches):
        ranks = np.searchsorted(cdf, rng.random(BATCH - n_uniform))
        ids = np.concatenate([ranking[np.minimum(ranks, ROWS - 1)], rng.integers(0, ROWS, size=n_uniform)])
        rng.shuffle(ids)
        out.append(torch.from_numpy(ids.astype(np.int64)))
    return out


def fill_table(t: torch.Tensor, seed: int = 7) -> None:
    g = torch.Generator().manual_seed(seed)
    chunk = 200_000
    for lo in range(0, t.shape[0], chunk):
        t[lo:lo + chunk].normal_(generator=g)


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """Polls SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.05):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
            self._thread = threading.Thread(target=self._run, args=(period_s,), daemon=True)
        except Exception:
            self._nv = None

    def _run(self, period_s):
        nv = self._nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            self._stop.wait(period_s)

    def start(self):
        if self._thread:
            self._thread.start()

    def stop(self) -> dict:
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=2)
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


# --------------------------------------------------------------------------- helpers
def measured_peaks() -> tuple:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return float(json.loads(p.read_text())["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s)"


def time_launches(fn, n: int, stream) -> float:
    """Mean device time in ms of n calls of fn, one CUDA-event pair per call."""
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
    torch.cuda.synchronize()
    for a, b in evs:
        a.record(stream)
        fn()
        b.record(stream)
    torch.cuda.synchronize()
    return sum(a.elapsed_time(b) for a, b in evs) / n


def hbm_bytes(n: int, n_hit: int) -> int:
    """Algorithmic HBM bytes of one fetch launch: per query id 8 + probe 12 (int64 key + int32
    slot) + the row written; hit rows are also read from HBM."""
    return n * (8 + 12) + n_hit * ROW_BYTES + n * ROW_BYTES


def measure_host_link(table: torch.Tensor, stream) -> dict:
    """Host-link ceiling, measured here: pinned H2D copy and a streaming UVA read kernel."""
    from shmtensor_b200._lib import check, lib
    nbytes = min(table.numel() * 4, 1 << 30)
    dst = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    src = table.view(torch.uint8).reshape(-1)[:nbytes]
    best_copy = min(time_launches(lambda: dst.copy_(src, non_blocking=True), 1, stream) for _ in range(5))
    sink = torch.zeros(1, dtype=torch.int64, device="cuda")
    ptr = table.data_ptr()
    best_read = min(time_launches(
        lambda: check(lib.shmt_stream_read(ptr, nbytes, sink.data_ptr(), stream.cuda_stream)), 1, stream)
        for _ in range(5))
    copy_gbs, read_gbs = nbytes / best_copy / 1e6, nbytes / best_read / 1e6
    return {"h2d_copy_gbs": round(copy_gbs, 2), "uva_read_kernel_gbs": round(read_gbs, 2),
            "peak_gbs": round(max(copy_gbs, read_gbs), 2)}


_REAL_STDOUT = None


def quiet_stdout() -> None:
    """Send everything libraries print on stdout (NCCL's version banner, for one) to stderr;
    stdout then carries nothing but the one JSON line written by emit()."""
    global _REAL_STDOUT
    if _REAL_STDOUT is None:
        sys.stdout.flush()
        _REAL_STDOUT = os.dup(1)
        os.dup2(2, 1)


def emit(line: dict) -> None:
    data = (json.dumps(line) + "\n").encode()
    if _REAL_STDOUT is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_REAL_STDOUT, data)


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


# --------------------------------------------------------------------------- reference arm
def run_reference(args) -> None:
    """The reference's CPU path for this fetch, on the host cores: torch.index_select over the
    host table (its ``cpu_fetch`` line).  Rank 0 only; no GPU work."""
    rank, _, world = dist_env()
    if rank != 0:
        return
    from oracle import oracle
    table = torch.empty(ROWS, DIM)
    fill_table(table)
    scores = make_scores()
    ranking = np.argsort(-scores, kind="stable")
    batches = make_batches(ranking, N_BATCHES, seed=100)
    for i in range(args.warmup):
        oracle.cpu_fetch_reference(table, batches[i % N_BATCHES])
    t0 = time.perf_counter()
    for i in range(args.steps):
        out = oracle.cpu_fetch_reference(table, batches[i % N_BATCHES])
    dt = time.perf_counter() - t0
    value = args.steps * BATCH * ROW_BYTES / dt / 1e9
    cores = torch.get_num_threads()
    line = {
        "impl": "reference", "metric": METRIC, "value": round(value, 3), "unit": UNIT,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(dt / args.steps * 1e3, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32 rows, int64 ids (byte copy)", "data": "synthetic (seeded)",
        "config": {"workload": WORKLOAD, "rows": ROWS, "dim": DIM, "batch": BATCH},
        "cpu_baseline": {"value": round(value, 3), "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"{args.steps} full batches of 500,000 ids; torch.index_select on the host "
                                   "table = the reference's cpu_fetch (example/test_cache_fetch.py:138), "
                                   f"{cores} threads of {os.cpu_count()} logical cores"},
        "e2e": {"value": round(value, 3), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    assert out.shape == (BATCH, DIM)
    emit(line)


# --------------------------------------------------------------------------- our arm
def run_ours(args) -> None:
    rank, local_rank, world = dist_env()
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    assert torch.cuda.is_available(), "bench.py needs a GPU (there is no CPU path)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    import torch.distributed as dist
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")  # stdout carries the one JSON line only
        dist.init_process_group("nccl", device_id=dev)

    import shmtensor_b200 as st
    from shmtensor_b200 import capi
    from shmtensor_b200.partition import PartitionedFeatureCache

    stream = torch.cuda.current_stream()

    # ---- data: host table shared by the ranks of the node, pinned; cache; batches
    if world > 1:
        name = f"shmt_bench_{os.environ.get('MASTER_PORT', '0')}"
        if rank == 0 and capi.file_exist(name):  # stale segment of a killed run
            p, fd = capi.open_shared_mem(name, ROWS * ROW_BYTES)
            capi.release_shared_mem(name, ROWS * ROW_BYTES, p, fd)
        dist.barrier()
        shm = st.ShmTensor(name, (ROWS, DIM), rank, world, None, torch.float32, pin_memory=True)
        table = shm.tensor_
        if rank == 0:
            fill_table(table)
        dist.barrier()
    else:
        shm = None
        table = torch.empty(ROWS, DIM)
        fill_table(table)
        capi.pin_memory(table)

    scores = make_scores()
    ranking = np.argsort(-scores, kind="stable")
    n_cached = int(ROWS * CACHE_FRACTION)
    cached_ids = torch.from_numpy(ranking[:n_cached].copy())
    batches_host = [b.pin_memory() for b in make_batches(ranking, N_BATCHES, seed=100 + rank)]
    batches = [b.to(dev) for b in batches_host]

    if world == 1:
        gpu_rows = capi.uva_fetch(table, cached_ids.to(dev))
        hmap = capi.CUCOStaticHashmap(cached_ids.to(dev), torch.arange(n_cached, dtype=torch.int32, device=dev),
                                      LOAD_FACTOR)
        fetch = lambda ids: capi.cache_fetch(table, gpu_rows, ids, hmap)
        query = hmap.query
        pcache = None
    else:
        pcache = PartitionedFeatureCache(table, cached_ids, load_factor=LOAD_FACTOR)
        fetch = pcache.fetch
        query = pcache.directory.query
    hit_counts = [int((query(b) >= 0).sum().item()) for b in batches]
    hit_rate = sum(hit_counts) / (N_BATCHES * BATCH)

    # ---- set-up, not timed: one streaming pass over the whole host table from this GPU, so that
    #      every page of it has been translated once (GPU TLB / IOMMU) before any step is timed
    from shmtensor_b200._lib import check as _check, lib as _lib_
    _sink = torch.zeros(1, dtype=torch.int64, device=dev)
    _check(_lib_.shmt_stream_read(table.data_ptr(), ROWS * ROW_BYTES, _sink.data_ptr(), stream.cuda_stream))
    torch.cuda.synchronize()

    # ---- parity on one batch before timing anything (bit-exact vs the host table)
    got = fetch(batches[0])
    want = torch.index_select(table, 0, batches_host[0])
    assert torch.equal(got.cpu().view(torch.int32), want.view(torch.int32)), "fetch is not bit-exact"
    del got, want

    # ---- warm-up, then the timed region: K launches, one CUDA-event pair each
    out = None
    for i in range(max(args.warmup, 3)):
        out = fetch(batches[i % N_BATCHES])  # held like in the timed loop: two output blocks get cached
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    region = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
    sampler = ClockSampler(local_rank, period_s=0.1)
    sampler.start()  # its first NVML queries are slow and can stall a launch: let them pass now
    for i in range(3):
        out = fetch(batches[i % N_BATCHES])
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    region[0].record(stream)
    for i, (a, b) in enumerate(evs):
        a.record(stream)
        out = fetch(batches[i % N_BATCHES])
        b.record(stream)
    region[1].record(stream)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    clocks = sampler.stop()
    region_ms = region[0].elapsed_time(region[1])
    kernel_ms = sum(a.elapsed_time(b) for a, b in evs) / args.steps
    per_launch = [a.elapsed_time(b) for a, b in evs]
    print(f"[rank {rank}] timed region {region_ms:.3f} ms, launches min/median/max "
          f"{min(per_launch):.3f}/{statistics.median(per_launch):.3f}/{max(per_launch):.3f} ms, "
          f"first five {[round(x, 3) for x in per_launch[:5]]}", file=sys.stderr, flush=True)
    if world > 1:
        t = torch.tensor([region_ms, kernel_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        region_ms, kernel_ms = t.tolist()
    ms_per_step = region_ms / args.steps
    value = world * BATCH * ROW_BYTES / (ms_per_step * 1e6)

    # ---- end to end through the public call: ids from pinned host memory each step, the last
    #      fetched row read back to pinned host memory
    ids_dev = torch.empty(BATCH, dtype=torch.int64, device=dev)
    tail = torch.empty(DIM, dtype=torch.float32).pin_memory()
    e2e_steps = args.steps
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    region[0].record(stream)
    for i in range(e2e_steps):
        ids_dev.copy_(batches_host[i % N_BATCHES], non_blocking=True)
        out = fetch(ids_dev)
        tail.copy_(out[-1], non_blocking=True)
        stream.synchronize()
    region[1].record(stream)
    torch.cuda.synchronize()
    e2e_ms = region[0].elapsed_time(region[1]) / e2e_steps
    e2e_wall_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = t.item()
    e2e_value = world * BATCH * ROW_BYTES / (e2e_ms * 1e6)

    line = {
        "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": round(ms_per_step, 5), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32 rows, int64 ids (byte copy)",
        "data": "synthetic (seeded)",
        "config": {"workload": WORKLOAD, "rows": ROWS, "dim": DIM, "batch": BATCH, "cached_rows": n_cached,
                   "hit_rate": round(hit_rate, 4),
                   "l2": "inputs larger than L2: 192 MB cached rows + 200 MB output per launch, "
                         f"{N_BATCHES} distinct query batches rotated",
                   "partition": "single GPU" if world == 1 else
                   f"hash-partitioned over {world} GPUs, NVLink P2P loads; the {pcache.replicated} hottest rows on every GPU"},
        "e2e": {"value": round(e2e_value, 2), "unit": UNIT, "h2d_bytes_per_step": BATCH * 8,
                "d2h_bytes_per_step": DIM * 4, "ms_per_step": round(e2e_ms, 5),
                "wall_ms_per_step": round(e2e_wall_ms, 5)},
        "gpu_launches": args.steps,
        "clocks": clocks,
    }

    # ---- N > 1: the NVLink regime -- ids all cached, (N-1)/N of the rows on a peer GPU
    if world > 1:
        from shmtensor_b200._lib import check, lib
        from shmtensor_b200.partition import _DeviceBuffer, share_device_buffer
        probe = _DeviceBuffer(256 << 20)
        ptrs, opened = share_device_buffer(probe)
        sink = torch.zeros(1, dtype=torch.int64, device=dev)
        peer = ptrs[(rank + 1) % world]
        peer_ms = min(time_launches(lambda: check(lib.shmt_stream_read(peer, 256 << 20, sink.data_ptr(),
                                                                        stream.cuda_stream)), 1, stream)
                      for _ in range(5))
        gen = torch.Generator().manual_seed(1000 + rank)
        hot_batches = [cached_ids[torch.randint(0, n_cached, (BATCH,), generator=gen)].to(dev) for _ in range(4)]
        for b in hot_batches[:2]:
            fetch(b)
        dist.barrier()
        ms_hit = time_launches(lambda c=[0]: (fetch(hot_batches[c[0] % 4]), c.__setitem__(0, c[0] + 1)), 40, stream)
        t = torch.tensor([ms_hit, peer_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_hit, peer_ms = t.tolist()
        peer_gbs = (256 << 20) / (peer_ms * 1e6)
        # rows that really came from a peer (the hottest ids are replicated on every rank)
        n_remote = sum(int(((pcache.directory.query(b) >> 40) != rank).sum().item()) for b in hot_batches) / 4
        t = torch.tensor([n_remote], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        remote_bytes = t.item() * ROW_BYTES
        line["roofline_all_hit_partitioned"] = {
            "bound": "nvlink", "kernel_ms": round(ms_hit, 5),
            "aggregate_gbs": round(world * BATCH * ROW_BYTES / (ms_hit * 1e6), 1),
            "achieved": round(remote_bytes / (ms_hit * 1e6), 1), "peak": round(peer_gbs, 1), "unit": "GB/s",
            "frac": round(remote_bytes / (ms_hit * 1e6) / peer_gbs, 4),
            "peak_source": "streaming read kernel over the next rank's IPC-mapped buffer, measured in this run",
            "what": "ids uniform over the cached set: about 1/N of the rows local, the rest read from peers over "
                    "NVLink; achieved = remote row bytes per rank (the least over ranks) / slowest rank's kernel time",
            "replicated_rows_per_gpu": pcache.replicated}
        # the batched alternative (NCCL all-to-all of ids, then of rows) on the same batches
        a2a = pcache.fetch_alltoall(batches[0])
        assert torch.equal(a2a.view(torch.int32), fetch(batches[0]).view(torch.int32)), "all-to-all route differs"
        def a2a_ms(bs, reps):
            for b in bs[:2]:
                pcache.fetch_alltoall(b)
            dist.barrier()
            t_ = time_launches(lambda c=[0]: (pcache.fetch_alltoall(bs[c[0] % len(bs)]), c.__setitem__(0, c[0] + 1)),
                               reps, stream)
            t_ = torch.tensor([t_], device=dev)
            dist.all_reduce(t_, op=dist.ReduceOp.MAX)
            return t_.item()
        line["alltoall_route"] = {"mixed_ms": round(a2a_ms(batches, 10), 4), "all_hit_ms": round(a2a_ms(hot_batches, 10), 4),
                                  "p2p_mixed_ms": round(ms_per_step, 4), "p2p_all_hit_ms": round(ms_hit, 4),
                                  "what": "PartitionedFeatureCache.fetch_alltoall (ids bucketed by owner, NCCL all-to-all of "
                                          "ids and of rows, misses read locally) against the fused peer-load kernel"}
        # the other way to spend N GPUs: every GPU keeps the cache budget of the 1-GPU run (480,000 rows),
        # so the partitioned cache holds N times as many ids and fewer rows cross the host link
        n_grown = min(world * n_cached, ROWS)
        grown = PartitionedFeatureCache(table, torch.from_numpy(ranking[:n_grown].copy()), load_factor=LOAD_FACTOR)
        got = grown.fetch(batches[0])
        assert torch.equal(got.cpu().view(torch.int32),
                           torch.index_select(table, 0, batches_host[0]).view(torch.int32)), "grown cache differs"
        del got
        grown_hits = sum(int((grown.directory.query(b) >= 0).sum().item()) for b in batches) / (N_BATCHES * BATCH)
        for b in batches[:3]:
            grown.fetch(b)
        dist.barrier()
        ms_grown = time_launches(lambda c=[0]: (grown.fetch(batches[c[0] % N_BATCHES]), c.__setitem__(0, c[0] + 1)),
                                 40, stream)
        t = torch.tensor([ms_grown], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_grown = t.item()
        line["cache_budget_per_gpu"] = {
            "cached_rows_total": n_grown, "cached_rows_per_gpu": n_grown // world, "hit_rate": round(grown_hits, 4),
            "ms_per_step": round(ms_grown, 5), "value": round(world * BATCH * ROW_BYTES / (ms_grown * 1e6), 2),
            "unit": UNIT,
            "what": "same batches; every GPU contributes the 1-GPU cache budget, so the partitioned cache grows "
                    "with N (the headline keeps the total cached set fixed and splits it)"}
        grown.close()
        torch.cuda.synchronize()
        dist.barrier()
        for p_ in opened:
            lib.shmt_ipc_close_handle(p_)
        dist.barrier()
        lib.shmt_dev_free(probe.ptr)

    # ---- rank 0, one GPU: roofline of the fetch kernel and the CPU baseline beside it
    if rank == 0 and world == 1:
        peak, peak_src = measured_peaks()
        link = measure_host_link(table, stream)
        n_hit = sum(hit_counts[i % N_BATCHES] for i in range(args.steps)) / args.steps
        alg = hbm_bytes(BATCH, int(n_hit))
        link_bytes = (BATCH - n_hit) * ROW_BYTES
        t_roof_ms = max(alg / (peak * 1e6), link_bytes / (link["peak_gbs"] * 1e6))
        line["roofline"] = {
            "bound": "hbm", "kernel": "row_gather_bulk_kernel<2> (fused probe + TMA bulk gather)",
            "achieved": round(alg / (kernel_ms * 1e6), 1), "peak": peak, "unit": "GB/s",
            "frac": round(alg / (kernel_ms * 1e6) / peak, 4), "peak_source": peak_src,
            # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel on this
            # workload, from the ncu capture summarised in profiles/row_gather_bulk_mixed.md
            "traffic": NCU_DRAM_BYTES_PER_LAUNCH, "algorithmic_bytes": int(alg),
            "traffic_source": "profiles/row_gather_bulk_mixed.md (ncu --set full, 2 launches; bytes per launch)",
            "kernel_ms": round(kernel_ms, 5),
            "note": "the 80%-hit batch is bound by the host link, not HBM: see roofline_link and "
                    "frac_of_bound (time at the binding ceiling / measured time)",
            "frac_of_bound": round(t_roof_ms / kernel_ms, 4),
        }
        line["roofline_link"] = {
            "bound": "host_link", "achieved": round(link_bytes / (kernel_ms * 1e6), 2), "peak": link["peak_gbs"],
            "unit": "GB/s", "frac": round(link_bytes / (kernel_ms * 1e6) / link["peak_gbs"], 4),
            "peak_source": "measured in this run", **link}
        # same kernel, all ids cached (HBM-bound regime) and no cache at all (link-bound regime)
        hot_batches = [cached_ids[torch.randint(0, n_cached, (BATCH,), generator=torch.Generator().manual_seed(s))].to(dev)
                       for s in range(4)]
        ms_hit = time_launches(lambda c=[0]: (fetch(hot_batches[c[0] % 4]), c.__setitem__(0, c[0] + 1)), 40, stream)
        alg_hit = hbm_bytes(BATCH, BATCH)
        line["roofline_all_hit"] = {"bound": "hbm", "achieved": round(alg_hit / (ms_hit * 1e6), 1), "peak": peak,
                                    "unit": "GB/s", "frac": round(alg_hit / (ms_hit * 1e6) / peak, 4),
                                    "frac_of_nominal_8TBs": round(alg_hit / (ms_hit * 1e6) / 8000, 4),
                                    "kernel_ms": round(ms_hit, 5), "peak_source": peak_src}
        # link-bound regime: ids drawn from the rows that are NOT cached, i.e. the population the
        # misses of the real batches come from (replaying the Zipf-hot ids against the host table
        # would hammer a few host cache lines thousands of times, which no cached run does)
        cold_ids = torch.from_numpy(ranking[n_cached:].copy())
        cold_batches = [cold_ids[torch.randint(0, cold_ids.numel(), (BATCH,), generator=torch.Generator().manual_seed(s))].to(dev)
                        for s in range(4)]
        for b in cold_batches[:2]:
            fetch(b)
        ms_miss = time_launches(lambda c=[0]: (fetch(cold_batches[c[0] % 4]), c.__setitem__(0, c[0] + 1)), 10, stream)
        line["roofline_all_miss"] = {"bound": "host_link", "achieved": round(BATCH * ROW_BYTES / (ms_miss * 1e6), 2),
                                     "peak": link["peak_gbs"], "unit": "GB/s",
                                     "frac": round(BATCH * ROW_BYTES / (ms_miss * 1e6) / link["peak_gbs"], 4),
                                     "kernel_ms": round(ms_miss, 5),
                                     "ids": "uniform over the 1,920,000 uncached rows, probed and missed"}
        # the reference's own fetch kernel on the same GPU and batches, when oracle/_ref was built
        try:
            from oracle import build_ref
            ref = build_ref.load_reference()
        except Exception as exc:  # noqa: BLE001
            ref = None
            line["reference_cuda"] = {"unavailable": f"reference build not loadable: {exc}"}
        if ref is not None:
            rmap = ref.CUCOStaticHashmap(cached_ids.to(dev), torch.arange(n_cached, dtype=torch.int32, device=dev),
                                         LOAD_FACTOR)
            def ref_ms(bs, n):
                for b in bs[:2]:
                    ref.cache_fetch(table, gpu_rows, b, rmap)
                return time_launches(lambda c=[0]: (ref.cache_fetch(table, gpu_rows, bs[c[0] % len(bs)], rmap),
                                                    c.__setitem__(0, c[0] + 1)), n, stream)
            r_mixed, r_hit, r_miss = ref_ms(batches, 20), ref_ms(hot_batches, 20), ref_ms(cold_batches, 5)
            line["reference_cuda"] = {
                "what": "the reference's MultiDimCacheFetchKernel (src/cache_feature_fetch.cu:106-129), compiled "
                        "unmodified, over a stand-in for its cuCollections map; same table, cache and batches",
                "mixed_ms": round(r_mixed, 5), "mixed_gbs": round(BATCH * ROW_BYTES / (r_mixed * 1e6), 2),
                "all_hit_ms": round(r_hit, 5), "all_hit_gbs": round(alg_hit / (r_hit * 1e6), 1),
                "all_miss_ms": round(r_miss, 5), "all_miss_gbs": round(BATCH * ROW_BYTES / (r_miss * 1e6), 2)}
            del rmap
        # CPU baseline: the reference's cpu_fetch line on this box's cores, bounded sample
        from oracle import oracle
        n_cpu = 20
        for i in range(3):
            oracle.cpu_fetch_reference(table, batches_host[i])
        t0 = time.perf_counter()
        for i in range(n_cpu):
            oracle.cpu_fetch_reference(table, batches_host[i % N_BATCHES])
        cpu_s = (time.perf_counter() - t0) / n_cpu
        cores = torch.get_num_threads()
        line["cpu_baseline"] = {
            "value": round(BATCH * ROW_BYTES / cpu_s / 1e9, 3), "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"{n_cpu} full batches of 500,000 ids after 3 warm-ups; torch.index_select on the pinned host "
                      f"table (the reference's cpu_fetch, example/test_cache_fetch.py:138); {cores} threads of "
                      f"{os.cpu_count()} logical cores"}

    if rank == 0:
        emit(line)

    # ---- orderly teardown: nothing in flight, peers unmapped before any shard is freed
    torch.cuda.synchronize()
    if pcache is not None:
        pcache.close()
    if world == 1:
        capi.unpin_memory(table)
    else:
        dist.barrier()
        del table, pcache
        shm = None
        dist.barrier()
        dist.destroy_process_group()


# --------------------------------------------------------------------------- sampling workload
G_NODES, G_EDGES, G_CAP, G_ALPHA = 2_400_000, 62_000_000, 10_000, 2.1
FANOUT = [15, 10, 5]
N_SEEDS = 1024
SAMPLING_WORKLOAD = ("1-GPU cached neighbour sampling + relabel: power-law CSR 2,400,000 nodes / 62,000,000 edges "
                     "(degree Zipf(2.1) capped at 10,000), int64 indptr, int32 indices, top 20% nodes by degree "
                     "cached in HBM, rest pinned host; 1,024 seeds, 3 hops fan-out [15,10,5], unique+relabel per hop")


def make_graph(seed: int = 3):
    """Seeded power-law CSR: capped Zipf degrees rescaled to the edge total; the neighbours of a
    row are an arithmetic progression modulo the node count (distinct within the row, spread
    uniformly over the nodes)."""
    rng = np.random.default_rng(seed)
    raw = np.minimum(rng.zipf(G_ALPHA, size=G_NODES), G_CAP).astype(np.float64)
    lo, hi = 0.1, 50.0
    for _ in range(60):  # bisection on the scale factor
        mid = 0.5 * (lo + hi)
        if np.minimum(np.floor(raw * mid), G_CAP).sum() > G_EDGES:
            hi = mid
        else:
            lo = mid
    deg = np.minimum(np.floor(raw * lo), G_CAP).astype(np.int64)
    short = G_EDGES - int(deg.sum())
    bump = rng.permutation(np.flatnonzero(deg < G_CAP))[:short]
    deg[bump] += 1
    indptr = np.zeros(G_NODES + 1, dtype=np.int64)
    np.cumsum(deg, out=indptr[1:])
    steps = np.array([7, 11, 13, 17, 19, 23, 29, 31, 37, 41, 43, 47, 53, 59, 61, 67], dtype=np.int64)  # coprime to 2.4M
    base = rng.integers(0, G_NODES, size=G_NODES)
    step = steps[rng.integers(0, steps.size, size=G_NODES)]
    row = np.repeat(np.arange(G_NODES, dtype=np.int64), deg)
    j = np.arange(indptr[-1], dtype=np.int64) - indptr[row]
    indices = ((base[row] + j * step[row]) % G_NODES).astype(np.int32)
    return indptr, indices, deg


def minibatch(capi, indptr, indices, gp, gi, hmap, seeds):
    """The reference's per-batch loop (python/shmtensor/sampling.py:124-143): hops over
    reversed(fan-out), relabel [seeds, neighbours], next frontier = unique."""
    edges = 0
    for k in reversed(FANOUT):
        if hmap is None:
            sub_indptr, sub_indices = capi.csr_sampling(indptr, indices, seeds, k, False)
        else:
            sub_indptr, sub_indices = capi.csr_cache_sampling(indptr, indices, gp, gi, hmap, seeds, k, False)
        seeds, _ = capi.tensor_relabel([seeds, sub_indices])
        edges += sub_indices.numel()
    return edges, seeds


def minibatch_fused(capi, indptr, indices, gp, gi, hmap, seeds):
    """The same mini-batch through the fused native call (what GPUSamplingDataloader uses)."""
    frontier, hops = capi.sample_minibatch(indptr, indices, seeds, list(reversed(FANOUT)), False, gp, gi, hmap)
    return sum(h[1].numel() for h in hops), frontier


def run_sampling(args) -> None:
    rank, local_rank, world = dist_env()
    if rank != 0:
        return
    indptr_n, indices_n, deg = make_graph()
    rng = np.random.default_rng(11)
    seed_batches = [rng.integers(0, G_NODES, size=N_SEEDS).astype(np.int32) for _ in range(32)]
    cores = torch.get_num_threads()
    line = {"metric": "sampled edges/s", "unit": "edges/s", "n_gpus": 1, "steps": args.steps,
            "warmup": max(args.warmup, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int64 indptr, int32 indices (integer / byte work)", "data": "synthetic (seeded)",
            "config": {"workload": SAMPLING_WORKLOAD, "nodes": G_NODES, "edges": int(indptr_n[-1]),
                       "fanout": FANOUT, "seeds": N_SEEDS, "hop_order": "reversed(fan-out), as the reference"}}

    if args.impl == "reference":
        # the reference has no CPU sampler (it compares against DGL): time the threaded CPU
        # restatement of its CUDA algorithm
        from oracle import build_oracle
        lib = build_oracle.load_cpu()
        def cpu_batch(seeds32):
            seeds = seeds32.astype(np.int64)
            edges = 0
            for k in reversed(FANOUT):
                sp = np.empty(seeds.size + 1, np.int64)
                so = np.empty(seeds.size * k, np.int32)
                nnz = lib.oracle_sample_hop(indptr_n.ctypes.data, indices_n.ctypes.data, 0, seeds.ctypes.data,
                                            seeds.size, k, 0, 7777, sp.ctypes.data, so.ctypes.data)
                cat = np.concatenate([seeds, so[:nnz].astype(np.int64)])
                uniq, rel = np.empty(cat.size, np.int64), np.empty(cat.size, np.int64)
                nu = lib.oracle_relabel(cat.ctypes.data, cat.size, uniq.ctypes.data, rel.ctypes.data)
                seeds = uniq[:nu].copy()
                edges += int(nnz)
            return edges
        for i in range(max(args.warmup, 1)):
            cpu_batch(seed_batches[i % 32])
        t0 = time.perf_counter()
        edges = sum(cpu_batch(seed_batches[i % 32]) for i in range(args.steps))
        dt = time.perf_counter() - t0
        v = edges / dt
        line.update({"impl": "reference", "value": round(v, 1), "ms_per_step": round(dt / args.steps * 1e3, 4),
                     "cpu_baseline": {"value": round(v, 1), "unit": "edges/s", "cores": lib.oracle_num_threads(),
                                      "kind": "port", "sample": f"{args.steps} full 3-hop mini-batches; threaded C++ "
                                      "restatement of the reference's sampler (seeds split over threads) + serial relabel"},
                     "e2e": {"value": round(v, 1), "unit": "edges/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
        emit(line)
        return

    assert torch.cuda.is_available(), "bench.py needs a GPU (there is no CPU path)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    from shmtensor_b200 import capi
    indptr, indices = torch.from_numpy(indptr_n), torch.from_numpy(indices_n)
    capi.pin_memory(indptr)
    capi.pin_memory(indices)
    n_cached = G_NODES // 5
    hot = torch.from_numpy(np.argsort(-deg, kind="stable")[:n_cached].copy()).to(dev)
    gp, gi = capi.create_subcsr(indptr, indices, hot)
    hmap = capi.CUCOStaticHashmap(hot.int(), torch.arange(n_cached, dtype=torch.int32, device=dev), 0.8)
    seeds_host = [torch.from_numpy(b).pin_memory() for b in seed_batches]
    seeds_dev = [b.to(dev) for b in seeds_host]
    stream = torch.cuda.current_stream()
    capi.set_sampling_seed(7777)
    for i in range(max(args.warmup, 3)):  # results held as in the timed loop, so its blocks get cached
        e, frontier = minibatch_fused(capi, indptr, indices, gp, gi, hmap, seeds_dev[i % 32])
    sampler = ClockSampler(local_rank, period_s=0.1)
    region = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
    torch.cuda.synchronize()
    sampler.start()
    region[0].record(stream)
    edges = 0
    for i in range(args.steps):
        e, frontier = minibatch_fused(capi, indptr, indices, gp, gi, hmap, seeds_dev[i % 32])
        edges += e
    region[1].record(stream)
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = region[0].elapsed_time(region[1]) / args.steps
    value = edges / args.steps / (ms * 1e-3)
    # end to end: seeds start in pinned host memory, the frontier size is read back
    seeds_buf = torch.empty(N_SEEDS, dtype=torch.int32, device=dev)
    torch.cuda.synchronize()
    region[0].record(stream)
    e2e_edges = 0
    for i in range(args.steps):
        seeds_buf.copy_(seeds_host[i % 32], non_blocking=True)
        e, frontier = minibatch_fused(capi, indptr, indices, gp, gi, hmap, seeds_buf)
        e2e_edges += e
        _ = frontier[-1].item()
    region[1].record(stream)
    torch.cuda.synchronize()
    e2e_ms = region[0].elapsed_time(region[1]) / args.steps
    # uncached (every row over UVA) and fully GPU-resident graph, for the cache's effect
    extra = {}
    variants = {"uva_only": (minibatch_fused, indptr, indices, None, None, None),
                "all_in_hbm": (minibatch_fused, indptr.to(dev), indices.to(dev), None, None, None),
                "call_per_hop_cached": (minibatch, indptr, indices, gp, gi, hmap),
                # not the configured workload: the whole indptr (19 MB) mirrored in HBM, so a cold
                # row costs one trip over the host link instead of two
                "cached_plus_indptr_in_hbm": (minibatch_fused, indptr.to(dev), indices, gp, gi, hmap)}
    for name, (fn, ip, ix, a, b, m) in variants.items():
        for i in range(3):
            fn(capi, ip, ix, a, b, m, seeds_dev[i])
        torch.cuda.synchronize()
        region[0].record(stream)
        ee = sum(fn(capi, ip, ix, a, b, m, seeds_dev[i % 32])[0] for i in range(50))
        region[1].record(stream)
        torch.cuda.synchronize()
        extra[name] = round(ee / (region[0].elapsed_time(region[1]) * 1e-3), 1)
    # same-box numbers of the reference's own CUDA kernels, when oracle/_ref was built
    ref_line = None
    try:
        from oracle import build_ref
        ref = build_ref.load_reference()
    except Exception as exc:  # noqa: BLE001
        ref, ref_line = None, {"unavailable": f"reference build not loadable: {exc}"}
    if ref is not None:
        indices64 = torch.from_numpy(indices_n.astype(np.int64))
        ref.pin_memory(indices64)
        rgp, rgi = ref.create_subcsr(indptr, indices64, hot)
        rmap = ref.CUCOStaticHashmap(hot.int(), torch.arange(n_cached, dtype=torch.int32, device=dev), 0.8)
        def ref_batch(seeds):
            ed = 0
            for k in reversed(FANOUT):
                sp, so = ref.csr_cache_sampling(indptr, indices64, rgp, rgi, rmap, seeds, k, False)
                seeds, _ = ref.tensor_relabel([seeds.long(), so])
                ed += so.numel()
            return ed
        for i in range(3):
            ref_batch(seeds_dev[i])
        torch.cuda.synchronize()
        region[0].record(stream)
        ee = sum(ref_batch(seeds_dev[i % 32]) for i in range(50))
        region[1].record(stream)
        torch.cuda.synchronize()
        ref_ms = region[0].elapsed_time(region[1]) / 50
        ref_line = {"edges_per_s": round(ee / 50 / (ref_ms * 1e-3), 1), "ms_per_step": round(ref_ms, 4),
                    "what": "the reference's own sampling + relabel kernels (compiled unmodified, int64 indices as it "
                            "requires equal dtypes) over a stand-in for its cuCollections map"}
        ref.unpin_memory(indices64)
    # CPU baseline beside it (bounded sample)
    from oracle import build_oracle
    lib = build_oracle.load_cpu()
    def cpu_batch(seeds32):
        seeds = seeds32.astype(np.int64)
        ed = 0
        for k in reversed(FANOUT):
            sp = np.empty(seeds.size + 1, np.int64)
            so = np.empty(seeds.size * k, np.int32)
            nnz = lib.oracle_sample_hop(indptr_n.ctypes.data, indices_n.ctypes.data, 0, seeds.ctypes.data,
                                        seeds.size, k, 0, 7777, sp.ctypes.data, so.ctypes.data)
            cat = np.concatenate([seeds, so[:nnz].astype(np.int64)])
            uniq, rel = np.empty(cat.size, np.int64), np.empty(cat.size, np.int64)
            nu = lib.oracle_relabel(cat.ctypes.data, cat.size, uniq.ctypes.data, rel.ctypes.data)
            seeds = uniq[:nu].copy()
            ed += int(nnz)
        return ed
    cpu_batch(seed_batches[0])
    t0 = time.perf_counter()
    ce = sum(cpu_batch(seed_batches[i]) for i in range(10))
    cpu_dt = time.perf_counter() - t0
    line.update({"value": round(value, 1), "ms_per_step": round(ms, 5), "edges_per_step": edges // args.steps,
                 "e2e": {"value": round(e2e_edges / args.steps / (e2e_ms * 1e-3), 1), "unit": "edges/s",
                         "h2d_bytes_per_step": N_SEEDS * 4, "d2h_bytes_per_step": 6 * 8 + 4, "ms_per_step": round(e2e_ms, 5)},
                 "gpu_launches": args.steps * 3 * 4, "api": "capi.sample_minibatch (all hops in one native call)", "clocks": clocks, "variants_edges_per_s": extra,
                 "reference_cuda": ref_line,
                 "cpu_baseline": {"value": round(ce / cpu_dt, 1), "unit": "edges/s", "cores": lib.oracle_num_threads(),
                                  "kind": "port", "sample": "10 full 3-hop mini-batches; threaded C++ restatement of the "
                                  "reference's sampler + serial relabel (the reference has no CPU sampler)"}})
    emit(line)
    capi.unpin_memory(indptr)
    capi.unpin_memory(indices)


# --------------------------------------------------------------------------- end-to-end mini-batch
MB_DIM = 128
MB_CACHE_FRACTION = 0.40
MINIBATCH_WORKLOAD = ("end-to-end mini-batch over a partitioned cache, config 4 scaled 1:46 to fit a short run: power-law "
                      "CSR 2,400,000 nodes / 62,000,000 edges, 128-d float32 features (1.2 GB) in pinned host memory; "
                      "the top 40% of nodes by degree have their adjacency cached on every GPU and their features "
                      "hash-partitioned over the GPUs; per GPU and step 1,024 seeds, fan-out [15,10,5], then the features "
                      "of every sampled node are fetched (remote hits over NVLink, misses over UVA)")


def run_minibatch(args) -> None:
    rank, local_rank, world = dist_env()
    indptr_n, indices_n, deg = make_graph()
    rng = np.random.default_rng(100 + rank)
    seed_batches = [rng.integers(0, G_NODES, size=N_SEEDS).astype(np.int32) for _ in range(32)]
    line = {"metric": "mini-batches/s (sampled edges/s, fetched feature GB/s)", "unit": "mini-batches/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "int32 ids, f32 rows (integer / byte work)",
            "data": "synthetic (seeded)",
            "config": {"workload": MINIBATCH_WORKLOAD, "nodes": G_NODES, "edges": int(indptr_n[-1]), "dim": MB_DIM,
                       "fanout": FANOUT, "seeds_per_gpu": N_SEEDS}}

    if args.impl == "reference":
        if rank != 0:
            return
        from oracle import build_oracle, oracle
        lib = build_oracle.load_cpu()
        feats = torch.empty(G_NODES, MB_DIM)
        fill_table(feats)
        def cpu_step(seeds32):
            seeds = seeds32.astype(np.int64)
            edges = 0
            for k in reversed(FANOUT):
                sp = np.empty(seeds.size + 1, np.int64)
                so = np.empty(seeds.size * k, np.int32)
                nnz = lib.oracle_sample_hop(indptr_n.ctypes.data, indices_n.ctypes.data, 0, seeds.ctypes.data,
                                            seeds.size, k, 0, 7777, sp.ctypes.data, so.ctypes.data)
                cat = np.concatenate([seeds, so[:nnz].astype(np.int64)])
                uniq, rel = np.empty(cat.size, np.int64), np.empty(cat.size, np.int64)
                nu = lib.oracle_relabel(cat.ctypes.data, cat.size, uniq.ctypes.data, rel.ctypes.data)
                seeds = uniq[:nu].copy()
                edges += int(nnz)
            out = oracle.cpu_fetch_reference(feats, torch.from_numpy(seeds))
            return edges, out.shape[0]
        for i in range(max(args.warmup, 1)):
            cpu_step(seed_batches[i % 32])
        t0 = time.perf_counter()
        tot = [cpu_step(seed_batches[i % 32]) for i in range(args.steps)]
        dt = (time.perf_counter() - t0) / args.steps
        line.update({"impl": "reference", "value": round(1 / dt, 2), "ms_per_step": round(dt * 1e3, 3),
                     "edges_per_s": round(sum(t[0] for t in tot) / args.steps / dt, 1),
                     "fetched_gbs": round(sum(t[1] for t in tot) / args.steps * MB_DIM * 4 / dt / 1e9, 3),
                     "cpu_baseline": {"value": round(1 / dt, 2), "unit": "mini-batches/s",
                                      "cores": lib.oracle_num_threads(), "kind": "port",
                                      "sample": f"{args.steps} full mini-batches: threaded C++ sampler + serial relabel "
                                                "+ torch.index_select on the host feature table"},
                     "e2e": {"value": round(1 / dt, 2), "unit": "mini-batches/s", "h2d_bytes_per_step": 0,
                             "d2h_bytes_per_step": 0}})
        emit(line)
        return

    assert torch.cuda.is_available(), "bench.py needs a GPU (there is no CPU path)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    import torch.distributed as dist
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    import shmtensor_b200 as st
    from shmtensor_b200 import capi
    from shmtensor_b200.partition import PartitionedFeatureCache
    stream = torch.cuda.current_stream()
    if world > 1:
        name = f"shmt_bench_mb_{os.environ.get('MASTER_PORT', '0')}"
        if rank == 0 and capi.file_exist(name):
            p, fd = capi.open_shared_mem(name, G_NODES * MB_DIM * 4)
            capi.release_shared_mem(name, G_NODES * MB_DIM * 4, p, fd)
        dist.barrier()
        shm = st.ShmTensor(name, (G_NODES, MB_DIM), rank, world, None, torch.float32, pin_memory=True)
        feats = shm.tensor_
        if rank == 0:
            fill_table(feats)
        dist.barrier()
    else:
        shm = None
        feats = torch.empty(G_NODES, MB_DIM)
        fill_table(feats)
        capi.pin_memory(feats)
    indptr, indices = torch.from_numpy(indptr_n), torch.from_numpy(indices_n)
    capi.pin_memory(indptr)
    capi.pin_memory(indices)
    n_cached = int(G_NODES * MB_CACHE_FRACTION)
    hot_n = np.argsort(-deg, kind="stable")[:n_cached].copy()
    hot = torch.from_numpy(hot_n).to(dev)
    gp, gi = capi.create_subcsr(indptr, indices, hot)
    gmap = capi.CUCOStaticHashmap(hot.int(), torch.arange(n_cached, dtype=torch.int32, device=dev), 0.8)
    fcache = PartitionedFeatureCache(feats, torch.from_numpy(hot_n))
    seeds_host = [torch.from_numpy(b).pin_memory() for b in seed_batches]
    seeds_buf = torch.empty(N_SEEDS, dtype=torch.int32, device=dev)
    tail = torch.empty(MB_DIM, dtype=torch.float32).pin_memory()
    capi.set_sampling_seed(7777 + rank)

    def step(i):
        seeds_buf.copy_(seeds_host[i % 32], non_blocking=True)
        frontier, hops = capi.sample_minibatch(indptr, indices, seeds_buf, list(reversed(FANOUT)), False, gp, gi, gmap)
        rows = fcache.fetch(frontier)
        return sum(h[1].numel() for h in hops), frontier, rows

    # parity of one full step: the fetched rows are the host rows of the frontier, bit for bit
    _, frontier, rows = step(0)
    assert torch.equal(rows.cpu().view(torch.int32), feats[frontier.cpu().long()].view(torch.int32))
    for i in range(max(args.warmup, 3)):
        e, frontier, rows = step(i)
    sampler = ClockSampler(local_rank, period_s=0.1)
    region = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler.start()
    region[0].record(stream)
    edges = n_rows = 0
    for i in range(args.steps):
        e, frontier, rows = step(i)
        tail.copy_(rows[-1], non_blocking=True)
        edges += e
        n_rows += rows.shape[0]
    region[1].record(stream)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    clocks = sampler.stop()
    ms = region[0].elapsed_time(region[1]) / args.steps
    t = torch.tensor([ms, float(edges), float(n_rows)], device=dev, dtype=torch.float64)
    if world > 1:
        tmax = t.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        ms, edges, n_rows = tmax[0].item(), t[1].item(), t[2].item()
    else:
        edges, n_rows = float(edges), float(n_rows)
    hits = int((fcache.directory.query(frontier.long()) >= 0).sum().item())
    v = world / (ms * 1e-3)
    line.update({"value": round(v, 1), "ms_per_step": round(ms, 5),
                 "edges_per_s": round(edges / args.steps / (ms * 1e-3), 1),
                 "fetched_gbs": round(n_rows / args.steps * MB_DIM * 4 / (ms * 1e6), 2),
                 "rows_fetched_per_gpu_step": round(n_rows / args.steps / world), "feature_hit_rate": round(hits / frontier.numel(), 4),
                 "e2e": {"value": round(v, 1), "unit": "mini-batches/s", "h2d_bytes_per_step": N_SEEDS * 4,
                         "d2h_bytes_per_step": MB_DIM * 4 + 9 * 8, "ms_per_step": round(ms, 5),
                         "note": "the timed loop is already end to end: seeds from pinned host memory, sizes and the "
                                 "last fetched row read back"},
                 "gpu_launches": args.steps * 10, "clocks": clocks})
    if rank == 0:
        emit(line)
    torch.cuda.synchronize()
    fcache.close()
    capi.unpin_memory(indptr)
    capi.unpin_memory(indices)
    if world == 1:
        capi.unpin_memory(feats)
    else:
        dist.barrier()
        del feats, fcache
        shm = None
        dist.barrier()
        dist.destroy_process_group()


# --------------------------------------------------------------------------- update workload
U_KEYS, U_DIM, U_LOOKUPS = 4_000_000, 256, 1_000_000
UPDATE_WORKLOAD = ("cache update path: fused insert/overwrite of 4,000,000 unique int64 keys (uniform over 2^40) with "
                   "256-d bfloat16 rows into an empty 1-GPU cache at load factor 0.5, then 1,000,000 lookups, "
                   "half present, half absent")


def run_update(args) -> None:
    rank, local_rank, world = dist_env()
    if rank != 0:
        return
    row_bytes = U_DIM * 2
    line = {"metric": "inserted+looked-up keys/s", "unit": "keys/s", "n_gpus": 1, "steps": args.steps,
            "warmup": max(args.warmup, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int64 keys, int32 slots, bf16 rows (byte copy)", "data": "synthetic (seeded)",
            "config": {"workload": UPDATE_WORKLOAD, "keys": U_KEYS, "row_bytes": row_bytes, "lookups": U_LOOKUPS}}
    rng = np.random.default_rng(5)
    keys_n = np.unique(rng.integers(0, 1 << 40, size=U_KEYS + 100_000))
    keys_n = rng.permutation(keys_n)[:U_KEYS].astype(np.int64)
    req_n = np.concatenate([keys_n[rng.integers(0, U_KEYS, size=U_LOOKUPS // 2)],
                            rng.integers(1 << 40, 1 << 41, size=U_LOOKUPS // 2)]).astype(np.int64)
    rng.shuffle(req_n)

    if args.impl == "reference":
        # CPU path: row write data[ids] = upd (example/test_cache_set.py:183-184) + an open-addressing
        # map built and queried on all cores (the reference's map is GPU-only)
        from oracle import build_oracle
        lib = build_oracle.load_cpu()
        rows = np.zeros((U_KEYS, row_bytes), np.uint8)
        rows[:] = np.arange(row_bytes, dtype=np.uint8)
        table_rows = np.empty_like(rows)
        slots = np.arange(U_KEYS, dtype=np.int64)
        cap = 1 << 23
        table = np.empty(2 * cap, np.int64)
        out = np.empty(U_LOOKUPS, np.int32)
        def step():
            lib.oracle_map_build_query(keys_n.ctypes.data, U_KEYS, table.ctypes.data, cap, req_n.ctypes.data,
                                       U_LOOKUPS, out.ctypes.data)
            lib.oracle_scatter(table_rows.ctypes.data, slots.ctypes.data, U_KEYS, row_bytes, rows.ctypes.data)
        for _ in range(max(args.warmup, 1)):
            step()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            step()
        dt = (time.perf_counter() - t0) / args.steps
        v = (U_KEYS + U_LOOKUPS) / dt
        line.update({"impl": "reference", "value": round(v, 1), "ms_per_step": round(dt * 1e3, 3),
                     "cpu_baseline": {"value": round(v, 1), "unit": "keys/s", "cores": lib.oracle_num_threads(),
                                      "kind": "port", "sample": f"{args.steps} full passes: threaded open-addressing "
                                      "build + query and a threaded row scatter"},
                     "e2e": {"value": round(v, 1), "unit": "keys/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
        emit(line)
        return

    assert torch.cuda.is_available(), "bench.py needs a GPU (there is no CPU path)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    from shmtensor_b200 import capi
    keys = torch.from_numpy(keys_n).to(dev)
    req = torch.from_numpy(req_n).to(dev)
    g = torch.Generator(device=dev).manual_seed(5)
    rows = torch.randn(U_KEYS, U_DIM, generator=g, device=dev).to(torch.bfloat16)
    slots = torch.arange(U_KEYS, dtype=torch.int32, device=dev)
    gpu = torch.empty(U_KEYS, U_DIM, dtype=torch.bfloat16, device=dev)
    stream = torch.cuda.current_stream()
    peak, peak_src = measured_peaks()

    def one_pass():
        m = capi.CUCOStaticHashmap.empty(2 * U_KEYS, torch.int64, torch.int32, dev)
        capi.cache_insert_set(gpu, keys, slots, rows, m)
        return m, m.query(req)

    for _ in range(max(args.warmup, 3)):
        m, out = one_pass()
    assert torch.equal(gpu.view(torch.int16), rows.view(torch.int16)) and m.size() == U_KEYS
    assert int((out >= 0).sum().item()) == U_LOOKUPS // 2
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    t_ins = t_q = 0.0
    torch.cuda.synchronize()
    for _ in range(args.steps):
        m = capi.CUCOStaticHashmap.empty(2 * U_KEYS, torch.int64, torch.int32, dev)
        ev[0].record(stream)
        capi.cache_insert_set(gpu, keys, slots, rows, m)
        ev[1].record(stream)
        out = m.query(req)
        ev[2].record(stream)
        torch.cuda.synchronize()
        t_ins += ev[0].elapsed_time(ev[1])
        t_q += ev[1].elapsed_time(ev[2])
    t_ins /= args.steps
    t_q /= args.steps
    # the reference-named overwrite of the same rows through the finished map (all hits)
    for _ in range(2):
        capi.cache_set(None, gpu, keys, rows, m)
    t_set = time_launches(lambda: capi.cache_set(None, gpu, keys, rows, m), 10, stream)
    b_set = U_KEYS * (8 + 12 + 2 * row_bytes)
    line["cache_set"] = {"ms": round(t_set, 4), "keys_per_s": round(U_KEYS / (t_set * 1e-3), 1),
                         "roofline": {"bound": "hbm", "achieved": round(b_set / (t_set * 1e6), 1), "peak": peak,
                                      "unit": "GB/s", "frac": round(b_set / (t_set * 1e6) / peak, 4)}}
    # plain map construction + query (CUCOStaticHashmap(keys, values, 0.5), the reference's flow),
    # and the reference's own map on the same GPU when oracle/_ref was built
    def build_query(mod):
        t0 = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        t0[0].record(stream)
        mm = mod.CUCOStaticHashmap(keys, slots, 0.5)
        t0[1].record(stream)
        r = mm.query(req)
        t0[2].record(stream)
        torch.cuda.synchronize()
        return t0[0].elapsed_time(t0[1]), t0[1].elapsed_time(t0[2]), r
    build_query(capi)
    b_ms, q_ms, r_ours = build_query(capi)
    line["map_build_query"] = {"build_ms": round(b_ms, 4), "query_ms": round(q_ms, 4)}
    try:
        from oracle import build_ref
        ref = build_ref.load_reference()
    except Exception:  # noqa: BLE001
        ref = None
    if ref is not None:
        build_query(ref)
        rb_ms, rq_ms, r_ref = build_query(ref)
        assert torch.equal(r_ours, r_ref), "map query differs from the reference's"
        line["map_build_query"]["reference_cuda"] = {"build_ms": round(rb_ms, 4), "query_ms": round(rq_ms, 4),
                                                     "what": "the reference's wrapper over a stand-in for cuCollections"}
    # cache turnover on the finished map: evict 10 % of the ids, admit as many new ones into the freed
    # rows (erased slots are taken again, so the table never fills); then the same back again
    n_turn = U_KEYS // 10
    evict, admit = keys[:n_turn].contiguous(), keys[:n_turn] + (1 << 41)
    t_er = t_ad = 0.0
    for a, b in ((evict, admit), (admit, evict), (evict, admit), (admit, evict)):
        t0 = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        t0[0].record(stream)
        freed = m.erase(a)
        t0[1].record(stream)
        m.insert(b, freed)
        t0[2].record(stream)
        torch.cuda.synchronize()
        t_er, t_ad = t0[0].elapsed_time(t0[1]), t0[1].elapsed_time(t0[2])
        assert m.size() == U_KEYS and torch.equal(m.query(b), freed) and bool((m.query(a) == -1).all())
    assert torch.equal(m.query(keys), slots)
    line["cache_turnover"] = {"ids": n_turn, "erase_ms": round(t_er, 4), "admit_ms": round(t_ad, 4),
                              "what": "shmt_map_erase of 10 % of the keys, then shmt_map_insert of as many new ids "
                                      "with the freed row numbers (host-synchronous calls, device time)"}
    # algorithmic bytes: insert+set per key 8 (key) + 4 (slot) + 16 (claim) + row read + row written;
    # lookup per key 8 + 12 + 4
    b_ins = U_KEYS * (8 + 4 + 16 + 2 * row_bytes)
    b_q = U_LOOKUPS * (8 + 12 + 4)
    line.update({"value": round((U_KEYS + U_LOOKUPS) / ((t_ins + t_q) * 1e-3), 1), "ms_per_step": round(t_ins + t_q, 4),
                 "insert_set": {"ms": round(t_ins, 4), "keys_per_s": round(U_KEYS / (t_ins * 1e-3), 1),
                                "roofline": {"bound": "hbm", "achieved": round(b_ins / (t_ins * 1e6), 1), "peak": peak,
                                             "unit": "GB/s", "frac": round(b_ins / (t_ins * 1e6) / peak, 4),
                                             "peak_source": peak_src}},
                 "lookup": {"ms": round(t_q, 4), "keys_per_s": round(U_LOOKUPS / (t_q * 1e-3), 1),
                            "roofline": {"bound": "hbm", "achieved": round(b_q / (t_q * 1e6), 1), "peak": peak,
                                         "unit": "GB/s", "frac": round(b_q / (t_q * 1e6) / peak, 4)}},
                 "gpu_launches": args.steps * 2})
    emit(line)


# --------------------------------------------------------------------------- scan + relabel workload
SR_SCAN_N, SR_IDS, SR_DISTINCT = 1 << 27, 1 << 25, 1 << 22
SR_WORKLOAD = ("prefix sum and relabel at sizes beyond L2: in-place inclusive scan of 134,217,728 int32 (512 MB) and of "
               "67,108,864 int64; relabel of 33,554,432 int64 ids drawn from 4,194,304 distinct values")


def run_scan_relabel(args) -> None:
    """One step = one int32 scan + one relabel.  Rows 16-17 of the hot path: src/thrust_scan.cu:9-18,
    src/tensor_relabel.cu:68-209."""
    rank, local_rank, world = dist_env()
    if rank != 0:
        return
    steps = min(args.steps, 30)
    line = {"metric": "scanned + relabelled elements/s", "unit": "elements/s", "n_gpus": 1, "steps": steps,
            "warmup": 3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int32 / int64 (integer adds, id compares)", "data": "synthetic (seeded)",
            "config": {"workload": SR_WORKLOAD, "scan_elements": SR_SCAN_N, "relabel_ids": SR_IDS,
                       "l2": "inputs larger than L2: 512 MB per scan, 256 MB of ids per relabel"}}
    rng = np.random.default_rng(17)
    if args.impl == "reference":
        # CPU path on a bounded sample: numpy cumsum (one thread) and the threaded relabel restatement
        from oracle import build_oracle
        lib = build_oracle.load_cpu()
        n_scan, n_ids = SR_SCAN_N // 8, SR_IDS // 8
        a = rng.integers(0, 3, size=n_scan).astype(np.int32)
        ids = rng.integers(0, SR_DISTINCT // 8, size=n_ids).astype(np.int64)
        uniq, rel = np.empty_like(ids), np.empty_like(ids)
        t_scan = t_rel = 0.0
        for i in range(steps + 1):
            t0 = time.perf_counter()
            np.cumsum(a, dtype=np.int32)
            t1 = time.perf_counter()
            lib.oracle_relabel(ids.ctypes.data, n_ids, uniq.ctypes.data, rel.ctypes.data)
            t2 = time.perf_counter()
            if i:
                t_scan += t1 - t0
                t_rel += t2 - t1
        dt = (t_scan + t_rel) / steps
        v = (n_scan + n_ids) / dt
        line.update({"impl": "reference", "value": round(v, 1), "ms_per_step": round(dt * 1e3, 3),
                     "scan_elements_per_s": round(n_scan * steps / t_scan, 1),
                     "relabel_ids_per_s": round(n_ids * steps / t_rel, 1),
                     "cpu_baseline": {"value": round(v, 1), "unit": "elements/s", "cores": lib.oracle_num_threads(),
                                      "kind": "port", "sample": f"{steps} passes over 1/8 of the workload: numpy cumsum "
                                      "(one thread) + hash relabel restatement"},
                     "e2e": {"value": round(v, 1), "unit": "elements/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
        emit(line)
        return

    assert torch.cuda.is_available(), "bench.py needs a GPU (there is no CPU path)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    from shmtensor_b200 import capi
    stream = torch.cuda.current_stream()
    peak, peak_src = measured_peaks()
    g = torch.Generator(device=dev).manual_seed(17)
    src32 = torch.randint(0, 3, (SR_SCAN_N,), generator=g, device=dev, dtype=torch.int32)
    src64 = torch.randint(0, 1 << 20, (SR_SCAN_N // 2,), generator=g, device=dev, dtype=torch.int64)
    ids = torch.randint(0, SR_DISTINCT, (SR_IDS,), generator=g, device=dev, dtype=torch.int64) * 2_000_003
    work32, work64 = torch.empty_like(src32), torch.empty_like(src64)

    def scan_ms(mod_scan, src, work, reps):
        ts = []
        for _ in range(reps):
            work.copy_(src)
            ts.append(time_launches(lambda: mod_scan(work), 1, stream))
        return statistics.median(ts)

    # parity at full size before timing: against torch.cumsum, and relabel through its defining properties
    work32.copy_(src32)
    capi.thrust_scan(work32)
    assert torch.equal(work32, torch.cumsum(src32, 0, dtype=torch.int32)), "scan differs from cumsum"
    uniq, (rel,) = capi.tensor_relabel([ids])
    assert torch.equal(uniq[rel], ids) and uniq.numel() == torch.unique(ids).numel(), "relabel is not a bijection"
    first = torch.full((uniq.numel(),), SR_IDS, dtype=torch.int64, device=dev).scatter_reduce_(
        0, rel, torch.arange(SR_IDS, device=dev), "amin")
    assert bool((first[1:] > first[:-1]).all()), "unique ids are not in first-occurrence order"
    del first
    t32 = scan_ms(capi.thrust_scan, src32, work32, steps)
    t64 = scan_ms(capi.thrust_scan, src64, work64, steps)
    for _ in range(3):
        capi.tensor_relabel([ids])
    t_rel = statistics.median(time_launches(lambda: capi.tensor_relabel([ids]), 1, stream) for _ in range(steps))
    b32, b64 = SR_SCAN_N * 8, SR_SCAN_N // 2 * 16
    # relabel: ids read by insert and compact (8 each), slot written + read + new id written (8 each x 3),
    # unique ids written; the table (12 bytes per slot at load <= 0.5) is written, read and cleaned
    cap = 1
    while cap < 2 * SR_IDS:
        cap <<= 1
    b_rel = SR_IDS * (8 + 8 + 8 * 3) + uniq.numel() * 8
    line.update({
        "value": round((SR_SCAN_N + SR_IDS) / ((t32 + t_rel) * 1e-3), 1), "ms_per_step": round(t32 + t_rel, 4),
        "scan_int32": {"ms": round(t32, 4), "elements_per_s": round(SR_SCAN_N / (t32 * 1e-3), 1),
                       "roofline": {"bound": "hbm", "achieved": round(b32 / (t32 * 1e6), 1), "peak": peak, "unit": "GB/s",
                                    "frac": round(b32 / (t32 * 1e6) / peak, 4), "peak_source": peak_src}},
        "scan_int64": {"ms": round(t64, 4), "elements_per_s": round(SR_SCAN_N // 2 / (t64 * 1e-3), 1),
                       "roofline": {"bound": "hbm", "achieved": round(b64 / (t64 * 1e6), 1), "peak": peak, "unit": "GB/s",
                                    "frac": round(b64 / (t64 * 1e6) / peak, 4)}},
        "relabel": {"ms": round(t_rel, 4), "ids_per_s": round(SR_IDS / (t_rel * 1e-3), 1), "unique": uniq.numel(),
                    "table_slots": cap,
                    "roofline": {"bound": "hbm", "achieved": round(b_rel / (t_rel * 1e6), 1), "peak": peak, "unit": "GB/s",
                                 "frac": round(b_rel / (t_rel * 1e6) / peak, 4),
                                 "note": "streamed bytes only; the random 12-byte table accesses (one sector each) "
                                         "are what bounds it"}},
        "roofline": {"bound": "hbm", "kernel": "scan_kernel (decoupled look-back, one pass)",
                     "achieved": round(b32 / (t32 * 1e6), 1), "peak": peak, "unit": "GB/s",
                     "frac": round(b32 / (t32 * 1e6) / peak, 4), "peak_source": peak_src, "traffic": None},
        "e2e": {"value": round((SR_SCAN_N + SR_IDS) / ((t32 + t_rel) * 1e-3), 1), "unit": "elements/s",
                "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 8,
                "note": "device-resident operands, as in their callers; relabel reads its unique count back"},
        "gpu_launches": steps * 4})
    # the reference's own kernels on the same GPU (thrust inclusive scan, its three-pass relabel)
    try:
        from oracle import build_ref
        ref = build_ref.load_reference()
    except Exception:  # noqa: BLE001
        ref = None
    if ref is not None:
        # its thrust_scan is a parallel for_each over ptr[i] += ptr[i-1] (src/thrust_scan.cu:9-18): one pass
        # over the data whose result depends on thread timing, so it is timed here but not compared
        r32 = scan_ms(ref.thrust_scan, src32, work32, steps)
        ru, rr = ref.tensor_relabel([ids])
        assert torch.equal(ru, uniq) and torch.equal(rr[0], rel), "relabel differs from the reference's"
        r_rel = statistics.median(time_launches(lambda: ref.tensor_relabel([ids]), 1, stream) for _ in range(steps))
        line["reference_cuda"] = {"scan_int32_ms": round(r32, 4), "relabel_ms": round(r_rel, 4),
                                  "what": "the reference's thrust_scan (a racy one-pass for_each, not a prefix sum) "
                                          "and tensor_relabel, compiled unmodified"}
    emit(line)



def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="fetch", choices=["fetch", "sampling", "update", "minibatch", "scan_relabel"],
                    help="fetch: the headline cached feature fetch; sampling: cached 3-hop sampling + relabel")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    args = ap.parse_args()
    quiet_stdout()
    if args.workload == "sampling":
        run_sampling(args)
    elif args.workload == "update":
        run_update(args)
    elif args.workload == "minibatch":
        run_minibatch(args)
    elif args.workload == "scan_relabel":
        run_scan_relabel(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
