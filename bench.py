#!/usr/bin/env python
"""Benchmark of the GPU-cache hot path: fetched feature GB/s and sampled edges/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload ...]

Headline workload (one step = one batch through the fused probe+gather kernel): a pinned host table
of 2,400,000 x 100 float32 rows, N(0,1); the top 20 % of rows by a seeded power-law score are
cached in HBM behind a static hashmap (int64 keys -> int32 slots, load factor 0.5); each
batch is 500,000 int64 ids, rank-Zipf(1.1) over the score ranking mixed with uniform rows so
that about 80 % hit the cache; misses are read from the host table through UVA.  With N > 1
ranks (torchrun), the cached rows are hash-partitioned over the GPUs and remote hits are read
over NVLink by the same kernel; every rank runs its own batches (weak scaling).

Prints one JSON line (rank 0).  ``value`` times the kernel with ids already on the GPU;
``e2e`` times the public call with the ids starting in pinned host memory and a read-back of
the last fetched row; ``e2e_host_result`` copies the whole result to pinned host memory as well.
The same line carries, as objects with their own rooflines and baselines, the rest of the
metric: ``sampling`` (cached 3-hop neighbour sampling + relabel, sampled edges/s) and ``update``
(fused insert/overwrite + lookups) at N = 1, and ``minibatch_c4`` (sampling + feature fetch over
the partitioned cache on the 111,000,000-node graph) at every N.  ``--workload`` runs one of them
alone.  ``--impl reference`` times the reference's CPU path for the same fetch (``data[q]`` =
torch.index_select on the host table, example/test_cache_fetch.py:138) on the host cores.
Data is synthetic and seeded.
"""
from __future__ import annotations

import argparse
import datetime
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
PG_TIMEOUT = datetime.timedelta(minutes=6)  # a rank that failed ends the others' next collective
LINK_BYTES_PER_ROW = 489  # PCIe read data per 400-byte row fetched from the host table (ncu pcie__read_bytes)
NCU_DRAM_BYTES_PER_LAUNCH = 203_000_000  # 63.8 MB read + 139.2 MB written (ncu, headline batch)
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


class PcieSampler:
    """Polls NVML's PCIe receive counter (bytes the GPU took in over its host link, averaged by
    the driver over 20 ms windows) while a loop runs.  Read-only."""

    def __init__(self, index: int, period_s: float = 0.03):
        self.kbs, self._stop, self._thread = [], threading.Event(), None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv, self._h = pynvml, pynvml.nvmlDeviceGetHandleByIndex(index)
            self._thread = threading.Thread(target=self._run, args=(period_s,), daemon=True)
        except Exception:  # noqa: BLE001
            self._nv = None

    def _run(self, period_s):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.kbs.append(nv.nvmlDeviceGetPcieThroughput(self._h, nv.NVML_PCIE_UTIL_RX_BYTES))
            except Exception:  # noqa: BLE001
                pass
            self._stop.wait(period_s)

    def start(self):
        if self._thread:
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=2)
        busy = [k for k in self.kbs if k > 1e6]  # windows in which the loop was running (> 1 GB/s)
        if not busy:
            return None
        return {"median_gbs": round(statistics.median(busy) * 1e3 / 1e9, 2), "max_gbs": round(max(busy) * 1e3 / 1e9, 2),
                "samples": len(busy)}


def measure_read_rate_ceilings(host_table: torch.Tensor, stream) -> dict:
    """Rates of independent small reads this GPU sustains, by the random-read probe: random
    32-byte sectors of a 4 GiB HBM buffer (what bounds hash probes and relabel tables beyond L2),
    of a 128 MiB buffer (a table that L2 largely holds), and random 16/32-byte reads of the pinned
    host table (what bounds sampling on rows whose adjacency is in host memory)."""
    from shmtensor_b200._lib import check, lib
    sink = torch.zeros(1, dtype=torch.int64, device="cuda")
    out = {}
    big = torch.empty(1 << 32, dtype=torch.uint8, device="cuda")
    def rate(ptr, nbytes, n_reads, unit):
        fn = lambda c=[0]: (check(lib.shmt_random_read(ptr, nbytes, n_reads, unit, c[0], sink.data_ptr(),
                                                       stream.cuda_stream)), c.__setitem__(0, c[0] + 1))
        fn()
        ms = min(time_launches(fn, 1, stream) for _ in range(5))
        return round(n_reads / (ms * 1e-3) / 1e9, 3)
    out["hbm_random_32B_reads_G_per_s_4GiB"] = rate(big.data_ptr(), 1 << 32, 1 << 26, 32)
    out["hbm_random_64B_reads_G_per_s_4GiB"] = rate(big.data_ptr(), 1 << 32, 1 << 26, 64)
    out["hbm_random_64B_reads_G_per_s_128MiB"] = rate(big.data_ptr(), 1 << 27, 1 << 26, 64)
    out["hbm_random_16B_reads_G_per_s_16MiB"] = rate(big.data_ptr(), 1 << 24, 1 << 26, 16)
    del big
    nbytes = host_table.numel() * host_table.element_size()
    out["host_link_random_16B_reads_G_per_s"] = rate(host_table.data_ptr(), nbytes, 1 << 22, 16)
    out["host_link_random_32B_reads_G_per_s"] = rate(host_table.data_ptr(), nbytes, 1 << 22, 32)
    out["host_link_random_128B_reads_G_per_s"] = rate(host_table.data_ptr(), nbytes, 1 << 22, 128)
    out["how"] = "shmt_random_read: independent reads at pseudo-random aligned offsets, 4 per thread in flight, best of 5"
    return out


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


def use_all_host_threads() -> int:
    """torchrun exports OMP_NUM_THREADS=1 to its workers; a CPU arm timed that way uses one core
    of the box.  Give torch (and OpenMP libraries loaded later) every core this process may run on."""
    n = len(os.sched_getaffinity(0))
    os.environ["OMP_NUM_THREADS"] = str(n)
    torch.set_num_threads(n)
    return n


def replicated_rows(n_cached: int, world: int) -> int:
    """Rows of the cached set that every GPU keeps (bench policy, both arms name it in `config`):
    the smallest head of the hotness ranking that takes half of the cached lookups of a batch,
    but at least the library's default."""
    if world <= 1:
        return 0
    from shmtensor_b200.partition import default_replication, head_for_mass
    w = 1.0 / np.arange(1, n_cached + 1, dtype=np.float64) ** ZIPF_ALPHA
    return max(default_replication(n_cached, world), head_for_mass(torch.from_numpy(w), 0.5))


def fetch_config(world: int, hit_rate: float, numa: str) -> dict:
    """`config` of the headline workload; both arms print exactly this."""
    n_cached = int(ROWS * CACHE_FRACTION)
    return {"workload": WORKLOAD, "rows": ROWS, "dim": DIM, "batch": BATCH, "cached_rows": n_cached,
            "hit_rate": round(hit_rate, 4),
            "l2": "inputs larger than L2: 192 MB cached rows + 200 MB output per launch, "
                  f"{N_BATCHES} distinct query batches rotated",
            "partition": "single GPU" if world == 1 else
            f"hash-partitioned over {world} GPUs, NVLink P2P loads; the {replicated_rows(n_cached, world)} "
            f"hottest rows on every GPU; host table pages: {numa}"}


def host_numa_mode(world: int) -> str:
    """Where the shared host table's pages go when several GPUs read it."""
    return "one rank's first touch" if world == 1 else os.environ.get("SHMT_BENCH_NUMA", "interleave")


def gpu_numa_node(index: int):
    """Memory node the GPU's PCIe root port hangs off (None if the kernel does not say)."""
    try:
        p = torch.cuda.get_device_properties(index)
        bdf = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        return int(Path(f"/sys/bus/pci/devices/{bdf}/numa_node").read_text())
    except Exception:  # noqa: BLE001
        return None


def pages_per_node(ptr: int) -> dict:
    """Pages of the mapping that starts at `ptr`, per memory node (/proc/self/numa_maps)."""
    try:
        want = f"{ptr:012x}"
        for ln in Path("/proc/self/numa_maps").read_text().splitlines():
            if ln.split(" ", 1)[0].rjust(12, "0") == want:
                return {tok.split("=")[0]: int(tok.split("=")[1]) for tok in ln.split() if tok[0] == "N" and "=" in tok}
    except Exception:  # noqa: BLE001
        pass
    return {}


# --------------------------------------------------------------------------- reference arm
def run_reference(args) -> None:
    """The reference's CPU path for this fetch, on the host cores: torch.index_select over the
    host table (its ``cpu_fetch`` line).  Rank 0 only."""
    rank, _, world = dist_env()
    if rank != 0:
        return
    from oracle import oracle
    cores = use_all_host_threads()
    table = torch.empty(ROWS, DIM)
    fill_table(table)
    scores = make_scores()
    ranking = np.argsort(-scores, kind="stable")
    batches = make_batches(ranking, N_BATCHES, seed=100)
    cached = np.zeros(ROWS, dtype=bool)
    cached[ranking[:int(ROWS * CACHE_FRACTION)]] = True
    hit_rate = float(np.mean([cached[b.numpy()].mean() for b in batches]))
    for i in range(args.warmup):
        oracle.cpu_fetch_reference(table, batches[i % N_BATCHES])
    t0 = time.perf_counter()
    for i in range(args.steps):
        out = oracle.cpu_fetch_reference(table, batches[i % N_BATCHES])
    dt = time.perf_counter() - t0
    value = args.steps * BATCH * ROW_BYTES / dt / 1e9
    # the reference's own script line ends on the GPU: `data[q.cpu()].cuda()`
    # (example/test_cache_fetch.py:138); timed as well when this box has a GPU
    gpu_resident = None
    if torch.cuda.is_available():
        n = max(3, min(args.steps, 10))
        oracle.cpu_fetch_reference(table, batches[0]).cuda()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for i in range(n):
            res = oracle.cpu_fetch_reference(table, batches[i % N_BATCHES]).cuda()
        torch.cuda.synchronize()
        gpu_resident = n * BATCH * ROW_BYTES / (time.perf_counter() - t0) / 1e9
        del res
    line = {
        "impl": "reference", "metric": METRIC, "value": round(value, 3), "unit": UNIT,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(dt / args.steps * 1e3, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32 rows, int64 ids (byte copy)", "data": "synthetic (seeded)",
        "config": fetch_config(args.gpus, hit_rate, host_numa_mode(args.gpus)),
        "cpu_baseline": {"value": round(value, 3), "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"{args.steps} full batches of 500,000 ids; torch.index_select on the host "
                                   "table = the reference's cpu_fetch (example/test_cache_fetch.py:138), "
                                   f"{cores} threads of {os.cpu_count()} logical cores"},
        "e2e": {"value": round(value, 3), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                "result_in": "host memory"},
        "e2e_gpu_resident": None if gpu_resident is None else {
            "value": round(gpu_resident, 3), "unit": UNIT, "h2d_bytes_per_step": BATCH * ROW_BYTES,
            "what": "data[q].cuda(): index_select on the host cores, then the 200 MB result copied to the GPU "
                    "(the line example/test_cache_fetch.py:138 times)"},
    }
    assert out.shape == (BATCH, DIM)
    emit(line)


# --------------------------------------------------------------------------- our arm
def bind_to_gpu_node(local_rank: int):
    """Run this rank's host threads on the cores of its GPU's memory node (where the kernel
    says which that is and the process may run there).  Returns (node, cores now allowed)."""
    node = gpu_numa_node(local_rank)
    try:
        if node is not None and node >= 0:
            txt = Path(f"/sys/devices/system/node/node{node}/cpulist").read_text().strip()
            cpus = set()
            for part in txt.split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
            cpus &= os.sched_getaffinity(0)
            if cpus:
                os.sched_setaffinity(0, cpus)
    except Exception:  # noqa: BLE001  placement of host threads is an optimisation only
        pass
    return node, len(os.sched_getaffinity(0))


def all_gather_floats(values, world, dev):
    """[rank][i] of a small list of floats."""
    import torch.distributed as dist
    t = torch.tensor(values, device=dev, dtype=torch.float64)
    if world == 1:
        return [t.tolist()]
    out = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(out, t)
    return [o.tolist() for o in out]


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
        dist.init_process_group("nccl", device_id=dev, timeout=PG_TIMEOUT)
    node, n_cores = bind_to_gpu_node(local_rank) if world > 1 else (gpu_numa_node(local_rank), len(os.sched_getaffinity(0)))

    import shmtensor_b200 as st
    from shmtensor_b200 import capi
    from shmtensor_b200._lib import check, lib
    from shmtensor_b200.partition import OWNER_SHIFT, PartitionedFeatureCache

    stream = torch.cuda.current_stream()
    numa_mode = host_numa_mode(world)

    # ---- data: host table shared by the ranks of the node, pinned; cache; batches
    if world > 1:
        name = f"shmt_bench_{os.environ.get('MASTER_PORT', '0')}"
        shm = st.ShmTensor(name, (ROWS, DIM), rank, world, None, torch.float32, pin_memory=True,
                           overwrite_stale=True, numa="interleave" if numa_mode == "interleave" else None)
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
        pcache = PartitionedFeatureCache(table, cached_ids, load_factor=LOAD_FACTOR,
                                         replicate=replicated_rows(n_cached, world))
        pcache.warm()
        fetch = pcache.fetch
        query = pcache.directory.query
    hit_counts = [int((query(b) >= 0).sum().item()) for b in batches]
    hit_rate = sum(hit_counts) / (N_BATCHES * BATCH)

    # ---- set-up, not timed: one streaming pass over the whole host table from this GPU, so that
    #      every page of it has been translated once (GPU TLB / IOMMU) before any step is timed
    _sink = torch.zeros(1, dtype=torch.int64, device=dev)
    check(lib.shmt_stream_read(table.data_ptr(), ROWS * ROW_BYTES, _sink.data_ptr(), stream.cuda_stream))
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
    sampler = ClockSampler(local_rank, period_s=0.005)
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
    my_kernel_ms, my_hit_rate = kernel_ms, hit_rate
    if world > 1:
        t = torch.tensor([region_ms, kernel_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        region_ms, kernel_ms = t.tolist()
    ms_per_step = region_ms / args.steps
    value = world * BATCH * ROW_BYTES / (ms_per_step * 1e6)

    # ---- end to end through the public call: ids from pinned host memory each step, the last
    #      fetched row read back to pinned host memory (the rows stay on the GPU, as the
    #      reference's result does) ...
    ids_dev = torch.empty(BATCH, dtype=torch.int64, device=dev)
    tail = torch.empty(DIM, dtype=torch.float32).pin_memory()

    def e2e_loop(read_back, steps):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        region[0].record(stream)
        for i in range(steps):
            ids_dev.copy_(batches_host[i % N_BATCHES], non_blocking=True)
            res = fetch(ids_dev)
            read_back(res)
            stream.synchronize()
        region[1].record(stream)
        torch.cuda.synchronize()
        ms = region[0].elapsed_time(region[1]) / steps
        wall = (time.perf_counter() - t0) * 1e3 / steps
        if world > 1:
            t_ = torch.tensor([ms], device=dev)
            dist.all_reduce(t_, op=dist.ReduceOp.MAX)
            ms = t_.item()
        return ms, wall

    e2e_serial_ms, _ = e2e_loop(lambda res: tail.copy_(res[-1], non_blocking=True), args.steps)

    # the same one step ahead: step i+1 (its ids on a second stream, its fetch, its read-back) is queued
    # before the host waits for step i's read-back, as a loader that knows its next batch does, so the GPU
    # does not idle while the host turns a step around; every step's ids still come from pinned host
    # memory and every step's result row is still read back and waited for
    pre_stream = torch.cuda.Stream()
    ids_two = [torch.empty(BATCH, dtype=torch.int64, device=dev) for _ in range(2)]
    tails = [torch.empty(DIM, dtype=torch.float32).pin_memory() for _ in range(2)]
    ids_ready = [torch.cuda.Event() for _ in range(2)]
    ids_free = [torch.cuda.Event() for _ in range(2)]
    step_done = [torch.cuda.Event() for _ in range(2)]

    def e2e_prefetched(steps):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        kept = [None, None]
        def issue(j):
            pre_stream.wait_event(ids_free[j % 2])     # the fetch that last read this id buffer is done
            with torch.cuda.stream(pre_stream):
                ids_two[j % 2].copy_(batches_host[j % N_BATCHES], non_blocking=True)
                ids_ready[j % 2].record(pre_stream)
            stream.wait_event(ids_ready[j % 2])
            kept[j % 2] = fetch(ids_two[j % 2])
            ids_free[j % 2].record(stream)
            tails[j % 2].copy_(kept[j % 2][-1], non_blocking=True)
            step_done[j % 2].record(stream)
        for e in ids_free:
            e.record(stream)
        t0 = time.perf_counter()
        region[0].record(stream)
        issue(0)
        for i in range(steps):
            if i + 1 < steps:
                issue(i + 1)
            step_done[i % 2].synchronize()             # the host has step i's row
        region[1].record(stream)
        torch.cuda.synchronize()
        ms = region[0].elapsed_time(region[1]) / steps
        wall = (time.perf_counter() - t0) * 1e3 / steps
        if world > 1:
            t_ = torch.tensor([ms], device=dev)
            dist.all_reduce(t_, op=dist.ReduceOp.MAX)
            ms = t_.item()
        return ms, wall

    e2e_prefetched(3)
    e2e_ms, e2e_wall_ms = e2e_prefetched(args.steps)
    e2e_value = world * BATCH * ROW_BYTES / (e2e_ms * 1e6)
    # ... and with the whole 200 MB result copied out to pinned host memory, which is where the
    # CPU arm's result lies: one step after the other, and pipelined (the copy of step i runs on a
    # second stream while step i+1 is fetched; two output buffers)
    full_host = [torch.empty(BATCH, DIM, dtype=torch.float32).pin_memory() for _ in range(2)]
    host_steps = max(4, min(args.steps, 20))
    e2e_loop(lambda res: full_host[0].copy_(res, non_blocking=True), 2)
    e2e_host_ms, _ = e2e_loop(lambda res: full_host[0].copy_(res, non_blocking=True), host_steps)
    assert torch.equal(full_host[0].view(torch.int32),
                       torch.index_select(table, 0, batches_host[(host_steps - 1) % N_BATCHES]).view(torch.int32))
    copy_stream = torch.cuda.Stream()
    copied = [torch.cuda.Event() for _ in range(2)]
    ids_pair = [torch.empty(BATCH, dtype=torch.int64, device=dev) for _ in range(2)]

    def pipelined(steps):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        region[0].record(stream)
        for i in range(steps):
            if i >= 2:
                copied[i % 2].synchronize()          # the host buffer of two steps ago has been filled
            ids_pair[i % 2].copy_(batches_host[i % N_BATCHES], non_blocking=True)
            res = fetch(ids_pair[i % 2])
            fetched = torch.cuda.Event()
            fetched.record(stream)
            copy_stream.wait_event(fetched)
            with torch.cuda.stream(copy_stream):
                full_host[i % 2].copy_(res, non_blocking=True)
                copied[i % 2].record(copy_stream)
            res.record_stream(copy_stream)
        stream.wait_stream(copy_stream)
        region[1].record(stream)
        torch.cuda.synchronize()
        ms = region[0].elapsed_time(region[1]) / steps
        if world > 1:
            t_ = torch.tensor([ms], device=dev)
            dist.all_reduce(t_, op=dist.ReduceOp.MAX)
            ms = t_.item()
        return ms

    pipelined(2)
    e2e_pipe_ms = pipelined(host_steps)
    for k in (host_steps - 2, host_steps - 1):
        assert torch.equal(full_host[k % 2].view(torch.int32),
                           torch.index_select(table, 0, batches_host[k % N_BATCHES]).view(torch.int32))
    del full_host

    line = {
        "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": round(ms_per_step, 5), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32 rows, int64 ids (byte copy)",
        "data": "synthetic (seeded)",
        "config": fetch_config(world, hit_rate, numa_mode),
        "e2e": {"value": round(e2e_value, 2), "unit": UNIT, "h2d_bytes_per_step": BATCH * 8,
                "d2h_bytes_per_step": DIM * 4, "ms_per_step": round(e2e_ms, 5),
                "wall_ms_per_step": round(e2e_wall_ms, 5),
                "result_in": "GPU memory (as the reference's cache_fetch returns it); one row read back",
                "how": "every step: 4 MB of ids from pinned host memory (on a second stream), the public call, one "
                       "fetched row read back and waited for by the host; step i+1 is queued before the host waits "
                       "for step i",
                "one_step_after_the_other": {"value": round(world * BATCH * ROW_BYTES / (e2e_serial_ms * 1e6), 2),
                                             "ms_per_step": round(e2e_serial_ms, 5),
                                             "how": "copy ids, call, read back, wait; only then the next step"}},
        "e2e_host_result": {"value": round(world * BATCH * ROW_BYTES / (e2e_pipe_ms * 1e6), 2), "unit": UNIT,
                            "h2d_bytes_per_step": BATCH * 8, "d2h_bytes_per_step": BATCH * ROW_BYTES,
                            "ms_per_step": round(e2e_pipe_ms, 5), "steps": host_steps,
                            "result_in": "pinned host memory: the whole fetched batch copied out every step, "
                                         "checked bit-exact; the copy of a step overlaps the fetch of the next",
                            "one_step_after_the_other": {
                                "value": round(world * BATCH * ROW_BYTES / (e2e_host_ms * 1e6), 2),
                                "ms_per_step": round(e2e_host_ms, 5)}},
        "gpu_launches": args.steps,
        "clocks": clocks,
    }

    # ---- N > 1: what every rank saw, the host link under concurrent load, the NVLink regime
    if world > 1:
        from shmtensor_b200.partition import _DeviceBuffer, share_device_buffer
        sink = torch.zeros(1, dtype=torch.int64, device=dev)
        n_hit = sum(hit_counts[i % N_BATCHES] for i in range(args.steps)) / args.steps
        # rows by where they came from (first batch): own shard, a peer's shard, the host table
        v = query(batches[0])
        n_local = int(((v >= 0) & ((v >> OWNER_SHIFT) == rank)).sum().item())
        n_remote = int(((v >= 0) & ((v >> OWNER_SHIFT) != rank)).sum().item())

        # host link with every GPU of the job reading at once: a streaming pass over the shared
        # table (the ceiling), then the same kernel as the headline on ids that all miss
        nbytes = ROWS * ROW_BYTES
        def timed_together(fn, reps):
            best = 1e30
            for _ in range(reps):
                dist.barrier()
                torch.cuda.synchronize()
                best = min(best, time_launches(fn, 1, stream))
            return best
        conc_ms = timed_together(lambda: check(lib.shmt_stream_read(table.data_ptr(), nbytes, sink.data_ptr(),
                                                                     stream.cuda_stream)), 4)
        cold_ids = torch.from_numpy(ranking[n_cached:].copy())
        g = torch.Generator().manual_seed(500 + rank)
        cold_batches = [cold_ids[torch.randint(0, cold_ids.numel(), (BATCH,), generator=g)].to(dev) for _ in range(2)]
        fetch(cold_batches[0])
        miss_ms = timed_together(lambda c=[0]: (fetch(cold_batches[c[0] % 2]), c.__setitem__(0, c[0] + 1)), 3)
        # one GPU at a time (rank 0, then the last rank: the two ends of the PCIe tree)
        solo = {}
        for r in sorted({0, world - 1}):
            dist.barrier()
            if rank == r:
                torch.cuda.synchronize()
                solo_ms = min(time_launches(lambda: check(lib.shmt_stream_read(
                    table.data_ptr(), nbytes, sink.data_ptr(), stream.cuda_stream)), 1, stream) for _ in range(3))
            else:
                solo_ms = 0.0
            t_ = torch.tensor([solo_ms], device=dev)
            dist.all_reduce(t_, op=dist.ReduceOp.MAX)
            solo[r] = round(nbytes / (t_.item() * 1e6), 2)
        per_rank = all_gather_floats([my_kernel_ms, BATCH - n_hit, float(node if node is not None else -1),
                                      nbytes / (conc_ms * 1e6), BATCH * ROW_BYTES / (miss_ms * 1e6),
                                      float(n_local), float(n_remote), float(n_cores)], world, dev)
        line["per_rank"] = [{
            "rank": r, "gpu_numa_node": int(p[2]), "host_cores_bound": int(p[7]), "kernel_ms": round(p[0], 4),
            "miss_rows_per_step": round(p[1]), "miss_gbs": round(p[1] * ROW_BYTES / (p[0] * 1e6), 2),
            "link_ceiling_concurrent_gbs": round(p[3], 2),
            "miss_frac_of_concurrent_ceiling": round(p[1] * ROW_BYTES / (p[0] * 1e6) / p[3], 4),
            "all_miss_concurrent_gbs": round(p[4], 2),
            "rows_local_remote_host_first_batch": [int(p[5]), int(p[6]), BATCH - int(p[5]) - int(p[6])],
        } for r, p in enumerate(per_rank)]
        line["roofline_link"] = {
            "bound": "host_link", "unit": "GB/s",
            "concurrent_peak_gbs": [round(p[3], 2) for p in per_rank],
            "concurrent_peak_total_gbs": round(sum(p[3] for p in per_rank), 1),
            "solo_peak_gbs": solo,
            "achieved": [round(p[1] * ROW_BYTES / (p[0] * 1e6), 2) for p in per_rank],
            "frac": [round(p[1] * ROW_BYTES / (p[0] * 1e6) / p[3], 4) for p in per_rank],
            "peak_source": "shmt_stream_read over the shared pinned host table, all ranks at the same time, "
                           "best of 4 (solo: one rank alone)",
            "host_table_pages_per_node": pages_per_node(table.data_ptr()), "numa_nodes": capi.numa_nodes(),
            "host_table_placement": numa_mode,
            "note": "the headline batch is bound by its misses over the host link; frac = a rank's miss bytes per "
                    "kernel time / what the same rank reads from the same table when all ranks stream from it"}

        # the NVLink regime: ids all cached, most rows on a peer
        probe = _DeviceBuffer(256 << 20)
        ptrs, opened = share_device_buffer(probe)
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
        n_rem = sum(int(((pcache.directory.query(b) >> OWNER_SHIFT) != rank).sum().item()) for b in hot_batches) / 4
        t = torch.tensor([n_rem], device=dev)
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
        # the other way to spend N GPUs: every GPU keeps the cache budget of the 1-GPU run (480,000 rows),
        # so the partitioned cache holds N times as many ids and fewer rows cross the host link
        n_grown = min(world * n_cached, ROWS)
        grown = PartitionedFeatureCache(table, torch.from_numpy(ranking[:n_grown].copy()), load_factor=LOAD_FACTOR,
                                        replicate=replicated_rows(n_cached, world))
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
            "traffic_source": "profiles/row_gather_bulk_mixed.md (ncu dram__bytes_read.sum + dram__bytes_write.sum per launch of the headline batch)",
            "kernel_ms": round(kernel_ms, 5),
            "note": "the 80%-hit batch is bound by the host link, not HBM: see roofline_link and "
                    "frac_of_bound (time at the binding ceiling / measured time)",
            "frac_of_bound": round(t_roof_ms / kernel_ms, 4),
        }
        line["roofline_link"] = {
            "bound": "host_link", "achieved": round(link_bytes / (kernel_ms * 1e6), 2), "peak": link["peak_gbs"],
            "unit": "GB/s", "frac": round(link_bytes / (kernel_ms * 1e6) / link["peak_gbs"], 4),
            "peak_source": "measured in this run", **link, "gpu_numa_node": node,
            # the same launch in bytes that actually cross the link: rows are read in whole lines
            "link_bytes_per_row": LINK_BYTES_PER_ROW,
            "achieved_link_bytes_gbs": round((BATCH - n_hit) * LINK_BYTES_PER_ROW / (kernel_ms * 1e6), 2),
            "frac_link_bytes": round((BATCH - n_hit) * LINK_BYTES_PER_ROW / (kernel_ms * 1e6) / link["peak_gbs"], 4),
            "link_bytes_source": "profiles/row_gather_bulk_mixed.md (ncu pcie__read_bytes.sum per launch / rows from the host)",
            "host_table_pages_per_node": pages_per_node(table.data_ptr())}
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
        pcie = PcieSampler(local_rank)
        pcie.start()
        ms_miss = time_launches(lambda c=[0]: (fetch(cold_batches[c[0] % 4]), c.__setitem__(0, c[0] + 1)), 40, stream)
        rx = pcie.stop()
        line["roofline_all_miss"] = {"bound": "host_link", "achieved": round(BATCH * ROW_BYTES / (ms_miss * 1e6), 2),
                                     "peak": link["peak_gbs"], "unit": "GB/s",
                                     "frac": round(BATCH * ROW_BYTES / (ms_miss * 1e6) / link["peak_gbs"], 4),
                                     "kernel_ms": round(ms_miss, 5),
                                     "ids": "uniform over the 1,920,000 uncached rows, probed and missed",
                                     # bytes the GPU received over PCIe while that loop ran, by NVML's counter
                                     "nvml_pcie_rx_gbs": rx,
                                     "link_bytes_per_row_by_nvml": None if not rx or not rx.get("median_gbs") else
                                     round(rx["median_gbs"] * 1e9 * (ms_miss * 1e-3) / BATCH, 1)}
        # ceilings of the kernels that are bound by a rate of small reads, not by bytes
        line["ceilings"] = measure_read_rate_ceilings(table, stream)
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

    # ---- orderly teardown of the fetch workload: nothing in flight, peers unmapped before any
    #      shard is freed
    torch.cuda.synchronize()
    if pcache is not None:
        pcache.close()
    if world == 1:
        capi.unpin_memory(table)
        del gpu_rows, hmap
    else:
        dist.barrier()
        del pcache
        shm = None
    del table, batches, out, fetch, query
    torch.cuda.empty_cache()

    # ---- the rest of the metric, in the same line: sampled edges/s and the cache update on one
    #      GPU; the end-to-end mini-batch over the partitioned cache on several
    if os.environ.get("SHMT_BENCH_ONLY_FETCH") != "1":
        sub_steps = max(5, min(args.steps, 50))
        def guarded(fn, *a):
            # a failure here must not cost the headline its line
            try:
                return fn(*a)
            except Exception as exc:  # noqa: BLE001
                import traceback
                traceback.print_exc(file=sys.stderr)
                return {"error": f"{type(exc).__name__}: {exc}"[:500]}
        if world == 1:
            line["sampling"] = guarded(sampling_object, sub_steps, local_rank, True)
            line["update"] = guarded(update_object, max(3, min(args.steps, 10)), local_rank)
        line["minibatch_c4"] = guarded(minibatch_object, max(5, min(args.steps, 20)), rank, local_rank, world)
    if rank == 0:
        emit(line)
    if world > 1:
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


def cpu_minibatch(lib, indptr_n, indices_n, seeds32):
    """One 3-hop mini-batch by the threaded C++ restatement of the reference's sampler and
    relabel (the reference has no CPU sampler of its own)."""
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
    return edges, seeds


def sampling_reference_line(args, line, indptr_n, indices_n, seed_batches) -> None:
    from oracle import build_oracle
    use_all_host_threads()
    lib = build_oracle.load_cpu()
    for i in range(max(args.warmup, 1)):
        cpu_minibatch(lib, indptr_n, indices_n, seed_batches[i % 32])
    t0 = time.perf_counter()
    edges = sum(cpu_minibatch(lib, indptr_n, indices_n, seed_batches[i % 32])[0] for i in range(args.steps))
    dt = time.perf_counter() - t0
    v = edges / dt
    line.update({"impl": "reference", "value": round(v, 1), "ms_per_step": round(dt / args.steps * 1e3, 4),
                 "cpu_baseline": {"value": round(v, 1), "unit": "edges/s", "cores": lib.oracle_num_threads(),
                                  "kind": "port", "sample": f"{args.steps} full 3-hop mini-batches; threaded C++ "
                                  "restatement of the reference's sampler (seeds split over threads) + serial relabel"},
                 "e2e": {"value": round(v, 1), "unit": "edges/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
    emit(line)


def sampling_object(steps: int, local_rank: int, full: bool = True) -> dict:
    """Config 3 on one GPU: sampled edges/s of the cached 3-hop mini-batch with relabel, its
    roofline, the reference's own CUDA kernels and the CPU restatement beside it."""
    dev = torch.device("cuda", local_rank)
    from shmtensor_b200 import capi
    from shmtensor_b200._lib import check, lib as shm_lib
    indptr_n, indices_n, deg = make_graph()
    rng = np.random.default_rng(11)
    seed_batches = [rng.integers(0, G_NODES, size=N_SEEDS).astype(np.int32) for _ in range(32)]
    obj = {"metric": "sampled edges/s", "unit": "edges/s", "steps": steps,
           "dtype": "int64 indptr, int32 indices (integer / byte work)",
           "config": {"workload": SAMPLING_WORKLOAD, "nodes": G_NODES, "edges": int(indptr_n[-1]),
                      "fanout": FANOUT, "seeds": N_SEEDS, "hop_order": "reversed(fan-out), as the reference"}}
    indptr, indices = torch.from_numpy(indptr_n), torch.from_numpy(indices_n)
    capi.pin_memory(indptr)
    capi.pin_memory(indices)
    n_cached = G_NODES // 5
    hot_n = np.argsort(-deg, kind="stable")[:n_cached].copy()
    hot = torch.from_numpy(hot_n).to(dev)
    gp, gi = capi.create_subcsr(indptr, indices, hot)
    hmap = capi.CUCOStaticHashmap(hot.int(), torch.arange(n_cached, dtype=torch.int32, device=dev), 0.8)
    seeds_host = [torch.from_numpy(b).pin_memory() for b in seed_batches]
    seeds_dev = [b.to(dev) for b in seeds_host]
    stream = torch.cuda.current_stream()
    capi.set_sampling_seed(7777)

    # parity of one full mini-batch before anything is timed: every hop a legal outcome of the
    # reference's sampler, relabel bit-equal to the oracle's (python/shmtensor/sampling.py:117-147)
    from oracle import oracle
    frontier, hops = capi.sample_minibatch(indptr, indices, seeds_dev[0], list(reversed(FANOUT)), False, gp, gi, hmap)
    cur = seed_batches[0]
    for (sp, sx, rel, nxt), k in zip(hops, reversed(FANOUT)):
        oracle.check_sample_bulk(indptr_n, indices_n, cur, k, False, sp.cpu().numpy(), sx.cpu().numpy(),
                                 distinct_rows=True)
        wu, (ws, wx) = oracle.tensor_relabel([cur.astype(np.int32), sx.cpu().numpy()])
        assert np.array_equal(nxt.cpu().numpy(), wu) and np.array_equal(rel.cpu().numpy(), wx), "relabel differs"
        cur = wu
    del frontier, hops

    def timed(fn, n, warm=3):
        for i in range(warm):
            keep = fn(i)
        region = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
        torch.cuda.synchronize()
        region[0].record(stream)
        edges = 0
        for i in range(n):
            e, keep = fn(i)
            edges += e
        region[1].record(stream)
        torch.cuda.synchronize()
        ms = region[0].elapsed_time(region[1]) / n
        return ms, edges / n

    sampler = ClockSampler(local_rank, period_s=0.1)
    sampler.start()
    ms, edges_per_step = timed(lambda i: minibatch_fused(capi, indptr, indices, gp, gi, hmap, seeds_dev[i % 32]), steps)
    obj["clocks"] = sampler.stop()
    value = edges_per_step / (ms * 1e-3)
    # end to end: seeds start in pinned host memory, the frontier size is read back
    seeds_buf = torch.empty(N_SEEDS, dtype=torch.int32, device=dev)
    def e2e_step(i):
        seeds_buf.copy_(seeds_host[i % 32], non_blocking=True)
        e, frontier = minibatch_fused(capi, indptr, indices, gp, gi, hmap, seeds_buf)
        _ = frontier[-1].item()
        return e, frontier
    e2e_ms, e2e_edges = timed(e2e_step, steps)
    obj.update({"value": round(value, 1), "ms_per_step": round(ms, 5), "edges_per_step": round(edges_per_step),
                "e2e": {"value": round(e2e_edges / (e2e_ms * 1e-3), 1), "unit": "edges/s",
                        "h2d_bytes_per_step": N_SEEDS * 4, "d2h_bytes_per_step": 9 * 8 + 4,
                        "ms_per_step": round(e2e_ms, 5)},
                "gpu_launches": steps * 9, "api": "capi.sample_minibatch (all hops in one native call)"})

    # like with like against the reference, which needs indptr and indices of one dtype: int64 / int64
    indices64 = torch.from_numpy(indices_n.astype(np.int64))
    capi.pin_memory(indices64)
    gp64, gi64 = capi.create_subcsr(indptr, indices64, hot)
    seeds64 = [b.long() for b in seeds_dev]
    ms64, e64 = timed(lambda i: minibatch_fused(capi, indptr, indices64, gp64, gi64, hmap, seeds64[i % 32]), steps)
    obj["int64_indices"] = {"value": round(e64 / (ms64 * 1e-3), 1), "ms_per_step": round(ms64, 5),
                            "what": "the same mini-batch with int64 indices, the only layout the reference accepts"}

    # roofline of the dominant kernel: the last hop's sampling kernel.  What bounds it is the rate
    # of small reads over the host link (row-offset pairs and picked neighbours of rows that are
    # not cached), so the ceiling is the random-read probe on the same pinned array.
    hop_seeds = []
    for i in range(8):
        s_ = seeds_dev[i]
        for k in list(reversed(FANOUT))[:-1]:
            _, sx = capi.csr_cache_sampling(indptr, indices, gp, gi, hmap, s_, k, False)
            s_, _ = capi.tensor_relabel([s_, sx])
        hop_seeds.append(s_)
    k_last = list(reversed(FANOUT))[-1]
    def last_hop(i):
        sp, sx = capi.csr_cache_sampling(indptr, indices, gp, gi, hmap, hop_seeds[i % 8], k_last, False)
        return sx.numel(), sx
    hop_ms, hop_edges = timed(last_hop, max(20, steps))
    fr = hop_seeds[0].cpu().numpy().astype(np.int64)
    is_hot = np.zeros(G_NODES, dtype=bool)
    is_hot[hot_n] = True
    cold = fr[~is_hot[fr]]
    d_cold = deg[cold].astype(np.float64)
    begin_cold = indptr_n[cold]
    # requests over the link per cold row: one for the row-offset pair, then one per distinct
    # 128-byte line of its adjacency list that is touched -- all lines of a row copied whole,
    # the expected number of distinct lines among k uniform picks otherwise
    lines = np.maximum(((begin_cold * 4) % 128 + d_cold * 4 + 127) // 128, 1)
    touched = np.where(d_cold <= k_last, lines, lines * (1.0 - (1.0 - 1.0 / lines) ** k_last))
    link_reads = int(cold.size + touched[d_cold > 0].sum())
    sink = torch.zeros(1, dtype=torch.int64, device=dev)
    n_probe = 1 << 21
    probe = lambda c=[0]: (check(shm_lib.shmt_random_read(indices.data_ptr(), indices.numel() * 4, n_probe, 16, c[0],
                                                          sink.data_ptr(), stream.cuda_stream)), c.__setitem__(0, c[0] + 1))
    probe()
    probe_ms = min(time_launches(probe, 1, stream) for _ in range(5))
    ceiling = n_probe / (probe_ms * 1e-3)
    peak, peak_src = measured_peaks()
    sizes = [(N_SEEDS, 0)]
    alg = 0
    cur_n = N_SEEDS
    frontier, hops = capi.sample_minibatch(indptr, indices, seeds_dev[0], list(reversed(FANOUT)), False, gp, gi, hmap)
    for sp, sx, rel, nxt in hops:
        nnz, nu = sx.numel(), nxt.numel()
        # per seed: id 4 + probe 12 + row offsets 16 + offset written 8; per edge: 4 read + 4 written;
        # relabel: ids read twice, slot + new id written and read, unique ids written
        alg += cur_n * (4 + 12 + 16 + 8) + nnz * 8 + (cur_n + nnz) * (4 + 4 + 4 * 3) + nu * 4
        cur_n = nu
    obj["roofline"] = {
        "bound": "host link, rate of small reads (not bytes)", "kernel": "sample_hop_kernel<int,16> (the last hop of reversed [15,10,5]: fan-out 15)",
        "kernel_ms": round(hop_ms, 5), "kernel_share_of_step": round(hop_ms / ms, 3),
        "link_reads_per_launch": link_reads, "achieved": round(link_reads / (hop_ms * 1e-3) / 1e9, 4),
        "peak": round(ceiling / 1e9, 4), "unit": "G reads/s", "frac": round(link_reads / (hop_ms * 1e-3) / ceiling, 4),
        "peak_source": "shmt_random_read: independent 16-byte reads (one request each) of the same pinned indices "
                       "array, 4 per thread in flight, measured in this run",
        "cold_rows_per_launch": int(cold.size), "frontier_rows_per_launch": int(fr.size),
        "algorithmic_bytes": int(alg), "hbm_achieved_gbs": round(alg / (ms * 1e6), 1), "hbm_peak": peak,
        "hbm_frac": round(alg / (ms * 1e6) / peak, 5), "hbm_peak_source": peak_src, "traffic": None,
        "note": "a cold row of the frontier costs one request for its row-offset pair and then one per 128-byte line of "
                "its adjacency list that a pick falls in, the second depending on the first; the link serves about 0.3 G "
                "such requests per second whatever their size, so bytes do not matter here"}

    if full:
        # uncached (every row over UVA) and fully GPU-resident graph, for the cache's effect
        extra = {}
        variants = {"uva_only": (minibatch_fused, indptr, indices, None, None, None),
                    "all_in_hbm": (minibatch_fused, indptr.to(dev), indices.to(dev), None, None, None),
                    "call_per_hop_cached": (minibatch, indptr, indices, gp, gi, hmap),
                    # not the configured workload: the whole indptr (19 MB) mirrored in HBM, so a cold
                    # row costs one trip over the host link instead of two
                    "cached_plus_indptr_in_hbm": (minibatch_fused, indptr.to(dev), indices, gp, gi, hmap)}
        for name, (fn, ip, ix, a, b, m) in variants.items():
            vms, ve = timed(lambda i: fn(capi, ip, ix, a, b, m, seeds_dev[i % 32]), min(steps, 30))
            extra[name] = round(ve / (vms * 1e-3), 1)
        obj["variants_edges_per_s"] = extra

    # same-box numbers of the reference's own CUDA kernels, when oracle/_ref was built
    ref_line = None
    try:
        from oracle import build_ref
        ref = build_ref.load_reference()
        if ref is None:
            ref_line = {"unavailable": "oracle/_ref has not been built"}
    except Exception as exc:  # noqa: BLE001
        ref, ref_line = None, {"unavailable": f"reference build not loadable: {exc}"}
    if ref is not None:
        rgp, rgi = ref.create_subcsr(indptr, indices64, hot)
        rmap = ref.CUCOStaticHashmap(hot.int(), torch.arange(n_cached, dtype=torch.int32, device=dev), 0.8)
        def ref_batch(i):
            seeds, ed = seeds_dev[i % 32], 0
            for k in reversed(FANOUT):
                sp, so = ref.csr_cache_sampling(indptr, indices64, rgp, rgi, rmap, seeds, k, False)
                seeds, _ = ref.tensor_relabel([seeds.long(), so])
                ed += so.numel()
            return ed, seeds
        ref_ms, ref_e = timed(ref_batch, min(steps, 30))
        ref_line = {"edges_per_s": round(ref_e / (ref_ms * 1e-3), 1), "ms_per_step": round(ref_ms, 4),
                    "ours_over_reference_int32_indices": round(value / (ref_e / (ref_ms * 1e-3)), 3),
                    "ours_over_reference_int64_indices": round(e64 / (ms64 * 1e-3) / (ref_e / (ref_ms * 1e-3)), 3),
                    "what": "the reference's own sampling + relabel kernels (compiled unmodified, int64 indices as it "
                            "requires equal dtypes) over a stand-in for its cuCollections map"}
    obj["reference_cuda"] = ref_line
    capi.unpin_memory(indices64)
    # CPU baseline beside it (bounded sample)
    from oracle import build_oracle
    use_all_host_threads()
    cpu = build_oracle.load_cpu()
    cpu_minibatch(cpu, indptr_n, indices_n, seed_batches[0])
    t0 = time.perf_counter()
    ce = sum(cpu_minibatch(cpu, indptr_n, indices_n, seed_batches[i])[0] for i in range(10))
    cpu_dt = time.perf_counter() - t0
    obj["cpu_baseline"] = {"value": round(ce / cpu_dt, 1), "unit": "edges/s", "cores": cpu.oracle_num_threads(),
                           "kind": "port", "sample": "10 full 3-hop mini-batches; threaded C++ restatement of the "
                           "reference's sampler + serial relabel (the reference has no CPU sampler)"}
    capi.unpin_memory(indptr)
    capi.unpin_memory(indices)
    del gp, gi, gp64, gi64, hmap, hops, frontier
    torch.cuda.empty_cache()
    return obj


def run_sampling(args) -> None:
    rank, local_rank, world = dist_env()
    if rank != 0:
        return
    line = {"metric": "sampled edges/s", "unit": "edges/s", "n_gpus": 1, "steps": args.steps,
            "warmup": max(args.warmup, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int64 indptr, int32 indices (integer / byte work)", "data": "synthetic (seeded)"}
    if args.impl == "reference":
        indptr_n, indices_n, deg = make_graph()
        rng = np.random.default_rng(11)
        seed_batches = [rng.integers(0, G_NODES, size=N_SEEDS).astype(np.int32) for _ in range(32)]
        line["config"] = {"workload": SAMPLING_WORKLOAD, "nodes": G_NODES, "edges": int(indptr_n[-1]),
                          "fanout": FANOUT, "seeds": N_SEEDS, "hop_order": "reversed(fan-out), as the reference"}
        sampling_reference_line(args, line, indptr_n, indices_n, seed_batches)
        return
    assert torch.cuda.is_available(), "bench.py needs a GPU (there is no CPU path)"
    torch.cuda.set_device(local_rank)
    line.update(sampling_object(args.steps, local_rank, full=True))
    emit(line)


# --------------------------------------------------------------------------- end-to-end mini-batch
C4_NODES, C4_EDGES, C4_DIM, C4_CAP, C4_CACHE_FRACTION = 111_000_000, 1_600_000_000, 128, 10_000, 0.40
C4_STEPS = [7, 11, 13, 17, 19, 23, 29, 31, 41, 43, 47, 53, 59, 61, 67, 71]  # coprime to 111,000,000 / 2^s


def c4_scale() -> tuple:
    """Config 4 needs 64 GB of host memory for its graph and features (111,000,000 x (8 + 512) bytes
    + 1,600,000,000 x 4 bytes), in shared memory that every rank maps.  Returns (divisor, why):
    1 when the box holds that, else the smallest power of two that makes it fit."""
    forced = os.environ.get("SHMT_BENCH_C4_SCALE")
    if forced:
        return int(forced), f"forced by SHMT_BENCH_C4_SCALE={forced}"
    limits = {}
    try:
        st_ = os.statvfs("/dev/shm")
        limits["/dev/shm free"] = st_.f_bavail * st_.f_frsize * 0.85
    except OSError:
        pass
    try:
        for ln in Path("/proc/meminfo").read_text().splitlines():
            if ln.startswith("MemAvailable:"):
                limits["MemAvailable"] = int(ln.split()[1]) * 1024 * 0.6
    except OSError:
        pass
    try:
        raw = Path("/sys/fs/cgroup/memory.max").read_text().strip()
        if raw != "max":
            limits["cgroup memory.max"] = int(raw) * 0.6
    except (OSError, ValueError):
        pass
    need = lambda d: (C4_NODES // d) * (8 + C4_DIM * 4) + (C4_EDGES // d) * 4
    limit_name, limit = min(limits.items(), key=lambda kv: kv[1]) if limits else ("unknown", float("inf"))
    d = 1
    while need(d) > limit and d < 1024:
        d *= 2
    gb = {k: round(v / 1e9, 1) for k, v in limits.items()}
    return d, (f"needs {need(1) / 1e9:.1f} GB of shared host memory; usable here {gb} (fractions of what the box reports)"
               + ("" if d == 1 else f"; bound by {limit_name}"))


def c4_degrees(n_nodes: int, n_edges: int, dev) -> torch.Tensor:
    """Out-degrees with a Zipf(2.0) tail: the integer part of a Pareto(1) draw, P(k) = 1/(k(k+1)),
    capped at 10,000 and rescaled so that they sum to the edge count.  Same on every rank (seeded
    generator of the same GPU model)."""
    g = torch.Generator(device=dev).manual_seed(404)
    u = torch.rand(n_nodes, generator=g, device=dev, dtype=torch.float64).clamp_(min=1.0 / (C4_CAP + 1))
    raw = torch.floor(1.0 / u).clamp_(max=C4_CAP)
    lo, hi = 0.1, 50.0
    for _ in range(60):
        mid = 0.5 * (lo + hi)
        if torch.floor(raw * mid).clamp_(max=C4_CAP).sum().item() > n_edges:
            hi = mid
        else:
            lo = mid
    deg = torch.floor(raw * lo).clamp_(max=C4_CAP).to(torch.int64)
    short = n_edges - int(deg.sum().item())
    bump = torch.nonzero(deg < C4_CAP).flatten()[:short]
    deg[bump] += 1
    return deg


def c4_fill_graph(indices_host: torch.Tensor, indptr_dev: torch.Tensor, n_nodes: int, lo_row: int, hi_row: int, dev) -> None:
    """Neighbours of rows [lo_row, hi_row): an arithmetic progression modulo the node count from a
    hashed start with a hashed prime step (distinct within a row, spread uniformly over the nodes),
    made on the GPU in pieces and copied into the shared host array."""
    steps = torch.tensor(C4_STEPS, device=dev, dtype=torch.int64)
    piece = 8_000_000
    for a in range(lo_row, hi_row, piece):
        b = min(a + piece, hi_row)
        e0, e1 = int(indptr_dev[a].item()), int(indptr_dev[b].item())
        if e1 == e0:
            continue
        rows = torch.arange(a, b, device=dev, dtype=torch.int64)
        deg = indptr_dev[a + 1:b + 1] - indptr_dev[a:b]
        row = torch.repeat_interleave(rows, deg)
        j = torch.arange(e0, e1, device=dev, dtype=torch.int64) - indptr_dev[row]
        base = (row * 2654435761 + 12345) % n_nodes
        step = steps[(row * 40503 >> 3) % len(C4_STEPS)]
        indices_host[e0:e1].copy_(((base + j * step) % n_nodes).to(torch.int32))
        del rows, deg, row, j, base, step


def c4_fill_features(feats_host: torch.Tensor, lo_row: int, hi_row: int, dev) -> None:
    """N(0,1) rows made on the GPU (one seeded generator per piece) and copied to the shared table."""
    piece = 2_000_000
    for a in range(lo_row, hi_row, piece):
        b = min(a + piece, hi_row)
        g = torch.Generator(device=dev).manual_seed(9000 + a // piece)
        feats_host[a:b].copy_(torch.randn(b - a, C4_DIM, generator=g, device=dev))


def minibatch_workload(n_nodes, n_edges, divisor) -> str:
    return ("end-to-end mini-batch over a partitioned cache (config 4" + ("" if divisor == 1 else f", scaled 1:{divisor}")
            + f"): power-law CSR {n_nodes:,} nodes / {n_edges:,} edges (degree tail Zipf(2.0), int64 indptr, int32 "
            f"indices), {C4_DIM}-d float32 features ({n_nodes * C4_DIM * 4 / 1e9:.1f} GB), graph and features in POSIX shared "
            f"memory mapped and pinned by every rank; every GPU holds the row offsets ({n_nodes * 8 / 1e9:.1f} GB) and the adjacency of the "
            "top 40% of nodes by degree, whose features are hash-partitioned over the GPUs; per GPU and step 1,024 seeds, fan-out "
            "[15,10,5], then the features of every sampled node are fetched (remote hits over NVLink, misses over UVA)")


def minibatch_object(steps: int, rank: int, local_rank: int, world: int) -> dict:
    """Config 4: sampling + relabel + feature fetch of every sampled node, per GPU and step, over
    a cache partitioned across the GPUs of the job.  Assumes the process group exists when
    world > 1.  Every rank returns the same object."""
    import torch.distributed as dist
    import shmtensor_b200 as st
    from shmtensor_b200 import capi
    from shmtensor_b200._lib import check, lib as shm_lib
    from shmtensor_b200.partition import PartitionedFeatureCache
    dev = torch.device("cuda", local_rank)
    stream = torch.cuda.current_stream()
    t_setup = time.perf_counter()
    divisor, why = c4_scale()
    n_nodes, n_edges = C4_NODES // divisor, C4_EDGES // divisor
    numa_mode = host_numa_mode(world) if world > 1 else None
    obj = {"metric": "mini-batches/s (sampled edges/s, fetched feature GB/s)", "unit": "mini-batches/s",
           "n_gpus": world, "steps": steps, "scaling": "weak",
           "dtype": "int32 ids, f32 rows (integer / byte work)",
           "config": {"workload": minibatch_workload(n_nodes, n_edges, divisor), "nodes": n_nodes, "edges": n_edges,
                      "dim": C4_DIM, "fanout": FANOUT, "seeds_per_gpu": N_SEEDS, "scale_divisor": divisor,
                      "scale_reason": why, "host_table_placement": numa_mode or "one rank's first touch"}}

    # ---- host side: three shared segments, pages placed, then pinned by every rank
    tag = os.environ.get("MASTER_PORT", str(os.getpid()))
    numa = "interleave" if numa_mode == "interleave" else None
    def shared(name, shape, dtype):
        if world > 1:
            return st.ShmTensor(f"shmt_c4_{name}_{tag}", shape, rank, world, None, dtype, pin_memory=True,
                                overwrite_stale=True, numa=numa)
        return st.ShmTensor(f"shmt_c4_{name}_{tag}", shape, 0, 1, None, dtype, pin_memory=True, overwrite_stale=True)
    shm_ptr, shm_idx, shm_feat = (shared("indptr", (n_nodes + 1,), torch.int64),
                                  shared("indices", (n_edges,), torch.int32),
                                  shared("feats", (n_nodes, C4_DIM), torch.float32))
    indptr, indices, feats = shm_ptr.tensor_, shm_idx.tensor_, shm_feat.tensor_
    t_mapped = time.perf_counter()

    deg = c4_degrees(n_nodes, n_edges, dev)
    indptr_dev = torch.zeros(n_nodes + 1, dtype=torch.int64, device=dev)
    torch.cumsum(deg, 0, out=indptr_dev[1:])
    if rank == 0:
        indptr.copy_(indptr_dev)
    # every rank writes its share of the edges (split by edge count) and of the feature rows
    cuts = torch.searchsorted(indptr_dev, torch.arange(world + 1, device=dev) * (n_edges // world)).tolist()
    cuts[0], cuts[-1] = 0, n_nodes
    c4_fill_graph(indices, indptr_dev, n_nodes, cuts[rank], cuts[rank + 1], dev)
    c4_fill_features(feats, rank * n_nodes // world, (rank + 1) * n_nodes // world, dev)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t_filled = time.perf_counter()

    # ---- caches: adjacency of the top 40 % by degree on every GPU (built from a temporary GPU copy
    #      of the edge array), their features partitioned over the GPUs
    n_cached = int(n_nodes * C4_CACHE_FRACTION)
    hot = torch.sort(deg, descending=True, stable=True).indices[:n_cached].contiguous()
    del deg
    indices_dev = indices.to(dev, non_blocking=True)
    gp, gi = capi.create_subcsr(indptr_dev, indices_dev, hot)
    del indices_dev   # the row offsets (0.9 GB) stay on the GPU: see `step`
    gmap = capi.CUCOStaticHashmap(hot.int(), torch.arange(n_cached, dtype=torch.int32, device=dev), 0.8)
    fcache = PartitionedFeatureCache(feats, hot, replicate=0)   # neighbours are uniform over the nodes: no hot head
    fcache.warm()
    del hot
    torch.cuda.empty_cache()
    t_cached = time.perf_counter()

    rng = np.random.default_rng(100 + rank)
    seed_batches = [rng.integers(0, n_nodes, size=N_SEEDS).astype(np.int32) for _ in range(32)]
    seeds_host = [torch.from_numpy(b).pin_memory() for b in seed_batches]
    seeds_buf = torch.empty(N_SEEDS, dtype=torch.int32, device=dev)
    tail = torch.empty(C4_DIM, dtype=torch.float32).pin_memory()
    capi.set_sampling_seed(7777 + rank)
    fan = list(reversed(FANOUT))

    # The sampler reads row offsets from the GPU copy (what GPUSamplingDataloader.create_cache does when
    # they fit in a quarter of its budget: a row whose adjacency is in host memory then costs one trip over
    # the host link instead of two) and the adjacency of rows that are not cached from the shared host array.
    def step(i):
        seeds_buf.copy_(seeds_host[i % 32], non_blocking=True)
        frontier, hops = capi.sample_minibatch(indptr_dev, indices, seeds_buf, fan, False, gp, gi, gmap)
        rows = fcache.fetch(frontier)
        return sum(h[1].numel() for h in hops), frontier, rows, hops

    # ---- parity of one full step on every rank: each hop a legal outcome of the reference's sampler,
    #      relabel as the oracle's, fetched rows the host rows of the frontier bit for bit
    from oracle import oracle
    _, frontier, rows, hops = step(0)
    indptr_n, indices_n = indptr.numpy(), indices.numpy()
    cur = seed_batches[0]
    for (sp, sx, rel, nxt), k in zip(hops, fan):
        oracle.check_sample_bulk(indptr_n, indices_n, cur, k, False, sp.cpu().numpy(), sx.cpu().numpy(), distinct_rows=True)
        wu, (ws, wx) = oracle.tensor_relabel([cur.astype(np.int32), sx.cpu().numpy()])
        assert np.array_equal(nxt.cpu().numpy(), wu) and np.array_equal(rel.cpu().numpy(), wx), "relabel differs"
        cur = wu
    assert torch.equal(rows.cpu().view(torch.int32), feats[frontier.cpu().long()].view(torch.int32)), "fetched rows differ"
    hits = int((fcache.directory.query(frontier.long()) >= 0).sum().item())
    hit_rate = hits / frontier.numel()
    del hops

    for i in range(3):
        e, frontier, rows, _ = step(i)
    sampler = ClockSampler(local_rank, period_s=0.1)
    region = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
    mid = [torch.cuda.Event(enable_timing=True) for _ in range(2 * steps)]
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler.start()
    region[0].record(stream)
    edges = n_rows = 0
    for i in range(steps):
        seeds_buf.copy_(seeds_host[i % 32], non_blocking=True)
        frontier, hops = capi.sample_minibatch(indptr_dev, indices, seeds_buf, fan, False, gp, gi, gmap)
        mid[2 * i].record(stream)
        rows = fcache.fetch(frontier)
        mid[2 * i + 1].record(stream)
        tail.copy_(rows[-1], non_blocking=True)
        edges += sum(h[1].numel() for h in hops)
        n_rows += rows.shape[0]
    region[1].record(stream)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    clocks = sampler.stop()
    ms = region[0].elapsed_time(region[1]) / steps
    fetch_ms = sum(mid[2 * i].elapsed_time(mid[2 * i + 1]) for i in range(steps)) / steps
    per_rank = all_gather_floats([ms, float(edges), float(n_rows), fetch_ms, hit_rate], world, dev)
    ms_max = max(p[0] for p in per_rank)
    edges_all, rows_all = sum(p[1] for p in per_rank), sum(p[2] for p in per_rank)

    # The same steps with the sampler on a stream of its own: the host queues the fetch of step i, then
    # samples step i+1 (a call that waits for its sizes), so the GPU runs that sampling beside the fetch.
    side = torch.cuda.Stream(device=dev)
    seeds_side = [torch.empty(N_SEEDS, dtype=torch.int32, device=dev) for _ in range(2)]

    def sample_ahead(i):
        with torch.cuda.stream(side):
            seeds_side[i % 2].copy_(seeds_host[i % 32], non_blocking=True)
            frontier, hops = capi.sample_minibatch(indptr_dev, indices, seeds_side[i % 2], fan, False, gp, gi, gmap)
            done = torch.cuda.Event()
            done.record(side)
        return frontier, hops, done

    def overlapped(n):
        edges = 0
        ahead = sample_ahead(0)
        for i in range(n):
            frontier, hops, done = ahead
            stream.wait_event(done)
            frontier.record_stream(stream)
            rows = fcache.fetch(frontier)
            tail.copy_(rows[-1], non_blocking=True)
            edges += sum(h[1].numel() for h in hops)
            if i + 1 < n:
                ahead = sample_ahead(i + 1)
        return edges
    overlapped(3)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    region[0].record(stream)
    overlapped(steps)
    region[1].record(stream)
    torch.cuda.synchronize()
    ms_ov_wall = (time.perf_counter() - t0) * 1e3 / steps
    if world > 1:
        dist.barrier()
    ms_ov = all_gather_floats([max(ms_ov_wall, region[0].elapsed_time(region[1]) / steps)], world, dev)
    ms_ov_max = max(p[0] for p in ms_ov)

    # the host link while every rank streams from the shared feature table at once: the ceiling
    # of the fetch's miss leg, which is what bounds a step
    sink = torch.zeros(1, dtype=torch.int64, device=dev)
    probe_bytes = min(feats.numel() * 4, 1 << 30)
    best = 1e30
    for _ in range(3):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        best = min(best, time_launches(lambda: check(shm_lib.shmt_stream_read(feats.data_ptr(), probe_bytes, sink.data_ptr(),
                                                                              stream.cuda_stream)), 1, stream))
    link = all_gather_floats([probe_bytes / (best * 1e6)], world, dev)
    miss_bytes = [(1 - p[4]) * p[2] / steps * C4_DIM * 4 for p in per_rank]

    obj.update({
        "value": round(world / (ms_max * 1e-3), 1), "ms_per_step": round(ms_max, 5),
        "edges_per_s": round(edges_all / steps / (ms_max * 1e-3), 1),
        "fetched_gbs": round(rows_all / steps * C4_DIM * 4 / (ms_max * 1e6), 2),
        "rows_fetched_per_gpu_step": round(rows_all / steps / world), "feature_hit_rate": round(hit_rate, 4),
        "per_rank_ms": [round(p[0], 4) for p in per_rank], "per_rank_fetch_ms": [round(p[3], 4) for p in per_rank],
        "sampling_a_step_ahead": {"value": round(world / (ms_ov_max * 1e-3), 1), "unit": "mini-batches/s",
                                  "ms_per_step": round(ms_ov_max, 5), "per_rank_ms": [round(p[0], 4) for p in ms_ov],
                                  "what": "the same steps with the sampler on its own stream, so that the sampling of "
                                          "step i+1 runs beside the feature fetch of step i (wall clock of the loop, "
                                          "slowest rank)"},
        "e2e": {"value": round(world / (ms_max * 1e-3), 1), "unit": "mini-batches/s", "h2d_bytes_per_step": N_SEEDS * 4,
                "d2h_bytes_per_step": C4_DIM * 4 + 9 * 8, "ms_per_step": round(ms_max, 5),
                "note": "the timed loop is end to end: seeds from pinned host memory, sizes and the last fetched "
                        "row read back"},
        "roofline": {"bound": "host_link", "kernel": "row_gather_bulk_kernel<2> (feature fetch of the frontier)",
                     "kernel_ms": [round(p[3], 4) for p in per_rank],
                     "achieved": [round(b / (p[3] * 1e6), 2) for b, p in zip(miss_bytes, per_rank)],
                     "peak": [round(l[0], 2) for l in link], "unit": "GB/s",
                     "frac": [round(b / (p[3] * 1e6) / l[0], 4) for b, p, l in zip(miss_bytes, per_rank, link)],
                     "peak_source": "shmt_stream_read over the shared pinned feature table, all ranks at once, this run",
                     "algorithmic_bytes": "rows x 512 B written + hit rows x 512 B read (HBM / NVLink) + miss rows x 512 B (host link)",
                     "traffic": None},
        "gpu_launches": steps * 10, "clocks": clocks,
        "setup_s": {"map_and_pin": round(t_mapped - t_setup, 1), "generate": round(t_filled - t_mapped, 1),
                    "build_caches": round(t_cached - t_filled, 1)},
        "host_pages_per_node": {"feats": pages_per_node(feats.data_ptr()), "indices": pages_per_node(indices.data_ptr())},
    })
    # CPU beside it: one GPU only (with more ranks the other processes' threads share the cores), bounded:
    # the threaded C++ sampler + relabel, then index_select on the table
    obj["cpu_baseline"] = None
    if world == 1:
        from oracle import build_oracle
        use_all_host_threads()
        cpu = build_oracle.load_cpu()
        def cpu_step(seeds32):
            e, fr = cpu_minibatch(cpu, indptr_n, indices_n, seeds32)
            return e, oracle.cpu_fetch_reference(feats, torch.from_numpy(fr)).shape[0]
        cpu_step(seed_batches[0])
        t0 = time.perf_counter()
        n_cpu = 3
        for i in range(n_cpu):
            cpu_step(seed_batches[1 + i])
        cpu_dt = (time.perf_counter() - t0) / n_cpu
        obj["cpu_baseline"] = {"value": round(1 / cpu_dt, 2), "unit": "mini-batches/s", "cores": cpu.oracle_num_threads(),
                               "kind": "port", "ms_per_step": round(cpu_dt * 1e3, 2),
                               "sample": f"{n_cpu} full mini-batches: threaded C++ sampler + serial relabel + "
                                         "torch.index_select on the shared feature table"}
    torch.cuda.synchronize()
    fcache.close()
    del fcache, gp, gi, gmap, indptr, indices, feats, indptr_n, indices_n, rows, frontier, indptr_dev
    shm_ptr = shm_idx = shm_feat = None
    torch.cuda.empty_cache()
    return obj


def run_minibatch(args) -> None:
    rank, local_rank, world = dist_env()
    if args.impl == "reference":
        if rank == 0:
            emit({"impl": "reference", "unavailable": "the CPU line of this workload is the cpu_baseline object of the "
                  "GPU arm's own run (it needs the same 64 GB of generated graph and features)"})
        return
    assert torch.cuda.is_available(), "bench.py needs a GPU (there is no CPU path)"
    torch.cuda.set_device(local_rank)
    import torch.distributed as dist
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank), timeout=PG_TIMEOUT)
        bind_to_gpu_node(local_rank)
    obj = minibatch_object(args.steps, rank, local_rank, world)
    line = {"metric": obj.pop("metric"), "value": obj.pop("value"), "unit": obj.pop("unit"), "n_gpus": world,
            "steps": args.steps, "warmup": 3, "ms_per_step": obj.pop("ms_per_step"), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "data": "synthetic (seeded)", **obj}
    if rank == 0:
        emit(line)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# --------------------------------------------------------------------------- update workload
U_KEYS, U_DIM, U_LOOKUPS = 4_000_000, 256, 1_000_000
UPDATE_WORKLOAD = ("cache update path: fused insert/overwrite of 4,000,000 unique int64 keys (uniform over 2^40) with "
                   "256-d bfloat16 rows into an empty 1-GPU cache at load factor 0.5, then 1,000,000 lookups, "
                   "half present, half absent")


def update_keys():
    rng = np.random.default_rng(5)
    keys_n = np.unique(rng.integers(0, 1 << 40, size=U_KEYS + 100_000))
    keys_n = rng.permutation(keys_n)[:U_KEYS].astype(np.int64)
    req_n = np.concatenate([keys_n[rng.integers(0, U_KEYS, size=U_LOOKUPS // 2)],
                            rng.integers(1 << 40, 1 << 41, size=U_LOOKUPS // 2)]).astype(np.int64)
    rng.shuffle(req_n)
    return keys_n, req_n


def update_cpu(steps: int, warmup: int, keys_n, req_n, sample: int = 1) -> dict:
    """CPU path: row write data[ids] = upd (example/test_cache_set.py:183-184) + an open-addressing
    map built and queried on all cores (the reference's map is GPU-only).  `sample` > 1 times the
    first 1/sample of the keys and lookups."""
    from oracle import build_oracle
    use_all_host_threads()
    lib = build_oracle.load_cpu()
    row_bytes = U_DIM * 2
    n_keys, n_req = U_KEYS // sample, U_LOOKUPS // sample
    rows = np.zeros((n_keys, row_bytes), np.uint8)
    rows[:] = np.arange(row_bytes, dtype=np.uint8)
    table_rows = np.empty_like(rows)
    slots = np.arange(n_keys, dtype=np.int64)
    cap = 1 << 23
    while cap // 2 >= 2 * n_keys:
        cap //= 2
    table = np.empty(2 * cap, np.int64)
    out = np.empty(n_req, np.int32)
    def step():
        lib.oracle_map_build_query(keys_n.ctypes.data, n_keys, table.ctypes.data, cap, req_n.ctypes.data,
                                   n_req, out.ctypes.data)
        lib.oracle_scatter(table_rows.ctypes.data, slots.ctypes.data, n_keys, row_bytes, rows.ctypes.data)
    for _ in range(max(warmup, 1)):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    v = (n_keys + n_req) / dt
    return {"value": round(v, 1), "unit": "keys/s", "cores": lib.oracle_num_threads(), "kind": "port",
            "ms_per_step": round(dt * 1e3, 3),
            "sample": f"{steps} passes over {'all' if sample == 1 else f'the first 1/{sample} of'} the keys and lookups: "
                      "threaded open-addressing build + query and a threaded row scatter"}


def update_object(steps: int, local_rank: int) -> dict:
    """Config 5 on one GPU: fused insert/overwrite of 4,000,000 keys with 512-byte rows into an
    empty cache, then 1,000,000 lookups; rooflines, the reference's map and the CPU beside it."""
    dev = torch.device("cuda", local_rank)
    from shmtensor_b200 import capi
    from shmtensor_b200._lib import check, lib as shm_lib
    row_bytes = U_DIM * 2
    obj = {"metric": "inserted+looked-up keys/s", "unit": "keys/s", "steps": steps,
           "dtype": "int64 keys, int32 slots, bf16 rows (byte copy)",
           "config": {"workload": UPDATE_WORKLOAD, "keys": U_KEYS, "row_bytes": row_bytes, "lookups": U_LOOKUPS}}
    keys_n, req_n = update_keys()
    keys_host, req_host = torch.from_numpy(keys_n).pin_memory(), torch.from_numpy(req_n).pin_memory()
    keys = keys_host.to(dev)
    req = req_host.to(dev)
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

    for _ in range(3):
        m, out = one_pass()
    # parity at full size: rows and slots bit-exact, absent keys -1
    assert torch.equal(gpu.view(torch.int16), rows.view(torch.int16)) and m.size() == U_KEYS
    assert int((out >= 0).sum().item()) == U_LOOKUPS // 2
    hit = out >= 0
    assert torch.equal(keys[out[hit].long()], req[hit]) and bool((req[~hit] >= (1 << 40)).all())
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    t_ins = t_q = 0.0
    torch.cuda.synchronize()
    for _ in range(steps):
        m = capi.CUCOStaticHashmap.empty(2 * U_KEYS, torch.int64, torch.int32, dev)
        ev[0].record(stream)
        capi.cache_insert_set(gpu, keys, slots, rows, m)
        ev[1].record(stream)
        out = m.query(req)
        ev[2].record(stream)
        torch.cuda.synchronize()
        t_ins += ev[0].elapsed_time(ev[1])
        t_q += ev[1].elapsed_time(ev[2])
    t_ins /= steps
    t_q /= steps
    # end to end: keys and lookups start in pinned host memory, the found slots go back to it
    # (the rows to insert are produced on the GPU, as the outputs of a training step are)
    keys_buf, req_buf = torch.empty_like(keys), torch.empty_like(req)
    out_host = torch.empty(U_LOOKUPS, dtype=torch.int32).pin_memory()
    e2e_n = max(3, min(steps, 5))
    torch.cuda.synchronize()
    ev[0].record(stream)
    for _ in range(e2e_n):
        keys_buf.copy_(keys_host, non_blocking=True)
        req_buf.copy_(req_host, non_blocking=True)
        mm = capi.CUCOStaticHashmap.empty(2 * U_KEYS, torch.int64, torch.int32, dev)
        capi.cache_insert_set(gpu, keys_buf, slots, rows, mm)
        out_host.copy_(mm.query(req_buf), non_blocking=True)
        stream.synchronize()
    ev[1].record(stream)
    torch.cuda.synchronize()
    e2e_ms = ev[0].elapsed_time(ev[1]) / e2e_n
    del mm, keys_buf, req_buf
    # the reference-named overwrite of the same rows through the finished map (all hits)
    for _ in range(2):
        capi.cache_set(None, gpu, keys, rows, m)
    t_set = time_launches(lambda: capi.cache_set(None, gpu, keys, rows, m), 10, stream)
    b_set = U_KEYS * (8 + 12 + 2 * row_bytes)
    obj["cache_set"] = {"ms": round(t_set, 4), "keys_per_s": round(U_KEYS / (t_set * 1e-3), 1),
                        "roofline": {"bound": "hbm", "kernel": "row_scatter_bulk_kernel<2>",
                                     "achieved": round(b_set / (t_set * 1e6), 1), "peak": peak,
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
    obj["map_build_query"] = {"build_ms": round(b_ms, 4), "query_ms": round(q_ms, 4)}
    try:
        from oracle import build_ref
        ref = build_ref.load_reference()
    except Exception:  # noqa: BLE001
        ref = None
    if ref is not None:
        build_query(ref)
        rb_ms, rq_ms, r_ref = build_query(ref)
        assert torch.equal(r_ours, r_ref), "map query differs from the reference's"
        # the reference's cache_set kernel on the same rows (bf16 viewed as int16: it rejects bf16)
        rm = ref.CUCOStaticHashmap(keys, slots, 0.5)
        g16, r16 = gpu.view(torch.int16), rows.view(torch.int16)
        for _ in range(2):
            ref.cache_set(g16, g16, keys, r16, rm)
        r_set = time_launches(lambda: ref.cache_set(g16, g16, keys, r16, rm), 5, stream)
        obj["reference_cuda"] = {"build_ms": round(rb_ms, 4), "query_ms": round(rq_ms, 4),
                                 "cache_set_ms": round(r_set, 4),
                                 "build_plus_set_plus_query_ms": round(rb_ms + r_set + rq_ms, 4),
                                 "what": "the reference's map wrapper (over a stand-in for cuCollections) and its "
                                         "MultiDimCacheSetKernel, compiled unmodified: build, overwrite all rows, query"}
        del rm
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
    obj["cache_turnover"] = {"ids": n_turn, "erase_ms": round(t_er, 4), "admit_ms": round(t_ad, 4),
                             "what": "shmt_map_erase of 10 % of the keys, then shmt_map_insert of as many new ids "
                                     "with the freed row numbers (host-synchronous calls, device time)"}
    # what bounds the lookups is the rate of random 64-byte window reads from a 256 MB table
    sink = torch.zeros(1, dtype=torch.int64, device=dev)
    tbl = torch.empty(m.memory_usage(), dtype=torch.uint8, device=dev)
    # measured twice: with as many reads per launch as the lookups have keys (a launch this short is
    # partly ramp and tail, for the probe as for the lookups), and with 16 times as many
    def window_rate(n_probe: int) -> float:
        probe = lambda c=[0]: (check(shm_lib.shmt_random_read(tbl.data_ptr(), tbl.numel(), n_probe, 64, c[0],
                                                              sink.data_ptr(), stream.cuda_stream)),
                               c.__setitem__(0, c[0] + 1))
        probe()
        return n_probe / (min(time_launches(probe, 1, stream) for _ in range(5)) * 1e-3)
    win_rate, win_rate_long = window_rate(U_LOOKUPS), window_rate(16 * U_LOOKUPS)
    del tbl
    # algorithmic bytes: insert+set per key 8 (key) + 4 (slot) + 16 (claim) + row read + row written;
    # lookup per key 8 + 12 + 4
    b_ins = U_KEYS * (8 + 4 + 16 + 2 * row_bytes)
    b_q = U_LOOKUPS * (8 + 12 + 4)
    obj.update({"value": round((U_KEYS + U_LOOKUPS) / ((t_ins + t_q) * 1e-3), 1), "ms_per_step": round(t_ins + t_q, 4),
                "roofline": {"bound": "hbm", "kernel": "insert_set_kernel<16,8> (probe-or-claim + row write)",
                             "kernel_ms": round(t_ins, 5), "algorithmic_bytes": b_ins,
                             "achieved": round(b_ins / (t_ins * 1e6), 1), "peak": peak, "unit": "GB/s",
                             "frac": round(b_ins / (t_ins * 1e6) / peak, 4), "peak_source": peak_src,
                             "traffic": 4_500_000_000,
                             "traffic_source": "profiles/insert_set_and_map_query.md (ncu, bytes per launch)"},
                "insert_set": {"ms": round(t_ins, 4), "keys_per_s": round(U_KEYS / (t_ins * 1e-3), 1)},
                "lookup": {"ms": round(t_q, 4), "keys_per_s": round(U_LOOKUPS / (t_q * 1e-3), 1),
                           "roofline": {"bound": "hbm, rate of random 64-byte window reads", "kernel": "map_query_kernel",
                                        "achieved": round(U_LOOKUPS / (t_q * 1e-3) / 1e9, 3),
                                        "peak": round(win_rate / 1e9, 3), "unit": "G reads/s",
                                        "frac": round(U_LOOKUPS / (t_q * 1e-3) / win_rate, 4),
                                        "peak_source": "shmt_random_read: as many independent 64-byte reads in one launch "
                                                       "as the lookups have keys, over a buffer of the table's size, "
                                                       "measured in this run",
                                        "peak_of_a_16x_longer_launch": round(win_rate_long / 1e9, 3),
                                        "hbm_bytes_frac": round(b_q / (t_q * 1e6) / peak, 4)}},
                "e2e": {"value": round((U_KEYS + U_LOOKUPS) / (e2e_ms * 1e-3), 1), "unit": "keys/s",
                        "h2d_bytes_per_step": (U_KEYS + U_LOOKUPS) * 8, "d2h_bytes_per_step": U_LOOKUPS * 4,
                        "ms_per_step": round(e2e_ms, 4), "steps": e2e_n},
                "gpu_launches": steps * 2})
    del m, gpu, rows, keys, req
    torch.cuda.empty_cache()
    obj["cpu_baseline"] = update_cpu(2, 1, keys_n, req_n, sample=4)
    return obj


def run_update(args) -> None:
    rank, local_rank, world = dist_env()
    if rank != 0:
        return
    line = {"metric": "inserted+looked-up keys/s", "unit": "keys/s", "n_gpus": 1, "steps": args.steps,
            "warmup": max(args.warmup, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int64 keys, int32 slots, bf16 rows (byte copy)", "data": "synthetic (seeded)",
            "config": {"workload": UPDATE_WORKLOAD, "keys": U_KEYS, "row_bytes": U_DIM * 2, "lookups": U_LOOKUPS}}
    if args.impl == "reference":
        keys_n, req_n = update_keys()
        cpu = update_cpu(args.steps, args.warmup, keys_n, req_n)
        line.update({"impl": "reference", "value": cpu["value"], "ms_per_step": cpu["ms_per_step"], "cpu_baseline": cpu,
                     "e2e": {"value": cpu["value"], "unit": "keys/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
        emit(line)
        return
    assert torch.cuda.is_available(), "bench.py needs a GPU (there is no CPU path)"
    torch.cuda.set_device(local_rank)
    line.update(update_object(args.steps, local_rank))
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
    # the scan on the reference's hot path is CUB's (src/cache_graph_sampling.cu:30-45); torch.cumsum is
    # CUB's DeviceScan as well: same bytes read and written (out of place, into a second buffer)
    cub32 = statistics.median(time_launches(lambda: torch.cumsum(src32, 0, dtype=torch.int32, out=work32), 1, stream)
                              for _ in range(steps))
    cub64 = statistics.median(time_launches(lambda: torch.cumsum(src64, 0, out=work64), 1, stream) for _ in range(steps))
    for _ in range(3):
        capi.tensor_relabel([ids])
    t_rel = statistics.median(time_launches(lambda: capi.tensor_relabel([ids]), 1, stream) for _ in range(steps))
    # the same ids numbered densely (0 .. SR_DISTINCT-1, as the nodes of a graph are): they all fit the
    # table, so each id is its own slot and the table's touched part stays in L2
    ids_dense = ids // 2_000_003
    ud, (rd,) = capi.tensor_relabel([ids_dense])
    assert torch.equal(ud[rd], ids_dense) and torch.equal(rd, rel) and torch.equal(ud * 2_000_003, uniq)
    del ud, rd
    t_rel_dense = statistics.median(time_launches(lambda: capi.tensor_relabel([ids_dense]), 1, stream)
                                    for _ in range(steps))
    del ids_dense
    b32, b64 = SR_SCAN_N * 8, SR_SCAN_N // 2 * 16
    # relabel: ids read by insert and compact (8 each), slot written + read + new id written (8 each x 3),
    # unique ids written; the table (12 bytes per slot at load <= 0.5) is written, read and cleaned
    cap = 1
    while cap < 2 * SR_IDS:
        cap <<= 1
    b_rel = SR_IDS * (8 + 8 + 8 * 3) + uniq.numel() * 8
    # what bounds relabel is the rate of random 16-byte slot accesses in a table beyond L2: per id one to
    # claim the slot / lower its first index and one to read the new id; per distinct id (at least) one to
    # confirm the first occurrence and write the new id, and one to empty the slot
    n_acc = 2 * SR_IDS + 2 * uniq.numel()
    from shmtensor_b200._lib import check, lib as shm_lib
    sink = torch.zeros(1, dtype=torch.int64, device=dev)
    tbl = torch.empty(cap * 16, dtype=torch.uint8, device=dev)
    n_probe = 1 << 26
    probe = lambda c=[0]: (check(shm_lib.shmt_random_read(tbl.data_ptr(), tbl.numel(), n_probe, 16, c[0], sink.data_ptr(),
                                                          stream.cuda_stream)), c.__setitem__(0, c[0] + 1))
    probe()
    slot_rate = n_probe / (min(time_launches(probe, 1, stream) for _ in range(5)) * 1e-3)
    del tbl
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
                    "dense_ids": {"ms": round(t_rel_dense, 4), "ids_per_s": round(SR_IDS / (t_rel_dense * 1e-3), 1),
                                  "what": "the same ids numbered 0 .. distinct-1 (ids as slots); the configured "
                                          "workload spreads its ids over 2^43 and is hashed"},
                    "roofline": {"bound": "hbm, rate of random 16-byte slot accesses (2 per id + 2 per distinct id)",
                                 "kernel": "relabel_insert / relabel_compact / relabel_remap",
                                 "slot_accesses": n_acc,
                                 "achieved": round(n_acc / (t_rel * 1e-3) / 1e9, 3), "peak": round(slot_rate / 1e9, 3),
                                 "unit": "G accesses/s", "frac": round(n_acc / (t_rel * 1e-3) / slot_rate, 4),
                                 "peak_source": "shmt_random_read, 16-byte reads over a buffer of the table's size "
                                                "(1 GiB), measured in this run",
                                 "streamed_bytes_frac_of_hbm": round(b_rel / (t_rel * 1e6) / peak, 4)}},
        "cub_scan": {"int32_ms": round(cub32, 4), "int64_ms": round(cub64, 4),
                     "int32_gbs": round(b32 / (cub32 * 1e6), 1), "int64_gbs": round(b64 / (cub64 * 1e6), 1),
                     "what": "torch.cumsum (cub::DeviceScan::InclusiveSum, out of place) on the same inputs: the "
                             "library scan the reference's hot path calls"},
        "roofline": {"bound": "hbm", "kernel": "scan_cluster_kernel<int> (persistent clusters, decoupled look-back, one pass)",
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
