"""Feature cache hash-partitioned over the GPUs of one node.

The reference is single-GPU; this is the multi-GPU form of its cached fetch.  Each of the
``world`` ranks (one process per GPU) keeps the rows of the cached ids it owns in one device
buffer.  Every rank holds the whole directory — a static hashmap id -> (owner << 40 | slot)
— so a probe never leaves local HBM; only row payloads cross NVLink, read by the same
per-row bulk copies, inside the same fused gather kernel, that serve local hits and host misses
(``shmt_fetch_partitioned``).  Peer buffers are mapped with CUDA IPC, handles exchanged through
``torch.distributed``.  There is no collective on the data path.

The hottest ids are kept by every rank (``replicate``): under a skewed access pattern a handful
of rows takes a large share of all lookups, and N-1 GPUs reading the same few lines of one
owner serialise on them (measured at 4 GPUs with a Zipf batch at 95 % hits: 1.8 ms per batch
without the replicas, 0.39 ms with them).
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import torch
import torch.distributed as dist

from . import capi
from ._lib import check, lib

OWNER_SHIFT = 40


def owner_of(ids: torch.Tensor, world: int) -> torch.Tensor:
    """Owner rank of each id: a multiplicative hash, so that consecutive (or degree-sorted)
    ids spread evenly.  Pure tensor arithmetic: identical on every rank, CPU or GPU."""
    h = (ids.to(torch.int64) * 0x9E3779B1) & 0xFFFFFFFF
    return (h >> 8) % world


def plan_partition(cached_ids: torch.Tensor, world: int):
    """(owner, slot) of every cached id: ``slot`` counts the ids of the same owner that
    come earlier in ``cached_ids``; also the number of rows each rank holds."""
    owner = owner_of(cached_ids, world)
    slot = torch.empty_like(owner)
    counts = []
    for r in range(world):
        mine = owner == r
        n = int(mine.sum().item())
        slot[mine] = torch.arange(n, dtype=torch.int64, device=owner.device)
        counts.append(n)
    return owner, slot, counts


def default_replication(n_cached: int, world: int) -> int:
    """Rows every rank keeps for itself: an eighth of its share of the cache, at least 1024."""
    if world <= 1:
        return 0
    return min(n_cached, max(1024, n_cached // (8 * world)))


def head_for_mass(hotness: torch.Tensor, mass: float) -> int:
    """Length of the shortest prefix of ``hotness`` (lookup counts or weights of the cached ids,
    hottest first) that takes the share ``mass`` of their total.  Under a skewed access pattern
    this is tiny next to the cache: half of a Zipf(1.1) stream over 480,000 rows falls on a few
    dozen of them."""
    h = hotness.to(torch.float64).flatten().cpu()
    if h.numel() == 0 or mass <= 0:
        return 0
    c = torch.cumsum(h, 0)
    target = min(max(float(mass), 0.0), 1.0) * float(c[-1])
    return min(int(torch.searchsorted(c, torch.tensor(target, dtype=torch.float64)).item()) + 1, h.numel())


def plan_directory(cached_ids: torch.Tensor, world: int, rank: int, replicate: int = 0):
    """What rank ``rank`` stores and how it sees the directory.  The first ``replicate`` ids of
    ``cached_ids`` (the hottest: callers pass ids hottest first) are kept by every rank, behind
    the rows it owns; the others are partitioned by ``plan_partition``.  Returns ``(values,
    my_ids, counts, replicate)``: the directory value ``owner << 40 | slot`` of every cached id
    as this rank sees it (a replicated id points at this rank's own copy), the ids whose rows
    this rank holds in slot order, and the number of partitioned rows per rank."""
    n = cached_ids.numel()
    rep = min(int(replicate), n) if world > 1 else 0
    rest = cached_ids[rep:]
    owner, slot, counts = plan_partition(rest, world)
    values = torch.empty(n, dtype=torch.int64, device=cached_ids.device)
    values[rep:] = (owner << OWNER_SHIFT) | slot
    values[:rep] = (rank << OWNER_SHIFT) | (counts[rank] + torch.arange(rep, dtype=torch.int64,
                                                                         device=cached_ids.device))
    my_ids = torch.cat([rest[owner == rank], cached_ids[:rep]])
    return values, my_ids, counts, rep


class _DeviceBuffer:
    """A cudaMalloc'ed block owned by libshmt, exposed to torch without a copy."""

    def __init__(self, nbytes: int, ptr: Optional[int] = None):
        self.nbytes = nbytes
        self.owned = ptr is None
        if ptr is None:
            out = C.c_void_p()
            check(lib.shmt_dev_alloc(max(nbytes, 16), C.byref(out)))
            ptr = out.value
        self.ptr = ptr
        self.__cuda_array_interface__ = {"shape": (max(nbytes, 1),), "typestr": "|u1",
                                         "data": (ptr, False), "version": 2}

    def tensor(self, dtype: torch.dtype, shape) -> torch.Tensor:
        flat = torch.as_tensor(self, device="cuda")[: self.nbytes]
        return flat.view(dtype).reshape(shape)


def share_device_buffer(buf: "_DeviceBuffer", group=None):
    """Map every rank's buffer into every other rank (CUDA IPC).  The allocation behind ``buf``
    should be whole 2 MB pages (``shmt_dev_alloc`` sees to it): a peer maps any other size with
    small pages, and random row reads from a buffer of several GB then run 10-20x slower.
    Returns ``(ptrs, opened)``:
    ``ptrs[r]`` is rank r's buffer as seen from this process, ``opened`` the mappings to close
    with ``shmt_ipc_close_handle`` (on every rank, with nothing in flight, before any free)."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    handle = (C.c_char * 64)()
    check(lib.shmt_ipc_get_handle(buf.ptr, handle))
    handles: List[bytes] = [b""] * world
    dist.all_gather_object(handles, bytes(handle.raw), group=group)
    ptrs, opened = [0] * world, []
    ptrs[rank] = buf.ptr
    for r, h in enumerate(handles):
        if r == rank:
            continue
        out = C.c_void_p()
        check(lib.shmt_ipc_open_handle(h, C.byref(out)))
        ptrs[r] = out.value
        opened.append(out.value)
    dist.barrier(group)
    return ptrs, opened


class PartitionedFeatureCache:
    """``fetch(ids)`` returns ``host_table[ids]`` on this rank's GPU, bit-exact, reading each
    row from the local shard, a peer's shard over NVLink, or pinned host memory."""

    def __init__(self, host_table: torch.Tensor, cached_ids: torch.Tensor, group=None,
                 load_factor: float = 0.5, replicate: Optional[int] = None,
                 hotness: Optional[torch.Tensor] = None, replicate_mass: float = 0.5):
        """``cached_ids`` hottest first.  Every rank keeps the first ``replicate`` of them; when
        that is not given but ``hotness`` (one weight per cached id, same order) is, the head
        that takes ``replicate_mass`` of the lookups is kept everywhere, and never less than
        the default share."""
        self.group = group
        distributed = dist.is_available() and dist.is_initialized()
        self.world = dist.get_world_size(group) if distributed else 1
        self.rank = dist.get_rank(group) if distributed else 0
        self.host_table = host_table
        self.device = torch.device("cuda", torch.cuda.current_device())
        row_shape = tuple(host_table.shape[1:])
        self.row_bytes = capi._row_bytes(host_table)

        cached_ids = cached_ids.to(torch.int64)   # the plan is made where the ids are (CPU or GPU)
        if replicate is None:
            replicate = default_replication(cached_ids.numel(), self.world)
            if hotness is not None and self.world > 1:
                replicate = max(replicate, head_for_mass(hotness, replicate_mass))
        values, mine, counts, self.replicated = plan_directory(cached_ids, self.world, self.rank, replicate)
        n_mine = mine.numel()

        # this rank's shard (the rows it owns, then its copy of the replicated rows), filled
        # straight from the host table by the UVA gather kernel
        self._buf = _DeviceBuffer(n_mine * self.row_bytes)
        self.shard = self._buf.tensor(host_table.dtype, (n_mine, *row_shape))
        if mine.numel():
            capi.uva_fetch(host_table, mine.to(self.device), out=self.shard)
        torch.cuda.synchronize()

        # peers' shards through CUDA IPC
        self._peer_ptrs: List[int] = [self._buf.ptr]
        self._opened: List[int] = []
        if self.world > 1:
            self._peer_ptrs, self._opened = share_device_buffer(self._buf, group)
        self._bases = (C.c_void_p * self.world)(*self._peer_ptrs)

        # directory on every rank: id -> owner << 40 | slot
        self.directory = capi.CUCOStaticHashmap(cached_ids.to(self.device),
                                                values.to(self.device), load_factor)
        self.counts = counts

    def warm(self) -> None:
        """One streaming pass over every peer's shard from this GPU, so that the first timed fetch
        does not pay for setting up the translations of memory it has never touched."""
        if self.world <= 1:
            return
        sink = torch.zeros(1, dtype=torch.int64, device=self.device)
        sizes = [c + self.replicated for c in self.counts]
        for r, (ptr, rows) in enumerate(zip(self._peer_ptrs, sizes)):
            nbytes = rows * self.row_bytes // 16 * 16
            if r != self.rank and nbytes >= 16:
                check(lib.shmt_stream_read(ptr, nbytes, sink.data_ptr(), capi._stream(self.device)))
        torch.cuda.synchronize()

    def fetch(self, ids: torch.Tensor) -> torch.Tensor:
        capi._check_cuda(ids, "ids")
        ids = ids.contiguous()
        out = torch.empty((ids.numel(), *self.host_table.shape[1:]), dtype=self.host_table.dtype,
                          device=ids.device)
        check(lib.shmt_fetch_partitioned(self.directory._handle, self._bases, self.world,
                                         OWNER_SHIFT, capi._ptr(self.host_table), capi._ptr(ids),
                                         capi._int_code(ids, "fetch"), ids.numel(), self.row_bytes,
                                         capi._ptr(out), capi._stream(ids.device)))
        return out

    def replace(self, evict_ids: torch.Tensor, admit_ids: torch.Tensor) -> int:
        """Turn the cache over in place: ``evict_ids`` leave it, ``admit_ids`` (distinct, not
        cached) take their rows, wherever those are: the directory names the owner of every id,
        so an admitted id simply inherits the (owner, row) of an evicted one.  Every rank makes
        the same call (a collective when there are several ranks, with no fetch in flight);
        each updates its own directory and fills the freed rows it owns from the host table.
        Ids held on every rank (the replicated hottest rows) cannot be evicted.  Admits at most
        as many ids as rows were freed, in order; returns how many.  ``evict_ids`` may list an
        id twice (it is evicted once); ``admit_ids`` must be distinct."""
        dev = self.device
        # every rank must pair the same freed row with the same admitted id: a duplicate would let
        # whichever thread erases first report the row, in an order that differs between ranks
        evict = torch.unique(evict_ids.to(dev, torch.int64), sorted=True).contiguous()
        admit = admit_ids.to(dev, torch.int64).contiguous()
        low = (1 << OWNER_SHIFT) - 1
        if self.replicated:
            seen = self.directory.query(evict)
            mine = (seen >> OWNER_SHIFT) == self.rank
            if bool((mine & ((seen & low) >= self.counts[self.rank]) & (seen >= 0)).any()):
                raise RuntimeError("PartitionedFeatureCache.replace: a replicated id cannot be evicted")
        freed = self.directory.erase(evict)
        freed = freed[freed >= 0]
        n = min(int(freed.numel()), int(admit.numel()))
        if n:
            admit, freed = admit[:n].contiguous(), freed[:n].contiguous()
            self.directory.insert(admit, freed)
            here = (freed >> OWNER_SHIFT) == self.rank
            if bool(here.any()):
                rows = (freed[here] & low).contiguous()
                capi.uva_set(self.shard, rows, capi.uva_fetch(self.host_table, admit[here].contiguous()))
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier(self.group)  # no rank reads a freed row of a peer before its owner refilled it
        return n

    def fetch_alltoall(self, ids: torch.Tensor) -> torch.Tensor:
        """The same result by the batched route: ids are bucketed by owner, exchanged with an
        NCCL all-to-all, gathered on the owner, and the rows come back with a second
        all-to-all; misses are read locally from the host table.  A collective, so every rank
        must call it, with batches of any size.  Kept for comparison with ``fetch``: direct
        peer loads need no exchange of ids and no staging copies."""
        capi._check_cuda(ids, "ids")
        ids = ids.contiguous()
        n, world = ids.numel(), self.world
        out = torch.empty((n, *self.host_table.shape[1:]), dtype=self.host_table.dtype, device=ids.device)
        value = self.directory.query(ids)
        miss = (value < 0).nonzero(as_tuple=True)[0]
        if miss.numel():
            out[miss] = capi.uva_fetch(self.host_table, ids[miss])
        hit = (value >= 0).nonzero(as_tuple=True)[0]
        owner = value[hit] >> OWNER_SHIFT
        order = torch.argsort(owner, stable=True)
        send_slots = (value[hit] & ((1 << OWNER_SHIFT) - 1))[order]
        send_counts = torch.bincount(owner, minlength=world)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        sc, rc = send_counts.tolist(), recv_counts.tolist()
        recv_slots = torch.empty(sum(rc), dtype=send_slots.dtype, device=ids.device)
        dist.all_to_all_single(recv_slots, send_slots, rc, sc, group=self.group)
        rows_out = self.shard[recv_slots]
        rows_in = torch.empty((sum(sc), *self.host_table.shape[1:]), dtype=self.host_table.dtype,
                              device=ids.device)
        dist.all_to_all_single(rows_in, rows_out, sc, rc, group=self.group)
        out[hit[order]] = rows_in
        return out

    def close(self) -> None:
        """Unmap the peers' buffers and free this rank's shard.  Call on every rank, between
        steps, with no fetch in flight; the ranks meet at a barrier before any memory goes."""
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier(self.group)
        for p in self._opened:
            lib.shmt_ipc_close_handle(p)
        self._opened = []
        if self.world > 1:
            dist.barrier(self.group)
        if self._buf is not None and self._buf.owned:
            self.shard = None
            lib.shmt_dev_free(self._buf.ptr)
            self._buf = None
