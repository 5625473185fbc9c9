"""``GPUSamplingDataloader`` — mini-batch neighbour sampling driven from Python.

Keeps the constructor, iteration protocol and helper methods of the reference's
python/shmtensor/sampling.py:30-237 (hops run over ``reversed(num_picks)``, the frontier of
the next hop is the relabelled unique set, ``create_cache`` keeps the hottest rows' adjacency
on the GPU behind a hashmap).  The DGL block the reference builds per hop is optional here:
pass ``block_fn`` (or have ``dgl`` installed and pass ``block_fn="dgl"``); without it each hop
yields the tuple ``(sub_indptr, relabel_indices, num_src, num_dst)``.
"""
from __future__ import annotations

import contextlib
import weakref
from typing import Callable, Optional

import torch
import torch.distributed as dist

from . import capi


def _dgl_block(sub_indptr, relabel_indices, num_src, num_dst, edge_ids=None):
    """CSC block as python/shmtensor/sampling.py:9-20 builds it (needs dgl).  The reference hands
    an empty edge-id tensor over; with ``with_edge_ids`` the block carries the real ones."""
    import dgl  # noqa: deferred so that the package works without dgl
    from dgl.heterograph import DGLBlock
    hgidx = dgl.heterograph_index.create_unitgraph_from_csr(
        2, num_src, num_dst, sub_indptr, relabel_indices,
        torch.Tensor() if edge_ids is None else edge_ids, formats=['coo', 'csr', 'csc'], transpose=True)
    return DGLBlock(hgidx, (['_N'], ['_N']), ['_E'])


def _plain_block(sub_indptr, relabel_indices, num_src, num_dst, edge_ids=None):
    if edge_ids is None:
        return sub_indptr, relabel_indices, num_src, num_dst
    return sub_indptr, relabel_indices, num_src, num_dst, edge_ids


class GPUSamplingDataloader:

    def __init__(self, indptr, indices, seeds, batchsize, num_picks, replace=False,
                 use_ddp=False, shuffle=True, drop_last=False,
                 block_fn: Optional[Callable] = None, fused: bool = True, with_edge_ids: bool = False,
                 own_stream: bool = False, edge_weights: Optional[torch.Tensor] = None):
        self.indptr, self.indices = indptr, indices
        self.batchsize, self.num_picks, self.replace = batchsize, num_picks, replace
        self.use_ddp, self.shuffle, self.drop_last = use_ddp, shuffle, drop_last
        self.block_fn = _dgl_block if block_fn == "dgl" else (block_fn or _plain_block)

        # fused: one native call per mini-batch; False keeps the reference's call-per-hop loop
        self.fused = fused
        # with_edge_ids (not in the reference): every block also gets the edge ids of its sampled
        # neighbours (positions in `indices`), passed to block_fn as a fifth argument
        self.with_edge_ids = with_edge_ids
        self.has_cache = False
        self.gpu_indptr = self.gpu_indices = self.hashmap = self.gpu_edge_base = None
        # edge_weights (not in the reference): float32, one per edge, parallel to `indices`; every hop
        # then picks neighbours in proportion to them (without replacement: fan-outs of at most 32)
        self.edge_weights = self.gpu_weights = None
        if edge_weights is not None:
            if edge_weights.dtype != torch.float32 or edge_weights.numel() != indices.numel():
                raise RuntimeError("GPUSamplingDataloader: edge_weights must be float32, one per edge")
            if with_edge_ids and fused:
                raise RuntimeError("GPUSamplingDataloader: edge ids with edge_weights need fused=False")
            self.edge_weights = edge_weights.contiguous()
            if not self.edge_weights.is_cuda:
                capi.pin_memory(self.edge_weights)
                weakref.finalize(self, capi.unpin_memory, self.edge_weights)
        # own_stream (not in the reference): sample on a stream of the loader's own.  The caller's
        # stream waits for each batch it is handed, but the sampling of a batch does not wait for
        # what the caller queued for the batch before it, so a consumer that queues its work and
        # comes back for the next batch (a feature fetch, a training step) has that work run on the
        # GPU beside the sampling of the next batch.
        self._side = None
        self._own_stream = own_stream
        self._raw = []

        # host-resident CSR arrays are registered so kernels can read them in place
        for t in (self.indptr, self.indices):
            if not t.is_cuda:
                capi.pin_memory(t)
                weakref.finalize(self, capi.unpin_memory, t)

        self.seeds = self._local_share(seeds)
        if self.shuffle:
            self._reshuffle()
        self.seeds = self.seeds.cuda()
        self._set_len()
        self.curr = 0
        if own_stream:
            self._side = torch.cuda.Stream(device=self.seeds.device)
        if self.fused and len(self.num_picks) <= 8:
            # scratch for the largest mini-batch this loader can issue, before the first one (the
            # scratch belongs to the stream the sampling runs on)
            with torch.cuda.stream(self._side) if self._side is not None else contextlib.nullcontext():
                capi.reserve_minibatch(max(1, min(self.batchsize, max(1, self.seeds.numel()))),
                                       list(reversed(self.num_picks)), self.seeds.device)

    # ------------------------------------------------------------------ seed bookkeeping
    def _local_share(self, seeds):
        """This rank's contiguous slice of the seeds (python/shmtensor/sampling.py:65-71)."""
        if not self.use_ddp:
            return seeds
        world, rank = dist.get_world_size(), dist.get_rank()
        part = (seeds.numel() + world - 1) // world
        return seeds[rank * part:(rank + 1) * part]

    def _reshuffle(self):
        self.seeds = self.seeds[torch.randperm(self.seeds.numel(), device=self.seeds.device)]

    def _set_len(self):
        n = self.seeds.numel()
        self.len = n // self.batchsize if self.drop_last else -(-n // self.batchsize)

    def __len__(self):
        return self.len

    def __iter__(self):
        if self.shuffle:
            self._reshuffle()
        self.curr = 0
        if self._side is not None:
            # the loader's stream sees the seeds, caches and arrays as the caller's stream left them
            self._side.wait_stream(torch.cuda.current_stream(self.seeds.device))
        return self

    def update_params(self, **kwargs):
        for k, v in kwargs.items():
            setattr(self, k, v)
        if "seeds" in kwargs or "use_ddp" in kwargs:
            self.seeds = self._local_share(self.seeds).cuda()
            self._set_len()

    # ------------------------------------------------------------------ one hop / one batch
    def _hop(self, seeds, num_pick):
        if self.has_cache:
            return capi.csr_cache_sampling(self.indptr, self.indices, self.gpu_indptr,
                                           self.gpu_indices, self.hashmap, seeds, num_pick,
                                           self.replace)
        return capi.csr_sampling(self.indptr, self.indices, seeds, num_pick, self.replace)

    def __next__(self):
        if self.curr >= self.len:
            raise StopIteration
        self._raw = []
        if self._side is None:
            batch = self._next_batch()
            self._raw = []
            return batch
        caller = torch.cuda.current_stream(self.seeds.device)
        with torch.cuda.stream(self._side):
            batch = self._next_batch()
            done = torch.cuda.Event()
            done.record(self._side)
        caller.wait_event(done)
        for t in self._raw:  # allocated on the loader's stream, used from here on by the caller's
            t.record_stream(caller)
        self._raw = []
        return batch

    def _next_batch(self):
        lo = self.curr * self.batchsize
        seeds = self.seeds[lo:lo + self.batchsize]
        self.curr += 1

        output_nodes, blocks = seeds, []
        if self.fused:
            # all hops in one native call: no host round trip between hops
            _, hops = capi.sample_minibatch(self.indptr, self.indices, seeds,
                                            list(reversed(self.num_picks)), self.replace,
                                            self.gpu_indptr if self.has_cache else None,
                                            self.gpu_indices if self.has_cache else None,
                                            self.hashmap if self.has_cache else None,
                                            self.gpu_edge_base if self.has_cache else None,
                                            return_eids=self.with_edge_ids, weights=self.edge_weights,
                                            gpu_weights=self.gpu_weights if self.has_cache else None)
            n_dst = seeds.numel()
            for hop in hops:
                sub_indptr, relabel_indices, frontier = hop[0], hop[2], hop[3]
                extra = (hop[4],) if self.with_edge_ids else ()
                self._raw += [sub_indptr, relabel_indices, frontier, *extra]
                blocks.insert(0, self.block_fn(sub_indptr, relabel_indices, frontier.numel(), n_dst, *extra))
                n_dst = frontier.numel()
            input_nodes = hops[-1][3].to(seeds.dtype)
            self._raw.append(input_nodes)
            return input_nodes, output_nodes, blocks
        for num_pick in reversed(self.num_picks):
            if self.edge_weights is not None:
                cached = dict(gpu_indptr=self.gpu_indptr, gpu_indices=self.gpu_indices, gpu_weights=self.gpu_weights,
                              gpu_edge_base=self.gpu_edge_base, hashmap=self.hashmap) if self.has_cache else {}
                got = capi.csr_weighted_sampling(self.indptr, self.indices, self.edge_weights, seeds, num_pick,
                                                 self.replace, return_eids=self.with_edge_ids, **cached)
                sub_indptr, sub_indices, extra = got[0], got[1], tuple(got[2:])
            elif self.with_edge_ids:
                cached = dict(gpu_indptr=self.gpu_indptr, gpu_indices=self.gpu_indices,
                              gpu_edge_base=self.gpu_edge_base, hashmap=self.hashmap) if self.has_cache else {}
                sub_indptr, sub_indices, eids = capi.csr_sampling_with_eids(self.indptr, self.indices, seeds,
                                                                           num_pick, self.replace, **cached)
                extra = (eids,)
            else:
                sub_indptr, sub_indices = self._hop(seeds, num_pick)
                extra = ()
            frontier, (_, relabel_indices) = capi.tensor_relabel([seeds, sub_indices])
            self._raw += [sub_indptr, relabel_indices, frontier, *extra]
            blocks.insert(0, self.block_fn(sub_indptr, relabel_indices, frontier.numel(),
                                           seeds.numel(), *extra))
            seeds = frontier
        return seeds, output_nodes, blocks

    # ------------------------------------------------------------------ cache management
    def create_cache(self, cache_capacity, hotness, replaceable=False):
        """Keep the hottest rows' adjacency on the GPU within ``cache_capacity`` bytes
        (python/shmtensor/sampling.py:149-189; same size model: adjacency bytes + one indptr
        entry + 1.25*2*4 bytes of map per row, map load factor 0.8, int32 keys/values).
        ``replaceable=True`` (not in the reference) builds a ``GraphCache`` instead of a compact
        sub-CSR, so that ``replace_cache`` can later swap rows without a rebuild."""
        if cache_capacity <= 0:
            return
        full_size = self.indptr.nbytes + self.indices.nbytes
        if full_size <= cache_capacity:  # everything fits: plain GPU CSR, no map
            self.has_cache = False
            self.indices, self.indptr = self.indices.cuda(), self.indptr.cuda()
            if self.edge_weights is not None:
                self.edge_weights = self.edge_weights.cuda()
            return

        degrees = (self.indptr[1:] - self.indptr[:-1]).cpu()
        # The row offsets are small next to the adjacency lists (8 bytes per node): when they
        # fit in a quarter of the budget they all go to the GPU first.  A row whose adjacency
        # stays on the host then costs one trip over the host link instead of two, and such
        # trips, not bytes, are what bound the sampler on cold rows.
        if not self.indptr.is_cuda and self.indptr.nbytes <= cache_capacity // 4:
            cache_capacity -= self.indptr.nbytes
            self.indptr = self.indptr.cuda()
        candidates = torch.sort(hotness, descending=True).indices
        cost = degrees[candidates.cpu()] * self.indices.element_size() \
            + self.indptr.element_size() + 1.25 * 2 * 4
        n_rows = int(torch.searchsorted(torch.cumsum(cost, dim=0), cache_capacity).item())
        candidates = candidates[:n_rows].cuda()
        if candidates.numel() == 0:
            return
        if self.with_edge_ids and replaceable:
            raise RuntimeError("create_cache: edge ids are kept for a compact cache only (replaceable=False)")
        if self.edge_weights is not None and replaceable:
            raise RuntimeError("create_cache: edge weights are kept for a compact cache only (replaceable=False)")
        if self.with_edge_ids:
            self.gpu_edge_base = capi.subcsr_edge_base(self.indptr, candidates)
        if replaceable:
            from .graph_cache import GraphCache
            self.graph_cache = GraphCache(self.indptr, self.indices, candidates)
            self.gpu_indptr, self.gpu_indices = self.graph_cache.gpu_indptr, self.graph_cache.gpu_indices
            self.hashmap = self.graph_cache.hashmap
            self.has_cache = True
            return
        self.gpu_indptr, self.gpu_indices = capi.create_subcsr(self.indptr, self.indices,
                                                               candidates)
        if self.edge_weights is not None:  # the cached rows' weights, laid out like their neighbours
            self.gpu_weights = capi.create_subcsr(self.indptr, self.edge_weights.view(torch.int32),
                                                  candidates)[1].view(torch.float32)
        slots = torch.arange(candidates.numel(), device='cuda', dtype=torch.int32)
        self.hashmap = capi.CUCOStaticHashmap(candidates.int(), slots, 0.8)
        self.has_cache = True

    def replace_cache(self, evict_nodes, admit_nodes):
        """Swap cached rows in place (needs ``create_cache(..., replaceable=True)``): the rows of
        ``evict_nodes`` leave the GPU, those of ``admit_nodes`` are copied into the freed space.
        Returns how many nodes were admitted.  Call between mini-batches."""
        gc = getattr(self, "graph_cache", None)
        if gc is None or not self.has_cache:
            raise RuntimeError("replace_cache: the cache was not created with replaceable=True")
        if self._side is not None:
            # batches already sampled on the loader's stream finish before the cache changes, and
            # the next one sees the change
            cur = torch.cuda.current_stream(self.seeds.device)
            cur.wait_stream(self._side)
        n = gc.replace(evict_nodes, admit_nodes)
        self.gpu_indptr, self.gpu_indices = gc.gpu_indptr, gc.gpu_indices
        if self._side is not None:
            self._side.wait_stream(cur)
        return n

    def clear_cache(self):
        self.has_cache = False
        self.gpu_indptr = self.gpu_indices = self.hashmap = self.gpu_edge_base = self.gpu_weights = None
        self.graph_cache = None

    def presampling(self):
        """One uncached epoch that counts how often each node is a seed (sampling hotness)
        and how often it appears in a frontier (feature hotness)
        (python/shmtensor/sampling.py:199-227)."""
        n_nodes = self.indptr.numel() - 1
        sampling_hotness = torch.zeros(n_nodes, device='cuda')
        feature_hotness = torch.zeros(n_nodes, device='cuda')
        one = torch.ones((), device='cuda')
        for b in range(self.len):
            seeds = self.seeds[b * self.batchsize:(b + 1) * self.batchsize]
            for num_pick in reversed(self.num_picks):
                sampling_hotness.index_add_(0, seeds.long(), one.expand(seeds.numel()))
                _, sub_indices = capi.csr_sampling(self.indptr, self.indices, seeds, num_pick,
                                                   self.replace)
                seeds, _ = capi.tensor_relabel([seeds, sub_indices])
                feature_hotness.index_add_(0, seeds.long(), one.expand(seeds.numel()))
        if self.use_ddp:
            dist.all_reduce(sampling_hotness)
            dist.all_reduce(feature_hotness)
        return sampling_hotness.cpu(), feature_hotness.cpu()

    def compute_weight_size(self, hotness):
        """(bytes of the full CSR, mean hotness-weighted bytes per touched row)
        (python/shmtensor/sampling.py:229-237)."""
        full_size = self.indptr.nbytes + self.indices.nbytes
        degree = (self.indptr[1:] - self.indptr[:-1]).clip(max=self.num_picks[0] * 1.3).float().cpu()
        hot = hotness > 0
        item = (degree[hot] * self.indices.element_size() + self.indptr.element_size()) * hotness[hot]
        return full_size, item.mean().item()
