"""A cached sub-graph whose rows can be evicted and admitted in place.

The reference builds its adjacency cache once (``create_subcsr``, src/cache_graph_sampling.cu:455-492,
called from python/shmtensor/sampling.py:149-189) and rebuilds it from scratch to change the cached
set.  Here the cached rows live in an arena with size-class free lists, so a turnover copies only
the admitted rows.

The layout is one the existing sampling kernels read unchanged.  They take a cached row's
bounds from ``gpu_indptr[v]`` and ``gpu_indptr[v + 1]``, where ``v`` is the value the hashmap
holds for the node.  A compact CSR stores ``v = slot``; this cache stores ``v = 2 * slot`` and
keeps ``(begin, end)`` of every slot side by side in ``bounds`` (passed as ``gpu_indptr``), so rows
need not be adjacent in ``gpu_indices`` and a slot can be pointed at another block at any time.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from . import capi
from ._lib import check, lib

_MIN_BLOCK = 8  # elements; blocks are powers of two from here up


def _block_class(deg: torch.Tensor) -> torch.Tensor:
    """Size class of a row of ``deg`` neighbours: the exponent of the smallest power-of-two block
    (at least 8 elements) that holds it.  Rows without neighbours take no block (class -1)."""
    d = torch.clamp(deg, min=1).to(torch.float64)
    c = torch.ceil(torch.log2(d)).to(torch.int64)
    c = torch.where((1 << c) < deg, c + 1, c)             # guard the float rounding of log2
    c = torch.clamp(c, min=_MIN_BLOCK.bit_length() - 1)
    return torch.where(deg > 0, c, torch.full_like(c, -1))


class GraphCache:
    """Adjacency lists of a set of nodes on the GPU, with in-place turnover.

    ``gpu_indptr`` / ``gpu_indices`` / ``hashmap`` plug into ``capi.csr_cache_sampling`` and
    ``capi.sample_minibatch`` like the outputs of ``create_subcsr`` and a
    ``CUCOStaticHashmap(nodes, arange)`` do.  ``arena_elements`` bounds the neighbour storage
    (power-of-two blocks: at most twice the cached edges are ever needed); ``replace`` raises
    when the admitted rows do not fit.
    """

    def __init__(self, indptr: torch.Tensor, indices: torch.Tensor, nodes: torch.Tensor,
                 arena_elements: int | None = None, load_factor: float = 0.5):
        capi._check_cuda(nodes, "nodes")
        self.indptr, self.indices = indptr, indices
        self.device = nodes.device
        nodes = nodes.contiguous()
        m = nodes.numel()
        begin = capi.subcsr_edge_base(indptr, nodes).to(torch.int64)
        end = capi.subcsr_edge_base(indptr, nodes + 1).to(torch.int64)
        deg = end - begin
        cls = _block_class(deg)
        sizes = torch.where(cls >= 0, 1 << torch.clamp(cls, min=0), torch.zeros_like(cls))
        offs = torch.cumsum(sizes, 0) - sizes
        used = int(sizes.sum().item())
        cap = int(arena_elements) if arena_elements is not None else max(used + used // 4, 1024)
        if used > cap:
            raise RuntimeError(f"GraphCache: {used} arena elements needed, {cap} given")
        self.arena = torch.empty(cap, dtype=indices.dtype, device=self.device)
        self._top = used                                   # bump pointer behind the last block
        self._free: Dict[int, List[torch.Tensor]] = {}     # class -> stacks of free block offsets
        self.bounds = torch.zeros(2 * m + 2, dtype=indptr.dtype, device=self.device)
        self.bounds[0:2 * m:2] = offs.to(indptr.dtype)
        self.bounds[1:2 * m:2] = (offs + deg).to(indptr.dtype)
        self._slot_class = cls                             # class of the block each slot holds
        self._fill(nodes, offs)
        values = (torch.arange(m, device=self.device, dtype=torch.int64) * 2)
        self.hashmap = capi.CUCOStaticHashmap(nodes.to(torch.int64), values, load_factor)

    # what the sampling entry points take
    gpu_indptr = property(lambda self: self.bounds)
    gpu_indices = property(lambda self: self.arena)

    def _fill(self, nodes: torch.Tensor, offs: torch.Tensor) -> None:
        """Copy the adjacency lists of ``nodes`` from the (host) CSR to ``arena[offs[i]:]``."""
        if nodes.numel() == 0:
            return
        offs = offs.to(self.indptr.dtype).contiguous()
        nodes = nodes.contiguous()
        check(lib.shmt_subcsr_fill(capi._ptr(self.indptr), capi._int_code(self.indptr, "GraphCache"),
                                   capi._ptr(self.indices), capi._int_code(self.indices, "GraphCache"),
                                   capi._ptr(nodes), capi._int_code(nodes, "GraphCache"), nodes.numel(),
                                   capi._ptr(offs), capi._ptr(self.arena), capi._stream(self.device)))

    def _take_blocks(self, cls: torch.Tensor) -> torch.Tensor:
        """One block per entry of ``cls`` (class -1: none): from the class's free list, else from
        the untouched end of the arena."""
        out = torch.zeros_like(cls)
        for c in torch.unique(cls).tolist():
            if c < 0:
                continue
            want = (cls == c).nonzero(as_tuple=True)[0]
            got: List[torch.Tensor] = []
            need = want.numel()
            stack = self._free.get(c, [])
            while need and stack:
                t = stack.pop()
                if t.numel() > need:
                    stack.append(t[need:])
                    t = t[:need]
                got.append(t)
                need -= t.numel()
            if need:
                size = 1 << c
                if self._top + need * size > self.arena.numel():
                    for t in got:                          # leave the free list as it was
                        stack.append(t)
                    raise RuntimeError("GraphCache.replace: the arena is full "
                                       f"({self._top} of {self.arena.numel()} elements used)")
                got.append(self._top + size * torch.arange(need, device=self.device, dtype=torch.int64))
                self._top += need * size
            self._free[c] = stack
            out[want] = torch.cat(got)
        return out

    def replace(self, evict_nodes: torch.Tensor, admit_nodes: torch.Tensor) -> int:
        """``evict_nodes`` leave the cache, ``admit_nodes`` (distinct, not cached) take their
        slots; only the admitted rows are copied.  Admits at most as many nodes as were evicted,
        in order; returns how many.  Must not overlap a sampling call that uses this cache."""
        dev = self.device
        evict = torch.unique(evict_nodes.to(dev, torch.int64), sorted=True)
        freed = self.hashmap.erase(evict)
        freed = freed[freed >= 0]
        slots = freed >> 1
        # the evicted rows' blocks go back to their classes
        cls_old = self._slot_class[slots]
        old_begin = self.bounds[2 * slots].to(torch.int64)
        for c in torch.unique(cls_old).tolist():
            if c >= 0:
                self._free.setdefault(c, []).append(old_begin[cls_old == c])
        self._slot_class[slots] = -1
        self.bounds[2 * slots + 1] = self.bounds[2 * slots]                # empty until reused
        n = min(int(slots.numel()), int(admit_nodes.numel()))
        if n == 0:
            return 0
        admit = admit_nodes.to(dev)[:n].contiguous()
        slots = slots[:n]
        begin = capi.subcsr_edge_base(self.indptr, admit).to(torch.int64)
        end = capi.subcsr_edge_base(self.indptr, admit + 1).to(torch.int64)
        deg = end - begin
        cls = _block_class(deg)
        offs = self._take_blocks(cls)
        self._fill(admit, offs)
        self._slot_class[slots] = cls
        self.bounds[2 * slots] = offs.to(self.bounds.dtype)
        self.bounds[2 * slots + 1] = (offs + deg).to(self.bounds.dtype)
        self.hashmap.insert(admit.to(torch.int64), slots * 2)
        return n

    def rows(self) -> int:
        return self.hashmap.size()

    def arena_used(self) -> int:
        """Arena elements handed out so far (free blocks inside that range are reused first)."""
        return self._top
