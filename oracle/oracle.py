"""CPU oracle for the GPU-cache hot path.  TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline /
reference arm may import this module, and only as the checker or the timed CPU
baseline.  Nothing under ``shmtensor_b200/`` imports it.

Each function restates, in numpy, what one piece of gpzlx1/ShmTensor computes
and cites the reference source it follows (paths inside that project).

Parity pins (known-answer vectors taken from the reference's own test scripts,
stored under ``tests/golden/`` and checked by ``tests/test_oracle.py``):

* relabel ............ example/test_cache_sampling.py:129-140 (full golden vector)
* sampling offsets ... example/test_cache_sampling.py:23-64   (sub_indptr, exact rows)
* sub-CSR ............ example/test_cache_sampling.py:75-84   (gpu_indptr, gpu_indices)
* fetch / set ........ example/test_cache_fetch.py:24-105, example/test_cache_set.py:24-147
                       (equality with ``data[query]`` / set-then-fetch round trip)
* hashmap ............ query -> stored value or -1; capacity = ceil(n / load_factor)
                       (include/cuco_hashmap.cuh:57-87).  The table itself is
                       NVIDIA/cuCollections (branch ``dev``, unpinned, not in the
                       reference tree); nothing of its layout is observable.
* scan ............... PARITY UNPINNED: the reference's thrust_scan races
                       (src/thrust_scan.cu:11-17) and no reference test calls it;
                       the oracle is the intended prefix sum with int32 wrap.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np


# --------------------------------------------------------------------------- hashmap
def hashmap_capacity(numel: int, load_factor: float) -> int:
    """include/cuco_hashmap.cuh:62 — ``std::ceil(numel / load_factor)``."""
    return int(math.ceil(numel / load_factor))


def hashmap_build(keys: np.ndarray, values: np.ndarray) -> Dict[int, int]:
    """include/cuco_hashmap.cuh:66-70 — bulk insert of (key, value); keys are unique, != -1."""
    return {int(k): int(v) for k, v in zip(keys.tolist(), values.tolist())}


def hashmap_query(table: Dict[int, int], requests: np.ndarray, key_dtype=np.int64,
                  value_dtype=np.int64) -> np.ndarray:
    """include/cuco_hashmap.cuh:81-87 + src/cuco_hashmap.cu:29 — requests are cast to the
    key dtype first; the answer is the stored value or -1, in the value dtype."""
    req = np.asarray(requests).astype(key_dtype)
    out = np.fromiter((table.get(int(r), -1) for r in req.reshape(-1).tolist()), dtype=np.int64,
                      count=req.size)
    return out.astype(value_dtype).reshape(req.shape)


def hashmap_erase(table: Dict[int, int], keys: np.ndarray) -> np.ndarray:
    """Removal of keys from the map: per key the value it had, or -1 (absent, or listed before
    in the same call).  The reference has no erase (its map is built once,
    include/cuco_hashmap.cuh:49-93); this states the contract of the added entry point."""
    return np.array([table.pop(int(k), -1) for k in np.asarray(keys).reshape(-1).tolist()],
                    dtype=np.int64)


# --------------------------------------------------------------------------- fetch / set
def uva_fetch(data: np.ndarray, indices: np.ndarray) -> np.ndarray:
    """src/cache_feature_fetch.cu:27-45 — ``out[i] = data[indices[i]]``."""
    return data[np.asarray(indices, dtype=np.int64)]


def cache_fetch_with_mask(uva_data: np.ndarray, gpu_data: np.ndarray, indices: np.ndarray,
                          mask: np.ndarray) -> np.ndarray:
    """src/cache_feature_fetch.cu:203-224 — row from ``gpu_data[mask[i]]`` if ``mask[i] >= 0``
    else from ``uva_data[indices[i]]``."""
    indices = np.asarray(indices, dtype=np.int64)
    mask = np.asarray(mask, dtype=np.int64)
    out = np.empty((indices.size, *uva_data.shape[1:]), dtype=uva_data.dtype)
    hit = mask >= 0
    out[hit] = gpu_data[mask[hit]]
    out[~hit] = uva_data[indices[~hit]]
    return out


def cache_fetch(uva_data: np.ndarray, gpu_data: np.ndarray, indices: np.ndarray,
                table: Dict[int, int], key_dtype=np.int64) -> np.ndarray:
    """src/cache_feature_fetch.cu:106-129 — probe, then as ``cache_fetch_with_mask``."""
    return cache_fetch_with_mask(uva_data, gpu_data, indices,
                                 hashmap_query(table, indices, key_dtype))


def cache_set_with_mask(uva_data: np.ndarray, gpu_data: np.ndarray, indices: np.ndarray,
                        update: np.ndarray, mask: np.ndarray) -> None:
    """src/cache_feature_set.cu:184-207 — in place; indices are unique (the reference's tests
    use unique ids, example/test_cache_set.py:30-31)."""
    indices = np.asarray(indices, dtype=np.int64)
    mask = np.asarray(mask, dtype=np.int64)
    hit = mask >= 0
    gpu_data[mask[hit]] = update[hit]
    uva_data[indices[~hit]] = update[~hit]


def cache_set(uva_data, gpu_data, indices, update, table, key_dtype=np.int64) -> None:
    """src/cache_feature_set.cu:93-116."""
    cache_set_with_mask(uva_data, gpu_data, indices, update,
                        hashmap_query(table, indices, key_dtype))


def uva_set(data: np.ndarray, indices: np.ndarray, update: np.ndarray) -> None:
    """src/cache_feature_set.cu:18-37."""
    data[np.asarray(indices, dtype=np.int64)] = update


def insert_set(table: Dict[int, int], gpu_data: np.ndarray, keys: np.ndarray, slots: np.ndarray,
               update: np.ndarray) -> None:
    """The added fused insert/overwrite: a new key takes ``slots[i]``, a known key keeps its
    slot; ``update[i]`` goes to that slot.  Equivalent to building the map from (keys, slots)
    (include/cuco_hashmap.cuh:66-70) and then ``cache_set`` with every id a hit."""
    for i, k in enumerate(np.asarray(keys).tolist()):
        s = table.setdefault(int(k), int(slots[i]))
        gpu_data[s] = update[i]


# --------------------------------------------------------------------------- scan
def scan_inclusive(a: np.ndarray) -> np.ndarray:
    """Intended semantics of src/thrust_scan.cu:9-18 (parity unpinned): prefix sum, wrapping."""
    return np.cumsum(a.astype(np.int64)).astype(a.dtype)


def scan_exclusive(a: np.ndarray) -> np.ndarray:
    """src/cache_graph_sampling.cu:30-45 — cub::DeviceScan::ExclusiveSum in place."""
    c = np.cumsum(a.astype(np.int64))
    out = np.empty_like(c)
    out[0] = 0
    out[1:] = c[:-1]
    return out.astype(a.dtype)


# --------------------------------------------------------------------------- relabel
def tensor_relabel(tensors: Sequence[np.ndarray]) -> Tuple[np.ndarray, List[np.ndarray]]:
    """src/tensor_relabel.cu:125-209, vectorised: distinct ids in first-occurrence order and,
    per input element, the index of its id in that list."""
    total = np.concatenate([np.asarray(t).reshape(-1) for t in tensors])
    if total.size == 0:
        return total, [np.asarray(t).reshape(-1) for t in tensors]
    uniq, first_idx, inverse = np.unique(total, return_index=True, return_inverse=True)
    order = np.argsort(first_idx, kind="stable")       # sorted ids -> first-occurrence order
    rank = np.empty_like(order)
    rank[order] = np.arange(order.size)
    unique = uniq[order].astype(total.dtype)
    relabel = rank[inverse].astype(total.dtype)
    sizes = np.cumsum([np.asarray(t).size for t in tensors])[:-1]
    return unique, np.split(relabel, sizes)


def tensor_relabel_literal(tensors: Sequence[np.ndarray]) -> Tuple[np.ndarray, List[np.ndarray]]:
    """src/tensor_relabel.cu:68-203 step by step (pure Python, small inputs only): table of
    ``1 << int(log2(numel) + 1)`` slots, ``hash = key & (cap - 1)``, probe
    ``pos = hash(pos + delta++)``, CAS the key in, keep the minimum input index per slot, flag
    elements that own their slot, exclusive-scan the flags, emit unique + remap."""
    total = np.concatenate([np.asarray(t).reshape(-1) for t in tensors]).astype(np.int64)
    numel = int(total.size)
    cap = 1 << int(math.log2(numel) + 1)
    keys = [-1] * cap
    index = [np.iinfo(np.int64).max] * cap

    def h(x: int) -> int:
        return x & (cap - 1)

    def probe(key: int, claim: bool) -> int:
        delta, pos = 1, h(key)
        while True:
            if keys[pos] == -1 and claim:
                keys[pos] = key
            if keys[pos] == key:
                return pos
            if keys[pos] == -1:
                return -1
            pos = h(pos + delta)
            delta += 1

    for i, k in enumerate(total.tolist()):                      # :147-154
        pos = probe(k, True)
        index[pos] = min(index[pos], i)
    flags = [1 if index[probe(k, False)] == i else 0 for i, k in enumerate(total.tolist())]
    prefix = np.concatenate([[0], np.cumsum(flags)])            # :161-170
    unique = np.empty(int(prefix[-1]), dtype=np.int64)
    value = [0] * cap
    for i, k in enumerate(total.tolist()):                      # :178-192
        pos = probe(k, False)
        if index[pos] == i:
            unique[prefix[i]] = k
            value[pos] = int(prefix[i])
    relabel = np.array([value[probe(k, False)] for k in total.tolist()], dtype=np.int64)  # :196-203
    dt = np.asarray(tensors[0]).dtype
    sizes = np.cumsum([np.asarray(t).size for t in tensors])[:-1]
    return unique.astype(dt), [r.astype(dt) for r in np.split(relabel, sizes)]


# --------------------------------------------------------------------------- sampling
def row_bounds(indptr: np.ndarray, seeds: np.ndarray, table: Optional[Dict[int, int]] = None,
               gpu_indptr: Optional[np.ndarray] = None, key_dtype=np.int64):
    """src/cache_graph_sampling.cu:70-73 / :259-268 — (begin, end, slot) per seed; ``slot`` is
    -1 for rows read from the host CSR."""
    seeds = np.asarray(seeds, dtype=np.int64)
    slot = np.full(seeds.size, -1, dtype=np.int64)
    if table is not None:
        slot = hashmap_query(table, seeds, key_dtype).astype(np.int64)
    begin = np.where(slot >= 0, 0, np.asarray(indptr, dtype=np.int64)[seeds])
    end = np.where(slot >= 0, 0, np.asarray(indptr, dtype=np.int64)[seeds + 1])
    if table is not None:
        g = np.asarray(gpu_indptr, dtype=np.int64)
        hit = slot >= 0
        begin[hit] = g[slot[hit]]
        end[hit] = g[slot[hit] + 1]
    return begin, end, slot


def sub_indptr(indptr, seeds, num_picks: int, replace: bool, table=None, gpu_indptr=None,
               key_dtype=np.int64) -> np.ndarray:
    """src/cache_graph_sampling.cu:74-83 — picks per seed ``replace ? (deg ? k : 0) : min(deg, k)``
    followed by an exclusive scan over n+1 entries; dtype of ``indptr``."""
    begin, end, _ = row_bounds(indptr, seeds, table, gpu_indptr, key_dtype)
    deg = end - begin
    cnt = np.where(deg == 0, 0, num_picks) if replace else np.minimum(deg, num_picks)
    out = np.zeros(cnt.size + 1, dtype=np.int64)
    np.cumsum(cnt, out=out[1:])
    return out.astype(np.asarray(indptr).dtype)


def csr_sampling(indptr, indices, seeds, num_picks: int, replace: bool,
                 rng: np.random.Generator, table=None, gpu_indptr=None, gpu_indices=None,
                 key_dtype=np.int64) -> Tuple[np.ndarray, np.ndarray]:
    """src/cache_graph_sampling.cu:109-145 and :163-176 (cached: :306-345, :366-378).

    deg <= k: the row is copied in CSR order.  Otherwise, without replacement, algorithm R:
    slots 0..k-1 start as positions 0..k-1 and every position i in [k, deg) draws
    ``r = rand % (i + 1)`` and takes slot r if r < k (the kernel's atomicMax keeps the
    largest i per slot, i.e. the serial order); with replacement, k draws ``rand % deg``.
    The random stream is numpy's, not cuRAND's: draws are comparable only in distribution.
    """
    begin, end, slot = row_bounds(indptr, seeds, table, gpu_indptr, key_dtype)
    ptr = sub_indptr(indptr, seeds, num_picks, replace, table, gpu_indptr, key_dtype).astype(np.int64)
    indices = np.asarray(indices)
    out = np.empty(int(ptr[-1]), dtype=indices.dtype)
    k = int(num_picks)
    for i in range(len(begin)):
        src = indices if slot[i] < 0 else np.asarray(gpu_indices)
        b, deg = int(begin[i]), int(end[i] - begin[i])
        o = int(ptr[i])
        if replace:
            if deg > 0:
                out[o:o + k] = src[b + rng.integers(0, deg, size=k)]
        elif deg <= k:
            out[o:o + deg] = src[b:b + deg]
        else:
            res = np.arange(k)
            draws = rng.integers(0, np.arange(k, deg) + 1)
            for pos, r in zip(range(k, deg), draws.tolist()):
                if r < k:
                    res[r] = pos
            out[o:o + k] = src[b + res]
    return ptr.astype(np.asarray(indptr).dtype), out


def create_subcsr(indptr, indices, seeds) -> Tuple[np.ndarray, np.ndarray]:
    """src/cache_graph_sampling.cu:455-492 — compact CSR of the rows ``seeds`` in that order."""
    indptr = np.asarray(indptr)
    indices = np.asarray(indices)
    seeds = np.asarray(seeds, dtype=np.int64)
    deg = indptr[seeds + 1].astype(np.int64) - indptr[seeds].astype(np.int64)
    gpu_indptr = np.zeros(seeds.size + 1, dtype=np.int64)
    np.cumsum(deg, out=gpu_indptr[1:])
    gpu_indices = np.empty(int(gpu_indptr[-1]), dtype=indices.dtype)
    for i, s in enumerate(seeds.tolist()):
        gpu_indices[gpu_indptr[i]:gpu_indptr[i + 1]] = indices[indptr[s]:indptr[s + 1]]
    return gpu_indptr.astype(indptr.dtype), gpu_indices


def check_sample(indptr, indices, seeds, num_picks: int, replace: bool, got_indptr, got_indices,
                 table=None, gpu_indptr=None, gpu_indices=None, key_dtype=np.int64,
                 positional: bool = False) -> None:
    """Assert that a sampler's output is a legal outcome of the reference algorithm:
    offsets exact; rows with deg <= k copied exactly (no replacement); every other sampled
    value lies in its row; without replacement no position is taken twice (checked on values
    when ``positional`` says the row values are distinct)."""
    want_ptr = sub_indptr(indptr, seeds, num_picks, replace, table, gpu_indptr, key_dtype)
    got_indptr = np.asarray(got_indptr)
    got_indices = np.asarray(got_indices)
    assert got_indptr.dtype == want_ptr.dtype, (got_indptr.dtype, want_ptr.dtype)
    assert np.array_equal(got_indptr, want_ptr), "sub_indptr differs"
    assert got_indices.size == int(want_ptr[-1])
    begin, end, slot = row_bounds(indptr, seeds, table, gpu_indptr, key_dtype)
    indices = np.asarray(indices)
    for i in range(len(begin)):
        src = indices if slot[i] < 0 else np.asarray(gpu_indices)
        row = src[int(begin[i]):int(end[i])]
        got = got_indices[int(want_ptr[i]):int(want_ptr[i + 1])]
        if not replace and row.size <= num_picks:
            assert np.array_equal(got, row), f"seed {i}: row not copied exactly"
            continue
        assert np.isin(got, row).all(), f"seed {i}: sampled value outside the row"
        if not replace and positional:
            assert np.unique(got).size == got.size, f"seed {i}: duplicate pick"


def check_sample_bulk(indptr, indices, seeds, num_picks: int, replace: bool, got_indptr, got_indices,
                      distinct_rows: bool = False) -> None:
    """The assertions of ``check_sample`` as whole-array numpy operations, for full-size
    workloads (a frontier of 100,000 seeds takes a second instead of minutes).  Rows are looked
    up in the host CSR only: a cached copy made by ``create_subcsr`` holds the same rows
    (src/cache_graph_sampling.cu:468-487), so membership in the host row is the same test.
    ``distinct_rows``: the values of every row are distinct, so a value taken twice without
    replacement is a position taken twice."""
    indptr = np.asarray(indptr)
    indices = np.asarray(indices)
    seeds = np.asarray(seeds).astype(np.int64)
    got_indptr, got_indices = np.asarray(got_indptr), np.asarray(got_indices)
    n = seeds.size
    begin = indptr[seeds].astype(np.int64)
    deg = indptr[seeds + 1].astype(np.int64) - begin
    cnt = np.where(deg > 0, num_picks, 0) if replace else np.minimum(deg, num_picks)
    want_ptr = np.concatenate([[0], np.cumsum(cnt)]).astype(indptr.dtype)
    assert got_indptr.dtype == want_ptr.dtype, (got_indptr.dtype, want_ptr.dtype)
    assert np.array_equal(got_indptr, want_ptr), "sub_indptr differs"
    nnz = int(want_ptr[-1])
    assert got_indices.size == nnz
    owner = np.repeat(np.arange(n, dtype=np.int64), cnt)            # seed index of every output
    within = np.arange(nnz, dtype=np.int64) - want_ptr[owner].astype(np.int64)
    exact = np.zeros(nnz, dtype=bool) if replace else deg[owner] <= num_picks
    assert np.array_equal(got_indices[exact], indices[begin[owner[exact]] + within[exact]]), \
        "a row with deg <= k was not copied exactly"
    rest = ~exact
    if not rest.any():
        return
    picked_from = np.unique(owner[rest])                            # seeds whose row was sampled
    d = deg[picked_from]
    row_owner = np.repeat(picked_from, d)
    start = np.concatenate([[0], np.cumsum(d)])[:-1]
    j = np.arange(int(d.sum()), dtype=np.int64) - np.repeat(start, d)
    row_keys = (row_owner << 32) | indices[np.repeat(begin[picked_from], d) + j].astype(np.int64)
    got_keys = (owner[rest] << 32) | got_indices[rest].astype(np.int64)
    assert np.isin(got_keys, row_keys).all(), "a sampled value lies outside its row"
    if distinct_rows and not replace:
        assert np.unique(got_keys).size == got_keys.size, "a position was picked twice"


# --------------------------------------------------------------------------- timed CPU lines
def cpu_fetch_reference(data, indices):
    """The reference's own CPU path for a feature fetch, ``data[q.cpu()]``
    (example/test_cache_fetch.py:138-139, the ``cpu_fetch`` line): torch's multithreaded
    index_select over the shared-memory / pinned host table."""
    import torch
    return torch.index_select(data, 0, indices)
