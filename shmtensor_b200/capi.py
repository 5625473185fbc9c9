"""Drop-in mirror of the reference's ``ShmTensorLib`` pybind module.

Same function names, keyword names, return shapes/dtypes and error behaviour as
the reference's ``src/pybind.cc:16-65``; the work is done by ``libshmt.so``
through its C-ABI.  PyTorch is only the tensor carrier here: this module checks
arguments, allocates outputs with ``torch.empty`` and passes raw pointers plus
torch's current CUDA stream.  There is no CPU implementation behind any of the
GPU entry points — they raise if no GPU / no library is available.

Differences a caller can see, all extensions:

* kernels run on torch's *current* stream (the reference uses the legacy
  default stream);
* ``indptr`` and ``indices`` may have different integer dtypes;
* payload rows may have any dtype (the reference rejects f16/bf16/bool);
* sampling draws differ from call to call (``set_sampling_seed`` pins them);
* ``CUCOStaticHashmap.insert`` / ``.empty`` and ``cache_insert_set`` exist.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import List, Sequence, Tuple

import torch

from . import _lib
from ._lib import I32, I64, check, lib

_INT_CODES = {torch.int32: I32, torch.int64: I64}
_CODE_DTYPES = {I32: torch.int32, I64: torch.int64}

_NPY_DTYPES = {
    "<f2": torch.float16, "<f4": torch.float32, "<f8": torch.float64, "|u1": torch.uint8,
    "|i1": torch.int8, "<i2": torch.int16, "<i4": torch.int32, "<i8": torch.int64,
    "|b1": torch.bool,
    # numpy has no bfloat16; writers that know the type (ml_dtypes, torch -> view(int16).numpy()
    # saved through a void view) store it as an opaque 2-byte item
    "<V2": torch.bfloat16, "|V2": torch.bfloat16,
}


# --------------------------------------------------------------------------- helpers
def _int_code(t: torch.Tensor, what: str) -> int:
    try:
        return _INT_CODES[t.dtype]
    except KeyError:
        raise RuntimeError(f"{what}: ID can only be int32 or int64, got {t.dtype}") from None


def _check_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")


def _check_contig(t: torch.Tensor, name: str) -> None:
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")


def _stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _ptr(t) -> int | None:
    if t is None:
        return None
    return t.data_ptr() if t.numel() else None


_contexts: dict = {}


def _ctx(device: torch.device) -> int:
    """libshmt context of (device, torch's current stream on it), created on first use.  A
    context's scratch serves one stream at a time, so every stream gets its own: calls issued
    from different torch streams can overlap on the GPU without sharing look-back state, result
    words or the relabel table."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    key = (idx, torch.cuda.current_stream(idx).cuda_stream)
    h = _contexts.get(key)
    if h is None:
        out = C.c_void_p()
        check(lib.shmt_ctx_create(idx, C.byref(out)))
        h = _contexts[key] = out.value
    return h


def reserve_minibatch(n_seeds: int, fanouts: Sequence[int], device="cuda") -> None:
    """Extension: size the current stream's context for ``sample_minibatch`` calls of up to
    ``n_seeds`` seeds with these fan-outs, so the first mini-batch does not stop to allocate."""
    device = torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    fan = (C.c_int64 * len(fanouts))(*[int(k) for k in fanouts])
    check(lib.shmt_ctx_reserve_minibatch(_ctx(device), int(n_seeds), fan, len(fanouts), _stream(device)))


def context_scratch_bytes(device="cuda") -> int:
    """Extension: device bytes the current stream's context holds."""
    device = torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    return lib.shmt_ctx_scratch_bytes(_ctx(device))


def _row_bytes(data: torch.Tensor) -> int:
    n = data.element_size()
    for s in data.shape[1:]:
        n *= s
    return n


_rng = {"seed": 7777, "calls": 0}
_ITEMSIZE = {torch.int32: 4, torch.int64: 8}
_minibatch_layouts: dict = {}


def set_sampling_seed(seed: int) -> None:
    """Pin the Philox key used by the samplers and restart the per-call counter.

    The reference hard-codes the seed 7777 (src/cache_graph_sampling.cu:201-204), so
    every call returns the same sample; here the key defaults to 7777 too but
    each call advances a counter.
    """
    _rng["seed"] = int(seed) & (2**64 - 1)
    _rng["calls"] = 0


# --------------------------------------------------------------------------- host memory
def create_shared_mem(name: str, size: int, pin_memory: bool = False,
                      exclusive: bool = False) -> Tuple[int, int]:
    """include/shm_memory.h:6-23 — returns ``(ptr, fd)``.  Extension: ``exclusive=True`` fails
    (``ShmtError``, code ``ERR_OS``) if a segment of that name already exists, in one atomic
    step instead of ``file_exist`` followed by a create."""
    p, fd = C.c_int64(), C.c_int64()
    fn = lib.shmt_shm_create_excl if exclusive else lib.shmt_shm_create
    check(fn(name.encode(), size, int(pin_memory), C.byref(p), C.byref(fd)))
    return p.value, fd.value


def unlink_shared_mem(name: str) -> None:
    """Extension: remove the name of a segment (one a killed run left behind, say).  Mappings
    that exist keep their memory; a name that does not exist is not an error."""
    check(lib.shmt_shm_unlink(name.encode()))


NUMA_INTERLEAVE, NUMA_BIND = 1, 2


def prefault(ptr: int, nbytes: int, n_threads: int = 0) -> None:
    """Extension: make the pages of a fresh (all-zero) host mapping present from several threads
    (default: one per core this process may run on, at most 32), before it is registered."""
    import os
    n = n_threads or min(32, len(os.sched_getaffinity(0)))
    check(lib.shmt_host_prefault(ptr, nbytes, n))


def numa_nodes() -> int:
    """Extension: number of memory nodes of this machine."""
    return lib.shmt_host_numa_nodes()


def numa_place(ptr: int, nbytes: int, policy: int = NUMA_INTERLEAVE, node: int = 0) -> None:
    """Extension: spread a fresh, page-aligned host mapping over all memory nodes
    (``NUMA_INTERLEAVE``) or put it on ``node`` (``NUMA_BIND``), before it is written and
    registered.  Decides which memory controllers and inter-socket links the GPUs' reads of a
    host table load."""
    check(lib.shmt_host_numa_place(ptr, nbytes, policy, node))


def open_shared_mem(name: str, size: int, pin_memory: bool = False) -> Tuple[int, int]:
    """include/shm_memory.h:25-39 — returns ``(ptr, fd)``."""
    p, fd = C.c_int64(), C.c_int64()
    check(lib.shmt_shm_open(name.encode(), size, int(pin_memory), C.byref(p), C.byref(fd)))
    return p.value, fd.value


def release_shared_mem(name: str, size: int, ptr: int, fd: int, pin_memory: bool = False) -> None:
    """include/shm_memory.h:41-49 — unregister, unmap, close and unlink."""
    check(lib.shmt_shm_release(name.encode(), size, ptr, fd, int(pin_memory)))


def _tensor_from_address(ptr: int, dtype: torch.dtype, shape: Sequence[int]) -> torch.Tensor:
    numel = 1
    for s in shape:
        numel *= int(s)
    itemsize = torch.empty((), dtype=dtype).element_size()
    if numel == 0:
        return torch.empty(tuple(shape), dtype=dtype)
    buf = (C.c_char * (numel * itemsize)).from_address(ptr)
    return torch.frombuffer(buf, dtype=dtype, count=numel).reshape(tuple(shape))


def open_shared_tensor(ptr: int, dtype: torch.dtype, shape: Sequence[int]) -> torch.Tensor:
    """include/shm_memory.h:51-56 — zero-copy CPU tensor over the mapping."""
    return _tensor_from_address(ptr, dtype, shape)


def file_exist(filename: str) -> bool:
    """include/utils.h:5-13 — does a POSIX shm segment of that name exist?"""
    return bool(lib.shmt_shm_exists(filename.encode()))


def open_mmap_tensor(filename: str, pin_memory: bool, read_only: bool = False):
    """src/mmap_tensor.cc:10-47 — returns ``(tensor, size, ptr, fd)``.  Extensions: ``read_only``
    maps the file without write permission (writing through the tensor then faults, as for any
    read-only mapping); an opaque 2-byte item (``V2``) is read as bfloat16."""
    info = _lib.NpyInfo()
    check(lib.shmt_npy_open(filename.encode(), int(bool(pin_memory)) | (2 if read_only else 0),
                            C.byref(info)))
    descr = info.descr.decode()
    try:
        if info.fortran_order:
            raise RuntimeError("fortran order is not supported")
        if descr not in _NPY_DTYPES:
            raise RuntimeError(f"parse_npy_header: failed to find dtype ({descr})")
    except RuntimeError:
        lib.shmt_npy_close(info.file_size, info.ptr, info.fd, int(pin_memory))
        raise
    shape = [info.shape[i] for i in range(info.ndim)]
    t = _tensor_from_address(info.ptr + info.data_offset, _NPY_DTYPES[descr], shape)
    return t, info.file_size, info.ptr, info.fd


def close_mmap_tensor(size: int, ptr: int, fd: int, pin_memory: bool) -> None:
    """src/mmap_tensor.cc:49-55."""
    check(lib.shmt_npy_close(size, ptr, fd, int(pin_memory)))


def pin_memory(data: torch.Tensor) -> None:
    """src/cache_feature_fetch.cu:6-9 — cudaHostRegister(Portable) of a CPU tensor in place."""
    _check_contig(data, "data")
    check(lib.shmt_host_register(data.data_ptr(), data.numel() * data.element_size()))


def _register_range(ptr: int, nbytes: int) -> None:
    check(lib.shmt_host_register(ptr, nbytes))


def unpin_memory(data: torch.Tensor) -> None:
    """src/cache_feature_fetch.cu:11-13."""
    check(lib.shmt_host_unregister(data.data_ptr()))


# --------------------------------------------------------------------------- hashmap
class CUCOStaticHashmap:
    """include/cuco_hashmap.h:12-25 — static map int32/int64 keys -> int32/int64 values.

    ``query`` returns the stored value or -1; ``capacity()`` is
    ``ceil(numel / load_factor)`` exactly as the reference reports it.
    """

    def __init__(self, keys: torch.Tensor, values: torch.Tensor, load_factor: float):
        _check_cuda(keys, "keys")
        _check_cuda(values, "values")
        kd = _int_code(keys, "keys")
        vd = _int_code(values, "values")
        if keys.numel() != values.numel():
            raise RuntimeError("keys and values must have the same number of elements")
        capacity = int(math.ceil(keys.numel() / load_factor))
        self._init_empty(capacity, kd, vd, keys.device, expected_keys=keys.numel())
        self.insert(keys, values)

    def _init_empty(self, capacity: int, kd: int, vd: int, device: torch.device,
                    expected_keys: int = 0) -> None:
        self._handle = None
        self._device = device
        self._kd, self._vd = kd, vd
        nbytes = lib.shmt_map_table_bytes(capacity, expected_keys)
        # table memory comes from torch's caching allocator, like the reference's torch_allocator
        self._table = torch.empty(nbytes, dtype=torch.uint8, device=device)
        out = C.c_void_p()
        check(lib.shmt_map_create(device.index, capacity, expected_keys, kd, vd, self._table.data_ptr(),
                                  _stream(device), C.byref(out)))
        self._handle = out.value

    @classmethod
    def empty(cls, capacity: int, key_dtype=torch.int64, value_dtype=torch.int64,
              device="cuda") -> "CUCOStaticHashmap":
        """Extension: an empty map with room for ``capacity`` keys (see ``insert``)."""
        self = cls.__new__(cls)
        device = torch.device(device)
        if device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        self._init_empty(int(capacity), _INT_CODES[key_dtype], _INT_CODES[value_dtype], device)
        return self

    def insert(self, keys: torch.Tensor, values: torch.Tensor) -> None:
        """Extension: insert_or_assign more pairs (keys != -1).  Raises on overflow."""
        _check_cuda(keys, "keys")
        _check_cuda(values, "values")
        keys = keys.contiguous().to(_CODE_DTYPES[self._kd])
        values = values.contiguous().to(_CODE_DTYPES[self._vd])
        check(lib.shmt_map_insert(self._handle, _ptr(keys), _ptr(values), keys.numel(),
                                  _stream(self._device)))

    def erase(self, keys: torch.Tensor) -> torch.Tensor:
        """Extension: remove ``keys``; returns per key the value it had, or -1 if it was absent.
        The freed slots are taken again by later ``insert`` calls."""
        _check_cuda(keys, "keys")
        keys = keys.contiguous().to(_CODE_DTYPES[self._kd])
        out = torch.empty(keys.shape, dtype=_CODE_DTYPES[self._vd], device=keys.device)
        check(lib.shmt_map_erase(self._handle, _ptr(keys), keys.numel(), _ptr(out),
                                 _stream(self._device)))
        return out

    def query(self, requests: torch.Tensor) -> torch.Tensor:
        _check_cuda(requests, "requests")
        if requests.dtype not in _INT_CODES:
            requests = requests.to(_CODE_DTYPES[self._kd])
        requests = requests.contiguous()
        out = torch.empty(requests.shape, dtype=_CODE_DTYPES[self._vd], device=requests.device)
        check(lib.shmt_map_query(self._handle, _ptr(requests), _INT_CODES[requests.dtype],
                                 requests.numel(), _ptr(out), _stream(requests.device)))
        return out

    def capacity(self) -> int:
        return lib.shmt_map_capacity(self._handle)

    def memory_usage(self) -> int:
        return lib.shmt_map_memory_usage(self._handle)

    def size(self) -> int:
        """Extension: number of distinct keys stored."""
        return lib.shmt_map_size(self._handle)

    @property
    def key_dtype(self) -> torch.dtype:
        return _CODE_DTYPES[self._kd]

    @property
    def value_dtype(self) -> torch.dtype:
        return _CODE_DTYPES[self._vd]

    def __del__(self, _destroy=lib.shmt_map_destroy):
        h = getattr(self, "_handle", None)
        if h is not None:
            self._handle = None
            _destroy(h)  # bound at definition: module globals may be gone at interpreter exit


# --------------------------------------------------------------------------- fetch / set
def _fetch(uva_data, gpu_data, indices, hashmap, mask, who, out=None):
    _check_cuda(indices, "indices")
    indices = indices.contiguous()
    idt = _int_code(indices, who)
    shape_src = uva_data if uva_data is not None else gpu_data
    _check_contig(shape_src, "data")
    if gpu_data is not None:
        _check_cuda(gpu_data, "gpu_data")
        _check_contig(gpu_data, "gpu_data")
    n = indices.numel()
    if out is None:
        out = torch.empty((n, *shape_src.shape[1:]), dtype=shape_src.dtype, device=indices.device)
    else:
        _check_cuda(out, "out")
        _check_contig(out, "out")
        if out.dtype != shape_src.dtype or tuple(out.shape) != (n, *shape_src.shape[1:]):
            raise RuntimeError(f"{who}: out must be a {(n, *shape_src.shape[1:])} tensor of {shape_src.dtype}")
    mdt = 0
    if mask is not None:
        _check_cuda(mask, "mask")
        mask = mask.contiguous()
        mdt = _int_code(mask, who)
    check(lib.shmt_fetch(hashmap._handle if hashmap is not None else None, _ptr(mask), mdt,
                         _ptr(uva_data), _ptr(gpu_data), _ptr(indices), idt, n,
                         _row_bytes(shape_src), _ptr(out), _stream(indices.device)))
    return out


def check_async(device="cuda") -> None:
    """Extension: wait for the current stream and raise if the last asynchronous call on this
    device's context (``thrust_scan`` / ``exclusive_scan_``) ended with a device-side error."""
    device = torch.device(device)
    check(lib.shmt_ctx_check(_ctx(device), _stream(device)))


def device_fault() -> int:
    """Extension: code left by a kernel whose bounded wait ran out (0 = none); synchronises."""
    code = C.c_int(0)
    check(lib.shmt_device_fault(C.byref(code)))
    return code.value


def uva_fetch(data: torch.Tensor, indices: torch.Tensor, out: torch.Tensor = None) -> torch.Tensor:
    """src/cache_feature_fetch.cu:47-87 — ``data[indices]`` read over UVA, result on the GPU.
    Extension: ``out`` receives the rows instead of a fresh tensor (filling a cache in place)."""
    return _fetch(data, None, indices, None, None, "uva_fetch", out)


def cache_fetch(uva_data: torch.Tensor, gpu_data: torch.Tensor, indices: torch.Tensor,
                hashmap: CUCOStaticHashmap) -> torch.Tensor:
    """src/cache_feature_fetch.cu:131-185 — hit rows from ``gpu_data``, misses from ``uva_data``."""
    return _fetch(uva_data, gpu_data, indices, hashmap, None, "cache_fetch")


def cache_fetch_with_mask(uva_data: torch.Tensor, gpu_data: torch.Tensor, indices: torch.Tensor,
                          mask: torch.Tensor) -> torch.Tensor:
    """src/cache_feature_fetch.cu:226-272 — like ``cache_fetch`` with slots given by ``mask``."""
    return _fetch(uva_data, gpu_data, indices, None, mask, "cache_fetch_with_mask")


def _set(uva_data, gpu_data, indices, update, hashmap, mask, who):
    _check_cuda(indices, "indices")
    _check_cuda(update, "update")
    indices = indices.contiguous()
    update = update.contiguous()
    idt = _int_code(indices, who)
    ref = uva_data if uva_data is not None else gpu_data
    _check_contig(ref, "data")
    if update.dtype != ref.dtype:
        raise RuntimeError(f"{who}: update has dtype {update.dtype}, the table {ref.dtype}")
    if update.numel() != indices.numel() * (_row_bytes(ref) // ref.element_size()):
        raise RuntimeError(f"{who}: update must hold one row per index")
    mdt = 0
    if mask is not None:
        _check_cuda(mask, "mask")
        mask = mask.contiguous()
        mdt = _int_code(mask, who)
    check(lib.shmt_set(hashmap._handle if hashmap is not None else None, _ptr(mask), mdt,
                       _ptr(uva_data), _ptr(gpu_data), _ptr(indices), idt, indices.numel(),
                       _row_bytes(ref), _ptr(update), _stream(indices.device)))


def uva_set(data: torch.Tensor, indices: torch.Tensor, update: torch.Tensor) -> None:
    """src/cache_feature_set.cu:39-75 — ``data[indices] = update`` written over UVA."""
    _set(data, None, indices, update, None, None, "uva_set")


def cache_set(uva_data: torch.Tensor, gpu_data: torch.Tensor, indices: torch.Tensor,
              update: torch.Tensor, hashmap: CUCOStaticHashmap) -> None:
    """src/cache_feature_set.cu:118-165 — hits overwrite the cached row, misses the host row."""
    _set(uva_data, gpu_data, indices, update, hashmap, None, "cache_set")


def cache_set_with_mask(uva_data: torch.Tensor, gpu_data: torch.Tensor, indices: torch.Tensor,
                        update: torch.Tensor, mask: torch.Tensor) -> None:
    """src/cache_feature_set.cu:209-248."""
    _set(uva_data, gpu_data, indices, update, None, mask, "cache_set_with_mask")


def cache_insert_set(gpu_data: torch.Tensor, indices: torch.Tensor, slots: torch.Tensor,
                     update: torch.Tensor, hashmap: CUCOStaticHashmap) -> None:
    """Extension: fused insert/overwrite.

    ``indices[i]`` is inserted with value ``slots[i]`` unless already present
    (then its stored slot is kept) and ``update[i]`` is written to that slot of
    ``gpu_data`` in the same kernel.  Raises if the map overflows.
    """
    for t, nm in ((gpu_data, "gpu_data"), (indices, "indices"), (slots, "slots"), (update, "update")):
        _check_cuda(t, nm)
    indices, slots, update = indices.contiguous(), slots.contiguous(), update.contiguous()
    _check_contig(gpu_data, "gpu_data")
    if update.dtype != gpu_data.dtype:
        raise RuntimeError("cache_insert_set: update and gpu_data dtypes differ")
    check(lib.shmt_insert_set(hashmap._handle, _ptr(gpu_data), _ptr(indices),
                              _int_code(indices, "cache_insert_set"), _ptr(slots),
                              _int_code(slots, "cache_insert_set"), indices.numel(),
                              _row_bytes(gpu_data), _ptr(update), _stream(indices.device)))


# --------------------------------------------------------------------------- scan / relabel
def cache_replace(uva_data: torch.Tensor, gpu_data: torch.Tensor, hashmap: CUCOStaticHashmap,
                  evict_ids: torch.Tensor, admit_ids: torch.Tensor) -> int:
    """Extension: turn the cache over in place.  The rows of ``evict_ids`` leave the cache; the ids
    of ``admit_ids`` (distinct, not cached yet) take their rows of ``gpu_data`` and are filled from
    ``uva_data`` by the UVA gather kernel.  The reference rebuilds the map and re-copies every
    row from the CPU to change the cached set (example/test_cache_set.py:57-61).  Admits at most
    as many ids as rows were freed, in order; returns how many.  An id listed twice in
    ``evict_ids`` is evicted once."""
    freed = hashmap.erase(torch.unique(evict_ids, sorted=True))
    freed = freed[freed >= 0]
    n = min(int(freed.numel()), int(admit_ids.numel()))
    if n == 0:
        return 0
    admit, rows = admit_ids[:n].contiguous(), freed[:n].contiguous()
    hashmap.insert(admit, rows)
    uva_set(gpu_data, rows, uva_fetch(uva_data, admit))
    return n


def thrust_scan(tensor: torch.Tensor) -> None:
    """src/thrust_scan.cu:9-18 — in-place inclusive prefix sum (int32; int64 also accepted)."""
    _check_cuda(tensor, "tensor")
    _check_contig(tensor, "tensor")
    check(lib.shmt_scan(_ctx(tensor.device), _ptr(tensor), _int_code(tensor, "thrust_scan"),
                        tensor.numel(), 0, _stream(tensor.device)))


def exclusive_scan_(tensor: torch.Tensor) -> None:
    """In-place exclusive prefix sum (the reference's internal cub_exclusiveSum)."""
    _check_cuda(tensor, "tensor")
    _check_contig(tensor, "tensor")
    check(lib.shmt_scan(_ctx(tensor.device), _ptr(tensor), _int_code(tensor, "exclusive_scan_"),
                        tensor.numel(), 1, _stream(tensor.device)))


def scan_static_(tensor: torch.Tensor, exclusive: bool = False) -> None:
    """Extension: in-place prefix sum that allocates nothing (``shmt_scan_static``).

    For callers that cannot allocate device memory where they need the scan: a component
    living inside an application that owns all device memory, or a loop with a latency
    bound that must never reach ``cudaMalloc``.  The scratch is a fixed array inside the
    library: at most 16,777,216 elements, and two calls that overlap on the same GPU
    corrupt each other.  Let the first call on a device happen before any stream capture.
    """
    _check_cuda(tensor, "tensor")
    _check_contig(tensor, "tensor")
    with torch.cuda.device(tensor.device):
        check(lib.shmt_scan_static(_ptr(tensor), _int_code(tensor, "scan_static_"), tensor.numel(),
                                   int(bool(exclusive)), _stream(tensor.device)))


def tensor_relabel(tensors: List[torch.Tensor]):
    """src/tensor_relabel.cu:125-209 — ``(unique, [relabelled ...])``.

    ``unique`` lists the distinct ids of ``cat(tensors)`` in first-occurrence
    order; each returned tensor holds, for its input, the index into ``unique``.
    """
    if len(tensors) == 0:
        raise RuntimeError("tensor_relabel: expected a non-empty list of tensors")
    dev = tensors[0].device
    dt = tensors[0].dtype
    for t in tensors:
        _check_cuda(t, "tensors")
        if t.device != dev:
            raise RuntimeError("tensor_relabel: all tensors must share a device")
        dt = torch.promote_types(dt, t.dtype)  # what the reference's torch::cat does
    code = _INT_CODES.get(dt)
    if code is None:
        raise RuntimeError(f"tensor_relabel: ID can only be int32 or int64, got {dt}")
    sizes = [t.numel() for t in tensors]
    parts = [t.contiguous().reshape(-1).to(dt) for t in tensors]
    if len(parts) > 8:
        parts = [torch.cat(parts, 0)]
    total = sum(sizes)
    unique = torch.empty(total, dtype=dt, device=dev)
    relabel = torch.empty(total, dtype=dt, device=dev)
    n_parts = len(parts)
    ptrs = (C.c_void_p * n_parts)(*[_ptr(p) for p in parts])
    lens = (C.c_int64 * n_parts)(*[p.numel() for p in parts])
    n_unique = C.c_int64(0)
    check(lib.shmt_relabel(_ctx(dev), ptrs, lens, n_parts, code, _ptr(unique), _ptr(relabel),
                           C.byref(n_unique), _stream(dev)))
    return unique[:n_unique.value], list(relabel.split_with_sizes(sizes, 0))


# --------------------------------------------------------------------------- sampling
def _sample(indptr, indices, gpu_indptr, gpu_indices, hashmap, seeds, num_picks, replace, who):
    _check_cuda(seeds, "seeds")
    seeds = seeds.contiguous()
    dev = seeds.device
    for t, nm in ((indptr, "indptr"), (indices, "indices")):
        _check_contig(t, nm)
    pdt, xdt, sdt = _int_code(indptr, who), _int_code(indices, who), _int_code(seeds, who)
    if hashmap is not None:
        _check_cuda(gpu_indptr, "gpu_indptr")
        _check_cuda(gpu_indices, "gpu_indices")
        if gpu_indptr.dtype != indptr.dtype or gpu_indices.dtype != indices.dtype:
            raise RuntimeError(f"{who}: the cached CSR must have the dtypes of the host CSR")
    n, k = seeds.numel(), int(num_picks)
    sub_indptr = torch.empty(n + 1, dtype=indptr.dtype, device=dev)
    sub_indices = torch.empty(n * k, dtype=indices.dtype, device=dev)
    nnz = C.c_int64(0)
    _rng["calls"] += 1
    check(lib.shmt_sample_hop(_ctx(dev), _ptr(indptr), pdt, _ptr(indices), xdt, _ptr(gpu_indptr),
                              _ptr(gpu_indices), hashmap._handle if hashmap is not None else None,
                              _ptr(seeds), sdt, n, k, int(bool(replace)), _rng["seed"],
                              _rng["calls"], sub_indptr.data_ptr(), _ptr(sub_indices),
                              C.byref(nnz), _stream(dev)))
    return sub_indptr, sub_indices[:nnz.value]


def csr_sampling(indptr: torch.Tensor, indices: torch.Tensor, seeds: torch.Tensor,
                 num_picks: int, replace: bool):
    """src/cache_graph_sampling.cu:179-220 — ``(sub_indptr, sub_indices)`` for one hop."""
    return _sample(indptr, indices, None, None, None, seeds, num_picks, replace, "csr_sampling")


def csr_cache_sampling(uva_indptr: torch.Tensor, uva_indices: torch.Tensor,
                       gpu_indptr: torch.Tensor, gpu_indices: torch.Tensor,
                       hashmap: CUCOStaticHashmap, seeds: torch.Tensor, num_picks: int,
                       replace: bool):
    """src/cache_graph_sampling.cu:382-426 — cached rows from the GPU CSR, the rest over UVA."""
    return _sample(uva_indptr, uva_indices, gpu_indptr, gpu_indices, hashmap, seeds, num_picks,
                   replace, "csr_cache_sampling")


def subcsr_edge_base(uva_indptr: torch.Tensor, seeds: torch.Tensor) -> torch.Tensor:
    """Extension: ``uva_indptr[seeds]`` on the GPU — where each row of a cached sub-CSR (built from
    the same ``seeds`` by ``create_subcsr``) starts in the full edge array."""
    _check_cuda(seeds, "seeds")
    seeds = seeds.contiguous()
    _check_contig(uva_indptr, "uva_indptr")
    out = torch.empty(seeds.numel(), dtype=uva_indptr.dtype, device=seeds.device)
    check(lib.shmt_subcsr_edge_base(_ptr(uva_indptr), _int_code(uva_indptr, "subcsr_edge_base"), _ptr(seeds),
                                    _int_code(seeds, "subcsr_edge_base"), seeds.numel(), _ptr(out),
                                    _stream(seeds.device)))
    return out


def csr_sampling_with_eids(indptr, indices, seeds, num_picks: int, replace: bool, gpu_indptr=None,
                           gpu_indices=None, gpu_edge_base=None, hashmap: "CUCOStaticHashmap | None" = None):
    """Extension: one hop like ``csr_sampling`` / ``csr_cache_sampling`` that also returns the edge
    id of every sampled neighbour (its position in ``indices``, dtype of ``indptr``):
    ``(sub_indptr, sub_indices, sub_eids)``.  The reference passes an empty edge-id tensor to its
    block builder (python/shmtensor/sampling.py:9-20).  With a cached graph give ``gpu_edge_base``
    from ``subcsr_edge_base``."""
    _check_cuda(seeds, "seeds")
    seeds = seeds.contiguous()
    dev = seeds.device
    who = "csr_sampling_with_eids"
    for t, nm in ((indptr, "indptr"), (indices, "indices")):
        _check_contig(t, nm)
    pdt, xdt, sdt = _int_code(indptr, who), _int_code(indices, who), _int_code(seeds, who)
    if hashmap is not None:
        for t, nm in ((gpu_indptr, "gpu_indptr"), (gpu_indices, "gpu_indices"), (gpu_edge_base, "gpu_edge_base")):
            if t is None:
                raise RuntimeError(f"{who}: a cached graph needs {nm}")
            _check_cuda(t, nm)
        if gpu_indptr.dtype != indptr.dtype or gpu_indices.dtype != indices.dtype or gpu_edge_base.dtype != indptr.dtype:
            raise RuntimeError(f"{who}: the cached CSR must have the dtypes of the host CSR")
    n, k = seeds.numel(), int(num_picks)
    sub_indptr = torch.empty(n + 1, dtype=indptr.dtype, device=dev)
    sub_indices = torch.empty(n * k, dtype=indices.dtype, device=dev)
    sub_eids = torch.empty(n * k, dtype=indptr.dtype, device=dev)
    nnz = C.c_int64(0)
    _rng["calls"] += 1
    check(lib.shmt_sample_hop_eids(_ctx(dev), _ptr(indptr), pdt, _ptr(indices), xdt, _ptr(gpu_indptr),
                                   _ptr(gpu_indices), _ptr(gpu_edge_base),
                                   hashmap._handle if hashmap is not None else None, _ptr(seeds), sdt, n, k,
                                   int(bool(replace)), _rng["seed"], _rng["calls"], sub_indptr.data_ptr(),
                                   _ptr(sub_indices), _ptr(sub_eids), C.byref(nnz), _stream(dev)))
    return sub_indptr, sub_indices[:nnz.value], sub_eids[:nnz.value]


def csr_weighted_sampling(indptr, indices, weights, seeds, num_picks: int, replace: bool, gpu_indptr=None,
                          gpu_indices=None, gpu_weights=None, hashmap: "CUCOStaticHashmap | None" = None,
                          gpu_edge_base=None, return_eids: bool = False):
    """Extension: one hop in which neighbours are picked with probabilities proportional to
    ``weights`` (float32, one per edge, parallel to ``indices``).  Without replacement (fan-out at
    most 32) this is sequential weighted sampling without replacement; with replacement the picks
    are independent.  Rows with ``deg <= num_picks`` are copied whole.  For a cached graph pass
    ``gpu_weights`` — ``create_subcsr(indptr, weights.view(torch.int32), cached_rows)[1]
    .view(torch.float32)`` makes them.  Returns ``(sub_indptr, sub_indices)`` or, with
    ``return_eids``, ``(sub_indptr, sub_indices, sub_eids)``.  The reference samples uniformly only."""
    _check_cuda(seeds, "seeds")
    seeds = seeds.contiguous()
    dev = seeds.device
    who = "csr_weighted_sampling"
    for t, nm in ((indptr, "indptr"), (indices, "indices"), (weights, "weights")):
        _check_contig(t, nm)
    if weights.dtype != torch.float32 or weights.numel() != indices.numel():
        raise RuntimeError(f"{who}: weights must be float32, one per edge")
    pdt, xdt, sdt = _int_code(indptr, who), _int_code(indices, who), _int_code(seeds, who)
    if hashmap is not None:
        for t, nm in ((gpu_indptr, "gpu_indptr"), (gpu_indices, "gpu_indices"), (gpu_weights, "gpu_weights")):
            if t is None:
                raise RuntimeError(f"{who}: a cached graph needs {nm}")
            _check_cuda(t, nm)
        if gpu_weights.dtype != torch.float32 or gpu_weights.numel() != gpu_indices.numel():
            raise RuntimeError(f"{who}: gpu_weights must be float32, one per cached edge")
        if return_eids and gpu_edge_base is None:
            raise RuntimeError(f"{who}: edge ids of a cached graph need gpu_edge_base")
    n, k = seeds.numel(), int(num_picks)
    sub_indptr = torch.empty(n + 1, dtype=indptr.dtype, device=dev)
    sub_indices = torch.empty(n * k, dtype=indices.dtype, device=dev)
    sub_eids = torch.empty(n * k, dtype=indptr.dtype, device=dev) if return_eids else None
    nnz = C.c_int64(0)
    _rng["calls"] += 1
    check(lib.shmt_sample_hop_weighted(_ctx(dev), _ptr(indptr), pdt, _ptr(indices), xdt, _ptr(weights),
                                       _ptr(gpu_indptr), _ptr(gpu_indices), _ptr(gpu_weights), _ptr(gpu_edge_base),
                                       hashmap._handle if hashmap is not None else None, _ptr(seeds), sdt, n, k,
                                       int(bool(replace)), _rng["seed"], _rng["calls"], sub_indptr.data_ptr(),
                                       _ptr(sub_indices), _ptr(sub_eids), C.byref(nnz), _stream(dev)))
    if return_eids:
        return sub_indptr, sub_indices[:nnz.value], sub_eids[:nnz.value]
    return sub_indptr, sub_indices[:nnz.value]


def sample_minibatch(indptr: torch.Tensor, indices: torch.Tensor, seeds: torch.Tensor,
                     fanouts: Sequence[int], replace: bool = False, gpu_indptr=None,
                     gpu_indices=None, hashmap: "CUCOStaticHashmap | None" = None,
                     gpu_edge_base=None, return_eids: bool = False, weights=None, gpu_weights=None):
    """Extension: all hops of a mini-batch in one native call (``shmt_sample_minibatch``).

    Equivalent to, for each ``k`` in ``fanouts`` in the given order::

        sub_indptr, sub_indices = csr_(cache_)sampling(..., seeds, k, replace)
        seeds, (_, relabel_indices) = tensor_relabel([seeds, sub_indices])

    but nothing is read back between hops; the host waits once.  Returns
    ``(frontier, hops)`` where ``hops[h] = (sub_indptr, sub_indices, relabel_indices,
    frontier_after_hop)``.  Seeds are converted to the dtype of ``indices``.  With ``return_eids``
    every hop's tuple ends with the edge ids of its sampled neighbours (positions in ``indices``,
    dtype of ``indptr``); a cached graph then needs ``gpu_edge_base`` (``subcsr_edge_base``).
    With ``weights`` (float32, one per edge; ``gpu_weights`` for the cached rows) every hop picks
    in proportion to them, as ``csr_weighted_sampling`` does (not together with ``return_eids``).
    """
    _check_cuda(seeds, "seeds")
    dev = seeds.device
    for t, nm in ((indptr, "indptr"), (indices, "indices")):
        _check_contig(t, nm)
    pdt, xdt = _int_code(indptr, "sample_minibatch"), _int_code(indices, "sample_minibatch")
    seeds = seeds.contiguous().to(indices.dtype)
    n_hops = len(fanouts)
    caps = [seeds.numel()]
    for k in fanouts:
        caps.append(caps[-1] * (1 + int(k)))
    # two allocations (one per dtype); the per-hop outputs are 16-byte aligned pieces of them,
    # handed to the library as raw addresses and turned into views only once sizes are known
    if return_eids and hashmap is not None and gpu_edge_base is None:
        raise RuntimeError("sample_minibatch: edge ids of a cached graph need gpu_edge_base")
    if weights is not None:
        if return_eids:
            raise RuntimeError("sample_minibatch: weights and return_eids cannot be combined")
        _check_contig(weights, "weights")
        if weights.dtype != torch.float32 or weights.numel() != indices.numel():
            raise RuntimeError("sample_minibatch: weights must be float32, one per edge")
        if hashmap is not None:
            if gpu_weights is None:
                raise RuntimeError("sample_minibatch: a cached graph needs gpu_weights")
            _check_cuda(gpu_weights, "gpu_weights")
            if gpu_weights.dtype != torch.float32 or gpu_weights.numel() != gpu_indices.numel():
                raise RuntimeError("sample_minibatch: gpu_weights must be float32, one per cached edge")
    key = (seeds.numel(), tuple(int(k) for k in fanouts), indptr.dtype, indices.dtype, bool(return_eids))
    layout = _minibatch_layouts.get(key)
    if layout is None:
        def plan(dtype, counts):
            item = _ITEMSIZE[dtype]
            step = 16 // item
            offs, lo = [], 0
            for c in counts:
                offs.append(lo)
                lo += -(-c // step) * step
            return offs + [lo], item
        p_off, p_item = plan(indptr.dtype, [caps[h] + 1 for h in range(n_hops)]
                             + ([caps[h] * int(fanouts[h]) for h in range(n_hops)] if return_eids else []))
        i_off, i_item = plan(indices.dtype, [caps[h] * int(fanouts[h]) for h in range(n_hops)]
                             + [caps[h + 1] for h in range(n_hops)] * 2)
        fan = (C.c_int64 * n_hops)(*[int(k) for k in fanouts])
        layout = _minibatch_layouts[key] = (p_off, p_item, i_off, i_item, fan)
    p_off, p_item, i_off, i_item, fan = layout
    p_pool = torch.empty(p_off[-1], dtype=indptr.dtype, device=dev)
    i_pool = torch.empty(i_off[-1], dtype=indices.dtype, device=dev)
    p_base, i_base = p_pool.data_ptr(), i_pool.data_ptr()
    VP = C.c_void_p * n_hops
    sizes = (C.c_int64 * (3 * n_hops))()
    offset = _rng["calls"] + 1
    _rng["calls"] += n_hops
    out_ptr = VP(*[p_base + p_off[h] * p_item for h in range(n_hops)])
    out_idx = VP(*[i_base + i_off[h] * i_item for h in range(n_hops)])
    out_rel = VP(*[i_base + i_off[n_hops + h] * i_item for h in range(n_hops)])
    out_front = VP(*[i_base + i_off[2 * n_hops + h] * i_item for h in range(n_hops)])
    map_handle = hashmap._handle if hashmap is not None else None
    if return_eids:
        out_eid = VP(*[p_base + p_off[n_hops + h] * p_item for h in range(n_hops)])
        check(lib.shmt_sample_minibatch_eids(
            _ctx(dev), _ptr(indptr), pdt, _ptr(indices), xdt, _ptr(gpu_indptr), _ptr(gpu_indices),
            _ptr(gpu_edge_base), map_handle, _ptr(seeds), seeds.numel(), fan, n_hops, int(bool(replace)),
            _rng["seed"], offset, out_ptr, out_idx, out_eid, out_rel, out_front, sizes, _stream(dev)))
    elif weights is not None:
        check(lib.shmt_sample_minibatch_weighted(
            _ctx(dev), _ptr(indptr), pdt, _ptr(indices), xdt, _ptr(weights), _ptr(gpu_indptr), _ptr(gpu_indices),
            _ptr(gpu_weights), map_handle, _ptr(seeds), seeds.numel(), fan, n_hops, int(bool(replace)),
            _rng["seed"], offset, out_ptr, out_idx, out_rel, out_front, sizes, _stream(dev)))
    else:
        check(lib.shmt_sample_minibatch(
            _ctx(dev), _ptr(indptr), pdt, _ptr(indices), xdt, _ptr(gpu_indptr), _ptr(gpu_indices),
            map_handle, _ptr(seeds), seeds.numel(), fan, n_hops, int(bool(replace)), _rng["seed"], offset,
            out_ptr, out_idx, out_rel, out_front, sizes, _stream(dev)))
    # one split per pool gives every exact-size view: per piece (skip, take, rest)
    cuts_p, cuts_i = [], [0] * (9 * n_hops)
    for h in range(n_hops):
        n_in, nnz, n_out = sizes[3 * h], sizes[3 * h + 1], sizes[3 * h + 2]
        room = p_off[h + 1] - p_off[h]
        cuts_p += [n_in + 1, room - n_in - 1]
        for piece, skip, take in ((h, 0, nnz), (n_hops + h, n_in, nnz), (2 * n_hops + h, 0, n_out)):
            room = i_off[piece + 1] - i_off[piece]
            cuts_i[3 * piece:3 * piece + 3] = [skip, take, room - skip - take]
    if return_eids:
        for h in range(n_hops):
            nnz = sizes[3 * h + 1]
            cuts_p += [nnz, p_off[n_hops + h + 1] - p_off[n_hops + h] - nnz]
    pv = p_pool.split_with_sizes(cuts_p)
    iv = i_pool.split_with_sizes(cuts_i)
    hops = [(pv[2 * h], iv[3 * h + 1], iv[3 * (n_hops + h) + 1], iv[3 * (2 * n_hops + h) + 1])
            + ((pv[2 * (n_hops + h)],) if return_eids else ())
            for h in range(n_hops)]
    return hops[-1][3], hops


def create_subcsr(uva_indptr: torch.Tensor, uva_indices: torch.Tensor, seeds: torch.Tensor):
    """src/cache_graph_sampling.cu:455-492 — compact GPU CSR of the rows ``seeds``, in order."""
    _check_cuda(seeds, "seeds")
    seeds = seeds.contiguous()
    dev = seeds.device
    _check_contig(uva_indptr, "uva_indptr")
    _check_contig(uva_indices, "uva_indices")
    pdt = _int_code(uva_indptr, "create_subcsr")
    xdt = _int_code(uva_indices, "create_subcsr")
    sdt = _int_code(seeds, "create_subcsr")
    n = seeds.numel()
    gpu_indptr = torch.empty(n + 1, dtype=uva_indptr.dtype, device=dev)
    nnz = C.c_int64(0)
    check(lib.shmt_subcsr_count(_ctx(dev), _ptr(uva_indptr), pdt, _ptr(seeds), sdt, n,
                                gpu_indptr.data_ptr(), C.byref(nnz), _stream(dev)))
    gpu_indices = torch.empty(nnz.value, dtype=uva_indices.dtype, device=dev)
    check(lib.shmt_subcsr_fill(_ptr(uva_indptr), pdt, _ptr(uva_indices), xdt, _ptr(seeds), sdt, n,
                               gpu_indptr.data_ptr(), _ptr(gpu_indices), _stream(dev)))
    return gpu_indptr, gpu_indices
