"""Host-resident tensors that GPU kernels read in place: ``ShmTensor`` and ``DiskTensor``.

Same constructor arguments, attributes (``tensor_``, ``ptr_``, ``fd_``, ``size_`` ...) and
life cycle as the reference's python/shmtensor/shm_tensor.py:19-88 and
python/shmtensor/disk_tensor.py:8-47, so scripts written against them keep working.
"""
from __future__ import annotations

import math
import os
import weakref

import torch
import torch.distributed as dist

from . import capi


class _HostTensorView:
    """What both kinds expose: the mapped tensor and pass-through metadata."""

    tensor_: torch.Tensor

    shape = property(lambda self: self.tensor_.shape)
    dtype = property(lambda self: self.tensor_.dtype)
    device = property(lambda self: self.tensor_.device)
    size = property(lambda self: self.tensor_.size)


class ShmTensor(_HostTensorView):
    """A tensor in a named POSIX shared-memory segment shared by the ranks of one node.

    Rank 0 of ``local_group`` creates the segment while the others wait, then they open it.
    With ``pin_memory`` every rank registers its mapping with CUDA so kernels can dereference it
    (UVA).  The segment is unmapped and unlinked when the object dies.

    Beyond the reference's constructor: the segment is created with ``O_EXCL`` (the reference
    tests ``file_exist`` on every rank and creates afterwards, so two jobs can both pass the
    test); ``overwrite_stale=True`` removes a segment of that name first, which is what a job
    wants whose previous run was killed before its finalizer ran; ``numa`` places the pages
    before anything is written: ``"interleave"`` over all memory nodes, or a node number.  A
    failure of the creating rank reaches every rank as an exception instead of a hang.
    """

    def __init__(self, name, shape, local_rank, local_world_size, local_group=None,
                 dtype=torch.float32, pin_memory=False, overwrite_stale=False, numa=None):
        nbytes = torch.empty((), dtype=dtype).element_size() * math.prod(shape)
        if nbytes <= 0:
            raise Exception("Invalid shape")
        self.name, self.shape_, self.dtype_ = name, shape, dtype
        self.pin_memory_ = pin_memory
        self.cur_rank, self.cur_world_size, self.cur_group = local_rank, local_world_size, local_group
        self.size_ = nbytes

        creator = local_rank == 0
        error = None
        if creator:
            try:
                if overwrite_stale:
                    capi.unlink_shared_mem(name)
                # registration waits until the pages are placed (a pinned page cannot move)
                self.ptr_, self.fd_ = capi.create_shared_mem(name, nbytes, False, exclusive=True)
                if numa is not None:
                    if numa == "interleave":
                        capi.numa_place(self.ptr_, nbytes, capi.NUMA_INTERLEAVE)
                    else:
                        capi.numa_place(self.ptr_, nbytes, capi.NUMA_BIND, int(numa))
                if pin_memory and nbytes >= (1 << 28):
                    capi.prefault(self.ptr_, nbytes)  # pages present before anyone pins them
            except Exception as exc:  # noqa: BLE001  told to every rank below
                error = "File name is already exist" if "already exists" in str(exc) else str(exc)
        error = self._agree(error, local_group)
        if error is not None:
            raise Exception(error)
        # every rank pins its own mapping, all at the same time
        if creator:
            if pin_memory:
                capi._register_range(self.ptr_, nbytes)
        else:
            self.ptr_, self.fd_ = capi.open_shared_mem(name, nbytes, pin_memory)

        # arguments only, no reference to self, or the object would never be collected
        self._shm_finalizer = weakref.finalize(self, capi.release_shared_mem, name, nbytes,
                                               self.ptr_, self.fd_, pin_memory)
        self.tensor_ = capi.open_shared_tensor(self.ptr_, dtype, shape)

    @staticmethod
    def _agree(error, group):
        """The creating rank's outcome, on every rank (also the point the others wait at)."""
        if not (dist.is_available() and dist.is_initialized()):
            return error
        src = dist.get_global_rank(group, 0) if group is not None else 0
        box = [error]
        dist.broadcast_object_list(box, src=src, group=group)
        return box[0]


class DiskTensor(_HostTensorView):
    """A ``.npy`` file mapped read/write (``MAP_SHARED``): writes through the tensor reach the
    file.  With ``pin_memory`` the whole mapping is registered with CUDA.  ``read_only=True``
    (not in the reference, which maps read/write only) opens and maps the file without write
    permission, for datasets on read-only media or shared between jobs."""

    def __init__(self, filename, pin_memory=False, read_only=False):
        assert os.path.exists(filename)
        assert filename.endswith('.npy')
        self.filename_, self.pin_memory_, self.read_only_ = filename, pin_memory, read_only
        self.tensor_, self.size_, self.ptr_, self.fd_ = capi.open_mmap_tensor(filename, pin_memory,
                                                                              read_only)
        self._disk_finalizer = weakref.finalize(self, capi.close_mmap_tensor, self.size_,
                                                self.ptr_, self.fd_, pin_memory)
