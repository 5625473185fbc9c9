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

    Rank 0 of ``local_group`` creates the segment while the others wait at a barrier, then
    they open it.  With ``pin_memory`` every rank registers its mapping with CUDA so kernels
    can dereference it (UVA).  The segment is unmapped and unlinked when the object dies.
    """

    def __init__(self, name, shape, local_rank, local_world_size, local_group=None,
                 dtype=torch.float32, pin_memory=False):
        nbytes = torch.empty((), dtype=dtype).element_size() * math.prod(shape)
        if nbytes <= 0:
            raise Exception("Invalid shape")
        self.name, self.shape_, self.dtype_ = name, shape, dtype
        self.pin_memory_ = pin_memory
        self.cur_rank, self.cur_world_size, self.cur_group = local_rank, local_world_size, local_group
        self.size_ = nbytes

        if capi.file_exist(name):
            raise Exception("File name is already exist")
        dist.barrier(local_group)  # nobody creates before everybody has looked

        creator = local_rank == 0
        if creator:
            self.ptr_, self.fd_ = capi.create_shared_mem(name, nbytes, pin_memory)
        dist.barrier(local_group)  # segment exists from here on
        if not creator:
            self.ptr_, self.fd_ = capi.open_shared_mem(name, nbytes, pin_memory)

        # arguments only, no reference to self, or the object would never be collected
        self._shm_finalizer = weakref.finalize(self, capi.release_shared_mem, name, nbytes,
                                               self.ptr_, self.fd_, pin_memory)
        self.tensor_ = capi.open_shared_tensor(self.ptr_, dtype, shape)


class DiskTensor(_HostTensorView):
    """A ``.npy`` file mapped read/write (``MAP_SHARED``): writes through the tensor reach the
    file.  With ``pin_memory`` the whole mapping is registered with CUDA."""

    def __init__(self, filename, pin_memory=False):
        assert os.path.exists(filename)
        assert filename.endswith('.npy')
        self.filename_, self.pin_memory_ = filename, pin_memory
        self.tensor_, self.size_, self.ptr_, self.fd_ = capi.open_mmap_tensor(filename, pin_memory)
        self._disk_finalizer = weakref.finalize(self, capi.close_mmap_tensor, self.size_,
                                                self.ptr_, self.fd_, pin_memory)
