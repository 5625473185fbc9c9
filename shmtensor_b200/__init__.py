"""shmtensor_b200 — the GPU-cache hot path of gpzlx1/ShmTensor rebuilt for B200 (sm_100a).

``capi`` mirrors the reference's ``ShmTensorLib`` module; ``ShmTensor``, ``DiskTensor`` and
``GPUSamplingDataloader`` mirror its ``shmtensor`` package (python/shmtensor/__init__.py:1-4).
``install_dropin()`` registers both under the reference's import names.
"""
from . import capi
from .dataloader import GPUSamplingDataloader
from .host_tensors import DiskTensor, ShmTensor

__all__ = ["capi", "ShmTensor", "DiskTensor", "GPUSamplingDataloader", "install_dropin"]


def install_dropin() -> None:
    """Make ``import ShmTensorLib`` and ``import shmtensor`` resolve to this package, so
    scripts written against the reference run unchanged."""
    import sys
    import types

    sys.modules.setdefault("ShmTensorLib", capi)
    if "shmtensor" not in sys.modules:
        mod = types.ModuleType("shmtensor")
        mod.capi, mod.ShmTensor, mod.DiskTensor = capi, ShmTensor, DiskTensor
        mod.GPUSamplingDataloader = GPUSamplingDataloader
        sys.modules["shmtensor"] = mod
