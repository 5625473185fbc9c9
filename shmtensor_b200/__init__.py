"""shmtensor_b200 — the GPU-cache hot path of gpzlx1/ShmTensor rebuilt for B200 (sm_100a).

``capi`` mirrors the reference's ``ShmTensorLib`` module; ``ShmTensor``, ``DiskTensor`` and
``GPUSamplingDataloader`` mirror its ``shmtensor`` package (python/shmtensor/__init__.py:1-4).
``install_dropin()`` registers both under the reference's import names.

Attributes load on first use, so ``python -m shmtensor_b200.build`` can (re)build the CUDA
library before anything tries to open it.
"""
import importlib

__all__ = ["capi", "ShmTensor", "DiskTensor", "GPUSamplingDataloader", "PartitionedFeatureCache",
           "GraphCache", "install_dropin"]

_LAZY = {
    "capi": ("shmtensor_b200.capi", None),
    "ShmTensor": ("shmtensor_b200.host_tensors", "ShmTensor"),
    "DiskTensor": ("shmtensor_b200.host_tensors", "DiskTensor"),
    "GPUSamplingDataloader": ("shmtensor_b200.dataloader", "GPUSamplingDataloader"),
    "PartitionedFeatureCache": ("shmtensor_b200.partition", "PartitionedFeatureCache"),
    "GraphCache": ("shmtensor_b200.graph_cache", "GraphCache"),
}


def __getattr__(name):
    try:
        module, attr = _LAZY[name]
    except KeyError:
        raise AttributeError(f"module 'shmtensor_b200' has no attribute {name!r}") from None
    mod = importlib.import_module(module)
    value = mod if attr is None else getattr(mod, attr)
    globals()[name] = value
    return value


def install_dropin() -> None:
    """Make ``import ShmTensorLib`` and ``import shmtensor`` resolve to this package, so
    scripts written against the reference run unchanged."""
    import sys
    import types

    capi = __getattr__("capi")
    sys.modules.setdefault("ShmTensorLib", capi)
    if "shmtensor" not in sys.modules:
        mod = types.ModuleType("shmtensor")
        mod.capi = capi
        for name in ("ShmTensor", "DiskTensor", "GPUSamplingDataloader"):
            setattr(mod, name, __getattr__(name))
        sys.modules["shmtensor"] = mod
