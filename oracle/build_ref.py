"""Compile the reference's own sources into ``oracle/_ref/ShmTensorLib.so``.

TEST AND BENCH INFRASTRUCTURE.  The sources are compiled where they lie (the reference checkout
named by the environment variable ``SHMT_REFERENCE_DIR`` or the first command-line argument,
unmodified; nothing is copied into this repository) with nvcc for sm_100a, against this
image's torch headers and ``oracle/ref_shim`` — a stand-in for the one header the reference's
build downloads (cuCollections, see ``oracle/ref_shim/cuco/static_map.cuh``).  The reference's
own build system (CMake + CPM download) is not run.  Output goes only to ``oracle/_ref/``
(git-ignored; it travels to the GPU box with the repository snapshot).

    SHMT_REFERENCE_DIR=<checkout of gpzlx1/ShmTensor> python oracle/build_ref.py
    python oracle/build_ref.py <checkout> [--force]      # about 5 minutes on 8 cores (torch headers)

Without a checkout an earlier build in ``oracle/_ref/`` is used as it is.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent


def reference_dir() -> Path | None:
    """The reference checkout to compile from: SHMT_REFERENCE_DIR, else a sibling directory named
    ``reference`` next to this repository; None if neither exists."""
    named = os.environ.get("SHMT_REFERENCE_DIR")
    for cand in ([Path(named)] if named else []) + [HERE.parent.parent / "reference"]:
        if (cand / "src" / "pybind.cc").exists():
            return cand
    return None


OUT_DIR = HERE / "_ref"
OUT = OUT_DIR / "ShmTensorLib.so"
SOURCES = ["src/pybind.cc", "src/cuco_hashmap.cu", "src/cache_feature_fetch.cu",
           "src/cache_feature_set.cu", "src/cache_graph_sampling.cu", "src/tensor_relabel.cu",
           "src/thrust_scan.cu", "src/mmap_tensor.cc", "src/cnpy.cc"]


def build_reference(force: bool = False, reference: Path | None = None) -> Path | None:
    REFERENCE = Path(reference) if reference else reference_dir()
    if REFERENCE is None:
        return OUT if OUT.exists() else None
    if OUT.exists() and not force:
        return OUT
    for stale in ([OUT] if OUT.exists() else []):
        stale.unlink()
    import torch
    from torch.utils import cpp_extension as ce
    OUT_DIR.mkdir(exist_ok=True)
    obj_dir = OUT_DIR / "obj"
    obj_dir.mkdir(exist_ok=True)
    inc = [str(HERE / "ref_shim"), str(REFERENCE / "include"), sysconfig.get_paths()["include"]]
    inc += ce.include_paths(device_type="cuda") if "device_type" in ce.include_paths.__code__.co_varnames \
        else ce.include_paths(cuda=True)
    flags = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
             "--expt-extended-lambda", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-w",
             "-DTORCH_EXTENSION_NAME=ShmTensorLib", "-DTORCH_API_INCLUDE_EXTENSION_H",
             f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}", "-x", "cu"]
    for i in inc:
        flags += ["-I", i]

    shim_time = max(f.stat().st_mtime for f in (HERE / "ref_shim").rglob("*") if f.is_file())

    def compile_one(rel: str) -> str:
        src = REFERENCE / rel
        obj = obj_dir / (src.stem + ".o")
        if obj.exists() and obj.stat().st_mtime > max(src.stat().st_mtime, shim_time):
            return str(obj)  # objects are kept between runs; a torch-including file takes minutes
        res = subprocess.run(["nvcc", *flags, "-c", str(src), "-o", str(obj)], capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed on {rel}:\n{res.stderr[-4000:]}")
        return str(obj)

    with ThreadPoolExecutor(max_workers=8) as pool:
        objs = list(pool.map(compile_one, SOURCES))
    lib_dir = str(Path(torch.__file__).parent / "lib")
    link = ["nvcc", "-shared", "-o", str(OUT), *objs, "-L", lib_dir, "-Xlinker", f"-rpath={lib_dir}",
            "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda", "-ltorch_python", "-lrt"]
    res = subprocess.run(link, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stderr[-4000:]}")
    return OUT


def load_reference():
    """Import the compiled reference module, or None if it has not been built."""
    if not OUT.exists():
        return None
    import importlib.util
    import torch  # noqa: F401  the extension needs torch's libraries loaded first
    spec = importlib.util.spec_from_file_location("ShmTensorLib", str(OUT))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    paths = [a for a in sys.argv[1:] if not a.startswith("--")]
    print(build_reference(force="--force" in sys.argv, reference=Path(paths[0]) if paths else None))
