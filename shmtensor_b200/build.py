"""Build ``libshmt.so`` (the CUDA kernels + C-ABI) in-tree with nvcc for sm_100a.

No torch headers are involved, so a full build takes seconds.  Objects are
rebuilt only when a source or header is newer than the object.

    python -m shmtensor_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
INCLUDE = PKG_DIR.parent / "include"
BUILD_DIR = PKG_DIR / "build"
LIB_PATH = PKG_DIR / "libshmt.so"

SOURCES = ["ctx.cu", "map.cu", "fetch_set.cu", "scan.cu", "relabel.cu", "sample.cu", "p2p.cu",
           "host_mem.cc"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found: libshmt.so cannot be built")


def _newest_header() -> float:
    hdrs = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(INCLUDE.glob("*.h"))
    return max(h.stat().st_mtime for h in hdrs)


def build(force: bool = False, verbose: bool = False, extra_flags: list[str] | None = None,
          out: Path | None = None) -> Path:
    """Compile every source for sm_100a and link ``libshmt.so``; returns its path.

    ``out`` names another output library (with its own object directory), for building a
    variant with ``extra_flags`` next to the installed one.
    """
    nvcc = _nvcc()
    LIB_PATH = Path(out) if out else globals()["LIB_PATH"]
    BUILD_DIR = LIB_PATH.parent / ("build_" + LIB_PATH.stem) if out else globals()["BUILD_DIR"]
    BUILD_DIR.mkdir(exist_ok=True, parents=True)
    hdr_time = _newest_header()
    flags = NVCC_FLAGS + ["-I", str(INCLUDE), "-I", str(CSRC)] + (extra_flags or [])
    if verbose:
        flags += ["-Xptxas", "-v"]

    def compile_one(name: str) -> tuple[Path, bool]:
        src = CSRC / name
        obj = BUILD_DIR / (src.stem + ".o")
        stale = force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_time)
        if stale:
            cmd = [nvcc, *flags, "-c", str(src), "-o", str(obj)]
            res = subprocess.run(cmd, capture_output=True, text=True)
            if res.returncode != 0:
                raise RuntimeError(f"nvcc failed on {name}:\n{res.stdout}\n{res.stderr}")
            if verbose:
                sys.stderr.write(res.stderr)
        return obj, stale

    with ThreadPoolExecutor(max_workers=min(8, len(SOURCES))) as pool:
        results = list(pool.map(compile_one, SOURCES))
    objs = [str(o) for o, _ in results]
    if force or any(stale for _, stale in results) or not LIB_PATH.exists():
        cmd = [nvcc, "-shared", "-o", str(LIB_PATH), *objs, "-lrt"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
