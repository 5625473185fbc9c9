"""Build the oracle's native pieces (test / bench infrastructure, not product code).

* ``oracle/liboracle_cpu.so`` — g++ -O3 -fopenmp build of ``oracle/cpu_ops.cc``, the threaded
  CPU restatement that ``bench.py`` times as the CPU baseline.

    python oracle/build_oracle.py
"""
from __future__ import annotations

import ctypes as C
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CPU_LIB = HERE / "liboracle_cpu.so"


def build_cpu(force: bool = False) -> Path:
    src = HERE / "cpu_ops.cc"
    if force or not CPU_LIB.exists() or CPU_LIB.stat().st_mtime < src.stat().st_mtime:
        # no -march=native: the library is built on one machine and may run on another
        cmd = ["g++", "-O3", "-fopenmp", "-shared", "-fPIC", "-o", str(CPU_LIB), str(src)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"g++ failed on cpu_ops.cc:\n{res.stderr}")
    return CPU_LIB


def load_cpu() -> C.CDLL:
    lib = C.CDLL(str(build_cpu()))
    vp, i64, i, u64 = C.c_void_p, C.c_int64, C.c_int, C.c_uint64
    lib.oracle_num_threads.restype = i
    lib.oracle_set_threads.restype = None
    lib.oracle_set_threads.argtypes = [i]
    import os
    lib.oracle_set_threads(len(os.sched_getaffinity(0)))  # whatever OMP_NUM_THREADS the launcher exported
    lib.oracle_gather.restype = None
    lib.oracle_gather.argtypes = [vp, vp, i64, i64, vp]
    lib.oracle_sample_hop.restype = i64
    lib.oracle_sample_hop.argtypes = [vp, vp, i, vp, i64, i64, i, u64, vp, vp]
    lib.oracle_map_build_query.restype = i64
    lib.oracle_map_build_query.argtypes = [vp, i64, vp, i64, vp, i64, vp]
    lib.oracle_scatter.restype = None
    lib.oracle_scatter.argtypes = [vp, vp, i64, i64, vp]
    lib.oracle_relabel.restype = i64
    lib.oracle_relabel.argtypes = [vp, i64, vp, vp]
    return lib


if __name__ == "__main__":
    print(build_cpu(force=True))
