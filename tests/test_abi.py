"""The C-ABI library loads and exports everything include/shmt.h declares (CPU only)."""
import ctypes as C
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def _declared():
    text = (ROOT / "include" / "shmt.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(shmt_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound():
    from shmtensor_b200 import _lib
    names = _declared()
    assert len(names) >= 35
    for n in names:
        assert hasattr(_lib.lib, n), f"{n} declared in shmt.h but not exported"
    assert sorted(_lib.SIGNATURES) == names, "ctypes table and header disagree"


def test_no_torch_symbols_in_the_library():
    import subprocess
    out = subprocess.run(["nm", "-D", "--undefined-only", str(ROOT / "shmtensor_b200" / "libshmt.so")],
                         capture_output=True, text=True).stdout
    assert "c10" not in out and "torch" not in out and "pybind" not in out


def test_invalid_arguments_return_status_not_crash():
    from shmtensor_b200 import _lib
    lib = _lib.lib
    assert lib.shmt_version() >= 100
    assert lib.shmt_scan(None, None, 0, 10, 0, None) == _lib.ERR_INVALID
    assert "ctx is null" in _lib.last_error()
    assert lib.shmt_fetch(None, None, 0, None, None, None, 7, 4, 16, None, None) == _lib.ERR_INVALID
    assert "int32 or int64" in _lib.last_error()
    assert lib.shmt_fetch(None, None, 0, None, None, None, 1, 0, 16, None, None) == _lib.OK  # n == 0
    assert lib.shmt_fetch(None, None, 0, None, None, None, 1, 4, 0, None, None) == _lib.ERR_INVALID
    assert lib.shmt_map_query(None, None, 0, 1, None, None) == _lib.ERR_INVALID
    assert lib.shmt_map_table_bytes(1000, 0) >= 1000 * 16
    assert lib.shmt_map_table_bytes(1000, 800) >= 1600 * 16
    p, fd = C.c_int64(), C.c_int64()
    assert lib.shmt_shm_open(b"/shmt_does_not_exist", 64, 0, C.byref(p), C.byref(fd)) == _lib.ERR_OS
    assert "fail to open" in _lib.last_error()
    with pytest.raises(_lib.ShmtError) as e:
        _lib.check(lib.shmt_relabel(None, None, None, 0, 0, None, None, None, None))
    assert e.value.code == _lib.ERR_INVALID


def test_product_never_imports_the_oracle():
    for f in (ROOT / "shmtensor_b200").rglob("*.py"):
        src = f.read_text()
        assert "oracle" not in src, f"{f} mentions the oracle"
    for f in (ROOT / "shmtensor_b200" / "csrc").iterdir():
        assert "oracle" not in f.read_text()
