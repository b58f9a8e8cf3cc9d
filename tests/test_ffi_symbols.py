"""The C-ABI library loads and exports exactly what include/m3scan.h declares
(no compute: this runs without a GPU)."""
import ctypes
import re
from pathlib import Path

from mamba_trainer_b200 import _ffi, build

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "m3scan.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return set(re.findall(r"\b(m3_[a-z0-9_]+)\s*\(", text))


def test_header_and_binding_agree():
    assert declared_symbols() == set(_ffi.SYMBOLS)


def test_library_builds_loads_and_exports_every_symbol():
    build.build()
    lib = _ffi.load()
    for name in declared_symbols():
        assert hasattr(lib, name), name
    assert lib.m3_version().decode().count(".") == 2


def test_struct_layouts_match_the_header():
    # 12 int32 then 14 pointers; 4, 4 and 14 pointers.
    assert ctypes.sizeof(_ffi.ScanDesc) == 12 * 4 + 14 * 8
    assert ctypes.sizeof(_ffi.ScanOut) == 4 * 8
    assert ctypes.sizeof(_ffi.ScanBwdIn) == 4 * 8
    assert ctypes.sizeof(_ffi.ScanGrads) == 14 * 8


def test_scratch_size_query_needs_no_gpu():
    lib = _ffi.load()
    d = _ffi.ScanDesc(batch=2, seq=256, heads=4, head_dim=64, d_state=64, rank=1, chunk=64, dtype=0,
                      discretization=0, dynamics=0, want_state=1, path=0)
    fwd = lib.m3_scan_scratch_bytes(ctypes.byref(d), 0)
    both = lib.m3_scan_scratch_bytes(ctypes.byref(d), 1)
    assert 0 < fwd < both
