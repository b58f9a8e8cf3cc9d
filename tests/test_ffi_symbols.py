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


def test_struct_layouts_match_the_header(tmp_path):
    """Sizes and field offsets of every structure, as a C compiler lays out include/m3scan.h,
    against the ctypes mirrors."""
    import subprocess
    pairs = [("m3_scan_desc", _ffi.ScanDesc, {"lambda": "lambda_"}), ("m3_scan_out", _ffi.ScanOut, {}),
             ("m3_scan_bwd_in", _ffi.ScanBwdIn, {}), ("m3_scan_grads", _ffi.ScanGrads, {}),
             ("m3_step_desc", _ffi.StepDesc, {"lambda": "lambda_"}), ("m3_step_out", _ffi.StepOut, {}),
             ("m3_host_in", _ffi.HostIn, {"lambda": "lambda_"}), ("m3_host_out", _ffi.HostOut, {}),
             ("m3_conv_desc", _ffi.ConvDesc, {}), ("m3_bc_desc", _ffi.BcDesc, {}),
             ("m3_act_desc", _ffi.ActDesc, {}), ("m3_gate_desc", _ffi.GateDesc, {}),
             ("m3_gate_norm_desc", _ffi.GateNormDesc, {})]
    inv = lambda ren: {v: k for k, v in ren.items()}
    lines = ["#include <stdio.h>", "#include <stddef.h>", f'#include "{ROOT / "include" / "m3scan.h"}"', "int main(void) {"]
    for cname, mirror, ren in pairs:
        lines.append(f'  printf("{cname} size %zu\\n", sizeof({cname}));')
        for fname, _ in mirror._fields_:
            cf = inv(ren).get(fname, fname)
            lines.append(f'  printf("{cname} {fname} %zu\\n", offsetof({cname}, {cf}));')
    lines += ["  return 0;", "}"]
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-std=c99", "-o", str(exe), str(src)], check=True)
    got = {}
    for ln in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.splitlines():
        cname, field, val = ln.split()
        got[(cname, field)] = int(val)
    for cname, mirror, _ in pairs:
        assert got[(cname, "size")] == ctypes.sizeof(mirror), cname
        for fname, _ in mirror._fields_:
            assert got[(cname, fname)] == getattr(mirror, fname).offset, (cname, fname)
    assert ctypes.sizeof(_ffi.ScanDesc) == 14 * 4 + 14 * 8


def test_scratch_size_query_needs_no_gpu():
    lib = _ffi.load()
    d = _ffi.ScanDesc(batch=2, seq=256, heads=4, head_dim=64, d_state=64, rank=1, chunk=64, dtype=0,
                      discretization=0, dynamics=0, want_state=1, path=0)
    fwd = lib.m3_scan_scratch_bytes(ctypes.byref(d), 0)
    both = lib.m3_scan_scratch_bytes(ctypes.byref(d), 1)
    assert 0 < fwd < both


def test_rust_sys_source_covers_the_header():
    """include/m3scan-sys/src/lib.rs (uncompiled here: the image has no Rust toolchain) declares every function
    of the header and nothing else, and lists every structure's fields in the header's order."""
    rs = (ROOT / "include" / "m3scan-sys" / "src" / "lib.rs").read_text()
    assert set(re.findall(r"pub fn (m3_[a-z0-9_]+)\s*\(", rs)) == declared_symbols()
    header = re.sub(r"/\*.*?\*/", "", (ROOT / "include" / "m3scan.h").read_text(), flags=re.S)
    for body, name in re.findall(r"typedef struct \{(.*?)\}\s*(m3_[a-z_]+);", header, flags=re.S):
        c_fields = []
        for decl in body.split(";"):
            decl = decl.strip()
            if not decl:
                continue
            for part in decl.split(","):
                c_fields.append(re.sub(r"\[\d+\]", "", part.strip().split()[-1].lstrip("*")))
        m = re.search(r"pub struct %s \{(.*?)\n\}" % name, rs, flags=re.S)
        assert m, name
        rs_fields = re.findall(r"pub ([a-z_0-9]+):", re.sub(r"//.*", "", m.group(1)))
        assert rs_fields == c_fields, name
