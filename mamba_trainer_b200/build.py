"""Build libm3scan.so (the C-ABI library) in-tree with nvcc for sm_100a.

    python -m mamba_trainer_b200.build [--force] [--verbose]

The library has no PyTorch dependency: it is plain CUDA behind `extern "C"`.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libm3scan.so"
SOURCES = ["m3_api.cu", "m3_generic_fwd.cu", "m3_generic_bwd.cu", "m3_noalloc.cu", "m3_tc_fwd.cu", "m3_tc_fwd_direct.cu", "m3_tc_bwd.cu", "m3_tc_bwd_direct.cu", "m3_step.cu",
           "m3_host_pipe.cu", "m3_conv.cu", "m3_mixer.cu", "m3_reduce.cu"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; libm3scan cannot be built")


def _stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))
    deps.append(PKG.parent / "include" / "m3scan.h")
    return any(p.stat().st_mtime > t for p in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every CUDA source into one shared library; returns its path."""
    if not force and not _stale():
        return LIB
    objdir = PKG / "build"
    objdir.mkdir(exist_ok=True)
    nvcc = _nvcc()
    common = [
        "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
        "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
    ]
    if verbose:
        common += ["-Xptxas", "-v"]
    procs = []
    objs = []
    for src in SOURCES:
        obj = objdir / (src + ".o")
        objs.append(str(obj))
        cmd = [nvcc, *common, "-c", str(CSRC / src), "-o", str(obj)]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode:
            sys.stderr.write(out)
        if p.returncode:
            raise RuntimeError(f"nvcc failed on {src}")
    link = [nvcc, "-shared", "-o", str(LIB), *objs, "-lcudart"]
    subprocess.run(link, check=True)
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
