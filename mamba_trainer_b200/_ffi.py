"""ctypes binding of libm3scan.so - the same declarations a Rust `-sys` crate would carry.

The structures mirror include/m3scan.h field for field.  Loading fails loudly when the
library has not been built: there is no CPU or eager fallback behind this module.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent / "libm3scan.so"

# m3_status
OK, ERR_SHAPE, ERR_RANK, ERR_CONFIG, ERR_UNSUPPORTED, ERR_CUDA, ERR_TIMEOUT, ERR_NULL = range(8)
# m3_dtype
F32, BF16 = 0, 1
# m3_path
PATH_AUTO, PATH_GENERIC, PATH_TENSOR = 0, 1, 2

GRAD_X, GRAD_B, GRAD_C, GRAD_DT, GRAD_A_LOG, GRAD_LAMBDA, GRAD_THETA, GRAD_D_SKIP, \
    GRAD_H0, GRAD_LAST_U0, GRAD_ANGLE0 = (1 << i for i in range(11))
GRAD_ALL = 0x7FF
NOALLOC_SCRATCH_BYTES = 16 << 20   # M3_NOALLOC_SCRATCH_BYTES


class ScanDesc(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "batch", "seq", "heads", "head_dim", "d_state", "rank", "chunk", "dtype",
        "discretization", "dynamics", "want_state", "path", "reverse_heads", "reserved0")] + [
        (n, C.c_void_p) for n in (
            "x", "b", "c", "dt", "lambda_", "theta", "a_log", "d_skip", "h0", "last_u0", "angle0",
            "a_raw", "g_raw", "w_raw")]


class ScanOut(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("y", "h", "last_u", "angle")]


class ScanBwdIn(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("dy", "dh", "dlast_u", "dangle")]


class ScanGrads(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in (
        "dx", "db", "dc", "ddt", "dlambda", "dtheta", "da_log", "dd_skip", "dh0", "dlast_u0", "dangle0",
        "da_raw", "dg_raw", "dw_raw")]


class StepDesc(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("batch", "heads", "head_dim", "d_state", "rank", "dtype",
                                         "discretization", "dynamics")] + [(n, C.c_void_p) for n in (
        "x", "b", "c", "dt", "lambda_", "theta", "a_log", "d_skip", "h", "last_u", "angle")]


class StepOut(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("y", "h", "last_u", "angle")]


class ConvDesc(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("batch", "seq", "channels", "kernel_size", "dtype", "activation")] + [
        ("x_stride", C.c_int64), ("y_stride", C.c_int64)] + [(n, C.c_void_p) for n in ("x", "history", "weight", "bias")] + [
        ("split", C.c_int32), ("reserved0", C.c_int32), ("y2_stride", C.c_int64), ("y2", C.c_void_p), ("dy2", C.c_void_p),
        ("n_reversed", C.c_int32), ("reversed_lo", C.c_int32 * 4), ("reversed_hi", C.c_int32 * 4), ("reserved1", C.c_int32)]


class BcDesc(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("batch", "seq", "heads", "groups", "d_state", "rank", "dtype", "has_norm")] + [
        ("eps", C.c_float), ("reserved0", C.c_int32), ("raw_stride", C.c_int64)] + [
        (n, C.c_void_p) for n in ("b_raw", "c_raw", "b_bias", "c_bias", "norm_weight")]


class ActDesc(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("batch", "seq", "heads", "dtype")] + [("stride", C.c_int64)] + [
        (n, C.c_void_p) for n in ("dt_raw", "lambda_raw", "dt_bias")]


class GateDesc(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("batch", "seq", "channels", "dtype")] + [("z_stride", C.c_int64)] + [
        (n, C.c_void_p) for n in ("y", "z")]


class GateNormDesc(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("batch", "seq", "channels", "dtype")] + [("z_stride", C.c_int64)] + [
        (n, C.c_void_p) for n in ("y", "z", "weight")] + [("eps", C.c_float)]


class HostIn(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("x", "b", "c", "dt", "lambda_", "theta", "dy")]


class HostOut(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("y", "dx", "db", "dc", "ddt", "dlambda", "dtheta", "da_log", "dd_skip")]


# name -> (restype, argtypes); every symbol include/m3scan.h declares.
SYMBOLS = {
    "m3_version": (C.c_char_p, []),
    "m3_ctx_create": (C.c_int, [C.c_int, C.POINTER(C.c_void_p)]),
    "m3_ctx_destroy": (C.c_int, [C.c_void_p]),
    "m3_ctx_set_stream": (C.c_int, [C.c_void_p, C.c_void_p]),
    "m3_sync": (C.c_int, [C.c_void_p]),
    "m3_ctx_set_wait_limit": (C.c_int, [C.c_void_p, C.c_uint32]),
    "m3_last_error": (C.c_char_p, [C.c_void_p]),
    "m3_launch_count": (C.c_uint64, [C.c_void_p]),
    "m3_alloc": (C.c_int, [C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p)]),
    "m3_free": (C.c_int, [C.c_void_p, C.c_void_p]),
    "m3_upload": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]),
    "m3_download": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]),
    "m3_scan_forward": (C.c_int, [C.c_void_p, C.POINTER(ScanDesc), C.POINTER(ScanOut), C.POINTER(C.c_void_p)]),
    "m3_scan_backward": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(ScanBwdIn), C.c_uint32, C.POINTER(ScanGrads)]),
    "m3_saved_free": (C.c_int, [C.c_void_p, C.c_void_p]),
    "m3_scan_scratch_bytes": (C.c_size_t, [C.POINTER(ScanDesc), C.c_int]),
    "m3_step_forward": (C.c_int, [C.c_void_p, C.POINTER(StepDesc), C.POINTER(StepOut)]),
    "m3_scan_forward_noalloc": (C.c_int, [C.c_void_p, C.POINTER(ScanDesc), C.POINTER(ScanOut)]),
    "m3_conv_forward": (C.c_int, [C.c_void_p, C.POINTER(ConvDesc), C.c_void_p, C.c_void_p]),
    "m3_conv_backward": (C.c_int, [C.c_void_p, C.POINTER(ConvDesc), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                   C.c_void_p]),
    "m3_bc_forward": (C.c_int, [C.c_void_p, C.POINTER(BcDesc), C.c_void_p, C.c_void_p]),
    "m3_bc_backward": (C.c_int, [C.c_void_p, C.POINTER(BcDesc)] + [C.c_void_p] * 7),
    "m3_dt_lambda_forward": (C.c_int, [C.c_void_p, C.POINTER(ActDesc), C.c_void_p, C.c_void_p]),
    "m3_dt_lambda_backward": (C.c_int, [C.c_void_p, C.POINTER(ActDesc)] + [C.c_void_p] * 5),
    "m3_gate_forward": (C.c_int, [C.c_void_p, C.POINTER(GateDesc), C.c_void_p]),
    "m3_gate_backward": (C.c_int, [C.c_void_p, C.POINTER(GateDesc), C.c_void_p, C.c_void_p, C.c_void_p]),
    "m3_gate_norm_forward": (C.c_int, [C.c_void_p, C.POINTER(GateNormDesc), C.c_void_p]),
    "m3_gate_norm_backward": (C.c_int, [C.c_void_p, C.POINTER(GateNormDesc), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "m3_host_alloc": (C.c_int, [C.c_size_t, C.POINTER(C.c_void_p)]),
    "m3_host_free": (C.c_int, [C.c_void_p]),
    "m3_host_pipe_create": (C.c_int, [C.c_void_p, C.POINTER(ScanDesc), C.c_int, C.POINTER(C.c_void_p)]),
    "m3_host_pipe_run": (C.c_int, [C.c_void_p, C.POINTER(HostIn), C.POINTER(HostOut), C.POINTER(C.c_uint64)]),
    "m3_host_pipe_wait": (C.c_int, [C.c_void_p, C.c_uint64]),
    "m3_host_pipe_destroy": (C.c_int, [C.c_void_p]),
}

_lib = None


def lib_path() -> Path:
    return _LIB_PATH


def load():
    """Load libm3scan.so and type its entry points.  Raises if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not _LIB_PATH.exists():
        raise RuntimeError(
            f"{_LIB_PATH} is missing: build it with `python -m mamba_trainer_b200.build` "
            "(there is no fallback implementation)")
    lib = C.CDLL(str(_LIB_PATH))
    for name, (res, args) in SYMBOLS.items():
        fn = getattr(lib, name)  # AttributeError if the library does not export it
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib
