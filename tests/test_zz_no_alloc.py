"""m3_scan_forward_noalloc, called straight through the C ABI.

The entry point serves hosts that may not allocate device memory while running (an
arena-owning server, a latency-bound decode loop): it must give what m3_scan_forward
gives, call after call, out of the scratch block built into the library.  This file is
collected last so that a run stopping at the first failure has already run the rest.
"""
import ctypes as C

import pytest
import torch

from mamba_trainer_b200 import _ffi, synthetic

pytestmark = pytest.mark.gpu


def _desc(t, w, want_state=True):
    p = lambda v: C.c_void_p(v.data_ptr()) if v is not None else None
    return _ffi.ScanDesc(
        batch=w.batch, seq=w.seq, heads=w.heads, head_dim=w.head_dim, d_state=w.d_state, rank=w.rank,
        chunk=w.chunk, dtype=_ffi.F32 if w.dtype == torch.float32 else _ffi.BF16, discretization=2,
        dynamics=1 if t["theta"] is not None else 0, want_state=int(want_state),
        path=_ffi.PATH_GENERIC,   # the no-alloc entry runs the generic family: compare like with like
        x=p(t["x"]), b=p(t["b"]), c=p(t["c"]), dt=p(t["dt"]), lambda_=p(t["lam"]), theta=p(t["theta"]),
        a_log=p(t["a_log"]), d_skip=p(t["d_skip"]), h0=None, last_u0=None, angle0=None)


def _outputs(t, w):
    y = torch.full_like(t["x"], float("nan"))
    st = lambda *s: torch.full(s, float("nan"), device="cuda")
    h, lu = st(w.batch, w.heads, w.head_dim, w.d_state), st(w.batch, w.heads, w.head_dim, w.d_state)
    ang = st(w.batch, w.heads, w.d_state // 2) if t["theta"] is not None else None
    p = lambda v: C.c_void_p(v.data_ptr()) if v is not None else None
    return (y, h, lu, ang), _ffi.ScanOut(y=p(y), h=p(h), last_u=p(lu), angle=p(ang))


@pytest.mark.parametrize("idx,kw", [(0, dict()), (3, dict(batch=1, heads=2, seq=300))])
def test_noalloc_forward_matches_the_allocating_one_twice(idx, kw):
    lib = _ffi.load()
    ctx = C.c_void_p()
    assert lib.m3_ctx_create(0, C.byref(ctx)) == _ffi.OK
    try:
        w = synthetic.WORKLOADS[idx].scaled(**kw) if kw else synthetic.WORKLOADS[idx]
        t = {k: (v.cuda() if v is not None else None) for k, v in synthetic.make_inputs(w, seed=4).items()}
        desc = _desc(t, w)
        assert lib.m3_scan_scratch_bytes(C.byref(desc), 0) <= _ffi.NOALLOC_SCRATCH_BYTES
        want, out = _outputs(t, w)
        assert lib.m3_scan_forward(ctx, C.byref(desc), C.byref(out), None) == _ffi.OK, lib.m3_last_error(ctx)
        assert lib.m3_sync(ctx) == _ffi.OK
        for call in range(2):
            got, out2 = _outputs(t, w)
            rc = lib.m3_scan_forward_noalloc(ctx, C.byref(desc), C.byref(out2))
            assert rc == _ffi.OK, lib.m3_last_error(ctx).decode()
            assert lib.m3_sync(ctx) == _ffi.OK
            for name, a, e in zip(("y", "h", "last_u", "angle"), got, want):
                if e is None:
                    continue
                a, e = a.float(), e.float()
                assert torch.isfinite(a).all(), f"{name} (call {call})"
                # same kernels on different scratch: the float32 tolerance of the parity tests
                assert ((a - e).abs() <= 1e-5 * max(1.0, float(e.abs().max())) + 1e-4 * e.abs()).all(), \
                    f"{name} (call {call})"
    finally:
        lib.m3_ctx_destroy(ctx)


def test_noalloc_refuses_what_does_not_fit():
    lib = _ffi.load()
    ctx = C.c_void_p()
    assert lib.m3_ctx_create(0, C.byref(ctx)) == _ffi.OK
    try:
        w = synthetic.WORKLOADS[1].scaled(batch=2)   # ~300 MB of scratch
        dummy = torch.zeros(1, device="cuda")
        p = C.c_void_p(dummy.data_ptr())
        desc = _ffi.ScanDesc(batch=w.batch, seq=w.seq, heads=w.heads, head_dim=w.head_dim, d_state=w.d_state,
                             rank=1, chunk=64, dtype=_ffi.BF16, discretization=2, dynamics=0, want_state=0, path=0,
                             x=p, b=p, c=p, dt=p, lambda_=p, theta=None, a_log=p, d_skip=None)
        assert lib.m3_scan_scratch_bytes(C.byref(desc), 0) > _ffi.NOALLOC_SCRATCH_BYTES
        out = _ffi.ScanOut(y=p, h=None, last_u=None, angle=None)
        assert lib.m3_scan_forward_noalloc(ctx, C.byref(desc), C.byref(out)) == _ffi.ERR_UNSUPPORTED
        assert b"scratch" in lib.m3_last_error(ctx)
    finally:
        lib.m3_ctx_destroy(ctx)
