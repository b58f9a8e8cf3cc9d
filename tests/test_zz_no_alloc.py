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
        path=_ffi.PATH_GENERIC,   # overridden per case
        x=p(t["x"]), b=p(t["b"]), c=p(t["c"]), dt=p(t["dt"]), lambda_=p(t["lam"]), theta=p(t["theta"]),
        a_log=p(t["a_log"]), d_skip=p(t["d_skip"]), h0=None, last_u0=None, angle0=None)


def _outputs(t, w):
    y = torch.full_like(t["x"], float("nan"))
    st = lambda *s: torch.full(s, float("nan"), device="cuda")
    h, lu = st(w.batch, w.heads, w.head_dim, w.d_state), st(w.batch, w.heads, w.head_dim, w.d_state)
    ang = st(w.batch, w.heads, w.d_state // 2) if t["theta"] is not None else None
    p = lambda v: C.c_void_p(v.data_ptr()) if v is not None else None
    return (y, h, lu, ang), _ffi.ScanOut(y=p(y), h=p(h), last_u=p(lu), angle=p(ang))


def _free_bytes():
    free, _ = torch.cuda.mem_get_info()
    return free


@pytest.mark.parametrize("idx,kw,path", [(0, dict(), _ffi.PATH_GENERIC),
                                         (3, dict(batch=1, heads=2, seq=300), _ffi.PATH_GENERIC),
                                         (3, dict(batch=1, heads=2, seq=300), _ffi.PATH_AUTO)])
def test_noalloc_forward_matches_the_allocating_one_twice(idx, kw, path):
    """Two calls in a row must both give what m3_scan_forward gives.  Between them a call of ANOTHER shape
    runs on the same built-in block, so that what the first call left there is not what the second would
    write anyway; the second call must not change the device's free memory (nothing is allocated once the
    library's kernels and the block have been touched); and one case is checked against the oracle itself,
    not only against the allocating entry point.  PATH_AUTO takes the tensor-core family, which needs no
    scratch when nothing is kept for a backward pass."""
    from tests._util import oracle_run, norm_rel
    lib = _ffi.load()
    ctx = C.c_void_p()
    assert lib.m3_ctx_create(0, C.byref(ctx)) == _ffi.OK
    try:
        w = synthetic.WORKLOADS[idx].scaled(**kw) if kw else synthetic.WORKLOADS[idx]
        t = {k: (v.cuda() if v is not None else None) for k, v in synthetic.make_inputs(w, seed=4).items()}
        desc = _desc(t, w)
        desc.path = path
        assert lib.m3_scan_scratch_bytes(C.byref(desc), 0) <= _ffi.NOALLOC_SCRATCH_BYTES
        want, out = _outputs(t, w)
        assert lib.m3_scan_forward(ctx, C.byref(desc), C.byref(out), None) == _ffi.OK, lib.m3_last_error(ctx)
        assert lib.m3_sync(ctx) == _ffi.OK
        # the other shape that runs in between (generic family, so it does use the block)
        w2 = synthetic.WORKLOADS[0].scaled(batch=1, heads=3, seq=150)
        t2 = {k: (v.cuda() if v is not None else None) for k, v in synthetic.make_inputs(w2, seed=9).items()}
        desc2 = _desc(t2, w2)
        for call in range(2):
            got, out2 = _outputs(t, w)
            torch.cuda.synchronize()
            before = _free_bytes()
            rc = lib.m3_scan_forward_noalloc(ctx, C.byref(desc), C.byref(out2))
            assert rc == _ffi.OK, lib.m3_last_error(ctx).decode()
            assert lib.m3_sync(ctx) == _ffi.OK
            if call == 1:
                assert _free_bytes() == before, "the second call changed the device's free memory"
            tight = path == _ffi.PATH_GENERIC
            for name, a, e in zip(("y", "h", "last_u", "angle"), got, want):
                if e is None:
                    continue
                a, e = a.float(), e.float()
                assert torch.isfinite(a).all(), f"{name} (call {call})"
                if tight:   # same kernels on different scratch: the float32 tolerance of the parity tests
                    assert ((a - e).abs() <= 1e-5 * max(1.0, float(e.abs().max())) + 1e-4 * e.abs()).all(), \
                        f"{name} (call {call})"
                else:       # the same tensor-core kernels: bit for bit
                    assert torch.equal(a, e), f"{name} (call {call})"
            if call == 0:
                _, out3 = _outputs(t2, w2)
                assert lib.m3_scan_forward_noalloc(ctx, C.byref(desc2), C.byref(out3)) == _ffi.OK
                assert lib.m3_sync(ctx) == _ffi.OK
        if idx == 3 and path == _ffi.PATH_GENERIC:   # against the float64 oracle (bf16 inputs: 2e-2)
            ey, est, _ = oracle_run({k: v for k, v in t.items() if v is not None}, w.chunk, True, torch.float64, False)
            assert norm_rel(got[0].float(), ey) <= 2e-2
            assert norm_rel(got[1].float(), est.h) <= 2e-2
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
                             rank=1, chunk=64, dtype=_ffi.BF16, discretization=2, dynamics=0, want_state=0,
                             path=_ffi.PATH_GENERIC,   # the family that needs the block (nothing is launched: refused first)
                             x=p, b=p, c=p, dt=p, lambda_=p, theta=None, a_log=p, d_skip=None)
        assert lib.m3_scan_scratch_bytes(C.byref(desc), 0) > _ffi.NOALLOC_SCRATCH_BYTES
        out = _ffi.ScanOut(y=p, h=None, last_u=None, angle=None)
        assert lib.m3_scan_forward_noalloc(ctx, C.byref(desc), C.byref(out)) == _ffi.ERR_UNSUPPORTED
        assert b"scratch" in lib.m3_last_error(ctx)
    finally:
        lib.m3_ctx_destroy(ctx)
