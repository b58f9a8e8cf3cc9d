"""Host side of the fused Mamba-3 scan: the reference's entry points over the C ABI.

`ScanInputs`, `ScanOutput`, `SsmState` and `mamba3_scan` keep the names, argument
meaning and error behaviour of src/ssm/scan.rs (:294-358, :361-443, :446-452,
:458-618).  Where the reference composes ~25 differentiable primitives and lets its
tape derive the backward pass, this module registers ONE node whose backward rule is
the library's hand-written adjoint - the arrangement `Var::record_with_mask`
(src/autograd/var.rs:169-204) gives a fused op in the reference.  PyTorch supplies
device memory, streams and the tape; all arithmetic happens in libm3scan.so.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import torch

from .. import _ffi
from ..error import ConfigError, NullError, RankError, ShapeError, UnsupportedError, from_status
from .config import Discretization

_DTYPES = {torch.float32: _ffi.F32, torch.bfloat16: _ffi.BF16}


class Context:
    """One m3_ctx per CUDA device; work is enqueued on torch's current stream."""

    _by_device: dict = {}

    def __init__(self, device_index: int):
        self.lib = _ffi.load()
        self.device_index = device_index
        handle = C.c_void_p()
        rc = self.lib.m3_ctx_create(device_index, C.byref(handle))
        if rc != _ffi.OK:
            raise from_status(rc, f"m3_ctx_create({device_index}) failed")
        self.handle = handle
        self._stream = None

    @classmethod
    def for_device(cls, device: torch.device) -> "Context":
        if device.type != "cuda":
            raise UnsupportedError(f"the fused scan runs on CUDA devices only, got {device}")
        idx = device.index if device.index is not None else torch.cuda.current_device()
        ctx = cls._by_device.get(idx)
        if ctx is None:
            ctx = cls._by_device[idx] = Context(idx)
        ctx.bind_current_stream()
        return ctx

    def bind_current_stream(self) -> None:
        stream = torch.cuda.current_stream(self.device_index).cuda_stream
        if stream != self._stream:
            self.check(self.lib.m3_ctx_set_stream(self.handle, C.c_void_p(stream)))
            self._stream = stream

    def check(self, rc: int) -> None:
        if rc != _ffi.OK:
            raise from_status(rc, self.lib.m3_last_error(self.handle).decode())

    def launch_count(self) -> int:
        return int(self.lib.m3_launch_count(self.handle))

    def sync(self) -> None:
        """Block until the context's work is done; raises DeviceTimeout if a kernel's bounded wait gave
        up since the last report (the same condition is also raised by the next scan call, which looks
        at the host-mapped flag on entry)."""
        self.check(self.lib.m3_sync(self.handle))

    def set_wait_limit(self, iterations: int) -> None:
        """Iteration limit of the kernels' bounded waits (0 = default); see m3_ctx_set_wait_limit."""
        self.check(self.lib.m3_ctx_set_wait_limit(self.handle, C.c_uint32(int(iterations))))


class _Saved:
    """Owns an m3_saved handle; freed when the tape node is dropped."""

    def __init__(self, ctx: Context, handle: C.c_void_p):
        self.ctx, self.handle = ctx, handle

    def __del__(self):
        if self.handle:
            try:
                self.ctx.lib.m3_saved_free(self.ctx.handle, self.handle)
            except Exception:  # interpreter shutdown
                pass
            self.handle = None


@dataclass
class SsmState:
    """State a Mamba-3 layer carries between windows (scan.rs:294-302)."""
    h: torch.Tensor                        # [batch, heads, head_dim, d_state]
    last_u: torch.Tensor                   # same shape
    angle: Optional[torch.Tensor] = None   # [batch, heads, d_state / 2]

    def num_elements(self) -> int:
        return self.h.numel() + self.last_u.numel() + (self.angle.numel() if self.angle is not None else 0)

    @staticmethod
    def zeros(batch, heads, head_dim, d_state, rotational, device) -> "SsmState":
        shape = (batch, heads, head_dim, d_state)
        return SsmState(
            torch.zeros(shape, device=device), torch.zeros(shape, device=device),
            torch.zeros((batch, heads, d_state // 2), device=device) if rotational else None)

    def detach(self) -> "SsmState":
        return SsmState(self.h.detach(), self.last_u.detach(),
                        self.angle.detach() if self.angle is not None else None)

    def clone(self) -> "SsmState":
        return SsmState(self.h, self.last_u, self.angle)


@dataclass
class ScanInputs:
    """Inputs to a full scan, after projection and normalisation (scan.rs:361-385)."""
    x: torch.Tensor        # [batch, seq, heads, head_dim, rank]
    b: torch.Tensor        # [batch, seq, heads, d_state, rank]
    c: torch.Tensor        # [batch, seq, heads, d_state, rank]
    dt: torch.Tensor       # [batch, seq, heads], positive
    a_log: torch.Tensor    # [heads]
    lambda_: Optional[torch.Tensor]  # [batch, seq, heads] in [0, 1]
    theta: Optional[torch.Tensor] = None    # [batch, seq, heads, d_state / 2]
    d_skip: Optional[torch.Tensor] = None   # [heads]
    state: Optional[SsmState] = None
    chunk_size: int = 64
    want_state: bool = True
    # Not in the reference: lets a caller that knows lambda is the constant of
    # Discretization::fixed_lambda skip reading it (lambda_ may then be None).
    discretization: Discretization = Discretization.LearnedTrapezoid
    path: int = _ffi.PATH_AUTO
    # The fused form of the bidirectional mixer (models/mamba3.rs:97-112): the last
    # `reverse_heads` heads walk time right to left.  The reference reverses those heads'
    # inputs before the scan (:352-370) and their output after it (:548-556); here the
    # kernels read and write those heads' tokens in reverse order instead.
    reverse_heads: int = 0

    @staticmethod
    def new(x, b, c, dt, a_log, lambda_) -> "ScanInputs":
        return ScanInputs(x, b, c, dt, a_log, lambda_)

    def with_theta(self, theta) -> "ScanInputs":
        self.theta = theta
        return self

    def with_skip(self, d_skip) -> "ScanInputs":
        self.d_skip = d_skip
        return self

    def with_state(self, state: SsmState) -> "ScanInputs":
        self.state = state
        return self

    def with_chunk_size(self, chunk_size: int) -> "ScanInputs":
        self.chunk_size = chunk_size
        return self

    def with_state_output(self, want_state: bool) -> "ScanInputs":
        self.want_state = want_state
        return self

    def with_discretization(self, discretization: Discretization) -> "ScanInputs":
        self.discretization = Discretization(discretization)
        return self

    def with_path(self, path: int) -> "ScanInputs":
        self.path = path
        return self

    def with_reverse_heads(self, reverse_heads: int) -> "ScanInputs":
        self.reverse_heads = int(reverse_heads)
        return self


@dataclass
class ScanOutput:
    """Result of a scan (scan.rs:446-452)."""
    y: torch.Tensor                 # [batch, seq, heads, head_dim, rank]
    state: Optional[SsmState]


def _ptr(t: Optional[torch.Tensor]):
    return C.c_void_p(t.data_ptr()) if t is not None else None


class _FusedScan(torch.autograd.Function):
    """The fused node: forward = m3_scan_forward, backward rule = m3_scan_backward."""

    @staticmethod
    def forward(fctx, opts, x, b, c, dt, a_log, lam, theta, d_skip, h0, last_u0, angle0):
        ctx = Context.for_device(x.device)
        B, T, H, P, R = x.shape
        N = b.shape[3]
        desc = _ffi.ScanDesc(
            batch=B, seq=T, heads=H, head_dim=P, d_state=N, rank=R, chunk=int(opts["chunk"]),
            dtype=_DTYPES[x.dtype], discretization=int(opts["disc"]),
            dynamics=1 if theta is not None else 0, want_state=1 if opts["want_state"] else 0,
            path=int(opts["path"]), reverse_heads=int(opts.get("rev", 0)),
            x=_ptr(x), b=_ptr(b), c=_ptr(c), dt=_ptr(dt), lambda_=_ptr(lam), theta=_ptr(theta),
            a_log=_ptr(a_log), d_skip=_ptr(d_skip), h0=_ptr(h0), last_u0=_ptr(last_u0), angle0=_ptr(angle0))
        y = torch.empty_like(x)
        h = lu = ang = None
        if opts["want_state"]:
            h = torch.empty((B, H, P, N), device=x.device, dtype=torch.float32)
            lu = torch.empty((B, H, P, N), device=x.device, dtype=torch.float32)
            if theta is not None:
                ang = torch.empty((B, H, N // 2), device=x.device, dtype=torch.float32)
        out = _ffi.ScanOut(y=_ptr(y), h=_ptr(h), last_u=_ptr(lu), angle=_ptr(ang))
        tensors = (x, b, c, dt, a_log, lam, theta, d_skip, h0, last_u0, angle0)
        # forward runs with grad mode off, so ask the node which parents are tracked
        # (the `wanted` mask of Var::record_with_mask); none => inference, no rule built.
        track = any(fctx.needs_input_grad)
        saved = C.c_void_p()
        ctx.check(ctx.lib.m3_scan_forward(ctx.handle, C.byref(desc), C.byref(out),
                                          C.byref(saved) if track else None))
        if track:
            fctx.m3 = ctx
            fctx.saved = _Saved(ctx, saved)
            fctx.save_for_backward(*[t for t in tensors if t is not None])
            fctx.present = [t is not None for t in tensors]
            fctx.set_materialize_grads(False)
        outs = [y] + [t for t in (h, lu, ang) if t is not None]
        fctx.n_state_out = len(outs) - 1
        fctx.has_angle = ang is not None
        return tuple(outs)

    @staticmethod
    def backward(fctx, dy, *dstate):
        ctx = fctx.m3
        ctx.bind_current_stream()
        it = iter(fctx.saved_tensors)
        x, b, c, dt, a_log, lam, theta, d_skip, h0, lu0, ang0 = (
            next(it) if p else None for p in fctx.present)
        dstate = list(dstate) + [None] * (3 - len(dstate))
        dh, dlu, dang = dstate[0], dstate[1], dstate[2] if fctx.has_angle else None
        if dy is None:
            dy = torch.zeros_like(x)
        need = fctx.needs_input_grad[1:]
        names = ("x", "b", "c", "dt", "a_log", "lam", "theta", "d_skip", "h0", "lu0", "ang0")
        inputs = dict(zip(names, (x, b, c, dt, a_log, lam, theta, d_skip, h0, lu0, ang0)))
        grads, mask = {}, 0
        for i, name in enumerate(names):
            t = inputs[name]
            if t is not None and need[i]:
                grads[name] = torch.empty_like(t)
                mask |= 1 << i
        cont = lambda t: t.contiguous() if t is not None else None
        dy, dh, dlu, dang = cont(dy), cont(dh), cont(dlu), cont(dang)
        bin_ = _ffi.ScanBwdIn(dy=_ptr(dy), dh=_ptr(dh), dlast_u=_ptr(dlu), dangle=_ptr(dang))
        g = lambda n: _ptr(grads.get(n))
        gout = _ffi.ScanGrads(dx=g("x"), db=g("b"), dc=g("c"), ddt=g("dt"), dlambda=g("lam"),
                              dtheta=g("theta"), da_log=g("a_log"), dd_skip=g("d_skip"),
                              dh0=g("h0"), dlast_u0=g("lu0"), dangle0=g("ang0"))
        ctx.check(ctx.lib.m3_scan_backward(ctx.handle, fctx.saved.handle, C.byref(bin_),
                                           C.c_uint32(mask), C.byref(gout)))
        return (None,) + tuple(grads.get(n) for n in names)


class _FusedSsd(torch.autograd.Function):
    """`ssd_chunked` as one node: the caller's own a, g, w (src/ssm/scan.rs:116-291)."""

    @staticmethod
    def forward(fctx, opts, x, b, c, a, g, w, h0):
        ctx = Context.for_device(x.device)
        B, T, H, P = x.shape
        N = b.shape[3]
        desc = _ffi.ScanDesc(
            batch=B, seq=T, heads=H, head_dim=P, d_state=N, rank=1, chunk=int(opts["chunk"]),
            dtype=_DTYPES[x.dtype], discretization=int(Discretization.LearnedTrapezoid), dynamics=0,
            want_state=1 if opts["want_state"] else 0, path=_ffi.PATH_GENERIC,
            x=_ptr(x), b=_ptr(b), c=_ptr(c), h0=_ptr(h0), a_raw=_ptr(a), g_raw=_ptr(g), w_raw=_ptr(w))
        y = torch.empty_like(x)
        h = torch.empty((B, H, P, N), device=x.device, dtype=torch.float32) if opts["want_state"] else None
        out = _ffi.ScanOut(y=_ptr(y), h=_ptr(h))
        track = any(fctx.needs_input_grad)
        saved = C.c_void_p()
        ctx.check(ctx.lib.m3_scan_forward(ctx.handle, C.byref(desc), C.byref(out),
                                          C.byref(saved) if track else None))
        if track:
            fctx.m3 = ctx
            fctx.saved = _Saved(ctx, saved)
            tensors = (x, b, c, a, g, w, h0)
            fctx.save_for_backward(*[t for t in tensors if t is not None])
            fctx.present = [t is not None for t in tensors]
            fctx.set_materialize_grads(False)
        return (y, h) if h is not None else (y,)

    @staticmethod
    def backward(fctx, dy, dh=None):
        ctx = fctx.m3
        ctx.bind_current_stream()
        it = iter(fctx.saved_tensors)
        x, b, c, a, g, w, h0 = (next(it) if p else None for p in fctx.present)
        if dy is None:
            dy = torch.zeros_like(x)
        need = fctx.needs_input_grad[1:]
        tensors = (x, b, c, a, g, w, h0)
        grads = [torch.empty_like(t) if (t is not None and need[i]) else None for i, t in enumerate(tensors)]
        mask = sum(bit for bit, gr in zip((_ffi.GRAD_X, _ffi.GRAD_B, _ffi.GRAD_C, _ffi.GRAD_DT, _ffi.GRAD_DT,
                                           _ffi.GRAD_DT, _ffi.GRAD_H0), grads) if gr is not None)
        dy = dy.contiguous()
        dh = dh.contiguous() if dh is not None else None
        bin_ = _ffi.ScanBwdIn(dy=_ptr(dy), dh=_ptr(dh))
        gout = _ffi.ScanGrads(dx=_ptr(grads[0]), db=_ptr(grads[1]), dc=_ptr(grads[2]), da_raw=_ptr(grads[3]),
                              dg_raw=_ptr(grads[4]), dw_raw=_ptr(grads[5]), dh0=_ptr(grads[6]))
        ctx.check(ctx.lib.m3_scan_backward(ctx.handle, fctx.saved.handle, C.byref(bin_), C.c_uint32(mask | 0xFF),
                                           C.byref(gout)))
        return (None,) + tuple(grads)


def ssd_chunked(x, b, c, a, g, w, initial_state=None, chunk_size: int = 64, want_state: bool = True):
    """The core one-channel scan with caller-supplied weights (src/ssm/scan.rs:116-126).

    x [B,T,H,P]; b, c [B,T,H,N]; a (log decay per step), g (diagonal weight), w (off-diagonal
    weight) [B,T,H]; initial_state [B,H,P,N].  Returns (y [B,T,H,P], state [B,H,P,N] or None).
    """
    _expect_rank(x, 4)                                   # scan.rs:127-128
    _expect_rank(b, 4)
    B, T, H, P = x.shape
    N = b.shape[3]
    if x.dtype not in _DTYPES:
        raise UnsupportedError(f"element type {x.dtype}: float32 and bfloat16 are served")
    if tuple(b.shape) != (B, T, H, N) or tuple(c.shape) != (B, T, H, N):
        raise ShapeError(f"b {tuple(b.shape)} / c {tuple(c.shape)} do not match x {tuple(x.shape)}")
    for name, t in (("a", a), ("g", g), ("w", w)):
        if tuple(t.shape) != (B, T, H):
            raise ShapeError(f"{name} has shape {tuple(t.shape)}, expected {(B, T, H)}")
    if initial_state is not None and tuple(initial_state.shape) != (B, H, P, N):
        raise ShapeError(f"initial_state has shape {tuple(initial_state.shape)}, expected {(B, H, P, N)}")
    if T == 0:                                           # scan.rs:134-144
        st = None
        if want_state:
            st = initial_state if initial_state is not None else torch.zeros((B, H, P, N), device=x.device)
        return x, st
    el = x.dtype
    big = lambda t: t.to(el).contiguous()
    h0 = initial_state.to(torch.float32).contiguous() if initial_state is not None else None
    outs = _FusedSsd.apply({"chunk": chunk_size, "want_state": bool(want_state)},
                           x.contiguous(), big(b), big(c), big(a), big(g), big(w), h0)
    return outs[0], (outs[1] if want_state else None)


def mamba3_step(x, b, c, dt, lambda_, a_log, theta, d_skip, state: SsmState,
                discretization: Discretization = Discretization.LearnedTrapezoid):
    """One decoding step (src/ssm/scan.rs:649-712), as a single launch; not differentiable.

    x [B,H,P,R]; b, c [B,H,N,R]; dt, lambda_ [B,H]; theta [B,H,N/2] or None; returns (y, SsmState).
    """
    _expect_rank(x, 4)
    B, H, P, R = x.shape
    N = b.shape[2]
    if x.dtype not in _DTYPES:
        raise UnsupportedError(f"element type {x.dtype}: float32 and bfloat16 are served")
    if tuple(b.shape) != (B, H, N, R) or tuple(c.shape) != (B, H, N, R):
        raise ShapeError(f"b {tuple(b.shape)} / c {tuple(c.shape)} do not match x {tuple(x.shape)}")
    if theta is not None and N % 2:
        raise ConfigError("rotational dynamics require an even d_state")
    disc = Discretization(discretization)
    if disc is Discretization.LearnedTrapezoid and lambda_ is None:
        raise NullError("LearnedTrapezoid needs a lambda tensor")
    ctx = Context.for_device(x.device)
    el = x.dtype
    big = lambda t: None if t is None else t.detach().to(el).contiguous()
    f32 = lambda t: None if t is None else t.detach().to(torch.float32).contiguous()
    xs, bs, cs, dts, lams, ths = big(x), big(b), big(c), big(dt), big(lambda_), big(theta)
    al, dk, h, lu = f32(a_log), f32(d_skip), f32(state.h), f32(state.last_u)
    ang = f32(state.angle) if (theta is not None and state.angle is not None) else None
    y = torch.empty_like(xs)
    h2, lu2 = torch.empty_like(h), torch.empty_like(lu)
    ang2 = torch.empty((B, H, N // 2), device=x.device, dtype=torch.float32) if theta is not None else None
    desc = _ffi.StepDesc(batch=B, heads=H, head_dim=P, d_state=N, rank=R, dtype=_DTYPES[el],
                         discretization=int(disc), dynamics=1 if theta is not None else 0,
                         x=_ptr(xs), b=_ptr(bs), c=_ptr(cs), dt=_ptr(dts),
                         lambda_=_ptr(lams) if disc is Discretization.LearnedTrapezoid else None, theta=_ptr(ths),
                         a_log=_ptr(al), d_skip=_ptr(dk), h=_ptr(h), last_u=_ptr(lu), angle=_ptr(ang))
    out = _ffi.StepOut(y=_ptr(y), h=_ptr(h2), last_u=_ptr(lu2), angle=_ptr(ang2))
    ctx.check(ctx.lib.m3_step_forward(ctx.handle, C.byref(desc), C.byref(out)))
    return y, SsmState(h2, lu2, ang2)


def shift_left(x: torch.Tensor, axis: int) -> torch.Tensor:
    """Shift along `axis` towards smaller indices, zero-filling the last slot (scan.rs:64-75)."""
    n = x.shape[axis]
    if n == 0:
        return x
    pad = torch.zeros_like(x.narrow(axis, 0, 1))
    if n == 1:
        return pad
    return torch.cat([x.narrow(axis, 1, n - 1), pad], dim=axis)


def _expect_rank(t: torch.Tensor, rank: int) -> None:
    if t.dim() != rank:
        raise RankError(rank, t.dim(), t.shape)


def mamba3_scan(inputs: ScanInputs) -> ScanOutput:
    """Run the Mamba-3 selective scan (scan.rs:458-618) as one fused device op."""
    x, b, c = inputs.x, inputs.b, inputs.c
    _expect_rank(x, 5)                                   # scan.rs:462
    _expect_rank(b, 5)
    _expect_rank(c, 5)
    B, T, H, P, R = x.shape
    N = b.shape[3]
    if x.dtype not in _DTYPES:
        raise UnsupportedError(f"element type {x.dtype}: float32 and bfloat16 are served")
    if tuple(b.shape) != (B, T, H, N, R) or tuple(c.shape) != (B, T, H, N, R):
        raise ShapeError(f"b {tuple(b.shape)} / c {tuple(c.shape)} do not match x {tuple(x.shape)}")
    disc = Discretization(inputs.discretization)
    lam = inputs.lambda_
    if disc is Discretization.LearnedTrapezoid and lam is None:
        raise NullError("LearnedTrapezoid needs a lambda tensor")
    if disc is not Discretization.LearnedTrapezoid:
        lam = None
    for name, t in (("dt", inputs.dt), ("lambda", lam)):
        if t is not None and tuple(t.shape) != (B, T, H):
            raise ShapeError(f"{name} has shape {tuple(t.shape)}, expected {(B, T, H)}")
    if tuple(inputs.a_log.shape) != (H,):
        raise ShapeError(f"a_log has shape {tuple(inputs.a_log.shape)}, expected {(H,)}")
    theta = inputs.theta
    if theta is not None:
        if N % 2:                                        # scan.rs:485-489
            raise ConfigError("rotational dynamics require an even d_state")
        if tuple(theta.shape) != (B, T, H, N // 2):
            raise ShapeError(f"theta has shape {tuple(theta.shape)}, expected {(B, T, H, N // 2)}")
    if inputs.d_skip is not None and tuple(inputs.d_skip.shape) != (H,):
        raise ShapeError(f"d_skip has shape {tuple(inputs.d_skip.shape)}, expected {(H,)}")
    if not 0 <= inputs.reverse_heads <= H:
        raise ConfigError(f"reverse_heads {inputs.reverse_heads} outside [0, heads = {H}]")
    st = inputs.state
    if st is not None:
        for name, t in (("h", st.h), ("last_u", st.last_u)):
            if tuple(t.shape) != (B, H, P, N):
                raise ShapeError(f"state.{name} has shape {tuple(t.shape)}, expected {(B, H, P, N)}")
        if st.angle is not None and theta is not None and tuple(st.angle.shape) != (B, H, N // 2):
            raise ShapeError(f"state.angle has shape {tuple(st.angle.shape)}")

    if T == 0:                                           # scan.rs:134-144: nothing to scan
        state = None
        if inputs.want_state:
            state = st.clone() if st is not None else SsmState.zeros(B, H, P, N, theta is not None, x.device)
        return ScanOutput(x, state)

    el = x.dtype
    big = lambda t: None if t is None else t.to(el).contiguous()
    f32 = lambda t: None if t is None else t.to(torch.float32).contiguous()
    opts = {"chunk": inputs.chunk_size, "disc": int(disc), "want_state": bool(inputs.want_state),
            "path": inputs.path, "rev": inputs.reverse_heads}
    outs = _FusedScan.apply(
        opts, x.contiguous(), big(b), big(c), big(inputs.dt), f32(inputs.a_log), big(lam), big(theta),
        f32(inputs.d_skip), f32(st.h) if st else None, f32(st.last_u) if st else None,
        f32(st.angle) if (st and theta is not None and st.angle is not None) else None)
    y = outs[0]
    state = None
    if inputs.want_state:
        state = SsmState(outs[1], outs[2], outs[3] if theta is not None else None)
    return ScanOutput(y, state)
