"""CPU oracle for the Mamba-3 SSD scan.  TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package may import this module: it exists so that the
CUDA path can be checked against a restatement of the reference algorithm, and
so that the benchmark can time a CPU baseline.  Parity status: PINNED - the
functions below are checked (tests/test_oracle.py) against

  * golden vectors produced by the reference's own PyTorch port of this path
    (bench/torch_mamba3.py ``ssd_chunked`` :47-129 and ``rotate_halves``
    :132-137), stored under tests/golden/ with the script that made them;
  * the directly unrolled recurrence of the reference's test-suite
    (tests/ssm.rs:58-106), restated in ``recurrence`` and extended to
    rotation / MIMO / skip / carried state the way ``mamba3_step``
    (src/ssm/scan.rs:649-712) evaluates a single token.

The composed scan follows src/ssm/scan.rs: ``ssd_chunked`` :116-291 and
``mamba3_scan`` :458-618.  It is written with differentiable torch ops so the
reference gradients come from autograd, as the reference's own tape produces
them.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch

LOG_DECAY_FLOOR = -60.0  # src/ssm/scan.rs:54-57
TWO_PI = 2.0 * math.pi


class _RoundedMatmul(torch.autograd.Function):
    """a @ b the way the reference's reduced-precision matmul mode evaluates it: both operands rounded
    to the narrow type once per call, products accumulated in float32, and every matmul of the backward
    rule evaluated the same way (src/tensor/ops/matmul.rs:94-128, :1832-1863; backward rules
    src/autograd/ops.rs:204-264).  Everything outside the matmuls stays in the wide type."""

    @staticmethod
    def forward(ctx, a, b, narrow):
        ctx.save_for_backward(a, b)
        ctx.narrow = narrow
        return _RoundedMatmul.mm(a, b, narrow)

    @staticmethod
    def mm(a, b, narrow):
        wide = a.dtype
        return (a.to(narrow).to(torch.float32) @ b.to(narrow).to(torch.float32)).to(wide)

    @staticmethod
    def backward(ctx, grad):
        a, b = ctx.saved_tensors
        ga = _RoundedMatmul.mm(grad, b.transpose(-1, -2), ctx.narrow)
        gb = _RoundedMatmul.mm(a.transpose(-1, -2), grad, ctx.narrow)
        return ga, gb, None


_MATMUL_NARROW = None   # None: exact matmuls in the tensors' own type


class matmul_precision:
    """Context manager: inside it every matmul of `ssd_chunked` runs in the reference's reduced-precision
    mode with `narrow` operands (e.g. torch.bfloat16).  Used to measure how far the REFERENCE's own bf16
    mode sits from exact arithmetic on a given input - the yardstick for the CUDA path's bf16 tolerances."""

    def __init__(self, narrow):
        self.narrow = narrow

    def __enter__(self):
        global _MATMUL_NARROW
        self.prev, _MATMUL_NARROW = _MATMUL_NARROW, self.narrow

    def __exit__(self, *exc):
        global _MATMUL_NARROW
        _MATMUL_NARROW = self.prev


def _mm(a, b):
    return a @ b if _MATMUL_NARROW is None else _RoundedMatmul.apply(a, b, _MATMUL_NARROW)


def wrap_angle(phi: torch.Tensor) -> torch.Tensor:
    """x - round(x / 2pi) * 2pi with an identity gradient.

    src/ssm/scan.rs:77-83 (``wrap_angle``) over
    src/tensor/ops/elemwise.rs:347-349 (``wrap_to``).
    """
    return phi - (torch.round(phi / TWO_PI) * TWO_PI).detach()


def rotate_by_angle(v: torch.Tensor, phi: torch.Tensor) -> torch.Tensor:
    """Rotate the halves (v[..., :n/2], v[..., n/2:]) of the last axis by -phi.

    src/tensor/ops/fused.rs:588-619 with ``from_angle``: the pair used is
    (cos phi, -sin phi), so out1 = x1 cos + x2 sin, out2 = -x1 sin + x2 cos.
    """
    half = v.shape[-1] // 2
    lo, hi = v[..., :half], v[..., half:]
    cs, sn = torch.cos(phi), torch.sin(phi)
    return torch.cat([lo * cs + hi * sn, hi * cs - lo * sn], dim=-1)


def trapezoid_weights(lam: torch.Tensor, dt: torch.Tensor):
    """g_t = lam_t dt_t ; w_t = g_t + (1 - lam_{t+1}) dt_{t+1}, last w = g.

    src/autograd/ops.rs:1169-1212, src/tensor/ops/fused.rs:2483-2503.
    Tensors are [B, T, H].
    """
    g = lam * dt
    nxt = (1.0 - lam) * dt
    f = torch.cat([nxt[:, 1:], torch.zeros_like(nxt[:, :1])], dim=1)
    return g, g + f


def _band(acum: torch.Tensor, w: torch.Tensor, g: torch.Tensor) -> torch.Tensor:
    """[rows, L] x3 -> [rows, L, L]; src/tensor/ops/fused.rs:2044-2070."""
    L = acum.shape[-1]
    diff = (acum.unsqueeze(-1) - acum.unsqueeze(-2)).clamp(LOG_DECAY_FLOOR, 0.0)
    idx = torch.arange(L)
    below = (idx.view(L, 1) > idx.view(1, L)).to(acum.dtype)
    diag = torch.eye(L, dtype=acum.dtype)
    weight = w.unsqueeze(-2) * below + g.unsqueeze(-2) * diag
    return diff.exp() * weight


def ssd_chunked(x, b, c, a, g, w, initial_state=None, chunk_size=64, want_state=True):
    """One-channel chunked SSD scan; src/ssm/scan.rs:116-291.

    x [B,T,H,P]; b, c [B,T,H,N]; a, g, w [B,T,H]; initial_state [B,H,P,N].
    Returns (y [B,T,H,P], state [B,H,P,N] or None).
    """
    assert x.dim() == 4 and b.dim() == 4
    B, T, H, P = x.shape
    N = b.shape[3]
    if T == 0:  # scan.rs:134-144
        st = None
        if want_state:
            st = initial_state if initial_state is not None else x.new_zeros(B, H, P, N)
        return x, st
    L = max(1, min(chunk_size, T))  # scan.rs:146
    pad = (L - T % L) % L
    Tp = T + pad
    C = Tp // L

    def pad_end(v):
        if pad == 0:
            return v
        z = v.new_zeros((v.shape[0], pad) + tuple(v.shape[2:]))
        return torch.cat([v, z], dim=1)

    x, b, c, a, g, w = (pad_end(v) for v in (x, b, c, a, g, w))
    x = x.reshape(B, C, L, H, P)
    b = b.reshape(B, C, L, H, N)
    c = c.reshape(B, C, L, H, N)
    a = a.reshape(B, C, L, H)
    g = g.reshape(B, C, L, H)
    w = w.reshape(B, C, L, H)
    acum = a.cumsum(2)

    def heads_first(v, last):
        return v.permute(0, 1, 3, 2, 4).reshape(B * C * H, L, last)

    def rows(v):
        return v.permute(0, 1, 3, 2).reshape(B * C * H, L)

    # 1. intra-chunk (scan.rs:192-205)
    band = _band(rows(acum), rows(w), rows(g))
    c_flat, b_flat, x_flat = heads_first(c, N), heads_first(b, N), heads_first(x, P)
    cb = _mm(c_flat, b_flat.transpose(1, 2))
    y_diag = _mm(cb * band, x_flat).reshape(B, C, H, L, P).permute(0, 1, 3, 2, 4)

    # 2. chunk summaries (scan.rs:208-216)
    last_acum = acum[:, :, L - 1:L]
    decay_to_end = (last_acum - acum).clamp(LOG_DECAY_FLOOR, 0.0).exp() * w
    weighted_x = x * decay_to_end.unsqueeze(4)
    chunk_state = _mm(
        weighted_x.permute(0, 1, 3, 4, 2).reshape(B * C * H, P, L), b_flat
    ).reshape(B, C, H, P, N)

    # 3. inter-chunk recurrence as a masked C x C product (scan.rs:219-251)
    chunk_decay = last_acum.reshape(B, C, H)
    through = chunk_decay.cumsum(1)
    before = through - chunk_decay
    kk = torch.arange(C)
    strict = (kk.view(C, 1) > kk.view(1, C)).to(x.dtype).view(1, C, C, 1)
    transfer = (before.unsqueeze(2) - through.unsqueeze(1)).clamp(
        LOG_DECAY_FLOOR, 0.0).exp() * strict
    carry_in = _mm(
        transfer.permute(0, 3, 1, 2).reshape(B * H, C, C),
        chunk_state.permute(0, 2, 1, 3, 4).reshape(B * H, C, P * N)
    ).reshape(B, H, C, P, N).permute(0, 2, 1, 3, 4)
    if initial_state is not None:
        scale = before.clamp(LOG_DECAY_FLOOR, 0.0).exp().reshape(B, C, H, 1, 1)
        carry_in = carry_in + initial_state.reshape(B, 1, H, P, N) * scale

    # 4. carry-in read by every position (scan.rs:254-268)
    c_dec = c * acum.clamp(LOG_DECAY_FLOOR, 0.0).exp().unsqueeze(4)
    y_off = _mm(
        heads_first(c_dec, N),
        carry_in.permute(0, 1, 2, 4, 3).reshape(B * C * H, N, P)
    ).reshape(B, C, H, L, P).permute(0, 1, 3, 2, 4)
    y = (y_diag + y_off).reshape(B, Tp, H, P)[:, :T]

    state = None
    if want_state:  # scan.rs:271-288
        tail = chunk_decay[:, C - 1].clamp(LOG_DECAY_FLOOR, 0.0).exp().reshape(B, H, 1, 1)
        state = carry_in[:, C - 1] * tail + chunk_state[:, C - 1]
    return y, state


@dataclass
class OracleState:
    """SsmState of src/ssm/scan.rs:294-302."""
    h: torch.Tensor                      # [B,H,P,N]
    last_u: torch.Tensor                 # [B,H,P,N]
    angle: Optional[torch.Tensor] = None  # [B,H,N/2]


def mamba3_scan(x, b, c, dt, a_log, lam, theta=None, d_skip=None, state=None,
                chunk_size=64, want_state=True):
    """The full scan, composed as R^2 one-channel scans; src/ssm/scan.rs:458-618.

    x [B,T,H,P,R]; b, c [B,T,H,N,R]; dt, lam [B,T,H]; a_log, d_skip [H];
    theta [B,T,H,N/2].  Returns (y [B,T,H,P,R], OracleState or None).
    """
    assert x.dim() == 5
    B, T, H, P, R = x.shape
    N = b.shape[3]
    a = dt * (-torch.exp(a_log)).reshape(1, 1, H)          # :470-475
    g, w = trapezoid_weights(lam, dt)                       # :479
    end_angle = None
    if theta is None:
        b_rot, c_rot = b, c
    else:                                                   # :482-519
        if N % 2:
            raise ValueError("rotational dynamics require an even d_state")
        phi = (dt.unsqueeze(3) * theta).cumsum(1)
        if state is not None and state.angle is not None:
            phi = phi + state.angle.unsqueeze(1)
        phi = wrap_angle(phi)
        table = phi.unsqueeze(3)

        def rot(v):
            return rotate_by_angle(v.permute(0, 1, 2, 4, 3), table).permute(0, 1, 2, 4, 3)

        b_rot, c_rot = rot(b), rot(c)
        if want_state:
            end_angle = phi[:, T - 1]
    carry = None
    if state is not None:                                   # :524-535
        first = ((1.0 - lam[:, 0]) * dt[:, 0]).reshape(B, H, 1, 1)
        carry = state.h + state.last_u * first
    outs, total = [], None
    for i in range(R):                                      # :545-589
        acc = None
        for j in range(R):
            y_ij, st = ssd_chunked(x[..., j], b_rot[..., j], c_rot[..., i], a, g, w,
                                   carry if j == 0 else None, chunk_size, want_state)
            acc = y_ij if acc is None else acc + y_ij
            if i == 0 and st is not None:
                total = st if total is None else total + st
        outs.append(acc.unsqueeze(4))
    y = torch.cat(outs, dim=4)
    if d_skip is not None:                                  # :594-597
        y = y + x * d_skip.reshape(1, 1, H, 1, 1)
    out_state = None
    if want_state:                                          # :600-615, :621-638
        h = total if total is not None else x.new_zeros(B, H, P, N)
        last_u = torch.einsum("bhpr,bhnr->bhpn", x[:, T - 1], b_rot[:, T - 1])
        out_state = OracleState(h, last_u, end_angle)
    return y, out_state


def reverse_bands_in_time(t: torch.Tensor, reverse_heads: int) -> torch.Tensor:
    """Reverse the time axis (1) of the last `reverse_heads` heads (axis 2) of a [B,T,H,...] tensor:
    what Tensor::reverse_bands does to the backward half of every direction-sensitive input of the
    bidirectional mixer, src/models/mamba3.rs:352-370 (an involution)."""
    if reverse_heads == 0:
        return t
    H = t.shape[2]
    return torch.cat([t[:, :, :H - reverse_heads], t[:, :, H - reverse_heads:].flip(1)], dim=2)


def mamba3_scan_bidirectional(x, b, c, dt, a_log, lam, theta=None, d_skip=None, state=None,
                              chunk_size=64, want_state=True, reverse_heads=0):
    """The scan as the bidirectional mixer runs it (src/models/mamba3.rs:352-370, :548-556): the last
    `reverse_heads` heads see x, B, C, dt, lambda, theta reversed in time, and their y is reversed
    back afterwards; the carried state is untouched (it is per head, not per token)."""
    r = lambda t: None if t is None else reverse_bands_in_time(t, reverse_heads)
    y, st = mamba3_scan(r(x), r(b), r(c), r(dt), a_log, r(lam), r(theta), d_skip, state, chunk_size, want_state)
    return r(y), st
