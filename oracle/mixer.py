"""CPU restatement (torch, any float dtype) of the mixer steps either side of the scan.

TEST INFRASTRUCTURE ONLY: imported by tests/, the smoke check and the CPU-baseline leg of the
benchmark; the product path never touches this module.

Pinned by tests/golden/conv_silu.npz and tests/golden/mixer_core.npz, which hold outputs of the
reference's own PyTorch port (bench/torch_mamba3.py:165-207) - see tests/golden/make_golden.py.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from . import m3_oracle as O


def causal_conv1d(x, weight, bias=None, history=None, activation: bool = True):
    """Depthwise causal convolution as a sum of zero-padded shifts, each scaled by its tap:
    CausalConv1d::apply_composed, src/nn/conv.rs:152-176 (tap k pairs with delay K-1-k), continued
    from `history` [B, K-1, C] as apply_with_history (:185-203), then the mixer's SiLU
    (src/models/mamba3.rs:401).  x [B, T, C]; weight [K, C]; bias [C].
    Returns (y [B, T, C], new_history [B, K-1, C])."""
    B, T, C = x.shape
    K = weight.shape[0]
    past = history if history is not None else x.new_zeros(B, K - 1, C)
    full = torch.cat([past, x], dim=1)                     # time index t maps to t + K - 1
    acc = None
    for delay in range(K):
        term = full[:, K - 1 - delay: K - 1 - delay + T] * weight[K - 1 - delay].reshape(1, 1, C)
        acc = term if acc is None else acc + term
    if bias is not None:
        acc = acc + bias.reshape(1, 1, C)
    y = F.silu(acc) if activation else acc
    return y, full[:, full.shape[1] - (K - 1):]


def rms_norm(v, weight=None, eps: float = 1e-5):
    """Var::rms_norm as RmsNorm::apply uses it (src/nn/norm.rs:95-105): v * rsqrt(mean(v^2) + eps) * weight."""
    out = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)
    return out * weight if weight is not None else out


class _Narrow(torch.autograd.Function):
    """Round to a narrow type and back, in both directions of the tape."""

    @staticmethod
    def forward(ctx, v, narrow):
        ctx.narrow = narrow
        return v.to(narrow).to(v.dtype)

    @staticmethod
    def backward(ctx, g):
        return g.to(ctx.narrow).to(g.dtype), None


def mixer_core(proj, p: dict, heads: int, head_dim: int, d_state: int, rank: int = 1, groups: Optional[int] = None,
               chunk: int = 64, learned_lambda: bool = True, rotational: bool = True, eps: float = 1e-5,
               conv_history=None, state=None, want_state: bool = False, fixed_lambda: float = 1.0,
               bidirectional: bool = False, scan_io_dtype=None, post_gate_norm: bool = False):
    """Everything Mamba3Mixer does between its input and output projections
    (src/models/mamba3.rs:340-461, :475-484, :540-556):
    split the projection into z | x B C | dt | lambda | theta, convolve x|B|C and apply SiLU, expand
    B / C groups to heads, add the per-head biases, RMS-normalise, move the rank axis last, softplus /
    sigmoid, scan, gate with SiLU(z).

    p: conv_w [K, d_inner + 2 bc], conv_b [same] or None, dt_bias [H], a_log [H], d_skip [H] or None,
    b_bias / c_bias [H, N] or None, norm_w [N] or None ("norm" False in p disables the norm);
    post_gate_norm: the scan's flattened output is RMS-normalised over d_inner, gain post_norm_w [d_inner] or
    None, before the gate (:478-482; the reference's port in bench/torch_mamba3.py has no such switch, so this
    branch is pinned only through rms_norm, which the B/C norm of the golden mixer vectors exercises).
    scan_io_dtype (e.g. torch.bfloat16): the scan's per-token inputs and its output pass through that
    type (rounded values, identity gradient, gradients rounded likewise) - the benchmark's "bf16 inputs"
    applied inside the mixer, where the CUDA path hands bf16 tensors from kernel to kernel.
    Returns (gated [B, T, d_inner], new conv history, OracleState or None)."""
    B, T, W = proj.shape
    H, P, N, R = heads, head_dim, d_state, rank
    G = groups or H
    d_inner, bc = H * P * R, G * N * R
    n_lam = H if learned_lambda else 0
    n_th = H * N // 2 if rotational else 0
    assert W == 2 * d_inner + 2 * bc + H + n_lam + n_th, "projection width"
    if bidirectional:
        # mamba3.rs:352-370: every piece is direction-major; the backward half of every piece that
        # feeds the convolution or the scan is reversed in time (z is not: the gate is per position).
        pieces, offset = [], d_inner
        for width in (d_inner, bc, bc, H, n_lam, n_th):
            if width:
                pieces.append((offset + width // 2, offset + width))
                offset += width
        cols = torch.zeros(W, dtype=torch.bool)
        for lo, hi in pieces:
            cols[lo:hi] = True
        proj = torch.where(cols.reshape(1, 1, W), proj.flip(1), proj)
    z, xbc, dt_raw, lam_raw, th_raw = torch.split(proj, [d_inner, d_inner + 2 * bc, H, n_lam, n_th], dim=-1)
    xbc, hist = causal_conv1d(xbc, p["conv_w"], p.get("conv_b"), conv_history, True)
    x, b_flat, c_flat = torch.split(xbc, [d_inner, bc, bc], dim=-1)

    def to_heads(v, bias):                                          # :409-436
        v = v.reshape(B, T, G, 1, R, N).expand(B, T, G, H // G, R, N).reshape(B, T, H, R, N)
        if bias is not None:
            v = v + bias.reshape(1, 1, H, 1, N)
        if p.get("norm", True):
            v = rms_norm(v, p.get("norm_w"), eps)
        return v.permute(0, 1, 2, 4, 3)

    b, c = to_heads(b_flat, p.get("b_bias")), to_heads(c_flat, p.get("c_bias"))
    x5 = x.reshape(B, T, H, P, R)
    dt = F.softplus(dt_raw + p["dt_bias"].reshape(1, 1, H))         # :440-442
    lam = torch.sigmoid(lam_raw) if learned_lambda else torch.full_like(dt, fixed_lambda)
    theta = th_raw.reshape(B, T, H, N // 2) if rotational else None
    if scan_io_dtype is not None:
        x5, b, c, dt, lam, theta = (None if v is None else _Narrow.apply(v, scan_io_dtype) for v in (x5, b, c, dt, lam, theta))
    y, st = O.mamba3_scan(x5, b, c, dt, p["a_log"], lam, theta, p.get("d_skip"), state, chunk, want_state)
    if scan_io_dtype is not None:
        y = _Narrow.apply(y, scan_io_dtype)
    y = y.reshape(B, T, d_inner)
    if bidirectional:                                               # :548-556: the backward heads' output back
        y = torch.cat([y[..., :d_inner // 2], y[..., d_inner // 2:].flip(1)], dim=-1)
    if post_gate_norm:
        y = rms_norm(y, p.get("post_norm_w"), eps)
    gated = y * F.silu(z)                                           # :475-484
    return gated, hist, st
