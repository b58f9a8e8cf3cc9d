"""Directly unrolled Mamba-3 recurrence.  TEST INFRASTRUCTURE ONLY.

``recurrence`` restates the independent check of the reference's test-suite,
tests/ssm.rs:58-106:

    h_t = alpha_t h_{t-1} + beta_t u_{t-1} + gamma_t u_t ,  y_t = C_t^T h_t
    alpha = exp(dt A), beta = (1 - lam) dt alpha, gamma = lam dt

and extends it, token by token, the way ``mamba3_step`` (src/ssm/scan.rs:649-712)
does: rotation of B and C by the running wrapped angle, u = sum_j x^(j) (x) B^(j),
one output per rank, the D skip, and a carried (h, last_u, angle).  float64 numpy
so it can also arbitrate between two fp32 implementations.

``lcg_noise`` and ``Case`` reproduce the deterministic inputs of
tests/ssm.rs:26-34 and :122-142 so the reference's own test cases can be replayed.
"""
from __future__ import annotations

import math

import numpy as np

_MASK = (1 << 64) - 1


def lcg_noise(n: int, seed: int) -> np.ndarray:
    """tests/ssm.rs:26-34 - values in [-1, 1), float32."""
    s = (seed * 6364136223846793005 + 1) & _MASK
    out = np.empty(n, dtype=np.float32)
    for i in range(n):
        s = (s * 6364136223846793005 + 1442695040888963407) & _MASK
        out[i] = np.float32(np.float32(s >> 33) / np.float32(1 << 31)) - np.float32(1.0)
    return out


class Case:
    """tests/ssm.rs:122-142 (seeds x=1, b=2, c=3, dt=7, lambda=11; theta=5 at :242)."""

    def __init__(self, batch, seq, heads, head_dim, state):
        bt = batch * seq * heads
        self.shape = (batch, seq, heads, head_dim, state)
        v = lcg_noise(bt, 7)
        self.dt = (np.float32(0.05) + np.float32(0.25) * (v + np.float32(1.0))).reshape(batch, seq, heads)
        v = lcg_noise(bt, 11)
        self.lam = (np.float32(0.5) * (v + np.float32(1.0)) * np.float32(0.98)
                    + np.float32(0.01)).reshape(batch, seq, heads)
        self.a_head = np.array([-(1.0 + 0.7 * i) for i in range(heads)], dtype=np.float32)
        self.a_log = np.log(-self.a_head).astype(np.float32)
        self.x = lcg_noise(batch * seq * heads * head_dim, 1).reshape(batch, seq, heads, head_dim)
        self.b = lcg_noise(batch * seq * heads * state, 2).reshape(batch, seq, heads, state)
        self.c = lcg_noise(batch * seq * heads * state, 3).reshape(batch, seq, heads, state)

    def theta(self):
        batch, seq, heads, _, state = self.shape
        return lcg_noise(batch * seq * heads * (state // 2), 5).reshape(batch, seq, heads, state // 2)


def _rot(v, phi):
    """v [..., N, R], phi [..., N/2] -> rotation of the halves of axis -2 by -phi."""
    half = v.shape[-2] // 2
    lo, hi = v[..., :half, :], v[..., half:, :]
    cs, sn = np.cos(phi)[..., None], np.sin(phi)[..., None]
    return np.concatenate([lo * cs + hi * sn, hi * cs - lo * sn], axis=-2)


def recurrence(x, b, c, dt, a_log, lam, theta=None, d_skip=None,
               h0=None, last_u0=None, angle0=None):
    """x [B,T,H,P,R]; b, c [B,T,H,N,R]; dt, lam [B,T,H]; theta [B,T,H,N/2].

    Returns (y [B,T,H,P,R], h [B,H,P,N], last_u [B,H,P,N], angle [B,H,N/2] or None),
    all float64.
    """
    x, b, c, dt, lam = (np.asarray(v, dtype=np.float64) for v in (x, b, c, dt, lam))
    B, T, H, P, R = x.shape
    N = b.shape[3]
    A = -np.exp(np.asarray(a_log, dtype=np.float64))
    h = np.zeros((B, H, P, N)) if h0 is None else np.asarray(h0, dtype=np.float64).copy()
    prev_u = np.zeros((B, H, P, N)) if last_u0 is None else np.asarray(last_u0, dtype=np.float64).copy()
    angle = None
    if theta is not None:
        theta = np.asarray(theta, dtype=np.float64)
        angle = np.zeros((B, H, N // 2)) if angle0 is None else np.asarray(angle0, dtype=np.float64).copy()
    y = np.zeros((B, T, H, P, R))
    for t in range(T):
        step, lm = dt[:, t], lam[:, t]                      # [B,H]
        alpha = np.exp(step * A[None, :])
        beta = (1.0 - lm) * step * alpha
        gamma = lm * step
        bt_, ct_ = b[:, t], c[:, t]                         # [B,H,N,R]
        if theta is not None:
            angle = angle + step[..., None] * theta[:, t]
            angle = angle - np.round(angle / (2 * math.pi)) * (2 * math.pi)
            bt_, ct_ = _rot(bt_, angle), _rot(ct_, angle)
        u = np.einsum("bhpr,bhnr->bhpn", x[:, t], bt_)
        h = alpha[..., None, None] * h + beta[..., None, None] * prev_u + gamma[..., None, None] * u
        prev_u = u
        yt = np.einsum("bhnr,bhpn->bhpr", ct_, h)
        if d_skip is not None:
            yt = yt + x[:, t] * np.asarray(d_skip, dtype=np.float64)[None, :, None, None]
        y[:, t] = yt
    return y, h, prev_u, angle
