"""Seeded synthetic scan inputs in the shapes and value distributions of the five
benchmark configurations (no dataset is involved: the scan's inputs are activations).

Distributions: x ~ N(0,1); dt = clamp(softplus(N(0,0.5) - 4.6), 1e-3, 0.1);
a_log ~ U(0, ln 16) per head (A = -exp(a_log)); D ~ N(0,1) per head;
lambda = sigmoid(N(0,1)) when learned; theta ~ U(0, pi) per (head, plane), repeated
over batch and time; B, C either N(0,1)/sqrt(N) or "rms": N(0,1) + bias N(0,0.02)
per (head, n), RMS-normalised over N (eps 1e-5), which is what the mixer feeds the
scan (src/models/mamba3.rs:424-433).  The upstream gradient dy ~ N(0,1).

bf16 configurations are generated in float32 and rounded once; the per-head
parameters stay float32.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, replace
from typing import Optional

import torch

from .ssm.config import Discretization


@dataclass(frozen=True)
class Workload:
    name: str
    batch: int
    seq: int
    heads: int
    head_dim: int
    d_state: int
    chunk: int
    rank: int
    dtype: torch.dtype
    discretization: Discretization
    rotational: bool
    bc: str  # "scaled" | "rms"

    @property
    def tokens(self) -> int:
        return self.batch * self.seq

    def elem_bytes(self) -> int:
        return 4 if self.dtype == torch.float32 else 2

    def bytes_per_token_head(self) -> int:
        """Algorithmic forward+backward HBM bytes per (token, head): inputs read twice,
        y written, dy read, every input gradient written; per-head parameters and
        implementation scratch not counted."""
        es = self.elem_bytes()
        ntheta = self.d_state // 2 if self.rotational else 0
        inputs = es * (self.head_dim * self.rank + 2 * self.d_state * self.rank + ntheta + 2)
        y = es * self.head_dim * self.rank
        return (inputs + y) + (inputs + y + inputs)

    def flops_per_token_head(self) -> int:
        """Forward+backward FLOPs per (token, head), folded MIMO, sequential state pass;
        backward counted as twice the forward."""
        L, R, N, P = self.chunk, self.rank, self.d_state, self.head_dim
        fwd = 2 * L * R * R * (N + P) + 4 * R * P * N + 2 * P * N // L
        return 3 * fwd

    def scaled(self, batch: Optional[int] = None, heads: Optional[int] = None, seq: Optional[int] = None):
        return replace(self, batch=batch or self.batch, heads=heads or self.heads, seq=seq or self.seq)


E, LT = Discretization.Euler, Discretization.LearnedTrapezoid
WORKLOADS = (
    Workload("cfg0_siso_euler_f32", 2, 256, 4, 64, 64, 64, 1, torch.float32, E, False, "scaled"),
    Workload("cfg1_siso_trapezoid_bf16", 8, 2048, 12, 64, 128, 64, 1, torch.bfloat16, LT, False, "rms"),
    Workload("cfg2_rotational_bf16", 8, 4096, 16, 64, 128, 64, 1, torch.bfloat16, LT, True, "rms"),
    Workload("cfg3_mimo4_rotational_bf16", 16, 4096, 32, 64, 128, 64, 4, torch.bfloat16, LT, True, "scaled"),
    Workload("cfg4_mimo2_scaling_bf16", 64, 16384, 32, 64, 128, 128, 2, torch.bfloat16, LT, True, "scaled"),
)


def make_inputs(w: Workload, seed: int = 0, device="cpu", with_state: bool = False) -> dict:
    """Tensors of one workload.  Generated on `device` from a generator seeded with
    `seed` (a CUDA generator and a CPU generator give different streams: tests that
    compare against a CPU oracle generate on the CPU and copy)."""
    dev = torch.device(device)
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)
    B, T, H, P, N, R = w.batch, w.seq, w.heads, w.head_dim, w.d_state, w.rank
    f32 = dict(device=dev, dtype=torch.float32, generator=gen)
    randn = lambda *s: torch.randn(*s, **f32)
    rand = lambda *s: torch.rand(*s, **f32)
    out = {"x": randn(B, T, H, P, R)}
    if w.bc == "rms":
        for name in ("b", "c"):
            bias = randn(H, N) * 0.02
            raw = randn(B, T, H, N, R) + bias.view(1, 1, H, N, 1)
            out[name] = raw * torch.rsqrt(raw.pow(2).mean(3, keepdim=True) + 1e-5)
    else:
        out["b"] = randn(B, T, H, N, R) / math.sqrt(N)
        out["c"] = randn(B, T, H, N, R) / math.sqrt(N)
    out["dt"] = torch.nn.functional.softplus(randn(B, T, H) * 0.5 - 4.6).clamp(1e-3, 0.1)
    out["a_log"] = rand(H) * math.log(16.0)
    out["d_skip"] = randn(H)
    if w.discretization is Discretization.LearnedTrapezoid:
        out["lam"] = torch.sigmoid(randn(B, T, H))
    elif w.discretization is Discretization.Trapezoid:
        out["lam"] = torch.full((B, T, H), 0.5, device=dev)
    else:
        out["lam"] = torch.ones((B, T, H), device=dev)
    if w.rotational:
        th = rand(H, N // 2) * math.pi
        out["theta"] = th.view(1, 1, H, N // 2).expand(B, T, H, N // 2).contiguous()
    else:
        out["theta"] = None
    out["dy"] = randn(B, T, H, P, R)
    if with_state:
        out["h0"] = randn(B, H, P, N) * 0.1
        out["last_u0"] = randn(B, H, P, N) * 0.1
        out["angle0"] = (rand(B, H, N // 2) * 2 - 1) * math.pi if w.rotational else None
    for k in ("x", "b", "c", "dt", "lam", "theta", "dy"):
        if out[k] is not None:
            out[k] = out[k].to(w.dtype)
    return out


def make_inputs_chunked(w: Workload, seed: int = 0, device="cpu", chunk: int = 8) -> dict:
    """The same distributions as `make_inputs`, generated `chunk` sequences at a time into tensors
    allocated once at their final element type: the float32 temporaries of the generator then stay a
    fraction of the result (a 64-sequence scaling workload would otherwise need twice its own size
    again while it is being made).  Chunk i is `make_inputs` of `chunk` sequences with seed
    `seed + i`; the per-head parameters (a_log, d_skip) are those of chunk 0."""
    if w.batch <= chunk:
        return make_inputs(w, seed=seed, device=device)
    out = None
    for i, b0 in enumerate(range(0, w.batch, chunk)):
        nb = min(chunk, w.batch - b0)
        part = make_inputs(w.scaled(batch=nb), seed=seed + i, device=device)
        if out is None:
            out = {}
            for k, v in part.items():
                if v is None or v.dim() < 3:
                    out[k] = v
                else:
                    out[k] = torch.empty((w.batch,) + tuple(v.shape[1:]), dtype=v.dtype, device=v.device)
        for k, v in part.items():
            if v is not None and v.dim() >= 3:
                out[k][b0:b0 + nb] = v
        del part
    return out
