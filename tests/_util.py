"""Helpers shared by the parity tests: run the oracle and the fused op on the same
tensors and compare with the stated tolerances."""
from __future__ import annotations

import numpy as np
import torch

from oracle import m3_oracle as O

GRAD_NAMES = ("x", "b", "c", "dt", "a_log", "lam", "theta", "d_skip", "h0", "last_u0", "angle0")


def ref_metric(a, e) -> float:
    """max |a - e| / (1 + |e|): the reference's own closeness measure (tests/ssm.rs:36-53)."""
    a = torch.as_tensor(np.asarray(a) if not torch.is_tensor(a) else a).double().cpu()
    e = torch.as_tensor(np.asarray(e) if not torch.is_tensor(e) else e).double().cpu()
    if a.numel() == 0:
        return 0.0
    return float(((a - e).abs() / (1.0 + e.abs())).max())


def norm_rel(a, e) -> float:
    """||a - e|| / ||e||."""
    a, e = a.detach().double().cpu(), e.detach().double().cpu()
    den = float(e.norm())
    return float((a - e).norm()) / den if den > 0 else float((a - e).norm())


def allclose_excess(a, e, rtol, atol) -> float:
    """max |a - e| / (atol + rtol |e|); <= 1 means within tolerance."""
    a, e = a.detach().double().cpu(), e.detach().double().cpu()
    if a.numel() == 0:
        return 0.0
    return float(((a - e).abs() / (atol + rtol * e.abs())).max())


def oracle_run(t: dict, chunk: int, want_state=True, dtype=torch.float64, grads=True,
               dstate=None, use_lam=True, reverse_heads=0, matmul_narrow=None):
    """Run the composed oracle on CPU.  `t` holds x, b, c, dt, a_log, lam, theta, d_skip
    and optionally h0, last_u0, angle0, dy.  Inputs are upcast (a bf16 tensor is used
    at its rounded value).  With `matmul_narrow` (e.g. torch.bfloat16) every matmul runs in the
    reference's reduced-precision mode (operands rounded once per call, float32 accumulation,
    src/tensor/ops/matmul.rs:94-128, :1832-1863).  Returns (y, state, {name: grad})."""
    if matmul_narrow is not None:
        with O.matmul_precision(matmul_narrow):
            return oracle_run(t, chunk, want_state, dtype, grads, dstate, use_lam, reverse_heads, None)
    names = [n for n in GRAD_NAMES if t.get(n) is not None]
    leaf = {n: t[n].detach().cpu().to(dtype).requires_grad_(grads) for n in names}
    st = None
    if "h0" in leaf:
        st = O.OracleState(leaf["h0"], leaf["last_u0"], leaf.get("angle0"))
    y, out = O.mamba3_scan_bidirectional(leaf["x"], leaf["b"], leaf["c"], leaf["dt"], leaf["a_log"], leaf["lam"],
                                         leaf.get("theta"), leaf.get("d_skip"), st, chunk, want_state, reverse_heads)
    g = {}
    if grads:
        loss = (y * t["dy"].detach().cpu().to(dtype)).sum()
        if dstate is not None and out is not None:
            loss = loss + (out.h * dstate["h"].cpu().to(dtype)).sum()
            loss = loss + (out.last_u * dstate["last_u"].cpu().to(dtype)).sum()
            if out.angle is not None and dstate.get("angle") is not None:
                loss = loss + (out.angle * dstate["angle"].cpu().to(dtype)).sum()
        gl = torch.autograd.grad(loss, [leaf[n] for n in names], allow_unused=True)
        g = {n: v for n, v in zip(names, gl) if v is not None}
    return y.detach(), out, g


def fused_run(t: dict, chunk: int, want_state=True, grads=True, dstate=None, discretization=None,
              path=0, device="cuda", reverse_heads=0):
    """Run the fused op on the GPU through the public host API (and so the C ABI)."""
    from mamba_trainer_b200.ssm import Discretization, ScanInputs, SsmState, mamba3_scan
    names = [n for n in GRAD_NAMES if t.get(n) is not None]
    leaf = {n: t[n].detach().to(device).requires_grad_(grads) for n in names}
    inp = ScanInputs.new(leaf["x"], leaf["b"], leaf["c"], leaf["dt"], leaf["a_log"], leaf.get("lam"))
    inp = inp.with_chunk_size(chunk).with_state_output(want_state).with_path(path).with_reverse_heads(reverse_heads)
    if discretization is not None:
        inp = inp.with_discretization(discretization)
    if "theta" in leaf:
        inp = inp.with_theta(leaf["theta"])
    if "d_skip" in leaf:
        inp = inp.with_skip(leaf["d_skip"])
    if "h0" in leaf:
        inp = inp.with_state(SsmState(leaf["h0"], leaf["last_u0"], leaf.get("angle0")))
    out = mamba3_scan(inp)
    g = {}
    if grads:
        loss = (out.y.float() * t["dy"].to(device).float()).sum()
        if dstate is not None and out.state is not None:
            loss = loss + (out.state.h * dstate["h"].to(device)).sum()
            loss = loss + (out.state.last_u * dstate["last_u"].to(device)).sum()
            if out.state.angle is not None and dstate.get("angle") is not None:
                loss = loss + (out.state.angle * dstate["angle"].to(device)).sum()
        use = [n for n in names if not (n == "lam" and discretization is not None and int(discretization) != 2)]
        gl = torch.autograd.grad(loss, [leaf[n] for n in use], allow_unused=True)
        g = {n: v.detach() for n, v in zip(use, gl) if v is not None}
    return out.y.detach(), out.state, g


def angle_close(a, e, tol) -> bool:
    """Angles compared on the circle (a wrap may land on +pi or -pi)."""
    a, e = a.detach().double().cpu(), e.detach().double().cpu()
    return float((torch.sin(a) - torch.sin(e)).abs().max()) < tol and \
        float((torch.cos(a) - torch.cos(e)).abs().max()) < tol


def reference_mode_error(t: dict, chunk: int, exact: dict, names, want_state=False) -> dict:
    """||r - e|| / ||e|| per gradient in `names`, where r comes from the oracle run in float32 with the
    REFERENCE's own bf16 matmul mode and e = `exact` from the float64 oracle on the same inputs: how far
    the reference's reduced-precision arithmetic itself sits from exact arithmetic.  The yardstick for
    gradients whose bf16 error is dominated by cancellation (d theta: the d phi of a stripe sum to zero;
    d a_log, d dt_bias: sums over every token)."""
    _, _, g = oracle_run(t, chunk, want_state, torch.float32, True, matmul_narrow=torch.bfloat16)
    return {n: norm_rel(g[n].double(), exact[n]) for n in names if n in g and n in exact}
