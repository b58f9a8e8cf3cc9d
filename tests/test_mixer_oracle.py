"""Pin the CPU restatement of the mixer steps around the scan against the reference port's outputs."""
from pathlib import Path

import numpy as np
import torch

from oracle import mixer as M

GOLD = Path(__file__).resolve().parent / "golden"
T64 = lambda a, g=False: torch.tensor(np.asarray(a, dtype=np.float64), requires_grad=g)


def rel_err(a, e):
    a, e = np.asarray(a, dtype=np.float64), np.asarray(e, dtype=np.float64)
    return float(np.max(np.abs(a - e) / (1.0 + np.abs(e)))) if a.size else 0.0


def conv_golden():
    z = np.load(GOLD / "conv_silu.npz")
    # the port keeps the taps as nn.Conv1d does, [C, 1, K]; tap k of [K, C] is w[:, 0, k]
    return z, np.ascontiguousarray(z["w"][:, 0, :].T)


def test_conv_silu_matches_reference_port():
    z, w = conv_golden()
    x, wt, b = T64(z["x"], True), T64(w, True), T64(z["b"], True)
    y, hist = M.causal_conv1d(x, wt, b)
    assert rel_err(y.detach(), z["y"]) < 1e-13
    dx, dw, db = torch.autograd.grad((y * T64(z["dy"])).sum(), [x, wt, b])
    assert rel_err(dx, z["dx"]) < 1e-13 and rel_err(db, z["db"]) < 1e-13
    assert rel_err(dw, z["dw"][:, 0, :].T) < 1e-12
    assert torch.equal(hist, x.detach()[:, -3:])


def test_conv_windows_with_history_equal_one_pass():
    """tests of apply_with_history in the reference (src/nn/conv.rs:185-203): two windows, the
    second continued from the first's history, equal the whole sequence."""
    z, w = conv_golden()
    x, wt, b = T64(z["x"]), T64(w), T64(z["b"])
    full, _ = M.causal_conv1d(x, wt, b)
    y1, h1 = M.causal_conv1d(x[:, :2], wt, b)          # shorter than the K-1 = 3 taps of history
    y2, h2 = M.causal_conv1d(x[:, 2:7], wt, b, h1)
    y3, _ = M.causal_conv1d(x[:, 7:], wt, b, h2)
    assert rel_err(torch.cat([y1, y2, y3], 1), full) < 1e-14


def core_golden():
    z = np.load(GOLD / "mixer_core.npz")
    p = {"conv_w": np.ascontiguousarray(z["conv_w"][:, 0, :].T), "conv_b": z["conv_b"], "dt_bias": z["dt_bias"],
         "a_log": z["a_log"], "d_skip": z["d_skip"], "b_bias": z["b_bias"], "c_bias": z["c_bias"], "norm_w": z["norm_w"]}
    return z, p


def test_mixer_core_matches_reference_port():
    """The whole stretch between the port's two projections: values and the gradient of every
    parameter and of the projection itself."""
    z, p = core_golden()
    B, T, H, P, N = (int(v) for v in z["dims"])
    proj = T64(z["proj"], True)
    pt = {k: T64(v, True) for k, v in p.items()}
    gated, _, _ = M.mixer_core(proj, pt, H, P, N, chunk=int(z["chunk"]), eps=float(z["eps"]))
    assert rel_err(gated.detach(), z["gated"]) < 1e-12
    names = list(pt)
    grads = torch.autograd.grad((gated * T64(z["dgated"])).sum(), [proj] + [pt[n] for n in names])
    assert rel_err(grads[0], z["dproj"]) < 1e-11
    for n, g in zip(names, grads[1:]):
        want = z["d_" + n]
        if n == "conv_w":
            want = want[:, 0, :].T
        assert rel_err(g, want) < 1e-11, n


def test_post_gate_norm_is_the_norm_of_the_ungated_output_times_the_gate():
    """SsmConfig::post_gate_norm (src/ssm/config.rs:113; Mamba3Mixer::finish, src/models/mamba3.rs:475-484;
    RmsNorm::apply, src/nn/norm.rs:95-105): gated' = rms_norm(y) * gain * silu(z) where the port's own path
    gives gated = y * silu(z).  The port has no such switch, so the branch is pinned through the port's vectors
    for everything up to y (y = gated / silu(z)) and the norm's definition written out here."""
    z, p = core_golden()
    B, T, H, P, N = (int(v) for v in z["dims"])
    d_inner = H * P
    proj = T64(z["proj"])
    pt = {k: T64(v) for k, v in p.items()}
    g = torch.Generator().manual_seed(4)
    pt["post_norm_w"] = 1.0 + 0.3 * torch.randn(d_inner, generator=g, dtype=torch.float64)
    got, _, _ = M.mixer_core(proj, pt, H, P, N, chunk=int(z["chunk"]), eps=float(z["eps"]), post_gate_norm=True)
    gate = torch.nn.functional.silu(proj[..., :d_inner])
    y = T64(z["gated"]) / gate                                   # the port's scan output, flattened
    want = y / torch.sqrt((y * y).mean(-1, keepdim=True) + float(z["eps"])) * pt["post_norm_w"] * gate
    assert rel_err(got, want) < 1e-9
    # without a gain the norm still applies
    del pt["post_norm_w"]
    got1, _, _ = M.mixer_core(proj, pt, H, P, N, chunk=int(z["chunk"]), eps=float(z["eps"]), post_gate_norm=True)
    assert rel_err(got1, want / (1.0 + 0.3 * torch.randn(d_inner, generator=torch.Generator().manual_seed(4), dtype=torch.float64))) < 1e-9
