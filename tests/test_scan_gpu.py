"""Parity of the fused CUDA scan with the oracle, through the host API and the C ABI.

Tolerances (written here, as the contract asks):
  float32 inputs:  |a - e| <= 1e-5 * scale + 1e-4 |e|, scale = max(1, max|e|) of the tensor
  bfloat16 inputs: ||a - e|| / ||e|| <= 2e-2 per tensor, and the reference's own
                   measure max |a - e| / (1 + |e|) <= 2e-2 * max(1, max|e|)
The expected values come from the float64 oracle fed the same (rounded) inputs, so a
correct kernel is never blamed for the float32 oracle's own rounding.
"""
import math

import numpy as np
import pytest
import torch

from mamba_trainer_b200 import synthetic
from mamba_trainer_b200.error import ConfigError, RankError, ShapeError
from mamba_trainer_b200.ssm import Discretization, ScanInputs, SsmState, mamba3_scan
from oracle.recurrence import Case, recurrence
from tests._util import (allclose_excess, angle_close, fused_run, norm_rel, oracle_run, ref_metric,
                         reference_mode_error)

pytestmark = pytest.mark.gpu


# How the float32 comparisons fare at the FLAT tolerance 1e-5 + 1e-4 |e| (no scaling of the absolute term
# by the tensor's magnitude): counted over the session and printed by the last test of this file.
F32_FLAT = {"tensors": 0, "pass_flat": 0, "worst_flat_excess": 0.0, "worst": ""}


def check_f32(name, a, e):
    scale = max(1.0, float(e.abs().max())) if e.numel() else 1.0
    ex = allclose_excess(a, e, 1e-4, 1e-5 * scale)
    flat = allclose_excess(a, e, 1e-4, 1e-5)
    F32_FLAT["tensors"] += 1
    F32_FLAT["pass_flat"] += int(flat <= 1.0)
    if flat > F32_FLAT["worst_flat_excess"]:
        F32_FLAT["worst_flat_excess"], F32_FLAT["worst"] = flat, f"{name} (max|e| = {scale:.1f})"
    assert ex <= 1.0, f"{name}: {ex:.2f}x over the float32 tolerance"


def check_bf16(name, a, e):
    scale = max(1.0, float(e.abs().max())) if e.numel() else 1.0
    nr, rm = norm_rel(a.float(), e), ref_metric(a.float(), e)
    assert nr <= 2e-2, f"{name}: norm-relative error {nr:.3e}"
    assert rm <= 2e-2 * scale, f"{name}: reference metric {rm:.3e} (scale {scale:.2f})"


def compare_all(t, chunk, check, want_state=True, dstate=None, discretization=None, path=0, reverse_heads=0):
    y, st, g = fused_run(t, chunk, want_state, True, dstate, discretization, path, reverse_heads=reverse_heads)
    ey, est, eg = oracle_run(t, chunk, want_state, torch.float64, True, dstate, reverse_heads=reverse_heads)
    check("y", y, ey)
    if want_state:
        check("h", st.h, est.h.detach())
        check("last_u", st.last_u, est.last_u.detach())
        if est.angle is not None:
            assert angle_close(st.angle, est.angle.detach(), 2e-3), "angle"
    else:
        assert st is None
    for n, e in eg.items():
        if n == "lam" and discretization is not None and int(discretization) != 2:
            continue
        assert n in g, f"missing gradient {n}"
        check("d" + n, g[n], e)


def case_tensors(case, rank1=True, theta=False, d_skip=None):
    f = lambda v: torch.tensor(v, dtype=torch.float32)
    t = {"x": f(case.x).unsqueeze(-1), "b": f(case.b).unsqueeze(-1), "c": f(case.c).unsqueeze(-1),
         "dt": f(case.dt), "lam": f(case.lam), "a_log": f(case.a_log)}
    if theta:
        t["theta"] = f(case.theta())
    if d_skip is not None:
        t["d_skip"] = f(np.asarray(d_skip, dtype=np.float32))
    t["dy"] = torch.randn(t["x"].shape, generator=torch.Generator().manual_seed(3))
    return t


def np_rec(t):
    g = lambda k: None if t.get(k) is None else t[k].double().numpy()
    return recurrence(g("x"), g("b"), g("c"), g("dt"), g("a_log"), g("lam"), g("theta"), g("d_skip"),
                      g("h0"), g("last_u0"), g("angle0"))


# ---- the reference's own scan tests, replayed against the fused op ----------------

@pytest.mark.parametrize("chunk", [1, 2, 3, 4, 8, 16])
def test_chunked_scan_matches_the_recurrence(chunk):
    """tests/ssm.rs:187-205, eps 2e-4."""
    t = case_tensors(Case(2, 12, 3, 4, 6))
    y, st, _ = fused_run(t, chunk, True, False)
    wy, wh, wu, _ = np_rec(t)
    assert ref_metric(y, wy) <= 2e-4 and ref_metric(st.h, wh) <= 2e-4 and ref_metric(st.last_u, wu) <= 2e-4


@pytest.mark.parametrize("seq", [1, 5, 7, 13])
def test_chunked_scan_handles_ragged_lengths(seq):
    """tests/ssm.rs:207-220."""
    t = case_tensors(Case(1, seq, 2, 3, 4))
    y, st, _ = fused_run(t, 4, True, False)
    wy, wh, _, _ = np_rec(t)
    assert ref_metric(y, wy) <= 2e-4 and ref_metric(st.h, wh) <= 2e-4


def test_euler_mode_reproduces_mamba2():
    """tests/ssm.rs:222-236: lambda = 1, and want_state = false returns no state."""
    case = Case(1, 8, 2, 3, 4)
    case.lam = np.ones_like(case.lam)
    t = case_tensors(case)
    wy, _, _, _ = np_rec(t)
    y, st, _ = fused_run(t, 4, False, False)
    assert st is None and ref_metric(y, wy) <= 2e-4
    t2 = dict(t, lam=None)  # the constant-lambda fast path must agree with lambda == 1
    y2, _, _ = fused_run(t2, 4, False, False, discretization=Discretization.Euler)
    assert ref_metric(y2, wy) <= 2e-4


def test_split_windows_match_a_single_pass():
    """tests/ssm.rs:238-310, eps 3e-4: cut at 5 of 12, state carried across the seam."""
    t = case_tensors(Case(2, 12, 2, 3, 4), theta=True)
    full_y, full_st, _ = fused_run(t, 4, True, False)
    cut = lambda s: {k: (v[:, s] if (v is not None and v.dim() >= 3) else v) for k, v in t.items()}
    y1, s1, _ = fused_run(cut(slice(0, 5)), 4, True, False)
    t2 = dict(cut(slice(5, 12)), h0=s1.h, last_u0=s1.last_u, angle0=s1.angle)
    y2, s2, _ = fused_run(t2, 4, True, False)
    assert ref_metric(torch.cat([y1, y2], 1), full_y) <= 3e-4
    assert ref_metric(s2.h, full_st.h) <= 3e-4


def test_step_recurrence_matches_the_chunked_scan():
    """tests/ssm.rs:312-380: rotation + D skip, token-by-token evaluation vs the scan."""
    t = case_tensors(Case(2, 9, 2, 3, 4), theta=True, d_skip=[0.3, -0.2])
    y, _, _ = fused_run(t, 4, True, False)
    wy, _, _, _ = np_rec(t)
    assert ref_metric(y, wy) <= 3e-4


def test_scan_is_differentiable():
    """tests/ssm.rs:382-426: d/dx of sum(y^2) against central differences."""
    case = Case(1, 6, 2, 3, 4)
    t = case_tensors(case)
    x = t["x"].cuda().requires_grad_(True)
    dev = {k: (v.cuda() if v is not None else None) for k, v in t.items()}

    def run(xv):
        inp = ScanInputs.new(xv, dev["b"], dev["c"], dev["dt"], dev["a_log"], dev["lam"])
        return mamba3_scan(inp.with_chunk_size(3).with_state_output(False)).y

    loss = (run(x) ** 2).sum()
    (analytic,) = torch.autograd.grad(loss, [x])
    eps = 1e-3
    for i in (0, 5, 17, 30):
        plus, minus = t["x"].clone().view(-1), t["x"].clone().view(-1)
        plus[i] += eps
        minus[i] -= eps
        f = lambda v: float((run(v.view_as(t["x"]).cuda()) ** 2).sum())
        numeric = (f(plus) - f(minus)) / (2 * eps)
        assert abs(float(analytic.view(-1)[i]) - numeric) < 2e-2 * (1 + abs(numeric))


# ---- all inputs' gradients, every variant, small float32 shapes --------------------

def small_inputs(B, T, H, P, N, R, rot, state, seed):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    u = lambda *s: torch.rand(*s, generator=g)
    t = {"x": r(B, T, H, P, R), "b": r(B, T, H, N, R), "c": r(B, T, H, N, R), "dt": u(B, T, H) * 0.5 + 0.05,
         "lam": u(B, T, H), "a_log": u(H), "d_skip": r(H), "dy": r(B, T, H, P, R)}
    t["theta"] = u(B, T, H, N // 2) * 3 if rot else None
    if state:
        t["h0"], t["last_u0"] = r(B, H, P, N), r(B, H, P, N)
        t["angle0"] = (u(B, H, N // 2) * 2 - 1) * 3 if rot else None
    ds = {"h": r(B, H, P, N), "last_u": r(B, H, P, N), "angle": r(B, H, N // 2) if rot else None}
    return t, ds


@pytest.mark.parametrize("B,T,H,P,N,R,L,rot,state", [
    (2, 12, 2, 3, 4, 2, 4, True, True),
    (1, 13, 2, 3, 4, 1, 4, False, False),
    (2, 7, 1, 5, 6, 3, 16, True, False),
    (1, 9, 2, 4, 4, 2, 3, True, True),
    (1, 70, 2, 8, 16, 4, 32, True, True),
    (2, 150, 3, 72, 80, 1, 64, False, True),
    (1, 130, 2, 16, 24, 5, 64, True, False),
])
def test_every_gradient_matches_the_oracle_f32(B, T, H, P, N, R, L, rot, state):
    t, ds = small_inputs(B, T, H, P, N, R, rot, state, seed=B * 100 + T)
    compare_all(t, L, check_f32, True, ds)


@pytest.mark.parametrize("disc", [Discretization.Euler, Discretization.Trapezoid])
def test_fixed_lambda_modes(disc):
    t, ds = small_inputs(2, 21, 2, 4, 6, 2, True, True, seed=5)
    t["lam"] = torch.full_like(t["lam"], disc.fixed_lambda())
    compare_all(t, 8, check_f32, True, ds, discretization=disc)


def test_grad_mask_and_repeatable_backward():
    t, _ = small_inputs(1, 20, 2, 4, 6, 2, True, False, seed=9)
    dev = {k: (v.cuda() if v is not None else None) for k, v in t.items()}
    dev["b"].requires_grad_(True)
    dev["a_log"].requires_grad_(True)
    inp = ScanInputs.new(dev["x"], dev["b"], dev["c"], dev["dt"], dev["a_log"], dev["lam"]).with_theta(dev["theta"])
    out = mamba3_scan(inp.with_chunk_size(8))
    loss = (out.y * dev["dy"]).sum()
    g1 = torch.autograd.grad(loss, [dev["b"], dev["a_log"]], retain_graph=True)
    g2 = torch.autograd.grad(loss, [dev["b"], dev["a_log"]])
    assert torch.equal(g1[0], g2[0]) and torch.equal(g1[1], g2[1])
    _, _, eg = oracle_run(t, 8, True)
    check_f32("db", g1[0], eg["b"])
    check_f32("da_log", g1[1], eg["a_log"])
    with torch.no_grad():
        y2 = mamba3_scan(inp).y
    assert not y2.requires_grad


# ---- the benchmark configurations ---------------------------------------------------

def test_config0_full_size_f32():
    w = synthetic.WORKLOADS[0]
    t = synthetic.make_inputs(w, seed=0)
    compare_all(t, w.chunk, check_f32, True, None)                       # lambda read as a tensor of ones
    compare_all(t, w.chunk, check_f32, False, None, discretization=Discretization.Euler)


@pytest.mark.parametrize("idx,batch,heads,seq", [(1, 1, 12, 2048), (2, 1, 4, 2048), (3, 4, 2, 1024), (4, 4, 2, 1024)])
def test_bf16_configs_reduced_batch(idx, batch, heads, seq):
    # Reduced so the CPU oracle finishes in seconds.  The per-head gradients (a_log, D) are sums
    # over every token of the shard with heavy cancellation: with bf16 tensor-core operands their
    # relative error shrinks with the number of tokens summed, so the MIMO cases keep 4 sequences.
    w = synthetic.WORKLOADS[idx].scaled(batch=batch, heads=heads, seq=seq)
    t = synthetic.make_inputs(w, seed=idx)
    compare_all(t, w.chunk, check_bf16, True, None)


@pytest.mark.parametrize("idx", [1, 2, 3, 4])
def test_bf16_configs_full_size(idx):
    """The benchmark configurations at their full size (config 4: one GPU's shard of the 8-way run,
    batch 8).  The oracle cannot run them whole, so: (a) sampled (batch, head) stripes - each an
    independent recurrence - against the oracle in float64, values, final state and every per-token
    gradient; (a') d a_log and d D of one head against the oracle summed over all of the head's stripes;
    (b) the backward pass is linear in dy: doubling dy doubles every gradient exactly;
    (c) two windows with the state carried across equal one pass (tests/ssm.rs:238-310)."""
    w = synthetic.WORKLOADS[idx]
    if idx == 4:
        w = w.scaled(batch=8)
    t = synthetic.make_inputs(w, seed=idx, device="cuda")
    names = [n for n in ("x", "b", "c", "dt", "lam", "theta", "a_log", "d_skip") if t.get(n) is not None]
    leaf = {n: t[n].detach().requires_grad_(True) for n in names}

    def build(sl=slice(None), state=None):
        inp = ScanInputs.new(leaf["x"][:, sl], leaf["b"][:, sl], leaf["c"][:, sl], leaf["dt"][:, sl], leaf["a_log"],
                             leaf["lam"][:, sl]).with_chunk_size(w.chunk).with_skip(leaf["d_skip"])
        if "theta" in leaf:
            inp = inp.with_theta(leaf["theta"][:, sl])
        return inp.with_state(state) if state is not None else inp

    out = mamba3_scan(build())
    grads = torch.autograd.grad(out.y, [leaf[n] for n in names], grad_outputs=t["dy"], retain_graph=True)
    g = dict(zip(names, grads))
    # (a) sampled stripes
    B, H = w.batch, w.heads
    for b_, h_ in ((0, 0), (B - 1, H - 1), (B // 2, H // 3)):
        cut = lambda v: v[b_:b_ + 1, :, h_:h_ + 1].detach().cpu()
        st = {n: cut(t[n]) for n in ("x", "b", "c", "dt", "lam", "theta", "dy") if t.get(n) is not None}
        st["a_log"], st["d_skip"] = t["a_log"][h_:h_ + 1].cpu(), t["d_skip"][h_:h_ + 1].cpu()
        ey, est, eg = oracle_run(st, w.chunk, True, torch.float64, True)
        check_bf16(f"y[{b_},{h_}]", cut(out.y), ey)
        check_bf16("h", out.state.h[b_:b_ + 1, h_:h_ + 1].cpu(), est.h.detach())
        check_bf16("last_u", out.state.last_u[b_:b_ + 1, h_:h_ + 1].cpu(), est.last_u.detach())
        if est.angle is not None:
            assert angle_close(out.state.angle[b_:b_ + 1, h_:h_ + 1].cpu(), est.angle.detach(), 2e-2)
        for n in ("x", "b", "c", "dt", "lam"):
            check_bf16(f"d{n}[{b_},{h_}]", cut(g[n]), eg[n])
        if "theta" in eg:
            # d theta = dt * (sum of d phi over every later step), and the d phi of a stripe sum to zero
            # (rotating B and C together changes nothing): the running sum is a difference of large
            # cancelling terms, so ANY bf16 rounding of matmul operands shows up amplified, growing with
            # sqrt(T).  The yardstick is the reference itself: its own bf16 matmul mode (oracle with
            # matmul_precision, src/tensor/ops/matmul.rs:94-128) on the same stripe is off from exact
            # arithmetic by 4-5 % (tests/test_oracle.py pins that figure); the CUDA path must be at least as
            # close as that, and meet the plain 2e-2 in the reference's own measure.
            a_, e_ = cut(g["theta"]).float(), eg["theta"]
            yard = reference_mode_error(st, w.chunk, eg, ("theta",))["theta"]
            assert ref_metric(a_, e_) <= 2e-2, f"dtheta[{b_},{h_}]: reference metric {ref_metric(a_, e_):.3e}"
            assert norm_rel(a_, e_) <= max(2e-2, yard), \
                f"dtheta[{b_},{h_}]: norm-relative error {norm_rel(a_, e_):.3e}, the reference's bf16 mode: {yard:.3e}"
    # (a') the per-head parameter gradients of ONE head: d a_log and d D sum over every batch row and token
    # of the head, so the oracle runs all B stripes of that head and its results are added up
    h_ = H // 3
    want = {"a_log": 0.0, "d_skip": 0.0}
    for b_ in range(B):
        cut = lambda v: v[b_:b_ + 1, :, h_:h_ + 1].detach().cpu()
        st = {n: cut(t[n]) for n in ("x", "b", "c", "dt", "lam", "theta", "dy") if t.get(n) is not None}
        st["a_log"], st["d_skip"] = t["a_log"][h_:h_ + 1].cpu(), t["d_skip"][h_:h_ + 1].cpu()
        _, _, eg = oracle_run(st, w.chunk, False, torch.float64, True)
        for n in want:
            want[n] = want[n] + eg[n].double()
    for n, e_ in want.items():
        a_ = g[n][h_:h_ + 1].detach().double().cpu()
        err = float((a_ - e_).abs() / e_.abs().clamp_min(1.0))
        assert err <= 2e-2, f"d{n}[head {h_}]: {float(a_):.6g} against {float(e_):.6g} ({err:.3e})"
    # (b) linearity in dy (a factor of two is exact in every format involved)
    g2 = torch.autograd.grad(out.y, [leaf[n] for n in names], grad_outputs=t["dy"] * 2)
    for n, a_, b2 in zip(names, grads, g2):
        assert torch.equal(a_ * 2, b2), n
    # (c) two windows, state carried
    half = (w.seq // 2 // 128) * 128
    with torch.no_grad():
        o1 = mamba3_scan(build(slice(0, half)))
        o2 = mamba3_scan(build(slice(half, w.seq), o1.state))
    check_bf16("windows y", torch.cat([o1.y, o2.y], 1), out.y.detach().float())
    check_bf16("windows h", o2.state.h, out.state.h.detach())


# ---- a bounded device-side wait that runs out (no fault, no hang: the kernels give up and say so) ----

@pytest.mark.parametrize("idx,kw", [(4, dict(batch=1, heads=2, seq=700)), (1, dict(batch=1, heads=2, seq=512)),
                                    (4, dict(batch=5, heads=32, seq=640))])
def test_a_wait_that_runs_out_is_reported_and_the_context_stays_usable(idx, kw):
    """Every device-side wait of the tensor-core kernels has an iteration limit.  With the limit set to one
    poll (m3_ctx_set_wait_limit) the first wait of every CTA gives up before its products or copies have
    finished: the kernels must return by themselves, the condition must surface as DeviceTimeout - at
    Context.sync() and, for callers that never sync, on entry to the next scan call - and once the limit
    is back to its default the same context must compute correct results again.  Covers the role-split
    kernels (rank 2, rotational), the direct form (rank 1, real dynamics) and stripes cut into time segments
    (160 stripes on 148 SMs: a CTA that gave up still raises its hand-over flag, and the wait for a
    predecessor's flag is bounded like every other)."""
    from mamba_trainer_b200.error import DeviceTimeout
    from mamba_trainer_b200.ssm import Context
    w = synthetic.WORKLOADS[idx].scaled(**kw)
    t = synthetic.make_inputs(w, seed=21)
    good_y, _, good_g = fused_run(t, w.chunk, False)
    ctx = Context.for_device(torch.device("cuda", torch.cuda.current_device()))
    ctx.sync()
    try:
        ctx.set_wait_limit(1)
        with pytest.raises(DeviceTimeout):
            fused_run(t, w.chunk, False)      # the forward gives up; the backward call may already see it on entry
            ctx.sync()                        # ... and if it was too early for that, the sync does
        torch.cuda.synchronize()
        try:
            ctx.sync()                        # whatever the backward raised meanwhile is reported once, then clear
        except DeviceTimeout:
            pass
        ctx.sync()
        fused_run(t, w.chunk, False, grads=False)
        torch.cuda.synchronize()
        with pytest.raises(DeviceTimeout):    # a caller that never syncs learns of it at its next call
            fused_run(t, w.chunk, False, grads=False)
    finally:
        ctx.set_wait_limit(0)
        torch.cuda.synchronize()
        try:
            ctx.sync()
        except DeviceTimeout:
            pass
    y, _, g = fused_run(t, w.chunk, False)
    assert torch.equal(y, good_y)
    for n in good_g:
        assert torch.equal(g[n], good_g[n]), n


# ---- error behaviour (src/ssm/scan.rs:462, :485-489; src/error.rs) -------------------

def test_errors_mirror_the_reference():
    t, _ = small_inputs(1, 4, 1, 2, 3, 1, False, False, seed=1)
    dev = {k: (v.cuda() if v is not None else None) for k, v in t.items()}
    with pytest.raises(RankError):
        mamba3_scan(ScanInputs.new(dev["x"][..., 0], dev["b"], dev["c"], dev["dt"], dev["a_log"], dev["lam"]))
    with pytest.raises(ConfigError):
        th = torch.zeros(1, 4, 1, 1, device="cuda")
        mamba3_scan(ScanInputs.new(dev["x"], dev["b"], dev["c"], dev["dt"], dev["a_log"], dev["lam"]).with_theta(th))
    with pytest.raises(ShapeError):
        mamba3_scan(ScanInputs.new(dev["x"], dev["b"], dev["c"], dev["dt"][:, :2], dev["a_log"], dev["lam"]))


def test_empty_sequence_passes_state_through():
    x = torch.zeros(2, 0, 3, 4, 1, device="cuda")
    b = torch.zeros(2, 0, 3, 6, 1, device="cuda")
    z = torch.zeros(2, 0, 3, device="cuda")
    st = SsmState(torch.randn(2, 3, 4, 6, device="cuda"), torch.randn(2, 3, 4, 6, device="cuda"))
    out = mamba3_scan(ScanInputs.new(x, b, b, z, torch.zeros(3, device="cuda"), z).with_state(st))
    assert out.y.shape == x.shape and torch.equal(out.state.h, st.h)


# ---- tensor-core family (tcgen05 / TMEM), explicit path = 2 --------------------------------

def tc_workload(rank, rot, seq, batch=2, heads=2, disc=Discretization.LearnedTrapezoid, bc="scaled"):
    return synthetic.Workload("tc_case", batch, seq, heads, 64, 128, 64, rank, torch.bfloat16, disc, rot, bc)


@pytest.mark.parametrize("rank,rot,seq,state,disc", [
    (1, False, 300, True, Discretization.LearnedTrapezoid),
    (1, True, 256, False, Discretization.LearnedTrapezoid),
    (1, False, 128, False, Discretization.Euler),
    (1, False, 200, True, Discretization.LearnedTrapezoid),    # bulk-copy path with a ragged last tile
    (1, False, 384, False, Discretization.Trapezoid),          # bulk-copy path, three full tiles
    (2, True, 200, True, Discretization.LearnedTrapezoid),
    (4, True, 130, True, Discretization.Trapezoid),
    (4, False, 64, False, Discretization.LearnedTrapezoid),
    (1, True, 1, True, Discretization.LearnedTrapezoid),
])
def test_tensor_core_forward(rank, rot, seq, state, disc):
    w = tc_workload(rank, rot, seq, disc=disc, bc="rms" if rank == 1 else "scaled")
    t = synthetic.make_inputs(w, seed=rank * 10 + seq, with_state=state)
    y, st, _ = fused_run(t, w.chunk, True, False, None, disc, path=2)
    ey, est, _ = oracle_run(t, w.chunk, True, torch.float64, False)
    check_bf16("y", y, ey)
    check_bf16("h", st.h, est.h)
    check_bf16("last_u", st.last_u, est.last_u)
    if rot:
        assert angle_close(st.angle, est.angle, 2e-2), "angle"


@pytest.mark.parametrize("rank,rot,seq,state,disc", [
    (1, False, 300, True, Discretization.LearnedTrapezoid),
    (1, True, 256, False, Discretization.LearnedTrapezoid),
    (1, False, 128, False, Discretization.Euler),
    (1, False, 200, True, Discretization.LearnedTrapezoid),    # bulk-copy path with a ragged last tile
    (1, False, 384, False, Discretization.Trapezoid),          # bulk-copy path, three full tiles
    (2, True, 200, True, Discretization.LearnedTrapezoid),
    (4, True, 130, True, Discretization.Trapezoid),
    (4, False, 64, False, Discretization.LearnedTrapezoid),
    (1, True, 1, True, Discretization.LearnedTrapezoid),
])
def test_tensor_core_backward(rank, rot, seq, state, disc):
    w = tc_workload(rank, rot, seq, disc=disc, bc="rms" if rank == 1 else "scaled")
    t = synthetic.make_inputs(w, seed=rank * 10 + seq + 1, with_state=state)
    g = torch.Generator().manual_seed(seq)
    ds = {"h": torch.randn(w.batch, w.heads, 64, 128, generator=g) * 0.1,
          "last_u": torch.randn(w.batch, w.heads, 64, 128, generator=g) * 0.1,
          "angle": torch.randn(w.batch, w.heads, 64, generator=g) * 0.1 if rot else None}
    compare_all(t, w.chunk, check_bf16, True, ds, discretization=disc, path=2)


@pytest.mark.parametrize("rank,rot,seq,rev", [(2, True, 1000, 1), (1, True, 1100, 0), (4, False, 520, 0), (2, False, 1000, 32)])
def test_time_segments_leave_results_unchanged(rank, rot, seq, rev):
    """With more stripes than SMs the kernels cut every stripe into time segments, possibly run by different
    CTAs, which hand the fp32 state (backward: its gradient) and the running angle over in global memory.
    The arithmetic and its order are those of whole stripes, so the results are identical: 160 stripes in one
    call (cut) against the same rows in calls of 64 and 96 stripes (never cut)."""
    w = tc_workload(rank, rot, seq, batch=5, heads=32)
    t = synthetic.make_inputs(w, seed=seq + rank, with_state=True)
    g = torch.Generator().manual_seed(seq)
    ds = {"h": torch.randn(w.batch, w.heads, 64, 128, generator=g) * 0.1,
          "last_u": torch.randn(w.batch, w.heads, 64, 128, generator=g) * 0.1,
          "angle": torch.randn(w.batch, w.heads, 64, generator=g) * 0.1 if rot else None}
    y, st, gr = fused_run(t, w.chunk, True, True, ds, path=2, reverse_heads=rev)
    per_head = ("a_log", "d_skip")
    sums = {}
    for lo, hi in ((0, 2), (2, 5)):
        tp = {k: (v if (v is None or k in per_head) else v[lo:hi]) for k, v in t.items()}
        dp = {k: (v if v is None else v[lo:hi]) for k, v in ds.items()}
        yp, sp, gp = fused_run(tp, w.chunk, True, True, dp, path=2, reverse_heads=rev)
        assert torch.equal(y[lo:hi], yp), "y"
        assert torch.equal(st.h[lo:hi], sp.h) and torch.equal(st.last_u[lo:hi], sp.last_u), "state"
        if rot:
            assert torch.equal(st.angle[lo:hi], sp.angle), "angle"
        for n, v in gp.items():
            if n in per_head:
                sums[n] = sums.get(n, 0) + v.double()
            else:
                assert torch.equal(gr[n][lo:hi], v), n
    for n, v in sums.items():
        assert torch.allclose(gr[n].double(), v, rtol=1e-4, atol=1e-4), n


def test_cut_stripe_launches_on_two_streams_do_not_wait_on_each_other():
    """Two launches whose CTAs wait on one another must not share the GPU (each could hold SMs the other's
    unscheduled CTAs are waited for on): the library chains them across streams.  Two cut-stripe scans
    enqueued back to back on two streams finish without a wait giving up and equal the same scans run alone."""
    from mamba_trainer_b200.ssm.scan import Context
    w = tc_workload(2, True, 2000, batch=5, heads=32)
    ts = [synthetic.make_inputs(w, seed=s_, device="cuda") for s_ in (11, 12)]

    def run(t):
        inp = ScanInputs.new(t["x"], t["b"], t["c"], t["dt"], t["a_log"], t["lam"]).with_chunk_size(w.chunk)
        inp = inp.with_theta(t["theta"]).with_skip(t["d_skip"]).with_state_output(False).with_path(2)
        with torch.no_grad():
            return mamba3_scan(inp).y

    alone = [run(t) for t in ts]
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    both = []
    for _ in range(3):
        for t, st in zip(ts, streams):
            with torch.cuda.stream(st):
                both.append(run(t))
    torch.cuda.synchronize()
    Context.for_device(torch.device("cuda")).sync()     # raises if a bounded wait gave up
    for i, y in enumerate(both):
        assert torch.equal(y, alone[i % 2]), i


def test_misaligned_rows_take_the_generic_family():
    """The tensor-core kernels move rows as 16-byte vectors and bulk tensor copies.  An input that is not
    16-byte aligned (a view that starts one element into its buffer) is served by the generic family when the
    path is left to the library, and refused when the tensor-core family is asked for by name."""
    from mamba_trainer_b200.error import UnsupportedError
    w = tc_workload(2, True, 200)
    t = synthetic.make_inputs(w, seed=9, device="cuda")
    flat = torch.empty(t["x"].numel() + 8, dtype=t["x"].dtype, device="cuda")
    off = flat[1:1 + t["x"].numel()].view(t["x"].shape)
    off.copy_(t["x"])
    assert off.data_ptr() % 16 != 0 and off.is_contiguous()

    def run(path):
        inp = ScanInputs.new(off, t["b"], t["c"], t["dt"], t["a_log"], t["lam"]).with_chunk_size(w.chunk)
        inp = inp.with_theta(t["theta"]).with_skip(t["d_skip"]).with_state_output(False).with_path(path)
        with torch.no_grad():
            return mamba3_scan(inp).y

    tc = {k: (v.cpu() if torch.is_tensor(v) else v) for k, v in t.items()}
    ey, _, _ = oracle_run(tc, w.chunk, False, torch.float64, False)
    check_bf16("y", run(0).cpu(), ey)
    with pytest.raises(UnsupportedError):
        run(2)


# ---- bidirectional mixer: the last heads walk right to left (models/mamba3.rs:352-370, :548-556) -----

@pytest.mark.parametrize("B,T,H,P,N,R,L,rot,state,rev", [
    (2, 12, 4, 3, 4, 2, 4, True, True, 2),      # the mixer's own split: half the heads
    (1, 13, 2, 3, 4, 1, 4, False, False, 2),    # every head reversed, ragged length
    (2, 70, 3, 8, 16, 4, 32, True, True, 1),    # one trailing head, chunk cap in play
    (1, 150, 2, 72, 80, 1, 64, False, True, 1),
])
def test_reversed_heads_match_the_oracle_f32(B, T, H, P, N, R, L, rot, state, rev):
    t, ds = small_inputs(B, T, H, P, N, R, rot, state, seed=B * 100 + T + rev)
    compare_all(t, L, check_f32, True, ds, reverse_heads=rev)


@pytest.mark.parametrize("rank,rot,seq,state,rev", [
    (1, False, 300, True, 1),
    (1, True, 256, False, 2),
    (2, True, 200, True, 1),
    (4, True, 130, True, 1),
])
def test_reversed_heads_tensor_core(rank, rot, seq, state, rev):
    w = tc_workload(rank, rot, seq, bc="rms" if rank == 1 else "scaled")
    t = synthetic.make_inputs(w, seed=rank * 10 + seq + 7, with_state=state)
    g = torch.Generator().manual_seed(seq)
    ds = {"h": torch.randn(w.batch, w.heads, 64, 128, generator=g) * 0.1,
          "last_u": torch.randn(w.batch, w.heads, 64, 128, generator=g) * 0.1,
          "angle": torch.randn(w.batch, w.heads, 64, generator=g) * 0.1 if rot else None}
    compare_all(t, w.chunk, check_bf16, True, ds, path=2, reverse_heads=rev)


def test_reversed_heads_equal_flipped_inputs_bitwise():
    """Walking a head right to left equals reversing that head's inputs, scanning left to right and
    reversing its output: the same arithmetic in the same order, so the results are identical."""
    from oracle.m3_oracle import reverse_bands_in_time as flip
    w = tc_workload(2, True, 200)
    t = synthetic.make_inputs(w, seed=3)
    y, _, g = fused_run(t, w.chunk, False, True, reverse_heads=1)
    tf = {k: (flip(v, 1) if k in ("x", "b", "c", "dt", "lam", "theta", "dy") else v) for k, v in t.items()}
    yf, _, gf = fused_run(tf, w.chunk, False, True)
    assert torch.equal(y.cpu(), flip(yf.cpu(), 1))
    for n in ("x", "b", "c", "dt", "lam", "theta"):
        assert torch.equal(g[n].cpu(), flip(gf[n].cpu(), 1)), n
    assert torch.equal(g["a_log"], gf["a_log"]) and torch.equal(g["d_skip"], gf["d_skip"])


# ---- ssd_chunked with the caller's own a, g, w (the reference's direct entry) ------------------------

def test_ssd_chunked_entry_matches_golden_and_oracle():
    """The reference port's golden vectors (tests/golden) through the CUDA path, values and all six
    gradients; then a carried state and a state gradient against the oracle."""
    from pathlib import Path
    from mamba_trainer_b200.ssm import ssd_chunked, shift_left
    from oracle import m3_oracle as O
    gold = Path(__file__).resolve().parent / "golden"
    for name in ("ssd_chunked_even", "ssd_chunked_ragged", "ssd_chunked_one_chunk"):
        z = np.load(gold / f"{name}.npz")
        leaves = [torch.tensor(z[k], dtype=torch.float32, device="cuda", requires_grad=True) for k in "xbcagw"]
        y, st = ssd_chunked(*leaves, None, int(z["chunk"]), True)
        check_f32("y " + name, y, torch.tensor(z["y"]))
        grads = torch.autograd.grad((y * torch.tensor(z["dy"], dtype=torch.float32, device="cuda")).sum(), leaves)
        for k, gr in zip("xbcagw", grads):
            check_f32(f"d{k} {name}", gr, torch.tensor(z[f"d{k}"]))
    # w built the reference's way: g + shift_left((1 - lambda) dt)   (tests/ssm.rs:176-184)
    case = Case(2, 12, 2, 3, 4)
    f = lambda v: torch.tensor(v, dtype=torch.float64)
    dt, lam = f(case.dt), f(case.lam)
    a, g = dt * f(case.a_head).view(1, 1, -1), lam * dt
    w = g + shift_left((1 - lam) * dt, 1)
    h0 = torch.randn(2, 2, 3, 4, dtype=torch.float64, generator=torch.Generator().manual_seed(2))
    dh = torch.randn(2, 2, 3, 4, dtype=torch.float64, generator=torch.Generator().manual_seed(3))
    cpu = [t.clone().requires_grad_(True) for t in (f(case.x), f(case.b), f(case.c), a, g, w, h0)]
    ey, est = O.ssd_chunked(*cpu[:6], cpu[6], 4, True)
    eg = torch.autograd.grad(ey.sum() + (est * dh).sum(), cpu)
    dev = [t.detach().float().cuda().requires_grad_(True) for t in cpu]
    y, st = ssd_chunked(*dev[:6], dev[6], 4, True)
    gg = torch.autograd.grad(y.sum() + (st * dh.float().cuda()).sum(), dev)
    check_f32("y", y, ey.detach())
    check_f32("state", st, est.detach())
    for n, a_, e_ in zip(("x", "b", "c", "a", "g", "w", "h0"), gg, eg):
        check_f32("d" + n, a_, e_)


def test_host_pipeline_matches_one_call():
    """Host-resident tensors through the sliced copy/compute pipeline equal one whole-batch call."""
    from mamba_trainer_b200.host_pipeline import HostScanPipeline
    w = tc_workload(2, True, 192, batch=5, heads=2)
    t = synthetic.make_inputs(w, seed=21)
    host = {n: t[n].pin_memory() for n in ("x", "b", "c", "dt", "lam", "theta", "dy")}
    params = {"a_log": t["a_log"].cuda().requires_grad_(True), "d_skip": t["d_skip"].cuda().requires_grad_(True)}
    pipe = HostScanPipeline(host, w.chunk, w.discretization, "cuda", slices=3)
    for _ in range(2):   # twice: buffers and streams are reused
        out = pipe.run(host, params, wait=True)
    y, _, g = fused_run(t, w.chunk, False, True)
    assert torch.equal(out["y"], y.cpu())
    for n in ("x", "b", "c", "dt", "lam", "theta"):
        assert torch.equal(out["d" + n], g[n].cpu()), n
    check_f32("da_log", out["da_log"], g["a_log"].cpu())     # summed over slices in a different order
    check_f32("dd_skip", out["dd_skip"], g["d_skip"].cpu())
    # Two runs in flight at once: each delivers into its own output set.
    host2 = dict(host, dy=(t["dy"] * 2).pin_memory())
    out1 = pipe.run(host, params)
    out2 = pipe.run(host2, params)
    pipe.wait(out1)
    assert torch.equal(out1["dx"], g["x"].cpu())
    pipe.wait(out2)
    assert torch.equal(out2["y"], y.cpu())
    assert torch.equal(out2["dx"], (g["x"] * 2).cpu())       # the adjoint is linear in dy (a power of two is exact)
    pipe.close()


def test_host_pipeline_single_slice_f32_generic_path():
    """One slice, float32, no rotation, constant lambda: the generic family through the same pipeline."""
    from mamba_trainer_b200.host_pipeline import HostScanPipeline
    t, _ = small_inputs(3, 37, 2, 8, 6, 2, False, False, seed=5)
    host = {n: t[n].pin_memory() for n in ("x", "b", "c", "dt", "dy")}
    params = {"a_log": t["a_log"].cuda().requires_grad_(True), "d_skip": t["d_skip"].cuda().requires_grad_(True)}
    pipe = HostScanPipeline(host, 16, Discretization.Trapezoid, "cuda", slices=1)
    out = pipe.run(host, params, wait=True)
    dev = {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in t.items()}
    for k in ("x", "b", "c", "dt", "a_log", "d_skip"):
        dev[k] = dev[k].detach().requires_grad_(True)
    inp = ScanInputs.new(dev["x"], dev["b"], dev["c"], dev["dt"], dev["a_log"], None).with_chunk_size(16)
    inp = inp.with_state_output(False).with_discretization(Discretization.Trapezoid).with_skip(dev["d_skip"])
    y = mamba3_scan(inp).y
    gr = torch.autograd.grad(y, [dev[k] for k in ("x", "b", "c", "dt", "a_log", "d_skip")], grad_outputs=dev["dy"])
    assert torch.equal(out["y"], y.detach().cpu())
    for n, gv in zip(("x", "b", "c", "dt", "a_log", "d_skip"), gr):
        assert torch.equal(out["d" + n], gv.cpu()), n
    pipe.close()


# ---- decode step ------------------------------------------------------------------------------------

@pytest.mark.parametrize("rank,dtype", [(1, torch.float32), (2, torch.float32), (4, torch.bfloat16)])
def test_step_matches_the_chunked_scan(rank, dtype):
    """tests/ssm.rs:312-380: mamba3_step token by token equals the scan (rotation + D skip), and the
    state it ends in equals the scan's."""
    from mamba_trainer_b200.ssm import mamba3_step
    g = torch.Generator().manual_seed(rank)
    B, T, H, P, N = 2, 9, 2, (3 if dtype == torch.float32 else 64), (4 if dtype == torch.float32 else 128)
    r = lambda *s: torch.randn(*s, generator=g)
    u = lambda *s: torch.rand(*s, generator=g)
    t = {"x": r(B, T, H, P, rank), "b": r(B, T, H, N, rank) / N ** 0.5, "c": r(B, T, H, N, rank) / N ** 0.5,
         "dt": u(B, T, H) * 0.5 + 0.05, "lam": u(B, T, H), "a_log": u(H), "theta": u(B, T, H, N // 2) * 3,
         "d_skip": torch.tensor([0.3, -0.2])}
    for k in ("x", "b", "c", "dt", "lam", "theta"):
        t[k] = t[k].to(dtype)
    y_scan, st_scan, _ = fused_run(t, 4, True, False)
    dev = {k: v.cuda() for k, v in t.items()}
    state = SsmState.zeros(B, H, P, N, True, "cuda")
    ys = []
    for i in range(T):
        y, state = mamba3_step(dev["x"][:, i], dev["b"][:, i], dev["c"][:, i], dev["dt"][:, i], dev["lam"][:, i],
                               dev["a_log"], dev["theta"][:, i], dev["d_skip"], state)
        ys.append(y.unsqueeze(1))
    y_step = torch.cat(ys, 1)
    tol = 3e-4 if dtype == torch.float32 else 2e-2
    assert ref_metric(y_step.float(), y_scan.float()) <= tol
    assert ref_metric(state.h, st_scan.h) <= tol and ref_metric(state.last_u, st_scan.last_u) <= tol
    assert angle_close(state.angle, st_scan.angle, 1e-3)


# ---- depthwise causal convolution + SiLU, the step in front of the scan (src/nn/conv.rs) ------------------

def _conv_case(B, T, Cn, K, seed, dtype=torch.float32, history=True, bias=True):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)
    t = {"x": r(B, T, Cn).to(dtype), "w": r(K, Cn) * 0.5, "b": r(Cn) * 0.3 if bias else None,
         "h": r(B, K - 1, Cn).to(dtype) if history else None, "dy": r(B, T, Cn).to(dtype)}
    return t


def _conv_compare(t, activation, rtol, atol):
    from mamba_trainer_b200.nn import causal_conv1d
    from oracle.mixer import causal_conv1d as oracle_conv
    names = [n for n in ("x", "w", "b", "h") if t[n] is not None]
    dev = {n: t[n].cuda().requires_grad_(True) for n in names}
    y, hist = causal_conv1d(dev["x"], dev["w"], dev.get("b"), dev.get("h"), activation, want_history=True)
    gr = torch.autograd.grad(y, [dev[n] for n in names], grad_outputs=t["dy"].cuda())
    cpu = {n: t[n].double().requires_grad_(True) for n in names}
    ey, ehist = oracle_conv(cpu["x"], cpu["w"], cpu.get("b"), cpu.get("h"), activation)
    eg = torch.autograd.grad(ey, [cpu[n] for n in names], grad_outputs=t["dy"].double())
    assert allclose_excess(y.float(), ey.detach(), rtol, atol) <= 1.0, "y"
    assert torch.equal(hist.cpu().double(), ehist.detach()), "history"
    for n, a_, e_ in zip(names, gr, eg):
        assert allclose_excess(a_.float(), e_, rtol, atol * max(1.0, float(e_.abs().max()))) <= 1.0, "d" + n


@pytest.mark.parametrize("B,T,Cn,K,history,bias,activation", [
    (2, 37, 24, 4, True, True, True),      # vector path, ragged run
    (1, 300, 8, 4, False, True, True),     # several time blocks
    (2, 2, 12, 4, True, False, True),      # shorter than the history
    (3, 50, 10, 3, True, True, False),     # scalar path (channels not a multiple of the vector), bare convolution
    (2, 19, 16, 1, False, True, True),     # a single tap
    (1, 40, 8, 2, True, True, True),
    (2, 33, 16, 7, True, True, True),      # the wide-kernel instantiation
])
def test_conv_silu_matches_the_oracle_f32(B, T, Cn, K, history, bias, activation):
    _conv_compare(_conv_case(B, T, Cn, K, seed=T + K, history=history, bias=bias), activation, 1e-4, 1e-5)


def test_conv_silu_bf16_on_a_column_band():
    """bf16 activations, x a column band of a wider projection (row stride > channels)."""
    from mamba_trainer_b200.nn import causal_conv1d
    from oracle.mixer import causal_conv1d as oracle_conv
    g = torch.Generator().manual_seed(9)
    B, T, W, Cn, K = 2, 130, 96, 64, 4
    proj = torch.randn(B, T, W, generator=g).bfloat16()
    w, b = torch.randn(K, Cn, generator=g) * 0.5, torch.randn(Cn, generator=g) * 0.3
    dy = torch.randn(B, T, Cn, generator=g).bfloat16()
    pd = proj.cuda().requires_grad_(True)
    wd, bd = w.cuda().requires_grad_(True), b.cuda().requires_grad_(True)
    y = causal_conv1d(pd[..., 16:16 + Cn], wd, bd)
    gp, gw, gb = torch.autograd.grad(y, [pd, wd, bd], grad_outputs=dy.cuda())
    pc = proj.double().requires_grad_(True)
    wc, bc = w.double().requires_grad_(True), b.double().requires_grad_(True)
    ey, _ = oracle_conv(pc[..., 16:16 + Cn], wc, bc)
    ep, ew, eb = torch.autograd.grad(ey, [pc, wc, bc], grad_outputs=dy.double())
    check_bf16("y", y, ey.detach())
    check_bf16("dx", gp, ep)
    check_bf16("dw", gw, ew)
    check_bf16("db", gb, eb)


def test_conv_silu_replays_the_reference_ports_vectors():
    from pathlib import Path
    from mamba_trainer_b200.nn import causal_conv1d
    z = np.load(Path(__file__).resolve().parent / "golden" / "conv_silu.npz")
    f = lambda a: torch.tensor(np.asarray(a), dtype=torch.float32).cuda().requires_grad_(True)
    x, w, b = f(z["x"]), f(np.ascontiguousarray(z["w"][:, 0, :].T)), f(z["b"])
    y = causal_conv1d(x, w, b)
    dx, dw, db = torch.autograd.grad(y, [x, w, b], grad_outputs=f(z["dy"]).detach())
    check_f32("y", y, torch.tensor(z["y"]))
    check_f32("dx", dx, torch.tensor(z["dx"]))
    check_f32("dw", dw, torch.tensor(np.ascontiguousarray(z["dw"][:, 0, :].T)))
    check_f32("db", db, torch.tensor(z["db"]))


# ---- the mixer between its two projections (src/models/mamba3.rs:340-461, :475-484) --------------------------

def _core_params(core, p):
    with torch.no_grad():
        for name, val in p.items():
            par = getattr(core, name)
            if par is not None and val is not None:
                par.copy_(torch.as_tensor(val, dtype=torch.float32))


def test_mixer_core_replays_the_reference_ports_vectors():
    """tests/golden/mixer_core.npz: the reference port's whole mixer interior, values and the gradient
    of the projection and of every parameter, through the CUDA path in float32."""
    from pathlib import Path
    from mamba_trainer_b200.nn import MixerCore, MixerShape
    z = np.load(Path(__file__).resolve().parent / "golden" / "mixer_core.npz")
    B, T, H, P, N = (int(v) for v in z["dims"])
    core = MixerCore(MixerShape(H, P, N), conv_kernel=int(z["kernel"]), chunk=int(z["chunk"]), eps=float(z["eps"]),
                     device="cuda")
    p = {"conv_w": np.ascontiguousarray(z["conv_w"][:, 0, :].T), "conv_b": z["conv_b"], "dt_bias": z["dt_bias"],
         "a_log": z["a_log"], "d_skip": z["d_skip"], "b_bias": z["b_bias"], "c_bias": z["c_bias"], "norm_w": z["norm_w"]}
    _core_params(core, p)
    proj = torch.tensor(z["proj"], dtype=torch.float32, device="cuda", requires_grad=True)
    out = core(proj)
    check_f32("gated", out, torch.tensor(z["gated"]))
    names = list(p)
    grads = torch.autograd.grad(out, [proj] + [getattr(core, n) for n in names],
                                grad_outputs=torch.tensor(z["dgated"], dtype=torch.float32, device="cuda"))
    check_f32("dproj", grads[0], torch.tensor(z["dproj"]))
    for n, g in zip(names, grads[1:]):
        want = z["d_" + n]
        check_f32("d" + n, g, torch.tensor(np.ascontiguousarray(want[:, 0, :].T) if n == "conv_w" else want))


@pytest.mark.parametrize("rank,groups,rot,learned,norm_gain", [
    (1, None, True, True, True),        # the reference port's configuration at tensor-core sizes
    (2, 1, True, True, True),           # MIMO, two heads sharing one group
    (1, None, False, False, False),     # real dynamics, Euler, norm without gain
])
def test_mixer_core_bf16_matches_the_oracle(rank, groups, rot, learned, norm_gain):
    from mamba_trainer_b200.nn import MixerCore, MixerShape
    from oracle.mixer import mixer_core as oracle_core
    H, P, N, B, T = 2, 64, 128, 6, 400   # enough tokens per head for the per-head sums (a_log, dt_bias) to average
    shape = MixerShape(H, P, N, rank, groups, learned, rot)
    torch.manual_seed(rank * 7 + (groups or 0))
    core = MixerCore(shape, chunk=64, norm_gain=norm_gain, device="cuda")
    g = torch.Generator().manual_seed(5)
    r = lambda *s: torch.randn(*s, generator=g)
    p = {"conv_w": r(4, shape.conv_channels) * 0.4, "conv_b": r(shape.conv_channels) * 0.2, "dt_bias": r(H) * 0.3 - 3.0,
         "a_log": torch.rand(H, generator=g) * 2, "d_skip": r(H), "b_bias": r(H, N) * 0.3, "c_bias": r(H, N) * 0.3,
         "norm_w": (1.0 + r(N) * 0.2) if norm_gain else None}
    _core_params(core, p)
    proj = r(B, T, shape.in_proj_width).bfloat16()
    dgated = r(B, T, shape.d_inner).bfloat16()
    pd = proj.cuda().requires_grad_(True)
    out = core(pd)
    names = [n for n in p if p[n] is not None]
    grads = torch.autograd.grad(out, [pd] + [getattr(core, n) for n in names], grad_outputs=dgated.cuda())
    pc = proj.double().requires_grad_(True)
    pt = {n: v.double().requires_grad_(True) for n, v in p.items() if v is not None}
    eo, _, _ = oracle_core(pc, pt, H, P, N, rank, groups, 64, learned, rot)
    eg = torch.autograd.grad(eo, [pc] + [pt[n] for n in names], grad_outputs=dgated.double())
    check_bf16("gated", out, eo.detach())
    # the projection's gradient band by band: the bands differ in scale by orders of magnitude
    di, bc = shape.d_inner, shape.bc_width
    cuts = {"z": (0, di), "x": (di, 2 * di), "B": (2 * di, 2 * di + bc), "C": (2 * di + bc, 2 * di + 2 * bc),
            "dt": (2 * di + 2 * bc, 2 * di + 2 * bc + H)}
    for name, (lo, hi) in cuts.items():
        check_bf16("dproj." + name, grads[0][..., lo:hi], eg[0][..., lo:hi])
    # every parameter gradient meets the plain bf16 tolerance (a_log and dt_bias are sums over every token
    # with heavy cancellation: the case has 2400 tokens per head so that they average)
    for n, a_, e_ in zip(names, grads[1:], eg[1:]):
        check_bf16("d" + n, a_, e_)


@pytest.mark.parametrize("rank,dtype", [(1, torch.float32), (2, torch.float32), (1, torch.bfloat16)])
def test_mixer_core_decode_matches_the_parallel_pass(rank, dtype):
    """tests/model.rs:141-200 (decode == parallel, < 2e-3): one pass over the whole sequence against a
    prefill window followed by single-position steps, each continuing from the carried cache."""
    from mamba_trainer_b200.nn import MixerCore, MixerShape
    small = dtype == torch.float32
    H, P, N = (2, 4, 6) if small else (2, 64, 128)
    B, T, split = 2, 19, 12
    shape = MixerShape(H, P, N, rank)
    torch.manual_seed(rank)
    core = MixerCore(shape, chunk=8, device="cuda")
    with torch.no_grad():
        core.b_bias.normal_(0, 0.3); core.c_bias.normal_(0, 0.3); core.conv_b.normal_(0, 0.2); core.d_skip.normal_()
    proj = torch.randn(B, T, shape.in_proj_width, device="cuda").to(dtype)
    with torch.no_grad():
        whole = core(proj)
    out1, cache = core.forward_cached(proj[:, :split])
    outs = [out1]
    for t in range(split, T):
        o, cache = core.forward_cached(proj[:, t:t + 1], cache)
        outs.append(o)
    got = torch.cat(outs, 1)
    tol = 2e-3 if small else 3e-2
    assert ref_metric(got.float(), whole.float()) <= tol, ref_metric(got.float(), whole.float())
    # and two windows of several positions each
    o1, ca = core.forward_cached(proj[:, :7])
    o2, _ = core.forward_cached(proj[:, 7:], ca)
    assert ref_metric(torch.cat([o1, o2], 1).float(), whole.float()) <= tol


@pytest.mark.parametrize("dtype,rank", [(torch.float32, 1), (torch.float32, 2), (torch.bfloat16, 1)])
def test_mixer_core_bidirectional_matches_the_oracle(dtype, rank):
    """Mamba3Mixer::with_bidirectional (mamba3.rs:97-112): direction-major bands, the second half of the
    heads right to left; the oracle reverses those bands in time around the one-direction path, the
    kernels walk them backwards in place."""
    from mamba_trainer_b200.nn import MixerCore, MixerShape
    from oracle.mixer import mixer_core as oracle_core
    small = dtype == torch.float32
    H, P, N = (4, 4, 8) if small else (2, 64, 128)
    B, T = 2, (23 if small else 200)
    shape = MixerShape(H, P, N, rank)
    torch.manual_seed(3 + rank)
    core = MixerCore(shape, chunk=8 if small else 64, bidirectional=True, device="cuda")
    g = torch.Generator().manual_seed(11)
    r = lambda *s: torch.randn(*s, generator=g)
    p = {"conv_w": r(4, shape.conv_channels) * 0.4, "conv_b": r(shape.conv_channels) * 0.2, "dt_bias": r(H) * 0.3 - 2.0,
         "a_log": torch.rand(H, generator=g), "d_skip": r(H), "b_bias": r(H, N) * 0.3, "c_bias": r(H, N) * 0.3,
         "norm_w": 1.0 + r(N) * 0.2}
    _core_params(core, p)
    proj = r(B, T, shape.in_proj_width).to(dtype)
    dgated = r(B, T, shape.d_inner).to(dtype)
    pd = proj.cuda().requires_grad_(True)
    out = core(pd)
    names = list(p)
    grads = torch.autograd.grad(out, [pd] + [getattr(core, n) for n in names], grad_outputs=dgated.cuda())
    pc = proj.double().requires_grad_(True)
    pt = {n: v.double().requires_grad_(True) for n, v in p.items()}
    eo, _, _ = oracle_core(pc, pt, H, P, N, rank, None, 8 if small else 64, True, True, bidirectional=True)
    eg = torch.autograd.grad(eo, [pc] + [pt[n] for n in names], grad_outputs=dgated.double())
    check = check_f32 if small else check_bf16
    check("gated", out, eo.detach())
    di, bc = shape.d_inner, shape.bc_width
    for name, (lo, hi) in {"z": (0, di), "x": (di, 2 * di), "B": (2 * di, 2 * di + bc), "C": (2 * di + bc, 2 * di + 2 * bc),
                           "dt": (2 * di + 2 * bc, 2 * di + 2 * bc + H)}.items():
        check("dproj." + name, grads[0][..., lo:hi], eg[0][..., lo:hi])
    for n, a_, e_ in zip(names, grads[1:], eg[1:]):
        if small or n not in ("a_log", "dt_bias"):
            check("d" + n, a_, e_)


@pytest.mark.parametrize("dtype,rank,channels_odd", [(torch.float32, 1, False), (torch.float32, 2, True), (torch.bfloat16, 2, False)])
def test_mixer_core_post_gate_norm_matches_the_oracle(dtype, rank, channels_odd):
    """SsmConfig::post_gate_norm (src/ssm/config.rs:113; Mamba3Mixer::finish, src/models/mamba3.rs:475-484): the
    scan's flattened output is RMS-normalised over d_inner, with a gain, before the gate.  Values, the
    projection's gradient band by band and every parameter gradient, the gain's included."""
    from mamba_trainer_b200.nn import MixerCore, MixerShape
    from mamba_trainer_b200.error import ConfigError
    from oracle.mixer import mixer_core as oracle_core
    small = dtype == torch.float32
    H, P, N = ((3, 5, 6) if channels_odd else (2, 4, 6)) if small else (2, 64, 128)
    B, T = (2, 21) if small else (4, 300)
    shape = MixerShape(H, P, N, rank)
    torch.manual_seed(17 + rank)
    core = MixerCore(shape, chunk=8 if small else 64, post_gate_norm=True, device="cuda")
    g = torch.Generator().manual_seed(23)
    r = lambda *s: torch.randn(*s, generator=g)
    p = {"conv_w": r(4, shape.conv_channels) * 0.4, "conv_b": r(shape.conv_channels) * 0.2, "dt_bias": r(H) * 0.3 - 2.0,
         "a_log": torch.rand(H, generator=g), "d_skip": r(H), "b_bias": r(H, N) * 0.3, "c_bias": r(H, N) * 0.3,
         "norm_w": 1.0 + r(N) * 0.2, "post_norm_w": 1.0 + r(shape.d_inner) * 0.3}
    _core_params(core, p)
    proj = r(B, T, shape.in_proj_width).to(dtype)
    dgated = r(B, T, shape.d_inner).to(dtype)
    pd = proj.cuda().requires_grad_(True)
    out = core(pd)
    names = list(p)
    grads = torch.autograd.grad(out, [pd] + [getattr(core, n) for n in names], grad_outputs=dgated.cuda())
    pc = proj.double().requires_grad_(True)
    pt = {n: v.double().requires_grad_(True) for n, v in p.items()}
    eo, _, _ = oracle_core(pc, pt, H, P, N, rank, None, 8 if small else 64, True, True, post_gate_norm=True)
    eg = torch.autograd.grad(eo, [pc] + [pt[n] for n in names], grad_outputs=dgated.double())
    check = check_f32 if small else check_bf16
    check("gated", out, eo.detach())
    di, bc = shape.d_inner, shape.bc_width
    for name, (lo, hi) in {"z": (0, di), "x": (di, 2 * di), "B": (2 * di, 2 * di + bc), "C": (2 * di + bc, 2 * di + 2 * bc),
                           "dt": (2 * di + 2 * bc, 2 * di + 2 * bc + H)}.items():
        check("dproj." + name, grads[0][..., lo:hi], eg[0][..., lo:hi])
    for n, a_, e_ in zip(names, grads[1:], eg[1:]):
        if small or n not in ("a_log", "dt_bias"):
            check("d" + n, a_, e_)
    # decode == parallel with the norm in place, and the reference's refusal for a bidirectional mixer
    with torch.no_grad():
        whole = core(proj.cuda())
        o1, cache = core.forward_cached(proj[:, :T - 1].cuda())
        o2, _ = core.forward_cached(proj[:, T - 1:].cuda(), cache)
    assert ref_metric(torch.cat([o1, o2], 1).float(), whole.float()) <= (2e-3 if small else 3e-2)
    with pytest.raises(ConfigError):
        MixerCore(MixerShape(2, 4, 6), bidirectional=True, post_gate_norm=True, device="cuda")


@pytest.mark.parametrize("Cn,W,off", [(1000, 1300, 100), (4096, 4300, 104), (1001, 1300, 99)])
def test_gate_norm_c_abi_edges(Cn, W, off):
    """m3_gate_norm_*: z as a band of a wider row, a norm without gain, outputs that are not wanted, and
    the channel limit; a warp per row, a block per row, and the element-wise kernels for rows that are not
    whole 16-byte vectors."""
    import ctypes as C
    from mamba_trainer_b200 import _ffi
    from mamba_trainer_b200.ssm.scan import Context
    from mamba_trainer_b200.error import UnsupportedError
    ctx = Context.for_device(torch.device("cuda"))
    lib, hd = ctx.lib, ctx.handle
    torch.manual_seed(2)
    B, T = 3, 37
    y = torch.randn(B, T, Cn, device="cuda")
    wide = torch.randn(B, T, W, device="cuda")
    dout = torch.randn(B, T, Cn, device="cuda")
    ptr = lambda t, off=0: C.c_void_p(t.data_ptr() + off * t.element_size()) if t is not None else None
    for gain in (None, 1.0 + 0.3 * torch.randn(Cn, device="cuda")):
        d = _ffi.GateNormDesc(batch=B, seq=T, channels=Cn, dtype=0, z_stride=W, y=ptr(y), z=ptr(wide, off), weight=ptr(gain), eps=1e-5)
        out, dy, dwide = torch.empty_like(y), torch.empty_like(y), torch.zeros_like(wide)
        dw = torch.full((Cn,), 7.0, device="cuda")
        ctx.check(lib.m3_gate_norm_forward(hd, C.byref(d), ptr(out)))
        ctx.check(lib.m3_gate_norm_backward(hd, C.byref(d), ptr(dout), ptr(dy), ptr(dwide, off), ptr(dw)))
        yd = y.double().requires_grad_(True)
        zd = wide[..., off:off + Cn].double().requires_grad_(True)
        gd = gain.double().requires_grad_(True) if gain is not None else None
        n = yd * torch.rsqrt(yd.pow(2).mean(-1, keepdim=True) + 1e-5)
        e = (n * gd if gd is not None else n) * torch.nn.functional.silu(zd)
        eg = torch.autograd.grad(e, [yd, zd] + ([gd] if gd is not None else []), grad_outputs=dout.double())
        check_f32("out", out, e.detach())
        check_f32("dy", dy, eg[0])
        check_f32("dz", dwide[..., off:off + Cn], eg[1])
        assert float(dwide[..., :off].abs().max()) == 0.0 and float(dwide[..., off + Cn:].abs().max()) == 0.0
        if gain is not None:
            check_f32("dweight", dw, eg[2])
            ctx.check(lib.m3_gate_norm_backward(hd, C.byref(d), ptr(dout), None, None, ptr(dw)))   # d gain alone
            check_f32("dweight alone", dw, eg[2])
        else:
            assert float((dw - 7.0).abs().max()) == 0.0      # no gain, nothing written
    big = _ffi.GateNormDesc(batch=1, seq=1, channels=8193, dtype=0, z_stride=0, y=ptr(y), z=ptr(y), weight=None, eps=1e-5)
    with pytest.raises(UnsupportedError):
        ctx.check(lib.m3_gate_norm_forward(hd, C.byref(big), ptr(y)))


def test_mixer_core_degenerate_lengths():
    """A single position and an empty window through the training path."""
    from mamba_trainer_b200.nn import MixerCore, MixerShape
    from oracle.mixer import mixer_core as oracle_core
    H, P, N = 2, 4, 6
    shape = MixerShape(H, P, N)
    torch.manual_seed(0)
    core = MixerCore(shape, chunk=4, device="cuda")
    p = {n: getattr(core, n).detach().cpu().double() for n in ("conv_w", "conv_b", "dt_bias", "a_log", "d_skip", "b_bias",
                                                              "c_bias", "norm_w")}
    proj = torch.randn(3, 1, shape.in_proj_width)
    pd = proj.cuda().requires_grad_(True)
    out = core(pd)
    (gp,) = torch.autograd.grad(out.sum(), [pd])
    pc = proj.double().requires_grad_(True)
    eo, _, _ = oracle_core(pc, p, H, P, N, chunk=4)
    (ep,) = torch.autograd.grad(eo.sum(), [pc])
    check_f32("gated", out, eo.detach())
    check_f32("dproj", gp, ep)
    empty = core(torch.zeros(3, 0, shape.in_proj_width, device="cuda", requires_grad=True))
    assert tuple(empty.shape) == (3, 0, shape.d_inner)


def test_zz_report_flat_float32_tolerance():
    """Not a check of its own: prints how many of the float32 tensor comparisons made by this file's tests
    also hold at the flat tolerance 1e-5 + 1e-4 |e| (run the whole file for the full count)."""
    n, ok = F32_FLAT["tensors"], F32_FLAT["pass_flat"]
    print(f"\nfloat32 comparisons: {ok} of {n} tensors within the flat 1e-5 + 1e-4|e|; "
          f"worst excess {F32_FLAT['worst_flat_excess']:.2f}x on {F32_FLAT['worst']}")
    assert ok <= n
