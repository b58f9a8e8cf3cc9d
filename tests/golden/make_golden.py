"""Generate the golden vectors under tests/golden/ from the REFERENCE's own code.

Run in a container that has the reference checked out (it is not needed to run the
tests):

    python tests/golden/make_golden.py <path to the mamba-trainer checkout>

It imports the reference's PyTorch port of the scan path (bench/torch_mamba3.py:
`ssd_chunked` :47-129, `rotate_halves` :132-137, `LOG_DECAY_FLOOR` :25) by file
path, feeds it the deterministic LCG inputs of the reference's test-suite
(tests/ssm.rs:26-34, :122-142) and stores inputs, outputs and autograd gradients
as float64 .npz files.  Nothing from the reference is copied: only its outputs.
"""
from __future__ import annotations

import importlib.util
import math
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
from oracle.recurrence import Case, lcg_noise  # noqa: E402  (LCG inputs only)


def load_reference(root: Path):
    spec = importlib.util.spec_from_file_location("ref_torch_mamba3", root / "bench" / "torch_mamba3.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def t64(a, grad=True):
    return torch.tensor(np.asarray(a, dtype=np.float64), requires_grad=grad)


def weights(case):
    dt, lam = t64(case.dt), t64(case.lam)
    a = dt * t64(case.a_head, False).view(1, 1, -1)
    g = lam * dt
    nxt = (1.0 - lam) * dt
    w = g + torch.cat([nxt[:, 1:], torch.zeros_like(nxt[:, :1])], dim=1)
    return a.detach().requires_grad_(), g.detach().requires_grad_(), w.detach().requires_grad_()


def ssd_case(ref, name, dims, chunk):
    case = Case(*dims)
    x, b, c = t64(case.x), t64(case.b), t64(case.c)
    a, g, w = weights(case)
    y = ref.ssd_chunked(x, b, c, a, g, w, chunk)
    dy = t64(lcg_noise(y.numel(), 13).reshape(y.shape), False)
    grads = torch.autograd.grad((y * dy).sum(), [x, b, c, a, g, w])
    np.savez(HERE / f"{name}.npz", dims=np.array(dims), chunk=chunk,
             x=x.detach().numpy(), b=b.detach().numpy(), c=c.detach().numpy(),
             a=a.detach().numpy(), g=g.detach().numpy(), w=w.detach().numpy(),
             y=y.detach().numpy(), dy=dy.numpy(),
             **{f"d{n}": v.numpy() for n, v in zip("xbcagw", grads)})


def rotate_case(ref):
    v = t64(lcg_noise(2 * 5 * 3 * 8, 21).reshape(2, 5, 3, 8))
    phi = t64(4.0 * lcg_noise(2 * 5 * 3 * 4, 22).reshape(2, 5, 3, 4))
    out = ref.rotate_halves(v, phi)
    go = t64(lcg_noise(out.numel(), 23).reshape(out.shape), False)
    dv, dphi = torch.autograd.grad((out * go).sum(), [v, phi])
    np.savez(HERE / "rotate_halves.npz", v=v.detach().numpy(), phi=phi.detach().numpy(),
             out=out.detach().numpy(), go=go.numpy(), dv=dv.numpy(), dphi=dphi.numpy())


def mixer_tail_case(ref):
    """The scan as the reference's mixer port drives it (bench/torch_mamba3.py:190-207):
    weights, wrapped cumulative angle, two rotations, ssd_chunked, D skip - SISO."""
    dims = (2, 11, 2, 3, 4)
    case = Case(*dims)
    x, b, c = t64(case.x), t64(case.b), t64(case.c)
    dt, lam = t64(case.dt), t64(case.lam)
    a_log = t64(case.a_log)
    theta = t64(case.theta())
    d_skip = t64(np.array([0.3, -0.2]))
    a = dt * (-torch.exp(a_log))
    g = lam * dt
    nxt = (1.0 - lam) * dt
    w = g + torch.cat([nxt[:, 1:], torch.zeros_like(nxt[:, :1])], dim=1)
    phi = (dt.unsqueeze(3) * theta).cumsum(1)
    phi = phi - (torch.round(phi / (2 * math.pi)) * 2 * math.pi).detach()
    y = ref.ssd_chunked(x, ref.rotate_halves(b, phi), ref.rotate_halves(c, phi), a, g, w, 4)
    y = y + x * d_skip.view(1, 1, -1, 1)
    dy = t64(lcg_noise(y.numel(), 13).reshape(y.shape), False)
    leaves = [x, b, c, dt, lam, a_log, theta, d_skip]
    grads = torch.autograd.grad((y * dy).sum(), leaves)
    names = ["x", "b", "c", "dt", "lam", "a_log", "theta", "d_skip"]
    np.savez(HERE / "mixer_tail.npz", dims=np.array(dims), chunk=4, y=y.detach().numpy(), dy=dy.numpy(),
             **{n: v.detach().numpy() for n, v in zip(names, leaves)},
             **{f"d_{n}": v.numpy() for n, v in zip(names, grads)})


def mixer_core_case(ref):
    """Everything the reference's mixer port does between its two projections
    (bench/torch_mamba3.py:165-207), run through the port's own Mamba3Mixer.forward in float64:
    split, depthwise causal convolution (:175), SiLU, B/C bias + RMS norm, softplus / sigmoid,
    angles and rotations, ssd_chunked, D skip, the SiLU(z) gate.  The projection's output and the
    output projection's input are captured with hooks; parameters get non-trivial values."""
    torch.manual_seed(0)
    d_model, H, P, N, chunk, K = 16, 2, 4, 6, 4, 4
    B, T = 2, 11
    m = ref.Mamba3Mixer(d_model, H, P, N, chunk, conv_kernel=K).double()
    noise = lambda shape, seed, s=1.0: torch.tensor(s * lcg_noise(int(np.prod(shape)), seed).reshape(shape), dtype=torch.float64)
    with torch.no_grad():
        m.conv.weight.copy_(noise(m.conv.weight.shape, 31, 0.6))
        m.conv.bias.copy_(noise(m.conv.bias.shape, 32, 0.3))
        m.dt_bias.copy_(noise((H,), 33) - 1.5)
        m.a_log.copy_(noise((H,), 34, 0.5) + 0.5)
        m.d_skip.copy_(noise((H,), 35))
        m.b_bias.copy_(noise((H, N), 36, 0.4))
        m.c_bias.copy_(noise((H, N), 37, 0.4))
        m.bc_norm.weight.copy_(1.0 + noise((N,), 38, 0.3))
    cap = {}
    def grab_proj(_mod, _inp, out):
        out.retain_grad()
        cap["proj"] = out
    def grab_gated(_mod, inp):
        inp[0].retain_grad()
        cap["gated"] = inp[0]
    h1 = m.in_proj.register_forward_hook(grab_proj)
    h2 = m.out_proj.register_forward_pre_hook(grab_gated)
    u = noise((B, T, d_model), 39, 2.0)
    m(u)
    h1.remove(); h2.remove()
    gated, proj = cap["gated"], cap["proj"]
    dgated = noise(tuple(gated.shape), 40)
    params = {"conv_w": m.conv.weight, "conv_b": m.conv.bias, "dt_bias": m.dt_bias, "a_log": m.a_log,
              "d_skip": m.d_skip, "b_bias": m.b_bias, "c_bias": m.c_bias, "norm_w": m.bc_norm.weight}
    grads = torch.autograd.grad((gated * dgated).sum(), [proj] + list(params.values()))
    np.savez(HERE / "mixer_core.npz", dims=np.array([B, T, H, P, N]), chunk=chunk, kernel=K, eps=m.bc_norm.eps,
             proj=proj.detach().numpy(), gated=gated.detach().numpy(), dgated=dgated.numpy(),
             dproj=grads[0].numpy(),
             **{n: v.detach().numpy() for n, v in params.items()},
             **{f"d_{n}": g.numpy() for n, g in zip(params, grads[1:])})
    # the convolution + SiLU step alone, as the port's forward applies it (:175-176)
    d_inner, bc = H * P, H * N
    xbc = proj.detach()[..., d_inner:2 * d_inner + 2 * bc].clone().requires_grad_(True)
    y = torch.nn.functional.silu(m.conv(xbc.transpose(1, 2))[..., :T].transpose(1, 2))
    dy = noise(tuple(y.shape), 41)
    gx, gw, gb = torch.autograd.grad((y * dy).sum(), [xbc, m.conv.weight, m.conv.bias])
    np.savez(HERE / "conv_silu.npz", x=xbc.detach().numpy(), w=m.conv.weight.detach().numpy(),
             b=m.conv.bias.detach().numpy(), y=y.detach().numpy(), dy=dy.numpy(), dx=gx.numpy(), dw=gw.numpy(),
             db=gb.numpy())


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <path to the mamba-trainer checkout>")
    root = Path(sys.argv[1])
    ref = load_reference(root)
    assert ref.LOG_DECAY_FLOOR == -60.0
    ssd_case(ref, "ssd_chunked_even", (2, 12, 3, 4, 6), 4)
    ssd_case(ref, "ssd_chunked_ragged", (1, 13, 2, 3, 4), 4)
    ssd_case(ref, "ssd_chunked_one_chunk", (1, 7, 2, 3, 4), 16)
    rotate_case(ref)
    mixer_tail_case(ref)
    mixer_core_case(ref)
    print("wrote", sorted(p.name for p in HERE.glob("*.npz")))


if __name__ == "__main__":
    main()
