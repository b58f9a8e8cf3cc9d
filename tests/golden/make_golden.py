"""Generate the golden vectors under tests/golden/ from the REFERENCE's own code.

Run in a container that has the reference checked out (it is not needed to run the
tests):

    python tests/golden/make_golden.py /root/reference

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


def main():
    root = Path(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
    ref = load_reference(root)
    assert ref.LOG_DECAY_FLOOR == -60.0
    ssd_case(ref, "ssd_chunked_even", (2, 12, 3, 4, 6), 4)
    ssd_case(ref, "ssd_chunked_ragged", (1, 13, 2, 3, 4), 4)
    ssd_case(ref, "ssd_chunked_one_chunk", (1, 7, 2, 3, 4), 16)
    rotate_case(ref)
    mixer_tail_case(ref)
    print("wrote", sorted(p.name for p in HERE.glob("*.npz")))


if __name__ == "__main__":
    main()
