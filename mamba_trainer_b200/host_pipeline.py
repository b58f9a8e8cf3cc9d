"""Scan forward + backward for callers whose tensors live in HOST memory.

The reference's tensors are device handles; a host-side caller (data loader output, a plugin
boundary that hands over host buffers) pays the PCIe copies around the op.  Because every batch
row is an independent recurrence, the call is cut into batch slices and run as a three-stage
pipeline - host-to-device copy, forward + backward, device-to-host copy - on three CUDA streams,
so the copies of one slice hide behind the kernels and the opposite-direction copies of its
neighbours.  Results are identical to one call on the whole batch (per-head parameter gradients
are summed over the slices in a fixed order).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .ssm.config import Discretization
from .ssm.scan import ScanInputs, mamba3_scan

_PER_TOKEN = ("x", "b", "c", "dt", "lam", "theta", "dy")
_PER_HEAD = ("a_log", "d_skip")


class HostScanPipeline:
    """Reusable pipeline for one problem shape.  `host` tensors must be pinned for the copies to
    be asynchronous; outputs are written into pinned tensors owned by the pipeline."""

    def __init__(self, host: Dict[str, Optional[torch.Tensor]], chunk: int, discretization: Discretization,
                 device, slices: int = 4):
        self.dev = torch.device(device)
        self.chunk, self.disc = chunk, Discretization(discretization)
        self.names = [n for n in _PER_TOKEN if host.get(n) is not None]
        if not self.disc.needs_lambda_projection() and "lam" in self.names:
            self.names.remove("lam")
        B = host["x"].shape[0]
        self.slices = max(1, min(slices, B))
        bounds = [round(i * B / self.slices) for i in range(self.slices + 1)]
        self.ranges = [(bounds[i], bounds[i + 1]) for i in range(self.slices)]
        width = max(hi - lo for lo, hi in self.ranges)
        self.stage = [{n: torch.empty((width,) + tuple(host[n].shape[1:]), dtype=host[n].dtype, device=self.dev)
                       for n in self.names} for _ in range(2)]
        self.grad_names = [n for n in self.names if n != "dy"]
        self.out = {"y": torch.empty(host["x"].shape, dtype=host["x"].dtype).pin_memory()}
        for n in self.grad_names:
            self.out["d" + n] = torch.empty(host[n].shape, dtype=host[n].dtype).pin_memory()
        H = host["x"].shape[2]
        for n in _PER_HEAD:   # per-head parameter gradients, float32 [heads]
            self.out["d" + n] = torch.empty((H,), dtype=torch.float32).pin_memory()
        self.s_in, self.s_out = torch.cuda.Stream(self.dev), torch.cuda.Stream(self.dev)
        self.h2d_bytes = sum(host[n].numel() * host[n].element_size() for n in self.names)
        self.d2h_bytes = sum(v.numel() * v.element_size() for v in self.out.values())

    def run(self, host: Dict[str, Optional[torch.Tensor]], params: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        """host: pinned per-token tensors; params: a_log / d_skip on the device (requires_grad)."""
        main = torch.cuda.current_stream(self.dev)
        done: List[torch.cuda.Event] = []
        keep = []
        psum = {n: None for n in _PER_HEAD if params.get(n) is not None}
        for i, (lo, hi) in enumerate(self.ranges):
            buf = self.stage[i % 2]
            with torch.cuda.stream(self.s_in):
                if i >= 2:
                    self.s_in.wait_event(done[i - 2])          # the staging buffer is free again
                elif i == 0:
                    self.s_in.wait_stream(main)
                for n in self.names:
                    buf[n][: hi - lo].copy_(host[n][lo:hi], non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(self.s_in)
            main.wait_event(ready)
            src = {n: buf[n][: hi - lo].detach().requires_grad_(n != "dy") for n in self.names}
            inp = ScanInputs.new(src["x"], src["b"], src["c"], src["dt"], params["a_log"], src.get("lam"))
            inp = inp.with_chunk_size(self.chunk).with_state_output(False).with_discretization(self.disc)
            if src.get("theta") is not None:
                inp = inp.with_theta(src["theta"])
            if params.get("d_skip") is not None:
                inp = inp.with_skip(params["d_skip"])
            y = mamba3_scan(inp).y
            wrt = [src[n] for n in self.grad_names] + [params[n] for n in psum]
            grads = torch.autograd.grad(y, wrt, grad_outputs=src["dy"])
            for n, gv in zip(psum, grads[len(self.grad_names):]):
                psum[n] = gv if psum[n] is None else psum[n] + gv
            ev = torch.cuda.Event()
            ev.record(main)
            done.append(ev)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(ev)
                self.out["y"][lo:hi].copy_(y, non_blocking=True)
                for n, gv in zip(self.grad_names, grads):
                    self.out["d" + n][lo:hi].copy_(gv, non_blocking=True)
            keep.append((y, grads))
        for n, gv in psum.items():
            self.out["d" + n].copy_(gv.float(), non_blocking=True)   # on the main stream, after the last slice
        main.wait_stream(self.s_out)
        self._keep = keep                                      # device results stay alive until the copies ran
        return self.out
