"""Scan forward + backward for callers whose tensors live in HOST memory.

The reference's tensors are device handles; a host-side caller (data loader output, a plugin
boundary that hands over host buffers) pays the PCIe copies around the op.  Because every batch
row is an independent recurrence, the call is cut into batch slices and run as a three-stage
pipeline - host-to-device copy, forward + backward, device-to-host copy - on three CUDA streams,
so the copies of one slice hide behind the kernels and the opposite-direction copies of its
neighbours.  The pipeline itself is native (m3_host_pipe_* in libm3scan): one library call enqueues
a whole run, so the host thread is not the bottleneck.  Results are identical to one call on the
whole batch (per-head parameter gradients are summed over the slices in a fixed order).
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, Optional

import torch

from . import _ffi
from .ssm.config import Discretization
from .ssm.scan import Context, _DTYPES

_PER_TOKEN = ("x", "b", "c", "dt", "lam", "theta", "dy")
_PER_HEAD = ("a_log", "d_skip")


def bind_host_thread_near(device) -> Optional[dict]:
    """Pin the calling process to the CPUs next to `device` (its PCIe root's NUMA node, as sysfs reports
    it), so that the page-locked buffers it allocates afterwards - a pinned page lives on the node of the
    thread that first touches it - sit on the memory controller the GPU's copies reach without crossing the
    socket interconnect.  With one process per GPU and none of them bound, every rank's staging buffers can
    land on one node and all host-to-device traffic of the box then shares that node's bandwidth.
    Returns {"node", "cpus"} or None where the platform gives no answer (no sysfs entry, node -1, or an
    empty intersection with the CPUs this process may use); nothing is changed in that case."""
    import os
    try:
        props = torch.cuda.get_device_properties(torch.device(device))
        addr = "%04x:%02x:%02x.0" % (props.pci_domain_id, props.pci_bus_id, props.pci_device_id)
        base = "/sys/bus/pci/devices/" + addr
        node = int(open(base + "/numa_node").read().strip())
        cpulist = open(base + "/local_cpulist").read().strip()
    except (OSError, ValueError, AttributeError):
        return None
    if node < 0 or not cpulist:
        return None
    cpus = set()
    for part in cpulist.split(","):
        lo, _, hi = part.partition("-")
        cpus.update(range(int(lo), int(hi or lo) + 1))
    cpus &= os.sched_getaffinity(0)
    if not cpus:
        return None
    os.sched_setaffinity(0, cpus)
    return {"node": node, "cpus": len(cpus)}


def _hp(t: Optional[torch.Tensor]):
    return C.c_void_p(t.data_ptr()) if t is not None else None


class HostScanPipeline:
    """Reusable pipeline for one problem shape.  `host` tensors must be pinned for the copies to
    be asynchronous; outputs are written into pinned tensors owned by the pipeline (`depth` sets,
    used in turn, so the results of one run stay valid while the next depth-1 runs are in flight)."""

    def __init__(self, host: Dict[str, Optional[torch.Tensor]], chunk: int, discretization: Discretization,
                 device, slices: int = 4, params: Optional[Dict[str, torch.Tensor]] = None,
                 path: int = _ffi.PATH_AUTO, depth: int = 2):
        self.dev = torch.device(device)
        self.chunk, self.disc = chunk, Discretization(discretization)
        self.names = [n for n in _PER_TOKEN if host.get(n) is not None]
        if not self.disc.needs_lambda_projection() and "lam" in self.names:
            self.names.remove("lam")
        x = host["x"]
        self.shape = tuple(x.shape)
        B, T, H, P, R = x.shape
        N = host["b"].shape[3]
        self.rot = "theta" in self.names
        self.slices = max(1, min(slices, B))
        self.grad_names = [n for n in self.names if n != "dy"]
        self.depth = max(1, int(depth))
        self._outs = []
        for _ in range(self.depth):
            out = {"y": torch.empty(x.shape, dtype=x.dtype).pin_memory()}
            for n in self.grad_names:
                out["d" + n] = torch.empty(host[n].shape, dtype=host[n].dtype).pin_memory()
            for n in _PER_HEAD:   # per-head parameter gradients, float32 [heads]
                out["d" + n] = torch.zeros((H,), dtype=torch.float32).pin_memory()
            self._outs.append(out)
        self.h2d_bytes = sum(host[n].numel() * host[n].element_size() for n in self.names)
        self.d2h_bytes = sum(v.numel() * v.element_size() for v in self._outs[0].values())
        self._desc_args = dict(
            batch=B, seq=T, heads=H, head_dim=P, d_state=N, rank=R, chunk=int(chunk), dtype=_DTYPES[x.dtype],
            discretization=int(self.disc.value), dynamics=1 if self.rot else 0, want_state=0, path=int(path))
        self._ctx = Context.for_device(self.dev)
        self._pipe = None
        self._params = None
        self._runs = 0
        self._tickets = {}
        if params is not None:
            self._create(params)

    def _create(self, params: Dict[str, torch.Tensor]) -> None:
        a_log, d_skip = params["a_log"].detach(), params.get("d_skip")
        d_skip = d_skip.detach() if d_skip is not None else None
        if a_log.dtype != torch.float32 or (d_skip is not None and d_skip.dtype != torch.float32):
            raise TypeError("a_log and d_skip are float32 device tensors")
        self._params = (a_log, d_skip)   # kept alive: the native pipeline holds their addresses
        desc = _ffi.ScanDesc(a_log=_hp(a_log), d_skip=_hp(d_skip), **self._desc_args)
        handle = C.c_void_p()
        self._ctx.check(self._ctx.lib.m3_host_pipe_create(self._ctx.handle, C.byref(desc), self.slices, C.byref(handle)))
        self._pipe = handle

    def run(self, host: Dict[str, Optional[torch.Tensor]], params: Dict[str, torch.Tensor],
            wait: bool = False) -> Dict[str, torch.Tensor]:
        """Enqueue one run.  host: pinned per-token tensors; params: a_log / d_skip on the device.
        Returns the pinned output tensors of this run; they are complete after `wait(outputs)`
        (or at once with wait=True)."""
        if self._pipe is None:
            self._create(params)
        elif params["a_log"].data_ptr() != self._params[0].data_ptr() or (
                self._params[1] is not None and params["d_skip"].data_ptr() != self._params[1].data_ptr()):
            raise ValueError("the pipeline was created for other parameter tensors")
        self._ctx.bind_current_stream()
        out = self._outs[self._runs % self.depth]
        hin = _ffi.HostIn(x=_hp(host["x"]), b=_hp(host["b"]), c=_hp(host["c"]), dt=_hp(host["dt"]),
                          lambda_=_hp(host.get("lam")) if "lam" in self.names else None,
                          theta=_hp(host.get("theta")) if self.rot else None, dy=_hp(host["dy"]))
        hout = _ffi.HostOut(y=_hp(out["y"]), dx=_hp(out["dx"]), db=_hp(out["db"]), dc=_hp(out["dc"]),
                            ddt=_hp(out["ddt"]), dlambda=_hp(out.get("dlam")), dtheta=_hp(out.get("dtheta")),
                            da_log=_hp(out["da_log"]), dd_skip=_hp(out["dd_skip"]) if self._params[1] is not None else None)
        ticket = C.c_uint64()
        self._ctx.check(self._ctx.lib.m3_host_pipe_run(self._pipe, C.byref(hin), C.byref(hout), C.byref(ticket)))
        self._tickets[id(out)] = ticket.value
        self._runs += 1
        if wait:
            self.wait(out)
        return out

    def wait(self, out: Optional[Dict[str, torch.Tensor]] = None) -> None:
        """Block until the run that produced `out` (default: the latest run) is in host memory."""
        if self._pipe is None or not self._tickets:
            return
        ticket = self._tickets[id(out)] if out is not None else max(self._tickets.values())
        self._ctx.check(self._ctx.lib.m3_host_pipe_wait(self._pipe, ticket))

    def close(self) -> None:
        if self._pipe is not None:
            self._ctx.lib.m3_host_pipe_destroy(self._pipe)
            self._pipe = None

    def __del__(self):
        try:
            self.close()
        except Exception:  # interpreter shutdown
            pass
