"""Benchmark of the fused Mamba-3 SSD scan: forward + backward Mtokens/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config I] [--impl ours|reference]

A step is one forward and one backward pass of the scan over one batch of synthetic
inputs (mamba_trainer_b200.synthetic).  Every rank runs the same per-GPU workload on
its own shard (weak scaling, no collective in the path).  Rank 0 prints one JSON line.
`--impl reference` times the CPU oracle (the restated reference composition) on the
host cores instead.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

from mamba_trainer_b200 import synthetic  # noqa: E402

# dram__bytes_read.sum + dram__bytes_write.sum of one tc_bwd_kernel launch, from the committed ncu
# capture of this workload (bytes per launch; None where no capture was taken).
NCU_TRAFFIC_BYTES = {"cfg1_siso_trapezoid_bf16": 267403520}

METRIC = "mamba3_ssd_scan_fwd_bwd_throughput"
UNIT = "Mtokens/s"


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """SM clock and throttle reasons sampled DURING the timed region: an NVML polling thread
    (2 ms period, so even a few-millisecond region gets samples), nvidia-smi as a fallback."""
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int):
        import threading
        self.sm, self.mask, self.max = [], 0, None
        self._stop = threading.Event()
        self._thread = None
        self._smi = None
        try:
            import pynvml
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(index).uuid)
            try:
                h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
            except Exception:
                h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
            get_reasons = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                pynvml.nvmlDeviceGetCurrentClocksThrottleReasons

            def poll():
                while not self._stop.is_set():
                    try:
                        self.sm.append(float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)))
                        self.mask |= int(get_reasons(h))
                    except Exception:
                        pass
                    time.sleep(0.002)

            self._thread = threading.Thread(target=poll, daemon=True)
            self._thread.start()
        except Exception:
            q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
                 "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
            try:
                self._smi = subprocess.Popen(
                    ["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-lms", "20", "-i", str(index)],
                    stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            except OSError:
                self._smi = None

    def stop(self) -> dict:
        reasons = []
        if self._thread is not None:
            self._stop.set()
            self._thread.join(timeout=1.0)
            reasons = sorted(n for bit, n in self.REASONS.items() if self.mask & bit)
        elif self._smi is not None:
            time.sleep(0.05)
            self._smi.terminate()
            try:
                out, _ = self._smi.communicate(timeout=5)
            except subprocess.TimeoutExpired:
                self._smi.kill()
                out, _ = self._smi.communicate()
            names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
            found = set()
            for line in out.splitlines():
                f = [v.strip() for v in line.split(",")]
                if len(f) < 6:
                    continue
                try:
                    self.sm.append(float(f[0]))
                    self.max = float(f[1])
                except ValueError:
                    continue
                found |= {n for n, v in zip(names, f[2:6]) if v.lower().startswith("active")}
            reasons = sorted(found)
        return {"sm_mhz": statistics.median(self.sm) if self.sm else None, "sm_max_mhz": self.max,
                "reasons": reasons, "samples": len(self.sm)}


def cpu_oracle_throughput(w, steps: int = 8, warmup: int = 1, budget_s: float = 20.0):
    """Time the CPU oracle (fp32, forward + backward) on a bounded slice of the workload: one batch row
    and two heads per step (the scan is independent across batch and heads, so throughput in
    token-heads/s carries over).  `warmup` untimed steps (at most 3), then up to `steps` timed ones, cut
    short when `budget_s` seconds are spent; the value is the mean over the timed steps."""
    from oracle import m3_oracle as O
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    heads = min(w.heads, 2)
    seq = min(w.seq, 2048)
    sw = w.scaled(batch=1, heads=heads, seq=seq)
    t = synthetic.make_inputs(sw, seed=0)
    names = [n for n in ("x", "b", "c", "dt", "a_log", "lam", "theta", "d_skip") if t.get(n) is not None]

    def one():
        leaf = {n: t[n].float().requires_grad_(True) for n in names}
        t0 = time.perf_counter()
        y, _ = O.mamba3_scan(leaf["x"], leaf["b"], leaf["c"], leaf["dt"], leaf["a_log"], leaf["lam"],
                             leaf.get("theta"), leaf.get("d_skip"), None, sw.chunk, False)
        torch.autograd.grad((y * t["dy"].float()).sum(), [leaf[n] for n in names])
        return time.perf_counter() - t0

    warm = max(1, min(warmup, 3))
    for _ in range(warm):
        one()
    times, t_start = [], time.perf_counter()
    while len(times) < max(1, steps) and (not times or time.perf_counter() - t_start < budget_s):
        times.append(one())
    mean = sum(times) / len(times)
    tok_heads_per_s = sw.tokens * sw.heads / mean
    value = tok_heads_per_s / w.heads / 1e6   # Mtokens/s of the full-head workload
    sample = (f"batch 1 x seq {seq} x {heads} of {w.heads} heads per step, fp32, mean of {len(times)} steps after "
              f"{warm} warm-up, scaled by heads")
    return value, cores, sample


def run_reference(args, w, rank):
    if rank != 0:
        return
    value, cores, sample = cpu_oracle_throughput(w, steps=args.steps, warmup=args.warmup, budget_s=120.0)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": w.tokens / (value * 1e6) * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": w.name, "batch_per_gpu": w.batch, "seq_len": w.seq, "heads": w.heads,
                   "head_dim": w.head_dim, "d_state": w.d_state, "rank": w.rank, "chunk": w.chunk,
                   "call": "CPU oracle (fp32 restatement of the reference's scan) on a bounded sample per step"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def mixer_core_leg(w, dev):
    """Secondary figure, not the headline: the whole stretch of the mixer between its two projections
    (convolution + SiLU, B/C bias + RMS norm + layout, dt / lambda activations, the scan, the gate)
    forward + backward as one tape node, on the workload's shapes with groups = heads."""
    from mamba_trainer_b200.nn import MixerCore, MixerShape
    shape = MixerShape(w.heads, w.head_dim, w.d_state, w.rank, None, True, w.rotational)
    core = MixerCore(shape, chunk=w.chunk, device=dev)
    g = torch.Generator(device=dev).manual_seed(1)
    proj = (torch.randn(w.batch, w.seq, shape.in_proj_width, device=dev, generator=g) * 0.5).to(w.dtype).requires_grad_(True)
    dg = torch.randn(w.batch, w.seq, shape.d_inner, device=dev, generator=g).to(w.dtype)
    params = list(core.parameters())

    def fb():
        return torch.autograd.grad(core(proj), [proj] + params, grad_outputs=dg)

    for _ in range(3):
        fb()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n = 10
    e0.record()
    for _ in range(n):
        fb()
    e1.record()
    torch.cuda.synchronize(dev)
    ms = e0.elapsed_time(e1) / n
    es = w.elem_bytes()
    # projection read by the forward and again by the backward, its gradient written, gated output
    # written and its gradient read: what an ideal single fused pass would move
    ideal = es * w.tokens * (3 * shape.in_proj_width + 2 * shape.d_inner)
    return {"value": w.tokens / (ms * 1e-3) / 1e6, "unit": UNIT, "ms_per_step": ms, "launches_per_step": 22,
            "in_proj_width": shape.in_proj_width, "ideal_bytes": ideal, "achieved_gbs_of_ideal": ideal / (ms * 1e-3) / 1e9}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--config", type=int, default=1)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--path", type=int, default=0, help="0 auto, 1 generic, 2 tensor-core")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    w = synthetic.WORKLOADS[args.config]
    if args.config == 4:
        # The scaling sweep shards its 64 sequences over 8 GPUs: 8 per GPU is one shard.
        w = w.scaled(batch=8)
    if args.impl == "reference":
        run_reference(args, w, rank)
        return

    from mamba_trainer_b200.ssm import Context, ScanInputs, mamba3_scan
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist_
        dist = dist_
        dist.init_process_group("nccl", device_id=dev)

    t = synthetic.make_inputs(w, seed=rank, device=dev)
    for n in ("x", "b", "c", "dt", "a_log", "lam", "theta", "d_skip"):
        if t.get(n) is not None:
            t[n].requires_grad_(True)
    names = [n for n in ("x", "b", "c", "dt", "a_log", "lam", "theta", "d_skip") if t.get(n) is not None]
    if not w.discretization.needs_lambda_projection():
        names.remove("lam")   # a constant lambda is not an input of the op

    def step(src, mid=None):
        inp = ScanInputs.new(src["x"], src["b"], src["c"], src["dt"], src["a_log"], src.get("lam"))
        inp = inp.with_chunk_size(w.chunk).with_state_output(False).with_discretization(w.discretization)
        inp = inp.with_path(args.path)
        if src.get("theta") is not None:
            inp = inp.with_theta(src["theta"])
        inp = inp.with_skip(src["d_skip"])
        out = mamba3_scan(inp)
        if mid is not None:
            mid.record()
        grads = torch.autograd.grad(out.y, [src[n] for n in names if src[n].requires_grad], grad_outputs=src["dy"])
        return out.y, grads

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # The timed steps call the C ABI directly (m3_scan_forward, m3_scan_backward, m3_saved_free) with
    # descriptors and output buffers prepared once: the autograd wrapper above costs 0.2-0.5 ms of host
    # time per step, more than the kernels of the smaller workloads take, and the number reported as
    # `value` is the device's.  Same library calls, same arguments; the first result is checked
    # against the wrapper's.
    import ctypes as C
    from mamba_trainer_b200 import _ffi
    from mamba_trainer_b200.ssm.scan import _DTYPES
    ctx = Context.for_device(dev)
    ctx.bind_current_stream()
    ptr = lambda v: C.c_void_p(v.data_ptr()) if v is not None else None
    B_, T_, H_, P_, R_ = t["x"].shape
    lam_in = t.get("lam") if w.discretization.needs_lambda_projection() else None
    desc = _ffi.ScanDesc(batch=B_, seq=T_, heads=H_, head_dim=P_, d_state=t["b"].shape[3], rank=R_, chunk=int(w.chunk),
                         dtype=_DTYPES[t["x"].dtype], discretization=int(w.discretization.value),
                         dynamics=1 if t.get("theta") is not None else 0, want_state=0, path=int(args.path),
                         x=ptr(t["x"]), b=ptr(t["b"]), c=ptr(t["c"]), dt=ptr(t["dt"]), lambda_=ptr(lam_in),
                         theta=ptr(t.get("theta")), a_log=ptr(t["a_log"]), d_skip=ptr(t["d_skip"]))
    abi_y = torch.empty_like(t["x"])
    abi_out = _ffi.ScanOut(y=ptr(abi_y))
    abi_g = {n: torch.empty_like(t[n]) for n in names}
    bits = {"x": _ffi.GRAD_X, "b": _ffi.GRAD_B, "c": _ffi.GRAD_C, "dt": _ffi.GRAD_DT, "a_log": _ffi.GRAD_A_LOG,
            "lam": _ffi.GRAD_LAMBDA, "theta": _ffi.GRAD_THETA, "d_skip": _ffi.GRAD_D_SKIP}
    abi_mask = 0
    for n in names:
        abi_mask |= bits[n]
    abi_in = _ffi.ScanBwdIn(dy=ptr(t["dy"]))
    abi_grads = _ffi.ScanGrads(dx=ptr(abi_g.get("x")), db=ptr(abi_g.get("b")), dc=ptr(abi_g.get("c")),
                               ddt=ptr(abi_g.get("dt")), dlambda=ptr(abi_g.get("lam")), dtheta=ptr(abi_g.get("theta")),
                               da_log=ptr(abi_g.get("a_log")), dd_skip=ptr(abi_g.get("d_skip")))

    def abi_step(mid=None):
        saved = C.c_void_p()
        ctx.check(ctx.lib.m3_scan_forward(ctx.handle, C.byref(desc), C.byref(abi_out), C.byref(saved)))
        if mid is not None:
            mid.record()
        ctx.check(ctx.lib.m3_scan_backward(ctx.handle, saved, C.byref(abi_in), C.c_uint32(abi_mask), C.byref(abi_grads)))
        ctx.check(ctx.lib.m3_saved_free(ctx.handle, saved))

    y_ref, g_ref = step(t)
    abi_step()
    torch.cuda.synchronize()
    if not torch.equal(y_ref, abi_y) or not all(torch.equal(a, abi_g[n]) for a, n in zip(g_ref, names)):
        raise RuntimeError("the direct C-ABI step and the autograd wrapper disagree")
    del y_ref, g_ref
    for _ in range(max(3, args.warmup)):
        abi_step()
    barrier()
    launches0 = ctx.launch_count()
    sampler = ClockSampler(local) if rank == 0 else None
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    marks = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    ev0.record()
    for i in range(args.steps):
        abi_step(marks[i][0])      # event between the forward and the backward launches
        marks[i][1].record()
    ev1.record()
    barrier()
    clocks = sampler.stop() if sampler else None
    launches = ctx.launch_count() - launches0
    ms = torch.tensor([ev0.elapsed_time(ev1)], device=dev)
    if dist is not None:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_total = float(ms)
    ms_step = ms_total / args.steps
    # per-launch durations of the two stripe kernels (the backward one dominates the step)
    bwd_ms = sum(m0.elapsed_time(m1) for m0, m1 in marks) / args.steps
    fwd_ms = (ev0.elapsed_time(marks[0][0]) + sum(marks[i][1].elapsed_time(marks[i + 1][0])
                                                   for i in range(args.steps - 1))) / args.steps
    value = world * w.tokens / (ms_step * 1e-3) / 1e6

    # End to end: every step starts from pinned HOST tensors (inputs and dy), runs forward +
    # backward through the package's host pipeline (batch slices; copies overlap the kernels) and
    # ends with y and every input gradient back in pinned host memory.
    from mamba_trainer_b200.host_pipeline import HostScanPipeline
    big = [n for n in ("x", "b", "c", "dt", "lam", "theta", "dy") if t.get(n) is not None]
    host = {n: t[n].detach().cpu().pin_memory() for n in big}
    params = {"a_log": t["a_log"], "d_skip": t["d_skip"]}
    pipe = HostScanPipeline(host, w.chunk, w.discretization, dev, slices=min(2, w.batch), params=params, depth=2)
    h2d, d2h = pipe.h2d_bytes, pipe.d2h_bytes

    # One run per step.  Up to two steps are in flight (each with its own pinned output set), so
    # consecutive steps overlap in the two PCIe directions; every step still copies all of its
    # inputs in and all of its results out, and the timed region ends when the last step's
    # results are in host memory.
    def e2e_steps(n):
        flying = []
        for _ in range(n):
            flying.append(pipe.run(host, params))
            if len(flying) == pipe.depth:
                pipe.wait(flying.pop(0))
        for out in flying:
            pipe.wait(out)

    e2e_steps(3)
    barrier()
    e_steps = max(3, min(args.steps, 10))
    ev0.record()
    e2e_steps(e_steps)
    ev1.record()
    barrier()
    ems = torch.tensor([ev0.elapsed_time(ev1)], device=dev)
    if dist is not None:
        dist.all_reduce(ems, op=dist.ReduceOp.MAX)
    e2e_value = world * w.tokens / (float(ems) / e_steps * 1e-3) / 1e6

    if rank == 0:
        peak, peak_kind = measured_peaks()
        th = w.tokens * w.heads
        alg_bytes = w.bytes_per_token_head() * th
        es = w.elem_bytes()
        inputs_b = es * (w.head_dim * w.rank + 2 * w.d_state * w.rank + (w.d_state // 2 if w.rotational else 0) + 2)
        y_b = es * w.head_dim * w.rank
        bwd_bytes = (2 * inputs_b + y_b) * th      # inputs re-read, dy read, every input gradient written
        fwd_bytes = (inputs_b + y_b) * th
        achieved = bwd_bytes / (bwd_ms * 1e-3) / 1e9
        whole = alg_bytes / (ms_step * 1e-3) / 1e9
        flops = w.flops_per_token_head() * th
        traffic = NCU_TRAFFIC_BYTES.get(w.name)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16" if w.dtype == torch.bfloat16 else "f32", "data": "synthetic",
            "config": {"workload": w.name, "batch_per_gpu": w.batch, "seq_len": w.seq, "heads": w.heads,
                       "head_dim": w.head_dim, "d_state": w.d_state, "rank": w.rank, "chunk": w.chunk,
                       "l2": "inputs larger than L2", "sharding": f"batch x heads, {world} shard(s), no collective",
                       "call": "C ABI: m3_scan_forward + m3_scan_backward per step, output buffers prepared once"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": traffic, "peak_kind": peak_kind,
                         "kernel": "tc_bwd_kernel (backward stripe kernel, with its two finalisation launches)",
                         "ms_per_launch": bwd_ms,
                         "forward": {"kernel": "tc_fwd_kernel", "ms_per_launch": fwd_ms,
                                     "achieved": fwd_bytes / (fwd_ms * 1e-3) / 1e9,
                                     "frac": fwd_bytes / (fwd_ms * 1e-3) / 1e9 / peak},
                         "whole_step": {"achieved": whole, "frac": whole / peak, "frac_of_8TBs": whole / 8000.0,
                                        "tflops": flops / (ms_step * 1e-3) / 1e12}},
            "clocks": clocks, "gpu_launches": int(launches),
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        }
        if world == 1:
            line["mixer_core"] = mixer_core_leg(w, dev)
        if not args.no_cpu_baseline and world == 1:
            v, cores, sample = cpu_oracle_throughput(w)
            line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
