"""Benchmark of the fused Mamba-3 SSD scan: forward + backward Mtokens/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config I] [--impl ours|reference]

A step is one forward and one backward pass of the scan over the workload's whole batch of synthetic
inputs (mamba_trainer_b200.synthetic).  The default workload is the scaling sweep (config 4: 64
sequences of 16384 tokens, 32 heads, rank 2, rotational, learned trapezoid): its 64 sequences are
cut over the ranks with `sharding.shard_plan` (strong scaling, no collective in the path), so one GPU
runs all 64.  Configs 0-3 run whole on every rank (weak scaling).  Rank 0 prints one JSON line.
`--impl reference` times the CPU oracle (the restated reference composition) on the host cores.
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

from mamba_trainer_b200 import sharding, synthetic  # noqa: E402

# dram__bytes_read.sum + dram__bytes_write.sum of ONE backward stripe-kernel launch per (token, head),
# from the committed ncu captures under profiles/ (a small case of the same instantiation; traffic is
# proportional to the token-heads a launch processes).  None where no capture was taken.
NCU_TRAFFIC_BYTES_PER_TOKEN_HEAD = {
    "cfg1_siso_trapezoid_bf16": 267403520 / (8 * 2048 * 12),
    # profiles/tc_fwd_bwd_kernels_cfg4.md: batch 4 x seq 4096 (whole stripes) and batch 8 x seq 4096 (stripes cut
    # into time segments, which adds the hand-over of the state between segments)
    "cfg4_mimo2_scaling_bf16": {"whole": 1722.7e6 / (4 * 4096 * 32), "split": 3560.8e6 / (8 * 4096 * 32)},
}


def traffic_per_token_head(w, sms: int):
    """The captured DRAM traffic per (token, head) of the instantiation this shard runs: the library cuts
    stripes in time when there are more stripes than SMs but fewer than six per SM (tc_segment_plan)."""
    v = NCU_TRAFFIC_BYTES_PER_TOKEN_HEAD.get(w.name)
    if isinstance(v, dict):
        stripes = w.batch * w.heads
        return v["split"] if sms < stripes < 6 * sms else v["whole"]
    return v

METRIC = "mamba3_ssd_scan_fwd_bwd_throughput"
UNIT = "Mtokens/s"
STRONG = {4}           # configs whose global batch is cut over the ranks


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


def cpu_sample_shape(w):
    """The bounded slice of a workload one CPU step runs: wide enough to occupy the host's cores
    (every batch row and head is an independent recurrence, so throughput in token-heads per second
    carries over), short enough that a forward + backward takes seconds.  Small workloads run whole."""
    if w.tokens * w.heads * w.rank * w.rank <= 8 * 2048 * 12:
        return w, "the whole workload"
    heads = min(w.heads, 16)
    seq = min(w.seq, 4096)
    batch = min(w.batch, 2)
    sw = w.scaled(batch=batch, heads=heads, seq=seq)
    note = f"batch {batch} x seq {seq} x {heads} of {w.heads} heads, scaled by batch x heads"
    if seq < w.seq:
        note += (f"; the sequence is cut from {w.seq} to {seq}, which flatters the CPU: the reference's inter-chunk "
                 "pass costs O(chunks^2) per sequence")
    return sw, note


def cpu_oracle_throughput(w, steps: int = 5, warmup: int = 1, budget_s: float = 25.0):
    """Time the CPU oracle (fp32, forward + backward, every host core) on `cpu_sample_shape(w)`.
    `warmup` untimed steps (at most 3), then `steps` timed ones (at least 5 unless `budget_s` seconds run
    out first, never fewer than 1); the value is the MEDIAN step, the spread (max - min) / median is
    reported beside it."""
    from oracle import m3_oracle as O
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    sw, note = cpu_sample_shape(w)
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
    want = max(5, steps)
    times, t_start = [], time.perf_counter()
    while len(times) < want and (not times or time.perf_counter() - t_start < budget_s):
        times.append(one())
    med = statistics.median(times)
    spread = (max(times) - min(times)) / med
    tok_heads_per_s = sw.tokens * sw.heads / med
    value = tok_heads_per_s / w.heads / 1e6   # Mtokens/s of the full-head workload
    sample = (f"{note}; fp32, median of {len(times)} steps after {warm} warm-up, "
              f"spread (max - min) / median = {spread:.3f}, {med * 1e3:.0f} ms per sampled step")
    return value, cores, sample, spread


def global_workload(config: int):
    return synthetic.WORKLOADS[config]


def run_reference(args, w, rank):
    if rank != 0:
        return
    value, cores, sample, spread = cpu_oracle_throughput(w, steps=args.steps, warmup=args.warmup, budget_s=120.0)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": w.tokens / (value * 1e6) * 1e3,
        "higher_is_better": True, "scaling": "strong" if args.config in STRONG else "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": workload_config(w, args.gpus, args.config),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample,
                         "spread": spread},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "ms_per_step is the whole workload's step time implied by the sampled throughput",
    }
    print(json.dumps(line), flush=True)


def workload_config(w, world, config):
    strong = config in STRONG
    return {"workload": w.name, "global_batch": w.batch * (1 if strong else world), "seq_len": w.seq, "heads": w.heads,
            "head_dim": w.head_dim, "d_state": w.d_state, "rank": w.rank, "chunk": w.chunk,
            "l2": "inputs larger than L2",
            "sharding": (f"batch x heads, {world} shard(s) of the global batch, no collective in the path" if strong
                         else f"every rank runs the whole workload on its own data ({world} replica(s))"),
            "call": "C ABI: m3_scan_forward + m3_scan_backward per step, output buffers prepared once"}


def mixer_core_leg(w, dev):
    """Secondary figure, not the headline: the whole stretch of the mixer between its two projections
    (convolution + SiLU, B/C bias + RMS norm + layout, dt / lambda activations, the scan, the gate)
    forward + backward as one tape node, on the workload's shapes with groups = heads."""
    from mamba_trainer_b200.nn import MixerCore, MixerShape
    from mamba_trainer_b200.ssm import Context
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
    ctx = Context.for_device(dev)
    l0 = ctx.launch_count()
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
    return {"value": w.tokens / (ms * 1e-3) / 1e6, "unit": UNIT, "ms_per_step": ms,
            "launches_per_step": (ctx.launch_count() - l0) / n,
            "in_proj_width": shape.in_proj_width, "ideal_bytes": ideal, "achieved_gbs_of_ideal": ideal / (ms * 1e-3) / 1e9}


def shard_check(dist, dev, w, rank, world):
    """The CUDA path across GPUs, outside every timed region: each rank builds the SAME seeded global
    inputs (a short-sequence copy of the workload), runs forward + backward on its `shard_plan` slice,
    the shards' y and dx are all-gathered and the per-head partial sums of d a_log / d D all-reduced
    over NCCL (device tensors; no kernel ever takes a peer's memory as an operand), and rank 0 compares
    with its own run of the unsharded problem: bit for bit for the per-token tensors, float32 tolerance
    for the per-head sums (their summation order differs)."""
    run_scan_fb = _run_scan_fb
    sw = w.scaled(seq=min(w.seq, 512))
    t = synthetic.make_inputs(sw, seed=1234, device=dev)
    shard = sharding.shard_plan(sw.batch, sw.heads, world, rank)
    local = sharding.shard_inputs(t, shard)
    y, g = run_scan_fb(local, sw)
    full_y = sharding.gather_per_token(y, sw.batch, sw.heads)
    full_dx = sharding.gather_per_token(g["x"], sw.batch, sw.heads)
    da = sharding.reduce_per_head(g["a_log"], sw.heads, shard)
    dd = sharding.reduce_per_head(g["d_skip"], sw.heads, shard)
    verdict = "ok"
    if rank == 0:
        ey, eg = run_scan_fb(t, sw)
        close = lambda a, e: bool(((a - e).abs() <= 1e-5 * max(1.0, float(e.abs().max())) + 1e-4 * e.abs()).all())
        bad = []
        if not torch.equal(full_y, ey):
            bad.append("y")
        if not torch.equal(full_dx, eg["x"]):
            bad.append("dx")
        if not close(da, eg["a_log"]):
            bad.append("da_log")
        if not close(dd, eg["d_skip"]):
            bad.append("dd_skip")
        if bad:
            verdict = "MISMATCH: " + ", ".join(bad)
    flag = torch.tensor([0 if verdict == "ok" else 1], device=dev)
    dist.broadcast(flag, 0)
    return verdict, {"seq_len": sw.seq, "global_batch": sw.batch, "gathered": ["y", "dx"], "reduced": ["da_log", "dd_skip"]}


def _run_scan_fb(t, w):
    """Forward + backward through the public host API on tensors already on the device."""
    from mamba_trainer_b200.ssm import ScanInputs, mamba3_scan
    names = [n for n in ("x", "b", "c", "dt", "a_log", "lam", "theta", "d_skip") if t.get(n) is not None]
    leaf = {n: t[n].detach().clone().requires_grad_(True) for n in names}
    inp = ScanInputs.new(leaf["x"], leaf["b"], leaf["c"], leaf["dt"], leaf["a_log"], leaf.get("lam"))
    inp = inp.with_chunk_size(w.chunk).with_state_output(False).with_discretization(w.discretization)
    if "theta" in leaf:
        inp = inp.with_theta(leaf["theta"])
    inp = inp.with_skip(leaf["d_skip"])
    y = mamba3_scan(inp).y
    gl = torch.autograd.grad(y, [leaf[n] for n in names], grad_outputs=t["dy"])
    return y.detach(), {n: v.detach() for n, v in zip(names, gl)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--config", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--path", type=int, default=0, help="0 auto, 1 generic, 2 tensor-core")
    ap.add_argument("--batch", type=int, default=0, help="override the workload's global batch (profiling of a small case)")
    ap.add_argument("--seq", type=int, default=0, help="override the workload's sequence length (profiling of a small case)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--mixer-core", action="store_true", help="add the secondary mixer-core figure")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    gw = global_workload(args.config)
    if args.batch:
        gw = gw.scaled(batch=args.batch)
    if args.seq:
        gw = gw.scaled(seq=args.seq)
    if args.impl == "reference":
        run_reference(args, gw, rank)
        return

    from mamba_trainer_b200.ssm import Context
    from mamba_trainer_b200.host_pipeline import bind_host_thread_near
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    # one process per GPU: keep this one, and the pinned staging buffers it will allocate, on the GPU's side
    # of the box (matters for the end-to-end leg once several ranks copy at the same time)
    numa = bind_host_thread_near(dev)
    dist = None
    if world > 1:
        import torch.distributed as dist_
        dist = dist_
        dist.init_process_group("nccl", device_id=dev)

    strong = args.config in STRONG
    fallback_note = None
    if strong:
        shard = sharding.shard_plan(gw.batch, gw.heads, world, rank)
        w = gw.scaled(batch=shard.n_batch, heads=shard.n_heads)
    else:
        w = gw
    # This rank's data: seeded by (config seed 0, rank), generated on the device in batch chunks so
    # that the float32 temporaries of the generator stay small beside the bf16 tensors they become.
    while True:
        try:
            t = synthetic.make_inputs_chunked(w, seed=1000 * rank, device=dev, chunk=8)
            break
        except torch.OutOfMemoryError:
            if w.batch <= 1:
                raise
            t = None
            torch.cuda.empty_cache()
            w = w.scaled(batch=max(1, w.batch // 2))
            fallback_note = f"allocation refused; per-rank batch reduced to {w.batch}"
    names = [n for n in ("x", "b", "c", "dt", "a_log", "lam", "theta", "d_skip") if t.get(n) is not None]
    if not w.discretization.needs_lambda_projection():
        names.remove("lam")   # a constant lambda is not an input of the op

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # The timed steps call the C ABI directly (m3_scan_forward, m3_scan_backward, m3_saved_free) with
    # descriptors and output buffers prepared once: the autograd wrapper costs 0.2-0.5 ms of host time per
    # step, more than the kernels of the smaller workloads take.  Same library calls, same arguments; on
    # workloads small enough to hold a second set of outputs the first result is checked against the wrapper's.
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

    abi_step()
    ctx.sync()   # also reads the device error flag: a bounded wait that gave up fails the run here
    in_bytes = sum(v.numel() * v.element_size() for v in t.values() if v is not None)
    if in_bytes < (8 << 30):
        y_ref, g_ref = _run_scan_fb(t, w)
        if not torch.equal(y_ref, abi_y) or not all(torch.equal(g_ref[n], abi_g[n]) for n in names):
            raise RuntimeError("the direct C-ABI step and the autograd wrapper disagree")
        del y_ref, g_ref
    warm = max(3, args.warmup)
    for _ in range(warm - 1):
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
    ctx.sync()   # the device error flag again: no timed step may have given up a wait
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
    ntok = torch.tensor([float(w.tokens)], device=dev)     # tokens this rank processed per step
    if dist is not None:
        dist.all_reduce(ntok, op=dist.ReduceOp.SUM)
    value = float(ntok) / (ms_step * 1e-3) / 1e6

    check, check_cfg = None, None
    if dist is not None and strong:
        check, check_cfg = shard_check(dist, dev, gw, rank, world)

    # End to end: every step starts from pinned HOST tensors (inputs and dy), runs forward + backward
    # through the package's host pipeline (batch slices; copies overlap the kernels) and ends with y and
    # every input gradient back in pinned host memory.  The scan is PCIe-bound there whatever the batch,
    # so a step moves at most 8 sequences of the rank's shard (56 GB of pinned memory per direction would
    # be needed for the whole scaling workload on one GPU); tokens per second count what was moved.
    e2e = None
    if not args.no_e2e:
        del abi_y, abi_g
        from mamba_trainer_b200.host_pipeline import HostScanPipeline
        eb = min(w.batch, 8)
        big = [n for n in ("x", "b", "c", "dt", "lam", "theta", "dy") if t.get(n) is not None]
        host = {n: t[n][:eb].detach().cpu().pin_memory() for n in big}
        params = {"a_log": t["a_log"], "d_skip": t["d_skip"]}
        for n in big:
            t[n] = None
        torch.cuda.empty_cache()
        pipe = HostScanPipeline(host, w.chunk, w.discretization, dev, slices=min(2, eb), params=params, depth=2)
        h2d, d2h = pipe.h2d_bytes, pipe.d2h_bytes

        # Up to two steps are in flight (each with its own pinned output set), so consecutive steps
        # overlap in the two PCIe directions; every step still copies all of its inputs in and all of
        # its results out, and the timed region ends when the last step's results are in host memory.
        def e2e_steps(n):
            flying = []
            for _ in range(n):
                flying.append(pipe.run(host, params))
                if len(flying) == pipe.depth:
                    pipe.wait(flying.pop(0))
            for out in flying:
                pipe.wait(out)

        # the two PCIe directions on their own (1 GiB each way, every rank at the same time): what the
        # end-to-end figure is made of
        def copy_rate(dst, src):
            barrier()
            c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            dst.copy_(src, non_blocking=True)
            torch.cuda.synchronize()
            c0.record()
            for _ in range(3):
                dst.copy_(src, non_blocking=True)
            c1.record()
            torch.cuda.synchronize()
            r = torch.tensor([3 * src.numel() / (c0.elapsed_time(c1) * 1e-3) / 1e9], device=dev)
            if dist is not None:
                dist.all_reduce(r, op=dist.ReduceOp.MIN)
            return float(r)
        probe_h = torch.empty(1 << 30, dtype=torch.uint8).pin_memory()
        probe_d = torch.empty(1 << 30, dtype=torch.uint8, device=dev)
        h2d_gbs, d2h_gbs = copy_rate(probe_d, probe_h), copy_rate(probe_h, probe_d)
        del probe_h, probe_d

        e2e_steps(2)
        barrier()
        e_steps = max(3, min(args.steps, 6))
        ev0.record()
        e2e_steps(e_steps)
        ev1.record()
        barrier()
        ctx.sync()
        ems = torch.tensor([ev0.elapsed_time(ev1)], device=dev)
        if dist is not None:
            dist.all_reduce(ems, op=dist.ReduceOp.MAX)
        e2e_value = world * eb * w.seq / (float(ems) / e_steps * 1e-3) / 1e6
        e2e = {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "sequences_per_step_per_gpu": eb, "steps": e_steps,
               "pcie_gbs_per_gpu": {"h2d": h2d_gbs, "d2h": d2h_gbs, "note": "slowest rank, all ranks copying at once"},
               "host_numa": numa}

    if rank == 0:
        peak, peak_kind = measured_peaks()
        th = w.tokens * w.heads        # token-heads one launch on this rank processes
        alg_bytes = w.bytes_per_token_head() * th
        es = w.elem_bytes()
        inputs_b = es * (w.head_dim * w.rank + 2 * w.d_state * w.rank + (w.d_state // 2 if w.rotational else 0) + 2)
        y_b = es * w.head_dim * w.rank
        bwd_bytes = (2 * inputs_b + y_b) * th      # inputs re-read, dy read, every input gradient written
        fwd_bytes = (inputs_b + y_b) * th
        achieved = bwd_bytes / (bwd_ms * 1e-3) / 1e9
        whole = alg_bytes / (ms_step * 1e-3) / 1e9
        flops = w.flops_per_token_head() * th
        per_th = traffic_per_token_head(w, torch.cuda.get_device_properties(dev).multi_processor_count)
        cfg = workload_config(gw, world, args.config)
        cfg["batch_per_gpu"] = w.batch
        # rank 1 with real dynamics takes the direct form of the stripe kernels, float32 the generic family
        direct = w.rank == 1 and not w.rotational
        if w.dtype != torch.bfloat16:
            fwd_name, bwd_name = "generic family (k_chunk_state ... k_chunk_out)", "generic family (kb_* kernels)"
        else:
            fwd_name = "tc_fwd_direct_kernel" if direct else "tc_fwd_kernel"
            bwd_name = "tc_bwd_direct_kernel" if direct else "tc_bwd_kernel"
        if fallback_note:
            cfg["fallback"] = fallback_note
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": warm, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong" if strong else "weak",
            "vs_baseline": None, "dtype": "bf16" if w.dtype == torch.bfloat16 else "f32", "data": "synthetic",
            "config": cfg,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": per_th * th if per_th else None, "peak_kind": peak_kind,
                         "kernel": bwd_name + " (backward stripe kernel, with its two finalisation launches)",
                         "ms_per_launch": bwd_ms, "algorithmic_bytes_per_launch": bwd_bytes,
                         "forward": {"kernel": fwd_name, "ms_per_launch": fwd_ms,
                                     "achieved": fwd_bytes / (fwd_ms * 1e-3) / 1e9,
                                     "frac": fwd_bytes / (fwd_ms * 1e-3) / 1e9 / peak},
                         "whole_step": {"achieved": whole, "frac": whole / peak, "frac_of_8TBs": whole / 8000.0,
                                        "tflops": flops / (ms_step * 1e-3) / 1e12}},
            "clocks": clocks, "gpu_launches": int(launches), "timed_region_ms": ms_total,
        }
        if e2e is not None:
            line["e2e"] = e2e
        if check is not None:
            line["shard_check"] = check
            line["shard_check_config"] = check_cfg
        if args.mixer_core and world == 1:
            line["mixer_core"] = mixer_core_leg(w.scaled(batch=min(w.batch, 8)), dev)
        if not args.no_cpu_baseline and world == 1:
            v, cores, sample, spread = cpu_oracle_throughput(gw)
            line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample,
                                    "spread": spread}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()
    if check is not None and check != "ok":
        sys.exit(3)


if __name__ == "__main__":
    main()
