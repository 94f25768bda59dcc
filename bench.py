"""Benchmark of the bound-propagation hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (config c4): ReLU-split branch-and-bound subdomains of an MLP
784-512x4-10 (fp32, He init, one input, eps 0.02, 9 margin specs).  One "step"
bounds one batch of 8192 subdomains per GPU: IBP under the split constraints,
adaptive alpha start, 10 alpha-CROWN Adam steps (11 lower-bound evaluations, 10
analytic gradients, 1 upper-bound evaluation at the best alpha), verdicts and,
with N > 1, the all-gather of bounds and verdicts.  Metric: BaB domains bounded/s
(whole job, all ranks).  `value` is measured with inputs resident in HBM, `e2e`
through the public API with pinned HOST buffers (H2D and D2H inside the timed
region).  `--impl reference` times the CPU restatement of the reference's own
PyTorch path (the oracle; the reference is pure Python and is not installed on
the GPU box) on a bounded sample of the same workload, on all host cores.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

DOMAINS_PER_GPU = 8192
ALPHA_STEPS = 10
LR = 0.1
# DRAM bytes of one backward-contraction launch of a 512x512 layer at 8192 domains (M = 73728 rows):
# ncu capture at 4096 domains (profiles/crown_tc_kernel_bwd_c4_4096domains.md) scaled x2 by the row count.
TRAFFIC_BYTES_PER_LAUNCH = 2 * (104.8e6 + 31.7e6)
METRIC = "bab_domains_bounded_per_s"
UNIT = "domains/s"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16": float(d["bf16_tflops"]), "bf16_sustained": float(d["bf16_tflops_sustained"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50", "-i", str(self.gpu_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons), "samples": len(sm)}


def build_host_batch(wl, root_pre, n_domains: int, rank: int):
    """Pinned host tensors of one subdomain batch for this rank (seeded per rank)."""
    from boundflow_b200 import workloads as W

    wl.generator = torch.Generator("cpu").manual_seed(1004_000 + rank)
    splits = W.make_split_domains(wl, root_pre, n_domains=n_domains)
    lo = wl.lo.expand(n_domains, -1).contiguous().pin_memory()
    up = wl.up.expand(n_domains, -1).contiguous().pin_memory()
    C = wl.C.expand(n_domains, -1, -1).contiguous().pin_memory()
    splits = [s.pin_memory() for s in splits]
    return lo, up, C, splits


def sweep_flops(widths, M):
    """Algorithmic flops of one backward sweep (one side) / one adjoint sweep for M coefficient rows."""
    bwd = sum(2.0 * M * widths[k] * widths[k + 1] for k in range(len(widths) - 1))
    adj = sum(2.0 * M * widths[k] * widths[k + 1] for k in range(len(widths) - 2))
    return bwd, adj


def cpu_baseline(sample_domains: int, reps: int = 1):
    """The oracle (CPU restatement of the reference's PyTorch path) on a bounded sample."""
    from boundflow_b200 import workloads as W
    from oracle import crown_oracle as O

    torch.set_num_threads(os.cpu_count() or 1)
    wl = W.make_workload("c4")
    root = O.forward_ibp_trace(wl.layers, O.box_input(wl.lo, wl.up))
    wl.generator = torch.Generator("cpu").manual_seed(1004_000)
    splits = W.make_split_domains(wl, root.pre, n_domains=sample_domains)
    inp = O.box_input(wl.lo.expand(sample_domains, -1).contiguous(), wl.up.expand(sample_domains, -1).contiguous())
    C = wl.C.expand(sample_domains, -1, -1).contiguous()
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        trace = O.forward_ibp_trace(wl.layers, inp, splits=splits)
        a0 = O.adaptive_alpha_init(trace)
        bl, bu, _, _ = O.alpha_crown(wl.layers, inp, C, steps=ALPHA_STEPS, lr=LR, alpha0=a0, trace=trace)
        _ = O.verdict(bl)
        times.append(time.perf_counter() - t0)
    times.sort()
    t = times[len(times) // 2]
    return sample_domains / t, t


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample = 2048
    t0 = time.perf_counter()
    for _ in range(max(args.warmup, 0) and 1):
        cpu_baseline(sample)
    vals = []
    for _ in range(max(1, min(args.steps, 3))):
        v, _t = cpu_baseline(sample)
        vals.append(v)
    v = sum(vals) / len(vals)
    cores = os.cpu_count() or 1
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": len(vals), "warmup": 1 if args.warmup else 0,
        "ms_per_step": 1e3 * sample / v, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "c4: MLP 784-512x4-10, ReLU-split BaB subdomains (10 split neurons), 10 alpha-CROWN steps, 9 specs", "domains_per_step": sample},
        "cpu_baseline": {"value": v, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"{sample} subdomains of the same workload per step, torch CPU ops on {cores} threads (the reference is pure Python/torch; its CPU path is restated by oracle/crown_oracle.py)"},
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": time.perf_counter() - t0,
    }
    print(json.dumps(line))


def crown_bounds_secondary(world: int, rank: int, dev, only=None):
    """Second half of the metric: CROWN bounds/s (one bound = one (input, spec) lower bound) on the
    input-sharded configurations, whole job over all ranks, device-timed, max over ranks.
      c1: IBP + CROWN (both sides), MLP 784-100-100-10, 64 inputs
      c2: CROWN with CROWN intermediate bounds, MNIST-shaped CNN, 256 inputs
      c3: alpha-CROWN, 20 Adam steps, MLP 784-256x5-10, 128 inputs
      c5: CROWN with full CROWN intermediate bounds, CIFAR-shaped CNN, 64 inputs"""
    import torch.distributed as dist

    from boundflow_b200 import _lib
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import AlphaState, adaptive_alpha_from_trace, ibp_trace, run_alpha_beta_crown_mlp, run_crown_ibp_mlp, run_crown_intermediate_mlp
    from boundflow_b200.dist import gather_domain_results, shard_range
    from boundflow_b200.ir import InputSpec

    lib = _lib.load()
    out = {}
    for name, reps in (("c1", 20), ("c2", 2), ("c3", 5), ("c5", 1)):
        if only is not None and name != only:
            continue
        wl = W.make_workload(name)
        n = wl.x.shape[0]
        a, b = shard_range(n, rank, world)
        lo, up, C = wl.lo[a:b].to(dev), wl.up[a:b].to(dev), wl.C[a:b].to(dev)
        spec = InputSpec.box(value_name="input", lower=lo, upper=up)

        def run():
            if name == "c1":
                res = run_crown_ibp_mlp(wl.module, spec, linear_spec_C=C).lower
            elif name == "c2":
                res = run_crown_intermediate_mlp(wl.module, spec, linear_spec_C=C, chunk_rows=512)[0].lower
            elif name == "c5":  # about 4096 coefficient rows per sweep
                res = run_crown_intermediate_mlp(wl.module, spec, linear_spec_C=C, chunk_rows=max(64, 4096 // max(1, b - a)))[0].lower
            else:
                tr = ibp_trace(wl.module, spec)
                a0 = adaptive_alpha_from_trace(tr)
                res = run_alpha_beta_crown_mlp(wl.module, spec, linear_spec_C=C, steps=20, lr=0.1, per_batch_params=True,
                                               warm_start_alpha=AlphaState(dict(zip(wl.relu_names, a0))))[0].lower
            verdict = torch.empty(res.shape[0], dtype=torch.int8, device=dev)
            _lib.check(lib.bf_verdict(res.data_ptr(), 0.0, 1e-6, verdict.data_ptr(), None, res.shape[0], res.shape[1],
                                      torch.cuda.current_stream().cuda_stream))
            return gather_domain_results(res, verdict, n) if world > 1 else (res, verdict)

        for _ in range(1 if name == "c5" else 2):
            run()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            run()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / reps
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        out[name] = {"bounds_per_s": n * 9 / (ms * 1e-3), "ms": ms, "inputs": n}
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--domains", type=int, default=DOMAINS_PER_GPU, help="subdomains per GPU per step")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--secondary-only", default=None, choices=["c1", "c2", "c3", "c5"],
                    help="time only this CROWN bounds/s configuration and print its figures (profiling aid)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
        return

    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the backend has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    from boundflow_b200.csrc import build as _build

    _build.build()
    from boundflow_b200 import _lib
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import bound_split_domains, ibp_trace
    from boundflow_b200.dist import gather_domain_results
    from boundflow_b200.ir import InputSpec

    lib = _lib.load()
    if args.secondary_only:
        sec = crown_bounds_secondary(world, rank, dev, only=args.secondary_only)
        if rank == 0:
            print(json.dumps({"crown_bounds_per_s": sec, "n_gpus": world}))
        if world > 1:
            dist.destroy_process_group()
        return
    warmup = max(int(args.warmup), 3)
    D = int(args.domains)
    wl = W.make_workload("c4")
    names = wl.relu_names
    root = ibp_trace(wl.module, InputSpec.box(value_name="input", lower=wl.lo.to(dev), upper=wl.up.to(dev)))
    root_pre = [(l.cpu(), u.cpu()) for l, u in zip(root.pre_l, root.pre_u)]
    h_lo, h_up, h_C, h_splits = build_host_batch(wl, root_pre, D, rank)
    d_lo, d_up, d_C = h_lo.to(dev), h_up.to(dev), h_C.to(dev)
    d_splits = {n: s.to(dev) for n, s in zip(names, h_splits)}
    d_spec = InputSpec.box(value_name="input", lower=d_lo, upper=d_up)
    n_total = D * world

    def step_resident():
        res = bound_split_domains(wl.module, d_spec, linear_spec_C=d_C, relu_split_state=d_splits, steps=ALPHA_STEPS, lr=LR)
        lower, verdict = gather_domain_results(res.lower, res.verdict, n_total) if world > 1 else (res.lower, res.verdict)
        return lower, verdict, res

    def step_e2e():
        spec = InputSpec.box(value_name="input", lower=h_lo.to(dev, non_blocking=True), upper=h_up.to(dev, non_blocking=True))
        res = bound_split_domains(
            wl.module, spec, linear_spec_C=h_C.to(dev, non_blocking=True),
            relu_split_state={n: s.to(dev, non_blocking=True) for n, s in zip(names, h_splits)}, steps=ALPHA_STEPS, lr=LR)
        lower, verdict = gather_domain_results(res.lower, res.verdict, n_total) if world > 1 else (res.lower, res.verdict)
        return lower.to("cpu"), verdict.to("cpu"), res.infeasible.to("cpu")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        out = None
        for _ in range(steps):
            out = fn()
        stop.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(stop)
        barrier()
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, out

    for _ in range(warmup):
        step_resident()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    lib.bf_kernel_timing_enable(1)
    launches0 = _lib.launch_count()
    ms_res, out = timed(step_resident, args.steps)
    launches = _lib.launch_count() - launches0
    n_l, t_l = ctypes.c_int(), ctypes.c_float()
    lib.bf_kernel_timing_read(0, ctypes.byref(n_l), ctypes.byref(t_l))
    n_a, t_a = ctypes.c_int(), ctypes.c_float()
    lib.bf_kernel_timing_read(1, ctypes.byref(n_a), ctypes.byref(t_a))
    lib.bf_kernel_timing_enable(0)

    for _ in range(2):
        step_e2e()
    ms_e2e, out_e2e = timed(step_e2e, args.steps)
    clocks = sampler.stop() if rank == 0 else None  # sampled over both timed regions (resident and end-to-end)

    secondary = crown_bounds_secondary(world, rank, dev)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    lower, verdict, res = out
    infeasible = int(res.infeasible.sum().item())
    proven = int(verdict.sum().item())
    peaks = measured_peaks()
    widths = [784, 512, 512, 512, 512, 10]
    M = D * 9
    bwd_flops, adj_flops = sweep_flops(widths, M)
    sweeps_per_step = ALPHA_STEPS + 2          # 11 lower evaluations + 1 upper
    bwd_total_flops = bwd_flops * sweeps_per_step * args.steps
    adj_total_flops = adj_flops * ALPHA_STEPS * args.steps
    fp32_equiv_peak = peaks["bf16_sustained"] / 6.0  # TF32 runs at half the bf16 rate; 3 TF32 MMAs per fp32-faithful product
    achieved = bwd_total_flops / (t_l.value * 1e-3) / 1e12 if t_l.value > 0 else None
    achieved_adj = adj_total_flops / (t_a.value * 1e-3) / 1e12 if t_a.value > 0 else None
    value = n_total * args.steps / (ms_res * 1e-3)
    e2e_value = n_total * args.steps / (ms_e2e * 1e-3)
    h2d = h_lo.numel() * 4 * 2 + h_C.numel() * 4 + sum(s.numel() for s in h_splits)
    d2h = n_total * 9 * 4 + n_total + D * 4
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warmup,
        "ms_per_step": ms_res / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {
            "workload": "c4: MLP 784-512x4-10, 1 input eps 0.02, ReLU-split BaB subdomains (10 split neurons each), 10 alpha-CROWN Adam steps lr 0.1, 9 margin specs",
            "domains_per_gpu_per_step": D, "domains_per_step": n_total, "alpha_steps": ALPHA_STEPS,
            "l2": "per-step working set (coefficient tensors, > 1 GB) exceeds the 126 MB L2; no explicit flush",
            "parallelism": f"domains sharded over {world} GPU(s), weights replicated, one all-gather of bounds+verdicts per step",
        },
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h), "ms_per_step": ms_e2e / args.steps},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "roofline": {
            "bound": "tensor", "kernel": "crown_tc_kernel<bwd> (ReLU-backward + Linear-backward contraction, tcgen05 3xTF32; the 10-wide top layer runs as a store-bound thin kernel)",
            "achieved": achieved, "peak": fp32_equiv_peak, "unit": "TFLOP/s", "frac": (achieved / fp32_equiv_peak) if achieved else None,
            "traffic": TRAFFIC_BYTES_PER_LAUNCH * (D / 8192.0),
            "traffic_source": "ncu dram__bytes_read+write of one 512x512-layer launch at 4096 domains, scaled by rows (profiles/)",
            "peak_source": f"{peaks['source']} bf16 sustained {peaks['bf16_sustained']} TFLOP/s / 6 = fp32-equivalent 3xTF32 tensor peak",
            "launches": n_l.value, "avg_launch_ms": (t_l.value / n_l.value) if n_l.value else None,
            "share_of_step": t_l.value / ms_res if ms_res else None,
        },
        "roofline_adjoint": {
            "kernel": "crown_tc_adjoint_kernel (gradient sweep, feature-major tcgen05 3xTF32)", "achieved": achieved_adj, "unit": "TFLOP/s",
            "frac": (achieved_adj / fp32_equiv_peak) if achieved_adj else None, "launches": n_a.value,
            "share_of_step": t_a.value / ms_res if ms_res else None,
        },
        "crown_bounds_per_s": secondary,
        "result_check": {"domains": n_total, "proven": proven, "infeasible_local": infeasible,
                         "mean_lower": float(lower[torch.isfinite(lower).all(dim=1)].mean().item())},
    }
    if not args.no_cpu_baseline and world == 1:
        sample = 2048
        v, t = cpu_baseline(sample)
        cores = os.cpu_count() or 1
        line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cores, "kind": "port",
                                "sample": f"{sample} subdomains of the same workload, one pass ({t:.1f} s), torch CPU ops on {cores} threads"}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
