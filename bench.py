"""Benchmark of the bound-propagation hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--scaling weak|strong]

Workload (config c4): ReLU-split branch-and-bound subdomains of an MLP
784-512x4-10 (fp32, He init, one input, eps 0.02, 9 margin specs).  One "step"
bounds one batch of 8192 subdomains per GPU: IBP under the split constraints,
adaptive alpha start, 10 alpha-CROWN Adam steps (11 lower-bound evaluations, 10
analytic gradients, 1 upper-bound evaluation at the best alpha), verdicts and,
with N > 1, the all-gather of bounds and verdicts.  Metric: BaB domains bounded/s
(whole job, all ranks).  `value` is measured with inputs resident in HBM, `e2e`
through the public API with pinned HOST buffers (H2D and D2H inside the timed
region; the input box and the spec rows, shared by all subdomains of one problem,
travel once and are repeated on the device).

`--scaling strong` splits ONE 8192-subdomain batch over the N GPUs instead of
giving every GPU its own batch.

`--impl reference` times the reference's own CPU implementation of the same step
on the host cores: the reference's functions from `oracle/_ref` (built by
`oracle/make_ref.py`) when present, else the CPU restatement `oracle/crown_oracle.py`,
on a bounded sample of the workload per step.

Other modes (profiling aids, one JSON line each): `--secondary-only cN` times one
CROWN bounds/s configuration, `--kernels` times single kernels on resident data and
reports their HBM / FP32 rooflines, `--conv-layers a,b --rows R` times the fused ReLU +
transposed-convolution layer call on the CNN configurations' layer shapes,
`--linear-layer D,S,n_cur,n_prev` times the ReLU + Linear backward layer call on one
synthetic layer (the kernel is chosen by the library's environment switches).
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
REFERENCE_SAMPLE = 512  # subdomains per step of the CPU arm (the same workload, a bounded sample)
# DRAM bytes of one backward-contraction launch of a 512x512 layer at 8192 domains (M = 73728 rows):
# ncu capture at 4096 domains (profiles/crown_tc_kernel_bwd_c4_4096domains.md) scaled x2 by the row count.
TRAFFIC_BYTES_PER_LAUNCH = 2 * (104.8e6 + 31.7e6)
METRIC = "bab_domains_bounded_per_s"
UNIT = "domains/s"
WORKLOAD = "c4: MLP 784-512x4-10, 1 input eps 0.02, ReLU-split BaB subdomains (10 split neurons each), 10 alpha-CROWN Adam steps lr 0.1, 9 margin specs"
FFMA_PEAK_TFLOPS = 148 * 128 * 2 * 1.965e9 / 1e12  # FP32 FMA lanes x 2 flop x max SM clock


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
    """Pinned host tensors of one subdomain batch for this rank (seeded per rank): the input box and the spec rows of
    the one problem the subdomains belong to, and one int8 split row per subdomain and ReLU layer."""
    from boundflow_b200 import workloads as W

    wl.generator = torch.Generator("cpu").manual_seed(1004_000 + rank)
    splits = W.make_split_domains(wl, root_pre, n_domains=n_domains)
    lo = wl.lo.contiguous().pin_memory()            # [1, 784]
    up = wl.up.contiguous().pin_memory()
    C = wl.C.contiguous().pin_memory()              # [1, 9, 10]
    splits = [s.pin_memory() for s in splits]
    return lo, up, C, splits


def sweep_flops(widths, M):
    """Algorithmic flops of one backward sweep (one side) / one adjoint sweep for M coefficient rows."""
    bwd = sum(2.0 * M * widths[k] * widths[k + 1] for k in range(len(widths) - 1))
    adj = sum(2.0 * M * widths[k] * widths[k + 1] for k in range(len(widths) - 2))
    return bwd, adj


# ---------------------------------------------------------------------------------------------
# CPU arm: the reference's own functions (oracle/_ref) or, when that is absent, the oracle port
# ---------------------------------------------------------------------------------------------
class CpuArm:
    """One c4 step (`sample` subdomains) on the host cores.  kind == "reference": the reference's
    `_forward_ibp_trace_mlp(relu_split_state=)`, its backward primitive `run_crown_ibp_mlp_from_forward_trace(relu_alpha=)`
    under torch autograd and torch.optim.Adam with the per-domain best-of rule of its alpha loop
    (alpha_beta_crown.py:747-923); kind == "port": `oracle/crown_oracle.py`, the restatement of the same functions."""

    def __init__(self, sample: int):
        from boundflow_b200 import workloads as W

        torch.set_num_threads(os.cpu_count() or 1)
        self.sample = int(sample)
        self.cores = os.cpu_count() or 1
        wl = W.make_workload("c4")
        self.wl = wl
        from oracle.make_ref import ref_path

        self.kind = "port"
        p = ref_path()
        if p is not None:
            if p not in sys.path:
                sys.path.insert(0, p)
            try:
                from boundflow.ir.task import BFTaskModule, BoundTask, TaskKind, TaskOp
                from boundflow.runtime.crown_ibp import _forward_ibp_trace_mlp, run_crown_ibp_mlp_from_forward_trace
                from boundflow.runtime.task_executor import InputSpec

                self._fwd, self._bwd, self._InputSpec = _forward_ibp_trace_mlp, run_crown_ibp_mlp_from_forward_trace, InputSpec
                src = wl.module.get_entry_task()
                ops = [TaskOp(op_type=o.op_type, name=o.name, inputs=list(o.inputs), outputs=list(o.outputs), attrs=dict(o.attrs)) for o in src.ops]
                task = BoundTask(task_id="t0", kind=TaskKind.INTERVAL_IBP, ops=ops, input_values=["input"], output_values=["out"])
                self.module = BFTaskModule(tasks=[task], entry_task_id="t0", bindings={"params": dict(wl.module.bindings["params"])})
                self.kind = "reference"
            except Exception as e:  # an unusable build of oracle/_ref: say so and time the port
                sys.stderr.write(f"bench: oracle/_ref is present but not importable ({e}); timing the oracle port instead\n")
        from oracle import crown_oracle as O

        self.O = O
        root = O.forward_ibp_trace(wl.layers, O.box_input(wl.lo, wl.up))
        wl.generator = torch.Generator("cpu").manual_seed(1004_000)
        self.splits = W.make_split_domains(wl, root.pre, n_domains=self.sample)
        self.lo = wl.lo.expand(self.sample, -1).contiguous()
        self.up = wl.up.expand(self.sample, -1).contiguous()
        self.C = wl.C.expand(self.sample, -1, -1).contiguous()

    def describe(self) -> str:
        what = ("the reference's own functions (oracle/_ref: _forward_ibp_trace_mlp + Adam over run_crown_ibp_mlp_from_forward_trace)"
                if self.kind == "reference" else "oracle/crown_oracle.py, the CPU restatement of the reference's functions (oracle/_ref not built)")
        return f"{self.sample} subdomains of the same workload per step, {what}, torch CPU ops on {self.cores} threads"

    def step(self) -> float:
        """One pass; returns seconds."""
        t0 = time.perf_counter()
        if self.kind == "reference":
            self._reference_step()
        else:
            O = self.O
            inp = O.box_input(self.lo, self.up)
            trace = O.forward_ibp_trace(self.wl.layers, inp, splits=self.splits)
            a0 = O.adaptive_alpha_init(trace)
            bl, _bu, _, _ = O.alpha_crown(self.wl.layers, inp, self.C, steps=ALPHA_STEPS, lr=LR, alpha0=a0, trace=trace)
            _ = O.verdict(bl)
        return time.perf_counter() - t0

    def _reference_step(self):
        names = self.wl.relu_names
        spec = self._InputSpec.box(value_name="input", lower=self.lo, upper=self.up)
        env, pre = self._fwd(self.module, spec, relu_split_state=dict(zip(names, self.splits)))
        alphas = {}
        for n in names:  # adaptive start: 1 where l >= 0 or (l < 0 < u and u > -l)
            l, u = pre[n].lower, pre[n].upper
            alphas[n] = ((l >= 0) | ((l < 0) & (u > 0) & (u > -l))).to(l.dtype).requires_grad_(True)
        opt = torch.optim.Adam(list(alphas.values()), lr=LR)
        best_m = best_l = None
        for step in range(ALPHA_STEPS + 1):
            b = self._bwd(self.module, spec, interval_env=env, relu_pre=pre, linear_spec_C=self.C, relu_alpha=alphas)
            m = b.lower.mean(dim=1)
            if best_m is None:
                best_m, best_l = m.detach().clone(), b.lower.detach().clone()
            else:
                imp = m.detach() > best_m
                best_m = torch.where(imp, m.detach(), best_m)
                best_l = torch.where(imp[:, None], b.lower.detach(), best_l)
            if step == ALPHA_STEPS:
                break
            opt.zero_grad(set_to_none=True)
            (-m.sum()).backward()
            opt.step()
            with torch.no_grad():
                for a in alphas.values():
                    a.clamp_(0.0, 1.0)
        return best_l.min(dim=1).values >= -1e-6

    def baseline(self):
        """1 warm-up pass + median of 3 passes -> (domains/s, seconds per pass)."""
        self.step()
        ts = sorted(self.step() for _ in range(3))
        return self.sample / ts[1], ts[1]


def bench_config(D: int, world: int, scaling: str):
    n_total = D * world if scaling == "weak" else D
    return {
        "workload": WORKLOAD,
        "domains_per_gpu_per_step": D if scaling == "weak" else D // world, "domains_per_step": n_total, "alpha_steps": ALPHA_STEPS,
        "l2": "per-step working set (coefficient tensors, > 1 GB) exceeds the 126 MB L2; no explicit flush",
        "parallelism": (f"domains sharded over {world} GPU(s), weights replicated, one all-gather of bounds+verdicts per step"
                        + ("" if scaling == "weak" else "; ONE batch split over the GPUs (strong scaling)")),
    }


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    t0 = time.perf_counter()
    arm = CpuArm(REFERENCE_SAMPLE)
    warmup, steps = max(int(args.warmup), 1), max(int(args.steps), 1)
    for _ in range(warmup):
        arm.step()
    total = sum(arm.step() for _ in range(steps))
    v = arm.sample * steps / total
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": steps, "warmup": warmup,
        "ms_per_step": 1e3 * total / steps, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": bench_config(int(args.domains), max(int(args.gpus), 1), args.scaling),
        "cpu_baseline": {"value": v, "unit": UNIT, "cores": arm.cores, "kind": arm.kind, "sample": arm.describe()},
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": f"a step of this arm bounds {arm.sample} of the config's subdomains (ms_per_step is that sample's time); value = subdomains/s",
        "wall_s": time.perf_counter() - t0,
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------
# kernel timing slots -> roofline objects
# ---------------------------------------------------------------------------------------------
def read_slots(lib):
    """{slot name: {launches, ms, bytes, flops}} of everything timed since bf_kernel_timing_enable(1)."""
    out = {}
    for s in range(int(lib.bf_kernel_timing_slots())):
        n, ms, by, fl = ctypes.c_int(), ctypes.c_float(), ctypes.c_double(), ctypes.c_double()
        lib.bf_kernel_timing_read_work(s, ctypes.byref(n), ctypes.byref(ms), ctypes.byref(by), ctypes.byref(fl))
        if n.value:
            out[lib.bf_kernel_timing_slot_name(s).decode()] = {"launches": n.value, "ms": ms.value, "bytes": by.value, "flops": fl.value}
    return out


def hbm_roofline(name, rec, peaks, note=""):
    gbs = rec["bytes"] / (rec["ms"] * 1e-3) / 1e9 if rec["ms"] > 0 else None
    tf = rec["flops"] / (rec["ms"] * 1e-3) / 1e12 if rec["ms"] > 0 else None
    r = {"kernel": name, "bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"] if gbs else None,
         "launches": rec["launches"], "avg_launch_us": 1e3 * rec["ms"] / rec["launches"], "algorithmic_bytes_per_launch": rec["bytes"] / rec["launches"],
         "fp32_tflops": tf, "fp32_frac_of_ffma_peak": tf / FFMA_PEAK_TFLOPS if tf else None, "peak_source": f"{peaks['source']} STREAM-style copy"}
    if note:
        r["note"] = note
    return r


def kernel_rooflines(dev, peaks):
    """Single kernels on resident data, CUDA events around every launch (the library's timing slots), inputs larger
    than L2 or an L2 flush between launches: the HBM-bound pieces of the path at the sizes of configurations c4 and c1."""
    from boundflow_b200 import _lib

    lib = _lib.load()
    st = torch.cuda.current_stream(dev).cuda_stream
    g = torch.Generator("cpu").manual_seed(5)
    flush = torch.empty(160 * 1024 * 1024, dtype=torch.uint8, device=dev)  # > 126 MB L2
    out = {}

    def timed(fn, reps, flush_between):
        for _ in range(3):
            fn()
        torch.cuda.synchronize(dev)
        lib.bf_kernel_timing_enable(1)
        for _ in range(reps):
            if flush_between:
                flush.fill_(1)
            fn()
        torch.cuda.synchronize(dev)
        slots = read_slots(lib)
        lib.bf_kernel_timing_enable(0)
        return slots

    # concretisation of c4's final coefficient rows: 73728 rows x 784
    B, S, n0 = 8192, 9, 784
    A = torch.randn(B * S, n0, generator=g).to(dev)
    mid, rad = torch.rand(B, n0, generator=g).to(dev), torch.rand(B, n0, generator=g).to(dev) * 0.02
    res = torch.empty(B, S, device=dev)
    s = timed(lambda: _lib.check(lib.bf_concretize(A.data_ptr(), mid.data_ptr(), rad.data_ptr(), None, res.data_ptr(), _lib.SIDE_LOWER, B, S, n0, st)), 10, False)
    out["concretize_kernel_c4_73728x784"] = hbm_roofline("concretize_kernel", s["concretize_kernel"], peaks, "input 231 MB > L2, no flush needed")
    del A
    # interval Linear layer of c4 (8192 domains, 512 -> 512, ReLU on load) and of c1 (64 inputs, 784 -> 100, weights dominate)
    for tag, Bq, K, N, relu_in, fl in (("c4_8192x512x512", 8192, 512, 512, 1, False), ("c1_64x784x100", 64, 784, 100, 0, True)):
        lo = torch.randn(Bq, K, generator=g).to(dev)
        up = lo + torch.rand(Bq, K, generator=g).to(dev)
        Wt, b = torch.randn(N, K, generator=g).to(dev), torch.randn(N, generator=g).to(dev)
        ol, ou = torch.empty(Bq, N, device=dev), torch.empty(Bq, N, device=dev)
        s = timed(lambda: _lib.check(lib.bf_ibp_linear(lo.data_ptr(), up.data_ptr(), _lib.IN_LOWER_UPPER, relu_in, Wt.data_ptr(), b.data_ptr(), None, 0, None, None,
                                                       ol.data_ptr(), ou.data_ptr(), None, Bq, K, N, st)), 10, fl)
        out[f"ibp_linear_kernel_{tag}"] = hbm_roofline("ibp_linear_kernel", s["ibp_linear_kernel"], peaks,
                                                       "compute-bound at this batch (FP32 FFMA): see fp32_frac_of_ffma_peak" if Bq > 1000 else "L2 flushed between launches; 0.3 MB of weights: launch-latency bound")
    # interval Conv2d of c5's second layer (64 inputs, 32x32x32 -> 32x16x16, k4 s2 p1) and c2's first at 256 inputs
    for tag, Bq, Ci, Hi, Co, k, stv, pd in (("c5conv2_64in", 64, 32, 32, 32, 4, 2, 1), ("c2conv1_256in", 256, 1, 28, 16, 4, 2, 1)):
        Ho = (Hi + 2 * pd - k) // stv + 1
        lo = torch.rand(Bq, Ci * Hi * Hi, generator=g).to(dev)
        up = lo + 0.01
        Wc, bc = torch.randn(Co, Ci, k, k, generator=g).to(dev), torch.randn(Co, generator=g).to(dev)
        ol, ou = torch.empty(Bq, Co * Ho * Ho, device=dev), torch.empty(Bq, Co * Ho * Ho, device=dev)
        s = timed(lambda: _lib.check(lib.bf_ibp_conv2d(lo.data_ptr(), up.data_ptr(), _lib.IN_LOWER_UPPER, 0, Wc.data_ptr(), bc.data_ptr(), None, 0, None, None,
                                                       ol.data_ptr(), ou.data_ptr(), None, Bq, Ci, Hi, Hi, Co, k, k, stv, stv, pd, pd, st)), 10, True)
        out[f"ibp_conv2d_kernel_{tag}"] = hbm_roofline("ibp_conv2d_kernel", s["ibp_conv2d_kernel"], peaks, "L2 flushed between launches")
    return out


CONV_LAYERS = {  # name: (Co, Ho, Wo, Ci, Hi, Wi, kernel, stride, padding) of the forward layer whose transpose is applied
    "c5conv2T": (32, 16, 16, 32, 32, 32, 4, 2, 1), "c5conv3T": (64, 16, 16, 32, 16, 16, 3, 1, 1), "c5conv4T": (64, 8, 8, 64, 16, 16, 4, 2, 1),
    "c5conv1T": (32, 32, 32, 3, 32, 32, 3, 1, 1), "c2conv2T": (32, 7, 7, 16, 14, 14, 4, 2, 1), "c2conv1T": (16, 14, 14, 1, 28, 28, 4, 2, 1),
}


def linear_layer_bench(dev, shape, reps):
    """Times the layer-level ReLU backward + Linear backward entry point (`bf_crown_relu_linear_bwd_packed`) on one
    synthetic layer `domains,specs,n_cur,n_prev`; the environment switches (BF_B200_BWD_PERSISTENT, BF_B200_BWD_PAIRS,
    BF_B200_FORCE_FFMA, BF_B200_TC_MIN_ROWS) select the kernel.  Result checked against a torch expression."""
    from boundflow_b200 import _lib

    B, S, K, N = (int(x) for x in shape.split(","))
    lib = _lib.load()
    g = torch.Generator().manual_seed(1)
    A = torch.randn(B, S, K, generator=g).to(dev)
    au, al, bu = (torch.rand(B, K, generator=g).to(dev) for _ in range(3))
    Wt = (torch.randn(K, N, generator=g) * 0.05).to(dev)
    bias = torch.randn(K, generator=g).to(dev)
    out, delta = torch.empty(B, S, N, device=dev), torch.empty(B, S, device=dev)
    st = torch.cuda.current_stream().cuda_stream
    nb = int(lib.bf_linear_pack_bytes(K, N))
    pack = torch.empty(nb, dtype=torch.uint8, device=dev)
    _lib.check(lib.bf_linear_pack(Wt.data_ptr(), K, N, pack.data_ptr(), nb, st))

    def call():
        _lib.check(lib.bf_crown_relu_linear_bwd_packed(A.data_ptr(), 0, au.data_ptr(), al.data_ptr(), bu.data_ptr(), None, None, Wt.data_ptr(),
                                                       bias.data_ptr(), pack.data_ptr(), out.data_ptr(), delta.data_ptr(), 0, B, S, K, N, st))

    for _ in range(3):
        call()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        call()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / reps
    ref = torch.where(A >= 0, A * al[:, None, :], A * au[:, None, :]) @ Wt
    return {"shape": [B, S, K, N], "rows": B * S, "us_per_launch": ms * 1e3, "tflops_fp32_equivalent": 2.0 * B * S * K * N / ms / 1e9,
            "max_abs_err_vs_torch": float((out - ref).abs().max()), "tc_launches": int(_lib.tc_launch_count())}


def conv_layer_bench(dev, names, rows, reps):
    """One `bf_crown_relu_conv2d_bwd` call per layer shape (ReLU scaling pass + transposed convolution, one side),
    CUDA events, multiply-accumulates per second."""
    from boundflow_b200 import _lib

    lib = _lib.load()
    out = {}
    for name in names:
        Co, Ho, Wo, Ci, Hi, Wi, k, stv, pd = CONV_LAYERS[name]
        S = 8
        B = max(1, rows // S)
        M = B * S
        g = torch.Generator("cpu").manual_seed(7)
        n = Co * Ho * Wo
        A = torch.randn(B, S, n, generator=g).to(dev)
        au, al, bu = (torch.rand(B, n, generator=g).to(dev) for _ in range(3))
        bl = torch.zeros(B, n, device=dev)
        Wc = torch.randn(Co, Ci, k, k, generator=g).to(dev)
        bias = torch.randn(Co, generator=g).to(dev)
        res = torch.empty(B, S, Ci * Hi * Wi, device=dev)
        delta = torch.empty(B, S, device=dev)
        nbytes = int(lib.bf_crown_relu_conv2d_bwd_scratch_bytes(B, S, Co, Ho, Wo))
        scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        st = torch.cuda.current_stream(dev).cuda_stream

        def run():
            _lib.check(lib.bf_crown_relu_conv2d_bwd(
                A.data_ptr(), _lib.SIDE_LOWER, au.data_ptr(), al.data_ptr(), bu.data_ptr(), bl.data_ptr(), Wc.data_ptr(), bias.data_ptr(),
                res.data_ptr(), delta.data_ptr(), 0, scratch.data_ptr(), nbytes, B, S, Ci, Hi, Wi, Co, Ho, Wo, k, k, stv, stv, pd, pd, st))

        for _ in range(3):
            run()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            run()
        e1.record()
        torch.cuda.synchronize(dev)
        ms = e0.elapsed_time(e1) / reps
        out[name] = {"rows": M, "ms": ms, "tmac_per_s": M * n * Ci * k * k / ms / 1e9}
    return out


def crown_bounds_secondary(world: int, rank: int, dev, only=None, with_slots=False):
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
                res = run_crown_intermediate_mlp(wl.module, spec, linear_spec_C=C, chunk_rows=2048)[0].lower
            elif name == "c5":
                # about 32768 coefficient rows per sweep (20 GB of coefficient buffers): the sweeps of one layer's identity rows are
                # independent, so larger chunks only make fewer, larger launches - same bounds bit for bit, 339 -> 284 ms at 64 inputs
                # against 4096 rows per sweep
                res = run_crown_intermediate_mlp(wl.module, spec, linear_spec_C=C, chunk_rows=max(64, 32768 // max(1, b - a)))[0].lower
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
        if with_slots:
            lib.bf_kernel_timing_enable(1)
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
        if with_slots:
            out[name]["kernels"] = read_slots(lib)
            lib.bf_kernel_timing_enable(0)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="weak: every GPU bounds its own batch of --domains subdomains; strong: ONE batch of --domains is split over the GPUs")
    ap.add_argument("--domains", type=int, default=DOMAINS_PER_GPU, help="subdomains per GPU per step (weak) or per step in all (strong)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true", help="skip the CROWN bounds/s configurations and the single-kernel rooflines")
    ap.add_argument("--secondary-only", default=None, choices=["c1", "c2", "c3", "c5"],
                    help="time only this CROWN bounds/s configuration and print its figures with per-kernel times (profiling aid)")
    ap.add_argument("--kernels", action="store_true", help="time single kernels on resident data and print their rooflines (profiling aid)")
    ap.add_argument("--conv-layers", default=None, help="comma-separated layer names: time the fused ReLU + transposed-convolution call (profiling aid)")
    ap.add_argument("--linear-layer", default=None, help="domains,specs,n_cur,n_prev: time the ReLU + Linear backward entry point on one layer (profiling aid)")
    ap.add_argument("--rows", type=int, default=2048, help="coefficient rows for --conv-layers")
    ap.add_argument("--reps", type=int, default=10, help="repetitions for --conv-layers")
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
        # the one collective of a step gathers a few hundred KB: it gains nothing from in-switch multicast buffers, and
        # without them a rank that ends does not touch its peers' mappings
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)

    from boundflow_b200.csrc import build as _build

    _build.build()
    from boundflow_b200 import _lib
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import bound_split_domains, ibp_trace
    from boundflow_b200.dist import gather_domain_results, shard_range
    from boundflow_b200.ir import InputSpec

    lib = _lib.load()
    peaks = measured_peaks()
    if args.secondary_only:
        sec = crown_bounds_secondary(world, rank, dev, only=args.secondary_only, with_slots=True)
        if rank == 0:
            print(json.dumps({"crown_bounds_per_s": sec, "n_gpus": world}))
        if world > 1:
            dist.destroy_process_group()
        return
    if args.kernels:
        print(json.dumps({"kernel_rooflines": kernel_rooflines(dev, peaks)}))
        return
    if args.conv_layers:
        print(json.dumps({"conv_layers": conv_layer_bench(dev, args.conv_layers.split(","), args.rows, args.reps)}))
        return
    if args.linear_layer:
        print(json.dumps({"linear_layer": linear_layer_bench(dev, args.linear_layer, args.reps)}))
        return
    warmup = max(int(args.warmup), 3)
    strong = args.scaling == "strong"
    n_total = int(args.domains) * (1 if strong else world)
    a_lo, a_hi = shard_range(n_total, rank, world)
    D = a_hi - a_lo  # subdomains bounded by this rank per step
    wl = W.make_workload("c4")
    names = wl.relu_names
    root = ibp_trace(wl.module, InputSpec.box(value_name="input", lower=wl.lo.to(dev), upper=wl.up.to(dev)))
    root_pre = [(l.cpu(), u.cpu()) for l, u in zip(root.pre_l, root.pre_u)]
    h_lo, h_up, h_C, h_splits = build_host_batch(wl, root_pre, D, rank)
    d_lo, d_up, d_C = h_lo.to(dev).expand(D, -1).contiguous(), h_up.to(dev).expand(D, -1).contiguous(), h_C.to(dev).expand(D, -1, -1).contiguous()
    d_splits = {n: s.to(dev) for n, s in zip(names, h_splits)}
    d_spec = InputSpec.box(value_name="input", lower=d_lo, upper=d_up)

    def step_resident():
        res = bound_split_domains(wl.module, d_spec, linear_spec_C=d_C, relu_split_state=d_splits, steps=ALPHA_STEPS, lr=LR)
        lower, verdict = gather_domain_results(res.lower, res.verdict, n_total) if world > 1 else (res.lower, res.verdict)
        return lower, verdict, res

    def step_e2e():
        # the public call fed from pinned host memory: box [1,784] x2, specs [1,9,10], one int8 split row per subdomain and layer
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
    launches0, tc0 = _lib.launch_count(), _lib.tc_launch_count()
    ms_res, out = timed(step_resident, args.steps)
    launches, tc_launches = _lib.launch_count() - launches0, _lib.tc_launch_count() - tc0
    slots = read_slots(lib)
    lib.bf_kernel_timing_enable(0)

    for _ in range(2):
        step_e2e()
    ms_e2e, out_e2e = timed(step_e2e, args.steps)
    clocks = sampler.stop() if rank == 0 else None  # sampled over both timed regions (resident and end-to-end)
    tc_status = wl_status = None
    from boundflow_b200.network import compile_chain

    tc_status = compile_chain(wl.module, (784,), dev).tc_status()

    secondary = None if args.no_secondary else crown_bounds_secondary(world, rank, dev)
    if world > 1:
        # every rank leaves the process group TOGETHER, before rank 0 goes on alone with the single-kernel timings, so
        # that no rank runs kernels while a peer tears its communicator down
        torch.cuda.synchronize(dev)
        dist.barrier()
        dist.destroy_process_group()
    kernels = None if (args.no_secondary or rank != 0) else kernel_rooflines(dev, peaks)

    if rank != 0:
        return

    lower, verdict, res = out
    infeasible = int(res.infeasible.sum().item())
    proven = int(verdict.sum().item())
    if tc_status != 0:
        raise SystemExit("bench: a bounded wait expired inside a tensor-core kernel (status word set): results are invalid")
    feasible_rows = lower[: res.infeasible.shape[0]][res.infeasible == 0]
    if not bool(torch.isfinite(feasible_rows).all()):
        raise SystemExit("bench: non-finite lower bound on a feasible subdomain")
    widths = [784, 512, 512, 512, 512, 10]
    bwd = slots.get("crown_bwd_contraction", {"launches": 0, "ms": 0.0, "bytes": 0.0, "flops": 0.0})
    adj = slots.get("crown_adjoint_contraction", {"launches": 0, "ms": 0.0, "bytes": 0.0, "flops": 0.0})
    fp32_equiv_peak = peaks["bf16_sustained"] / 6.0  # TF32 runs at half the bf16 rate; 3 TF32 MMAs per fp32-faithful product
    achieved = bwd["flops"] / (bwd["ms"] * 1e-3) / 1e12 if bwd["ms"] > 0 else None
    achieved_adj = adj["flops"] / (adj["ms"] * 1e-3) / 1e12 if adj["ms"] > 0 else None
    value = n_total * args.steps / (ms_res * 1e-3)
    e2e_value = n_total * args.steps / (ms_e2e * 1e-3)
    h2d = h_lo.numel() * 4 * 2 + h_C.numel() * 4 + sum(s.numel() for s in h_splits)
    d2h = n_total * 9 * 4 + n_total + D * 4
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warmup,
        "ms_per_step": ms_res / args.steps, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": bench_config(int(args.domains), world, args.scaling),
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h), "ms_per_step": ms_e2e / args.steps,
                "note": "input box [1,784] x2 and spec rows [1,9,10] travel once per step and are repeated on the device; one int8 split row per subdomain and ReLU layer"},
        "gpu_launches": int(launches), "gpu_tensor_core_launches": int(tc_launches),
        "clocks": clocks,
        "roofline": {
            "bound": "tensor", "kernel": "crown_tc_kernel<bwd> (ReLU-backward + Linear-backward contraction, tcgen05 3xTF32)",
            "achieved": achieved, "peak": fp32_equiv_peak, "unit": "TFLOP/s", "frac": (achieved / fp32_equiv_peak) if achieved else None,
            "traffic": TRAFFIC_BYTES_PER_LAUNCH * (D / 8192.0),
            "traffic_source": "ncu dram__bytes_read+write of one 512x512-layer launch at 4096 domains, scaled by rows (profiles/)",
            "peak_source": f"{peaks['source']} bf16 sustained {peaks['bf16_sustained']} TFLOP/s / 6 = fp32-equivalent 3xTF32 tensor peak",
            "launches": bwd["launches"], "avg_launch_ms": (bwd["ms"] / bwd["launches"]) if bwd["launches"] else None,
            "algorithmic_flops_per_launch": (bwd["flops"] / bwd["launches"]) if bwd["launches"] else None,
            "share_of_step": bwd["ms"] / ms_res if ms_res else None,
        },
        "roofline_adjoint": {
            "kernel": "crown_tc_adjoint_kernel (gradient sweep, feature-major tcgen05 3xTF32)", "achieved": achieved_adj, "unit": "TFLOP/s",
            "frac": (achieved_adj / fp32_equiv_peak) if achieved_adj else None, "launches": adj["launches"],
            "share_of_step": adj["ms"] / ms_res if ms_res else None,
        },
        # HBM-bound kernels: inside the timed c4 step (live event pairs), and single kernels at the configurations' sizes
        "roofline_hbm": {
            "in_step": {n: hbm_roofline(n, slots[n], peaks) for n in ("crown_bwd_thin_kernel", "adam_step_kernel", "ibp_linear_kernel") if n in slots},
            "single_kernels": kernels,
        },
        "kernel_share_of_step": {n: r["ms"] / ms_res for n, r in slots.items()},
        "crown_bounds_per_s": secondary,
        "result_check": {"domains": n_total, "proven": proven, "infeasible_local": infeasible, "tc_status": tc_status,
                         "mean_lower": float(lower[torch.isfinite(lower).all(dim=1)].mean().item())},
    }
    if not args.no_cpu_baseline and world == 1:
        arm = CpuArm(REFERENCE_SAMPLE)
        v, t = arm.baseline()
        line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": arm.cores, "kind": arm.kind,
                                "sample": arm.describe() + f"; 1 warm-up pass, median of 3 ({t:.2f} s per pass)"}
    print(json.dumps(line))


if __name__ == "__main__":
    main()
