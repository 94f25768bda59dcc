"""Parity of the headline path (configuration c4 on the tcgen05 kernels, and c3) pinned three ways:

1. golden outputs of the reference at 32 split subdomains (288 coefficient rows, i.e. on the tensor-core
   kernels -- the launch counter is checked);
2. a float64 evaluation of the same bounds at the alpha the CUDA loop returned ("truth"): the tcgen05 path, the
   FP32 FFMA path and the fp32 oracle are all measured against it;
3. the trajectory of the Adam loop after 1, 2, 5, 10 (20) steps against the reference's own float32 trajectory,
   with the reference's float32-vs-float64 distance stored beside it (tests/golden/adam_divergence.npz).

Tolerance everywhere: |got - ref| <= 1e-4 + 1e-5 |ref| unless a test states and measures otherwise.
"""
import os

import numpy as np
import pytest
import torch

from tests.helpers import ATOL, RTOL, assert_close

pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("tc_from_256_rows")]


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available()
    from boundflow_b200.csrc import build

    build.build()
    return torch.device("cuda", 0)


class _ForceFFMA:
    def __enter__(self):
        os.environ["BF_B200_FORCE_FFMA"] = "1"

    def __exit__(self, *exc):
        os.environ.pop("BF_B200_FORCE_FFMA", None)


def _c4(D, dev):
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import ibp_trace
    from boundflow_b200.ir import InputSpec
    from oracle import crown_oracle as O

    wl = W.make_workload("c4")
    root = O.forward_ibp_trace(wl.layers, O.box_input(wl.lo, wl.up))
    splits = W.make_split_domains(wl, root.pre, n_domains=D)
    lo, up = wl.lo.expand(D, -1).contiguous(), wl.up.expand(D, -1).contiguous()
    spec = InputSpec.box(value_name="input", lower=lo.to(dev), upper=up.to(dev))
    C = wl.C.expand(D, -1, -1).contiguous()
    trace = ibp_trace(wl.module, spec, relu_split_state={n: s.to(dev) for n, s in zip(wl.relu_names, splits)})
    return wl, splits, lo, up, C, trace


def _strict_excess(got, ref):
    """max over elements of |got - ref| / (1e-4 + 1e-5 |ref|): <= 1 means inside the strict tolerance."""
    got = torch.as_tensor(np.asarray(got.detach().cpu() if torch.is_tensor(got) else got), dtype=torch.float64)
    ref = torch.as_tensor(np.asarray(ref.detach().cpu() if torch.is_tensor(ref) else ref), dtype=torch.float64)
    return float(((got - ref).abs() / (ATOL + RTOL * ref.abs())).max())


def test_c4_golden_runs_on_tensor_cores(dev, golden):
    """The reference's c4 outputs (32 subdomains) reproduced with every contraction on the tcgen05 kernels."""
    from boundflow_b200 import _lib
    from boundflow_b200.crown import adaptive_alpha_from_trace, alpha_crown_from_trace, crown_from_trace

    g = golden("c4_split_alpha.npz")
    wl, splits, lo, up, C, trace = _c4(32, dev)
    assert int(trace.infeasible.sum()) == 0
    a0 = adaptive_alpha_from_trace(trace)
    tc0 = _lib.tc_launch_count()
    lo0, up0 = crown_from_trace(trace, C.to(dev), relu_alpha=dict(zip(wl.relu_names, a0)))
    n_eval = _lib.tc_launch_count() - tc0
    assert n_eval >= 8, f"one lower and one upper sweep over 4 wide layers must launch 8 tcgen05 contractions, saw {n_eval}"
    assert_close(lo0, g["step0_lower"], "step-0 lower on tensor cores")
    assert_close(up0, g["step0_upper"], "step-0 upper on tensor cores")
    tc1 = _lib.tc_launch_count()
    best_l, best_u, best_a, _, _ = alpha_crown_from_trace(trace, C.to(dev), a0, steps=10, lr=0.1)
    torch.cuda.synchronize()
    assert trace.chain.tc_status() == 0
    # 11 lower sweeps + 1 upper sweep (4 contractions each) + 10 gradient sweeps (4 each)
    assert _lib.tc_launch_count() - tc1 == 12 * 4 + 10 * 4
    # optimised bounds: see test_adam_trajectory_c4 for the step-by-step measurement behind this band
    ex_l, ex_u = _strict_excess(best_l, g["best_lower"]), _strict_excess(best_u, g["best_upper"])
    print(f"c4 golden, 10 steps on tensor cores: |err| / strict tolerance = {ex_l:.2f} (lower), {ex_u:.2f} (upper)")
    assert ex_l <= 3.0 and ex_u <= 3.0
    got_m, ref_m = best_l.mean(dim=1).cpu(), torch.as_tensor(g["best_lower"]).mean(dim=1)
    assert_close(got_m, ref_m, "per-domain objective after 10 steps")
    with _ForceFFMA():
        ffma_l, ffma_u, _, _, _ = alpha_crown_from_trace(trace, C.to(dev), a0, steps=10, lr=0.1)
    assert_close(ffma_l, g["best_lower"], "FFMA path, 10 steps, lower")
    assert_close(ffma_u, g["best_upper"], "FFMA path, 10 steps, upper")


@pytest.mark.parametrize("cfg", ["c4", "c3"])
def test_adam_trajectory_against_reference(dev, golden, cfg):
    """Best-of bounds after k Adam steps against the reference's float32 run of the same k.

    Measured on B200 (printed below): the FFMA path and the c3 runs stay within 5e-7 relative of the reference's
    trajectory for every k, as close as the reference's own float32 and float64 runs are to each other (3e-7, stored
    in the fixture).  The tcgen05 path (3xTF32: operands carry 22 significant bits and the tensor core's accumulation
    truncates, about four times the rounding noise of FP32 FFMA) matches to 5e-7 for k <= 2 and then drifts -- Adam turns
    a gradient entry whose sign differs at rounding level into a full +-lr move -- to 1.4e-6 at k = 5 and 1.4e-5 at
    k = 10 on c4.  Bands asserted: the strict tolerance wherever it was measured to hold; for the tcgen05 path at
    k >= 10 three times the strict band on single elements AND the strict tolerance on the per-domain objective.
    No best-of tie is involved: the reference's best and second-best iteration differ by >= 4.6e-5 relative
    (`*_hist_lower` in the fixture), far above these distances."""
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import AlphaState, adaptive_alpha_from_trace, alpha_crown_from_trace, ibp_trace, run_alpha_beta_crown_mlp
    from boundflow_b200.ir import InputSpec

    d = golden("adam_divergence.npz")
    if cfg == "c4":
        wl, splits, lo, up, C, trace = _c4(32, dev)
        a0 = adaptive_alpha_from_trace(trace)
        ks = (1, 2, 5, 10)

        def run(k):
            return alpha_crown_from_trace(trace, C.to(dev), a0, steps=k, lr=0.1)[0]
    else:
        wl = W.make_workload("c3", batch=8)
        spec = InputSpec.box(value_name="input", lower=wl.lo.to(dev), upper=wl.up.to(dev))
        trace = ibp_trace(wl.module, spec)
        a0 = adaptive_alpha_from_trace(trace)
        ks = (1, 2, 5, 10, 20)

        def run(k):
            return run_alpha_beta_crown_mlp(wl.module, spec, linear_spec_C=wl.C.to(dev), steps=k, lr=0.1, per_batch_params=True,
                                            warm_start_alpha=AlphaState(dict(zip(wl.relu_names, a0))))[0].lower

    # the reference's best-of is unambiguous in these runs
    hist = d[f"{cfg}_hist_lower"].astype(np.float64)
    m = np.sort(hist.mean(axis=2), axis=0)[::-1]
    assert float(((m[0] - m[1]) / np.abs(m[0])).min()) > 2e-5
    for path in ("tensor", "ffma"):
        for k in ks:
            if path == "ffma":
                with _ForceFFMA():
                    got = run(k)
            else:
                got = run(k)
            ref32, ref64 = d[f"{cfg}_f32_lower_{k}"], d[f"{cfg}_f64_lower_{k}"]
            ex = _strict_excess(got, ref32)
            ref_ex = _strict_excess(ref32, ref64)
            print(f"{cfg} {path} k={k}: |err| / strict tolerance = {ex:.3f} (reference float32 vs float64: {ref_ex:.3f})")
            band = 3.0 if (path == "tensor" and k >= 10) else 1.0
            assert ex <= band, f"{cfg} {path} after {k} steps: {ex:.2f} x the strict tolerance"
            assert_close(got.mean(dim=1), torch.as_tensor(ref32).mean(dim=1), f"{cfg} {path} objective after {k} steps")


def _truth_errors(name, wl, lo, up, C, splits, sel, got_l, got_u, alpha_sel):
    """Errors of `got` against the float64 oracle at `alpha_sel`, and the fp32 oracle's own errors against it."""
    from oracle import crown_oracle as O

    layers64 = O.layers_to(wl.layers, torch.float64)
    sp = None if splits is None else [s[sel] for s in splits]
    out = {}
    for tag, layers, dt in (("f64", layers64, torch.float64), ("f32", wl.layers, torch.float32)):
        inp = O.box_input(lo[sel].to(dt), up[sel].to(dt))
        tr = O.forward_ibp_trace(layers, inp, splits=sp)
        l, u = O.crown_backward(layers, inp, tr, C[sel].to(dt), alpha=[a.to(dt) for a in alpha_sel])
        out[tag] = (l, u)
    t_l, t_u = out["f64"]
    res = {"oracle_f32": max(_strict_excess(out["f32"][0], t_l), _strict_excess(out["f32"][1], t_u)),
           "got": max(_strict_excess(got_l, t_l), _strict_excess(got_u, t_u))}
    rel = float(((got_l.double().cpu() - t_l).abs() / t_l.abs()).max())
    print(f"{name}: |err| / strict tolerance vs float64 truth: CUDA {res['got']:.3f}, fp32 oracle {res['oracle_f32']:.3f}; CUDA max rel err {rel:.2e}")
    return res


@pytest.mark.parametrize("path", ["tensor", "ffma"])
def test_float64_truth_c4_full_batch(dev, path):
    """8192 subdomains, 10 Adam steps; 256 of them re-evaluated in float64 at the returned alpha.  Done = the CUDA
    result is inside the strict tolerance of the float64 value, or no further from it than twice the fp32 oracle."""
    from boundflow_b200.crown import adaptive_alpha_from_trace, alpha_crown_from_trace

    D = 8192
    wl, splits, lo, up, C, trace = _c4_fast(D, dev)
    feasible = (trace.infeasible == 0).cpu()
    a0 = adaptive_alpha_from_trace(trace)
    ctx = _ForceFFMA() if path == "ffma" else None
    if ctx:
        ctx.__enter__()
    try:
        best_l, best_u, best_a, _, _ = alpha_crown_from_trace(trace, C.to(dev), a0, steps=10, lr=0.1)
        torch.cuda.synchronize()
    finally:
        if ctx:
            ctx.__exit__()
    assert trace.chain.tc_status() == 0
    sel = torch.nonzero(feasible).flatten()[:: max(1, int(feasible.sum()) // 256)][:256]
    res = _truth_errors(f"c4 {path}", wl, lo, up, C, splits, sel, best_l[sel.to(dev)], best_u[sel.to(dev)], [a[sel.to(dev)].cpu() for a in best_a])
    assert res["got"] <= 1.0 or res["got"] <= 2.0 * res["oracle_f32"]


def _c4_fast(D, dev):
    """Full-size batch with a vectorised split draw (10 unstable neurons per domain: 3, 3, 2, 2 per layer)."""
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import ibp_trace
    from boundflow_b200.ir import InputSpec
    from oracle import crown_oracle as O

    wl = W.make_workload("c4")
    root = O.forward_ibp_trace(wl.layers, O.box_input(wl.lo, wl.up))
    g = torch.Generator("cpu").manual_seed(4)
    splits = []
    for r, (l, u) in enumerate(root.pre):
        idx = torch.nonzero(((l < 0) & (u > 0)).reshape(-1)).flatten()
        s = torch.zeros(D, l.shape[1], dtype=torch.int8)
        k = 3 if r < 2 else 2
        pick = idx[torch.randint(0, len(idx), (D, k), generator=g)]
        sign = (torch.randint(0, 2, (D, k), generator=g) * 2 - 1).to(torch.int8)
        s.scatter_(1, pick, sign)
        splits.append(s)
    lo, up = wl.lo.expand(D, -1).contiguous(), wl.up.expand(D, -1).contiguous()
    spec = InputSpec.box(value_name="input", lower=lo.to(dev), upper=up.to(dev))
    C = wl.C.expand(D, -1, -1).contiguous()
    trace = ibp_trace(wl.module, spec, relu_split_state={n: s.to(dev) for n, s in zip(wl.relu_names, splits)})
    return wl, splits, lo, up, C, trace


@pytest.mark.parametrize("path", ["tensor", "ffma"])
def test_float64_truth_c3(dev, path):
    """c3 (128 inputs, 20 Adam steps): 32 inputs re-evaluated in float64 at the returned alpha."""
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import AlphaState, adaptive_alpha_from_trace, ibp_trace, run_alpha_beta_crown_mlp
    from boundflow_b200.ir import InputSpec

    wl = W.make_workload("c3")
    spec = InputSpec.box(value_name="input", lower=wl.lo.to(dev), upper=wl.up.to(dev))
    trace = ibp_trace(wl.module, spec)
    a0 = adaptive_alpha_from_trace(trace)
    ctx = _ForceFFMA() if path == "ffma" else None
    if ctx:
        ctx.__enter__()
    try:
        bounds, a_state, _b, _s = run_alpha_beta_crown_mlp(wl.module, spec, linear_spec_C=wl.C.to(dev), steps=20, lr=0.1, per_batch_params=True,
                                                         warm_start_alpha=AlphaState(dict(zip(wl.relu_names, a0))))
        torch.cuda.synchronize()
    finally:
        if ctx:
            ctx.__exit__()
    sel = torch.arange(0, 128, 4)
    alpha_sel = [a_state.alpha_by_relu_input[n][sel.to(dev)].cpu() for n in wl.relu_names]
    res = _truth_errors(f"c3 {path}", wl, wl.lo, wl.up, wl.C, None, sel, bounds.lower[sel.to(dev)], bounds.upper[sel.to(dev)], alpha_sel)
    assert res["got"] <= 1.0 or res["got"] <= 2.0 * res["oracle_f32"]
