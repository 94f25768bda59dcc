"""The upper, gap and both objectives of the per-domain alpha loop on the GPU, against the reference's
`run_alpha_beta_crown_mlp(objective=...)` outputs (tests/golden/objectives.npz, lb_weight 1.0, ub_weight 0.5)."""
import pytest
import torch

from tests.helpers import assert_close

pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("tc_from_256_rows")]

CASES = (("upper", "mean"), ("gap", "mean"), ("both", "mean"), ("upper", "min"), ("gap", "min"), ("both", "softmin"), ("gap", "softmin"))


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available()
    from boundflow_b200.csrc import build

    build.build()
    return torch.device("cuda", 0)


@pytest.mark.parametrize("cfg", ["c1", "c3"])
@pytest.mark.parametrize("objective,reduce", CASES)
def test_matches_reference_golden(dev, golden, cfg, objective, reduce):
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import AlphaState, adaptive_alpha_from_trace, ibp_trace, run_alpha_beta_crown_mlp
    from boundflow_b200.ir import InputSpec

    g = golden("objectives.npz")
    wl = W.make_workload(cfg, batch=8)
    spec = InputSpec.box(value_name="input", lower=wl.lo.to(dev), upper=wl.up.to(dev))
    a0 = adaptive_alpha_from_trace(ibp_trace(wl.module, spec))
    for k in (1, 3, 10):
        b, _a, _b, stats = run_alpha_beta_crown_mlp(wl.module, spec, linear_spec_C=wl.C.to(dev), steps=k, lr=0.1, per_batch_params=True,
                                                   warm_start_alpha=AlphaState(dict(zip(wl.relu_names, a0))), objective=objective,
                                                   spec_reduce=reduce, soft_tau=float(g[f"{cfg}_tau"]), lb_weight=1.0, ub_weight=0.5)
        assert stats.objective == objective
        assert_close(b.lower, g[f"{cfg}_{objective}_{reduce}_lower_{k}"], f"{cfg} {objective}/{reduce} lower after {k} steps")
        assert_close(b.upper, g[f"{cfg}_{objective}_{reduce}_upper_{k}"], f"{cfg} {objective}/{reduce} upper after {k} steps")


def test_tensor_core_rows_split_domains_and_argument_errors(dev):
    """c3 at 32 inputs (288 / 576 coefficient rows: tcgen05 kernels) against the oracle, with a split assignment
    present (the beta term stays out of these objectives and the start beta comes back); bad arguments raise."""
    from boundflow_b200 import _lib
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import adaptive_alpha_from_trace, alpha_crown_from_trace, ibp_trace
    from boundflow_b200.ir import InputSpec
    from oracle import crown_oracle as O

    wl = W.make_workload("c3", batch=32)
    spec = InputSpec.box(value_name="input", lower=wl.lo.to(dev), upper=wl.up.to(dev))
    inp = O.box_input(wl.lo, wl.up)
    root = O.forward_ibp_trace(wl.layers, inp)
    g = torch.Generator("cpu").manual_seed(5)
    splits = []
    for l, u in root.pre:
        s8 = torch.zeros(l.shape, dtype=torch.int8)
        for b in range(l.shape[0]):
            idx = torch.nonzero((l[b] < 0) & (u[b] > 0)).flatten()
            pick = idx[torch.randint(0, len(idx), (2,), generator=g)]
            s8[b, pick] = (torch.randint(0, 2, (2,), generator=g) * 2 - 1).to(torch.int8)
        splits.append(s8)
    trace = ibp_trace(wl.module, spec, relu_split_state={n: s.to(dev) for n, s in zip(wl.relu_names, splits)})
    keep = torch.nonzero((trace.infeasible == 0).cpu()).flatten()
    assert len(keep) >= 16
    a0 = adaptive_alpha_from_trace(trace)
    tr = O.forward_ibp_trace(wl.layers, inp, splits=splits)
    for obj, red, tau in (("upper", "mean", 1.0), ("gap", "softmin", 80.0), ("both", "min", 1.0)):
        t0 = _lib.tc_launch_count()
        got = alpha_crown_from_trace(trace, wl.C.to(dev), a0, steps=3, lr=0.1, spec_reduce=red, soft_tau=tau, objective=obj, lb_weight=0.7,
                                     ub_weight=1.3, beta_splits=[s.to(dev) for s in splits])
        assert _lib.tc_launch_count() > t0
        assert len(got) == 6 and all(float(b.abs().max()) == 0.0 for b in got[5])
        ref_l, ref_u, _a, _t = O.alpha_crown(wl.layers, inp, wl.C, steps=3, lr=0.1, alpha0=[a.cpu() for a in a0], trace=tr, spec_reduce=red,
                                             soft_tau=tau, objective=obj, lb_weight=0.7, ub_weight=1.3, splits=splits)
        assert_close(got[0][keep.to(dev)], ref_l[keep], f"{obj}/{red} lower, 3 steps")
        assert_close(got[1][keep.to(dev)], ref_u[keep], f"{obj}/{red} upper, 3 steps")
    with pytest.raises(ValueError):
        alpha_crown_from_trace(trace, wl.C.to(dev), a0, steps=1, lr=0.1, objective="tightest")
    with pytest.raises(ValueError):
        alpha_crown_from_trace(trace, wl.C.to(dev), a0, steps=1, lr=0.1, objective="gap", spec_reduce="sum")
    with pytest.raises(NotImplementedError):
        alpha_crown_from_trace(trace, wl.C.to(dev), a0, steps=1, lr=0.1, objective="both", ub_weight=-1.0)


SHARED_CASES = (("lower", "min"), ("lower", "softmin"), ("upper", "mean"), ("gap", "min"), ("both", "softmin"), ("both", "mean"))


@pytest.mark.parametrize("cfg,batch", [("c1", 8), ("c2", 4)])
def test_shared_alpha_objectives_match_reference_golden(dev, golden, cfg, batch):
    """The shared-alpha loop (`run_alpha_crown_mlp`) with the objectives and reductions beyond lower / mean, on an
    MLP and on a CNN, against tests/golden/shared_objectives.npz (lb_weight 1.0, ub_weight 0.5)."""
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import run_alpha_beta_crown_mlp, run_alpha_crown_mlp
    from boundflow_b200.ir import InputSpec

    g = golden("shared_objectives.npz")
    wl = W.make_workload(cfg, batch=batch)
    spec = InputSpec.box(value_name="input", lower=wl.lo.to(dev), upper=wl.up.to(dev))
    for obj, red in SHARED_CASES:
        for k in (1, 6):
            b, st, stats = run_alpha_crown_mlp(wl.module, spec, linear_spec_C=wl.C.to(dev), steps=k, lr=0.1, objective=obj, spec_reduce=red,
                                               soft_tau=float(g[f"{cfg}_tau"]), lb_weight=1.0, ub_weight=0.5)
            assert stats.objective == obj and stats.spec_reduce == red
            assert_close(b.lower, g[f"{cfg}_{obj}_{red}_lower_{k}"], f"{cfg} shared {obj}/{red} lower after {k}")
            assert_close(b.upper, g[f"{cfg}_{obj}_{red}_upper_{k}"], f"{cfg} shared {obj}/{red} upper after {k}")
    # the alpha-beta function in its shared mode takes the same route (alpha start 0.5 in both functions)
    b, _a, _bt, _s = run_alpha_beta_crown_mlp(wl.module, spec, linear_spec_C=wl.C.to(dev), steps=6, lr=0.1, per_batch_params=False, objective="gap",
                                             spec_reduce="min", soft_tau=float(g[f"{cfg}_tau"]))
    assert_close(b.lower, g[f"{cfg}_gap_min_lower_6"], f"{cfg} alpha-beta function, shared gap/min lower")
    assert_close(b.upper, g[f"{cfg}_gap_min_upper_6"], f"{cfg} alpha-beta function, shared gap/min upper")


def test_single_spec_row_and_single_input_against_oracle(dev):
    """Edge shapes of the objective kernels: one input with one spec row (every reduction degenerates to the row itself)
    and one input with nine rows, per-domain and shared parameters, against the oracle."""
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import adaptive_alpha_from_trace, alpha_crown_from_trace, ibp_trace, shared_alpha_crown_from_trace
    from boundflow_b200.ir import InputSpec
    from oracle import crown_oracle as O

    wl = W.make_workload("c1", batch=1)
    spec = InputSpec.box(value_name="input", lower=wl.lo.to(dev), upper=wl.up.to(dev))
    trace = ibp_trace(wl.module, spec)
    a0 = adaptive_alpha_from_trace(trace)
    inp = O.box_input(wl.lo, wl.up)
    tr = O.forward_ibp_trace(wl.layers, inp)
    for C in (wl.C[:, :1], wl.C):
        for obj, red in (("both", "min"), ("gap", "softmin"), ("upper", "min"), ("lower", "softmin")):
            got = alpha_crown_from_trace(trace, C.to(dev), a0, steps=3, lr=0.1, objective=obj, spec_reduce=red, soft_tau=0.7, lb_weight=1.0, ub_weight=2.0)
            ref_l, ref_u, _a, _t = O.alpha_crown(wl.layers, inp, C, steps=3, lr=0.1, alpha0=[a.cpu() for a in a0], trace=tr, objective=obj,
                                                 spec_reduce=red, soft_tau=0.7, lb_weight=1.0, ub_weight=2.0)
            assert_close(got[0], ref_l, f"per-domain {obj}/{red} lower, S={C.shape[1]}")
            assert_close(got[1], ref_u, f"per-domain {obj}/{red} upper, S={C.shape[1]}")
            a_sh = [torch.full((n,), 0.5, device=dev) for n in trace.chain.relu_widths]
            got = shared_alpha_crown_from_trace(trace, C.to(dev), a_sh, steps=3, lr=0.1, objective=obj, spec_reduce=red, soft_tau=0.7, lb_weight=1.0,
                                                ub_weight=2.0)
            ref_l, ref_u, _a, _t = O.alpha_crown_shared(wl.layers, inp, C, steps=3, lr=0.1, trace=tr, objective=obj, spec_reduce=red, soft_tau=0.7,
                                                        lb_weight=1.0, ub_weight=2.0)
            assert_close(got[0], ref_l, f"shared {obj}/{red} lower, S={C.shape[1]}")
            assert_close(got[1], ref_u, f"shared {obj}/{red} upper, S={C.shape[1]}")
