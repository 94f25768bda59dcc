"""IBP and CROWN on graphs that are not chains (residual add, fan-out), against the reference's outputs."""
import pytest
import torch

from tests.helpers import assert_close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available()
    from boundflow_b200.csrc import build

    build.build()
    return torch.device("cuda", 0)


@pytest.mark.parametrize("name", ["residual_s1", "residual_s2", "fanout_mlp", "mini_resnet", "concat_cnn", "concat_mlp"])
def test_graph_matches_reference_golden(dev, golden, name):
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import needs_graph_path, run_crown_ibp_mlp
    from boundflow_b200.executor import CudaTaskExecutor
    from boundflow_b200.ir import InputSpec

    g = golden("graph_cases.npz")
    module, _x, lo, up, C = W.make_graph_cases()[name]
    assert needs_graph_path(module)
    spec = InputSpec.box(value_name="input", lower=lo.to(dev), upper=up.to(dev))
    ibp = CudaTaskExecutor().run_ibp(module, spec)
    assert_close(ibp.lower, g[f"{name}_ibp_lower"], "ibp lower")
    assert_close(ibp.upper, g[f"{name}_ibp_upper"], "ibp upper")
    crown = run_crown_ibp_mlp(module, spec, linear_spec_C=None if C is None else C.to(dev))
    assert_close(crown.lower, g[f"{name}_crown_lower"], "crown lower")
    assert_close(crown.upper, g[f"{name}_crown_upper"], "crown upper")
    # CROWN is never looser than IBP here by more than rounding, and the bounds are ordered
    assert bool((crown.lower <= crown.upper + 1e-5).all())


def test_chain_modules_keep_the_fused_path_and_unsupported_modes_are_refused(dev):
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import needs_graph_path, run_alpha_beta_crown_mlp
    from boundflow_b200.ir import InputSpec

    assert not needs_graph_path(W.make_workload("c1").module)
    assert not needs_graph_path(W.make_workload("c2", batch=1).module)
    module, _x, lo, up, C = W.make_graph_cases()["fanout_mlp"]
    spec = InputSpec.box(value_name="input", lower=lo.to(dev), upper=up.to(dev))
    with pytest.raises(ValueError):
        run_alpha_beta_crown_mlp(module, spec, linear_spec_C=C.to(dev), steps=1, lr=0.1, per_batch_params=True, objective="tightest")
    with pytest.raises(ValueError):            # sum goes with the per-domain lower objective only
        run_alpha_beta_crown_mlp(module, spec, linear_spec_C=C.to(dev), steps=1, lr=0.1, per_batch_params=True, objective="gap", spec_reduce="sum")
    with pytest.raises(NotImplementedError):   # a negative weight would flip the sign decisions of the gradient sweep
        run_alpha_beta_crown_mlp(module, spec, linear_spec_C=C.to(dev), steps=1, lr=0.1, per_batch_params=True, objective="both", ub_weight=-1.0)


@pytest.mark.parametrize("name", ["residual_s1", "residual_s2", "fanout_mlp", "mini_resnet", "concat_cnn", "concat_mlp"])
def test_graph_alpha_and_alpha_beta_match_reference_golden(dev, golden, name):
    """The per-domain alpha loop and the alpha-beta loop with ReLU splits on graphs that are not chains, against the
    reference's `run_alpha_beta_crown_mlp` outputs (tests/golden/graph_alpha.npz), plus plain CROWN with a split and an
    explicit alpha against the graph oracle."""
    import numpy as np

    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import AlphaState, run_alpha_beta_crown_mlp, run_crown_ibp_mlp
    from boundflow_b200.dag import forward_ibp_dag
    from boundflow_b200.ir import InputSpec
    from oracle import graph_oracle as GO

    g = golden("graph_alpha.npz")
    module, _x, lo, up, C = W.make_graph_cases()[name]
    B = int(lo.shape[0])
    spec = InputSpec.box(value_name="input", lower=lo.to(dev), upper=up.to(dev))
    Cd = None if C is None else C.to(dev)
    tr = forward_ibp_dag(module, spec)
    adaptive = lambda t: {x: ((t.pre_l[x] >= 0) | ((t.pre_l[x] < 0) & (t.pre_u[x] > 0) & (t.pre_u[x] > -t.pre_l[x]))).float() for x in t.pre_l}  # noqa: E731
    a0 = adaptive(tr)
    for steps in (1, 4):
        b, a, _bt, stats = run_alpha_beta_crown_mlp(module, spec, linear_spec_C=Cd, steps=steps, lr=0.1, per_batch_params=True,
                                                   warm_start_alpha=AlphaState(dict(a0)))
        assert_close(b.lower.reshape(B, -1), g[f"{name}_alpha_lower_{steps}"].reshape(B, -1), f"alpha lower after {steps}")
        assert_close(b.upper.reshape(B, -1), g[f"{name}_alpha_upper_{steps}"].reshape(B, -1), f"alpha upper after {steps}")
        assert set(a.alpha_by_relu_input) == set(tr.pre_l) == set(stats.relu_inputs)
    splits = {x: torch.from_numpy(np.asarray(g[f"{name}_split_{x}"])).to(torch.int8).to(dev) for x in tr.pre_l}
    tr_s = forward_ibp_dag(module, spec, splits)
    assert int(tr_s.infeasible.sum()) == 0
    b, _a, bt, _s = run_alpha_beta_crown_mlp(module, spec, linear_spec_C=Cd, relu_split_state=splits, steps=3, lr=0.1, per_batch_params=True,
                                            warm_start_alpha=AlphaState(adaptive(tr_s)))
    assert_close(b.lower.reshape(B, -1), g[f"{name}_beta_lower_3"].reshape(B, -1), "alpha-beta lower after 3")
    assert_close(b.upper.reshape(B, -1), g[f"{name}_beta_upper_3"].reshape(B, -1), "alpha-beta upper after 3")
    for x in tr.pre_l:
        assert_close(bt.beta_by_relu_input[x].reshape(B, -1), g[f"{name}_beta_{x}_3"], f"beta {x} after 3", atol=1e-5)
    # plain CROWN with splits, an explicit alpha and a lower-side add term, against the graph oracle
    gen = torch.Generator("cpu").manual_seed(3)
    alpha = {x: torch.rand(B, int(tr.pre_l[x].shape[1]), generator=gen) for x in tr.pre_l}
    add = {x: -0.05 * torch.rand(B, int(tr.pre_l[x].shape[1]), generator=gen) * splits[x].cpu().float() for x in tr.pre_l}
    got = run_crown_ibp_mlp(module, spec, linear_spec_C=Cd, relu_split_state=splits, relu_alpha={x: a.to(dev) for x, a in alpha.items()},
                            relu_pre_add_coeff_l={x: a.to(dev) for x, a in add.items()})
    env, pre = GO.forward_ibp_graph(module, lo, up, splits={x: s.cpu() for x, s in splits.items()})
    n_out = env["out"][0].reshape(B, -1).shape[1]
    Cb = torch.eye(n_out).unsqueeze(0).expand(B, -1, -1) if C is None else (C if C.dim() == 3 else C.unsqueeze(0).expand(B, -1, -1))
    ref_l, ref_u = GO.crown_backward_graph(module, env, pre, Cb, lo, up, alpha=alpha, add_l=add)
    assert_close(got.lower.reshape(B, -1), ref_l, "CROWN lower with split, alpha and add term")
    assert_close(got.upper.reshape(B, -1), ref_u, "CROWN upper with split, alpha and add term")


GRAPH_OBJECTIVE_CASES = (("upper", "mean"), ("gap", "min"), ("both", "softmin"), ("lower", "softmin"), ("lower", "min"))
GRAPH_SHARED_CASES = (("lower", "mean"), ("gap", "mean"), ("both", "min"), ("upper", "softmin"))


@pytest.mark.parametrize("name", ["residual_s1", "residual_s2", "fanout_mlp", "mini_resnet", "concat_cnn", "concat_mlp"])
def test_graph_objectives_and_shared_mode_match_reference_golden(dev, golden, name):
    """On graphs that are not chains: the upper / gap / both objectives and the min / softmin reductions with per-domain
    parameters, the shared-parameter mode of `run_alpha_beta_crown_mlp` (with and without beta) and `run_alpha_crown_mlp`,
    against the reference's outputs (tests/golden/graph_objectives.npz; lb_weight 1.0, ub_weight 0.5)."""
    import numpy as np

    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import AlphaState, run_alpha_beta_crown_mlp, run_alpha_crown_mlp
    from boundflow_b200.dag import forward_ibp_dag
    from boundflow_b200.ir import InputSpec

    g, ga = golden("graph_objectives.npz"), golden("graph_alpha.npz")
    module, _x, lo, up, C = W.make_graph_cases()[name]
    B = int(lo.shape[0])
    spec = InputSpec.box(value_name="input", lower=lo.to(dev), upper=up.to(dev))
    Cd = None if C is None else C.to(dev)
    tr = forward_ibp_dag(module, spec)
    a0 = {x: ((tr.pre_l[x] >= 0) | ((tr.pre_l[x] < 0) & (tr.pre_u[x] > 0) & (tr.pre_u[x] > -tr.pre_l[x]))).float() for x in tr.pre_l}
    kw = {"soft_tau": float(g["tau"]), "lb_weight": 1.0, "ub_weight": 0.5}
    for obj, red in GRAPH_OBJECTIVE_CASES:
        for steps in (1, 4):
            b, a, _bt, stats = run_alpha_beta_crown_mlp(module, spec, linear_spec_C=Cd, steps=steps, lr=0.1, per_batch_params=True, objective=obj,
                                                       spec_reduce=red, warm_start_alpha=AlphaState(dict(a0)), **kw)
            assert stats.objective == obj and stats.spec_reduce == red
            assert_close(b.lower.reshape(B, -1), g[f"{name}_{obj}_{red}_lower_{steps}"].reshape(B, -1), f"{obj}/{red} lower after {steps}")
            assert_close(b.upper.reshape(B, -1), g[f"{name}_{obj}_{red}_upper_{steps}"].reshape(B, -1), f"{obj}/{red} upper after {steps}")
    for obj, red in GRAPH_SHARED_CASES:
        b, a, _bt, _s = run_alpha_beta_crown_mlp(module, spec, linear_spec_C=Cd, steps=4, lr=0.1, per_batch_params=False, objective=obj, spec_reduce=red, **kw)
        assert_close(b.lower.reshape(B, -1), g[f"{name}_shared_{obj}_{red}_lower_4"].reshape(B, -1), f"shared {obj}/{red} lower")
        assert_close(b.upper.reshape(B, -1), g[f"{name}_shared_{obj}_{red}_upper_4"].reshape(B, -1), f"shared {obj}/{red} upper")
        for x, v in a.alpha_by_relu_input.items():   # the ReLU input's shape without the batch axis
            assert tuple(v.shape) == tuple(tr.shape[x])
    b, st, stats = run_alpha_crown_mlp(module, spec, linear_spec_C=Cd, steps=4, lr=0.1)
    assert_close(b.lower.reshape(B, -1), g[f"{name}_alpha_crown_lower_4"].reshape(B, -1), "run_alpha_crown_mlp lower")
    assert_close(b.upper.reshape(B, -1), g[f"{name}_alpha_crown_upper_4"].reshape(B, -1), "run_alpha_crown_mlp upper")
    for x, v in st.alpha_by_relu_input.items():
        assert_close(v.reshape(-1), g[f"{name}_alpha_crown_alpha_{x}"], f"shared alpha {x}", atol=1e-5)
    if f"{name}_shared_beta_lower_3" in g:
        splits = {x: torch.from_numpy(np.asarray(ga[f"{name}_split_{x}"])).to(torch.int8).to(dev) for x in tr.pre_l}
        b, _a, bt, _s = run_alpha_beta_crown_mlp(module, spec, linear_spec_C=Cd, relu_split_state=splits, steps=3, lr=0.1, per_batch_params=False)
        assert_close(b.lower.reshape(B, -1), g[f"{name}_shared_beta_lower_3"].reshape(B, -1), "shared alpha-beta lower after 3")
        assert_close(b.upper.reshape(B, -1), g[f"{name}_shared_beta_upper_3"].reshape(B, -1), "shared alpha-beta upper after 3")
        for x in tr.pre_l:
            assert_close(bt.beta_by_relu_input[x].reshape(-1), g[f"{name}_shared_beta_{x}_3"], f"shared beta {x} after 3", atol=1e-5)


@pytest.mark.parametrize("name", ["fanout_mlp", "mini_resnet", "concat_cnn"])
def test_trace_level_functions_on_graphs_match_reference_golden(dev, golden, name):
    """`forward_ibp_trace_mlp(relu_pre_constraints=...)`, `run_crown_ibp_mlp_from_forward_trace` (with the trace it left in
    the environment, and with bounds handed over as plain tensors) and the ReLU-influence variant on graphs that are
    not chains (tests/golden/graph_trace.npz)."""
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import (forward_ibp_trace_mlp, run_crown_ibp_mlp_from_forward_trace,
                                      run_crown_ibp_mlp_with_relu_influence_from_forward_trace)
    from boundflow_b200.ir import InputSpec, IntervalState

    g = golden("graph_trace.npz")
    module, _x, lo, up, C = W.make_graph_cases()[name]
    B = int(lo.shape[0])
    spec = InputSpec.box(value_name="input", lower=lo.to(dev), upper=up.to(dev))
    env, relu_pre = forward_ibp_trace_mlp(module, spec)
    n_out = int(env["out"].lower.reshape(B, -1).shape[1])
    Cd = (C if C is not None else torch.eye(n_out).unsqueeze(0).expand(B, -1, -1).contiguous()).to(dev)
    cons = {x: IntervalState(lower=st.lower + 0.1 * (st.upper - st.lower), upper=st.upper - 0.1 * (st.upper - st.lower)) for x, st in relu_pre.items()}
    env2, pre2 = forward_ibp_trace_mlp(module, spec, relu_pre_constraints=cons)
    for x, st in pre2.items():
        assert tuple(st.lower.shape) == tuple(relu_pre[x].lower.shape)
        assert_close(st.lower.reshape(B, -1), g[f"{name}_cons_pre_{x}_lower"], f"constrained pre {x} lower")
        assert_close(st.upper.reshape(B, -1), g[f"{name}_cons_pre_{x}_upper"], f"constrained pre {x} upper")
    assert_close(env2["out"].lower, g[f"{name}_cons_out_lower"], "constrained ibp lower")
    assert_close(env2["out"].upper, g[f"{name}_cons_out_upper"], "constrained ibp upper")
    crown = run_crown_ibp_mlp_from_forward_trace(module, spec, interval_env=env2, relu_pre=pre2, linear_spec_C=Cd)
    assert_close(crown.lower.reshape(B, -1), g[f"{name}_cons_crown_lower"].reshape(B, -1), "crown on the constrained trace, lower")
    assert_close(crown.upper.reshape(B, -1), g[f"{name}_cons_crown_upper"].reshape(B, -1), "crown on the constrained trace, upper")
    # bounds handed over as copies (no device trace to reuse): the same result
    plain_env = {k: v for k, v in env2.items() if k != "__trace__"}
    plain_pre = {x: IntervalState(lower=st.lower.clone(), upper=st.upper.clone()) for x, st in pre2.items()}
    again = run_crown_ibp_mlp_from_forward_trace(module, spec, interval_env=plain_env, relu_pre=plain_pre, linear_spec_C=Cd)
    assert_close(again.lower, crown.lower, "crown from copied bounds, lower")
    assert_close(again.upper, crown.upper, "crown from copied bounds, upper")
    bounds, infl = run_crown_ibp_mlp_with_relu_influence_from_forward_trace(module, spec, interval_env=env, relu_pre=relu_pre, linear_spec_C=Cd)
    assert_close(bounds.lower.reshape(B, -1), g[f"{name}_infl_lower"].reshape(B, -1), "influence call lower")
    assert_close(bounds.upper.reshape(B, -1), g[f"{name}_infl_upper"].reshape(B, -1), "influence call upper")
    assert list(infl) == list(relu_pre)
    for x, v in infl.items():
        assert tuple(v.shape) == tuple(relu_pre[x].lower.shape)
        assert_close(v.reshape(B, -1), g[f"{name}_infl_{x}"], f"influence {x}")
    # constraint errors as in the reference
    bad = dict(cons)
    first = next(iter(bad))
    bad[first] = IntervalState(lower=relu_pre[first].upper + 1.0, upper=relu_pre[first].upper + 2.0)
    with pytest.raises(ValueError, match="infeasible ReLU pre-activation intersection"):
        forward_ibp_trace_mlp(module, spec, relu_pre_constraints=bad)
    with pytest.raises(ValueError, match="schema differs"):
        forward_ibp_trace_mlp(module, spec, relu_pre_constraints={x: IntervalState(lower=st.lower[:, :1], upper=st.upper[:, :1]) for x, st in cons.items()})
    with pytest.raises(ValueError, match="identities differ"):
        forward_ibp_trace_mlp(module, spec, relu_pre_constraints={**cons, "not_a_relu_input": cons[first]})


@pytest.mark.parametrize("name", ["grouped_dilated_chain", "depthwise_residual"])
def test_grouped_and_dilated_convolutions_match_reference_golden(dev, golden, name):
    """Conv2d with groups and dilation on a chain (fused sweeps) and on a residual graph (per-value walker), through the
    dense-equivalent weights: IBP, CROWN-IBP and the per-domain alpha loop (tests/golden/grouped_dilated.npz)."""
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import AlphaState, forward_ibp_trace_mlp, needs_graph_path, run_alpha_beta_crown_mlp, run_crown_ibp_mlp
    from boundflow_b200.executor import CudaTaskExecutor
    from boundflow_b200.ir import InputSpec

    g = golden("grouped_dilated.npz")
    module, _x, lo, up, _C = W.make_grouped_dilated_cases()[name]
    assert needs_graph_path(module) == (name == "depthwise_residual")
    B = int(lo.shape[0])
    spec = InputSpec.box(value_name="input", lower=lo.to(dev), upper=up.to(dev))
    ibp = CudaTaskExecutor().run_ibp(module, spec)
    assert_close(ibp.lower.reshape(B, -1), g[f"{name}_ibp_lower"].reshape(B, -1), "ibp lower")
    assert_close(ibp.upper.reshape(B, -1), g[f"{name}_ibp_upper"].reshape(B, -1), "ibp upper")
    crown = run_crown_ibp_mlp(module, spec)
    assert_close(crown.lower.reshape(B, -1), g[f"{name}_crown_lower"].reshape(B, -1), "crown lower")
    assert_close(crown.upper.reshape(B, -1), g[f"{name}_crown_upper"].reshape(B, -1), "crown upper")
    _env, relu_pre = forward_ibp_trace_mlp(module, spec)
    a0 = {x: ((st.lower >= 0) | ((st.lower < 0) & (st.upper > 0) & (st.upper > -st.lower))).float() for x, st in relu_pre.items()}
    b, _a, _bt, _s = run_alpha_beta_crown_mlp(module, spec, steps=3, lr=0.1, per_batch_params=True, warm_start_alpha=AlphaState(a0))
    assert_close(b.lower.reshape(B, -1), g[f"{name}_alpha_lower_3"].reshape(B, -1), "alpha lower after 3")
    assert_close(b.upper.reshape(B, -1), g[f"{name}_alpha_upper_3"].reshape(B, -1), "alpha upper after 3")


@pytest.mark.parametrize("name", ["mini_resnet", "fanout_mlp"])
def test_warm_starts_on_graphs(dev, name):
    """Warm starts in the value's own shape: a shared alpha of 0.5 equals the default start of `run_alpha_crown_mlp`, a
    per-domain one the default of `run_alpha_beta_crown_mlp(per_batch_params=True)`; the shared mode refuses a
    batch-specific warm start like the reference."""
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import AlphaState, run_alpha_beta_crown_mlp, run_alpha_crown_mlp
    from boundflow_b200.dag import forward_ibp_dag
    from boundflow_b200.ir import InputSpec

    module, _x, lo, up, C = W.make_graph_cases()[name]
    B = int(lo.shape[0])
    spec = InputSpec.box(value_name="input", lower=lo.to(dev), upper=up.to(dev))
    Cd = None if C is None else C.to(dev)
    tr = forward_ibp_dag(module, spec)
    shared = AlphaState({x: torch.full(tuple(tr.shape[x]), 0.5, device=dev) for x in tr.pre_l})
    a, _sa, _ = run_alpha_crown_mlp(module, spec, linear_spec_C=Cd, steps=3, lr=0.1)
    b, sb, _ = run_alpha_crown_mlp(module, spec, linear_spec_C=Cd, steps=3, lr=0.1, warm_start=shared)
    assert torch.equal(a.lower, b.lower) and torch.equal(a.upper, b.upper)
    assert {k: tuple(v.shape) for k, v in sb.alpha_by_relu_input.items()} == {x: tuple(tr.shape[x]) for x in tr.pre_l}
    per_domain = AlphaState({x: torch.full((B,) + tuple(tr.shape[x]), 0.5, device=dev) for x in tr.pre_l})
    c, _a, _b, _s = run_alpha_beta_crown_mlp(module, spec, linear_spec_C=Cd, steps=3, lr=0.1, per_batch_params=True, warm_start_alpha=per_domain)
    d, _a, _b, _s = run_alpha_beta_crown_mlp(module, spec, linear_spec_C=Cd, steps=3, lr=0.1, per_batch_params=True)
    assert torch.equal(c.lower, d.lower) and torch.equal(c.upper, d.upper)
    with pytest.raises(ValueError):
        run_alpha_crown_mlp(module, spec, linear_spec_C=Cd, steps=1, lr=0.1, warm_start=per_domain)


def test_building_blocks_against_torch(dev):
    """bf_crown_relu_bwd (incl. rows wider than one chunk) and bf_accumulate."""
    from boundflow_b200 import _lib

    lib = _lib.load()
    g = torch.Generator("cpu").manual_seed(11)
    s = torch.cuda.current_stream(dev).cuda_stream
    for B, S, n in ((3, 5, 37), (2, 3, 9001)):
        A = torch.randn(B, S, n, generator=g)
        au, al, bu = (torch.rand(B, n, generator=g) for _ in range(3))
        bl = torch.zeros(B, n)
        d0 = torch.randn(B, S, generator=g)
        Ad, aud, ald, bud, bld = (t.to(dev).contiguous() for t in (A, au, al, bu, bl))
        nb = int(lib.bf_crown_relu_bwd_scratch_bytes(B, S, n))
        scratch = torch.empty(max(nb, 16), dtype=torch.uint8, device=dev)
        for side in (0, 1):
            pos = A >= 0
            if side == 0:
                slope, icpt = torch.where(pos, al.unsqueeze(1), au.unsqueeze(1)), torch.where(pos, bl.unsqueeze(1), bu.unsqueeze(1))
            else:
                slope, icpt = torch.where(pos, au.unsqueeze(1), al.unsqueeze(1)), torch.where(pos, bu.unsqueeze(1), bl.unsqueeze(1))
            out, dd = torch.empty(B, S, n, device=dev), d0.to(dev).clone()
            _lib.check(lib.bf_crown_relu_bwd(Ad.data_ptr(), side, aud.data_ptr(), ald.data_ptr(), bud.data_ptr(), bld.data_ptr(), out.data_ptr(),
                                             dd.data_ptr(), 1, scratch.data_ptr(), scratch.numel(), B, S, n, s))
            assert_close(out, A * slope, f"A_prev side {side}")
            assert_close(dd, d0 + (A * icpt).sum(dim=2), f"delta side {side}", rtol=1e-4)
    x, y = torch.randn(1000, generator=g), torch.randn(1000, generator=g)
    xd = x.to(dev)
    _lib.check(lib.bf_accumulate(xd.data_ptr(), y.to(dev).data_ptr(), 1000, s))
    assert_close(xd, x + y, "accumulate")


def test_graph_loop_building_blocks_against_torch(dev):
    """bf_relu_split_apply, bf_rows_add_broadcast, bf_adjoint_start_box, bf_rows_conv2d_fwd, bf_relu_adjoint_rows and
    bf_conv2d_dense_rows against plain torch expressions of their definitions."""
    import torch.nn.functional as F

    from boundflow_b200 import _lib

    lib = _lib.load()
    g = torch.Generator("cpu").manual_seed(23)
    s = torch.cuda.current_stream(dev).cuda_stream
    B, S, n = 3, 5, 70
    # split on bounds, with one domain made infeasible on purpose (l > 0 there and the split says "inactive")
    l = torch.randn(B, n, generator=g) - 0.3
    u = l + torch.rand(B, n, generator=g) * 2
    sp = torch.randint(-1, 2, (B, n), generator=g).to(torch.int8)
    l[1, 7], u[1, 7], sp[1, 7] = 0.5, 0.9, -1
    ld, ud, spd = l.to(dev).clone(), u.to(dev).clone(), sp.to(dev)
    bad = torch.zeros(B, dtype=torch.int32, device=dev)
    _lib.check(lib.bf_relu_split_apply(ld.data_ptr(), ud.data_ptr(), spd.data_ptr(), n, bad.data_ptr(), B, n, s))
    want_l = torch.where(sp > 0, l.clamp(min=0), l)
    want_u = torch.where(sp < 0, u.clamp(max=0), u)
    assert torch.equal(ld.cpu(), want_l) and torch.equal(ud.cpu(), want_u)
    assert bad.cpu().tolist() == (want_l > want_u).any(dim=1).int().tolist() and bad.cpu().tolist()[1] == 1
    # broadcast add, per domain and shared
    A = torch.randn(B, S, n, generator=g)
    v = torch.randn(B, n, generator=g)
    Ad, vd, v0d = A.to(dev).clone(), v.to(dev), v[0].to(dev).contiguous()   # device operands stay referenced until the calls have run
    _lib.check(lib.bf_rows_add_broadcast(Ad.data_ptr(), vd.data_ptr(), n, B, S, n, s))
    assert torch.equal(Ad.cpu(), A + v.unsqueeze(1))
    Ad = A.to(dev).clone()
    _lib.check(lib.bf_rows_add_broadcast(Ad.data_ptr(), v0d.data_ptr(), 0, B, S, n, s))
    assert torch.equal(Ad.cpu(), A + v[0])
    # adjoint start vector
    mid, rad = torch.rand(B, n, generator=g), torch.rand(B, n, generator=g) * 0.1
    A[0, 0, :5] = 0.0
    Ad, midd, radd = A.to(dev).clone(), mid.to(dev), rad.to(dev)
    _lib.check(lib.bf_adjoint_start_box(Ad.data_ptr(), midd.data_ptr(), radd.data_ptr(), B, S, n, s))
    assert torch.equal(Ad.cpu(), mid.unsqueeze(1) - torch.sign(A) * rad.unsqueeze(1))
    # forward convolution of rows
    Ci, Hi, Co, k, st, pd = 3, 9, 4, 3, 2, 1
    Ho = (Hi + 2 * pd - k) // st + 1
    X = torch.randn(B * S, Ci, Hi, Hi, generator=g)
    Wc, bc = torch.randn(Co, Ci, k, k, generator=g), torch.randn(Co, generator=g)
    out = torch.empty(B * S, Co, Ho, Ho, device=dev)
    Xd, Wd, bd = X.to(dev), Wc.to(dev), bc.to(dev)
    _lib.check(lib.bf_rows_conv2d_fwd(Xd.data_ptr(), Wd.data_ptr(), bd.data_ptr(), out.data_ptr(), B * S, Ci, Hi, Hi, Co, Ho, Ho,
                                      k, k, st, st, pd, pd, s))
    assert_close(out, F.conv2d(X, Wc, bc, st, pd), "rows conv2d forward", atol=1e-5)
    # ReLU adjoint step with both gradient sums
    G, Ah = torch.randn(B, S, n, generator=g), torch.randn(B, S, n, generator=g)
    au, al, bu = torch.rand(B, n, generator=g), torch.rand(B, n, generator=g), torch.rand(B, n, generator=g)
    grad0, gsum0 = torch.randn(B, n, generator=g), torch.randn(B, n, generator=g)
    Gd, gr, gs = G.to(dev).clone(), grad0.to(dev).clone(), gsum0.to(dev).clone()
    Ahd, aud, ald, bud, l2d, u2d = (x.to(dev).contiguous() for x in (Ah, au, al, bu, l, u))
    _lib.check(lib.bf_relu_adjoint_rows(Gd.data_ptr(), Ahd.data_ptr(), aud.data_ptr(), ald.data_ptr(), bud.data_ptr(), l2d.data_ptr(),
                                        u2d.data_ptr(), gr.data_ptr(), gs.data_ptr(), None, B, S, n, s))
    sel = Ah >= 0
    amb = ((l < 0) & (u > 0)).unsqueeze(1)
    assert_close(Gd, torch.where(sel, al.unsqueeze(1) * G, au.unsqueeze(1) * G + bu.unsqueeze(1)), "relu adjoint output", atol=1e-6)
    assert_close(gr, grad0 + (torch.where(sel & amb, Ah * G, torch.zeros_like(G))).sum(dim=1), "alpha gradient sums", atol=1e-5)
    assert_close(gs, gsum0 + G.sum(dim=1), "beta gradient sums", atol=1e-5)
    # the same step with a weight per row on the beta sums (min / softmin objectives with beta parameters)
    rw = torch.rand(B, S, generator=g)
    Gd, gr, gs, rwd = G.to(dev).clone(), grad0.to(dev).clone(), gsum0.to(dev).clone(), rw.to(dev)
    _lib.check(lib.bf_relu_adjoint_rows(Gd.data_ptr(), Ahd.data_ptr(), aud.data_ptr(), ald.data_ptr(), bud.data_ptr(), l2d.data_ptr(),
                                        u2d.data_ptr(), gr.data_ptr(), gs.data_ptr(), rwd.data_ptr(), B, S, n, s))
    assert_close(gr, grad0 + (torch.where(sel & amb, Ah * G, torch.zeros_like(G))).sum(dim=1), "alpha gradient sums (weighted call)", atol=1e-5)
    assert_close(gs, gsum0 + (rw.unsqueeze(2) * G).sum(dim=1), "weighted beta gradient sums", atol=1e-5)
