"""alpha-CROWN with alpha shared across the batch (`run_alpha_crown_mlp`) on the GPU, against the
reference's own outputs (tests/golden/shared_alpha.npz) and the oracle."""
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


def test_c3_matches_reference_golden(dev, golden):
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import crown_from_trace, ibp_trace, run_alpha_crown_mlp
    from boundflow_b200.ir import InputSpec

    g = golden("shared_alpha.npz")
    wl = W.make_workload("c3", batch=8)
    spec = InputSpec.box(value_name="input", lower=wl.lo.to(dev), upper=wl.up.to(dev))
    b1, _s1, _ = run_alpha_crown_mlp(wl.module, spec, linear_spec_C=wl.C.to(dev), steps=1, lr=0.1)
    assert_close(b1.lower, g["c3_lower_1step"], "one-step lower")
    assert_close(b1.upper, g["c3_upper_1step"], "one-step upper")
    b, st, stats = run_alpha_crown_mlp(wl.module, spec, linear_spec_C=wl.C.to(dev), steps=10, lr=0.1)
    # optimised bounds: Adam amplifies rounding-level differences, see tests/test_gpu_parity.py::test_c3_alpha_crown
    assert_close(b.lower, g["c3_lower"], "lower")
    assert_close(b.upper, g["c3_upper"], "upper")
    assert float(b.lower.mean()) >= float(torch.as_tensor(g["c3_lower"]).mean()) - 2e-4 * abs(float(torch.as_tensor(g["c3_lower"]).mean()))
    assert stats.relu_inputs == tuple(wl.relu_names)
    for n in wl.relu_names:
        a = st.alpha_by_relu_input[n]
        assert a.dim() == 1, "alpha has the ReLU input's shape, no batch axis"
        assert float(a.min()) >= 0.0 and float(a.max()) <= 1.0
        assert float((a.cpu() - torch.as_tensor(g[f"c3_alpha_{n}"]).reshape(-1)).abs().mean()) < 2e-3
    # the returned bounds are one strict evaluation at the returned alpha
    trace = ibp_trace(wl.module, spec)
    lo_chk, up_chk = crown_from_trace(trace, wl.C.to(dev), relu_alpha=st.alpha_by_relu_input)
    assert_close(lo_chk, b.lower, "lower at best alpha")
    assert_close(up_chk, b.upper, "upper at best alpha")


def test_c4_split_domains_match_reference_golden_and_oracle(dev, golden):
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import run_alpha_crown_mlp
    from boundflow_b200.ir import InputSpec
    from oracle import crown_oracle as O

    g = golden("shared_alpha.npz")
    wl = W.make_workload("c4")
    root = O.forward_ibp_trace(wl.layers, O.box_input(wl.lo, wl.up))
    D = 24
    splits = W.make_split_domains(wl, root.pre, n_domains=D)
    lo, up = wl.lo.expand(D, -1).contiguous(), wl.up.expand(D, -1).contiguous()
    spec = InputSpec.box(value_name="input", lower=lo.to(dev), upper=up.to(dev))
    state = {n: s.to(dev) for n, s in zip(wl.relu_names, splits)}
    C = wl.C.expand(D, -1, -1).contiguous().to(dev)
    b, st, _ = run_alpha_crown_mlp(wl.module, spec, linear_spec_C=C, steps=10, lr=0.1, relu_split_state=state)
    assert_close(b.lower, g["c4_lower"], "lower")
    assert_close(b.upper, g["c4_upper"], "upper")
    # one Adam step is insensitive to rounding: strict against the oracle (216 coefficient rows: FFMA and tensor-core sizes mix)
    b1, _s, _ = run_alpha_crown_mlp(wl.module, spec, linear_spec_C=C, steps=1, lr=0.1, relu_split_state=state)
    o1 = O.alpha_crown_shared(wl.layers, O.box_input(lo, up), wl.C.expand(D, -1, -1), steps=1, lr=0.1, splits=splits)
    assert_close(b1.lower, o1[0], "one-step lower")
    assert_close(b1.upper, o1[1], "one-step upper")


def test_warm_start_zero_steps_and_refusals(dev):
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import AlphaState, run_alpha_crown_mlp, run_crown_ibp_mlp
    from boundflow_b200.ir import InputSpec

    wl = W.make_workload("c3", batch=3)
    spec = InputSpec.box(value_name="input", lower=wl.lo.to(dev), upper=wl.up.to(dev))
    # steps=0 with warm start alpha = 0: the lower relaxation slope is 0 on every unstable neuron
    b0, st0, _ = run_alpha_crown_mlp(wl.module, spec, linear_spec_C=wl.C.to(dev), steps=0, alpha_init=0.0)
    ref = run_crown_ibp_mlp(wl.module, spec, linear_spec_C=wl.C.to(dev), relu_alpha={n: torch.zeros_like(a) for n, a in st0.alpha_by_relu_input.items()})
    assert_close(b0.lower, ref.lower, "steps=0 lower")
    assert_close(b0.upper, ref.upper, "steps=0 upper")
    warm = AlphaState({n: torch.full_like(a, 0.25) for n, a in st0.alpha_by_relu_input.items()})
    bw, stw, _ = run_alpha_crown_mlp(wl.module, spec, linear_spec_C=wl.C.to(dev), steps=0, warm_start=warm)
    for n in wl.relu_names:
        assert float((stw.alpha_by_relu_input[n] - 0.25).abs().max()) == 0.0
    # the other objectives and reductions run (tests/test_gpu_objectives.py pins them); unknown names and a
    # non-positive softmin temperature raise like the reference
    with pytest.raises(ValueError):
        run_alpha_crown_mlp(wl.module, spec, linear_spec_C=wl.C.to(dev), objective="tightest")
    with pytest.raises(ValueError):
        run_alpha_crown_mlp(wl.module, spec, linear_spec_C=wl.C.to(dev), spec_reduce="softmin", soft_tau=0.0)
    with pytest.raises(ValueError):
        run_alpha_crown_mlp(wl.module, spec, linear_spec_C=wl.C.to(dev), spec_reduce="sum")


def test_shared_alpha_beta_matches_reference_golden(dev, golden):
    """per_batch_params=False of run_alpha_beta_crown_mlp: one alpha row and one beta row for all domains."""
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import crown_from_trace, ibp_trace, run_alpha_beta_crown_mlp
    from boundflow_b200.ir import InputSpec
    from oracle import crown_oracle as O

    g = golden("shared_alpha.npz")
    wl = W.make_workload("c4")
    root = O.forward_ibp_trace(wl.layers, O.box_input(wl.lo, wl.up))
    D = 24
    splits = W.make_split_domains(wl, root.pre, n_domains=D)
    lo, up = wl.lo.expand(D, -1).contiguous(), wl.up.expand(D, -1).contiguous()
    spec = InputSpec.box(value_name="input", lower=lo.to(dev), upper=up.to(dev))
    state = {n: s.to(dev) for n, s in zip(wl.relu_names, splits)}
    C = wl.C.expand(D, -1, -1).contiguous().to(dev)
    b1, _a1, _b1, _ = run_alpha_beta_crown_mlp(wl.module, spec, linear_spec_C=C, relu_split_state=state, steps=1, lr=0.1, per_batch_params=False)
    assert_close(b1.lower, g["c4_ab_lower_1step"], "one-step lower")
    assert_close(b1.upper, g["c4_ab_upper_1step"], "one-step upper")
    b, a_st, b_st, stats = run_alpha_beta_crown_mlp(wl.module, spec, linear_spec_C=C, relu_split_state=state, steps=10, lr=0.1, per_batch_params=False)
    assert_close(b.lower, g["c4_ab_lower"], "lower")
    assert_close(b.upper, g["c4_ab_upper"], "upper")
    for n, sp in zip(wl.relu_names, splits):
        bt = b_st.beta_by_relu_input[n]
        assert bt.dim() == 1 and float(bt.min()) >= 0.0
        assert float(bt.cpu()[(sp != 0).sum(dim=0) == 0].abs().max()) == 0.0, "beta moves only where some domain has a split"
        assert float((bt.cpu() - torch.as_tensor(g[f"c4_ab_beta_{n}"]).reshape(-1)).abs().max()) <= 0.05
    assert len(stats.branch_choices) == D
    # the returned bounds are one strict evaluation at the returned shared alpha and beta
    trace = ibp_trace(wl.module, spec, relu_split_state=state)
    add = {n: -b_st.beta_by_relu_input[n].unsqueeze(0) * s.to(dev).float() for n, s in zip(wl.relu_names, splits)}
    lo_chk, up_chk = crown_from_trace(trace, C, relu_alpha=a_st.alpha_by_relu_input, relu_pre_add_coeff_l=add)
    assert_close(lo_chk, b.lower, "lower at best alpha/beta")
    assert_close(up_chk, b.upper, "upper at best alpha")
    # beta does not make the whole-batch objective worse than alpha alone
    ba, _x, _y, _z = run_alpha_beta_crown_mlp(wl.module, spec, linear_spec_C=C, relu_split_state=state, steps=10, lr=0.1,
                                              per_batch_params=False, optimize_beta=False)
    assert float(b.lower.mean()) >= float(ba.lower.mean()) - 1e-3 * abs(float(ba.lower.mean()))
