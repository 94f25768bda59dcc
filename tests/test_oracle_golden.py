"""Pins the CPU oracle against outputs of the reference itself (tests/golden/*.npz,
made by tests/golden/make_golden.py) and against the literal known-answer cases of
the reference's own tests."""
import numpy as np
import pytest
import torch

from boundflow_b200 import workloads as W
from oracle import crown_oracle as O
from tests.helpers import assert_close, workload_checksum


def _check_inputs(wl, g):
    assert np.allclose(workload_checksum(wl), g["input_checksum"], rtol=1e-12, atol=0), "seeded inputs drifted from the golden run"


def test_c1_ibp_and_crown(golden):
    g = golden("c1_ibp_crown.npz")
    wl = W.make_workload("c1")
    _check_inputs(wl, g)
    inp = O.box_input(wl.lo, wl.up)
    lower, upper, trace = O.crown_ibp(wl.layers, inp, wl.C)
    assert_close(trace.out[0], g["ibp_lower"], "ibp lower")
    assert_close(trace.out[1], g["ibp_upper"], "ibp upper")
    assert_close(trace.pre[0][0], g["pre1_lower"], "pre1 lower")
    assert_close(trace.pre[1][1], g["pre2_upper"], "pre2 upper")
    assert_close(lower, g["crown_lower"], "crown lower")
    assert_close(upper, g["crown_upper"], "crown upper")
    lo2, up2, _ = O.crown_ibp(wl.layers, O.linf_box(wl.x, wl.eps), wl.C)
    assert_close(lo2, g["crown_linf_lower"], "crown linf lower")
    assert_close(up2, g["crown_linf_upper"], "crown linf upper")


def test_c2_cnn(golden):
    g = golden("c2_cnn.npz")
    wl = W.make_workload("c2", batch=8)
    _check_inputs(wl, g)
    lower, upper, trace = O.crown_ibp(wl.layers, O.box_input(wl.lo, wl.up), wl.C)
    assert_close(trace.out[0], g["ibp_lower"], "ibp lower")
    assert_close(trace.out[1], g["ibp_upper"], "ibp upper")
    assert_close(lower, g["crown_lower"], "crown lower")
    assert_close(upper, g["crown_upper"], "crown upper")
    wl4 = W.make_workload("c2", batch=4)
    lo4, up4, tr4 = O.crown_with_intermediate_crown(wl4.layers, O.box_input(wl4.lo, wl4.up), wl4.C)
    assert_close(lo4, g["full_lower"], "full-crown lower")
    assert_close(up4, g["full_upper"], "full-crown upper")
    for r, name in enumerate(wl4.relu_names):
        assert_close(tr4.pre[r][0].reshape(4, -1)[:, ::7], g[f"pre_{name}_lower"], f"pre {name} lower")
        assert_close(tr4.pre[r][1].reshape(4, -1)[:, ::7], g[f"pre_{name}_upper"], f"pre {name} upper")


def test_c3_alpha(golden):
    g = golden("c3_alpha.npz")
    wl = W.make_workload("c3", batch=8)
    _check_inputs(wl, g)
    inp = O.box_input(wl.lo, wl.up)
    lower, upper, trace = O.crown_ibp(wl.layers, inp, wl.C)
    assert_close(lower, g["plain_lower"], "plain lower")
    assert_close(upper, g["plain_upper"], "plain upper")
    a0 = O.adaptive_alpha_init(trace)
    lo0, up0 = O.crown_backward(wl.layers, inp, trace, wl.C, alpha=a0)
    assert_close(lo0, g["step0_lower"], "step0 lower")
    assert_close(up0, g["step0_upper"], "step0 upper")
    grads, _ = O.alpha_gradient(wl.layers, inp, trace, wl.C, a0)
    for r, name in enumerate(wl.relu_names):
        assert_close(grads[r], g[f"grad0_{name}"], f"grad0 {name}", atol=1e-5, rtol=1e-4)
    bl, bu, ba, _ = O.alpha_crown(wl.layers, inp, wl.C, steps=20, lr=0.1, alpha0=a0, spec_reduce="mean")
    assert_close(bl, g["best_lower"], "alpha best lower")
    assert_close(bu, g["best_upper"], "alpha best upper")
    sl, su, _, _ = O.alpha_crown(wl.layers, inp, wl.C, steps=20, lr=0.1, alpha0=a0, spec_reduce="sum")
    # The mean-objective runs above follow the reference's trajectory to 1e-7.  With the sum objective every
    # gradient is 9x larger relative to Adam's eps = 1e-8: alpha entries whose exact gradient is zero carry a
    # rounding residue r and move by lr * r / (|r| + 1e-8), i.e. by almost +-lr once |r| is 9x larger, with the
    # sign of the residue -- which depends on the order of operations.  Measured distance between this
    # restatement and the reference's primitives after 20 such steps: 5.5e-5 relative.
    assert_close(sl, g["sum_best_lower"], "alpha(sum) best lower", rtol=1e-4)
    assert (bl.mean(dim=1) >= lo0.mean(dim=1) - 1e-6).all()


def test_c4_split_alpha(golden):
    g = golden("c4_split_alpha.npz")
    wl = W.make_workload("c4")
    _check_inputs(wl, g)
    root = O.forward_ibp_trace(wl.layers, O.box_input(wl.lo, wl.up))
    D = 32
    splits = W.make_split_domains(wl, root.pre, n_domains=D)
    chk = np.array([int(s.to(torch.int64).sum()) for s in splits] + [int(s.to(torch.int64).abs().sum()) for s in splits])
    assert (chk == g["split_checksum"]).all()
    inp = O.box_input(wl.lo.expand(D, -1).contiguous(), wl.up.expand(D, -1).contiguous())
    C = wl.C.expand(D, -1, -1).contiguous()
    trace = O.forward_ibp_trace(wl.layers, inp, splits=splits)
    assert not trace.infeasible.any()
    for r, name in enumerate(wl.relu_names):
        assert_close(trace.pre[r][0], g[f"pre_{name}_lower"], f"pre {name} lower")
        assert_close(trace.pre[r][1], g[f"pre_{name}_upper"], f"pre {name} upper")
    a0 = O.adaptive_alpha_init(trace)
    lo0, up0 = O.crown_backward(wl.layers, inp, trace, C, alpha=a0)
    assert_close(lo0, g["step0_lower"], "step0 lower")
    bl, bu, _, _ = O.alpha_crown(wl.layers, inp, C, steps=10, lr=0.1, alpha0=a0, trace=trace)
    assert_close(bl, g["best_lower"], "best lower")
    assert_close(bu, g["best_upper"], "best upper")


def test_c5_cnn(golden):
    g = golden("c5_cnn.npz")
    wl = W.make_workload("c5", batch=2)
    _check_inputs(wl, g)
    lower, upper, trace = O.crown_ibp(wl.layers, O.box_input(wl.lo, wl.up), wl.C)
    assert_close(trace.out[0], g["ibp_lower"], "ibp lower")
    assert_close(lower, g["crown_lower"], "crown lower")
    assert_close(upper, g["crown_upper"], "crown upper")


def test_bruteforce_grid_known_answer():
    """Toy 2-2-2 network of the reference's grid test
    (tests/test_phase6b_crown_ibp_mlp.py:153-175): bounds must contain every
    point of a 41x41 grid in float64 to 1e-9."""
    dt = torch.float64
    x0 = torch.tensor([[0.2, -0.1]], dtype=dt)
    layers = [
        {"op": "linear", "W": torch.tensor([[1.3, -0.7], [-0.4, 0.9]], dtype=dt), "b": torch.tensor([0.05, -0.02], dtype=dt)},
        {"op": "relu"},
        {"op": "linear", "W": torch.tensor([[-1.2, 0.8], [0.6, -0.5]], dtype=dt), "b": torch.tensor([0.1, -0.3], dtype=dt)},
    ]
    inp = O.linf_box(x0, 0.3)
    lower, upper, _ = O.crown_ibp(layers, inp, None)
    grid = torch.linspace(-0.3, 0.3, steps=41, dtype=dt)
    xs = torch.stack([x0[0] + torch.stack([dx, dy]) for dx in grid for dy in grid])
    ys = O.concrete_forward(layers, xs)
    assert (ys >= lower - 1e-9).all() and (ys <= upper + 1e-9).all()


def test_alpha_gradient_sign_selection_formula():
    """Closed form of the reference's known-answer test
    (tests/test_phase7a_pr10_relu_dense_reference.py:132-162):
    d/dalpha sum(outputs) = sum over rows of A_u[A_u<0 & amb] + A_l[A_l>=0 & amb]."""
    dt = torch.float64
    g = torch.Generator("cpu").manual_seed(5)
    l = torch.tensor([[0.5, -2.0, -1.0, -0.3]], dtype=dt)
    u = torch.tensor([[1.0, -0.5, 2.0, 0.9]], dtype=dt)
    A_u = torch.randn(1, 3, 4, generator=g, dtype=dt)
    A_l = torch.randn(1, 3, 4, generator=g, dtype=dt)
    alpha = torch.tensor([[0.2, 0.3, 0.6, 0.8]], dtype=dt, requires_grad=True)
    au, bu, al, bl = O.relu_slopes(l, u, alpha)
    out = O.relu_backward(A_u, A_l, torch.zeros(1, 3, dtype=dt), torch.zeros(1, 3, dtype=dt), au, bu, al, bl)
    sum(o.sum() for o in out).backward()
    amb = ((l < 0) & (u > 0)).unsqueeze(1)
    expected = (torch.where((A_u < 0) & amb, A_u, torch.zeros_like(A_u)) + torch.where((A_l >= 0) & amb, A_l, torch.zeros_like(A_l))).sum(dim=(0, 1))
    assert torch.allclose(alpha.grad[0], expected, atol=1e-12, rtol=1e-12)
    assert torch.equal(alpha.grad[0, :2], torch.zeros(2, dtype=dt))


def test_fused_region_reference_vectors(golden):
    """The oracle's ReLU-backward + affine-backward equals the reference's eager
    fused-region executor (runtime/fused_crown.py:330-400) on seeded requests."""
    g = golden("fused_region.npz")
    gen = torch.Generator("cpu").manual_seed(77)
    D, S, n_cur, n_prev = 5, 9, 37, 53
    A_u = torch.randn(D, S, n_cur, generator=gen)
    A_l = torch.randn(D, S, n_cur, generator=gen)
    l = torch.randn(D, n_cur, generator=gen) - 0.2
    u = l + torch.rand(D, n_cur, generator=gen) * 2.0
    Wt = torch.randn(n_cur, n_prev, generator=gen)
    bias = torch.randn(n_cur, generator=gen)
    au, bu, al, bl = O.relu_relax(l, u)
    z = torch.zeros(D, S)
    sA_u, sA_l, d_u, d_l = O.relu_backward(A_u, A_l, z, z, au, bu, al, bl)
    P_u, d_u = O.linear_backward(sA_u, d_u, Wt, bias)
    P_l, d_l = O.linear_backward(sA_l, d_l, Wt, bias)
    assert_close(P_u, g["lin_A_prev_u"], "A_prev_u")
    assert_close(P_l, g["lin_A_prev_l"], "A_prev_l")
    assert_close(d_u, g["lin_delta_u"], "delta_u")
    assert_close(d_l, g["lin_delta_l"], "delta_l")


def test_c4_alpha_beta_and_branch_choices(golden):
    """The verbatim reference function `run_alpha_beta_crown_mlp` (alpha and beta optimised,
    per-domain parameters) and its widest-gap branching hint on 32 split subdomains."""
    g = golden("c4_split_alpha_beta.npz")
    wl = W.make_workload("c4")
    root = O.forward_ibp_trace(wl.layers, O.box_input(wl.lo, wl.up))
    D = 32
    splits = W.make_split_domains(wl, root.pre, n_domains=D)
    inp = O.box_input(wl.lo.expand(D, -1).contiguous(), wl.up.expand(D, -1).contiguous())
    C = wl.C.expand(D, -1, -1).contiguous()
    trace = O.forward_ibp_trace(wl.layers, inp, splits=splits)
    choices = O.branch_choices(trace)
    got = np.array([[-1, -1] if c is None else list(c) for c in choices])
    assert (got == g["branch_choices"]).all()
    a0 = O.adaptive_alpha_init(trace)
    bl, bu, ba, bb, _ = O.alpha_crown(wl.layers, inp, C, steps=10, lr=0.1, alpha0=a0, splits=splits, trace=trace,
                                      optimize_beta=True, return_beta=True)
    assert_close(bl, g["best_lower"], "alpha-beta best lower")
    assert_close(bu, g["best_upper"], "alpha-beta best upper")
    for r, name in enumerate(wl.relu_names):
        assert_close(bb[r], g[f"beta_{name}"], f"beta {name}", atol=1e-5, rtol=1e-4)
    # beta moves only where a split exists and stays non-negative
    for r in range(len(splits)):
        assert float(bb[r].min()) >= 0.0
        assert float(bb[r][splits[r] == 0].abs().max()) == 0.0


def test_lp_ball_inputs(golden):
    """L2 / L1 balls: dual-norm first layer and concretisation (MLP), bounding-box forward pass (CNN)."""
    g = golden("lp_ball.npz")
    for tag, wl in (("c1", W.make_workload("c1")), ("c2", W.make_workload("c2", batch=4))):
        assert np.allclose(workload_checksum(wl), g[f"{tag}_input_checksum"], rtol=1e-12, atol=0)
        for pname, p in (("l2", 2), ("l1", 1)):
            inp = O.lp_ball(wl.x, float(g[f"{tag}_{pname}_eps"]), p)
            lower, upper, trace = O.crown_ibp(wl.layers, inp, wl.C)
            assert_close(trace.out[0], g[f"{tag}_{pname}_ibp_lower"], f"{tag} {pname} ibp lower")
            assert_close(trace.out[1], g[f"{tag}_{pname}_ibp_upper"], f"{tag} {pname} ibp upper")
            assert_close(lower, g[f"{tag}_{pname}_crown_lower"], f"{tag} {pname} crown lower")
            assert_close(upper, g[f"{tag}_{pname}_crown_upper"], f"{tag} {pname} crown upper")


def test_shared_alpha(golden):
    """`run_alpha_crown_mlp`: one alpha per neuron for the whole batch, whole-batch best-of."""
    g = golden("shared_alpha.npz")
    wl = W.make_workload("c3", batch=8)
    assert np.allclose(workload_checksum(wl), g["c3_input_checksum"], rtol=1e-12, atol=0)
    inp = O.box_input(wl.lo, wl.up)
    lo1, up1, _a1, _ = O.alpha_crown_shared(wl.layers, inp, wl.C, steps=1, lr=0.1)
    assert_close(lo1, g["c3_lower_1step"], "c3 one-step lower")
    assert_close(up1, g["c3_upper_1step"], "c3 one-step upper")
    lo, up, a, _ = O.alpha_crown_shared(wl.layers, inp, wl.C, steps=10, lr=0.1)
    # the optimised trajectory amplifies rounding (see test_c3_alpha): relative tolerance 3e-4
    assert_close(lo, g["c3_lower"], "c3 lower")
    assert_close(up, g["c3_upper"], "c3 upper")
    for r, n in enumerate(wl.relu_names):
        assert float((a[r] - torch.as_tensor(g[f"c3_alpha_{n}"]).reshape(-1)).abs().mean()) < 2e-3

    wl = W.make_workload("c4")
    root = O.forward_ibp_trace(wl.layers, O.box_input(wl.lo, wl.up))
    D = 24
    splits = W.make_split_domains(wl, root.pre, n_domains=D)
    assert (np.array([int(s.to(torch.int64).abs().sum()) for s in splits]) == g["c4_split_checksum"]).all()
    inp = O.box_input(wl.lo.expand(D, -1).contiguous(), wl.up.expand(D, -1).contiguous())
    lo, up, a, _ = O.alpha_crown_shared(wl.layers, inp, wl.C.expand(D, -1, -1), steps=10, lr=0.1, splits=splits)
    assert_close(lo, g["c4_lower"], "c4 lower")
    assert_close(up, g["c4_upper"], "c4 upper")


def test_shared_alpha_beta(golden):
    """`run_alpha_beta_crown_mlp(per_batch_params=False)`: shared alpha and beta on split c4 domains."""
    g = golden("shared_alpha.npz")
    wl = W.make_workload("c4")
    root = O.forward_ibp_trace(wl.layers, O.box_input(wl.lo, wl.up))
    D = 24
    splits = W.make_split_domains(wl, root.pre, n_domains=D)
    inp = O.box_input(wl.lo.expand(D, -1).contiguous(), wl.up.expand(D, -1).contiguous())
    C = wl.C.expand(D, -1, -1)
    lo1, up1, _a, _b, _ = O.alpha_crown_shared(wl.layers, inp, C, steps=1, lr=0.1, splits=splits, optimize_beta=True)
    assert_close(lo1, g["c4_ab_lower_1step"], "one-step lower")
    assert_close(up1, g["c4_ab_upper_1step"], "one-step upper")
    lo, up, a, b, _ = O.alpha_crown_shared(wl.layers, inp, C, steps=10, lr=0.1, splits=splits, optimize_beta=True)
    assert_close(lo, g["c4_ab_lower"], "lower")
    assert_close(up, g["c4_ab_upper"], "upper")
    for r, n in enumerate(wl.relu_names):
        ref_b = torch.as_tensor(g[f"c4_ab_beta_{n}"]).reshape(-1)
        assert float(b[r].min()) >= 0.0
        assert float((b[r] - ref_b).abs().max()) <= 0.05


def test_spec_fused_ibp(golden):
    """Margins C @ logits by IBP with the spec merged into the last layer (batched-W linear)."""
    g = golden("spec_fused_ibp.npz")
    for tag in ("c1", "c3"):
        wl = W.make_workload(tag) if tag == "c1" else W.make_workload(tag, batch=8)
        assert np.allclose(workload_checksum(wl), g[f"{tag}_input_checksum"], rtol=1e-12, atol=0)
        body = wl.layers[:-1]   # ... linear, relu | last linear
        assert body[-1]["op"] == "relu" and wl.layers[-1]["op"] == "linear"
        tr = O.forward_ibp_trace(body[:-1], O.box_input(wl.lo, wl.up))
        l, u = torch.relu(tr.out[0]), torch.relu(tr.out[1])
        Wl, bl = wl.layers[-1]["W"], wl.layers[-1]["b"]
        lo, up = O.ibp_linear_batched(l, u, torch.matmul(wl.C, Wl), torch.matmul(wl.C, bl))
        assert_close(lo, g[f"{tag}_lower"], f"{tag} lower")
        assert_close(up, g[f"{tag}_upper"], f"{tag} upper")


def test_first_layer_certificate(golden):
    g = golden("first_layer_certificate.npz")
    _module, layers, _x, lo, up, cases = W.make_certificate_cases()
    assert [n for n, _ in cases] == [str(n) for n in g["names"]]
    inp = O.box_input(lo, up)
    for k, (name, row) in enumerate(cases):
        assert (row.numpy() == g["split_rows"][k]).all()
        bad, best = O.first_layer_certificate(layers[0]["W"], layers[0]["b"], inp, row)
        assert bad == bool(g["infeasible"][k]), name
        if bad:
            # the value at which the loop stopped; an early exit one step apart moves it, so compare loosely
            assert best < -1e-6 and abs(best - float(g["max_value"][k])) <= 0.5 * abs(float(g["max_value"][k])) + 1e-3, name


def test_relu_objective_influence(golden):
    g = golden("relu_influence.npz")
    for tag, batch in (("c1", 8), ("c2", 3)):
        wl = W.make_workload(tag, batch=batch)
        assert np.allclose(workload_checksum(wl), g[f"{tag}_input_checksum"], rtol=1e-12, atol=0)
        inp = O.box_input(wl.lo, wl.up)
        trace = O.forward_ibp_trace(wl.layers, inp)
        infl = []
        lo, up = O.crown_backward(wl.layers, inp, trace, wl.C, influence_out=infl)
        assert_close(lo, g[f"{tag}_lower"], "lower")
        assert_close(up, g[f"{tag}_upper"], "upper")
        assert len(infl) == len(wl.relu_names)
        for r, n in enumerate(wl.relu_names):
            assert_close(infl[r].reshape(batch, -1), g[f"{tag}_influence_{n}"], f"{tag} influence {n}")


def test_alpha_crown_on_lp_balls(golden):
    g = golden("lp_alpha.npz")
    wl = W.make_workload("c3", batch=8)
    assert np.allclose(workload_checksum(wl), g["input_checksum"], rtol=1e-12, atol=0)
    for pname, p in (("l2", 2), ("l1", 1)):
        inp = O.lp_ball(wl.x, float(g[f"{pname}_eps"]), p)
        trace = O.forward_ibp_trace(wl.layers, inp)
        a0 = O.adaptive_alpha_init(trace)
        lo1, up1, _a, _ = O.alpha_crown(wl.layers, inp, wl.C, steps=1, lr=0.1, alpha0=a0, trace=trace)
        assert_close(lo1, g[f"{pname}_lower_1"], f"{pname} one-step lower")
        assert_close(up1, g[f"{pname}_upper_1"], f"{pname} one-step upper")
        lo, up, _a, _ = O.alpha_crown(wl.layers, inp, wl.C, steps=10, lr=0.1, alpha0=a0, trace=trace)
        assert_close(lo, g[f"{pname}_lower_10"], f"{pname} lower")
        assert_close(up, g[f"{pname}_upper_10"], f"{pname} upper")


def test_alpha_crown_on_a_conv_chain(golden):
    g = golden("conv_alpha.npz")
    wl = W.make_workload("c2", batch=4)
    assert np.allclose(workload_checksum(wl), g["input_checksum"], rtol=1e-12, atol=0)
    inp = O.box_input(wl.lo, wl.up)
    trace = O.forward_ibp_trace(wl.layers, inp)
    a0 = O.adaptive_alpha_init(trace)
    for steps, rtol in ((1, 3e-5), (6, 3e-4)):
        lo, up, _a, _ = O.alpha_crown(wl.layers, inp, wl.C, steps=steps, lr=0.1, alpha0=a0, trace=trace)
        assert_close(lo, g[f"per_domain_lower_{steps}"], f"per-domain lower {steps}", rtol=rtol)
        assert_close(up, g[f"per_domain_upper_{steps}"], f"per-domain upper {steps}", rtol=rtol)
        lo, up, _a, _ = O.alpha_crown_shared(wl.layers, inp, wl.C, steps=steps, lr=0.1, trace=trace)
        assert_close(lo, g[f"shared_lower_{steps}"], f"shared lower {steps}", rtol=rtol)
        assert_close(up, g[f"shared_upper_{steps}"], f"shared upper {steps}", rtol=rtol)


def test_min_and_softmin_spec_reductions(golden):
    """`run_alpha_beta_crown_mlp(spec_reduce="min" | "softmin")` of the reference (alpha_beta_crown.py:535-612, 787-818)."""
    g = golden("spec_reduce.npz")
    for cfg in ("c1", "c3"):
        wl = W.make_workload(cfg, batch=8)
        inp = O.box_input(wl.lo, wl.up)
        trace = O.forward_ibp_trace(wl.layers, inp)
        a0 = O.adaptive_alpha_init(trace)
        for red in ("min", "softmin"):
            for k in (1, 3, 10):
                lo, up, _a, _t = O.alpha_crown(wl.layers, inp, wl.C, steps=k, lr=0.1, alpha0=a0, trace=trace, spec_reduce=red,
                                               soft_tau=float(g[f"{cfg}_tau"]))
                assert_close(lo, g[f"{cfg}_{red}_lower_{k}"], f"{cfg} {red} lower after {k}")
                assert_close(up, g[f"{cfg}_{red}_upper_{k}"], f"{cfg} {red} upper after {k}")


OBJECTIVE_CASES = (("upper", "mean"), ("gap", "mean"), ("both", "mean"), ("upper", "min"), ("gap", "min"), ("both", "softmin"), ("gap", "softmin"))


def test_upper_gap_both_objectives(golden):
    """`run_alpha_beta_crown_mlp(objective="upper" | "gap" | "both")` of the reference (alpha_beta_crown.py:535-612, 807-818),
    lb_weight 1.0 and ub_weight 0.5."""
    g = golden("objectives.npz")
    for cfg in ("c1", "c3"):
        wl = W.make_workload(cfg, batch=8)
        inp = O.box_input(wl.lo, wl.up)
        trace = O.forward_ibp_trace(wl.layers, inp)
        a0 = O.adaptive_alpha_init(trace)
        for obj, red in OBJECTIVE_CASES:
            for k in (1, 3, 10):
                lo, up, _a, _t = O.alpha_crown(wl.layers, inp, wl.C, steps=k, lr=0.1, alpha0=a0, trace=trace, spec_reduce=red,
                                               soft_tau=float(g[f"{cfg}_tau"]), objective=obj, lb_weight=1.0, ub_weight=0.5)
                assert_close(lo, g[f"{cfg}_{obj}_{red}_lower_{k}"], f"{cfg} {obj}/{red} lower after {k}")
                assert_close(up, g[f"{cfg}_{obj}_{red}_upper_{k}"], f"{cfg} {obj}/{red} upper after {k}")


def _conv_beta_splits(g, wl):
    shapes = {"h1": (16, 14, 14), "h2": (32, 7, 7), "h3": (100,)}
    return [torch.from_numpy(np.asarray(g[f"split_{n}"])).to(torch.int8).reshape((4,) + shapes[n]) for n in wl.relu_names]


def test_alpha_beta_crown_on_a_conv_chain(golden):
    """`run_alpha_beta_crown_mlp(relu_split_state=...)` of the reference on the CNN c2: beta parameters on conv ReLUs
    (alpha_beta_crown.py:615-640 with the conv backward step crown_ibp.py:1106-1173)."""
    g = golden("conv_beta.npz")
    wl = W.make_workload("c2", batch=4)
    assert np.allclose(workload_checksum(wl), g["input_checksum"], rtol=1e-12, atol=0)
    assert list(wl.relu_names) == ["h1", "h2", "h3"]
    splits = _conv_beta_splits(g, wl)
    inp = O.box_input(wl.lo, wl.up)
    trace = O.forward_ibp_trace(wl.layers, inp, splits=splits)
    a0 = O.adaptive_alpha_init(trace)
    for steps in (1, 3, 8):
        lo, up, _a, beta, _t = O.alpha_crown(wl.layers, inp, wl.C, steps=steps, lr=0.1, alpha0=a0, trace=trace, splits=splits,
                                             optimize_beta=True, return_beta=True)
        assert_close(lo, g[f"per_domain_lower_{steps}"], f"per-domain lower {steps}")
        assert_close(up, g[f"per_domain_upper_{steps}"], f"per-domain upper {steps}")
        for n, b in zip(wl.relu_names, beta):
            assert_close(b.reshape(4, -1), g[f"per_domain_beta_{n}_{steps}"], f"beta {n} after {steps}", atol=1e-5)
    lo, up, _a, _b, _t = O.alpha_crown_shared(wl.layers, inp, wl.C, steps=3, lr=0.1, trace=trace, splits=splits, optimize_beta=True)
    assert_close(lo, g["shared_lower_3"], "shared lower 3")
    assert_close(up, g["shared_upper_3"], "shared upper 3")


def test_first_layer_certificate_over_a_conv_first_layer(golden):
    """The conv2d branch of the reference's half-space collection (alpha_beta_crown.py:325-387)."""
    g = golden("conv_certificate.npz")
    _module, layers, _x, lo, up, cases = W.make_conv_certificate_cases()
    assert [n for n, _ in cases] == [str(n) for n in g["names"]]
    conv = layers[0]
    Wd, bd = O.conv2d_dense_rows(conv["W"], conv["b"], conv["stride"], conv["padding"], (1, 6, 6), (4, 6, 6))
    inp = O.box_input(lo.reshape(1, -1), up.reshape(1, -1))
    for k, (name, row) in enumerate(cases):
        assert (row.numpy() == g["split_rows"][k]).all()
        bad, best = O.first_layer_certificate(Wd, bd, inp, row)
        assert bad == bool(g["infeasible"][k]), name
        if bad:
            assert best < -1e-6 and abs(best - float(g["max_value"][k])) <= 0.5 * abs(float(g["max_value"][k])) + 1e-3, name


@pytest.mark.parametrize("kind", ["linear", "conv"])
def test_first_layer_certificate_over_two_input_branches(golden, kind):
    """Half-spaces collected from two ReLUs that both sit on the input value (alpha_beta_crown.py:264-387): the oracle's
    certificate on the stacked rows of both branches against the reference (graph_certificate.npz)."""
    g = golden("graph_certificate.npz")
    module, _x, lo, up, cases = W.make_graph_certificate_cases(kind)
    assert [n for n, _ in cases] == [str(n) for n in g[f"{kind}_names"]]
    P = module.bindings["params"]
    Wd = torch.cat([P["Wa"].reshape(6, -1), P["Wb"].reshape(2, -1)])
    bd = torch.cat([P["ba"], P["bb"]])
    inp = O.box_input(lo.reshape(1, -1), up.reshape(1, -1))
    for k, (name, rows) in enumerate(cases):
        bad, best = O.first_layer_certificate(Wd, bd, inp, torch.cat([rows["ha"], rows["hb"]]))
        assert bad == bool(g[f"{kind}_infeasible"][k]), name
        if bad:
            ref = float(g[f"{kind}_max_value"][k])
            assert best < -1e-6 and abs(best - ref) <= 0.5 * abs(ref) + 1e-3, name


def _lp_certificate_problems():
    """(tag, dense first-layer rows, biases, centre, [(name, split row over those rows)]) of the three case families."""
    module, layers, x, _lo, _up, cases = W.make_certificate_cases()
    yield "mlp", layers[0]["W"], layers[0]["b"], x, cases
    _module, layers, x, _lo, _up, cases = W.make_conv_certificate_cases()
    conv = layers[0]
    Wd, bd = O.conv2d_dense_rows(conv["W"], conv["b"], conv["stride"], conv["padding"], (1, 6, 6), (4, 6, 6))
    yield "cnn", Wd, bd, x, cases
    module, x, _lo, _up, cases = W.make_graph_certificate_cases("linear")
    P = module.bindings["params"]
    yield "graph", torch.cat([P["Wa"], P["Wb"]]), torch.cat([P["ba"], P["bb"]]), x, [(n, torch.cat([r["ha"], r["hb"]])) for n, r in cases]


def test_first_layer_certificate_on_lp_balls(golden):
    """The certificate's maximum over an L2 / L1 ball is a.centre + eps * dual norm (alpha_beta_crown.py:439-441, 476-478
    call the perturbation's concretize_affine); MLP, Conv2d first layer and two-branch graph cases (lp_certificate.npz)."""
    g = golden("lp_certificate.npz")
    for tag, Wd, bd, x, cases in _lp_certificate_problems():
        assert [n for n, _ in cases] == [str(n) for n in g[f"{tag}_names"]]
        for pname, p in (("l2", 2), ("l1", 1)):
            inp = O.lp_ball(x.reshape(1, -1), float(g[f"{tag}_{pname}_eps"]), p)
            for k, (name, row) in enumerate(cases):
                bad, best = O.first_layer_certificate(Wd, bd, inp, row)
                assert bad == bool(g[f"{tag}_{pname}_infeasible"][k]), (tag, pname, name)
                if bad:
                    ref = float(g[f"{tag}_{pname}_max_value"][k])
                    assert best < -1e-6 and abs(best - ref) <= 0.5 * abs(ref) + 1e-3, (tag, pname, name)


GRAPH_NAMES = ["residual_s1", "residual_s2", "fanout_mlp", "mini_resnet", "concat_cnn", "concat_mlp"]


@pytest.mark.parametrize("name", GRAPH_NAMES)
def test_graph_oracle_crown_and_alpha_beta(golden, name):
    """oracle/graph_oracle.py against the reference on the non-chain graphs: CROWN-IBP (graph_cases.npz), the per-domain
    alpha loop and the alpha-beta loop with splits (graph_alpha.npz)."""
    from oracle import graph_oracle as GO

    gc, ga = golden("graph_cases.npz"), golden("graph_alpha.npz")
    module, _x, lo, up, C = W.make_graph_cases()[name]
    B = lo.shape[0]
    env, relu_pre = GO.forward_ibp_graph(module, lo, up)
    out_l, out_u = env["out"]
    assert_close(out_l, gc[f"{name}_ibp_lower"], "ibp lower")
    assert_close(out_u, gc[f"{name}_ibp_upper"], "ibp upper")
    n_out = out_l.reshape(B, -1).shape[1]
    y_mid = GO.concrete_forward_graph(module, (lo + up) / 2)   # the sampler of the soundness tests: inside the interval bounds
    assert bool((y_mid >= out_l - 1e-5).all()) and bool((y_mid <= out_u + 1e-5).all())
    Cb = torch.eye(n_out).unsqueeze(0).expand(B, -1, -1) if C is None else (C if C.dim() == 3 else C.unsqueeze(0).expand(B, -1, -1))
    lower, upper = GO.crown_backward_graph(module, env, relu_pre, Cb, lo, up)
    assert_close(lower, gc[f"{name}_crown_lower"].reshape(B, -1), "crown lower")
    assert_close(upper, gc[f"{name}_crown_upper"].reshape(B, -1), "crown upper")
    a0 = GO.adaptive_alpha_init_graph(relu_pre)
    for steps in (1, 4):
        lo_a, up_a, _a, _b = GO.alpha_crown_graph(module, lo, up, Cb, steps=steps, lr=0.1, alpha0=a0)
        assert_close(lo_a, ga[f"{name}_alpha_lower_{steps}"].reshape(B, -1), f"alpha lower after {steps}")
        assert_close(up_a, ga[f"{name}_alpha_upper_{steps}"].reshape(B, -1), f"alpha upper after {steps}")
    splits = {x: torch.from_numpy(np.asarray(ga[f"{name}_split_{x}"])).to(torch.int8) for x in relu_pre}
    _env, pre_split = GO.forward_ibp_graph(module, lo, up, splits=splits)
    a1 = GO.adaptive_alpha_init_graph(pre_split)
    lo_b, up_b, _a, beta = GO.alpha_crown_graph(module, lo, up, Cb, steps=3, lr=0.1, alpha0=a1, splits=splits, optimize_beta=True)
    assert_close(lo_b, ga[f"{name}_beta_lower_3"].reshape(B, -1), "alpha-beta lower after 3")
    assert_close(up_b, ga[f"{name}_beta_upper_3"].reshape(B, -1), "alpha-beta upper after 3")
    for x, b in beta.items():
        assert_close(b, ga[f"{name}_beta_{x}_3"], f"beta {x} after 3", atol=1e-5)


def test_beta_with_min_and_softmin_reductions(golden):
    """beta parameters together with the min / softmin reductions of the lower objective (alpha_beta_crown.py:763-805):
    the oracles against the reference on c4 subdomains, the CNN c2 and two non-chain graphs (beta_reduce.npz)."""
    from oracle import graph_oracle as GO

    g = golden("beta_reduce.npz")
    tau = float(g["c4_tau"])
    for D, steps in ((8, (1, 3, 6)), (40, (3,))):
        wl = W.make_workload("c4")
        root = O.forward_ibp_trace(wl.layers, O.box_input(wl.lo, wl.up))
        splits = W.make_split_domains(wl, root.pre, n_domains=D)
        inp = O.box_input(wl.lo.expand(D, -1).contiguous(), wl.up.expand(D, -1).contiguous())
        tr = O.forward_ibp_trace(wl.layers, inp, splits=splits)
        a0 = O.adaptive_alpha_init(tr)
        C = wl.C.expand(D, -1, -1).contiguous()
        for red in ("min", "softmin"):
            for k in steps:
                lo, up, _a, beta, _t = O.alpha_crown(wl.layers, inp, C, steps=k, lr=0.1, alpha0=a0, splits=splits, trace=tr, optimize_beta=True,
                                                     return_beta=True, spec_reduce=red, soft_tau=tau)
                assert_close(lo, g[f"c4_{D}_{red}_lower_{k}"], f"c4 {D} domains {red} lower after {k}")
                assert_close(up, g[f"c4_{D}_{red}_upper_{k}"], f"c4 {D} domains {red} upper after {k}")
                for n, b in zip(wl.relu_names, beta):
                    assert_close(b, g[f"c4_{D}_{red}_beta_{n}_{k}"], f"beta {n}", atol=1e-5)
            if D == 8:
                lo, up, _a, beta, _t = O.alpha_crown_shared(wl.layers, inp, C, steps=4, lr=0.1, splits=splits, trace=tr, optimize_beta=True,
                                                            spec_reduce=red, soft_tau=tau)
                assert_close(lo, g[f"c4_8_shared_{red}_lower_4"], f"c4 shared {red} lower")
                assert_close(up, g[f"c4_8_shared_{red}_upper_4"], f"c4 shared {red} upper")
                for n, b in zip(wl.relu_names, beta):
                    assert_close(b, g[f"c4_8_shared_{red}_beta_{n}_4"], f"shared beta {n}", atol=1e-5)
    cb = golden("conv_beta.npz")
    wl = W.make_workload("c2", batch=4)
    inp = O.box_input(wl.lo, wl.up)
    splits = [torch.from_numpy(np.asarray(cb[f"split_{n}"])).to(torch.int8).reshape(4, -1) for n in wl.relu_names]
    tr = O.forward_ibp_trace(wl.layers, inp, splits=splits)
    a0 = O.adaptive_alpha_init(tr)
    for red in ("min", "softmin"):
        lo, up, _a, beta, _t = O.alpha_crown(wl.layers, inp, wl.C, steps=4, lr=0.1, alpha0=a0, splits=splits, trace=tr, optimize_beta=True,
                                             return_beta=True, spec_reduce=red, soft_tau=float(g["c2_tau"]))
        assert_close(lo, g[f"c2_{red}_lower_4"], f"c2 {red} lower")
        assert_close(up, g[f"c2_{red}_upper_4"], f"c2 {red} upper")
        for n, b in zip(wl.relu_names, beta):
            assert_close(b.reshape(4, -1), g[f"c2_{red}_beta_{n}_4"], f"c2 beta {n}", atol=1e-5)
    ga = golden("graph_alpha.npz")
    for name in ("fanout_mlp", "residual_s1"):
        module, _x, lo, up, C = W.make_graph_cases()[name]
        B = lo.shape[0]
        env, relu_pre = GO.forward_ibp_graph(module, lo, up)
        n_out = env["out"][0].reshape(B, -1).shape[1]
        Cb = torch.eye(n_out).unsqueeze(0).expand(B, -1, -1) if C is None else (C if C.dim() == 3 else C.unsqueeze(0).expand(B, -1, -1))
        splits = {x: torch.from_numpy(np.asarray(ga[f"{name}_split_{x}"])).to(torch.int8) for x in relu_pre}
        _env, pre_split = GO.forward_ibp_graph(module, lo, up, splits=splits)
        a1 = GO.adaptive_alpha_init_graph(pre_split)
        lo_b, up_b, _a, beta = GO.alpha_crown_graph(module, lo, up, Cb, steps=3, lr=0.1, alpha0=a1, splits=splits, optimize_beta=True,
                                                    spec_reduce="softmin", soft_tau=float(g["graph_tau"]))
        assert_close(lo_b, g[f"{name}_softmin_lower_3"].reshape(B, -1), f"{name} softmin lower")
        assert_close(up_b, g[f"{name}_softmin_upper_3"].reshape(B, -1), f"{name} softmin upper")
        for x, b in beta.items():
            assert_close(b, g[f"{name}_softmin_beta_{x}_3"], f"{name} beta {x}", atol=1e-5)
        lo_b, up_b, _a, beta = GO.alpha_crown_graph(module, lo, up, Cb, steps=3, lr=0.1, splits=splits, optimize_beta=True, spec_reduce="min",
                                                    per_batch_params=False)
        assert_close(lo_b, g[f"{name}_shared_min_lower_3"].reshape(B, -1), f"{name} shared min lower")
        assert_close(up_b, g[f"{name}_shared_min_upper_3"].reshape(B, -1), f"{name} shared min upper")
        for x, b in beta.items():
            assert_close(b.reshape(-1), g[f"{name}_shared_min_beta_{x}_3"], f"{name} shared beta {x}", atol=1e-5)


@pytest.mark.parametrize("name", ["fanout_mlp", "concat_mlp", "residual_s1"])
def test_graph_oracle_on_lp_balls(golden, name):
    """L2 / L1 ball inputs on non-chain graphs (graph_lp.npz): IBP of the output, CROWN-IBP, the per-domain alpha loop."""
    from oracle import graph_oracle as GO

    g = golden("graph_lp.npz")
    module, x, _lo, _up, C = W.make_graph_cases()[name]
    B = x.shape[0]
    for pname, p in (("l2", 2), ("l1", 1)):
        eps = float(g[f"{name}_{pname}_eps"])
        lo, up, ball = x - eps, x + eps, (p, eps)
        env, relu_pre = GO.forward_ibp_graph(module, lo, up, ball=ball)
        assert_close(env["out"][0], g[f"{name}_{pname}_ibp_lower"], f"{pname} ibp lower")
        assert_close(env["out"][1], g[f"{name}_{pname}_ibp_upper"], f"{pname} ibp upper")
        n_out = env["out"][0].reshape(B, -1).shape[1]
        Cb = torch.eye(n_out).unsqueeze(0).expand(B, -1, -1) if C is None else (C if C.dim() == 3 else C.unsqueeze(0).expand(B, -1, -1))
        lower, upper = GO.crown_backward_graph(module, env, relu_pre, Cb, lo, up, ball=ball)
        assert_close(lower, g[f"{name}_{pname}_crown_lower"].reshape(B, -1), f"{pname} crown lower")
        assert_close(upper, g[f"{name}_{pname}_crown_upper"].reshape(B, -1), f"{pname} crown upper")
        a0 = GO.adaptive_alpha_init_graph(relu_pre)
        lo_a, up_a, _a, _b = GO.alpha_crown_graph(module, lo, up, Cb, steps=3, lr=0.1, alpha0=a0, ball=ball)
        assert_close(lo_a, g[f"{name}_{pname}_alpha_lower_3"].reshape(B, -1), f"{pname} alpha lower after 3")
        assert_close(up_a, g[f"{name}_{pname}_alpha_upper_3"].reshape(B, -1), f"{pname} alpha upper after 3")


@pytest.mark.parametrize("name", ["fanout_mlp", "mini_resnet", "concat_cnn"])
def test_graph_oracle_trace_level_functions(golden, name):
    """`_forward_ibp_trace_mlp(relu_pre_constraints=...)`, `run_crown_ibp_mlp_from_forward_trace` and the ReLU-influence
    variant on non-chain graphs (graph_trace.npz)."""
    from oracle import graph_oracle as GO

    g = golden("graph_trace.npz")
    module, _x, lo, up, C = W.make_graph_cases()[name]
    B = lo.shape[0]
    env, relu_pre = GO.forward_ibp_graph(module, lo, up)
    n_out = env["out"][0].reshape(B, -1).shape[1]
    Cb = torch.eye(n_out).unsqueeze(0).expand(B, -1, -1) if C is None else (C if C.dim() == 3 else C.unsqueeze(0).expand(B, -1, -1))
    cons = {x: (l + 0.1 * (u - l), u - 0.1 * (u - l)) for x, (l, u) in relu_pre.items()}
    env2, pre2 = GO.forward_ibp_graph(module, lo, up, constraints=cons)
    for x, (l, u) in pre2.items():
        assert_close(l.reshape(B, -1), g[f"{name}_cons_pre_{x}_lower"], f"constrained pre {x} lower")
        assert_close(u.reshape(B, -1), g[f"{name}_cons_pre_{x}_upper"], f"constrained pre {x} upper")
    assert_close(env2["out"][0], g[f"{name}_cons_out_lower"], "constrained ibp lower")
    assert_close(env2["out"][1], g[f"{name}_cons_out_upper"], "constrained ibp upper")
    lower, upper = GO.crown_backward_graph(module, env2, pre2, Cb, lo, up)
    assert_close(lower, g[f"{name}_cons_crown_lower"].reshape(B, -1), "crown on the constrained trace, lower")
    assert_close(upper, g[f"{name}_cons_crown_upper"].reshape(B, -1), "crown on the constrained trace, upper")
    infl = {}
    lower, upper = GO.crown_backward_graph(module, env, relu_pre, Cb, lo, up, influence_out=infl)
    assert_close(lower, g[f"{name}_infl_lower"].reshape(B, -1), "influence call lower")
    assert set(infl) == set(relu_pre)
    for x, v in infl.items():
        assert_close(v.reshape(B, -1), g[f"{name}_infl_{x}"], f"influence {x}")


def test_add_coefficients_on_both_sides(golden):
    """`relu_pre_add_coeff_u` / `_l` (crown_ibp.py:1270-1296) on the MLP c1 and on the fan-out graph (add_coeff.npz)."""
    from oracle import graph_oracle as GO

    g = golden("add_coeff.npz")
    wl = W.make_workload("c1", batch=8)
    inp = O.box_input(wl.lo, wl.up)
    tr = O.forward_ibp_trace(wl.layers, inp)
    rows = lambda key, n: torch.as_tensor(g[key]).reshape(-1, n).expand(8, n)  # noqa: E731
    widths = [l.shape[1] for l, _u in tr.pre]
    add_u = [rows(f"c1_add_u_{n}", w) for n, w in zip(wl.relu_names, widths)]
    add_l = [rows(f"c1_add_l_{n}", w) for n, w in zip(wl.relu_names, widths)]
    lo, up = O.crown_backward(wl.layers, inp, tr, wl.C, add_l=add_l, add_u=add_u)
    assert_close(lo, g["c1_lower"], "c1 lower with both terms")
    assert_close(up, g["c1_upper"], "c1 upper with both terms")
    lo, up = O.crown_backward(wl.layers, inp, tr, wl.C, add_u=add_u)
    assert_close(lo, g["c1_u_only_lower"], "c1 lower with the upper term only")
    assert_close(up, g["c1_u_only_upper"], "c1 upper with the upper term only")
    module, _x, blo, bup, C = W.make_graph_cases()["fanout_mlp"]
    B = blo.shape[0]
    env, relu_pre = GO.forward_ibp_graph(module, blo, bup)
    gu = {x: torch.as_tensor(g[f"fanout_add_u_{x}"]).reshape(B, -1) for x in relu_pre}
    gl = {x: torch.as_tensor(g[f"fanout_add_l_{x}"]).reshape(B, -1) for x in relu_pre}
    lo, up = GO.crown_backward_graph(module, env, relu_pre, C, blo, bup, add_l=gl, add_u=gu)
    assert_close(lo, g["fanout_lower"], "fan-out graph lower")
    assert_close(up, g["fanout_upper"], "fan-out graph upper")


@pytest.mark.parametrize("name", ["grouped_dilated_chain", "depthwise_residual"])
def test_grouped_and_dilated_convolutions(golden, name):
    """Conv2d with groups and dilation (domains/interval.py:57-74, crown_ibp.py:1127-1170): IBP, CROWN-IBP and the
    per-domain alpha loop of the reference (grouped_dilated.npz) against the graph oracle, which walks chains too."""
    from oracle import graph_oracle as GO

    g = golden("grouped_dilated.npz")
    module, _x, lo, up, _C = W.make_grouped_dilated_cases()[name]
    B = lo.shape[0]
    env, relu_pre = GO.forward_ibp_graph(module, lo, up)
    assert_close(env["out"][0], g[f"{name}_ibp_lower"], "ibp lower")
    assert_close(env["out"][1], g[f"{name}_ibp_upper"], "ibp upper")
    n_out = env["out"][0].reshape(B, -1).shape[1]
    Cb = torch.eye(n_out).unsqueeze(0).expand(B, -1, -1)
    lower, upper = GO.crown_backward_graph(module, env, relu_pre, Cb, lo, up)
    assert_close(lower, g[f"{name}_crown_lower"].reshape(B, -1), "crown lower")
    assert_close(upper, g[f"{name}_crown_upper"].reshape(B, -1), "crown upper")
    lo_a, up_a, _a, _b = GO.alpha_crown_graph(module, lo, up, Cb, steps=3, lr=0.1, alpha0=GO.adaptive_alpha_init_graph(relu_pre))
    assert_close(lo_a, g[f"{name}_alpha_lower_3"].reshape(B, -1), "alpha lower after 3")
    assert_close(up_a, g[f"{name}_alpha_upper_3"].reshape(B, -1), "alpha upper after 3")
    # the dense equivalent the CUDA path uses gives the same convolution
    from boundflow_b200.network import dense_conv_weight

    for op in module.get_entry_task().ops:
        if op.op_type == "conv2d":
            Wg = module.bindings["params"][op.inputs[1]]
            x = torch.randn(2, Wg.shape[1] * int(op.attrs["groups"]), 9, 9)
            ref = torch.nn.functional.conv2d(x, Wg, None, op.attrs["stride"], op.attrs["padding"], op.attrs["dilation"], op.attrs["groups"])
            got = torch.nn.functional.conv2d(x, dense_conv_weight(Wg, op.attrs), None, op.attrs["stride"], op.attrs["padding"])
            assert_close(got, ref, f"dense equivalent of {op.name}", atol=1e-5)


@pytest.mark.parametrize("name", ["mul_gate", "permute_cnn", "spec_linear"])
def test_executor_only_ops(golden, name):
    """The op types that only the interval executors handle (mul, permute, spec_linear; task_executor.py:184-350), on a box
    and on an L2 ball, against `PythonTaskExecutor.run_ibp` (executor_ops.npz)."""
    from oracle import graph_oracle as GO

    g = golden("executor_ops.npz")
    module, x, lo, up = W.make_executor_op_cases()[name]
    env, _pre = GO.forward_ibp_graph(module, lo, up)
    assert_close(env["out"][0], g[f"{name}_box_lower"], "box lower")
    assert_close(env["out"][1], g[f"{name}_box_upper"], "box upper")
    if x.dim() == 2:
        env, _pre = GO.forward_ibp_graph(module, x - 0.2, x + 0.2, ball=(2, 0.2))
        assert_close(env["out"][0], g[f"{name}_l2_lower"], "L2 ball lower")
        assert_close(env["out"][1], g[f"{name}_l2_upper"], "L2 ball upper")


GRAPH_OBJECTIVE_CASES = (("upper", "mean"), ("gap", "min"), ("both", "softmin"), ("lower", "softmin"), ("lower", "min"))
GRAPH_SHARED_CASES = (("lower", "mean"), ("gap", "mean"), ("both", "min"), ("upper", "softmin"))


@pytest.mark.parametrize("name", GRAPH_NAMES)
def test_graph_oracle_objectives_and_shared_mode(golden, name):
    """oracle/graph_oracle.py against the reference on the non-chain graphs (graph_objectives.npz): the other
    objectives and reductions with per-domain parameters, the shared-parameter mode, and shared alpha + beta."""
    from oracle import graph_oracle as GO

    g, ga = golden("graph_objectives.npz"), golden("graph_alpha.npz")
    module, _x, lo, up, C = W.make_graph_cases()[name]
    B = lo.shape[0]
    env, relu_pre = GO.forward_ibp_graph(module, lo, up)
    n_out = env["out"][0].reshape(B, -1).shape[1]
    Cb = torch.eye(n_out).unsqueeze(0).expand(B, -1, -1) if C is None else (C if C.dim() == 3 else C.unsqueeze(0).expand(B, -1, -1))
    a0 = GO.adaptive_alpha_init_graph(relu_pre)
    kw = {"soft_tau": float(g["tau"]), "lb_weight": 1.0, "ub_weight": 0.5}
    for obj, red in GRAPH_OBJECTIVE_CASES:
        for steps in (1, 4):
            lo_a, up_a, _a, _b = GO.alpha_crown_graph(module, lo, up, Cb, steps=steps, lr=0.1, alpha0=a0, objective=obj, spec_reduce=red, **kw)
            assert_close(lo_a, g[f"{name}_{obj}_{red}_lower_{steps}"].reshape(B, -1), f"{obj}/{red} lower after {steps}")
            assert_close(up_a, g[f"{name}_{obj}_{red}_upper_{steps}"].reshape(B, -1), f"{obj}/{red} upper after {steps}")
    for obj, red in GRAPH_SHARED_CASES:
        lo_a, up_a, _a, _b = GO.alpha_crown_graph(module, lo, up, Cb, steps=4, lr=0.1, objective=obj, spec_reduce=red, per_batch_params=False, **kw)
        assert_close(lo_a, g[f"{name}_shared_{obj}_{red}_lower_4"].reshape(B, -1), f"shared {obj}/{red} lower")
        assert_close(up_a, g[f"{name}_shared_{obj}_{red}_upper_4"].reshape(B, -1), f"shared {obj}/{red} upper")
    # `run_alpha_crown_mlp` is the shared mode with lower / mean
    lo_a, up_a, al, _b = GO.alpha_crown_graph(module, lo, up, Cb, steps=4, lr=0.1, per_batch_params=False)
    assert_close(lo_a, g[f"{name}_alpha_crown_lower_4"].reshape(B, -1), "run_alpha_crown_mlp lower")
    assert_close(up_a, g[f"{name}_alpha_crown_upper_4"].reshape(B, -1), "run_alpha_crown_mlp upper")
    for x, a in al.items():
        assert_close(a.reshape(-1), g[f"{name}_alpha_crown_alpha_{x}"], f"shared alpha {x}", atol=1e-5)
    if f"{name}_shared_beta_lower_3" in g:
        splits = {x: torch.from_numpy(np.asarray(ga[f"{name}_split_{x}"])).to(torch.int8) for x in relu_pre}
        lo_b, up_b, _a, beta = GO.alpha_crown_graph(module, lo, up, Cb, steps=3, lr=0.1, splits=splits, optimize_beta=True, per_batch_params=False)
        assert_close(lo_b, g[f"{name}_shared_beta_lower_3"].reshape(B, -1), "shared alpha-beta lower after 3")
        assert_close(up_b, g[f"{name}_shared_beta_upper_3"].reshape(B, -1), "shared alpha-beta upper after 3")
        for x, b in beta.items():
            assert_close(b.reshape(-1), g[f"{name}_shared_beta_{x}_3"], f"shared beta {x} after 3", atol=1e-5)


SHARED_OBJECTIVE_CASES = (("lower", "min"), ("lower", "softmin"), ("upper", "mean"), ("gap", "min"), ("both", "softmin"), ("both", "mean"))


def test_shared_alpha_objectives_and_reductions(golden):
    """`run_alpha_crown_mlp(objective=..., spec_reduce=...)` of the reference (alpha_crown.py:67-134, 137-261)."""
    g = golden("shared_objectives.npz")
    for cfg, batch in (("c1", 8), ("c2", 4)):
        wl = W.make_workload(cfg, batch=batch)
        inp = O.box_input(wl.lo, wl.up)
        trace = O.forward_ibp_trace(wl.layers, inp)
        for obj, red in SHARED_OBJECTIVE_CASES:
            for k in (1, 6):
                lo, up, _a, _t = O.alpha_crown_shared(wl.layers, inp, wl.C, steps=k, lr=0.1, trace=trace, objective=obj, spec_reduce=red,
                                                      soft_tau=float(g[f"{cfg}_tau"]), lb_weight=1.0, ub_weight=0.5)
                assert_close(lo, g[f"{cfg}_{obj}_{red}_lower_{k}"], f"{cfg} shared {obj}/{red} lower after {k}")
                assert_close(up, g[f"{cfg}_{obj}_{red}_upper_{k}"], f"{cfg} shared {obj}/{red} upper after {k}")
