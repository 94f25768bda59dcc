"""First-layer infeasibility certificate per domain (`bf_first_layer_certificate`)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available()
    from boundflow_b200.csrc import build

    build.build()
    return torch.device("cuda", 0)


def test_cases_match_reference_golden_and_oracle(dev, golden):
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import first_layer_certificate
    from boundflow_b200.ir import InputSpec
    from oracle import crown_oracle as O

    g = golden("first_layer_certificate.npz")
    module, layers, _x, lo, up, cases = W.make_certificate_cases()
    D = len(cases)
    spec = InputSpec.box(value_name="input", lower=lo.expand(D, -1).contiguous().to(dev), upper=up.expand(D, -1).contiguous().to(dev))
    rows = torch.stack([r for _n, r in cases]).to(dev)
    flags, best, count = first_layer_certificate(module, spec, {"h1": rows})
    flags, best, count = flags.cpu(), best.cpu(), count.cpu()
    inp = O.box_input(lo, up)
    for k, (name, row) in enumerate(cases):
        assert int(count[k]) == int((row != 0).sum()), name
        assert int(flags[k]) == int(bool(g["infeasible"][k])), name
        o_bad, o_best = O.first_layer_certificate(layers[0]["W"], layers[0]["b"], inp, row)
        assert bool(flags[k]) == o_bad, name
        if o_best is not None:
            # same trajectory as the oracle up to rounding; an exit one step apart moves the value slightly
            assert abs(float(best[k]) - o_best) <= 0.25 * abs(o_best) + 1e-4, (name, float(best[k]), o_best)


def test_shared_row_many_halfspaces_and_single_node_precheck(dev):
    from boundflow_b200 import _lib
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import first_layer_certificate, run_alpha_beta_crown_mlp
    from boundflow_b200.ir import InputSpec

    module, _layers, _x, lo, up, cases = W.make_certificate_cases()
    case = dict(cases)
    spec3 = InputSpec.box(value_name="input", lower=lo.expand(3, -1).contiguous().to(dev), upper=up.expand(3, -1).contiguous().to(dev))
    # one split row shared by all domains (stride 0)
    flags, _b, _c = first_layer_certificate(module, spec3, {"h1": case["pair_contradiction_needs_steps"].to(dev)})
    assert flags.cpu().tolist() == [1, 1, 1]
    assert int(_lib.load().bf_first_layer_certificate_max_halfspaces()) == 16
    # no split on the first ReLU: nothing to test
    wide = torch.zeros(16, dtype=torch.int8)
    flags, _b, cnt = first_layer_certificate(module, spec3, {"h1": wide.to(dev)})
    assert flags.cpu().tolist() == [0, 0, 0] and cnt.cpu().tolist() == [0, 0, 0]
    # the single-node alpha-beta call returns the reference's "infeasible" result shape
    spec1 = InputSpec.box(value_name="input", lower=lo.to(dev), upper=up.to(dev))
    bounds, a, b, stats = run_alpha_beta_crown_mlp(module, spec1, relu_split_state={"h1": case["pair_contradiction_uniform_weights"].unsqueeze(0).to(dev)},
                                                   steps=2, lr=0.1, per_batch_params=True)
    assert stats.feasibility == "infeasible" and tuple(bounds.lower.shape) == (1, 1) and not a.alpha_by_relu_input
    bounds, a, b, stats = run_alpha_beta_crown_mlp(module, spec1, relu_split_state={"h1": case["feasible_pair"].unsqueeze(0).to(dev)},
                                                   steps=2, lr=0.1, per_batch_params=True)
    assert stats.feasibility == "unknown" and tuple(bounds.lower.shape) == (1, 5)


def test_conv_first_layer_cases_match_reference_golden_and_oracle(dev, golden):
    """Conv2d first layer: the half-space rows of the neurons that are split somewhere in the batch come from
    `bf_conv2d_dense_rows` (checked against the oracle's dense matrix), the certificate itself from the same kernel."""
    from boundflow_b200 import _lib
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import first_layer_certificate, run_alpha_beta_crown_mlp
    from boundflow_b200.ir import InputSpec
    from oracle import crown_oracle as O

    g = golden("conv_certificate.npz")
    module, layers, _x, lo, up, cases = W.make_conv_certificate_cases()
    conv = layers[0]
    Wd, bd = O.conv2d_dense_rows(conv["W"], conv["b"], conv["stride"], conv["padding"], (1, 6, 6), (4, 6, 6))
    # the row kernel on every neuron plus one index outside the layer (zero row)
    lib = _lib.load()
    idx = torch.arange(145, dtype=torch.int32, device=dev)
    rows = torch.full((145, 36), float("nan"), device=dev)
    rb = torch.full((145,), float("nan"), device=dev)
    Wc, bc = conv["W"].to(dev).contiguous(), conv["b"].to(dev).contiguous()
    _lib.check(lib.bf_conv2d_dense_rows(Wc.data_ptr(), bc.data_ptr(), idx.data_ptr(), 145, rows.data_ptr(), rb.data_ptr(), 1, 6, 6, 4, 6, 6, 3, 3,
                                        1, 1, 1, 1, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert torch.equal(rows[:144].cpu(), Wd) and torch.equal(rb[:144].cpu(), bd)
    assert float(rows[144].abs().max()) == 0.0 and float(rb[144]) == 0.0
    D = len(cases)
    spec = InputSpec.box(value_name="input", lower=lo.expand(D, -1, -1, -1).contiguous().to(dev), upper=up.expand(D, -1, -1, -1).contiguous().to(dev))
    split = torch.stack([r for _n, r in cases]).reshape(D, 4, 6, 6).to(dev)
    flags, best, count = first_layer_certificate(module, spec, {"h1": split})
    flags, best, count = flags.cpu(), best.cpu(), count.cpu()
    inp = O.box_input(lo.reshape(1, -1), up.reshape(1, -1))
    for k, (name, row) in enumerate(cases):
        assert int(count[k]) == int((row != 0).sum()), name
        assert int(flags[k]) == int(bool(g["infeasible"][k])), name
        o_bad, o_best = O.first_layer_certificate(Wd, bd, inp, row)
        assert bool(flags[k]) == o_bad, name
        if o_best is not None:
            assert abs(float(best[k]) - o_best) <= 0.25 * abs(o_best) + 1e-4, (name, float(best[k]), o_best)
    # the single-node pre-check of the alpha-beta function on a conv first layer
    case = dict(cases)
    spec1 = InputSpec.box(value_name="input", lower=lo.to(dev), upper=up.to(dev))
    _bounds, a, _b, stats = run_alpha_beta_crown_mlp(module, spec1, relu_split_state={"h1": case["border_pixel_contradiction"].reshape(1, 4, 6, 6).to(dev)},
                                                    steps=2, lr=0.1, per_batch_params=True)
    assert stats.feasibility == "infeasible" and not a.alpha_by_relu_input
    bounds, _a, _b, stats = run_alpha_beta_crown_mlp(module, spec1, relu_split_state={"h1": case["feasible_pair"].reshape(1, 4, 6, 6).to(dev)},
                                                    steps=2, lr=0.1, per_batch_params=True)
    assert stats.feasibility == "unknown" and tuple(bounds.lower.shape) == (1, 5)


@pytest.mark.parametrize("kind", ["linear", "conv"])
def test_two_input_branches_of_a_graph_match_reference_golden_and_oracle(dev, golden, kind):
    """A graph that is not a chain: two ReLUs sit on ops that read the input value, and a contradiction may span both
    (tests/golden/graph_certificate.npz).  All cases as one batch of domains, then the single-node pre-check."""
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import first_layer_certificate, needs_graph_path, run_alpha_beta_crown_mlp
    from boundflow_b200.ir import InputSpec
    from oracle import crown_oracle as O

    g = golden("graph_certificate.npz")
    module, _x, lo, up, cases = W.make_graph_certificate_cases(kind)
    assert needs_graph_path(module)
    D = len(cases)
    rep = (D,) + (-1,) * (lo.dim() - 1)
    spec = InputSpec.box(value_name="input", lower=lo.expand(*rep).contiguous().to(dev), upper=up.expand(*rep).contiguous().to(dev))
    tail = () if kind == "linear" else (1, 1)
    split = {k: torch.stack([rows[k] for _n, rows in cases]).reshape((D, -1) + tail).to(dev) for k in ("ha", "hb")}
    flags, best, count = first_layer_certificate(module, spec, split)
    flags, best, count = flags.cpu(), best.cpu(), count.cpu()
    P = module.bindings["params"]
    Wd, bd = torch.cat([P["Wa"].reshape(6, -1), P["Wb"].reshape(2, -1)]), torch.cat([P["ba"], P["bb"]])
    inp = O.box_input(lo.reshape(1, -1), up.reshape(1, -1))
    for k, (name, rows) in enumerate(cases):
        row = torch.cat([rows["ha"], rows["hb"]])
        assert int(count[k]) == int((row != 0).sum()), name
        assert int(flags[k]) == int(bool(g[f"{kind}_infeasible"][k])), name
        o_bad, o_best = O.first_layer_certificate(Wd, bd, inp, row)
        assert bool(flags[k]) == o_bad, name
        if o_best is not None:
            assert abs(float(best[k]) - o_best) <= 0.25 * abs(o_best) + 1e-4, (name, float(best[k]), o_best)
    # one split row shared by the batch on one branch, per-domain rows on the other
    mixed = {"ha": dict(cases)["cross_branch_contradiction_needs_steps"]["ha"].to(dev), "hb": split["hb"]}
    flags2, _b, _c = first_layer_certificate(module, spec, mixed)
    want = [int(bool((rows["hb"] == 1).any())) for _n, rows in cases]   # ha[0] active contradicts either neuron of hb being active
    assert flags2.cpu().tolist() == want
    # the single-node pre-check of the alpha-beta function on a graph
    case = dict(cases)
    spec1 = InputSpec.box(value_name="input", lower=lo.to(dev), upper=up.to(dev))
    one = lambda rows: {k: v.reshape((1, -1) + tail).to(dev) for k, v in rows.items()}  # noqa: E731
    bounds, a, _b, stats = run_alpha_beta_crown_mlp(module, spec1, relu_split_state=one(case["cross_branch_contradiction_uniform_weights"]), steps=2,
                                                   lr=0.1, per_batch_params=True)
    assert stats.feasibility == "infeasible" and tuple(bounds.lower.shape) == (1, 1) and not a.alpha_by_relu_input
    bounds, a, _b, stats = run_alpha_beta_crown_mlp(module, spec1, relu_split_state=one(case["cross_branch_feasible"]), steps=2, lr=0.1,
                                                   per_batch_params=True)
    assert stats.feasibility == "unknown" and tuple(bounds.lower.shape) == (1, 3)


@pytest.mark.parametrize("pname,p", [("l2", 2), ("l1", 1)])
def test_lp_ball_inputs_match_reference_golden_and_oracle(dev, golden, pname, p):
    """L2 / L1 ball inputs (tests/golden/lp_certificate.npz): a Linear first layer, a Conv2d first layer and the two-branch
    graph, every case family as one batch of domains; then the single-node pre-check of the alpha-beta function."""
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import first_layer_certificate, run_alpha_beta_crown_mlp
    from boundflow_b200.ir import InputSpec
    from oracle import crown_oracle as O

    g = golden("lp_certificate.npz")
    mk = InputSpec.l2 if p == 2 else InputSpec.l1

    def check(tag, module, x, split, Wd, bd, rows):
        D = len(rows)
        eps = float(g[f"{tag}_{pname}_eps"])
        spec = mk(value_name="input", center=x.expand((D,) + tuple(x.shape[1:])).contiguous().to(dev), eps=eps)
        flags, best, count = first_layer_certificate(module, spec, split)
        flags, best, count = flags.cpu(), best.cpu(), count.cpu()
        inp = O.lp_ball(x.reshape(1, -1), eps, p)
        for k, (name, row) in enumerate(rows):
            assert int(count[k]) == int((row != 0).sum()), (tag, name)
            assert int(flags[k]) == int(bool(g[f"{tag}_{pname}_infeasible"][k])), (tag, name)
            o_bad, o_best = O.first_layer_certificate(Wd, bd, inp, row)
            assert bool(flags[k]) == o_bad, (tag, name)
            if o_best is not None:
                assert abs(float(best[k]) - o_best) <= 0.25 * abs(o_best) + 1e-4, (tag, name, float(best[k]), o_best)

    module, layers, x, _lo, _up, cases = W.make_certificate_cases()
    check("mlp", module, x, {"h1": torch.stack([r for _n, r in cases]).to(dev)}, layers[0]["W"], layers[0]["b"], cases)
    case = dict(cases)
    spec1 = mk(value_name="input", center=x.to(dev), eps=float(g[f"mlp_{pname}_eps"]))
    bounds, a, _b, stats = run_alpha_beta_crown_mlp(module, spec1, relu_split_state={"h1": case["pair_contradiction_uniform_weights"].unsqueeze(0).to(dev)},
                                                   steps=2, lr=0.1, per_batch_params=True)
    assert stats.feasibility == "infeasible" and tuple(bounds.lower.shape) == (1, 1) and not a.alpha_by_relu_input
    cmodule, layers, x, _lo, _up, cases = W.make_conv_certificate_cases()
    conv = layers[0]
    Wd, bd = O.conv2d_dense_rows(conv["W"], conv["b"], conv["stride"], conv["padding"], (1, 6, 6), (4, 6, 6))
    check("cnn", cmodule, x, {"h1": torch.stack([r for _n, r in cases]).reshape(len(cases), 4, 6, 6).to(dev)}, Wd, bd, cases)
    gmodule, x, _lo, _up, cases = W.make_graph_certificate_cases("linear")
    P = gmodule.bindings["params"]
    rows = [(n, torch.cat([r["ha"], r["hb"]])) for n, r in cases]
    split = {k: torch.stack([r[k] for _n, r in cases]).to(dev) for k in ("ha", "hb")}
    check("graph", gmodule, x, split, torch.cat([P["Wa"], P["Wb"]]), torch.cat([P["ba"], P["bb"]]), rows)


def test_single_node_wrapper_and_capability_query(dev):
    """`check_first_layer_infeasible_split` (one node: "infeasible" with a certificate, else "unknown" with the reason) and
    `get_crown_ibp_mlp_stats` (which modules `run_crown_ibp_mlp` takes)."""
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import check_first_layer_infeasible_split, get_crown_ibp_mlp_stats
    from boundflow_b200.ir import InputSpec

    module, _layers, _x, lo, up, cases = W.make_certificate_cases()
    case = dict(cases)
    spec1 = InputSpec.box(value_name="input", lower=lo.to(dev), upper=up.to(dev))
    st = check_first_layer_infeasible_split(module, spec1, relu_split_state={"h1": case["pair_contradiction_needs_steps"].unsqueeze(0).to(dev)})
    assert st.feasibility == "infeasible" and st.infeasible_certificate["type"] == "convex_combo_max_negative"
    assert st.infeasible_certificate["max_value"] < -1e-6 and st.infeasible_certificate["n_halfspaces"] == 2
    st = check_first_layer_infeasible_split(module, spec1, relu_split_state={"h1": case["feasible_pair"].unsqueeze(0).to(dev)})
    assert st.feasibility == "unknown" and st.infeasible_certificate is None
    st = check_first_layer_infeasible_split(module, spec1, relu_split_state={"h1": case["no_split"].unsqueeze(0).to(dev)})
    assert st.feasibility == "unknown" and "no first-layer split halfspaces" in st.reason
    spec3 = InputSpec.box(value_name="input", lower=lo.expand(3, -1).contiguous().to(dev), upper=up.expand(3, -1).contiguous().to(dev))
    st = check_first_layer_infeasible_split(module, spec3, relu_split_state={"h1": case["pair_contradiction_needs_steps"].to(dev)})
    assert st.feasibility == "unknown" and st.reason == "skip (batch!=1)"
    assert get_crown_ibp_mlp_stats(module).supported
    assert get_crown_ibp_mlp_stats(W.make_graph_cases()["mini_resnet"][0]).supported
    bad = get_crown_ibp_mlp_stats(W.make_executor_op_cases()["permute_cnn"][0])
    assert not bad.supported and "permute" in bad.reason and bad.ops_seen[2] == "permute"
