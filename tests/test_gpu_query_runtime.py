"""`CudaQueryRuntime.execute`: the `query_runtime=` hook of the reference's BaB driver."""
from types import SimpleNamespace

import pytest
import torch

from tests.helpers import assert_close

pytestmark = pytest.mark.gpu

OPTS = {"alpha_steps": 5, "alpha_lr": 0.1, "alpha_init": 0.5, "beta_init": 0.0, "objective": "lower", "spec_reduce": "mean",
        "soft_tau": 1.0, "lb_weight": 1.0, "ub_weight": 1.0}


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available()
    from boundflow_b200.csrc import build

    build.build()
    return torch.device("cuda", 0)


def _requests(dev, D, method="alpha-beta-CROWN", opts=OPTS, prefix="q"):
    from boundflow_b200 import workloads as W
    from boundflow_b200.ir import InputSpec
    from oracle import crown_oracle as O

    wl = W.make_workload("c4")
    root = O.forward_ibp_trace(wl.layers, O.box_input(wl.lo, wl.up))
    splits = W.make_split_domains(wl, root.pre, n_domains=D)
    reqs = []
    for i in range(D):
        spec = InputSpec.box(value_name="input", lower=wl.lo.to(dev), upper=wl.up.to(dev))
        payload = SimpleNamespace(input_spec=spec, linear_spec_c=wl.C[0].to(dev),
                                  split_by_relu_input={n: s[i].to(dev) for n, s in zip(wl.relu_names, splits)},
                                  warm_alpha_by_relu_input={}, warm_beta_by_relu_input={})
        query = SimpleNamespace(query_id=f"{prefix}{i}", bound_method=SimpleNamespace(value=method), execution_options=dict(opts))
        reqs.append(SimpleNamespace(query=query, payload=payload))
    return wl, splits, reqs


def test_batch_equals_direct_call_and_keeps_order(dev):
    from boundflow_b200.crown import run_alpha_beta_crown_mlp
    from boundflow_b200.ir import InputSpec
    from boundflow_b200.query_runtime import CudaQueryRuntime

    D = 12
    wl, splits, reqs = _requests(dev, D)
    rt = CudaQueryRuntime(max_batch_size=5)  # 12 nodes -> batches of 5, 5, 2
    out = rt.execute(wl.module, reqs)
    assert [qid for qid, _ in out] == [f"q{i}" for i in range(D)]
    spec = InputSpec.box(value_name="input", lower=wl.lo.expand(D, -1).contiguous().to(dev), upper=wl.up.expand(D, -1).contiguous().to(dev))
    state = {n: s.to(dev) for n, s in zip(wl.relu_names, splits)}
    b, a, bt, stats = run_alpha_beta_crown_mlp(wl.module, spec, linear_spec_C=wl.C.expand(D, -1, -1).contiguous().to(dev), relu_split_state=state,
                                               steps=5, lr=0.1, alpha_init=0.5, per_batch_params=True)
    for i, (_qid, r) in enumerate(out):
        assert r.status == "ok"
        assert tuple(r.lower.shape) == (1, 9)
        # every node is an independent optimisation: batching 5+5+2 or 12 at once gives the same numbers
        assert_close(r.lower, b.lower[i : i + 1], f"node {i} lower")
        assert_close(r.upper, b.upper[i : i + 1], f"node {i} upper")
        assert r.branch == stats.branch_choices[i]
        for n in wl.relu_names:
            assert tuple(r.alpha_by_relu_input[n].shape) == tuple(a.alpha_by_relu_input[n].shape[1:])
            assert float(r.beta_by_relu_input[n].min()) >= 0.0
    assert rt.audit()["batches"] == 3 and rt.audit()["queries"] == D


def test_infeasible_node_is_reported_alone(dev):
    from boundflow_b200.query_runtime import CudaQueryRuntime

    wl, splits, reqs = _requests(dev, 4)
    # node 2: force a neuron inactive whose lower bound is positive under the other clamps -> empty set
    name = wl.relu_names[0]
    from oracle import crown_oracle as O

    root = O.forward_ibp_trace(wl.layers, O.box_input(wl.lo, wl.up))
    stable_on = int(torch.nonzero(root.pre[0][0][0] > 0)[0])
    bad = reqs[2].payload.split_by_relu_input[name].clone()
    bad[stable_on] = -1
    reqs[2].payload.split_by_relu_input[name] = bad
    out = CudaQueryRuntime().execute(wl.module, reqs)
    assert [r.status for _q, r in out] == ["ok", "ok", "infeasible", "ok"]
    assert out[2][1].lower is None


def test_mixed_groups_and_alpha_only(dev):
    from boundflow_b200.query_runtime import CudaQueryRuntime

    wl, _s, ab = _requests(dev, 3, prefix="ab")
    _wl, _s2, al = _requests(dev, 2, method="alpha-CROWN", opts={**OPTS, "alpha_steps": 2}, prefix="al")
    mixed = [ab[0], al[0], ab[1], al[1], ab[2]]
    out = CudaQueryRuntime().execute(wl.module, mixed)
    assert [q for q, _ in out] == ["ab0", "al0", "ab1", "al1", "ab2"]
    assert all(r.status == "ok" for _q, r in out)
    assert out[1][1].branch is None and not out[1][1].beta_by_relu_input
    with pytest.raises(ValueError):
        bad = _requests(dev, 1, method="CROWN")[2]
        CudaQueryRuntime().execute(wl.module, bad)
    assert CudaQueryRuntime().execute(wl.module, []) == []


@pytest.mark.parametrize("objective,reduce", [("gap", "min"), ("lower", "softmin"), ("upper", "mean")])
def test_objective_and_reduction_options_reach_the_loop(dev, objective, reduce):
    """The replay options of a query (`objective`, `spec_reduce`, `soft_tau`, `lb_weight`, `ub_weight`; bab_query.py:860-864)
    select the same loop as a direct call with those arguments."""
    from boundflow_b200.crown import run_alpha_beta_crown_mlp
    from boundflow_b200.ir import InputSpec
    from boundflow_b200.query_runtime import CudaQueryRuntime

    D = 6
    opts = dict(OPTS, objective=objective, spec_reduce=reduce, soft_tau=20.0, lb_weight=1.0, ub_weight=0.5)
    wl, splits, reqs = _requests(dev, D, opts=opts)
    out = CudaQueryRuntime().execute(wl.module, reqs)
    spec = InputSpec.box(value_name="input", lower=wl.lo.expand(D, -1).contiguous().to(dev), upper=wl.up.expand(D, -1).contiguous().to(dev))
    state = {n: s.to(dev) for n, s in zip(wl.relu_names, splits)}
    b, _a, _bt, _stats = run_alpha_beta_crown_mlp(wl.module, spec, linear_spec_C=wl.C.expand(D, -1, -1).contiguous().to(dev), relu_split_state=state,
                                                 steps=5, lr=0.1, alpha_init=0.5, per_batch_params=True, objective=objective, spec_reduce=reduce,
                                                 soft_tau=20.0, lb_weight=1.0, ub_weight=0.5)
    for i, (_qid, r) in enumerate(out):
        assert r.status == "ok"
        assert_close(r.lower, b.lower[i : i + 1], f"node {i} lower")
        assert_close(r.upper, b.upper[i : i + 1], f"node {i} upper")


def _node_requests(module_spec_rows, C_rows, split_rows, opts, method="alpha-beta-CROWN"):
    reqs = []
    for i, spec in enumerate(module_spec_rows):
        payload = SimpleNamespace(input_spec=spec, linear_spec_c=None if C_rows is None else C_rows[i],
                                  split_by_relu_input={n: s[i] for n, s in split_rows.items()}, warm_alpha_by_relu_input={}, warm_beta_by_relu_input={})
        query = SimpleNamespace(query_id=f"n{i}", bound_method=SimpleNamespace(value=method), execution_options=dict(opts))
        reqs.append(SimpleNamespace(query=query, payload=payload))
    return reqs


def test_graph_module_and_lp_ball_nodes(dev, golden):
    """Nodes of a graph that is not a chain (splits of tests/golden/graph_alpha.npz) and nodes with an L2-ball input set go
    through the whole-query functions: the same numbers as one direct call on the stacked batch, the branching hint of
    every node, and an empty node reported alone."""
    import numpy as np

    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import run_alpha_beta_crown_mlp
    from boundflow_b200.ir import InputSpec
    from boundflow_b200.query_runtime import CudaQueryRuntime

    ga = golden("graph_alpha.npz")
    module, _x, lo, up, C = W.make_graph_cases()["fanout_mlp"]
    B = int(lo.shape[0])
    split = {"h": torch.from_numpy(np.asarray(ga["fanout_mlp_split_h"])).to(torch.int8).to(dev)}
    specs = [InputSpec.box(value_name="input", lower=lo[i : i + 1].to(dev), upper=up[i : i + 1].to(dev)) for i in range(B)]
    reqs = _node_requests(specs, C.to(dev), split, OPTS)
    rt = CudaQueryRuntime()
    out = rt.execute(module, reqs)
    whole = InputSpec.box(value_name="input", lower=lo.to(dev), upper=up.to(dev))
    b, _a, bt, stats = run_alpha_beta_crown_mlp(module, whole, linear_spec_C=C.to(dev), relu_split_state=split, steps=5, lr=0.1, alpha_init=0.5,
                                               per_batch_params=True)
    for i, (qid, r) in enumerate(out):
        assert qid == f"n{i}" and r.status == "ok"
        assert_close(r.lower, b.lower[i : i + 1], f"graph node {i} lower")
        assert_close(r.upper, b.upper[i : i + 1], f"graph node {i} upper")
        assert_close(r.beta_by_relu_input["h"], bt.beta_by_relu_input["h"][i], f"graph node {i} beta", atol=1e-6)
        assert r.branch == stats.branch_choices[i]
    # the hint: widest unstable gap of the (split) pre-activation bounds, first index on ties
    from boundflow_b200.dag import forward_ibp_dag

    tr = forward_ibp_dag(module, whole, split)
    gap = torch.where((tr.pre_l["h"] < 0) & (tr.pre_u["h"] > 0), tr.pre_u["h"] - tr.pre_l["h"], torch.full_like(tr.pre_l["h"], -1.0))
    assert [c[1] for c in stats.branch_choices] == gap.argmax(dim=1).cpu().tolist() and all(c[0] == "h" for c in stats.branch_choices)
    # an empty node (a neuron forced inactive whose lower bound is positive) is reported alone
    tr0 = forward_ibp_dag(module, whole)
    on = int(torch.nonzero(tr0.pre_l["h"][1] > 0)[0])
    bad = {"h": split["h"].clone()}
    bad["h"][1, on] = -1
    out = rt.execute(module, _node_requests(specs, C.to(dev), bad, OPTS))
    assert [r.status for _q, r in out] == ["ok", "infeasible", "ok", "ok", "ok"]
    assert_close(out[0][1].lower, b.lower[0:1], "node 0 beside the empty node")
    # L2-ball nodes on the chain c1
    wl = W.make_workload("c1", batch=6)
    specs = [InputSpec.l2(value_name="input", center=wl.x[i : i + 1].to(dev), eps=0.1) for i in range(6)]
    out = rt.execute(wl.module, _node_requests(specs, wl.C.to(dev), {}, OPTS, method="alpha-CROWN"))
    b, _a, _bt, _s = run_alpha_beta_crown_mlp(wl.module, InputSpec.l2(value_name="input", center=wl.x.to(dev), eps=0.1), linear_spec_C=wl.C.to(dev),
                                             steps=5, lr=0.1, alpha_init=0.5, per_batch_params=True)
    for i, (_qid, r) in enumerate(out):
        assert r.status == "ok" and r.branch is None
        assert_close(r.lower, b.lower[i : i + 1], f"L2 node {i} lower")
        assert_close(r.upper, b.upper[i : i + 1], f"L2 node {i} upper")
