"""L2 / L1 ball input sets on the GPU (dual-norm first layer, dual-norm concretisation),
against the reference's own outputs (tests/golden/lp_ball.npz) and the oracle."""
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


@pytest.mark.parametrize("tag,batch", [("c1", None), ("c2", 4)])
@pytest.mark.parametrize("pname,p", [("l2", 2), ("l1", 1)])
def test_lp_ball_matches_reference_golden(dev, golden, tag, batch, pname, p):
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import run_crown_ibp_mlp
    from boundflow_b200.executor import CudaTaskExecutor
    from boundflow_b200.ir import InputSpec

    g = golden("lp_ball.npz")
    wl = W.make_workload(tag) if batch is None else W.make_workload(tag, batch=batch)
    mk = InputSpec.l2 if p == 2 else InputSpec.l1
    spec = mk(value_name="input", center=wl.x.to(dev), eps=float(g[f"{tag}_{pname}_eps"]))
    ibp = CudaTaskExecutor().run_ibp(wl.module, spec)
    assert_close(ibp.lower, g[f"{tag}_{pname}_ibp_lower"], "ibp lower")
    assert_close(ibp.upper, g[f"{tag}_{pname}_ibp_upper"], "ibp upper")
    crown = run_crown_ibp_mlp(wl.module, spec, linear_spec_C=wl.C.to(dev))
    assert_close(crown.lower, g[f"{tag}_{pname}_crown_lower"], "crown lower")
    assert_close(crown.upper, g[f"{tag}_{pname}_crown_upper"], "crown upper")


@pytest.mark.parametrize("p", [1, 2, 3])
def test_lp_entry_points_against_torch(dev, p):
    """bf_row_dual_norms and bf_concretize_lp on ragged sizes (p = 3 encodes the L-inf ball)."""
    from boundflow_b200 import _lib

    lib = _lib.load()
    g = torch.Generator("cpu").manual_seed(5 + p)
    Wm = torch.randn(37, 301, generator=g)
    A = torch.randn(3, 7, 301, generator=g)
    x0 = torch.randn(3, 301, generator=g)
    b = torch.randn(3, 7, generator=g)
    eps = 0.37

    def dual(t):
        if p == 2:
            return torch.linalg.vector_norm(t, ord=2, dim=-1)
        return t.abs().amax(dim=-1) if p == 1 else t.abs().sum(dim=-1)

    Wd, Ad, xd, bd = (t.to(dev).contiguous() for t in (Wm, A, x0, b))
    s = torch.cuda.current_stream(dev).cuda_stream
    out = torch.empty(37, device=dev)
    _lib.check(lib.bf_row_dual_norms(_lib.ptr(Wd), 37, 301, p, eps, _lib.ptr(out), s))
    assert_close(out, eps * dual(Wm), "row dual norms")
    for side, sgn in ((0, -1.0), (1, 1.0)):
        o = torch.empty(3, 7, device=dev)
        _lib.check(lib.bf_concretize_lp(_lib.ptr(Ad), _lib.ptr(xd), eps, p, _lib.ptr(bd), _lib.ptr(o), side, 3, 7, 301, s))
        ref = (A * x0[:, None, :]).sum(-1) + sgn * eps * dual(A) + b
        assert_close(o, ref, f"concretize side {side}")


@pytest.mark.parametrize("pname,p", [("l2", 2), ("l1", 1)])
def test_alpha_crown_on_lp_ball_matches_reference_golden_and_oracle_gradient(dev, golden, pname, p):
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import AlphaState, adaptive_alpha_from_trace, alpha_grad_from_trace, ibp_trace, run_alpha_beta_crown_mlp
    from boundflow_b200.ir import InputSpec
    from oracle import crown_oracle as O

    g = golden("lp_alpha.npz")
    wl = W.make_workload("c3", batch=8)
    mk = InputSpec.l2 if p == 2 else InputSpec.l1
    eps = float(g[f"{pname}_eps"])
    spec = mk(value_name="input", center=wl.x.to(dev), eps=eps)
    trace = ibp_trace(wl.module, spec)
    a0 = adaptive_alpha_from_trace(trace)
    warm = AlphaState(dict(zip(wl.relu_names, a0)))
    for steps, rtol in ((1, 1e-5), (10, 1e-5)):
        b, _a, _b, _s = run_alpha_beta_crown_mlp(wl.module, spec, linear_spec_C=wl.C.to(dev), steps=steps, lr=0.1,
                                                warm_start_alpha=warm, per_batch_params=True)
        assert_close(b.lower, g[f"{pname}_lower_{steps}"], f"lower after {steps} steps", rtol=rtol)
        assert_close(b.upper, g[f"{pname}_upper_{steps}"], f"upper after {steps} steps", rtol=rtol)
    # the analytic gradient (adjoint sweep started from centre - eps * d||A_0||_q/dA_0) against autograd through the oracle
    inp = O.lp_ball(wl.x, eps, p)
    otrace = O.forward_ibp_trace(wl.layers, inp)
    mid_alpha = [torch.full_like(a, 0.4) for a in a0]
    grads, lower = alpha_grad_from_trace(trace, wl.C.to(dev), mid_alpha)
    ref_grads, ref_lower = O.alpha_gradient(wl.layers, inp, otrace, wl.C, [a.cpu() for a in mid_alpha])
    assert_close(lower, ref_lower, "lower at alpha = 0.4")
    for r, (gg, rg) in enumerate(zip(grads, ref_grads)):
        scale = float(rg.abs().max()) + 1e-12
        assert float((gg.cpu() - rg).abs().max()) <= 2e-4 * scale + 1e-6, f"gradient of ReLU {r}"


@pytest.mark.parametrize("name", ["fanout_mlp", "concat_mlp", "residual_s1"])
@pytest.mark.parametrize("pname,p", [("l2", 2), ("l1", 1)])
def test_lp_ball_on_graphs_matches_reference_golden(dev, golden, name, pname, p):
    """L2 / L1 balls on graphs that are not chains (tests/golden/graph_lp.npz): a Linear op on the input value uses the
    dual row norms, a Conv2d op the bounding box; the sweep ends in the Lp concretisation and the gradient sweep
    starts from the Lp adjoint point."""
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import AlphaState, run_alpha_beta_crown_mlp, run_crown_ibp_mlp
    from boundflow_b200.dag import forward_ibp_dag
    from boundflow_b200.executor import CudaTaskExecutor
    from boundflow_b200.ir import InputSpec

    g = golden("graph_lp.npz")
    module, x, _lo, _up, C = W.make_graph_cases()[name]
    B = int(x.shape[0])
    mk = InputSpec.l2 if p == 2 else InputSpec.l1
    spec = mk(value_name="input", center=x.to(dev), eps=float(g[f"{name}_{pname}_eps"]))
    Cd = None if C is None else C.to(dev)
    ibp = CudaTaskExecutor().run_ibp(module, spec)
    assert_close(ibp.lower.reshape(B, -1), g[f"{name}_{pname}_ibp_lower"].reshape(B, -1), "ibp lower")
    assert_close(ibp.upper.reshape(B, -1), g[f"{name}_{pname}_ibp_upper"].reshape(B, -1), "ibp upper")
    crown = run_crown_ibp_mlp(module, spec, linear_spec_C=Cd)
    assert_close(crown.lower.reshape(B, -1), g[f"{name}_{pname}_crown_lower"].reshape(B, -1), "crown lower")
    assert_close(crown.upper.reshape(B, -1), g[f"{name}_{pname}_crown_upper"].reshape(B, -1), "crown upper")
    tr = forward_ibp_dag(module, spec)
    a0 = {k: ((tr.pre_l[k] >= 0) | ((tr.pre_l[k] < 0) & (tr.pre_u[k] > 0) & (tr.pre_u[k] > -tr.pre_l[k]))).float() for k in tr.pre_l}
    b, _a, _bt, _s = run_alpha_beta_crown_mlp(module, spec, linear_spec_C=Cd, steps=3, lr=0.1, per_batch_params=True, warm_start_alpha=AlphaState(a0))
    assert_close(b.lower.reshape(B, -1), g[f"{name}_{pname}_alpha_lower_3"].reshape(B, -1), "alpha lower after 3")
    assert_close(b.upper.reshape(B, -1), g[f"{name}_{pname}_alpha_upper_3"].reshape(B, -1), "alpha upper after 3")
