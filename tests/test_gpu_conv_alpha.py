"""alpha-CROWN on a conv chain (Conv2d backward steps in the sweeps, forward convolution + ReLU adjoint step
in the gradient sweep), against the reference's outputs and autograd through the oracle."""
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


def test_c2_matches_reference_golden(dev, golden):
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import AlphaState, adaptive_alpha_from_trace, ibp_trace, run_alpha_beta_crown_mlp, run_alpha_crown_mlp
    from boundflow_b200.ir import InputSpec

    g = golden("conv_alpha.npz")
    wl = W.make_workload("c2", batch=4)
    spec = InputSpec.box(value_name="input", lower=wl.lo.to(dev), upper=wl.up.to(dev))
    trace = ibp_trace(wl.module, spec)
    warm = AlphaState(dict(zip(wl.relu_names, adaptive_alpha_from_trace(trace))))
    for steps, rtol in ((1, 1e-5), (6, 1e-5)):
        b, a, _b, _s = run_alpha_beta_crown_mlp(wl.module, spec, linear_spec_C=wl.C.to(dev), steps=steps, lr=0.1, warm_start_alpha=warm,
                                               per_batch_params=True)
        assert_close(b.lower, g[f"per_domain_lower_{steps}"], f"per-domain lower after {steps}", rtol=rtol)
        assert_close(b.upper, g[f"per_domain_upper_{steps}"], f"per-domain upper after {steps}", rtol=rtol)
        bs, st, _ = run_alpha_crown_mlp(wl.module, spec, linear_spec_C=wl.C.to(dev), steps=steps, lr=0.1)
        assert_close(bs.lower, g[f"shared_lower_{steps}"], f"shared lower after {steps}", rtol=rtol)
        assert_close(bs.upper, g[f"shared_upper_{steps}"], f"shared upper after {steps}", rtol=rtol)
    # alpha keeps the pre-activation's shape
    assert tuple(a.alpha_by_relu_input[wl.relu_names[0]].shape) == (4, 16, 14, 14)
    assert tuple(st.alpha_by_relu_input[wl.relu_names[0]].shape) == (16, 14, 14)


def test_conv_gradient_against_oracle_autograd(dev):
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import alpha_grad_from_trace, ibp_trace
    from boundflow_b200.ir import InputSpec
    from oracle import crown_oracle as O

    wl = W.make_workload("c2", batch=3)
    spec = InputSpec.box(value_name="input", lower=wl.lo.to(dev), upper=wl.up.to(dev))
    trace = ibp_trace(wl.module, spec)
    alphas = [torch.full((3, n), 0.35, device=dev) for n in trace.chain.relu_widths]
    grads, lower = alpha_grad_from_trace(trace, wl.C.to(dev), alphas)
    inp = O.box_input(wl.lo, wl.up)
    otrace = O.forward_ibp_trace(wl.layers, inp)
    ref_grads, ref_lower = O.alpha_gradient(wl.layers, inp, otrace, wl.C, [a.cpu() for a in alphas])
    assert_close(lower, ref_lower, "lower at alpha = 0.35")
    for r, (gg, rg) in enumerate(zip(grads, ref_grads)):
        scale = float(rg.abs().max()) + 1e-12
        assert float((gg.cpu() - rg.reshape(3, -1)).abs().max()) <= 2e-4 * scale + 1e-6, f"gradient of ReLU {r}"


def test_beta_on_the_linear_relu_of_a_conv_chain_matches_oracle(dev):
    """A split on the Linear ReLU only of a conv chain (the conv ReLUs carry a zero split term), against the oracle."""
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import run_alpha_beta_crown_mlp
    from boundflow_b200.ir import InputSpec
    from oracle import crown_oracle as O

    wl = W.make_workload("c2", batch=2)
    spec = InputSpec.box(value_name="input", lower=wl.lo.to(dev), upper=wl.up.to(dev))
    s3 = torch.zeros(2, 100, dtype=torch.int8)
    s3[:, 3] = 1
    s3[:, 40] = -1
    b, _a, bt, _s = run_alpha_beta_crown_mlp(wl.module, spec, linear_spec_C=wl.C.to(dev), relu_split_state={wl.relu_names[2]: s3.to(dev)},
                                            steps=4, lr=0.1, per_batch_params=True)
    inp = O.box_input(wl.lo, wl.up)
    splits = [None, None, s3]
    lo, up, _al, beta, _t = O.alpha_crown(wl.layers, inp, wl.C, steps=4, lr=0.1, splits=splits, optimize_beta=True, return_beta=True)
    assert_close(b.lower, lo, "lower after 4 steps")
    assert_close(b.upper, up, "upper after 4 steps")
    assert_close(bt.beta_by_relu_input[wl.relu_names[2]].reshape(2, -1), beta[2], "beta of the Linear ReLU", atol=1e-5)


def test_c2_alpha_beta_with_splits_matches_reference_golden(dev, golden):
    """beta parameters on conv ReLUs: the split term enters the ReLU scaling pass in front of the transposed
    convolution, its gradient comes from the per-domain sums of the adjoint values (tests/golden/conv_beta.npz, the
    reference's `run_alpha_beta_crown_mlp(relu_split_state=...)` on c2 with three split neurons per ReLU and input)."""
    import numpy as np

    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import AlphaState, adaptive_alpha_from_trace, ibp_trace, run_alpha_beta_crown_mlp
    from boundflow_b200.ir import InputSpec

    g = golden("conv_beta.npz")
    wl = W.make_workload("c2", batch=4)
    shapes = {"h1": (16, 14, 14), "h2": (32, 7, 7), "h3": (100,)}
    splits = {n: torch.from_numpy(np.asarray(g[f"split_{n}"])).to(torch.int8).reshape((4,) + shapes[n]).to(dev) for n in wl.relu_names}
    spec = InputSpec.box(value_name="input", lower=wl.lo.to(dev), upper=wl.up.to(dev))
    trace = ibp_trace(wl.module, spec, relu_split_state=splits)
    warm = AlphaState(dict(zip(wl.relu_names, adaptive_alpha_from_trace(trace))))
    from oracle import crown_oracle as O

    inp = O.box_input(wl.lo, wl.up)
    otrace = O.forward_ibp_trace(wl.layers, inp, splits=[s.cpu() for s in splits.values()])
    for steps in (1, 3, 8):
        b, a, bt, _s = run_alpha_beta_crown_mlp(wl.module, spec, linear_spec_C=wl.C.to(dev), relu_split_state=splits, steps=steps, lr=0.1,
                                               warm_start_alpha=warm, per_batch_params=True)
        assert_close(b.lower, g[f"per_domain_lower_{steps}"], f"per-domain lower after {steps}")
        # The upper bound is not what the loop optimises, so it follows the rounding of the alpha trajectory to first
        # order: after 8 Adam steps it sits 1.6x the strict tolerance from the reference's (measured), while the same
        # upper bound evaluated by the oracle AT the returned alpha agrees strictly.
        assert_close(b.upper, g[f"per_domain_upper_{steps}"], f"per-domain upper after {steps}", rtol=1e-5 if steps < 8 else 3e-5)
        _lo_at, up_at = O.crown_backward(wl.layers, inp, otrace, wl.C, alpha=[a.alpha_by_relu_input[n].reshape(4, -1).cpu() for n in wl.relu_names])
        assert_close(b.upper, up_at, f"upper after {steps} against the oracle at the returned alpha")
        for n in wl.relu_names:
            assert tuple(bt.beta_by_relu_input[n].shape) == (4,) + shapes[n]
            # beta itself is an Adam iterate (normalised steps of 0.1): strict up to 3 steps, 1.2x the strict tolerance
            # after 8 (measured; the lower bound it produces stays strict)
            assert_close(bt.beta_by_relu_input[n].reshape(4, -1), g[f"per_domain_beta_{n}_{steps}"], f"beta {n} after {steps}",
                         atol=1e-5 if steps < 8 else 3e-4)
    b, _a, _bt, _s = run_alpha_beta_crown_mlp(wl.module, spec, linear_spec_C=wl.C.to(dev), relu_split_state=splits, steps=3, lr=0.1,
                                             per_batch_params=False)
    assert_close(b.lower, g["shared_lower_3"], "shared lower after 3")
    assert_close(b.upper, g["shared_upper_3"], "shared upper after 3")
