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


def test_beta_on_a_conv_chain_is_refused(dev):
    from boundflow_b200 import workloads as W
    from boundflow_b200._lib import BackendError
    from boundflow_b200.crown import run_alpha_beta_crown_mlp
    from boundflow_b200.ir import InputSpec

    wl = W.make_workload("c2", batch=2)
    spec = InputSpec.box(value_name="input", lower=wl.lo.to(dev), upper=wl.up.to(dev))
    split = {wl.relu_names[2]: torch.zeros(2, 100, dtype=torch.int8, device=dev)}
    split[wl.relu_names[2]][:, 3] = 1
    with pytest.raises((BackendError, NotImplementedError)):
        run_alpha_beta_crown_mlp(wl.module, spec, linear_spec_C=wl.C.to(dev), relu_split_state=split, steps=1, lr=0.1, per_batch_params=True)
