"""Per-ReLU objective influence of the backward coefficients (`bf_chain_crown_influence`)."""
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


@pytest.mark.parametrize("tag,batch", [("c1", 8), ("c2", 3)])
def test_matches_reference_golden(dev, golden, tag, batch):
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import forward_ibp_trace_mlp, run_crown_ibp_mlp_with_relu_influence_from_forward_trace
    from boundflow_b200.ir import InputSpec

    g = golden("relu_influence.npz")
    wl = W.make_workload(tag, batch=batch)
    spec = InputSpec.box(value_name="input", lower=wl.lo.to(dev), upper=wl.up.to(dev))
    env, pre = forward_ibp_trace_mlp(wl.module, spec)
    bounds, infl = run_crown_ibp_mlp_with_relu_influence_from_forward_trace(
        wl.module, spec, interval_env=env, relu_pre=pre, linear_spec_C=wl.C.to(dev))
    assert_close(bounds.lower, g[f"{tag}_lower"], "lower")
    assert_close(bounds.upper, g[f"{tag}_upper"], "upper")
    assert list(infl) == list(wl.relu_names)
    for n in wl.relu_names:
        assert tuple(infl[n].shape) == tuple(pre[n].lower.shape)
        assert_close(infl[n].reshape(batch, -1), g[f"{tag}_influence_{n}"], f"influence {n}")
