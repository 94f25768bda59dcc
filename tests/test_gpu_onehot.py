"""Identity spec rows without an identity tensor (`bf_chain_crown_onehot`): the sweep that bounds an
intermediate value neuron by neuron must equal the dense sweep with C = rows of the identity."""
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


@pytest.mark.parametrize("name,batch", [("c2", 3), ("c3", 5), ("c5", 1)])
def test_onehot_rows_equal_dense_identity(dev, name, batch):
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import crown_from_trace, ibp_trace
    from boundflow_b200.ir import InputSpec

    wl = W.make_workload(name, batch=batch)
    spec = InputSpec.box(value_name="input", lower=wl.lo.to(dev), upper=wl.up.to(dev))
    trace = ibp_trace(wl.module, spec)
    chain = trace.chain
    for r in range(1, len(chain.relu_input_names)):
        n = chain.relu_widths[r]
        # ragged window that crosses channel / row boundaries and ends at the last neuron
        for first, cnt in ((0, min(7, n)), (max(0, n - 37), min(37, n)), (n // 3, min(50, n - n // 3))):
            eye = torch.eye(n, dtype=torch.float32, device=dev)[first : first + cnt]
            lo_d, up_d = crown_from_trace(trace, eye, output_value=chain.relu_input_names[r])
            lo_o, up_o = crown_from_trace(trace, None, output_value=chain.relu_input_names[r], identity_rows=(first, cnt))
            assert_close(lo_o, lo_d, f"{name} relu {r} rows {first}+{cnt} lower")
            assert_close(up_o, up_d, f"{name} relu {r} rows {first}+{cnt} upper")


def test_onehot_rejects_bad_windows(dev):
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import crown_from_trace, ibp_trace
    from boundflow_b200.ir import InputSpec

    wl = W.make_workload("c3", batch=2)
    spec = InputSpec.box(value_name="input", lower=wl.lo.to(dev), upper=wl.up.to(dev))
    trace = ibp_trace(wl.module, spec)
    name = trace.chain.relu_input_names[1]
    n = trace.chain.relu_widths[1]
    with pytest.raises(ValueError):
        crown_from_trace(trace, None, output_value=name, identity_rows=(n - 3, 4))
    with pytest.raises(ValueError):
        crown_from_trace(trace, None, output_value=name, identity_rows=(-1, 4))


def test_intermediate_recipe_on_mlp_matches_oracle(dev):
    """The recipe with a Linear layer under every bounded value (weight-row copy as first step)."""
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import run_crown_intermediate_mlp
    from boundflow_b200.ir import InputSpec
    from oracle import crown_oracle as O

    wl = W.make_workload("c1")
    lo, up, C = wl.lo[:6], wl.up[:6], wl.C[:6]
    spec = InputSpec.box(value_name="input", lower=lo.to(dev), upper=up.to(dev))
    got, pre = run_crown_intermediate_mlp(wl.module, spec, linear_spec_C=C.to(dev), chunk_rows=64)
    ref_l, ref_u, ref_tr = O.crown_with_intermediate_crown(wl.layers, O.box_input(lo, up), C, chunk=64)
    assert_close(got.lower, ref_l, "lower")
    assert_close(got.upper, ref_u, "upper")
    for r, nm in enumerate(wl.relu_names):
        assert_close(pre[nm].lower, ref_tr.pre[r][0], f"pre {nm} lower")
        assert_close(pre[nm].upper, ref_tr.pre[r][1], f"pre {nm} upper")
