"""The min and softmin spec reductions of the alpha loop's lower-bound objective on the GPU, against the
reference's `run_alpha_beta_crown_mlp(spec_reduce=...)` outputs (tests/golden/spec_reduce.npz)."""
import pytest
import torch

from tests.helpers import assert_close

pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("tc_from_256_rows")]


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available()
    from boundflow_b200.csrc import build

    build.build()
    return torch.device("cuda", 0)


@pytest.mark.parametrize("cfg", ["c1", "c3"])
@pytest.mark.parametrize("reduce", ["min", "softmin"])
def test_matches_reference_golden(dev, golden, cfg, reduce):
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import AlphaState, adaptive_alpha_from_trace, ibp_trace, run_alpha_beta_crown_mlp
    from boundflow_b200.ir import InputSpec

    g = golden("spec_reduce.npz")
    wl = W.make_workload(cfg, batch=8)
    spec = InputSpec.box(value_name="input", lower=wl.lo.to(dev), upper=wl.up.to(dev))
    a0 = adaptive_alpha_from_trace(ibp_trace(wl.module, spec))
    for k in (1, 3, 10):
        b, _a, _b, stats = run_alpha_beta_crown_mlp(wl.module, spec, linear_spec_C=wl.C.to(dev), steps=k, lr=0.1, per_batch_params=True,
                                                   warm_start_alpha=AlphaState(dict(zip(wl.relu_names, a0))), spec_reduce=reduce,
                                                   soft_tau=float(g[f"{cfg}_tau"]))
        assert stats.spec_reduce == reduce
        assert_close(b.lower, g[f"{cfg}_{reduce}_lower_{k}"], f"{cfg} {reduce} lower after {k} steps")
        assert_close(b.upper, g[f"{cfg}_{reduce}_upper_{k}"], f"{cfg} {reduce} upper after {k} steps")


def test_tensor_core_rows_and_argument_errors(dev):
    """288 coefficient rows (tcgen05 kernels) against the oracle; min / softmin refuse beta and a non-positive tau."""
    from boundflow_b200 import _lib
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import adaptive_alpha_from_trace, alpha_crown_from_trace, ibp_trace
    from boundflow_b200.ir import InputSpec
    from oracle import crown_oracle as O

    wl = W.make_workload("c3", batch=32)
    spec = InputSpec.box(value_name="input", lower=wl.lo.to(dev), upper=wl.up.to(dev))
    trace = ibp_trace(wl.module, spec)
    a0 = adaptive_alpha_from_trace(trace)
    inp = O.box_input(wl.lo, wl.up)
    tr = O.forward_ibp_trace(wl.layers, inp)
    for red, tau in (("min", 1.0), ("softmin", 80.0)):
        t0 = _lib.tc_launch_count()
        got = alpha_crown_from_trace(trace, wl.C.to(dev), a0, steps=2, lr=0.1, spec_reduce=red, soft_tau=tau)
        assert _lib.tc_launch_count() > t0
        ref_l, ref_u, _a, _t = O.alpha_crown(wl.layers, inp, wl.C, steps=2, lr=0.1, alpha0=[a.cpu() for a in a0], trace=tr, spec_reduce=red, soft_tau=tau)
        assert_close(got[0], ref_l, f"{red} lower, 2 steps")
        assert_close(got[1], ref_u, f"{red} upper, 2 steps")
    with pytest.raises(ValueError):
        alpha_crown_from_trace(trace, wl.C.to(dev), a0, steps=1, lr=0.1, spec_reduce="softmin", soft_tau=0.0)
    with pytest.raises(NotImplementedError):
        alpha_crown_from_trace(trace, wl.C.to(dev), a0, steps=1, lr=0.1, spec_reduce="min", beta_splits=[None] * 5)
