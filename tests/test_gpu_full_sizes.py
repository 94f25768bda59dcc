"""Full-size configurations through size-independent properties: c1 (64 inputs), c2 (256 inputs, CROWN with CROWN
intermediate bounds), c3 (128 inputs, 20 alpha steps), c5 (64 inputs, full intermediate CROWN).  The oracle is used on
small slices only; the rest are invariants of the method: sampled soundness, ordering, refinement never loosens a bound,
each input's result does not depend on what else is in the batch."""
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


def _spec(lo, up, dev):
    from boundflow_b200.ir import InputSpec

    return InputSpec.box(value_name="input", lower=lo.to(dev), upper=up.to(dev))


@pytest.mark.parametrize("name,chunk,n_samples", [("c2", 512, 300), ("c5", 64, 60)])
def test_cnn_intermediate_crown_full_size(dev, name, chunk, n_samples):
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import ibp_trace, run_crown_ibp_mlp, run_crown_intermediate_mlp
    from oracle import crown_oracle as O

    wl = W.make_workload(name)   # the configuration's own batch size
    B = wl.x.shape[0]
    spec = _spec(wl.lo, wl.up, dev)
    got, pre = run_crown_intermediate_mlp(wl.module, spec, linear_spec_C=wl.C.to(dev), chunk_rows=chunk)
    lower, upper = got.lower.cpu(), got.upper.cpu()
    assert tuple(lower.shape) == (B, 9) and torch.isfinite(lower).all() and torch.isfinite(upper).all()
    assert (lower <= upper + 1e-4).all()
    # refinement only intersects: every refined pre-activation box lies inside the IBP box
    trace = ibp_trace(wl.module, spec)
    for r, n in enumerate(wl.relu_names):
        l0, u0 = trace.pre_l[r].cpu(), trace.pre_u[r].cpu()
        slack = 1e-5 * float(u0.abs().max()) + 1e-5
        assert (pre[n].lower.reshape(B, -1).cpu() >= l0 - slack).all(), n
        assert (pre[n].upper.reshape(B, -1).cpu() <= u0 + slack).all(), n
    # and the final bounds are at least as tight as CROWN-IBP on average (each is valid; tighter boxes give tighter relaxations)
    plain = run_crown_ibp_mlp(wl.module, spec, linear_spec_C=wl.C.to(dev))
    assert float(lower.mean()) >= float(plain.lower.cpu().mean()) - 1e-4
    assert float(upper.mean()) <= float(plain.upper.cpu().mean()) + 1e-4
    # sampled soundness on a slice of the batch
    sel = slice(0, 8)
    inp = O.box_input(wl.lo[sel], wl.up[sel])
    wlo, wup = O.sample_soundness(wl.layers, inp, wl.C[sel], lower[sel], upper[sel], n=n_samples, seed=3)
    assert wlo <= 1e-4 and wup <= 1e-4
    # batch independence: the first two inputs alone give the same numbers
    alone, _ = run_crown_intermediate_mlp(wl.module, _spec(wl.lo[:2], wl.up[:2], dev), linear_spec_C=wl.C[:2].to(dev), chunk_rows=chunk)
    assert_close(alone.lower, lower[:2], "batch independence (lower)")
    assert_close(alone.upper, upper[:2], "batch independence (upper)")


def test_c1_and_c3_full_size(dev):
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import AlphaState, adaptive_alpha_from_trace, ibp_trace, run_alpha_beta_crown_mlp, run_crown_ibp_mlp
    from oracle import crown_oracle as O

    wl = W.make_workload("c1")
    got = run_crown_ibp_mlp(wl.module, _spec(wl.lo, wl.up, dev), linear_spec_C=wl.C.to(dev))
    ref_l, ref_u, _ = O.crown_ibp(wl.layers, O.box_input(wl.lo, wl.up), wl.C)   # 64 inputs: the oracle is fast enough
    assert_close(got.lower, ref_l, "c1 lower")
    assert_close(got.upper, ref_u, "c1 upper")

    wl = W.make_workload("c3")
    spec = _spec(wl.lo, wl.up, dev)
    trace = ibp_trace(wl.module, spec)
    a0 = adaptive_alpha_from_trace(trace)
    warm = AlphaState(dict(zip(wl.relu_names, a0)))
    b20, a20, _b, _s = run_alpha_beta_crown_mlp(wl.module, spec, linear_spec_C=wl.C.to(dev), steps=20, lr=0.1, warm_start_alpha=warm, per_batch_params=True)
    b0, _a, _b, _s = run_alpha_beta_crown_mlp(wl.module, spec, linear_spec_C=wl.C.to(dev), steps=0, lr=0.1, warm_start_alpha=warm, per_batch_params=True)
    B = wl.x.shape[0]
    assert tuple(b20.lower.shape) == (B, 9)
    # best-of-steps is never below the start, per input
    assert (b20.lower.mean(dim=1) >= b0.lower.mean(dim=1) - 1e-6 * b0.lower.mean(dim=1).abs()).all()
    assert (b20.lower <= b20.upper + 1e-2).all()
    for n in wl.relu_names:
        a = a20.alpha_by_relu_input[n]
        assert float(a.min()) >= 0.0 and float(a.max()) <= 1.0
    # the oracle, evaluated once at the returned alpha, reproduces the returned bounds on a slice
    sel = slice(0, 6)
    inp = O.box_input(wl.lo[sel], wl.up[sel])
    tr = O.forward_ibp_trace(wl.layers, inp)
    lo_ref, up_ref = O.crown_backward(wl.layers, inp, tr, wl.C[sel], alpha=[a20.alpha_by_relu_input[n][sel].reshape(6, -1).cpu() for n in wl.relu_names])
    assert_close(b20.lower[sel], lo_ref, "oracle at returned alpha (lower)")
    assert_close(b20.upper[sel], up_ref, "oracle at returned alpha (upper)")
