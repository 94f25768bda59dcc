"""The tcgen05 (3xTF32) contraction path against the FP32 FFMA path and the CPU oracle.

The chain drivers pick the tensor-core kernels when B*S >= 256 and the layer is at least
32 wide; BF_B200_FORCE_FFMA=1 (read at every launch) forces the FFMA tiles, which gives
an A/B comparison of the two implementations on identical inputs."""
import os

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


class _ffma:
    def __enter__(self):
        os.environ["BF_B200_FORCE_FFMA"] = "1"

    def __exit__(self, *a):
        os.environ.pop("BF_B200_FORCE_FFMA", None)


class _adjoint_kernel:
    """Pins the tensor-core adjoint kernel: "fm" = feature-major (features on the MMA's M side, the default
    once its 256x256 CTAs fill the GPU), "rows" = row-major; read at every launch."""

    def __init__(self, which):
        self.var = {"fm": "BF_B200_ADJ_FEATURE_MAJOR", "rows": "BF_B200_ADJ_ROWMAJOR"}[which]

    def __enter__(self):
        os.environ[self.var] = "1"

    def __exit__(self, *a):
        os.environ.pop(self.var, None)


def _spec(wl, dev):
    from boundflow_b200.ir import InputSpec

    return InputSpec.box(value_name="input", lower=wl.lo.to(dev), upper=wl.up.to(dev))


def _launch_delta(fn):
    from boundflow_b200 import _lib

    n0 = _lib.launch_count()
    out = fn()
    return out, _lib.launch_count() - n0


def test_tc_crown_matches_ffma_and_oracle_c3(dev):
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import adaptive_alpha_from_trace, crown_from_trace, ibp_trace
    from oracle import crown_oracle as O

    wl = W.make_workload("c3", batch=64)   # M = 576 rows, layers 256 wide
    spec = _spec(wl, dev)
    C = wl.C.to(dev)
    trace = ibp_trace(wl.module, spec)
    a0 = adaptive_alpha_from_trace(trace)
    alpha = dict(zip(trace.chain.relu_input_names, a0))
    lo_tc, up_tc = crown_from_trace(trace, C, relu_alpha=alpha)
    with _ffma():
        lo_ff, up_ff = crown_from_trace(trace, C, relu_alpha=alpha)
    torch.cuda.synchronize()
    assert trace.chain.tc_status() == 0
    assert not torch.equal(lo_tc, lo_ff), "the two paths should not be the same kernel"
    assert_close(lo_tc, lo_ff, "tc vs ffma lower")
    assert_close(up_tc, up_ff, "tc vs ffma upper")
    inp = O.box_input(wl.lo, wl.up)
    tr = O.forward_ibp_trace(wl.layers, inp)
    lo_ref, up_ref = O.crown_backward(wl.layers, inp, tr, wl.C, alpha=[a.cpu() for a in a0])
    assert_close(lo_tc, lo_ref, "tc vs oracle lower")
    assert_close(up_tc, up_ref, "tc vs oracle upper")


@pytest.mark.parametrize("adjoint", ["fm", "rows"])
def test_tc_gradient_matches_ffma_and_oracle(dev, adjoint):
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import adaptive_alpha_from_trace, alpha_grad_from_trace, ibp_trace
    from oracle import crown_oracle as O

    wl = W.make_workload("c3", batch=40)   # M = 360: a ragged last row tile
    spec = _spec(wl, dev)
    C = wl.C.to(dev)
    trace = ibp_trace(wl.module, spec)
    a0 = adaptive_alpha_from_trace(trace)
    a0 = [0.25 + 0.5 * a for a in a0]      # interior alpha: both sign branches carry gradient
    with _adjoint_kernel(adjoint):
        g_tc, lo_tc = alpha_grad_from_trace(trace, C, a0)
    with _ffma():
        g_ff, lo_ff = alpha_grad_from_trace(trace, C, a0)
    torch.cuda.synchronize()
    assert trace.chain.tc_status() == 0
    assert_close(lo_tc, lo_ff, "lower")
    inp = O.box_input(wl.lo, wl.up)
    tr = O.forward_ibp_trace(wl.layers, inp)
    g_ref, lo_ref = O.alpha_gradient(wl.layers, inp, tr, wl.C, [a.cpu() for a in a0])
    assert_close(lo_tc, lo_ref, "lower vs oracle")
    for r in range(len(g_tc)):
        scale = float(g_ref[r].abs().max())
        assert_close(g_tc[r], g_ff[r], f"grad {r} tc vs ffma", atol=2e-5 * scale, rtol=1e-4)
        assert_close(g_tc[r], g_ref[r], f"grad {r} tc vs oracle", atol=2e-5 * scale, rtol=1e-4)


@pytest.mark.parametrize("adjoint", ["fm", "rows"])
@pytest.mark.parametrize("widths,B,S", [((784, 200, 136, 10), 60, 5), ((100, 72, 40, 33, 7), 300, 1), ((64, 512, 300, 10), 29, 9),
                                        ((48, 130, 260, 10), 37, 12)])
def test_tc_ragged_shapes(dev, widths, B, S, adjoint):
    """Layer widths that are not multiples of the 32-wide k-block or the column tile,
    row counts that are not multiples of 128, and S values that put several domains in
    one 8-row group."""
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import alpha_grad_from_trace, crown_from_trace, ibp_trace
    from boundflow_b200.ir import InputSpec
    from oracle import crown_oracle as O

    net = W.NetSpec((widths[0],), [("fc", w) for w in widths[1:]])
    g = torch.Generator("cpu").manual_seed(sum(widths))
    layers, module, names = W.build_chain(net, g)
    x = torch.rand(B, widths[0], generator=g)
    lo, up = x - 0.05, x + 0.05
    C = torch.randn(B, S, widths[-1], generator=g)
    spec = InputSpec.box(value_name="input", lower=lo.to(dev), upper=up.to(dev))
    trace = ibp_trace(module, spec)
    alpha = [torch.rand(B, w, generator=g) for w in widths[1:-1]]
    amap = dict(zip(names, [a.to(dev) for a in alpha]))
    (lo_tc, up_tc), n_launch = _launch_delta(lambda: crown_from_trace(trace, C.to(dev), relu_alpha=amap))
    inp = O.box_input(lo, up)
    tr = O.forward_ibp_trace(layers, inp)
    lo_ref, up_ref = O.crown_backward(layers, inp, tr, C, alpha=alpha)
    torch.cuda.synchronize()
    assert trace.chain.tc_status() == 0
    scale = max(1.0, float(lo_ref.abs().max()))
    assert_close(lo_tc, lo_ref, "lower", atol=1e-4 + 2e-6 * scale)
    assert_close(up_tc, up_ref, "upper", atol=1e-4 + 2e-6 * scale)
    with _adjoint_kernel(adjoint):
        grads, lower = alpha_grad_from_trace(trace, C.to(dev), [a.to(dev) for a in alpha])
    torch.cuda.synchronize()
    assert trace.chain.tc_status() == 0
    g_ref, _ = O.alpha_gradient(layers, inp, tr, C, alpha)
    for r in range(len(grads)):
        s = max(1e-3, float(g_ref[r].abs().max()))
        assert_close(grads[r], g_ref[r], f"grad {r}", atol=3e-5 * s, rtol=1e-4)


@pytest.mark.parametrize("adjoint", ["fm", "rows"])
def test_tc_is_deterministic(dev, adjoint):
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import adaptive_alpha_from_trace, alpha_crown_from_trace, ibp_trace

    wl = W.make_workload("c3", batch=48)
    trace = ibp_trace(wl.module, _spec(wl, dev))
    a0 = adaptive_alpha_from_trace(trace)
    with _adjoint_kernel(adjoint):
        r1 = alpha_crown_from_trace(trace, wl.C.to(dev), a0, steps=4, lr=0.1)
        r2 = alpha_crown_from_trace(trace, wl.C.to(dev), a0, steps=4, lr=0.1)
    torch.cuda.synchronize()
    assert trace.chain.tc_status() == 0
    assert torch.equal(r1[0], r2[0]) and torch.equal(r1[1], r2[1])
    for a, b in zip(r1[2], r2[2]):
        assert torch.equal(a, b)


@pytest.mark.parametrize("switch", ["BF_B200_BWD_PERSISTENT", "BF_B200_BWD_PAIRS"])
def test_opt_in_backward_kernels_match_oracle(dev, switch):
    """The two opt-in variants of the backward contraction on a problem with several tiles per CTA and on ragged
    small ones: the persistent warp-specialised kernel (double-buffered accumulators in tensor memory, narrower tiles
    when few row blocks exist) and the CTA-pair kernel (clusters of two row blocks, tcgen05 cta_group::2, each CTA
    holding half of every weight image; 360 rows = 3 row blocks leave one pair with an empty second CTA)."""
    import os

    from boundflow_b200 import _lib
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import adaptive_alpha_from_trace, alpha_crown_from_trace, crown_from_trace, ibp_trace
    from boundflow_b200.ir import InputSpec
    from oracle import crown_oracle as O

    os.environ[switch] = "1"
    try:
        for name, batch in (("c3", 40), ("c1", 64)):   # 360 and 576 rows: narrow tiles, partial row blocks
            wl = W.make_workload(name, batch=batch)
            trace = ibp_trace(wl.module, _spec(wl, dev))
            a0 = adaptive_alpha_from_trace(trace)
            t0 = _lib.tc_launch_count()
            lo, up = crown_from_trace(trace, wl.C.to(dev), relu_alpha=dict(zip(trace.chain.relu_input_names, a0)))
            assert _lib.tc_launch_count() > t0
            inp = O.box_input(wl.lo, wl.up)
            tr = O.forward_ibp_trace(wl.layers, inp)
            lo_ref, up_ref = O.crown_backward(wl.layers, inp, tr, wl.C, alpha=[a.cpu() for a in a0])
            assert_close(lo, lo_ref, f"{name} lower")
            assert_close(up, up_ref, f"{name} upper")
        # c4 at 4096 subdomains: 288 row blocks x 2 column tiles on 148 SMs -> four tiles per CTA, both accumulator buffers reused
        wl = W.make_workload("c4")
        D = 4096
        root = O.forward_ibp_trace(wl.layers, O.box_input(wl.lo, wl.up))
        g = torch.Generator("cpu").manual_seed(11)
        splits = []
        for r, (l, u) in enumerate(root.pre):
            idx = torch.nonzero(((l < 0) & (u > 0)).reshape(-1)).flatten()
            s8 = torch.zeros(D, l.shape[1], dtype=torch.int8)
            pick = idx[torch.randint(0, len(idx), (D, 3), generator=g)]
            s8.scatter_(1, pick, (torch.randint(0, 2, (D, 3), generator=g) * 2 - 1).to(torch.int8))
            splits.append(s8)
        lo_b, up_b = wl.lo.expand(D, -1).contiguous(), wl.up.expand(D, -1).contiguous()
        spec = InputSpec.box(value_name="input", lower=lo_b.to(dev), upper=up_b.to(dev))
        trace = ibp_trace(wl.module, spec, relu_split_state={n: s.to(dev) for n, s in zip(wl.relu_names, splits)})
        a0 = adaptive_alpha_from_trace(trace)
        C = wl.C.expand(D, -1, -1).contiguous()
        best_l, best_u, best_a, _, _ = alpha_crown_from_trace(trace, C.to(dev), a0, steps=2, lr=0.1)
        torch.cuda.synchronize()
        assert trace.chain.tc_status() == 0
        sel = torch.nonzero((trace.infeasible == 0).cpu()).flatten()[::257][:16]
        inp = O.box_input(lo_b[sel], up_b[sel])
        tr = O.forward_ibp_trace(wl.layers, inp, splits=[s[sel] for s in splits])
        lo_ref, up_ref = O.crown_backward(wl.layers, inp, tr, C[sel], alpha=[a[sel.to(dev)].cpu() for a in best_a])
        assert_close(best_l[sel.to(dev)], lo_ref, "c4 lower at the returned alpha")
        assert_close(best_u[sel.to(dev)], up_ref, "c4 upper at the returned alpha")
    finally:
        os.environ.pop(switch, None)
