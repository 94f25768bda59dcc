"""Soundness by sampling: every bound of every configuration holds on 10^4 points per input set.

The sampler is test infrastructure: plain torch forward passes in float64 on the GPU of the same seeded networks
(`workloads.py`), nothing of the library under test.  A bound is violated when a sampled output leaves
[lower, upper] by more than the parity tolerance 1e-4 + 1e-5 |bound| (the bounds are fp32 results).

  c1  IBP and CROWN, all 64 inputs
  c2  CROWN with CROWN intermediate bounds, 8 inputs
  c3  alpha-CROWN (20 Adam steps), 8 inputs
  c4  alpha-CROWN (10 steps) on 8 ReLU-split subdomains; only samples that satisfy the split constraints count
      (the number of survivors is reported and must reach 10^3 per subdomain)
  c5  CROWN with full CROWN intermediate bounds, 8 inputs
  conv chain and non-chain graphs with ReLU splits (alpha-beta), graphs on L2 / L1 balls, grouped / dilated convolutions
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

N_SAMPLES = 10_000


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available()
    from boundflow_b200.csrc import build

    build.build()
    return torch.device("cuda", 0)


def _layers64(layers, dev):
    return [{k: (v.to(device=dev, dtype=torch.float64) if torch.is_tensor(v) else v) for k, v in layer.items()} for layer in layers]


def _forward(layers, x, record_pre=False):
    """Concrete forward pass of a chain (float64); optionally returns the inputs of every ReLU."""
    import torch.nn.functional as F

    pre = []
    for layer in layers:
        op = layer["op"]
        if op == "linear":
            x = x.matmul(layer["W"].t())
            if layer.get("b") is not None:
                x = x + layer["b"]
        elif op == "conv2d":
            x = F.conv2d(x, layer["W"], layer.get("b"), layer["stride"], layer["padding"])
        elif op == "relu":
            if record_pre:
                pre.append(x.flatten(1))
            x = torch.relu(x)
        elif op == "flatten":
            x = x.flatten(1)
        else:
            raise NotImplementedError(op)
    return (x, pre) if record_pre else x


def _worst_violation(layers, lo, up, C, lower, upper, dev, n=N_SAMPLES, seed=0, chunk=2500):
    """max over inputs, samples and spec rows of (lower - y) and (y - upper), each divided by the tolerance of that bound."""
    L = _layers64(layers, dev)
    g = torch.Generator(device=dev).manual_seed(seed)
    worst = 0.0
    for b in range(lo.shape[0]):
        lo_b, up_b = lo[b].to(dev, torch.float64), up[b].to(dev, torch.float64)
        Cb = C[b].to(dev, torch.float64)
        lb, ub = lower[b].to(dev, torch.float64), upper[b].to(dev, torch.float64)
        tol_l, tol_u = 1e-4 + 1e-5 * lb.abs(), 1e-4 + 1e-5 * ub.abs()
        for s in range(0, n, chunk):
            m = min(chunk, n - s)
            r = torch.rand((m,) + tuple(lo_b.shape), generator=g, device=dev, dtype=torch.float64)
            if s == 0:
                r[0] = 0.0   # the corners lo and up themselves
                r[1] = 1.0
            y = _forward(L, lo_b + r * (up_b - lo_b)).matmul(Cb.t())   # [m, S]
            worst = max(worst, float(((lb - y) / tol_l).max()), float(((y - ub) / tol_u).max()))
    return worst


def test_c1_ibp_and_crown_sound_on_all_inputs(dev):
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import run_crown_ibp_mlp
    from boundflow_b200.executor import CudaTaskExecutor
    from boundflow_b200.ir import InputSpec

    wl = W.make_workload("c1")
    spec = InputSpec.box(value_name="input", lower=wl.lo.to(dev), upper=wl.up.to(dev))
    got = run_crown_ibp_mlp(wl.module, spec, linear_spec_C=wl.C.to(dev))
    w = _worst_violation(wl.layers, wl.lo, wl.up, wl.C, got.lower, got.upper, dev, seed=1)
    print(f"c1 CROWN: worst violation / tolerance = {w:.3f}")
    assert w <= 1.0
    ibp = CudaTaskExecutor().run_ibp(wl.module, spec)
    eye = torch.eye(10).unsqueeze(0).expand(wl.x.shape[0], -1, -1)
    w = _worst_violation(wl.layers, wl.lo, wl.up, eye, ibp.lower, ibp.upper, dev, seed=2)
    print(f"c1 IBP: worst violation / tolerance = {w:.3f}")
    assert w <= 1.0


@pytest.mark.parametrize("name", ["c2", "c5"])
def test_cnn_crown_with_intermediate_crown_sound(dev, name):
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import run_crown_intermediate_mlp
    from boundflow_b200.ir import InputSpec

    wl = W.make_workload(name, batch=8)
    spec = InputSpec.box(value_name="input", lower=wl.lo.to(dev), upper=wl.up.to(dev))
    bounds, _pre = run_crown_intermediate_mlp(wl.module, spec, linear_spec_C=wl.C.to(dev), chunk_rows=512)
    w = _worst_violation(wl.layers, wl.lo, wl.up, wl.C, bounds.lower, bounds.upper, dev, seed=3)
    print(f"{name} CROWN with CROWN intermediates, 8 inputs x 10^4 samples: worst violation / tolerance = {w:.3f}")
    assert w <= 1.0


def test_c3_alpha_crown_sound(dev, tc_from_256_rows):
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import AlphaState, adaptive_alpha_from_trace, ibp_trace, run_alpha_beta_crown_mlp
    from boundflow_b200.ir import InputSpec

    wl = W.make_workload("c3", batch=32)   # 288 coefficient rows: the tensor-core kernels
    spec = InputSpec.box(value_name="input", lower=wl.lo.to(dev), upper=wl.up.to(dev))
    a0 = adaptive_alpha_from_trace(ibp_trace(wl.module, spec))
    bounds, _a, _b, _s = run_alpha_beta_crown_mlp(wl.module, spec, linear_spec_C=wl.C.to(dev), steps=20, lr=0.1, per_batch_params=True,
                                                warm_start_alpha=AlphaState(dict(zip(wl.relu_names, a0))))
    sel = slice(0, 8)
    w = _worst_violation(wl.layers, wl.lo[sel], wl.up[sel], wl.C[sel], bounds.lower[sel], bounds.upper[sel], dev, seed=4)
    print(f"c3 alpha-CROWN (20 steps): worst violation / tolerance = {w:.3f}")
    assert w <= 1.0


def test_c4_split_subdomains_sound_on_constraint_satisfying_samples(dev, tc_from_256_rows):
    """Eight subdomains whose ten split neurons take the sign they have at a point of the box (so the subdomain is
    not empty); samples are the box corners, uniform points and perturbations of that point at several scales, and
    only samples that satisfy all ten split constraints are checked."""
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import bound_split_domains
    from boundflow_b200.ir import InputSpec
    from oracle import crown_oracle as O

    wl = W.make_workload("c4")
    D = 32   # 288 coefficient rows: the tensor-core kernels; the first 8 subdomains are sampled
    root = O.forward_ibp_trace(wl.layers, O.box_input(wl.lo, wl.up))
    L = _layers64(wl.layers, dev)
    g = torch.Generator(device=dev).manual_seed(9)
    lo, up = wl.lo[0].to(dev, torch.float64), wl.up[0].to(dev, torch.float64)
    anchors = lo + torch.rand((D, 784), generator=g, device=dev, dtype=torch.float64) * (up - lo)
    _y, pre_at_anchor = _forward(L, anchors, record_pre=True)
    unstable = [torch.nonzero(((l < 0) & (u > 0)).reshape(-1)).flatten().to(dev) for l, u in root.pre]
    splits = [torch.zeros(D, l.shape[1], dtype=torch.int8, device=dev) for l, _ in root.pre]
    per_layer = (3, 3, 2, 2)
    for r, idx in enumerate(unstable):
        pick = idx[torch.randint(0, len(idx), (D, per_layer[r]), generator=g, device=dev)]
        sign = torch.where(pre_at_anchor[r].gather(1, pick) >= 0, 1, -1).to(torch.int8)
        splits[r].scatter_(1, pick, sign)
    spec = InputSpec.box(value_name="input", lower=wl.lo.to(dev), upper=wl.up.to(dev))   # one box, repeated on the device
    res = bound_split_domains(wl.module, spec, linear_spec_C=wl.C.to(dev), relu_split_state=dict(zip(wl.relu_names, splits)), steps=10, lr=0.1)
    assert int(res.infeasible.sum()) == 0
    C = wl.C[0].to(dev, torch.float64)
    worst, fewest = 0.0, None
    for d in range(8):
        lb, ub = res.lower[d].to(torch.float64), res.upper[d].to(torch.float64)
        tol_l, tol_u = 1e-4 + 1e-5 * lb.abs(), 1e-4 + 1e-5 * ub.abs()
        survivors = 0
        for scale in (None, 0.3, 0.1, 0.03, 0.01):
            r = torch.rand((N_SAMPLES // 5, 784), generator=g, device=dev, dtype=torch.float64)
            if scale is None:
                x = lo + r * (up - lo)
            else:
                x = torch.minimum(torch.maximum(anchors[d] + scale * (r - 0.5) * (up - lo), lo), up)
            x[0] = anchors[d]
            y, pre = _forward(L, x, record_pre=True)
            ok = torch.ones(x.shape[0], dtype=torch.bool, device=dev)
            for rr in range(4):
                s = splits[rr][d].to(torch.float64)
                ok &= ~(((s > 0) & (pre[rr] < 0)) | ((s < 0) & (pre[rr] > 0))).any(dim=1)
            survivors += int(ok.sum())
            if ok.any():
                yy = y[ok].matmul(C.t())
                worst = max(worst, float(((lb - yy) / tol_l).max()), float(((yy - ub) / tol_u).max()))
        fewest = survivors if fewest is None else min(fewest, survivors)
    print(f"c4 alpha-CROWN on split subdomains: worst violation / tolerance = {worst:.3f}; fewest constraint-satisfying samples per subdomain = {fewest} of {N_SAMPLES}")
    assert fewest >= 1000
    assert worst <= 1.0


def _anchored_splits(fwd, lo, up, unstable, dev, per_relu=3, seed=0):
    """A split assignment per input that is satisfiable by construction: `per_relu` unstable neurons of every ReLU take the
    sign their pre-activation has at an anchor point of the box.  unstable: name -> bool [B, n].  Returns (anchors, name ->
    int8 [B, n])."""
    g = torch.Generator(device=dev).manual_seed(seed)
    B = lo.shape[0]
    lo64, up64 = lo.to(dev, torch.float64), up.to(dev, torch.float64)
    anchors = lo64 + torch.rand(lo64.shape, generator=g, device=dev, dtype=torch.float64) * (up64 - lo64)
    _y, pre = fwd(anchors)
    splits = {}
    for x, mask in unstable.items():
        s8 = torch.zeros(mask.shape, dtype=torch.int8, device=dev)
        p = pre[x].reshape(B, -1)
        for b in range(B):
            idx = torch.nonzero(mask[b].to(dev)).flatten()
            if len(idx) == 0:
                continue
            pick = idx[torch.randint(0, len(idx), (per_relu,), generator=g, device=dev)]
            s8[b, pick] = torch.where(p[b, pick] >= 0, 1, -1).to(torch.int8)
        splits[x] = s8
    return anchors, splits


def _split_soundness(name, fwd, lo, up, anchors, splits_flat, C, lower, upper, dev, n=N_SAMPLES, seed=0):
    """Worst violation / tolerance over the samples that satisfy each input's ReLU splits (uniform points of the box and
    perturbations of the anchor at several scales), and the fewest surviving samples per input.
    `fwd(x) -> (y, pre: name -> tensor)` in float64; splits_flat: name -> int8 [B, n]."""
    g = torch.Generator(device=dev).manual_seed(seed)
    worst, fewest = 0.0, None
    B = lo.shape[0]
    for b in range(B):
        lo_b, up_b = lo[b].to(dev, torch.float64), up[b].to(dev, torch.float64)
        Cb = C[b].to(dev, torch.float64)
        lb, ub = lower[b].to(dev, torch.float64), upper[b].to(dev, torch.float64)
        tol_l, tol_u = 1e-4 + 1e-5 * lb.abs(), 1e-4 + 1e-5 * ub.abs()
        survivors = 0
        for scale in (None, 0.3, 0.1, 0.03, 0.01):
            m = n // 5
            r = torch.rand((m,) + tuple(lo_b.shape), generator=g, device=dev, dtype=torch.float64)
            x = lo_b + r * (up_b - lo_b) if scale is None else torch.minimum(torch.maximum(anchors[b] + scale * (r - 0.5) * (up_b - lo_b), lo_b), up_b)
            x[0] = anchors[b]
            y, pre = fwd(x)
            ok = torch.ones(m, dtype=torch.bool, device=dev)
            for xn, s in splits_flat.items():
                sb = s[b].to(dev, torch.float64)
                p = pre[xn].reshape(m, -1)
                ok &= ~(((sb > 0) & (p < 0)) | ((sb < 0) & (p > 0))).any(dim=1)
            k = int(ok.sum())
            survivors += k
            if k:
                yy = y[ok].reshape(k, -1).matmul(Cb.t())
                worst = max(worst, float(((lb - yy) / tol_l).max()), float(((yy - ub) / tol_u).max()))
        fewest = survivors if fewest is None else min(fewest, survivors)
    print(f"{name}: worst violation / tolerance = {worst:.3f}; fewest split-satisfying samples per input = {fewest} of {n}")
    return worst, fewest


def test_conv_alpha_beta_with_splits_sound(dev):
    """alpha-beta-CROWN on the CNN c2 (4 inputs) with three split neurons on each conv ReLU and on the Linear ReLU
    (beta parameters on all three), 8 Adam steps."""
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import ibp_trace, run_alpha_beta_crown_mlp
    from boundflow_b200.ir import InputSpec

    wl = W.make_workload("c2", batch=4)
    shapes = {"h1": (16, 14, 14), "h2": (32, 7, 7), "h3": (100,)}
    spec = InputSpec.box(value_name="input", lower=wl.lo.to(dev), upper=wl.up.to(dev))
    tr = ibp_trace(wl.module, spec)
    unstable = {n: (tr.pre_l[r] < 0) & (tr.pre_u[r] > 0) for r, n in enumerate(wl.relu_names)}
    L = _layers64(wl.layers, dev)

    def fwd(x):
        y, pre = _forward(L, x, record_pre=True)
        return y, dict(zip(wl.relu_names, pre))

    anchors, flat = _anchored_splits(fwd, wl.lo, wl.up, unstable, dev, seed=20)
    splits = {n: flat[n].reshape((4,) + shapes[n]) for n in wl.relu_names}
    b, _a, bt, _s = run_alpha_beta_crown_mlp(wl.module, spec, linear_spec_C=wl.C.to(dev), relu_split_state=splits, steps=8, lr=0.1, per_batch_params=True)
    assert any(float(v.abs().max()) > 0 for v in bt.beta_by_relu_input.values()), "beta never moved"
    worst, fewest = _split_soundness("c2 alpha-beta with splits", fwd, wl.lo, wl.up, anchors, flat, wl.C, b.lower, b.upper, dev, seed=21)
    assert fewest >= 1000 and worst <= 1.0


@pytest.mark.parametrize("name", ["residual_s2", "mini_resnet", "concat_cnn", "fanout_mlp"])
def test_graph_alpha_beta_with_splits_sound(dev, name):
    """alpha-beta-CROWN on graphs that are not chains, two split neurons per ReLU and input, 6 Adam steps."""
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import run_alpha_beta_crown_mlp
    from boundflow_b200.dag import forward_ibp_dag
    from boundflow_b200.ir import InputSpec
    from oracle import graph_oracle as GO

    module, _x, lo, up, C = W.make_graph_cases()[name]
    B = int(lo.shape[0])
    spec = InputSpec.box(value_name="input", lower=lo.to(dev), upper=up.to(dev))
    tr = forward_ibp_dag(module, spec)
    unstable = {x: (tr.pre_l[x] < 0) & (tr.pre_u[x] > 0) for x in tr.pre_l}
    fwd = lambda x: GO.concrete_forward_graph(module, x, record_pre=True)  # noqa: E731
    anchors, flat = _anchored_splits(fwd, lo, up, unstable, dev, per_relu=2, seed=30)
    b, _a, _bt, _s = run_alpha_beta_crown_mlp(module, spec, linear_spec_C=None if C is None else C.to(dev), relu_split_state=flat, steps=6, lr=0.1,
                                             per_batch_params=True)
    n_out = int(b.lower.reshape(B, -1).shape[1])
    Cb = torch.eye(n_out).unsqueeze(0).expand(B, -1, -1) if C is None else (C if C.dim() == 3 else C.unsqueeze(0).expand(B, -1, -1))
    worst, fewest = _split_soundness(f"{name} alpha-beta with splits", fwd, lo, up, anchors, flat, Cb, b.lower.reshape(B, -1), b.upper.reshape(B, -1),
                                     dev, seed=31)
    assert fewest >= 1000 and worst <= 1.0


def _graph_violation(module, points, Cb, lower, upper):
    """Worst violation (in units of the parity tolerance) of C @ f(x) in [lower, upper] over points [B, n, *shape]."""
    from oracle import graph_oracle as GO

    B, n = points.shape[0], points.shape[1]
    worst = 0.0
    for b in range(B):
        y = GO.concrete_forward_graph(module, points[b]).reshape(n, -1)
        v = torch.einsum("so,no->ns", Cb[b].to(y), y)
        lo_b, up_b = lower[b].to(y), upper[b].to(y)
        tol_l, tol_u = 1e-4 + 1e-5 * lo_b.abs(), 1e-4 + 1e-5 * up_b.abs()
        worst = max(worst, float(((lo_b - v) / tol_l).max()), float(((v - up_b) / tol_u).max()))
    return worst


@pytest.mark.parametrize("name", ["fanout_mlp", "residual_s1", "concat_mlp"])
@pytest.mark.parametrize("p", [2, 1])
def test_graph_bounds_on_lp_balls_sound(dev, name, p):
    """CROWN-IBP and the per-domain alpha loop (6 steps) on L2 / L1 balls over graphs that are not chains: 10^4 points per
    input, drawn inside the ball (random directions scaled to random radii, plus points on the sphere / at the vertices)."""
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import run_alpha_beta_crown_mlp, run_crown_ibp_mlp
    from boundflow_b200.ir import InputSpec

    module, x, _lo, _up, C = W.make_graph_cases()[name]
    B = int(x.shape[0])
    eps = 0.25 if p == 2 else 0.6
    mk = InputSpec.l2 if p == 2 else InputSpec.l1
    spec = mk(value_name="input", center=x.to(dev), eps=eps)
    Cd = None if C is None else C.to(dev)
    crown = run_crown_ibp_mlp(module, spec, linear_spec_C=Cd)
    alpha, _a, _bt, _s = run_alpha_beta_crown_mlp(module, spec, linear_spec_C=Cd, steps=6, lr=0.1, per_batch_params=True)
    g = torch.Generator("cpu").manual_seed(40 + p)
    n0 = x[0].numel()
    d = torch.randn(B, N_SAMPLES, n0, generator=g, dtype=torch.float64)
    if p == 2:
        d = d / d.norm(dim=2, keepdim=True)
    else:   # L1 ball: a point of the simplex with random signs
        e = -torch.log(torch.rand(B, N_SAMPLES, n0, generator=g, dtype=torch.float64))
        d = torch.sign(d) * e / e.sum(dim=2, keepdim=True)
        k = torch.randint(0, n0, (B, N_SAMPLES // 10), generator=g)   # vertices: all of eps on one coordinate
        d[:, : N_SAMPLES // 10] = torch.nn.functional.one_hot(k, n0).double() * torch.sign(d[:, : N_SAMPLES // 10])
    r = torch.rand(B, N_SAMPLES, 1, generator=g, dtype=torch.float64) ** (1.0 / n0)
    r[:, : N_SAMPLES // 4] = 1.0   # a quarter of the points on the boundary
    pts = (x.double().reshape(B, 1, n0) + eps * r * d).reshape((B, N_SAMPLES) + tuple(x.shape[1:]))
    n_out = int(crown.lower.reshape(B, -1).shape[1])
    Cb = torch.eye(n_out).unsqueeze(0).expand(B, -1, -1) if C is None else (C if C.dim() == 3 else C.unsqueeze(0).expand(B, -1, -1))
    for what, bnd in (("CROWN", crown), ("alpha-CROWN", alpha)):
        worst = _graph_violation(module, pts, Cb.double(), bnd.lower.reshape(B, -1).cpu().double(), bnd.upper.reshape(B, -1).cpu().double())
        assert worst <= 1.0, f"{name} L{p} {what}: worst violation {worst:.2f} x tolerance"


@pytest.mark.parametrize("name", ["grouped_dilated_chain", "depthwise_residual"])
def test_grouped_and_dilated_convolutions_sound(dev, name):
    """CROWN-IBP and 6 alpha steps on the grouped / dilated convolution cases: 10^4 box samples per input through a
    float64 forward pass with torch's own grouped, dilated conv2d."""
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import run_alpha_beta_crown_mlp, run_crown_ibp_mlp
    from boundflow_b200.ir import InputSpec

    module, _x, lo, up, _C = W.make_grouped_dilated_cases()[name]
    B = int(lo.shape[0])
    spec = InputSpec.box(value_name="input", lower=lo.to(dev), upper=up.to(dev))
    crown = run_crown_ibp_mlp(module, spec)
    alpha, _a, _bt, _s = run_alpha_beta_crown_mlp(module, spec, steps=6, lr=0.1, per_batch_params=True)
    g = torch.Generator("cpu").manual_seed(50)
    u01 = torch.rand((B, N_SAMPLES) + tuple(lo.shape[1:]), generator=g, dtype=torch.float64)
    u01[:, : N_SAMPLES // 4] = torch.round(u01[:, : N_SAMPLES // 4])   # a quarter of the points at box corners
    pts = lo.double().unsqueeze(1) + u01 * (up - lo).double().unsqueeze(1)
    n_out = int(crown.lower.reshape(B, -1).shape[1])
    Cb = torch.eye(n_out, dtype=torch.float64).unsqueeze(0).expand(B, -1, -1)
    for what, bnd in (("CROWN", crown), ("alpha-CROWN", alpha)):
        worst = _graph_violation(module, pts, Cb, bnd.lower.reshape(B, -1).cpu().double(), bnd.upper.reshape(B, -1).cpu().double())
        assert worst <= 1.0, f"{name} {what}: worst violation {worst:.2f} x tolerance"
