"""Seeded synthetic verification workloads (networks, input boxes, margin specs, ReLU splits).

Five configurations, all fp32 and generated on the CPU so that every consumer
(the CUDA backend, the CPU oracle, the reference itself) sees identical bits:

  c1  MLP 784-100-100-10,            64 inputs,  eps 0.02,  IBP + CROWN
  c2  CNN 1x28x28 [16k4s2p1, 32k4s2p1, fc100, fc10], 256 inputs, eps 0.1, CROWN with CROWN intermediates
  c3  MLP 784-256x5-10,              128 inputs, eps 0.015, alpha-CROWN 20 steps lr 0.1
  c4  MLP 784-512x4-10,              1 input, eps 0.02, batches of 8192 ReLU-split subdomains, 10 alpha steps
  c5  CNN 3x32x32 [32k3s1p1, 32k4s2p1, 64k3s1p1, 64k4s2p1, fc512, fc10], 64 inputs, eps 2/255

Inputs are uniform [0,1] tensors shaped like MNIST / CIFAR images (no dataset
items are used); weights are He-normal, biases N(0, 0.1^2); the input set is the
L-inf ball clipped to [0,1], i.e. a per-element box; the 9 spec rows per input
are logit[y] - logit[j], j != y, with y the clean arg-max.

The module layout mirrors the reference's hand-built test fixtures
(tests/test_phase6b_crown_ibp_mlp.py:10-27 in the reference): a single
INTERVAL_IBP task whose ops are linear/conv2d/relu/flatten with parameters in
`module.bindings["params"]`.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .ir import BFTaskModule, BoundTask, TaskKind, TaskOp


@dataclass
class NetSpec:
    input_shape: Tuple[int, ...]
    # ("conv", out_ch, k, stride, pad) | ("fc", out)
    body: Sequence[tuple]


NETS: Dict[str, NetSpec] = {
    "c1": NetSpec((784,), [("fc", 100), ("fc", 100), ("fc", 10)]),
    "c2": NetSpec((1, 28, 28), [("conv", 16, 4, 2, 1), ("conv", 32, 4, 2, 1), ("fc", 100), ("fc", 10)]),
    "c3": NetSpec((784,), [("fc", 256)] * 5 + [("fc", 10)]),
    "c4": NetSpec((784,), [("fc", 512)] * 4 + [("fc", 10)]),
    "c5": NetSpec(
        (3, 32, 32),
        [("conv", 32, 3, 1, 1), ("conv", 32, 4, 2, 1), ("conv", 64, 3, 1, 1), ("conv", 64, 4, 2, 1), ("fc", 512), ("fc", 10)],
    ),
}
DEFAULTS = {
    "c1": dict(batch=64, eps=0.02),
    "c2": dict(batch=256, eps=0.1),
    "c3": dict(batch=128, eps=0.015),
    "c4": dict(batch=1, eps=0.02),
    "c5": dict(batch=64, eps=2.0 / 255.0),
}
SEEDS = {"c1": 1001, "c2": 1002, "c3": 1003, "c4": 1004, "c5": 1005}


@dataclass
class Workload:
    name: str
    module: BFTaskModule
    layers: List[dict]            # chain description (op dicts holding CPU tensors)
    x: torch.Tensor               # [B, *input_shape]
    lo: torch.Tensor              # clipped box lower
    up: torch.Tensor              # clipped box upper
    C: torch.Tensor               # [B, 9, 10]
    labels: torch.Tensor          # [B]
    eps: float
    relu_names: List[str] = field(default_factory=list)
    generator: Optional[torch.Generator] = None


def build_chain(spec: NetSpec, g: torch.Generator, *, scale: Optional[Sequence[int]] = None):
    """Draw the parameters in layer order and return (layers, module)."""
    layers: List[dict] = []
    ops: List[TaskOp] = []
    params: Dict[str, torch.Tensor] = {}
    shape = tuple(spec.input_shape)
    cur = "input"
    relu_names: List[str] = []
    body = list(spec.body)
    for k, item in enumerate(body, start=1):
        last = k == len(body)
        if item[0] == "conv":
            _, oc, ks, st, pd = item
            ic, h, w = shape
            fan_in = ic * ks * ks
            W = torch.randn((oc, ic, ks, ks), generator=g) * math.sqrt(2.0 / fan_in)
            b = torch.randn((oc,), generator=g) * 0.1
            ho = (h + 2 * pd - ks) // st + 1
            wo = (w + 2 * pd - ks) // st + 1
            layers.append({"op": "conv2d", "W": W, "b": b, "stride": (st, st), "padding": (pd, pd)})
            out = f"h{k}"
            ops.append(TaskOp("conv2d", f"conv{k}", [cur, f"W{k}", f"b{k}"], [out], {"stride": (st, st), "padding": (pd, pd)}))
            shape = (oc, ho, wo)
        else:
            if len(shape) == 3:
                layers.append({"op": "flatten"})
                flat = f"f{k}"
                ops.append(TaskOp("flatten", f"flatten{k}", [cur], [flat], {"start_dim": 1, "end_dim": -1}))
                cur = flat
                shape = (shape[0] * shape[1] * shape[2],)
            n_out = int(item[1])
            fan_in = shape[0]
            W = torch.randn((n_out, fan_in), generator=g) * math.sqrt(2.0 / fan_in)
            b = torch.randn((n_out,), generator=g) * 0.1
            layers.append({"op": "linear", "W": W, "b": b})
            out = "out" if last else f"h{k}"
            ops.append(TaskOp("linear", f"linear{k}", [cur, f"W{k}", f"b{k}"], [out]))
            shape = (n_out,)
        params[f"W{k}"] = W
        params[f"b{k}"] = b
        cur = out
        if not last:
            layers.append({"op": "relu"})
            relu_names.append(cur)
            ops.append(TaskOp("relu", f"relu{k}", [cur], [f"r{k}"]))
            cur = f"r{k}"
    task = BoundTask(task_id="t0", kind=TaskKind.INTERVAL_IBP, ops=ops, input_values=["input"], output_values=["out"])
    module = BFTaskModule(tasks=[task], entry_task_id="t0", bindings={"params": params})
    return layers, module, relu_names


def clean_forward(layers: List[dict], x: torch.Tensor) -> torch.Tensor:
    import torch.nn.functional as F

    for layer in layers:
        op = layer["op"]
        if op == "linear":
            x = x.matmul(layer["W"].t()) + layer["b"]
        elif op == "conv2d":
            x = F.conv2d(x, layer["W"], layer["b"], layer["stride"], layer["padding"])
        elif op == "relu":
            x = torch.relu(x)
        elif op == "flatten":
            x = x.flatten(1)
    return x


def margin_specs(logits: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """C[b,k,:] = e_y - e_j for the k-th j != y in ascending j."""
    B, O = logits.shape
    y = logits.argmax(dim=1)
    C = torch.zeros(B, O - 1, O, dtype=logits.dtype)
    for b in range(B):
        k = 0
        for j in range(O):
            if j == int(y[b]):
                continue
            C[b, k, int(y[b])] = 1.0
            C[b, k, j] = -1.0
            k += 1
    return C, y


def make_workload(name: str, *, batch: Optional[int] = None, eps: Optional[float] = None, net: Optional[NetSpec] = None, seed: Optional[int] = None) -> Workload:
    """Build configuration `name` (c1..c5); `batch` draws only the first inputs
    of the same stream so a reduced batch is a prefix of the full one."""
    spec = net or NETS[name]
    d = DEFAULTS[name]
    full_batch = int(d["batch"])
    B = int(batch) if batch is not None else full_batch
    e = float(eps) if eps is not None else float(d["eps"])
    g = torch.Generator("cpu").manual_seed(int(seed) if seed is not None else SEEDS[name])
    layers, module, relu_names = build_chain(spec, g)
    x_full = torch.rand((max(B, full_batch),) + tuple(spec.input_shape), generator=g)
    x = x_full[:B].contiguous()
    logits = clean_forward(layers, x)
    C, y = margin_specs(logits)
    lo = torch.clamp(x - e, min=0.0)
    up = torch.clamp(x + e, max=1.0)
    return Workload(name=name, module=module, layers=layers, x=x, lo=lo, up=up, C=C, labels=y, eps=e, relu_names=relu_names, generator=g)


def make_split_domains(wl: Workload, root_pre: Sequence[Tuple[torch.Tensor, torch.Tensor]], *, n_domains: int, n_split: int = 10) -> List[torch.Tensor]:
    """ReLU-split subdomains of the single-input configuration (c4).

    `root_pre` are the root's pre-activation bounds per ReLU ([1,n_k] each).
    For every domain, `n_split` neurons are drawn without replacement from the
    root's unstable set (l<0<u) and assigned active(+1)/inactive(-1) with equal
    probability.  Returns one int8 [n_domains, n_k] tensor per ReLU.  Draws
    continue the workload's generator stream, so they are reproducible.
    """
    g = wl.generator
    unstable: List[Tuple[int, int]] = []
    for r, (l, u) in enumerate(root_pre):
        lf, uf = l.reshape(-1), u.reshape(-1)
        idx = torch.nonzero((lf < 0) & (uf > 0)).flatten().tolist()
        unstable.extend((r, j) for j in idx)
    if len(unstable) < n_split:
        raise ValueError(f"only {len(unstable)} unstable neurons at the root, need {n_split}")
    splits = [torch.zeros(n_domains, l.reshape(-1).shape[0], dtype=torch.int8) for l, _ in root_pre]
    U = len(unstable)
    for d in range(n_domains):
        pick = torch.randperm(U, generator=g)[:n_split].tolist()
        sign = torch.rand(n_split, generator=g) < 0.5
        for t, p in enumerate(pick):
            r, j = unstable[p]
            splits[r][d, j] = 1 if bool(sign[t]) else -1
    return splits


def make_certificate_cases(seed: int = 1009):
    """Small MLP 12-16-5 and split rows on its first ReLU that exercise the first-layer infeasibility
    certificate: rows 1 and 2 of the first layer are negative multiples of row 0 (shifted down), so
    "neuron 0 active" contradicts "neuron 1 active" (found with uniform weights) and "neuron 2 active"
    (needs the optimiser: the best weights are 2/3, 1/3).  Returns (module, layers, x, lo, up, cases)
    with cases = list of (name, int8 split row [16])."""
    g = torch.Generator("cpu").manual_seed(seed)
    n0, n1, n2 = 12, 16, 5
    W1 = torch.randn(n1, n0, generator=g) * math.sqrt(2.0 / n0)
    b1 = torch.randn(n1, generator=g) * 0.1
    W2 = torch.randn(n2, n1, generator=g) * math.sqrt(2.0 / n1)
    b2 = torch.randn(n2, generator=g) * 0.1
    x = torch.rand(1, n0, generator=g)
    b1[0] = b1[0] - (W1[0] @ x[0] + b1[0])  # neuron 0 is zero at the centre: unstable over the box
    W1[1], b1[1] = -W1[0], -b1[0] - 0.05
    W1[2], b1[2] = -2.0 * W1[0], -2.0 * b1[0] - 0.09
    lo, up = (x - 0.3).clamp(0, 1), (x + 0.3).clamp(0, 1)
    params = {"W1": W1, "b1": b1, "W2": W2, "b2": b2}
    ops = [TaskOp("linear", "fc1", ["input", "W1", "b1"], ["h1"]), TaskOp("relu", "relu1", ["h1"], ["r1"]),
           TaskOp("linear", "fc2", ["r1", "W2", "b2"], ["out"])]
    task = BoundTask(task_id="t0", kind=TaskKind.INTERVAL_IBP, ops=ops, input_values=["input"], output_values=["out"])
    module = BFTaskModule(tasks=[task], entry_task_id="t0", bindings={"params": params})
    layers = [{"op": "linear", "W": W1, "b": b1}, {"op": "relu"}, {"op": "linear", "W": W2, "b": b2}]

    def row(**kw):
        r = torch.zeros(n1, dtype=torch.int8)
        for k, v in kw.items():
            r[int(k[1:])] = v
        return r

    pre_l = (W1.clamp(min=0) @ lo[0] + W1.clamp(max=0) @ up[0] + b1)
    pre_u = (W1.clamp(min=0) @ up[0] + W1.clamp(max=0) @ lo[0] + b1)
    unstable = [int(j) for j in torch.nonzero((pre_l < 0) & (pre_u > 0)).reshape(-1) if int(j) > 2]
    off = [int(j) for j in torch.nonzero(pre_u < 0).reshape(-1)]
    cases = [
        ("no_split", row()),
        ("one_feasible", row(n0=1)),
        ("pair_contradiction_uniform_weights", row(n0=1, n1=1)),
        ("pair_contradiction_needs_steps", row(n0=1, n2=1)),
        ("triple_with_bystander", row(**{"n0": 1, "n2": 1, f"n{unstable[0]}": -1})),
        ("feasible_pair", row(**{f"n{unstable[0]}": 1, f"n{unstable[1]}": -1})),
    ]
    if off:
        cases.append(("single_halfspace_infeasible", row(**{f"n{off[0]}": 1})))
    return module, layers, x, lo, up, cases


def make_conv_certificate_cases(seed: int = 1013):
    """Small CNN (1x6x6 -> conv 4 channels k3 s1 p1 -> ReLU -> flatten -> Linear 5) and split rows on its first
    ReLU for the first-layer infeasibility certificate over a Conv2d first layer: filter 1 is minus filter 0 (shifted
    down) and filter 2 is minus twice filter 0, so at one pixel "channel 0 active" contradicts "channel 1 active"
    (uniform weights) and "channel 2 active" (needs the optimiser); a border pixel exercises the taps that fall into
    the padding.  Returns (module, layers, x, lo, up, cases) with cases = list of (name, int8 split row [144])."""
    g = torch.Generator("cpu").manual_seed(seed)
    Co, H = 4, 6
    Wc = torch.randn(Co, 1, 3, 3, generator=g) * math.sqrt(2.0 / 9)
    bc = torch.randn(Co, generator=g) * 0.1
    x = torch.rand(1, 1, H, H, generator=g)
    z0 = torch.nn.functional.conv2d(x, Wc[:1], None, 1, 1)[0, 0]
    bc[0] = -z0[2, 3]  # channel 0 is zero at pixel (2,3) at the centre: unstable over the box
    Wc[1], bc[1] = -Wc[0], -bc[0] - 0.05
    Wc[2], bc[2] = -2.0 * Wc[0], -2.0 * bc[0] - 0.09
    W2 = torch.randn(5, Co * H * H, generator=g) * math.sqrt(2.0 / (Co * H * H))
    b2 = torch.randn(5, generator=g) * 0.1
    lo, up = (x - 0.3).clamp(0, 1), (x + 0.3).clamp(0, 1)
    params = {"Wc": Wc, "bc": bc, "W2": W2, "b2": b2}
    ops = [TaskOp("conv2d", "conv1", ["input", "Wc", "bc"], ["h1"], attrs={"stride": 1, "padding": 1}),
           TaskOp("relu", "relu1", ["h1"], ["r1"]), TaskOp("flatten", "flat", ["r1"], ["f1"], attrs={"start_dim": 1, "end_dim": -1}),
           TaskOp("linear", "fc", ["f1", "W2", "b2"], ["out"])]
    task = BoundTask(task_id="t0", kind=TaskKind.INTERVAL_IBP, ops=ops, input_values=["input"], output_values=["out"])
    module = BFTaskModule(tasks=[task], entry_task_id="t0", bindings={"params": params})
    layers = [{"op": "conv2d", "W": Wc, "b": bc, "stride": (1, 1), "padding": (1, 1)}, {"op": "relu"}, {"op": "flatten"},
              {"op": "linear", "W": W2, "b": b2}]

    def row(*entries):
        r = torch.zeros(Co * H * H, dtype=torch.int8)
        for (c, h, w, v) in entries:
            r[(c * H + h) * H + w] = v
        return r

    cases = [
        ("no_split", row()),
        ("one_feasible", row((0, 2, 3, 1))),
        ("pair_contradiction_uniform_weights", row((0, 2, 3, 1), (1, 2, 3, 1))),
        ("pair_contradiction_needs_steps", row((0, 2, 3, 1), (2, 2, 3, 1))),
        ("border_pixel_contradiction", row((0, 0, 0, 1), (1, 0, 0, 1))),
        ("different_pixels", row((0, 2, 3, 1), (1, 4, 1, 1))),
        ("triple_with_bystander", row((0, 2, 3, 1), (2, 2, 3, 1), (3, 1, 1, -1))),
        ("feasible_pair", row((0, 2, 3, 1), (3, 1, 1, -1))),
    ]
    return module, layers, x, lo, up, cases


def make_graph_certificate_cases(kind: str = "linear", seed: int = 1019):
    """Two-branch graph for the first-layer infeasibility certificate on a graph that is not a chain: branches "ha" (6
    neurons) and "hb" (2 neurons) both read the input, a ReLU on each, concat, Linear head.  kind "linear": the input is a
    vector of 8 and the branches are Linear ops; kind "conv": the input is 2x2x2 and the branches are Conv2d ops with
    2x2 kernels (one output pixel, the same weights reshaped), so both kinds pose the same half-spaces.  Row 0 of
    branch a is pinned to be unstable; row 0 of branch b is minus that row (so "ha[0] active" contradicts "hb[0] active"
    across the two ReLUs, uniform weights) and row 1 is minus twice the row (needs the optimiser).
    Returns (module, x, lo, up, cases) with cases = list of (name, {"ha": int8 [6], "hb": int8 [2]})."""
    if kind not in ("linear", "conv"):
        raise ValueError(kind)
    g = torch.Generator("cpu").manual_seed(seed)
    Wa = torch.randn(6, 8, generator=g) * 0.5
    ba = torch.randn(6, generator=g) * 0.1
    x = torch.rand(1, 8, generator=g)
    ba[0] = -float(Wa[0] @ x.reshape(-1))   # ha[0] is zero at the centre: unstable over the box
    Wb = torch.stack([-Wa[0], -2.0 * Wa[0]])
    bb = torch.stack([-ba[0] - 0.05, -2.0 * ba[0] - 0.09])
    Wh = torch.randn(3, 8, generator=g) * 0.5
    bh = torch.randn(3, generator=g) * 0.1
    lo, up = (x - 0.3).clamp(0, 1), (x + 0.3).clamp(0, 1)
    if kind == "linear":
        ops = [TaskOp("linear", "branch_a", ["input", "Wa", "ba"], ["ha"]), TaskOp("relu", "relu_a", ["ha"], ["ra"]),
               TaskOp("linear", "branch_b", ["input", "Wb", "bb"], ["hb"]), TaskOp("relu", "relu_b", ["hb"], ["rb"]),
               TaskOp("concat", "cat", ["ra", "rb"], ["hc"], {"axis": 1}), TaskOp("linear", "head", ["hc", "Wh", "bh"], ["out"])]
        params = {"Wa": Wa, "ba": ba, "Wb": Wb, "bb": bb, "Wh": Wh, "bh": bh}
    else:
        k2 = {"stride": (1, 1), "padding": (0, 0), "dilation": (1, 1), "groups": 1}
        ops = [TaskOp("conv2d", "branch_a", ["input", "Wa", "ba"], ["ha"], k2), TaskOp("relu", "relu_a", ["ha"], ["ra"]),
               TaskOp("conv2d", "branch_b", ["input", "Wb", "bb"], ["hb"], k2), TaskOp("relu", "relu_b", ["hb"], ["rb"]),
               TaskOp("concat", "cat", ["ra", "rb"], ["hc"], {"axis": 1}),
               TaskOp("flatten", "flatten", ["hc"], ["flat"], {"start_dim": 1, "end_dim": -1}), TaskOp("linear", "head", ["flat", "Wh", "bh"], ["out"])]
        params = {"Wa": Wa.reshape(6, 2, 2, 2).clone(), "ba": ba, "Wb": Wb.reshape(2, 2, 2, 2).clone(), "bb": bb, "Wh": Wh, "bh": bh}
        x, lo, up = x.reshape(1, 2, 2, 2), lo.reshape(1, 2, 2, 2), up.reshape(1, 2, 2, 2)
    task = BoundTask(task_id="graph_cert", kind=TaskKind.INTERVAL_IBP, ops=ops, input_values=["input"], output_values=["out"])
    module = BFTaskModule(tasks=[task], entry_task_id="graph_cert", bindings={"params": params})

    def rows(a=(), b=()):
        ra, rb = torch.zeros(6, dtype=torch.int8), torch.zeros(2, dtype=torch.int8)
        for i, v in a:
            ra[i] = v
        for i, v in b:
            rb[i] = v
        return {"ha": ra, "hb": rb}

    cases = [
        ("no_split", rows()),
        ("one_feasible", rows(a=[(0, 1)])),
        ("cross_branch_contradiction_uniform_weights", rows(a=[(0, 1)], b=[(0, 1)])),
        ("cross_branch_contradiction_needs_steps", rows(a=[(0, 1)], b=[(1, 1)])),
        ("cross_branch_feasible", rows(a=[(0, 1)], b=[(0, -1)])),
        ("second_branch_only", rows(b=[(0, 1), (1, 1)])),
        ("triple_with_bystander", rows(a=[(0, 1), (3, -1)], b=[(1, 1)])),
    ]
    return module, x, lo, up, cases


def make_grouped_dilated_cases(seed: int = 1021):
    """Conv2d ops with groups and dilation: a chain (4x10x10 -> conv 8 ch k3 p1 groups 2 -> ReLU -> conv 8 ch k3 p2
    dilation 2 groups 4 -> ReLU -> flatten -> Linear 5) and a residual graph whose main branch is a depthwise 3x3
    convolution (groups = channels) beside a 1x1 skip.  Returns {name: (module, x, lo, up, C)}."""
    g = torch.Generator("cpu").manual_seed(seed)

    def rn(*shape, fan):
        return torch.randn(*shape, generator=g) * math.sqrt(2.0 / fan)

    def mod(tid, ops, params):
        task = BoundTask(task_id=tid, kind=TaskKind.INTERVAL_IBP, ops=ops, input_values=["input"], output_values=["out"])
        return BFTaskModule(tasks=[task], entry_task_id=tid, bindings={"params": params})

    cases = {}
    ops = [
        TaskOp("conv2d", "conv1", ["input", "w1", "b1"], ["h1"], {"stride": (1, 1), "padding": (1, 1), "dilation": (1, 1), "groups": 2}),
        TaskOp("relu", "relu1", ["h1"], ["r1"]),
        TaskOp("conv2d", "conv2", ["r1", "w2", "b2"], ["h2"], {"stride": (1, 1), "padding": (2, 2), "dilation": (2, 2), "groups": 4}),
        TaskOp("relu", "relu2", ["h2"], ["r2"]),
        TaskOp("flatten", "flatten", ["r2"], ["flat"], {"start_dim": 1, "end_dim": -1}),
        TaskOp("linear", "head", ["flat", "wh", "bh"], ["out"]),
    ]
    params = {"w1": rn(8, 2, 3, 3, fan=18), "b1": rn(8, fan=200), "w2": rn(8, 2, 3, 3, fan=18), "b2": rn(8, fan=200),
              "wh": rn(5, 800, fan=800), "bh": rn(5, fan=200)}
    x = torch.rand(3, 4, 10, 10, generator=g)
    cases["grouped_dilated_chain"] = (mod("gd_chain", ops, params), x, (x - 0.03).clamp(0, 1), (x + 0.03).clamp(0, 1), None)
    ops = [
        TaskOp("conv2d", "depthwise", ["input", "wd", "bd"], ["hd"], {"stride": (2, 2), "padding": (1, 1), "dilation": (1, 1), "groups": 3}),
        TaskOp("relu", "relu_d", ["hd"], ["rd"]),
        TaskOp("conv2d", "skip", ["input", "ws", "bs"], ["hs"], {"stride": (2, 2), "padding": (0, 0), "dilation": (1, 1), "groups": 1}),
        TaskOp("add", "merge", ["rd", "hs"], ["sum"]),
        TaskOp("relu", "relu_out", ["sum"], ["rout"]),
        TaskOp("flatten", "flatten", ["rout"], ["flat"], {"start_dim": 1, "end_dim": -1}),
        TaskOp("linear", "head", ["flat", "wh", "bh"], ["out"]),
    ]
    params = {"wd": rn(3, 1, 3, 3, fan=9), "bd": rn(3, fan=200), "ws": rn(3, 3, 1, 1, fan=3), "bs": rn(3, fan=200),
              "wh": rn(4, 48, fan=48), "bh": rn(4, fan=200)}
    x = torch.rand(2, 3, 8, 8, generator=g)
    cases["depthwise_residual"] = (mod("dw_residual", ops, params), x, (x - 0.04).clamp(0, 1), (x + 0.04).clamp(0, 1), None)
    return cases


def make_executor_op_cases(seed: int = 1023):
    """Small modules with the op types that only the interval executors handle (task_executor.py:184-350): an elementwise
    product of two branches, a permute behind a convolution and a `spec_linear` output op.
    Returns {name: (module, x, lo, up)}."""
    g = torch.Generator("cpu").manual_seed(seed)

    def rn(*shape, fan):
        return torch.randn(*shape, generator=g) * math.sqrt(2.0 / fan)

    def mod(tid, ops, params):
        task = BoundTask(task_id=tid, kind=TaskKind.INTERVAL_IBP, ops=ops, input_values=["input"], output_values=["out"])
        return BFTaskModule(tasks=[task], entry_task_id=tid, bindings={"params": params})

    def box(x, eps):
        return (x - eps).clamp(0, 1), (x + eps).clamp(0, 1)

    k3 = {"stride": (1, 1), "padding": (1, 1), "dilation": (1, 1), "groups": 1}
    cases = {}
    ops = [TaskOp("linear", "a", ["input", "wa", "ba"], ["ha"]), TaskOp("linear", "b", ["input", "wb", "bb"], ["hb"]),
           TaskOp("relu", "gate", ["hb"], ["rb"]), TaskOp("mul", "product", ["ha", "rb"], ["m"]), TaskOp("linear", "head", ["m", "wh", "bh"], ["out"])]
    params = {"wa": rn(5, 6, fan=6), "ba": rn(5, fan=50), "wb": rn(5, 6, fan=6), "bb": rn(5, fan=50), "wh": rn(3, 5, fan=5), "bh": rn(3, fan=50)}
    x = torch.rand(4, 6, generator=g)
    cases["mul_gate"] = (mod("mul_gate", ops, params), x) + box(x, 0.08)
    ops = [TaskOp("conv2d", "conv", ["input", "wc", "bc"], ["hc"], k3), TaskOp("relu", "relu", ["hc"], ["rc"]),
           TaskOp("permute", "to_nhwc", ["rc"], ["pc"], {"dims": [0, 2, 3, 1]}),
           TaskOp("flatten", "flatten", ["pc"], ["flat"], {"start_dim": 1, "end_dim": -1}), TaskOp("linear", "head", ["flat", "wh", "bh"], ["out"])]
    params = {"wc": rn(3, 2, 3, 3, fan=18), "bc": rn(3, fan=50), "wh": rn(4, 48, fan=48), "bh": rn(4, fan=50)}
    x = torch.rand(3, 2, 4, 4, generator=g)
    cases["permute_cnn"] = (mod("permute_cnn", ops, params), x) + box(x, 0.05)
    ops = [TaskOp("linear", "body", ["input", "w1", "b1"], ["h1"]), TaskOp("relu", "relu", ["h1"], ["r1"]),
           TaskOp("linear", "logits", ["r1", "w2", "b2"], ["logits"]), TaskOp("spec_linear", "spec", ["logits", "Cspec"], ["out"])]
    params = {"w1": rn(7, 6, fan=6), "b1": rn(7, fan=50), "w2": rn(4, 7, fan=7), "b2": rn(4, fan=50), "Cspec": torch.randn(5, 3, 4, generator=g)}
    x = torch.rand(5, 6, generator=g)
    cases["spec_linear"] = (mod("spec_linear", ops, params), x) + box(x, 0.06)
    return cases


def make_graph_cases(seed: int = 1011):
    """Small graphs that are not chains, shaped like the reference's end-to-end fixtures
    (tests/test_phase7a_pr12_e2e_crown_runtime.py:98-239): a residual CNN block with a projection skip
    (stride 1 and stride 2), an MLP whose hidden value feeds a ReLU path and a direct path (fan-out),
    and a two-block mini ResNet.  Returns {name: (module, x, lo, up, C)}; weights are scaled He-normal."""
    g = torch.Generator("cpu").manual_seed(seed)

    def rn(*shape, fan):
        return torch.randn(*shape, generator=g) * math.sqrt(2.0 / fan)

    def mod(tid, ops, params):
        task = BoundTask(task_id=tid, kind=TaskKind.INTERVAL_IBP, ops=ops, input_values=["input"], output_values=["out"])
        return BFTaskModule(tasks=[task], entry_task_id=tid, bindings={"params": params})

    def box(x, eps):
        return (x - eps).clamp(0, 1), (x + eps).clamp(0, 1)

    cases = {}
    for name, down in (("residual_s1", False), ("residual_s2", True)):
        st, sp = ((2, 2), 4) if down else ((1, 1), 7)
        ops = [
            TaskOp("conv2d", "main1", ["input", "wm1", "bm1"], ["hm1"], {"stride": st, "padding": (1, 1), "dilation": (1, 1), "groups": 1}),
            TaskOp("relu", "main_relu", ["hm1"], ["rm1"]),
            TaskOp("conv2d", "main2", ["rm1", "wm2", "bm2"], ["hm2"], {"stride": (1, 1), "padding": (1, 1), "dilation": (1, 1), "groups": 1}),
            TaskOp("conv2d", "skip", ["input", "ws", "bs"], ["hs"], {"stride": st, "padding": (0, 0), "dilation": (1, 1), "groups": 1}),
            TaskOp("add", "merge", ["hm2", "hs"], ["sum"]),
            TaskOp("relu", "out_relu", ["sum"], ["rout"]),
            TaskOp("flatten", "flatten", ["rout"], ["flat"], {"start_dim": 1, "end_dim": -1}),
            TaskOp("linear", "head", ["flat", "wh", "bh"], ["out"]),
        ]
        params = {"wm1": rn(3, 2, 3, 3, fan=18), "bm1": rn(3, fan=200), "wm2": rn(3, 3, 3, 3, fan=27), "bm2": rn(3, fan=200),
                  "ws": rn(3, 2, 1, 1, fan=2), "bs": rn(3, fan=200), "wh": rn(4, 3 * sp * sp, fan=3 * sp * sp), "bh": rn(4, fan=200)}
        x = torch.rand(3, 2, 7, 7, generator=g)
        cases[name] = (mod(name, ops, params), x) + box(x, 0.05) + (None,)
    ops = [
        TaskOp("linear", "shared", ["input", "w1", "b1"], ["h"]), TaskOp("relu", "relu", ["h"], ["r"]),
        TaskOp("linear", "direct", ["h", "wd", "bd"], ["d"]), TaskOp("linear", "relu_path", ["r", "wr", "br"], ["q"]),
        TaskOp("add", "merge", ["d", "q"], ["out"]),
    ]
    params = {"w1": rn(24, 10, fan=10), "b1": rn(24, fan=200), "wd": rn(6, 24, fan=24), "bd": rn(6, fan=200), "wr": rn(6, 24, fan=24), "br": rn(6, fan=200)}
    x = torch.rand(5, 10, generator=g)
    cases["fanout_mlp"] = (mod("fanout", ops, params), x) + box(x, 0.1) + (torch.randn(5, 3, 6, generator=g),)
    conv = {"stride": (1, 1), "padding": (1, 1), "dilation": (1, 1), "groups": 1}
    down = {"stride": (2, 2), "padding": (1, 1), "dilation": (1, 1), "groups": 1}
    proj = {"stride": (2, 2), "padding": (0, 0), "dilation": (1, 1), "groups": 1}
    ops = [
        TaskOp("conv2d", "stem", ["input", "ws", "bs"], ["hs"], conv), TaskOp("relu", "stem_relu", ["hs"], ["r0"]),
        TaskOp("conv2d", "b1c1", ["r0", "w11", "b11"], ["h11"], conv), TaskOp("relu", "b1_relu", ["h11"], ["r11"]),
        TaskOp("conv2d", "b1c2", ["r11", "w12", "b12"], ["h12"], conv), TaskOp("add", "b1_add", ["r0", "h12"], ["s1"]),
        TaskOp("relu", "b1_out", ["s1"], ["r1"]),
        TaskOp("conv2d", "b2c1", ["r1", "w21", "b21"], ["h21"], down), TaskOp("relu", "b2_relu", ["h21"], ["r21"]),
        TaskOp("conv2d", "b2c2", ["r21", "w22", "b22"], ["h22"], conv), TaskOp("conv2d", "b2_skip", ["r1", "wp", "bp"], ["hp"], proj),
        TaskOp("add", "b2_add", ["h22", "hp"], ["s2"]), TaskOp("relu", "b2_out", ["s2"], ["r2"]),
        TaskOp("flatten", "flatten", ["r2"], ["flat"], {"start_dim": 1, "end_dim": -1}),
        TaskOp("linear", "head", ["flat", "wh", "bh"], ["out"]),
    ]
    c0, c1 = 4, 6
    params = {"ws": rn(c0, 3, 3, 3, fan=27), "bs": rn(c0, fan=200), "w11": rn(c0, c0, 3, 3, fan=9 * c0), "b11": rn(c0, fan=200),
              "w12": rn(c0, c0, 3, 3, fan=9 * c0), "b12": rn(c0, fan=200), "w21": rn(c1, c0, 3, 3, fan=9 * c0), "b21": rn(c1, fan=200),
              "w22": rn(c1, c1, 3, 3, fan=9 * c1), "b22": rn(c1, fan=200), "wp": rn(c1, c0, 1, 1, fan=c0), "bp": rn(c1, fan=200),
              "wh": rn(5, c1 * 4 * 4, fan=c1 * 16), "bh": rn(5, fan=200)}
    x = torch.rand(2, 3, 8, 8, generator=g)
    cases["mini_resnet"] = (mod("mini_resnet", ops, params), x) + box(x, 0.02) + (None,)
    # channel concatenation of two conv branches, and feature concatenation of two linear branches
    k3 = {"stride": (1, 1), "padding": (1, 1), "dilation": (1, 1), "groups": 1}
    k1 = {"stride": (1, 1), "padding": (0, 0), "dilation": (1, 1), "groups": 1}
    ops = [
        TaskOp("conv2d", "branch_a", ["input", "wa", "ba"], ["ha"], k3), TaskOp("conv2d", "branch_b", ["input", "wb", "bb"], ["hb"], k1),
        TaskOp("concat", "cat", ["ha", "hb"], ["hc"], {"axis": 1}), TaskOp("relu", "relu1", ["hc"], ["rc"]),
        TaskOp("conv2d", "down", ["rc", "wd", "bd"], ["hd"], down), TaskOp("relu", "relu2", ["hd"], ["rd"]),
        TaskOp("flatten", "flatten", ["rd"], ["flat"], {"start_dim": 1, "end_dim": -1}),
        TaskOp("linear", "head", ["flat", "wh", "bh"], ["out"]),
    ]
    params = {"wa": rn(2, 3, 3, 3, fan=27), "ba": rn(2, fan=200), "wb": rn(3, 3, 1, 1, fan=3), "bb": rn(3, fan=200),
              "wd": rn(4, 5, 3, 3, fan=45), "bd": rn(4, fan=200), "wh": rn(3, 4 * 3 * 3, fan=36), "bh": rn(3, fan=200)}
    x = torch.rand(2, 3, 6, 6, generator=g)
    cases["concat_cnn"] = (mod("concat_cnn", ops, params), x) + box(x, 0.03) + (None,)
    ops = [
        TaskOp("linear", "left", ["input", "wl", "bl"], ["hl"]), TaskOp("linear", "right", ["input", "wr", "br"], ["hr"]),
        TaskOp("relu", "relu_l", ["hl"], ["rl"]),
        TaskOp("concat", "cat", ["rl", "hr"], ["hc"], {"axis": -1}), TaskOp("relu", "relu_c", ["hc"], ["rc"]),
        TaskOp("linear", "head", ["rc", "wh", "bh"], ["out"]),
    ]
    params = {"wl": rn(7, 9, fan=9), "bl": rn(7, fan=200), "wr": rn(5, 9, fan=9), "br": rn(5, fan=200), "wh": rn(4, 12, fan=12), "bh": rn(4, fan=200)}
    x = torch.rand(4, 9, generator=g)
    cases["concat_mlp"] = (mod("concat_mlp", ops, params), x) + box(x, 0.08) + (torch.randn(4, 2, 4, generator=g),)
    return cases
