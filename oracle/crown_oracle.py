"""CPU restatement of BoundFlow's IBP -> CROWN -> concretise -> alpha-CROWN path.

TEST INFRASTRUCTURE ONLY.  This module is the checker for the CUDA kernels: the
test-suite, the smoke check and the benchmark's CPU-baseline leg may import it;
nothing in the shipped package does.  It uses plain torch CPU tensor ops (the
reference's own arithmetic library), is dtype generic (float32 / float64) and
follows the reference function by function; every function cites the reference
file:line it restates (paths are relative to the reference project root).

Parity status: PINNED.  `tests/golden/make_golden.py` runs the reference's own
functions (imported from the reference checkout) on seeded inputs and stores
their outputs under `tests/golden/*.npz`; `tests/test_oracle_golden.py` checks
this restatement against those vectors and against the literal known-answer
cases the reference's tests hold.

Network description used throughout: a chain `layers`, a list of dicts
  {"op": "linear", "W": [out,in], "b": [out] or None}
  {"op": "conv2d", "W": [O,I,kh,kw], "b": [O] or None, "stride": (sh,sw), "padding": (ph,pw)}
  {"op": "relu"}
  {"op": "flatten"}
The input set is a per-element box [lo, up] (an L-inf ball is the box
[x0-eps, x0+eps] with midpoint x0 and radius eps, see `linf_box`).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

Layers = List[dict]


def layers_to(layers: "Layers", dtype: torch.dtype) -> "Layers":
    """The same chain with its parameters cast to `dtype` (float64 evaluations serve as "truth" for the fp32 paths)."""
    return [{k: (v.to(dtype) if torch.is_tensor(v) else v) for k, v in layer.items()} for layer in layers]


# ----------------------------------------------------------------------------
# input sets
# ----------------------------------------------------------------------------
@dataclass
class InputSet:
    """Midpoint/radius view of the input perturbation set.

    Box: perturbation.py:297-298 and 345-346 (`midpoint=(lower+upper)/2`,
    `radius=(upper-lower)/2`).  L-inf ball: perturbation.py:201-215 uses the
    centre itself and the scalar eps.
    """

    mid: torch.Tensor
    rad: torch.Tensor
    lo: torch.Tensor
    up: torch.Tensor
    p: Optional[int] = None   # 1 or 2: an Lp ball of radius eps around `mid` (then lo/up are its bounding box)
    eps: float = 0.0


def lp_ball(x0: torch.Tensor, eps: float, p: int) -> "InputSet":
    """L1 / L2 ball (`LpBallPerturbation`, perturbation.py:73-222).  Its
    bounding box is centre +- eps for every p (perturbation.py:97-100)."""
    if p not in (1, 2):
        raise ValueError("p must be 1 or 2 (use linf_box for the L-inf ball)")
    rad = torch.full_like(x0, float(eps))
    return InputSet(mid=x0, rad=rad, lo=x0 - float(eps), up=x0 + float(eps), p=int(p), eps=float(eps))


def _dual_row_norm(A: torch.Tensor, p: int) -> torch.Tensor:
    """Dual norm over the last axis: p=2 -> L2, p=1 -> max |.| (perturbation.py:121-126, 204-209)."""
    return torch.linalg.vector_norm(A, ord=2, dim=-1) if p == 2 else A.abs().amax(dim=-1)


def box_input(lo: torch.Tensor, up: torch.Tensor) -> InputSet:
    return InputSet(mid=(lo + up) / 2.0, rad=(up - lo) / 2.0, lo=lo, up=up)


def linf_box(x0: torch.Tensor, eps: float) -> InputSet:
    rad = torch.full_like(x0, float(eps))
    return InputSet(mid=x0, rad=rad, lo=x0 - float(eps), up=x0 + float(eps))


# ----------------------------------------------------------------------------
# IBP transformers
# ----------------------------------------------------------------------------
def ibp_first_linear(inp: InputSet, W: torch.Tensor, b: Optional[torch.Tensor]):
    """First affine layer straight from the input set.

    Box: `BoxPerturbation.concretize_matmul` perturbation.py:282-325
    (`midpoint @ W^T`, `radius @ |W|^T`).  L-inf: perturbation.py:102-134 gives
    the same numbers with radius == eps (`eps * |W|.sum(1)`).
    """
    mid = inp.mid.reshape(inp.mid.shape[0], -1)
    rad = inp.rad.reshape(inp.rad.shape[0], -1)
    center = mid.matmul(W.t())
    if inp.p is not None:  # L1/L2 ball: eps * dual row norm, the same for every batch row (perturbation.py:117-128)
        dev = (inp.eps * _dual_row_norm(W, inp.p)).unsqueeze(0)
    else:
        dev = rad.matmul(W.abs().t())
    lower, upper = center - dev, center + dev
    if b is not None:
        lower, upper = lower + b, upper + b
    return lower, upper


def ibp_linear(l: torch.Tensor, u: torch.Tensor, W: torch.Tensor, b: Optional[torch.Tensor]):
    """`IntervalDomain.affine_transformer` linear branch, domains/interval.py:79-86."""
    w_pos = torch.clamp(W, min=0.0)
    w_neg = torch.clamp(W, max=0.0)
    y_l = l.matmul(w_pos.t()) + u.matmul(w_neg.t())
    y_u = u.matmul(w_pos.t()) + l.matmul(w_neg.t())
    if b is not None:
        y_l, y_u = y_l + b, y_u + b
    return y_l, y_u


def ibp_conv2d(l, u, W, b, stride, padding, dilation=(1, 1), groups=1):
    """`IntervalDomain.affine_transformer` conv2d branch, domains/interval.py:57-74."""
    w_pos = torch.clamp(W, min=0.0)
    w_neg = torch.clamp(W, max=0.0)
    y_l = F.conv2d(l, w_pos, None, stride, padding, dilation, groups) + F.conv2d(u, w_neg, None, stride, padding, dilation, groups)
    y_u = F.conv2d(u, w_pos, None, stride, padding, dilation, groups) + F.conv2d(l, w_neg, None, stride, padding, dilation, groups)
    if b is not None:
        y_l = y_l + b.view(1, -1, 1, 1)
        y_u = y_u + b.view(1, -1, 1, 1)
    return y_l, y_u


def ibp_linear_batched(l: torch.Tensor, u: torch.Tensor, W: torch.Tensor, b: Optional[torch.Tensor]):
    """Linear layer with one weight matrix per batch element, W [B,S,I], b [B,S]: the
    batched branch of `PythonTaskExecutor.run_ibp` (runtime/task_executor.py:231-245),
    which evaluates a module whose last layer carries the merged output spec
    (`_fuse_linear_spec_into_last_linear`, planner/interval_v1.py:85-163)."""
    mid = (l + u) / 2.0
    diff = (u - l) / 2.0
    center = torch.bmm(mid.unsqueeze(1), W.transpose(-1, -2)).squeeze(1)
    dev = torch.bmm(diff.unsqueeze(1), W.abs().transpose(-1, -2)).squeeze(1)
    lower, upper = center - dev, center + dev
    if b is not None:
        lower, upper = lower + b, upper + b
    return lower, upper


def apply_relu_split(l: torch.Tensor, u: torch.Tensor, split: torch.Tensor):
    """`_apply_relu_split`, runtime/crown_ibp.py:70-98.

    split in {-1,0,+1} with the pre-activation's shape (a leading batch axis of
    1 or a missing batch axis broadcasts, runtime/relu_shape_utils.py:82-115).
    Returns the clamped bounds and a per-domain `infeasible` mask; the reference
    raises ValueError for the whole batch when any entry has lower > upper
    (crown_ibp.py:92-95) -- callers that mirror that behaviour test `.any()`.
    """
    shape = l.shape
    B = shape[0]
    lf, uf = l.reshape(B, -1), u.reshape(B, -1)
    s = split.reshape(-1, lf.shape[1]) if split.dim() >= 1 and split.numel() != 1 else split.reshape(1, 1)
    s = s.expand(B, lf.shape[1])
    lf = torch.where(s > 0, torch.maximum(lf, torch.zeros_like(lf)), lf)
    uf = torch.where(s < 0, torch.minimum(uf, torch.zeros_like(uf)), uf)
    infeasible = (lf > uf).any(dim=1)
    return lf.reshape(shape), uf.reshape(shape), infeasible


@dataclass
class ForwardTrace:
    """What `_forward_ibp_trace_mlp` (crown_ibp.py:101-342) returns, positionally.

    pre[i]  : (l, u) bounds of the i-th ReLU's input after constraint/split clamps
    shapes  : per-layer output shapes without batch (input shape first)
    out     : IBP bounds of the chain output
    infeasible : [B] bool, any split/constraint made lower > upper
    """

    pre: List[Tuple[torch.Tensor, torch.Tensor]]
    shapes: List[Tuple[int, ...]]
    out: Tuple[torch.Tensor, torch.Tensor]
    infeasible: torch.Tensor


def forward_ibp_trace(
    layers: Layers,
    inp: InputSet,
    *,
    splits: Optional[Sequence[Optional[torch.Tensor]]] = None,
    constraints: Optional[Sequence[Tuple[torch.Tensor, torch.Tensor]]] = None,
) -> ForwardTrace:
    """One IBP sweep recording every ReLU pre-activation, crown_ibp.py:101-342.

    The first linear layer consumes the input set exactly
    (crown_ibp.py:151-159); a first conv2d uses the bounding box
    (crown_ibp.py:173-178).  `constraints[i]` is intersected with the i-th
    pre-activation (crown_ibp.py:186-209) before `splits[i]` is applied
    (crown_ibp.py:210-213).
    """
    B = inp.mid.shape[0]
    at_input = True
    cur_l, cur_u = inp.lo, inp.up
    cur_inp = inp
    pre: List[Tuple[torch.Tensor, torch.Tensor]] = []
    shapes: List[Tuple[int, ...]] = [tuple(inp.mid.shape[1:])]
    infeasible = torch.zeros(B, dtype=torch.bool)
    relu_idx = 0
    for layer in layers:
        op = layer["op"]
        if op == "linear":
            if at_input:
                cur_l, cur_u = ibp_first_linear(cur_inp, layer["W"], layer.get("b"))
            else:
                cur_l, cur_u = ibp_linear(cur_l, cur_u, layer["W"], layer.get("b"))
            at_input = False
        elif op == "conv2d":
            cur_l, cur_u = ibp_conv2d(cur_l, cur_u, layer["W"], layer.get("b"), layer["stride"], layer["padding"],
                                      layer.get("dilation", (1, 1)), layer.get("groups", 1))
            at_input = False
        elif op == "relu":
            if constraints is not None:
                c_l, c_u = constraints[relu_idx]
                cur_l = torch.maximum(cur_l, c_l)
                cur_u = torch.minimum(cur_u, c_u)
                infeasible |= (cur_l > cur_u).reshape(B, -1).any(dim=1)
            if splits is not None and splits[relu_idx] is not None:
                cur_l, cur_u, bad = apply_relu_split(cur_l, cur_u, splits[relu_idx])
                infeasible |= bad
            pre.append((cur_l, cur_u))
            relu_idx += 1
            cur_l, cur_u = torch.relu(cur_l), torch.relu(cur_u)  # interval.py:88-91
        elif op == "flatten":
            if at_input:
                cur_inp = InputSet(
                    mid=cur_inp.mid.flatten(1), rad=cur_inp.rad.flatten(1), lo=cur_inp.lo.flatten(1), up=cur_inp.up.flatten(1),
                    p=cur_inp.p, eps=cur_inp.eps,
                )
            cur_l, cur_u = cur_l.flatten(1), cur_u.flatten(1)
        else:
            raise NotImplementedError(op)
        shapes.append(tuple(cur_l.shape[1:]))
    return ForwardTrace(pre=pre, shapes=shapes, out=(cur_l, cur_u), infeasible=infeasible)


# ----------------------------------------------------------------------------
# ReLU relaxation and backward transformers
# ----------------------------------------------------------------------------
def relu_relax(l: torch.Tensor, u: torch.Tensor):
    """`_relu_relax`, crown_ibp.py:722-758.

    pos = l>=0 -> slope 1; neg = u<=0 -> slope 0 (the later masked write wins
    when l == u == 0); otherwise upper line u/(u-l) with intercept -l*u/(u-l),
    lower slope 0.  The denominator is clamped at the dtype's machine epsilon.
    """
    pos = l >= 0
    neg = u <= 0
    amb = (~pos) & (~neg)
    denom = (u - l).clamp_min(torch.finfo(l.dtype).eps)
    a = u / denom
    one, zero = torch.ones_like(l), torch.zeros_like(l)
    alpha_u = torch.where(amb, a, torch.where(neg, zero, one))
    beta_u = torch.where(amb, -l * a, zero)
    alpha_l = torch.where(amb, zero, torch.where(neg, zero, one))
    beta_l = zero
    return alpha_u, beta_u, alpha_l, beta_l


def relu_slopes(l, u, alpha: Optional[torch.Tensor]):
    """`_relu_backward_relaxation`, crown_ibp.py:1176-1208: flattened slopes with
    the alpha override `clamp(alpha,0,1)` (crown_ibp.py:1001) applied only where
    l < 0 < u (crown_ibp.py:1199-1201)."""
    B = l.shape[0]
    lf, uf = l.reshape(B, -1), u.reshape(B, -1)
    alpha_u, beta_u, alpha_l, beta_l = relu_relax(lf, uf)
    if alpha is not None:
        a = alpha.reshape(-1, lf.shape[1]).expand(B, lf.shape[1]).clamp(0.0, 1.0)
        amb = (lf < 0) & (uf > 0)
        alpha_l = torch.where(amb, a, alpha_l)
    return alpha_u, beta_u, alpha_l, beta_l


def relu_backward(A_u, A_l, b_u, b_l, alpha_u, beta_u, alpha_l, beta_l, add_u=None, add_l=None):
    """`_backprop_relu_step_dense_reference`, crown_ibp.py:1262-1298.

    A_* are [B,S,n]; slopes [B,n]; add_* (the beta term, [B,n]) is broadcast
    over S and added after scaling.
    """
    sel_a = torch.where(A_u >= 0, alpha_u.unsqueeze(1), alpha_l.unsqueeze(1))
    sel_b = torch.where(A_u >= 0, beta_u.unsqueeze(1), beta_l.unsqueeze(1))
    out_b_u = b_u + (A_u * sel_b).sum(dim=2)
    out_A_u = A_u * sel_a
    if add_u is not None:
        out_A_u = out_A_u + add_u.unsqueeze(1)
    sel_a = torch.where(A_l >= 0, alpha_l.unsqueeze(1), alpha_u.unsqueeze(1))
    sel_b = torch.where(A_l >= 0, beta_l.unsqueeze(1), beta_u.unsqueeze(1))
    out_b_l = b_l + (A_l * sel_b).sum(dim=2)
    out_A_l = A_l * sel_a
    if add_l is not None:
        out_A_l = out_A_l + add_l.unsqueeze(1)
    return out_A_u, out_A_l, out_b_u, out_b_l


def linear_backward(A, b, W, bias):
    """`_backprop_linear_step`, crown_ibp.py:1073-1090: A' = A @ W
    (linear_operator.py:585-586 `einsum bko,oi->bki`), b' = b + A @ bias
    (linear_operator.py:374-383)."""
    b_out = b + torch.einsum("bko,o->bk", A, bias) if bias is not None else b
    return torch.einsum("bko,oi->bki", A, W), b_out


def conv2d_output_padding(in_hw, out_hw, k, stride, padding, dilation=(1, 1)):
    """linear_operator.py:140-163 / crown_ibp.py:1589-1596: output_padding = H_in - ((H_out-1)*s - 2p + d*(k-1) + 1)."""
    return tuple(
        int(in_hw[i]) - ((int(out_hw[i]) - 1) * stride[i] - 2 * padding[i] + dilation[i] * (k[i] - 1) + 1) for i in range(2)
    )


def conv2d_backward(A, b, W, bias, stride, padding, in_shape, out_shape, dilation=(1, 1), groups=1):
    """`_backprop_conv2d_step`, crown_ibp.py:1106-1173, with
    `Conv2dLinearOperator.to_dense` (linear_operator.py:1067-1092): the
    coefficient rows [B,S,C_o*H_o*W_o] go through conv_transpose2d with batch =
    B*S; the bias term is sum over (c,h,w) of A*bias[c] (crown_ibp.py:1149-1152).
    """
    B, S = A.shape[0], A.shape[1]
    A4 = A.reshape(B * S, *out_shape)
    b_out = b
    if bias is not None:
        b_out = b + (A4.sum(dim=(2, 3)) * bias.view(1, -1)).sum(dim=1).reshape(B, S)
    opad = conv2d_output_padding(in_shape[1:], out_shape[1:], W.shape[2:], stride, padding, dilation)
    prev = F.conv_transpose2d(A4, W, None, stride, padding, opad, groups, dilation)
    return prev.reshape(B, S, -1), b_out


def conv2d_dense_rows(W, bias, stride, padding, in_shape, out_shape):
    """Dense matrix [C_o*H_o*W_o, C_i*H_i*W_i] and bias vector of a Conv2d layer, the rows that the reference's
    first-layer certificate builds one at a time for a conv first layer (alpha_beta_crown.py:346-387: a one-hot
    coefficient row through `DenseLinearOperator.conv2d_right(...).to_dense()`, bias = bias[channel])."""
    n1 = int(out_shape[0]) * int(out_shape[1]) * int(out_shape[2])
    eye = torch.eye(n1, dtype=W.dtype).reshape(1, n1, n1)
    rows, bvec = conv2d_backward(eye, torch.zeros(1, n1, dtype=W.dtype), W, bias, stride, padding, in_shape, out_shape)
    return rows[0], bvec[0]


def concretize(inp: InputSet, A, b, side: str):
    """`BoxPerturbation.concretize_affine`, perturbation.py:327-359:
    lower = A.mid - |A|.rad + b, upper = A.mid + |A|.rad + b.  (L-inf ball:
    perturbation.py:201-215, identical with rad == eps.)"""
    B = A.shape[0]
    mid = inp.mid.reshape(B, 1, -1)
    rad = inp.rad.reshape(B, 1, -1)
    center = (A * mid).sum(dim=2)
    if inp.p is not None:  # perturbation.py:201-222: eps * ||A_row||_q
        dev = inp.eps * _dual_row_norm(A, inp.p)
    else:
        dev = (A.abs() * rad).sum(dim=2)
    return (center - dev + b) if side == "lower" else (center + dev + b)


# ----------------------------------------------------------------------------
# CROWN backward sweep
# ----------------------------------------------------------------------------
def relu_layer_indices(layers: Layers) -> List[int]:
    return [i for i, layer in enumerate(layers) if layer["op"] == "relu"]


def crown_backward(
    layers: Layers,
    inp: InputSet,
    trace: ForwardTrace,
    C: Optional[torch.Tensor],
    *,
    alpha: Optional[Sequence[Optional[torch.Tensor]]] = None,
    add_l: Optional[Sequence[Optional[torch.Tensor]]] = None,
    upto: Optional[int] = None,
    influence_out: Optional[List[torch.Tensor]] = None,
    add_u: Optional[Sequence[Optional[torch.Tensor]]] = None,
):
    """`_run_crown_backward_from_trace`, crown_ibp.py:1669-2051, for chains.

    Bounds `C @ value` where value is the output of `layers[:upto]` (default:
    the whole chain; crown_ibp.py:1722 `output_value=`).  C is [B,S,O] (or
    [S,O], broadcast; or None = identity, crown_ibp.py:672-719).  `alpha[i]`
    overrides the i-th ReLU's lower slope, `add_l[i]` is the beta term added to
    the lower coefficients (alpha_beta_crown.py:615-640).  Returns (lower, upper)
    both [B,S].  `influence_out` (a list) receives, per ReLU in chain order, the objective
    influence max(max_s |A_u|, max_s |A_l|) [B,n_r] of the coefficients that reach the ReLU
    (crown_ibp.py:1810-1834).
    """
    n_layers = len(layers) if upto is None else int(upto)
    B = inp.mid.shape[0]
    out_shape = trace.shapes[n_layers]
    out_dim = 1
    for d in out_shape:
        out_dim *= int(d)
    dtype = inp.mid.dtype
    if C is None:
        C = torch.eye(out_dim, dtype=dtype).unsqueeze(0).expand(B, out_dim, out_dim)
    elif C.dim() == 2:
        C = C.unsqueeze(0).expand(B, C.shape[0], C.shape[1])
    A_u, A_l = C.clone(), C.clone()
    S = A_u.shape[1]
    b_u = torch.zeros(B, S, dtype=dtype)
    b_l = torch.zeros(B, S, dtype=dtype)
    relu_ids = relu_layer_indices(layers)
    for idx in range(n_layers - 1, -1, -1):
        layer = layers[idx]
        op = layer["op"]
        if op == "linear":
            A_u, b_u = linear_backward(A_u, b_u, layer["W"], layer.get("b"))
            A_l, b_l = linear_backward(A_l, b_l, layer["W"], layer.get("b"))
        elif op == "conv2d":
            in_shape, o_shape = trace.shapes[idx], trace.shapes[idx + 1]
            dg = (layer.get("dilation", (1, 1)), layer.get("groups", 1))
            A_u, b_u = conv2d_backward(A_u, b_u, layer["W"], layer.get("b"), layer["stride"], layer["padding"], in_shape, o_shape, *dg)
            A_l, b_l = conv2d_backward(A_l, b_l, layer["W"], layer.get("b"), layer["stride"], layer["padding"], in_shape, o_shape, *dg)
        elif op == "relu":
            r = relu_ids.index(idx)
            l, u = trace.pre[r]
            if influence_out is not None:
                influence_out.insert(0, torch.maximum(A_u.abs().amax(dim=1), A_l.abs().amax(dim=1)))
            a = alpha[r] if alpha is not None else None
            alpha_u, beta_u, alpha_l, beta_l = relu_slopes(l, u, a)
            add = add_l[r] if add_l is not None else None
            add_up = add_u[r] if add_u is not None else None  # relu_pre_add_coeff_u, crown_ibp.py:1270-1278
            A_u, A_l, b_u, b_l = relu_backward(A_u, A_l, b_u, b_l, alpha_u, beta_u, alpha_l, beta_l, add_up, add)
        elif op == "flatten":
            pass  # coefficients are kept flattened; reshape is a view (crown_ibp.py:1093-1103)
        else:
            raise NotImplementedError(op)
    lower = concretize(inp, A_l, b_l, "lower")
    upper = concretize(inp, A_u, b_u, "upper")
    return lower, upper


def crown_ibp(layers: Layers, inp: InputSet, C, *, splits=None, alpha=None):
    """`run_crown_ibp_mlp`, crown_ibp.py:2054-2133: IBP trace then one backward sweep."""
    trace = forward_ibp_trace(layers, inp, splits=splits)
    lower, upper = crown_backward(layers, inp, trace, C, alpha=alpha)
    return lower, upper, trace


def crown_with_intermediate_crown(layers: Layers, inp: InputSet, C, *, chunk: int = 512):
    """CROWN whose intermediate (ReLU-input) bounds are themselves CROWN bounds.

    Composition of reference primitives as in
    runtime/native_intermediate_refinement.py:923-988: for every ReLU input in
    graph order bound it with an identity spec
    (`run_crown_ibp_mlp_from_forward_trace(output_value=name)`), intersect with
    the current bounds (maximum/minimum), re-propagate IBP under the constraints
    (`_forward_ibp_trace_mlp(relu_pre_constraints=...)`), and finally bound the
    spec rows.  Identity rows are processed in chunks to bound memory.
    """
    trace = forward_ibp_trace(layers, inp)
    relu_ids = relu_layer_indices(layers)
    B = inp.mid.shape[0]
    cons = [(l.clone(), u.clone()) for l, u in trace.pre]
    for r, idx in enumerate(relu_ids):
        if r == 0:
            continue  # the first pre-activation's CROWN bound equals its IBP bound
        shape = trace.shapes[idx]
        n = 1
        for d in shape:
            n *= int(d)
        lo_rows, up_rows = [], []
        eye = torch.eye(n, dtype=inp.mid.dtype)
        for s in range(0, n, chunk):
            Cc = eye[s : s + chunk]
            lo_c, up_c = crown_backward(layers, inp, trace, Cc, upto=idx)
            lo_rows.append(lo_c)
            up_rows.append(up_c)
        new_l = torch.cat(lo_rows, dim=1).reshape(B, *shape)
        new_u = torch.cat(up_rows, dim=1).reshape(B, *shape)
        cons[r] = (torch.maximum(cons[r][0], new_l), torch.minimum(cons[r][1], new_u))
        trace = forward_ibp_trace(layers, inp, constraints=cons)
        cons = [(l.clone(), u.clone()) for l, u in trace.pre]
    lower, upper = crown_backward(layers, inp, trace, C)
    return lower, upper, trace


# ----------------------------------------------------------------------------
# alpha-CROWN
# ----------------------------------------------------------------------------
def adaptive_alpha_init(trace: ForwardTrace) -> List[torch.Tensor]:
    """Adaptive lower-slope start, native_alpha_beta_optimizer_schedule.py:635-656:
    1 where l >= 0 or (l < 0 < u and u > -l), else 0."""
    out = []
    for l, u in trace.pre:
        lf, uf = l.reshape(l.shape[0], -1), u.reshape(u.shape[0], -1)
        out.append(((lf >= 0) | ((lf < 0) & (uf > 0) & (uf > -lf))).to(l.dtype))
    return out


def alpha_crown(
    layers: Layers,
    inp: InputSet,
    C,
    *,
    steps: int,
    lr: float,
    alpha0: Optional[Sequence[torch.Tensor]] = None,
    alpha_init: float = 0.5,
    splits=None,
    spec_reduce: str = "mean",
    trace: Optional[ForwardTrace] = None,
    optimize_beta: bool = False,
    return_beta: bool = False,
    soft_tau: float = 1.0,
    objective: str = "lower",
    lb_weight: float = 1.0,
    ub_weight: float = 1.0,
):
    """Per-domain alpha (and optionally beta) optimisation, `run_alpha_beta_crown_mlp`
    with `per_batch_params=True` restated (alpha_beta_crown.py:716-923).
    Objectives (alpha_beta_crown.py:807-818): "lower" maximises reduce(lower), "upper" minimises
    reduce(upper), "gap" minimises reduce(upper - lower), "both" maximises
    lb_weight * reduce(lower) - ub_weight * reduce(upper); upper-side reductions take max / softmax
    where the lower side takes min / softmin (787-805).  The beta term enters the lower objective
    only (763-785): the other objectives run the alpha-only evaluation.
    With `optimize_beta` every ReLU also gets a per-domain beta >= 0 (start 0) whose
    split term -beta*s*[s != 0] is added to the lower coefficients
    (`_beta_to_relu_pre_add_coeff`, alpha_beta_crown.py:615-640) and which the same Adam
    instance updates; without it beta stays at zero, i.e. the alpha-only loop.

    steps+1 bound evaluations (756); metric_b = mean (or sum) over specs of the
    lower bound (787-805); per-domain best with strict improvement, step 0
    initialises (821-866); loss = -sum_b metric_b (913); torch Adam with default
    betas/eps (747); projection alpha in [0,1] (919-921).  Returns the best
    (lower, upper) per domain, the best alpha per ReLU, and the trace.
    """
    if trace is None:
        trace = forward_ibp_trace(layers, inp, splits=splits)
    B = inp.mid.shape[0]
    dtype = inp.mid.dtype
    alphas = []
    for r, (l, _u) in enumerate(trace.pre):
        n = l.reshape(B, -1).shape[1]
        if alpha0 is not None:
            a = alpha0[r].reshape(-1, n).expand(B, n).to(dtype).clone()
        else:
            a = torch.full((B, n), float(alpha_init), dtype=dtype)
        alphas.append(a.requires_grad_(True))
    betas: List[torch.Tensor] = []
    split_f: List[Optional[torch.Tensor]] = []
    if optimize_beta:
        for r, (l, _u) in enumerate(trace.pre):
            n = l.reshape(B, -1).shape[1]
            betas.append(torch.zeros(B, n, dtype=dtype, requires_grad=True))
            sp = splits[r] if (splits is not None and splits[r] is not None) else None
            split_f.append(None if sp is None else sp.reshape(-1, n).expand(B, n).to(dtype))
    opt = torch.optim.Adam(alphas + betas, lr=float(lr))
    best_metric = None
    best_lower = best_upper = None
    best_alpha: List[torch.Tensor] = []
    best_beta: List[torch.Tensor] = []
    for step in range(int(steps) + 1):
        add_l = None
        if optimize_beta and objective == "lower":
            add_l = [None if sf is None else -bt * sf * (sf != 0).to(dtype) for bt, sf in zip(betas, split_f)]
        lower, upper = crown_backward(layers, inp, trace, C, alpha=alphas, add_l=add_l)

        # spec reductions (alpha_beta_crown.py:787-805): mean | min | softmin, plus sum
        def _reduce(x, direction):
            if spec_reduce == "mean":
                return x.mean(dim=1)
            if spec_reduce == "sum":
                return x.sum(dim=1)
            if spec_reduce == "min":
                return x.min(dim=1).values if direction == "min" else x.max(dim=1).values
            if spec_reduce == "softmin":
                tau = float(soft_tau)
                return -tau * torch.logsumexp(-x / tau, dim=1) if direction == "min" else tau * torch.logsumexp(x / tau, dim=1)
            raise ValueError(spec_reduce)

        if objective == "lower":
            metric_b = _reduce(lower, "min")
        elif objective == "upper":
            metric_b = -_reduce(upper, "max")
        elif objective == "gap":
            metric_b = -_reduce(upper - lower, "max")
        elif objective == "both":
            metric_b = float(lb_weight) * _reduce(lower, "min") - float(ub_weight) * _reduce(upper, "max")
        else:
            raise ValueError(objective)
        if best_metric is None:
            best_metric = metric_b.detach().clone()
            best_lower, best_upper = lower.detach().clone(), upper.detach().clone()
            best_alpha = [a.detach().clone() for a in alphas]
            best_beta = [b.detach().clone() for b in betas]
        else:
            improve = metric_b.detach() > best_metric
            best_metric = torch.where(improve, metric_b.detach(), best_metric)
            best_lower = torch.where(improve.unsqueeze(1), lower.detach(), best_lower)
            best_upper = torch.where(improve.unsqueeze(1), upper.detach(), best_upper)
            best_alpha = [torch.where(improve.unsqueeze(1), a.detach(), p) for a, p in zip(alphas, best_alpha)]
            best_beta = [torch.where(improve.unsqueeze(1), b.detach(), p) for b, p in zip(betas, best_beta)]
        if step == int(steps):
            break
        loss = -metric_b.sum()
        if not loss.requires_grad:
            break
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        with torch.no_grad():
            for a in alphas:
                a.clamp_(0.0, 1.0)
            for b in betas:
                b.clamp_(0.0)
    if return_beta:
        return best_lower, best_upper, best_alpha, best_beta, trace
    return best_lower, best_upper, best_alpha, trace


def alpha_crown_shared(layers: Layers, inp: InputSet, C, *, steps: int, lr: float, alpha0: Optional[Sequence[torch.Tensor]] = None,
                       alpha_init: float = 0.5, splits=None, trace: Optional[ForwardTrace] = None, optimize_beta: bool = False,
                       objective: str = "lower", spec_reduce: str = "mean", soft_tau: float = 1.0, lb_weight: float = 1.0,
                       ub_weight: float = 1.0):
    """alpha (and optionally beta) shared by every domain and spec row: `run_alpha_crown_mlp`
    (alpha_crown.py:137-261) and the `per_batch_params=False` mode of `run_alpha_beta_crown_mlp`
    (alpha_beta_crown.py:716-923), restated for objective="lower", spec_reduce="mean".
    Parameters have the ReLU input's shape without the batch axis (alpha start `alpha_init`,
    beta start 0); steps+1 evaluations; metric = mean over all lower bounds; strict best-of on
    that scalar keeps the whole batch's bounds and parameters (alpha_crown.py:215-220,
    alpha_beta_crown.py:877-903); loss = -metric (alpha_beta_crown.py:913), torch Adam, alpha
    clamped to [0,1], beta to >= 0.  Returns best (lower, upper), best alpha list, trace and,
    with `optimize_beta`, the best beta list before the trace."""
    if trace is None:
        trace = forward_ibp_trace(layers, inp, splits=splits)
    B = inp.mid.shape[0]
    dtype = inp.mid.dtype
    alphas, betas, split_f = [], [], []
    for r, (l, _u) in enumerate(trace.pre):
        n = l.reshape(B, -1).shape[1]
        a = alpha0[r].reshape(n).to(dtype).clone() if alpha0 is not None else torch.full((n,), float(alpha_init), dtype=dtype)
        alphas.append(a.requires_grad_(True))
        if optimize_beta:
            betas.append(torch.zeros(n, dtype=dtype, requires_grad=True))
            sp = splits[r] if (splits is not None and splits[r] is not None) else None
            split_f.append(None if sp is None else sp.reshape(-1, n).expand(B, n).to(dtype))
    opt = torch.optim.Adam(alphas + betas, lr=float(lr)) if alphas else None
    best_metric = None
    best = None
    for step in range(int(steps) + 1):
        add_l = None
        if optimize_beta:
            add_l = [None if sf is None else -bt.unsqueeze(0) * sf for bt, sf in zip(betas, split_f)]
        lower, upper = crown_backward(layers, inp, trace, C, alpha=[a.unsqueeze(0).expand(B, -1) for a in alphas], add_l=add_l)

        # `_reduce_over_specs` / `_objective_metric`, alpha_crown.py:67-112: per-domain reduction, then the batch mean
        def _reduce(x, direction):
            if spec_reduce == "mean":
                return x.mean()
            if spec_reduce == "min":
                return (x.min(dim=1).values if direction == "min" else x.max(dim=1).values).mean()
            tau = float(soft_tau)
            return ((-tau * torch.logsumexp(-x / tau, dim=1)) if direction == "min" else (tau * torch.logsumexp(x / tau, dim=1))).mean()

        if objective == "lower":
            metric = _reduce(lower, "min")
        elif objective == "upper":
            metric = -_reduce(upper, "max")
        elif objective == "gap":
            metric = -_reduce(upper - lower, "max")
        elif objective == "both":
            metric = float(lb_weight) * _reduce(lower, "min") - float(ub_weight) * _reduce(upper, "max")
        else:
            raise ValueError(objective)
        if best_metric is None or float(metric.detach()) > best_metric:
            best_metric = float(metric.detach())
            best = (lower.detach().clone(), upper.detach().clone(), [a.detach().clone() for a in alphas], [b.detach().clone() for b in betas])
        if step == int(steps) or opt is None:
            break
        loss = -metric
        if not loss.requires_grad:
            break
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        with torch.no_grad():
            for a in alphas:
                a.clamp_(0.0, 1.0)
            for b in betas:
                b.clamp_(0.0)
    if optimize_beta:
        return best[0], best[1], best[2], best[3], trace
    return best[0], best[1], best[2], trace


def branch_choices(trace: ForwardTrace) -> List[Optional[Tuple[int, int]]]:
    """Widest-unstable-gap branching hint, `_branch_choices_from_relu_pre`
    (alpha_beta_crown.py:145-182): per domain the (ReLU index, neuron index) with the largest
    u - l among neurons with l < 0 < u; earlier ReLUs win ties (strict improvement), the first
    index wins inside a ReLU (argmax); None when no neuron is unstable."""
    B = trace.pre[0][0].shape[0]
    best_gap = torch.full((B,), float("-inf"), dtype=trace.pre[0][0].dtype)
    best: List[Optional[Tuple[int, int]]] = [None] * B
    for r, (l, u) in enumerate(trace.pre):
        lf, uf = l.reshape(B, -1), u.reshape(B, -1)
        amb = (lf < 0) & (uf > 0)
        gap = torch.where(amb, (uf - lf).clamp_min(0.0), torch.full_like(lf, float("-inf")))
        row_best = gap.max(dim=1).values
        row_idx = gap.argmax(dim=1)
        improve = row_best > best_gap
        best_gap = torch.where(improve, row_best, best_gap)
        for i in torch.nonzero(improve).flatten().tolist():
            best[i] = (r, int(row_idx[i]))
    return best


def alpha_gradient(layers: Layers, inp: InputSet, trace: ForwardTrace, C, alphas: Sequence[torch.Tensor], spec_reduce="mean"):
    """Gradient of `-sum_b reduce_s lower[b,s]` w.r.t. each per-domain alpha via
    autograd through `crown_backward` -- the quantity the reference's
    `loss.backward()` (alpha_beta_crown.py:913-917) hands to Adam."""
    leaves = [a.detach().clone().requires_grad_(True) for a in alphas]
    lower, _ = crown_backward(layers, inp, trace, C, alpha=leaves)
    metric_b = lower.mean(dim=1) if spec_reduce == "mean" else lower.sum(dim=1)
    (-metric_b.sum()).backward()
    return [a.grad if a.grad is not None else torch.zeros_like(a) for a in leaves], lower.detach()


# ----------------------------------------------------------------------------
# verdicts and soundness
# ----------------------------------------------------------------------------
def first_layer_certificate(W1: torch.Tensor, b1: Optional[torch.Tensor], inp: InputSet, split_row: torch.Tensor, *,
                            steps: int = 200, lr: float = 0.1, tol: float = 1e-6):
    """`_is_infeasible_split_first_layer_convex_combo` (alpha_beta_crown.py:391-532) for one domain
    (`inp` has batch size 1) and a Linear first layer: half-spaces s_j*(W1[j].x + b1[j]) >= 0 of the
    split neurons in ascending j (262-322); one half-space: its maximum over the input set (439-468);
    else logits = 0, Adam(lr) on max_x (sum w_i a_i).x + sum w_i c_i with w = softmax(logits),
    best value tracked before each update, early exit below -tol (470-512).
    Returns (infeasible: bool, smallest value seen or None without half-spaces)."""
    idx = torch.nonzero(split_row.reshape(-1) != 0).reshape(-1)
    if idx.numel() == 0:
        return False, None
    sgn = split_row.reshape(-1)[idx].to(W1.dtype)
    a_mat = (sgn.unsqueeze(1) * W1[idx]).detach()
    c_vec = (sgn * (b1[idx] if b1 is not None else torch.zeros_like(sgn))).detach()

    def value(a, c):
        return concretize(inp, a.view(1, 1, -1), c.view(1, 1), "upper").squeeze()

    if idx.numel() == 1:
        v = float(value(a_mat[0], c_vec[0]))
        return v < -float(tol), v
    logits = torch.zeros(idx.numel(), dtype=W1.dtype, requires_grad=True)
    opt = torch.optim.Adam([logits], lr=float(lr))
    best = None
    for _ in range(int(steps)):
        w = torch.softmax(logits, dim=0)
        ub = value((w.unsqueeze(1) * a_mat).sum(dim=0), (w * c_vec).sum())
        v = float(ub.detach())
        best = v if best is None or v < best else best
        if v < -float(tol):
            return True, best
        opt.zero_grad(set_to_none=True)
        ub.backward()
        opt.step()
    return best < -float(tol), best


def verdict(lower: torch.Tensor, threshold: float = 0.0, tol: float = 1e-6) -> torch.Tensor:
    """bab.py:881-895: a domain is proven iff min over specs of the lower bound
    is >= threshold - tol."""
    return lower.min(dim=1).values >= (threshold - tol)


def concrete_forward(layers: Layers, x: torch.Tensor) -> torch.Tensor:
    """Plain forward evaluation of the chain (task_executor.py:574-784 restated
    for chains) used by the sampling soundness check."""
    for layer in layers:
        op = layer["op"]
        if op == "linear":
            x = x.matmul(layer["W"].t())
            if layer.get("b") is not None:
                x = x + layer["b"]
        elif op == "conv2d":
            x = F.conv2d(x, layer["W"], layer.get("b"), layer["stride"], layer["padding"], layer.get("dilation", (1, 1)), layer.get("groups", 1))
        elif op == "relu":
            x = torch.relu(x)
        elif op == "flatten":
            x = x.flatten(1)
        else:
            raise NotImplementedError(op)
    return x


def sample_soundness(layers: Layers, inp: InputSet, C, lower, upper, *, n: int, seed: int, splits=None, chunk: int = 1000):
    """Worst violation of `lower <= C f(x) <= upper` over n uniform samples per
    box (tests/test_phase6b_crown_ibp_mlp.py:68-110 style).  With `splits`, only
    samples that satisfy every split constraint count.  Returns
    (max(lower - y), max(y - upper)) over valid samples (<= 0 means sound)."""
    g = torch.Generator("cpu").manual_seed(int(seed))
    B = inp.lo.shape[0]
    worst_lo = torch.tensor(-float("inf"), dtype=torch.float64)
    worst_up = torch.tensor(-float("inf"), dtype=torch.float64)
    Cb = C if C.dim() == 3 else C.unsqueeze(0).expand(B, *C.shape)
    relu_ids = relu_layer_indices(layers)
    for s in range(0, n, chunk):
        m = min(chunk, n - s)
        r = torch.rand((m,) + tuple(inp.lo.shape), generator=g, dtype=inp.lo.dtype)
        xs = inp.lo.unsqueeze(0) + r * (inp.up - inp.lo).unsqueeze(0)
        x = xs.reshape(m * B, *inp.lo.shape[1:]).to(torch.float64)
        valid = torch.ones(m * B, dtype=torch.bool)
        ri = 0
        for i, layer in enumerate(layers):
            if layer["op"] == "relu" and splits is not None and splits[ri] is not None:
                sp = splits[ri].reshape(-1, x[0].numel()).expand(B, -1).repeat(m, 1)
                xf = x.reshape(m * B, -1)
                valid &= ~(((sp > 0) & (xf < 0)) | ((sp < 0) & (xf > 0))).any(dim=1)
            if layer["op"] == "relu":
                ri += 1
            lay = {k: (v.to(torch.float64) if torch.is_tensor(v) else v) for k, v in layer.items()}
            x = concrete_forward([lay], x)
        y = torch.einsum("bso,mbo->mbs", Cb.to(torch.float64), x.reshape(m, B, -1))
        v = valid.reshape(m, B, 1).expand_as(y)
        if v.any():
            worst_lo = torch.maximum(worst_lo, (lower.unsqueeze(0).to(torch.float64) - y)[v].max())
            worst_up = torch.maximum(worst_up, (y - upper.unsqueeze(0).to(torch.float64))[v].max())
    return float(worst_lo), float(worst_up)
