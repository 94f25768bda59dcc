"""IBP and CROWN on single-task graphs that are not chains (residual add, fan-out, concat).

The reference's backward sweep (`_run_crown_backward_from_trace`,
boundflow/runtime/crown_ibp.py:1669-2051) keeps one coefficient state per VALUE
(`adjoints`), walks the ops in reverse order and accumulates every op's contribution
into the states of its inputs: `add` hands the same coefficients to both inputs and its
bias to the first dynamic one (`_split_bias_once`, 922-937), `concat` slices the
coefficients along the channel axis (1978-2030), a value consumed twice (fan-out) sums
what arrives (`_accumulate_backward_state`, 879-913).  This module does the same with
the layer-level entry points of the C ABI: `bf_crown_relu_linear_bwd` /
`bf_crown_relu_conv2d_bwd` without slopes (affine backward), `bf_crown_relu_bwd`
(ReLU backward), `bf_accumulate`, `bf_concretize`; the forward pass uses
`bf_ibp_linear` / `bf_ibp_conv2d` / `bf_interval_relu` / `bf_interval_add`.
Chains should use `crown.py`, whose sweeps are fused and tensor-core backed; this is the
general path.  Boxes and L-inf balls only.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping, Optional, Tuple

import torch

from . import _lib
from .crown import _alpha_rows, _cuda_device, _f32, _split_tensor, _stream_ptr
from .ir import IntervalState, input_mid_rad, lp_ball_of, normalize_input_spec
from .network import dense_conv_weight


def _numel(shape) -> int:
    n = 1
    for d in shape:
        n *= int(d)
    return n


def _pair(v) -> Tuple[int, int]:
    if isinstance(v, (tuple, list)):
        return int(v[0]), int(v[1])
    return int(v), int(v)


@dataclass
class DagTrace:
    """Forward IBP result: bounds (flat [B,n]) and shape (without batch) of every value."""

    lower: Dict[str, torch.Tensor] = field(default_factory=dict)
    upper: Dict[str, torch.Tensor] = field(default_factory=dict)
    shape: Dict[str, Tuple[int, ...]] = field(default_factory=dict)
    relu_inputs: List[str] = field(default_factory=list)
    # bounds of every ReLU input after its split (crown_ibp.py:210-214); the value's own entry stays unsplit
    pre_l: Dict[str, torch.Tensor] = field(default_factory=dict)
    pre_u: Dict[str, torch.Tensor] = field(default_factory=dict)
    infeasible: Optional[torch.Tensor] = None  # int32 [B]: a split left some neuron with lower > upper
    B: int = 0
    mid: Optional[torch.Tensor] = None
    rad: Optional[torch.Tensor] = None
    input_name: str = ""
    norm_p: int = 0     # _lib.NORM_BOX, or 1 / 2 for an L1 / L2 ball (then mid = centre and rad = eps, the bounding box)
    eps: float = 0.0


def _params(module: Any, device: torch.device) -> Dict[str, torch.Tensor]:
    """Parameters as fp32 device tensors; the weight of a grouped or dilated Conv2d op is replaced by its dense
    equivalent (`network.dense_conv_weight`), so every step of the walkers sees groups = 1, dilation = 1."""
    raw = module.bindings.get("params", {})
    out = {}
    for k, v in (raw.items() if isinstance(raw, dict) else []):
        t = v if torch.is_tensor(v) else torch.as_tensor(v)
        out[k] = _f32(t, device)
    dense_for: Dict[str, Tuple[int, Tuple[int, int]]] = {}
    for op in module.get_entry_task().ops:
        if op.op_type != "conv2d" or len(op.inputs) < 2 or op.inputs[1] not in out:
            continue
        key = (int(op.attrs.get("groups", 1)), _pair(op.attrs.get("dilation", 1)))
        if dense_for.setdefault(op.inputs[1], key) != key:
            raise NotImplementedError(f"weight '{op.inputs[1]}' is shared by Conv2d ops with different groups / dilation")
    for name, (groups, dilation) in dense_for.items():
        out[name] = dense_conv_weight(out[name], {"groups": groups, "dilation": dilation})
    return out


def forward_ibp_dag(module: Any, input_spec: Any, relu_split_state: Optional[Mapping[str, torch.Tensor]] = None,
                    relu_pre_constraints: Optional[Mapping[str, Any]] = None) -> DagTrace:
    """One IBP pass over the ops in order (`_forward_ibp_trace_mlp`, crown_ibp.py:101-342); `relu_split_state` maps
    the name of a ReLU input to its int8 split assignment ([B, *shape] or one shared row); `relu_pre_constraints` maps
    every ReLU input, in graph order, to an interval that its bounds are intersected with before the split
    (crown_ibp.py:186-209, 338-341)."""
    lib = _lib.load()
    spec = normalize_input_spec(input_spec)
    ball = lp_ball_of(spec)
    device = _cuda_device(spec.center)
    task = module.get_entry_task()
    params = _params(module, device)
    B = int(spec.center.shape[0])
    tr = DagTrace(B=B, input_name=spec.value_name)
    tr.infeasible = torch.zeros(B, dtype=torch.int32, device=device)
    if ball is not None:
        # L1 / L2 ball (LpBallPerturbation, perturbation.py:73-222): a Linear op on the input value uses the dual row norms,
        # every other consumer the bounding box centre -/+ eps (crown_ibp.py:126-134, 173-175)
        tr.norm_p, tr.eps = int(ball[0]), float(ball[1])
        tr.mid = _f32(spec.center, device).reshape(B, -1).contiguous()
        tr.rad = torch.full_like(tr.mid, tr.eps)
        tr.lower[spec.value_name], tr.upper[spec.value_name] = tr.mid - tr.eps, tr.mid + tr.eps
    else:
        mid, rad, lo, up = input_mid_rad(spec)
        tr.mid, tr.rad = _f32(mid, device).reshape(B, -1), _f32(rad, device).reshape(B, -1)
        tr.lower[spec.value_name], tr.upper[spec.value_name] = _f32(lo, device).reshape(B, -1), _f32(up, device).reshape(B, -1)
    input_views = {spec.value_name}   # the input value and its flatten / reshape views (crown_ibp.py:267-330)
    tr.shape[spec.value_name] = tuple(int(d) for d in spec.center.shape[1:])
    s = _stream_ptr(device)
    for op in task.ops:
        t, out = op.op_type, op.outputs[0]
        if t in ("linear", "conv2d"):
            x = op.inputs[0]
            W = params[op.inputs[1]]
            b = params[op.inputs[2]] if len(op.inputs) == 3 else None
            at_input = x in input_views
            if t == "linear":
                n_in, n_out = int(W.shape[1]), int(W.shape[0])
                if _numel(tr.shape[x]) != n_in:
                    raise ValueError(f"linear '{op.name}': weight {tuple(W.shape)} does not match input shape {tr.shape[x]}")
                yl, yu = torch.empty(B, n_out, device=device), torch.empty(B, n_out, device=device)
                if at_input and ball is not None:
                    row_dev = torch.empty(n_out, dtype=torch.float32, device=device)
                    _lib.check(lib.bf_row_dual_norms(_lib.ptr(W), n_out, n_in, tr.norm_p, tr.eps, _lib.ptr(row_dev), s))
                    _lib.check(lib.bf_ibp_linear_lp(_lib.ptr(tr.mid), _lib.ptr(row_dev), _lib.ptr(W), _lib.ptr(b), None, 0, None, None,
                                                    _lib.ptr(yl), _lib.ptr(yu), None, B, n_in, n_out, s))
                else:
                    a, bb, mode = (tr.mid, tr.rad, _lib.IN_MID_RAD) if at_input else (tr.lower[x], tr.upper[x], _lib.IN_LOWER_UPPER)
                    _lib.check(lib.bf_ibp_linear(_lib.ptr(a), _lib.ptr(bb), mode, 0, _lib.ptr(W), _lib.ptr(b), None, 0, None, None,
                                                 _lib.ptr(yl), _lib.ptr(yu), None, B, n_in, n_out, s))
                tr.shape[out] = (n_out,)
            else:
                Ci, Hi, Wi = tr.shape[x]
                Co, _ci, kh, kw = (int(d) for d in W.shape)
                st, pd = _pair(op.attrs.get("stride", 1)), _pair(op.attrs.get("padding", 0))
                Ho, Wo = (Hi + 2 * pd[0] - kh) // st[0] + 1, (Wi + 2 * pd[1] - kw) // st[1] + 1
                yl, yu = torch.empty(B, Co * Ho * Wo, device=device), torch.empty(B, Co * Ho * Wo, device=device)
                _lib.check(lib.bf_ibp_conv2d(_lib.ptr(tr.lower[x]), _lib.ptr(tr.upper[x]), _lib.IN_LOWER_UPPER, 0, _lib.ptr(W), _lib.ptr(b),
                                             None, 0, None, None, _lib.ptr(yl), _lib.ptr(yu), None, B, Ci, Hi, Wi, Co, kh, kw,
                                             st[0], st[1], pd[0], pd[1], s))
                tr.shape[out] = (Co, Ho, Wo)
            tr.lower[out], tr.upper[out] = yl, yu
        elif t == "relu":
            x = op.inputs[0]
            tr.relu_inputs.append(x)
            pl, pu = tr.lower[x], tr.upper[x]
            if relu_pre_constraints is not None:
                c = relu_pre_constraints.get(x)
                shape_x = (B,) + tuple(tr.shape[x])
                if (c is None or not hasattr(c, "lower") or tuple(c.lower.shape) != shape_x or tuple(c.upper.shape) != shape_x
                        or not bool(torch.isfinite(c.lower).all()) or not bool(torch.isfinite(c.upper).all()) or not bool((c.lower <= c.upper).all())):
                    raise ValueError(f"ReLU pre-activation constraint schema differs for {x}")
                n = _numel(tr.shape[x])
                pl, pu = pl.clone(), pu.clone()
                cl, cu = _f32(c.lower, device).reshape(B, n).contiguous(), _f32(c.upper, device).reshape(B, n).contiguous()
                empty = torch.zeros(B, dtype=torch.int32, device=device)
                _lib.check(lib.bf_interval_intersect(_lib.ptr(pl), _lib.ptr(pu), _lib.ptr(cl), _lib.ptr(cu), _lib.ptr(empty), B, n, s))
                if int(empty.sum()) != 0:
                    raise ValueError(f"infeasible ReLU pre-activation intersection for {x}")
            sp = relu_split_state.get(x) if relu_split_state else None
            if sp is not None:
                n = _numel(tr.shape[x])
                t8, stride = _split_tensor(sp, B, n, device, x)
                pl, pu = pl.clone(), pu.clone()
                _lib.check(lib.bf_relu_split_apply(_lib.ptr(pl), _lib.ptr(pu), _lib.ptr(t8), stride, _lib.ptr(tr.infeasible), B, n, s))
            tr.pre_l[x], tr.pre_u[x] = pl, pu
            yl, yu = torch.empty_like(pl), torch.empty_like(pu)
            _lib.check(lib.bf_interval_relu(_lib.ptr(pl), _lib.ptr(pu), _lib.ptr(yl), _lib.ptr(yu), yl.numel(), s))
            tr.lower[out], tr.upper[out], tr.shape[out] = yl, yu, tr.shape[x]
        elif t == "add":
            a, b2 = op.inputs
            for nm in (a, b2):
                if nm not in tr.lower:
                    if nm not in params:
                        raise KeyError(f"missing value in interval_env/params: {nm}")
                    c = params[nm].reshape(1, -1).expand(B, -1).contiguous()
                    tr.lower[nm], tr.upper[nm], tr.shape[nm] = c, c, tuple(int(d) for d in params[nm].shape[-len(tr.shape[a if nm == b2 else b2]):])
            if tr.shape[a] != tr.shape[b2]:
                raise NotImplementedError(f"add supports exact same-shape non-broadcast inputs; got {tr.shape[a]} and {tr.shape[b2]}")
            yl, yu = torch.empty_like(tr.lower[a]), torch.empty_like(tr.upper[a])
            _lib.check(lib.bf_interval_add(_lib.ptr(tr.lower[a]), _lib.ptr(tr.upper[a]), _lib.ptr(tr.lower[b2]), _lib.ptr(tr.upper[b2]),
                                           _lib.ptr(yl), _lib.ptr(yu), yl.numel(), s))
            tr.lower[out], tr.upper[out], tr.shape[out] = yl, yu, tr.shape[a]
        elif t in ("flatten", "reshape"):
            x = op.inputs[0]
            if t == "flatten":
                if int(op.attrs.get("start_dim", 1)) != 1 or int(op.attrs.get("end_dim", -1)) != -1:
                    raise NotImplementedError("only flatten(start_dim=1, end_dim=-1) is supported")
                shp: Tuple[int, ...] = (_numel(tr.shape[x]),)
            else:
                shp = tuple(int(d) for d in op.attrs.get("shape", ()))[1:]
                if _numel(shp) != _numel(tr.shape[x]):
                    raise NotImplementedError("reshape must keep the batch axis and the element count")
            tr.lower[out], tr.upper[out], tr.shape[out] = tr.lower[x], tr.upper[x], shp
            if x in input_views:
                input_views.add(out)
        elif t == "concat":
            if int(op.attrs.get("axis", 1)) not in (1, -len(tr.shape[op.inputs[0]])):
                raise NotImplementedError("concat is supported along the channel axis (axis=1) only")
            shapes = [tr.shape[n] for n in op.inputs]
            if any(sh[1:] != shapes[0][1:] for sh in shapes):
                raise ValueError("concat inputs differ in their trailing dimensions")
            tr.lower[out] = torch.cat([tr.lower[n] for n in op.inputs], dim=1)  # channel-major flat layout: plain concatenation
            tr.upper[out] = torch.cat([tr.upper[n] for n in op.inputs], dim=1)
            tr.shape[out] = (sum(sh[0] for sh in shapes),) + tuple(shapes[0][1:])
        else:
            raise NotImplementedError(f"unsupported op_type in the CUDA graph backend: {t}")
    if relu_pre_constraints is not None and tuple(relu_pre_constraints) != tuple(dict.fromkeys(tr.relu_inputs)):
        raise ValueError("ReLU pre-activation constraint identities differ")
    return tr


class _State:
    """Coefficients [B,S,n] and bias [B,S] of one side for one value."""

    __slots__ = ("A", "d")

    def __init__(self, A: torch.Tensor, d: torch.Tensor):
        self.A, self.d = A, d


def _spec_rows(linear_spec_C: Optional[torch.Tensor], B: int, n_out: int, device: torch.device) -> torch.Tensor:
    if linear_spec_C is None:
        return torch.eye(n_out, dtype=torch.float32, device=device).unsqueeze(0).expand(B, n_out, n_out).contiguous()
    C = _f32(linear_spec_C, device)
    C = (C.unsqueeze(0).expand(B, -1, -1) if C.dim() == 2 else C).contiguous()
    if int(C.shape[0]) != B or int(C.shape[2]) != n_out:
        raise ValueError(f"linear_spec_C shape {tuple(C.shape)} does not match batch {B} and output width {n_out}")
    return C


def _relax(lib, tr: DagTrace, relu_alpha: Optional[Mapping[str, torch.Tensor]], s) -> Dict[str, Tuple[torch.Tensor, torch.Tensor, torch.Tensor]]:
    """Slopes / intercepts of every ReLU from its (split) pre-activation bounds; alpha overrides the lower slope of
    unstable neurons (crown_ibp.py:1176-1208)."""
    device, B = tr.mid.device, tr.B
    relax = {}
    for x in tr.relu_inputs:
        if x in relax:
            continue
        n = _numel(tr.shape[x])
        au, bu, al = (torch.empty(B, n, device=device) for _ in range(3))
        a, stride = (None, 0)
        if relu_alpha is not None and x in relu_alpha and relu_alpha[x] is not None:
            a, stride = _alpha_rows(relu_alpha[x], B, n, device, x)
        _lib.check(lib.bf_relu_relax(_lib.ptr(tr.pre_l[x]), _lib.ptr(tr.pre_u[x]), _lib.ptr(a), stride, _lib.ptr(au), _lib.ptr(bu), _lib.ptr(al), B, n, s))
        relax[x] = (au, bu, al)
    return relax


def _sweep(lib, module: Any, tr: DagTrace, params: Dict[str, torch.Tensor], relax, C: torch.Tensor, side: int, output_value: str, *,
           add_l: Optional[Mapping[str, torch.Tensor]] = None, ahat: Optional[Dict[str, torch.Tensor]] = None):
    """One backward sweep of one side.  Returns (bounds [B,S], final coefficients [B,S,n0]).  `add_l[x]` ([B,n], e.g. the
    split term of beta-CROWN on the lower side) is added to this side's coefficients behind ReLU x; `ahat` (a dict) receives the
    coefficients that arrive at every ReLU's output, which the gradient sweep needs."""
    device, B = tr.mid.device, tr.B
    task = module.get_entry_task()
    S = int(C.shape[1])
    s = _stream_ptr(device)
    dynamic = set(tr.lower) - set(params)
    adj: Dict[str, _State] = {output_value: _State(C.clone(), torch.zeros(B, S, device=device))}

    def push(name: str, A: torch.Tensor, d: torch.Tensor) -> None:
        cur = adj.get(name)
        if cur is None:
            adj[name] = _State(A, d)
            return
        _lib.check(lib.bf_accumulate(_lib.ptr(cur.A), _lib.ptr(A), A.numel(), s))
        _lib.check(lib.bf_accumulate(_lib.ptr(cur.d), _lib.ptr(d), d.numel(), s))

    for op in reversed(task.ops):
        out = op.outputs[0]
        st = adj.pop(out, None)
        if st is None:
            continue
        t = op.op_type
        if t == "linear":
            W = params[op.inputs[1]]
            b = params[op.inputs[2]] if len(op.inputs) == 3 else None
            n_cur, n_prev = int(W.shape[0]), int(W.shape[1])
            Ap = torch.empty(B, S, n_prev, device=device)
            pack = _lib.LINEAR_PACKS.get(W, B * S, s)  # tensor-core path for large coefficient blocks
            _lib.check(lib.bf_crown_relu_linear_bwd_packed(_lib.ptr(st.A), side, None, None, None, None, None, _lib.ptr(W), _lib.ptr(b),
                                                           _lib.ptr(pack), _lib.ptr(Ap), _lib.ptr(st.d), 1, B, S, n_cur, n_prev, s))
            push(op.inputs[0], Ap, st.d)
        elif t == "conv2d":
            W = params[op.inputs[1]]
            b = params[op.inputs[2]] if len(op.inputs) == 3 else None
            Ci, Hi, Wi = tr.shape[op.inputs[0]]
            Co, Ho, Wo = tr.shape[out]
            kh, kw = int(W.shape[2]), int(W.shape[3])
            sth, pdh = _pair(op.attrs.get("stride", 1)), _pair(op.attrs.get("padding", 0))
            Ap = torch.empty(B, S, Ci * Hi * Wi, device=device)
            nb = int(lib.bf_crown_relu_conv2d_bwd_scratch_bytes(B, S, Co, Ho, Wo))
            scratch = torch.empty(max(nb, 16), dtype=torch.uint8, device=device)
            _lib.check(lib.bf_crown_relu_conv2d_bwd(_lib.ptr(st.A), side, None, None, None, None, _lib.ptr(W), _lib.ptr(b), _lib.ptr(Ap),
                                                    _lib.ptr(st.d), 1, _lib.ptr(scratch), scratch.numel(), B, S, Ci, Hi, Wi, Co, Ho, Wo,
                                                    kh, kw, sth[0], sth[1], pdh[0], pdh[1], s))
            push(op.inputs[0], Ap, st.d)
        elif t == "relu":
            x = op.inputs[0]
            n = _numel(tr.shape[x])
            au, bu, al = relax[x]
            zb = torch.zeros(B, n, device=device)
            nb = int(lib.bf_crown_relu_bwd_scratch_bytes(B, S, n))
            scratch = torch.empty(max(nb, 16), dtype=torch.uint8, device=device)
            Ap = torch.empty_like(st.A)
            _lib.check(lib.bf_crown_relu_bwd(_lib.ptr(st.A), side, _lib.ptr(au), _lib.ptr(al), _lib.ptr(bu), _lib.ptr(zb), _lib.ptr(Ap),
                                             _lib.ptr(st.d), 1, _lib.ptr(scratch), scratch.numel(), B, S, n, s))
            if ahat is not None:
                ahat[x] = st.A  # left untouched by the call above
            if add_l is not None and add_l.get(x) is not None:
                _lib.check(lib.bf_rows_add_broadcast(_lib.ptr(Ap), _lib.ptr(add_l[x]), n, B, S, n, s))
            push(x, Ap, st.d)
        elif t == "add":
            d = st.d
            dyn = []
            for nm in op.inputs:
                if nm in dynamic:
                    dyn.append(nm)
                else:  # a constant operand adds A . value to the bias (crown_ibp.py:1948-1950)
                    const = tr.lower[nm].reshape(B, 1, -1)
                    d = d + (st.A * const).sum(dim=2)
            for k, nm in enumerate(dyn):
                # the same coefficients for every operand; the bias travels with the first one only
                push(nm, st.A.clone() if k + 1 < len(dyn) or nm in adj else st.A, d if k == 0 else torch.zeros_like(d))
        elif t in ("flatten", "reshape"):
            push(op.inputs[0], st.A, st.d)
        elif t == "concat":
            start = 0
            for k, nm in enumerate(op.inputs):
                w = _numel(tr.shape[nm])
                push(nm, st.A[:, :, start : start + w].contiguous(), st.d if k == 0 else torch.zeros_like(st.d))
                start += w
        else:
            raise NotImplementedError(f"run_crown_ibp_mlp unsupported op_type in backward: {t}")
    if tr.input_name not in adj:
        raise RuntimeError(f"backward did not reach input value {tr.input_name}")
    fin = adj[tr.input_name]
    res = torch.empty(B, S, device=device)
    if tr.norm_p != _lib.NORM_BOX:
        _lib.check(lib.bf_concretize_lp(_lib.ptr(fin.A), _lib.ptr(tr.mid), tr.eps, tr.norm_p, _lib.ptr(fin.d), _lib.ptr(res), side, B, S,
                                        int(tr.mid.shape[1]), s))
    else:
        _lib.check(lib.bf_concretize(_lib.ptr(fin.A), _lib.ptr(tr.mid), _lib.ptr(tr.rad), _lib.ptr(fin.d), _lib.ptr(res), side, B, S,
                                     int(tr.mid.shape[1]), s))
    return res, fin.A


def _output_value(module: Any, tr: DagTrace, output_value: Optional[str]) -> str:
    task = module.get_entry_task()
    if output_value is None:
        if len(task.output_values) != 1:
            raise ValueError(f"task has {len(task.output_values)} outputs; specify output_value explicitly")
        output_value = task.output_values[0]
    if output_value not in tr.shape:
        raise KeyError(f"missing value in interval_env/params: {output_value}")
    return output_value


def crown_dag(module: Any, input_spec: Any, linear_spec_C: Optional[torch.Tensor], *, output_value: Optional[str] = None,
              trace: Optional[DagTrace] = None, relu_split_state: Optional[Mapping[str, torch.Tensor]] = None,
              relu_alpha: Optional[Mapping[str, torch.Tensor]] = None,
              relu_pre_add_coeff_l: Optional[Mapping[str, torch.Tensor]] = None,
              relu_pre_add_coeff_u: Optional[Mapping[str, torch.Tensor]] = None) -> Tuple[torch.Tensor, torch.Tensor, DagTrace]:
    """CROWN-IBP on a graph: IBP bounds for every ReLU input (with the ReLU splits, if any), then one backward sweep
    per side; `relu_alpha` overrides the lower slopes of unstable neurons, `relu_pre_add_coeff_l` / `_u` is added to the
    lower / upper coefficients behind a ReLU (crown_ibp.py:1270-1296, 2136-2152).  Returns (lower, upper) [B,S] CUDA
    tensors and the trace."""
    lib = _lib.load()
    spec = normalize_input_spec(input_spec)
    tr = trace if trace is not None else forward_ibp_dag(module, spec, relu_split_state)
    if int(tr.infeasible.sum()) != 0:
        raise ValueError("infeasible relu split: lower > upper")
    device, B = tr.mid.device, tr.B
    params = _params(module, device)
    output_value = _output_value(module, tr, output_value)
    C = _spec_rows(linear_spec_C, B, _numel(tr.shape[output_value]), device)
    s = _stream_ptr(device)
    relax = _relax(lib, tr, relu_alpha, s)
    def terms(raw):
        if not raw:
            return None
        return {x: _f32(v, device).reshape(-1, _numel(tr.shape[x])).expand(B, -1).contiguous() for x, v in raw.items() if v is not None}

    lo, _ = _sweep(lib, module, tr, params, relax, C, _lib.SIDE_LOWER, output_value, add_l=terms(relu_pre_add_coeff_l))
    up, _ = _sweep(lib, module, tr, params, relax, C, _lib.SIDE_UPPER, output_value, add_l=terms(relu_pre_add_coeff_u))
    return lo, up, tr


def crown_influence_dag(module: Any, input_spec: Any, linear_spec_C: Optional[torch.Tensor], *, output_value: Optional[str] = None,
                        trace: Optional[DagTrace] = None):
    """CROWN-IBP on a graph plus, per ReLU input, max(max_s |A_u|, max_s |A_l|) of the coefficients that arrive at the
    ReLU's output in the two sweeps (`run_crown_ibp_mlp_with_relu_influence_from_forward_trace`, crown_ibp.py:1810-1834,
    2201-2240).  Returns (lower, upper, {name: [B, n]}, trace); a ReLU the sweep never reaches has no entry."""
    lib = _lib.load()
    spec = normalize_input_spec(input_spec)
    tr = trace if trace is not None else forward_ibp_dag(module, spec)
    device, B = tr.mid.device, tr.B
    params = _params(module, device)
    output_value = _output_value(module, tr, output_value)
    C = _spec_rows(linear_spec_C, B, _numel(tr.shape[output_value]), device)
    S = int(C.shape[1])
    s = _stream_ptr(device)
    relax = _relax(lib, tr, None, s)
    at_l: Dict[str, torch.Tensor] = {}
    at_u: Dict[str, torch.Tensor] = {}
    lo, _ = _sweep(lib, module, tr, params, relax, C, _lib.SIDE_LOWER, output_value, ahat=at_l)
    up, _ = _sweep(lib, module, tr, params, relax, C, _lib.SIDE_UPPER, output_value, ahat=at_u)
    influence: Dict[str, torch.Tensor] = {}
    for x in at_l:
        n = _numel(tr.shape[x])
        out = torch.zeros(B, n, dtype=torch.float32, device=device)
        for A in (at_l[x], at_u[x]):
            _lib.check(lib.bf_rows_colmax_abs(_lib.ptr(A), _lib.ptr(out), B, S, n, s))
        influence[x] = out
    return lo, up, influence, tr


def _adjoint_forward(lib, module: Any, tr: DagTrace, params: Dict[str, torch.Tensor], relax, A0: torch.Tensor, ahat: Dict[str, torch.Tensor],
                     grad: Dict[str, torch.Tensor], gsum: Optional[Dict[str, torch.Tensor]], S: int,
                     row_weight: Optional[torch.Tensor] = None) -> None:
    """Gradient sweep: the lower bound of row s equals C[s] . f_s(h0), where f_s is the network with every ReLU
    replaced by the line the backward sweep chose for that row and h0 = mid - sgn(A0) * rad.  Pushing h0 forward through
    the graph gives, at every ReLU input, the value g with d lower / d alpha = [l<0<u][Ahat>=0] Ahat * g and
    d lower / d add = g (`bf_relu_adjoint_rows` accumulates both per domain; `row_weight` [B,S] weights the rows of the
    second sum, the first one is weighted through `ahat`)."""
    device, B = tr.mid.device, tr.B
    task = module.get_entry_task()
    s = _stream_ptr(device)
    if tr.norm_p != _lib.NORM_BOX:
        _lib.check(lib.bf_adjoint_start_lp(_lib.ptr(A0), _lib.ptr(tr.mid), tr.eps, tr.norm_p, B, S, int(tr.mid.shape[1]), s))
    else:
        _lib.check(lib.bf_adjoint_start_box(_lib.ptr(A0), _lib.ptr(tr.mid), _lib.ptr(tr.rad), B, S, int(tr.mid.shape[1]), s))
    h: Dict[str, torch.Tensor] = {tr.input_name: A0}
    for op in task.ops:
        t, out = op.op_type, op.outputs[0]
        if t == "linear":
            x = op.inputs[0]
            if x not in h:
                continue
            W = params[op.inputs[1]]
            b = params[op.inputs[2]] if len(op.inputs) == 3 else None
            n_out, n_in = int(W.shape[0]), int(W.shape[1])
            Wt = _TRANSPOSED.get(W)
            g = torch.empty(B, S, n_out, device=device)
            # rows x W^T: the backward entry point on the transposed weight, no slopes, no bias term
            _lib.check(lib.bf_crown_relu_linear_bwd(_lib.ptr(h[x]), _lib.SIDE_LOWER, None, None, None, None, None, _lib.ptr(Wt), None,
                                                    _lib.ptr(g), None, 0, B, S, n_in, n_out, s))
            if b is not None:
                _lib.check(lib.bf_rows_add_broadcast(_lib.ptr(g), _lib.ptr(b), 0, B, S, n_out, s))
            h[out] = g
        elif t == "conv2d":
            x = op.inputs[0]
            if x not in h:
                continue
            W = params[op.inputs[1]]
            b = params[op.inputs[2]] if len(op.inputs) == 3 else None
            Ci, Hi, Wi = tr.shape[x]
            Co, Ho, Wo = tr.shape[out]
            sth, pdh = _pair(op.attrs.get("stride", 1)), _pair(op.attrs.get("padding", 0))
            g = torch.empty(B, S, Co * Ho * Wo, device=device)
            _lib.check(lib.bf_rows_conv2d_fwd(_lib.ptr(h[x]), _lib.ptr(W), _lib.ptr(b), _lib.ptr(g), B * S, Ci, Hi, Wi, Co, Ho, Wo, int(W.shape[2]),
                                              int(W.shape[3]), sth[0], sth[1], pdh[0], pdh[1], s))
            h[out] = g
        elif t == "relu":
            x = op.inputs[0]
            if x not in h or x not in ahat:   # no coefficients arrived here: the value does not reach the output
                continue
            n = _numel(tr.shape[x])
            au, bu, al = relax[x]
            G = h[x].clone()                  # x may feed other ops as well
            _lib.check(lib.bf_relu_adjoint_rows(_lib.ptr(G), _lib.ptr(ahat[x]), _lib.ptr(au), _lib.ptr(al), _lib.ptr(bu), _lib.ptr(tr.pre_l[x]),
                                                _lib.ptr(tr.pre_u[x]), _lib.ptr(grad[x]), _lib.ptr(gsum[x]) if gsum is not None else None,
                                                _lib.ptr(row_weight) if (gsum is not None and row_weight is not None) else None, B, S, n, s))
            h[out] = G
        elif t == "add":
            terms = [nm for nm in op.inputs if nm in h]
            if not terms:
                continue
            acc = h[terms[0]].clone()
            for nm in terms[1:]:
                _lib.check(lib.bf_accumulate(_lib.ptr(acc), _lib.ptr(h[nm]), acc.numel(), s))
            for nm in op.inputs:
                if nm in params and nm not in h:   # constant operand
                    c = params[nm].reshape(-1).contiguous()
                    _lib.check(lib.bf_rows_add_broadcast(_lib.ptr(acc), _lib.ptr(c), 0, B, S, int(c.numel()), s))
            h[out] = acc
        elif t in ("flatten", "reshape"):
            if op.inputs[0] in h:
                h[out] = h[op.inputs[0]]
        elif t == "concat":
            if all(nm in h for nm in op.inputs):
                h[out] = torch.cat([h[nm] for nm in op.inputs], dim=2)
        else:
            raise NotImplementedError(f"unsupported op_type in the gradient sweep: {t}")


class _TransposedWeights:
    """W^T copies for the forward Linear step of the gradient sweep, one per weight tensor.  Like the packed-weight
    cache, an entry is keyed by storage address, shape, device and in-place version counter and keeps the weight tensor
    itself alive, so an address cannot be reused by another tensor while its transpose is cached; least recently used
    entries are dropped beyond `capacity`."""

    def __init__(self, capacity: int = 32):
        self.capacity = int(capacity)
        self._entries: Dict[Tuple[int, Tuple[int, ...], Optional[int], int], Tuple[torch.Tensor, torch.Tensor]] = {}

    def get(self, W: torch.Tensor) -> torch.Tensor:
        key = (W.data_ptr(), tuple(W.shape), W.device.index, int(W._version))
        hit = self._entries.pop(key, None)
        if hit is None:
            hit = (W, W.t().contiguous())
            while len(self._entries) >= self.capacity:
                self._entries.pop(next(iter(self._entries)))
        self._entries[key] = hit  # most recently used last
        return hit[1]


_TRANSPOSED = _TransposedWeights()


def alpha_beta_crown_dag(module: Any, input_spec: Any, linear_spec_C: Optional[torch.Tensor], *, steps: int, lr: float,
                         alpha0: Optional[Mapping[str, torch.Tensor]] = None, alpha_init: float = 0.5,
                         relu_split_state: Optional[Mapping[str, torch.Tensor]] = None, optimize_beta: bool = False,
                         beta0: Optional[Mapping[str, torch.Tensor]] = None, beta_init: float = 0.0, spec_reduce: str = "mean",
                         soft_tau: float = 1.0, objective: str = "lower", lb_weight: float = 1.0, ub_weight: float = 1.0,
                         per_batch_params: bool = True, output_value: Optional[str] = None):
    """alpha (and beta) loop on a graph that is not a chain: `run_alpha_beta_crown_mlp` (alpha_beta_crown.py:716-923),
    whose sweep is the reference's generic graph backward.  steps + 1 evaluations; each is one lower sweep that keeps
    the coefficients at every ReLU, the objective with strict best-of, one gradient sweep and one Adam step per ReLU.

    `per_batch_params=True`: one parameter row and one best-of per domain; False: one row shared by the batch and a
    whole-batch best-of on the mean of the per-domain objectives.  `objective` lower | upper | gap | both (807-818):
    upper runs on the negated spec rows, gap / both on the rows followed by their negations (2S rows per domain, row
    weights from the objective's derivative scale the kept coefficients before the gradient sweep).  `spec_reduce`
    mean | min | softmin (787-805), plus sum for lower.  beta enters objective="lower" only (763-785).
    Returns (best_lower, best_upper, best_alpha dict, best_beta dict, trace); alpha / beta are [B, n] ([1, n] in the
    shared mode) per ReLU input name."""
    lib = _lib.load()
    codes = {"mean": _lib.REDUCE_MEAN, "sum": _lib.REDUCE_SUM, "min": _lib.REDUCE_MIN, "softmin": _lib.REDUCE_SOFTMIN}
    if objective not in ("lower", "upper", "gap", "both"):
        raise ValueError(f"objective={objective!r}: expected lower | upper | gap | both")
    if spec_reduce not in codes or (spec_reduce == "sum" and (objective != "lower" or not per_batch_params)):
        raise ValueError(f"spec_reduce={spec_reduce!r}: expected mean | min | softmin (sum with the per-domain lower objective only)")
    if spec_reduce == "softmin" and float(soft_tau) <= 0.0:
        raise ValueError(f"soft_tau must be >0, got {soft_tau}")
    paired = objective in ("gap", "both")
    if paired and (float(lb_weight) < 0.0 or float(ub_weight) < 0.0):
        raise NotImplementedError("the CUDA backend takes non-negative lb_weight / ub_weight (a row weight must not flip the sign decisions of the gradient sweep)")
    weighted = paired or spec_reduce in ("min", "softmin")
    with_beta = bool(optimize_beta and relu_split_state and objective == "lower")
    spec = normalize_input_spec(input_spec)
    tr = forward_ibp_dag(module, spec, relu_split_state)
    if int(tr.infeasible.sum()) != 0:
        raise ValueError("infeasible relu split: lower > upper")
    device, B = tr.mid.device, tr.B
    params = _params(module, device)
    output_value = _output_value(module, tr, output_value)
    C0 = _spec_rows(linear_spec_C, B, _numel(tr.shape[output_value]), device)
    S0 = int(C0.shape[1])
    C = -C0 if objective == "upper" else (torch.cat([C0, -C0], dim=1).contiguous() if paired else C0)
    S = int(C.shape[1])
    M = B * S
    s = _stream_ptr(device)
    names = list(dict.fromkeys(tr.relu_inputs))
    width = {x: _numel(tr.shape[x]) for x in names}
    rows = B if per_batch_params else 1

    def start(raw, x, init):
        n = width[x]
        if raw is not None and x in raw and raw[x] is not None:
            t, _ = _alpha_rows(raw[x], rows, n, device, x)
            if not per_batch_params and int(t.shape[0]) != 1:
                raise ValueError(f"warm start [{x}] is batch-specific; expected the shared shape {tuple(tr.shape[x])}")
            return t.expand(rows, n).contiguous().clone()
        return torch.full((rows, n), float(init), dtype=torch.float32, device=device)

    zeros = lambda x, r=B: torch.zeros(r, width[x], dtype=torch.float32, device=device)  # noqa: E731
    alpha = {x: start(alpha0, x, alpha_init) for x in names}
    best_alpha = {x: alpha[x].clone() for x in names}
    m, v = ({x: zeros(x, rows) for x in names} for _ in range(2))
    grad, slope = ({x: zeros(x) for x in names} for _ in range(2))
    beta = {x: start(beta0, x, beta_init) for x in names}
    best_beta = {x: beta[x].clone() for x in names}
    splits: Dict[str, Tuple[Optional[torch.Tensor], int]] = {}
    if with_beta:
        mb, vb = ({x: zeros(x, rows) for x in names} for _ in range(2))
        gsum, addv = ({x: zeros(x) for x in names} for _ in range(2))
        for x in names:
            sp = relu_split_state.get(x)
            if sp is not None:
                splits[x] = _split_tensor(sp, B, width[x], device, x)
            else:
                splits[x] = (torch.zeros(1, width[x], dtype=torch.int8, device=device), 0) if per_batch_params else (None, 0)
        if per_batch_params:
            for x in names:  # split term of the start beta
                _lib.check(lib.bf_beta_adam_step(_lib.ptr(beta[x]), _lib.ptr(mb[x]), _lib.ptr(vb[x]), _lib.ptr(gsum[x]), _lib.ptr(splits[x][0]),
                                                 splits[x][1], None, None, _lib.ptr(addv[x]), 0, float(lr), codes[spec_reduce], S, 0, B, width[x], s))
    best_rows = torch.empty(B, S, dtype=torch.float32, device=device)
    best_metric = torch.empty(rows, dtype=torch.float32, device=device)
    improve = torch.zeros(rows, dtype=torch.int32, device=device)
    row_weight = torch.empty(B, S, dtype=torch.float32, device=device) if weighted else None
    if not per_batch_params:
        scratch = torch.empty(max(int(lib.bf_shared_adam_scratch_floats(B, width[x])) for x in names) if names else 1, dtype=torch.float32, device=device)
        if weighted:
            dom_rows = torch.empty(B, S, dtype=torch.float32, device=device)
            dom_metric = torch.empty(B, dtype=torch.float32, device=device)
            dom_improve = torch.zeros(B, dtype=torch.int32, device=device)
    obj_code = _lib.OBJECTIVE_GAP if objective == "gap" else _lib.OBJECTIVE_BOTH
    # d loss / d lower of the Adam steps: row weights already carry 1/S of a paired mean
    per_domain_reduce = _lib.REDUCE_SUM if paired else codes[spec_reduce]
    shared_scale = (-1.0 / B) if weighted else (-1.0 / M)

    def select(cur, rows_out, metric_out, improve_out, first, rw):
        if paired:
            _lib.check(lib.bf_alpha_select_best_paired(_lib.ptr(cur), _lib.ptr(rows_out), _lib.ptr(metric_out), _lib.ptr(improve_out), first, obj_code,
                                                       codes[spec_reduce], float(soft_tau), float(lb_weight), float(ub_weight), _lib.ptr(rw), B, S0, s))
        else:
            _lib.check(lib.bf_alpha_select_best(_lib.ptr(cur), _lib.ptr(rows_out), _lib.ptr(metric_out), _lib.ptr(improve_out), first,
                                                codes[spec_reduce], float(soft_tau), _lib.ptr(rw), B, S, s))

    for t in range(int(steps) + 1):
        last = t == int(steps)
        relax = _relax(lib, tr, alpha, s)
        if with_beta and not per_batch_params:
            for x in names:
                if splits[x][0] is not None:
                    _lib.check(lib.bf_shared_beta_add(_lib.ptr(beta[x]), _lib.ptr(splits[x][0]), splits[x][1], _lib.ptr(addv[x]), B, width[x], s))
        ahat: Dict[str, torch.Tensor] = {}
        cur, A0 = _sweep(lib, module, tr, params, relax, C, _lib.SIDE_LOWER, output_value, add_l=addv if with_beta else None, ahat=ahat)
        rw = row_weight if (weighted and not last) else None
        if per_batch_params:
            select(cur, best_rows, best_metric, improve, 1 if t == 0 else 0, rw)
        else:
            if weighted:  # per-domain objective and its derivative (no per-domain best-of), then the batch mean
                select(cur, dom_rows, dom_metric, dom_improve, 1, rw)
                _lib.check(lib.bf_shared_metric(_lib.ptr(dom_metric), B, _lib.ptr(best_metric), _lib.ptr(improve), 1 if t == 0 else 0, s))
            else:
                _lib.check(lib.bf_shared_metric(_lib.ptr(cur), M, _lib.ptr(best_metric), _lib.ptr(improve), 1 if t == 0 else 0, s))
            _lib.check(lib.bf_copy_if(_lib.ptr(cur), _lib.ptr(best_rows), M, _lib.ptr(improve), s))
        if not last:
            if weighted:
                done = set()
                for x, A in ahat.items():
                    if A.data_ptr() not in done:
                        done.add(A.data_ptr())
                        _lib.check(lib.bf_rows_scale(_lib.ptr(A), _lib.ptr(row_weight), M, width[x], s))
            _adjoint_forward(lib, module, tr, params, relax, A0, ahat, grad, gsum if with_beta else None, S, row_weight if weighted else None)
        upd = 0 if last else 1
        for x in names:
            n = width[x]
            if per_batch_params:
                _lib.check(lib.bf_alpha_adam_step(_lib.ptr(alpha[x]), _lib.ptr(m[x]), _lib.ptr(v[x]), _lib.ptr(grad[x]), _lib.ptr(improve), _lib.ptr(best_alpha[x]),
                                                  _lib.ptr(tr.pre_l[x]), _lib.ptr(tr.pre_u[x]), _lib.ptr(slope[x]), t, float(lr), per_domain_reduce, S,
                                                  upd, B, n, s))
                if with_beta:
                    _lib.check(lib.bf_beta_adam_step(_lib.ptr(beta[x]), _lib.ptr(mb[x]), _lib.ptr(vb[x]), _lib.ptr(gsum[x]), _lib.ptr(splits[x][0]),
                                                     splits[x][1], _lib.ptr(improve), _lib.ptr(best_beta[x]), _lib.ptr(addv[x]), t, float(lr),
                                                     per_domain_reduce, S, upd, B, n, s))
            else:
                _lib.check(lib.bf_shared_adam_step(_lib.ptr(alpha[x]), _lib.ptr(m[x]), _lib.ptr(v[x]), _lib.ptr(grad[x]), None, 0, _lib.ptr(scratch),
                                                   _lib.ptr(improve), _lib.ptr(best_alpha[x]), t, float(lr), shared_scale, upd, 0, B, n, s))
                if with_beta:
                    sp, st = splits[x]  # without a split on this ReLU the beta gradient is identically zero: snapshot only
                    _lib.check(lib.bf_shared_adam_step(_lib.ptr(beta[x]), _lib.ptr(mb[x]), _lib.ptr(vb[x]), _lib.ptr(gsum[x]), _lib.ptr(sp), st,
                                                       _lib.ptr(scratch), _lib.ptr(improve), _lib.ptr(best_beta[x]), t, float(lr), shared_scale,
                                                       upd if sp is not None else 0, 1, B, n, s))
    if paired:
        return best_rows[:, :S0].contiguous(), -best_rows[:, S0:], best_alpha, best_beta, tr
    # the other side at each domain's best alpha (beta acts on the lower side only)
    relax = _relax(lib, tr, best_alpha, s)
    other, _ = _sweep(lib, module, tr, params, relax, C, _lib.SIDE_UPPER, output_value)
    if objective == "upper":
        return -other, -best_rows, best_alpha, best_beta, tr
    return best_rows, other, best_alpha, best_beta, tr


def first_layer_certificate_dag(module: Any, input_spec: Any, relu_split_state: Mapping[str, torch.Tensor], *, steps: int = 200,
                                lr: float = 0.1, tol: float = 1e-6):
    """First-layer infeasibility certificate on a graph (`_is_infeasible_split_first_layer_convex_combo`,
    alpha_beta_crown.py:255-532): every ReLU whose input is produced by a Linear or Conv2d op that reads the input value
    contributes the half-spaces of its split neurons (264-387); the rows of all of them are stacked and handed to the
    certificate kernel.  Returns (infeasible int32 [B]: 1 found / 0 none, best_value [B], n_halfspaces int32 [B])."""
    lib = _lib.load()
    spec = normalize_input_spec(input_spec)
    ball = lp_ball_of(spec)
    device = _cuda_device(spec.center)
    B = int(spec.center.shape[0])
    if ball is not None:
        mid, rad = _f32(spec.center, device).reshape(B, -1).contiguous(), None
    else:
        mid, rad, _lo, _up = input_mid_rad(spec)
        mid, rad = _f32(mid, device).reshape(B, -1).contiguous(), _f32(rad, device).reshape(B, -1).contiguous()
    n0 = int(mid.shape[1])
    infeasible = torch.zeros(B, dtype=torch.int32, device=device)
    best = torch.full((B,), float("inf"), dtype=torch.float32, device=device)
    count = torch.zeros(B, dtype=torch.int32, device=device)
    task = module.get_entry_task()
    params = _params(module, device)
    producer = {op.outputs[0]: op for op in task.ops}
    in_shape = tuple(int(d) for d in spec.center.shape[1:])
    s = _stream_ptr(device)
    W_parts, b_parts, sp_parts, per_domain = [], [], [], False
    seen = set()
    for op in task.ops:
        if op.op_type != "relu" or op.inputs[0] in seen:
            continue
        x = op.inputs[0]
        seen.add(x)
        raw = relu_split_state.get(x) if relu_split_state else None
        prod = producer.get(x)
        if raw is None or prod is None or prod.op_type not in ("linear", "conv2d") or not prod.inputs or prod.inputs[0] != spec.value_name:
            continue
        W = params[prod.inputs[1]]
        b = params[prod.inputs[2]] if len(prod.inputs) == 3 else None
        if prod.op_type == "linear":
            n1 = int(W.shape[0])
        else:
            if len(in_shape) != 3:
                continue
            Ci, Hi, Wi = in_shape
            kh, kw = int(W.shape[2]), int(W.shape[3])
            sth, pdh = _pair(prod.attrs.get("stride", 1)), _pair(prod.attrs.get("padding", 0))
            Co = int(W.shape[0])
            Ho, Wo = (Hi + 2 * pdh[0] - kh) // sth[0] + 1, (Wi + 2 * pdh[1] - kw) // sth[1] + 1
            n1 = Co * Ho * Wo
        sp, stride = _split_tensor(raw, B, n1, device, x)
        cols = torch.nonzero((sp != 0).any(dim=0)).flatten()   # neurons split in at least one domain, ascending
        U = int(cols.numel())
        if U == 0:
            continue
        if prod.op_type == "linear":
            W_rows = W.index_select(0, cols).contiguous()
            b_rows = b.index_select(0, cols).contiguous() if b is not None else torch.zeros(U, dtype=torch.float32, device=device)
        else:
            W_rows = torch.empty(U, n0, dtype=torch.float32, device=device)
            b_rows = torch.empty(U, dtype=torch.float32, device=device)
            rows = cols.to(torch.int32).contiguous()
            _lib.check(lib.bf_conv2d_dense_rows(_lib.ptr(W), _lib.ptr(b), _lib.ptr(rows), U, _lib.ptr(W_rows), _lib.ptr(b_rows), Ci, Hi, Wi, Co, Ho, Wo,
                                                kh, kw, sth[0], sth[1], pdh[0], pdh[1], s))
        W_parts.append(W_rows)
        b_parts.append(b_rows)
        sp_parts.append(sp[:, cols])
        per_domain = per_domain or stride != 0
    if not W_parts:
        return infeasible, best, count
    rows_sp = B if per_domain else 1
    W_all, b_all = torch.cat(W_parts, dim=0).contiguous(), torch.cat(b_parts, dim=0).contiguous()
    sp_all = torch.cat([p.expand(rows_sp, -1) for p in sp_parts], dim=1).contiguous()
    U = int(W_all.shape[0])
    if ball is not None:
        _lib.check(lib.bf_first_layer_certificate_lp(_lib.ptr(sp_all), U if per_domain else 0, _lib.ptr(W_all), _lib.ptr(b_all), _lib.ptr(mid), float(ball[1]),
                                                     int(ball[0]), _lib.ptr(infeasible), _lib.ptr(best), _lib.ptr(count), int(steps), float(lr),
                                                     float(tol), B, U, n0, s))
    else:
        _lib.check(lib.bf_first_layer_certificate(_lib.ptr(sp_all), U if per_domain else 0, _lib.ptr(W_all), _lib.ptr(b_all), _lib.ptr(mid), _lib.ptr(rad),
                                                  _lib.ptr(infeasible), _lib.ptr(best), _lib.ptr(count), int(steps), float(lr), float(tol), B, U, n0, s))
    return infeasible, best, count


def run_crown_ibp_dag(module: Any, input_spec: Any, *, linear_spec_C: Optional[torch.Tensor] = None,
                      output_value: Optional[str] = None, relu_alpha: Optional[Mapping[str, torch.Tensor]] = None,
                      relu_pre_add_coeff_l: Optional[Mapping[str, torch.Tensor]] = None,
                      relu_split_state: Optional[Mapping[str, torch.Tensor]] = None,
                      relu_pre_add_coeff_u: Optional[Mapping[str, torch.Tensor]] = None) -> IntervalState:
    """`run_crown_ibp_mlp` (crown_ibp.py:2054-2133) for graphs with add / concat / fan-out."""
    lo, up, _tr = crown_dag(module, input_spec, linear_spec_C, output_value=output_value, relu_split_state=relu_split_state,
                            relu_alpha=relu_alpha, relu_pre_add_coeff_l=relu_pre_add_coeff_l, relu_pre_add_coeff_u=relu_pre_add_coeff_u)
    dev = normalize_input_spec(input_spec).center.device
    return IntervalState(lower=lo.to(dev), upper=up.to(dev))


def run_ibp_dag(module: Any, input_spec: Any, *, output_value: Optional[str] = None) -> IntervalState:
    """IBP bounds of a value of the graph, shaped like the value."""
    tr = forward_ibp_dag(module, input_spec)
    task = module.get_entry_task()
    name = output_value or task.output_values[0]
    if name not in tr.shape:
        raise KeyError(f"missing value in env/params: {name}")
    dev = normalize_input_spec(input_spec).center.device
    shape = (tr.B,) + tuple(tr.shape[name])
    return IntervalState(lower=tr.lower[name].reshape(shape).to(dev), upper=tr.upper[name].reshape(shape).to(dev))
