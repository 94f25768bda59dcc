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
from .crown import _cuda_device, _f32, _stream_ptr
from .ir import IntervalState, input_mid_rad, lp_ball_of, normalize_input_spec


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
    B: int = 0
    mid: Optional[torch.Tensor] = None
    rad: Optional[torch.Tensor] = None
    input_name: str = ""


def _params(module: Any, device: torch.device) -> Dict[str, torch.Tensor]:
    raw = module.bindings.get("params", {})
    out = {}
    for k, v in (raw.items() if isinstance(raw, dict) else []):
        t = v if torch.is_tensor(v) else torch.as_tensor(v)
        out[k] = _f32(t, device)
    return out


def forward_ibp_dag(module: Any, input_spec: Any) -> DagTrace:
    """One IBP pass over the ops in order (`_forward_ibp_trace_mlp`, crown_ibp.py:101-342, without splits)."""
    lib = _lib.load()
    spec = normalize_input_spec(input_spec)
    if lp_ball_of(spec) is not None:
        raise NotImplementedError("the graph path supports boxes and L-inf balls")
    device = _cuda_device(spec.center)
    task = module.get_entry_task()
    params = _params(module, device)
    mid, rad, lo, up = input_mid_rad(spec)
    B = int(spec.center.shape[0])
    tr = DagTrace(B=B, input_name=spec.value_name)
    tr.mid, tr.rad = _f32(mid, device).reshape(B, -1), _f32(rad, device).reshape(B, -1)
    tr.lower[spec.value_name], tr.upper[spec.value_name] = _f32(lo, device).reshape(B, -1), _f32(up, device).reshape(B, -1)
    tr.shape[spec.value_name] = tuple(int(d) for d in spec.center.shape[1:])
    s = _stream_ptr(device)
    for op in task.ops:
        t, out = op.op_type, op.outputs[0]
        if t in ("linear", "conv2d"):
            x = op.inputs[0]
            W = params[op.inputs[1]]
            b = params[op.inputs[2]] if len(op.inputs) == 3 else None
            at_input = x == spec.value_name
            if t == "linear":
                n_in, n_out = int(W.shape[1]), int(W.shape[0])
                if _numel(tr.shape[x]) != n_in:
                    raise ValueError(f"linear '{op.name}': weight {tuple(W.shape)} does not match input shape {tr.shape[x]}")
                yl, yu = torch.empty(B, n_out, device=device), torch.empty(B, n_out, device=device)
                a, bb, mode = (tr.mid, tr.rad, _lib.IN_MID_RAD) if at_input else (tr.lower[x], tr.upper[x], _lib.IN_LOWER_UPPER)
                _lib.check(lib.bf_ibp_linear(_lib.ptr(a), _lib.ptr(bb), mode, 0, _lib.ptr(W), _lib.ptr(b), None, 0, None, None,
                                             _lib.ptr(yl), _lib.ptr(yu), None, B, n_in, n_out, s))
                tr.shape[out] = (n_out,)
            else:
                if int(op.attrs.get("groups", 1)) != 1 or _pair(op.attrs.get("dilation", 1)) != (1, 1):
                    raise NotImplementedError("conv2d with dilation or groups is not supported by the CUDA backend")
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
            yl, yu = torch.empty_like(tr.lower[x]), torch.empty_like(tr.upper[x])
            _lib.check(lib.bf_interval_relu(_lib.ptr(tr.lower[x]), _lib.ptr(tr.upper[x]), _lib.ptr(yl), _lib.ptr(yu), yl.numel(), s))
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
    return tr


class _State:
    """Coefficients [B,S,n] and bias [B,S] of one side for one value."""

    __slots__ = ("A", "d")

    def __init__(self, A: torch.Tensor, d: torch.Tensor):
        self.A, self.d = A, d


def crown_dag(module: Any, input_spec: Any, linear_spec_C: Optional[torch.Tensor], *, output_value: Optional[str] = None,
              trace: Optional[DagTrace] = None) -> Tuple[torch.Tensor, torch.Tensor, DagTrace]:
    """CROWN-IBP on a graph: IBP bounds for every ReLU input, then one backward sweep per side.
    Returns (lower, upper) [B,S] CUDA tensors and the forward trace."""
    lib = _lib.load()
    spec = normalize_input_spec(input_spec)
    tr = trace if trace is not None else forward_ibp_dag(module, spec)
    device, B = tr.mid.device, tr.B
    task = module.get_entry_task()
    params = _params(module, device)
    if output_value is None:
        if len(task.output_values) != 1:
            raise ValueError(f"task has {len(task.output_values)} outputs; specify output_value explicitly")
        output_value = task.output_values[0]
    if output_value not in tr.shape:
        raise KeyError(f"missing value in interval_env/params: {output_value}")
    n_out = _numel(tr.shape[output_value])
    if linear_spec_C is None:
        C = torch.eye(n_out, dtype=torch.float32, device=device).unsqueeze(0).expand(B, n_out, n_out).contiguous()
    else:
        C = _f32(linear_spec_C, device)
        C = (C.unsqueeze(0).expand(B, -1, -1) if C.dim() == 2 else C).contiguous()
        if int(C.shape[0]) != B or int(C.shape[2]) != n_out:
            raise ValueError(f"linear_spec_C shape {tuple(C.shape)} does not match batch {B} and output width {n_out}")
    S = int(C.shape[1])
    s = _stream_ptr(device)
    # ReLU relaxations from the IBP pre-activations
    relax: Dict[str, Tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = {}
    for x in tr.relu_inputs:
        n = _numel(tr.shape[x])
        au, bu, al = (torch.empty(B, n, device=device) for _ in range(3))
        _lib.check(lib.bf_relu_relax(_lib.ptr(tr.lower[x]), _lib.ptr(tr.upper[x]), None, 0, _lib.ptr(au), _lib.ptr(bu), _lib.ptr(al), B, n, s))
        relax[x] = (au, bu, al)
    zero_beta: Dict[int, torch.Tensor] = {}
    dynamic = set(tr.lower) - set(params)

    outs = []
    for side in (_lib.SIDE_LOWER, _lib.SIDE_UPPER):
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
                zb = zero_beta.get(n)
                if zb is None:
                    zb = zero_beta[n] = torch.zeros(B, n, device=device)
                nb = int(lib.bf_crown_relu_bwd_scratch_bytes(B, S, n))
                scratch = torch.empty(max(nb, 16), dtype=torch.uint8, device=device)
                Ap = torch.empty_like(st.A)
                _lib.check(lib.bf_crown_relu_bwd(_lib.ptr(st.A), side, _lib.ptr(au), _lib.ptr(al), _lib.ptr(bu), _lib.ptr(zb), _lib.ptr(Ap),
                                                 _lib.ptr(st.d), 1, _lib.ptr(scratch), scratch.numel(), B, S, n, s))
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
        _lib.check(lib.bf_concretize(_lib.ptr(fin.A), _lib.ptr(tr.mid), _lib.ptr(tr.rad), _lib.ptr(fin.d), _lib.ptr(res), side, B, S,
                                     int(tr.mid.shape[1]), s))
        outs.append(res)
    return outs[0], outs[1], tr


def run_crown_ibp_dag(module: Any, input_spec: Any, *, linear_spec_C: Optional[torch.Tensor] = None,
                      output_value: Optional[str] = None) -> IntervalState:
    """`run_crown_ibp_mlp` (crown_ibp.py:2054-2133) for graphs with add / concat / fan-out."""
    lo, up, _tr = crown_dag(module, input_spec, linear_spec_C, output_value=output_value)
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
