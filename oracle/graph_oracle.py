"""CPU restatement of the reference's bound propagation on single-task graphs that are not chains
(residual add, concat, fan-out).  TEST INFRASTRUCTURE ONLY: nothing in the product imports this file.

It follows `_forward_ibp_trace_mlp` (boundflow/runtime/crown_ibp.py:101-342) for the interval pass and the generic
backward sweep `_run_crown_backward_from_trace` (crown_ibp.py:1669-2051) for CROWN: one coefficient state per VALUE,
ops walked in reverse, `add` handing the same coefficients to both operands and its bias to the first dynamic one
(`_split_bias_once`, 922-937), `concat` slicing along the channel axis (1978-2030), a value with several consumers
summing what arrives (`_accumulate_backward_state`, 879-913).  The alpha / beta loop is the per-domain mode of
`run_alpha_beta_crown_mlp` (boundflow/runtime/alpha_beta_crown.py:716-923) with torch autograd through the sweep,
exactly as the reference does it.  Pinned by tests/golden/graph_cases.npz and tests/golden/graph_alpha.npz, both
generated from the reference.  The per-op arithmetic is shared with oracle/crown_oracle.py.
"""
from __future__ import annotations

from typing import Any, Dict, List, Mapping, Optional, Tuple

import torch
import torch.nn.functional as F

from . import crown_oracle as O


def _pair(v) -> Tuple[int, int]:
    if isinstance(v, (tuple, list)):
        return int(v[0]), int(v[1])
    return int(v), int(v)


def _task(module: Any):
    return module.get_entry_task()


def _params(module: Any, dtype) -> Dict[str, torch.Tensor]:
    return {k: torch.as_tensor(v).to(dtype) for k, v in module.bindings.get("params", {}).items()}


def _input_set(lo: torch.Tensor, up: torch.Tensor, ball):
    """The input set as the chain oracle's InputSet: the box [lo, up], or with ball = (p, eps) the L1 / L2 ball around the
    box's midpoint (lo / up are then its bounding box centre -/+ eps)."""
    B = lo.shape[0]
    if ball is None:
        return O.box_input(lo.reshape(B, -1), up.reshape(B, -1))
    return O.lp_ball(((lo + up) / 2.0).reshape(B, -1), float(ball[1]), int(ball[0]))


def forward_ibp_graph(module: Any, lo: torch.Tensor, up: torch.Tensor, *, input_name: str = "input", splits: Optional[Mapping[str, torch.Tensor]] = None,
                      ball=None, constraints: Optional[Mapping[str, Tuple[torch.Tensor, torch.Tensor]]] = None):
    """Interval pass.  Returns (env, relu_pre): name -> (lower, upper) in the value's own shape; relu_pre holds the
    bounds of every ReLU input AFTER its split (crown_ibp.py:210-214), env[x] stays unsplit.  With `ball` = (p, eps) a
    Linear op on the input value (or a flatten / reshape of it) uses the ball's dual row norms (perturbation.py:102-134),
    every other consumer the bounding box (crown_ibp.py:126-134, 173-175).  `constraints[x]` = (lower, upper) is
    intersected with the bounds of ReLU input x before its split (crown_ibp.py:186-209)."""
    dtype = lo.dtype
    P = _params(module, dtype)
    env: Dict[str, Tuple[torch.Tensor, torch.Tensor]] = {input_name: (lo, up)}
    views = {input_name}
    relu_pre: Dict[str, Tuple[torch.Tensor, torch.Tensor]] = {}
    B = lo.shape[0]

    def get(name):
        if name in env:
            return env[name]
        c = P[name]
        c = c.unsqueeze(0).expand((B,) + tuple(c.shape)) if c.dim() == 0 or c.shape[0] != B else c
        return (c, c)

    for op in _task(module).ops:
        t, out = op.op_type, op.outputs[0]
        if t == "linear":
            l, u = get(op.inputs[0])
            W = P[op.inputs[1]]
            b = P[op.inputs[2]] if len(op.inputs) == 3 else None
            if op.inputs[0] in views:
                env[out] = O.ibp_first_linear(_input_set(l, u, ball), W, b)
            else:
                env[out] = O.ibp_linear(l.reshape(B, -1), u.reshape(B, -1), W, b)
        elif t == "conv2d":
            l, u = get(op.inputs[0])
            W = P[op.inputs[1]]
            b = P[op.inputs[2]] if len(op.inputs) == 3 else None
            env[out] = O.ibp_conv2d(l, u, W, b, _pair(op.attrs.get("stride", 1)), _pair(op.attrs.get("padding", 0)),
                                    _pair(op.attrs.get("dilation", 1)), int(op.attrs.get("groups", 1)))
        elif t == "relu":
            x = op.inputs[0]
            l, u = get(x)
            if constraints is not None:
                cl, cu = constraints[x]
                l, u = torch.maximum(l, cl.reshape(l.shape)), torch.minimum(u, cu.reshape(u.shape))
                if bool((l > u).any()):
                    raise ValueError(f"infeasible ReLU pre-activation intersection for {x}")
            if splits is not None and x in splits and splits[x] is not None:
                l, u, _infeasible = O.apply_relu_split(l, u, splits[x])
            relu_pre[x] = (l, u)
            env[out] = (l.clamp(min=0), u.clamp(min=0))
        elif t == "add":
            (al, au), (bl, bu) = get(op.inputs[0]), get(op.inputs[1])
            env[out] = (al + bl, au + bu)
        elif t in ("flatten", "reshape"):
            l, u = get(op.inputs[0])
            shp = (B, -1) if t == "flatten" else (B,) + tuple(int(d) for d in op.attrs.get("shape", ()))[1:]
            env[out] = (l.reshape(shp), u.reshape(shp))
            if op.inputs[0] in views:
                views.add(out)
        elif t == "concat":
            ls, us = zip(*[get(n) for n in op.inputs])
            env[out] = (torch.cat(ls, dim=1), torch.cat(us, dim=1))
        elif t == "mul":  # IntervalDomain.elementwise_transformer("mul"), domains/interval.py:102-112
            (al, au), (bl, bu) = get(op.inputs[0]), get(op.inputs[1])
            cand = torch.stack([al * bl, al * bu, au * bl, au * bu], dim=0)
            env[out] = (cand.min(dim=0).values, cand.max(dim=0).values)
        elif t in ("permute", "transpose"):  # task_executor.py:334-346
            l, u = get(op.inputs[0])
            dims = [int(d) for d in op.attrs["dims"]]
            env[out] = (l.permute(*dims), u.permute(*dims))
        elif t == "spec_linear":  # y = C @ logits with C [B,S,O], task_executor.py:185-213
            l, u = get(op.inputs[0])
            Cm = P[op.inputs[1]]
            c_pos, c_neg = Cm.clamp(min=0.0), Cm.clamp(max=0.0)
            env[out] = ((c_pos * l.unsqueeze(1) + c_neg * u.unsqueeze(1)).sum(dim=-1), (c_pos * u.unsqueeze(1) + c_neg * l.unsqueeze(1)).sum(dim=-1))
        else:
            raise NotImplementedError(t)
    return env, relu_pre


def crown_backward_graph(module: Any, env, relu_pre, C, lo, up, *, input_name: str = "input", output_name: Optional[str] = None,
                         alpha: Optional[Mapping[str, torch.Tensor]] = None, add_l: Optional[Mapping[str, torch.Tensor]] = None, ball=None,
                         influence_out: Optional[Dict[str, torch.Tensor]] = None, add_u: Optional[Mapping[str, torch.Tensor]] = None):
    """Backward sweep for both sides and box concretisation.  C [B,S,n_out]; alpha / add_l: name of the ReLU input ->
    [B, n] (flattened).  Returns (lower, upper) [B,S]; differentiable in alpha and add_l."""
    task = _task(module)
    dtype = lo.dtype
    P = _params(module, dtype)
    B, S = C.shape[0], C.shape[1]
    out_name = output_name or task.output_values[0]
    shape = {n: tuple(v[0].shape[1:]) for n, v in env.items()}
    zero = torch.zeros(B, S, dtype=dtype)
    # state per value: [A_u, A_l, b_u, b_l], coefficients flattened to [B,S,n]
    adj: Dict[str, List[torch.Tensor]] = {out_name: [C, C, zero, zero]}

    def push(name, Au, Al, bu, bl):
        if name in adj:
            s = adj[name]
            adj[name] = [s[0] + Au, s[1] + Al, s[2] + bu, s[3] + bl]
        else:
            adj[name] = [Au, Al, bu, bl]

    for op in reversed(task.ops):
        out = op.outputs[0]
        st = adj.pop(out, None)
        if st is None:
            continue
        Au, Al, bu, bl = st
        t = op.op_type
        if t == "linear":
            W = P[op.inputs[1]]
            b = P[op.inputs[2]] if len(op.inputs) == 3 else None
            Au2, bu2 = O.linear_backward(Au, bu, W, b)
            Al2, bl2 = O.linear_backward(Al, bl, W, b)
            push(op.inputs[0], Au2, Al2, bu2, bl2)
        elif t == "conv2d":
            W = P[op.inputs[1]]
            b = P[op.inputs[2]] if len(op.inputs) == 3 else None
            st_, pd_ = _pair(op.attrs.get("stride", 1)), _pair(op.attrs.get("padding", 0))
            dg = (_pair(op.attrs.get("dilation", 1)), int(op.attrs.get("groups", 1)))
            Au2, bu2 = O.conv2d_backward(Au, bu, W, b, st_, pd_, shape[op.inputs[0]], shape[out], *dg)
            Al2, bl2 = O.conv2d_backward(Al, bl, W, b, st_, pd_, shape[op.inputs[0]], shape[out], *dg)
            push(op.inputs[0], Au2, Al2, bu2, bl2)
        elif t == "relu":
            x = op.inputs[0]
            l, u = relu_pre[x]
            if influence_out is not None:  # crown_ibp.py:1810-1834: the coefficients that arrive at the ReLU's output
                influence_out[x] = torch.maximum(Au.abs().amax(dim=1), Al.abs().amax(dim=1)).detach()
            a = alpha.get(x) if alpha is not None else None
            au_, bu_, al_, bl_ = O.relu_slopes(l, u, a)
            ad = add_l.get(x) if add_l is not None else None
            ad_u = add_u.get(x) if add_u is not None else None
            Au2, Al2, bu2, bl2 = O.relu_backward(Au, Al, bu, bl, au_, bu_, al_, bl_, add_u=ad_u, add_l=ad)
            push(x, Au2, Al2, bu2, bl2)
        elif t == "add":
            dyn = [n for n in op.inputs if n in env]
            for n in op.inputs:
                if n not in env:  # constant operand: A . value joins the bias (crown_ibp.py:1948-1950)
                    c = P[n].reshape(1, 1, -1)
                    bu, bl = bu + (Au * c).sum(dim=2), bl + (Al * c).sum(dim=2)
            for k, n in enumerate(dyn):
                push(n, Au, Al, bu if k == 0 else torch.zeros_like(bu), bl if k == 0 else torch.zeros_like(bl))
        elif t in ("flatten", "reshape"):
            push(op.inputs[0], Au, Al, bu, bl)
        elif t == "concat":
            start = 0
            for k, n in enumerate(op.inputs):
                w = 1
                for d in shape[n]:
                    w *= int(d)
                push(n, Au[:, :, start : start + w], Al[:, :, start : start + w], bu if k == 0 else torch.zeros_like(bu),
                     bl if k == 0 else torch.zeros_like(bl))
                start += w
        else:
            raise NotImplementedError(t)
    Au, Al, bu, bl = adj[input_name]
    inp = _input_set(lo, up, ball)
    return O.concretize(inp, Al, bl, "lower"), O.concretize(inp, Au, bu, "upper")


def adaptive_alpha_init_graph(relu_pre) -> Dict[str, torch.Tensor]:
    """alpha start 1 where l >= 0 or (l < 0 < u and u > -l), else 0 (native_alpha_beta_optimizer_schedule.py:644-656)."""
    out = {}
    for x, (l, u) in relu_pre.items():
        B = l.shape[0]
        lf, uf = l.reshape(B, -1), u.reshape(B, -1)
        out[x] = ((lf >= 0) | ((lf < 0) & (uf > 0) & (uf > -lf))).to(l.dtype)
    return out


def alpha_crown_graph(module: Any, lo, up, C, *, steps: int, lr: float, alpha0: Optional[Mapping[str, torch.Tensor]] = None,
                      alpha_init: float = 0.5, splits: Optional[Mapping[str, torch.Tensor]] = None, optimize_beta: bool = False,
                      input_name: str = "input", objective: str = "lower", spec_reduce: str = "mean", soft_tau: float = 1.0,
                      lb_weight: float = 1.0, ub_weight: float = 1.0, per_batch_params: bool = True, ball=None):
    """alpha (and beta) loop on a graph: `run_alpha_beta_crown_mlp`, alpha_beta_crown.py:716-923, with per-domain
    parameters and best-of (`per_batch_params=True`) or one parameter row for the batch and a whole-batch best-of on
    the mean of the per-domain objectives (False; `run_alpha_crown_mlp`, alpha_crown.py:137-261, is this mode without
    beta).  Objectives lower | upper | gap | both (807-818), reductions mean | sum | min | softmin over the spec rows
    (787-805; max / softmax on the upper side); beta enters the lower objective only (763-785).
    Returns (best_lower, best_upper, best_alpha dict, best_beta dict)."""
    env, relu_pre = forward_ibp_graph(module, lo, up, input_name=input_name, splits=splits, ball=ball)
    B, dtype = lo.shape[0], lo.dtype
    names = list(relu_pre)
    rows = B if per_batch_params else 1
    use_beta = bool(optimize_beta and objective == "lower")
    alphas, betas, split_f = {}, {}, {}
    for x in names:
        n = relu_pre[x][0].reshape(B, -1).shape[1]
        a = (alpha0[x].reshape(-1, n).expand(rows, n).to(dtype).clone() if alpha0 is not None and x in alpha0
             else torch.full((rows, n), float(alpha_init), dtype=dtype))
        alphas[x] = a.requires_grad_(True)
        if use_beta:
            betas[x] = torch.zeros(rows, n, dtype=dtype, requires_grad=True)
            sp = splits.get(x) if splits is not None else None
            split_f[x] = None if sp is None else sp.reshape(-1, n).expand(B, n).to(dtype)
    opt = torch.optim.Adam(list(alphas.values()) + list(betas.values()), lr=float(lr))

    def reduce(x, direction):
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

    best = None
    for step in range(int(steps) + 1):
        add_l = None
        if use_beta:
            add_l = {x: (-betas[x] * split_f[x]) for x in names if split_f[x] is not None}
        a_rows = {x: a.expand(B, -1) for x, a in alphas.items()}
        lower, upper = crown_backward_graph(module, env, relu_pre, C, lo, up, input_name=input_name, alpha=a_rows, add_l=add_l, ball=ball)
        if objective == "lower":
            metric_b = reduce(lower, "min")
        elif objective == "upper":
            metric_b = -reduce(upper, "max")
        elif objective == "gap":
            metric_b = -reduce(upper - lower, "max")
        elif objective == "both":
            metric_b = float(lb_weight) * reduce(lower, "min") - float(ub_weight) * reduce(upper, "max")
        else:
            raise ValueError(objective)
        snap = lambda d: {x: t.detach().clone() for x, t in d.items()}  # noqa: E731
        if per_batch_params:
            m = metric_b.detach()
            if best is None:
                best = [m.clone(), lower.detach().clone(), upper.detach().clone(), snap(alphas), snap(betas)]
            else:
                imp = m > best[0]
                best[0] = torch.where(imp, m, best[0])
                best[1] = torch.where(imp.unsqueeze(1), lower.detach(), best[1])
                best[2] = torch.where(imp.unsqueeze(1), upper.detach(), best[2])
                best[3] = {x: torch.where(imp.unsqueeze(1), a.detach(), best[3][x]) for x, a in alphas.items()}
                best[4] = {x: torch.where(imp.unsqueeze(1), b.detach(), best[4][x]) for x, b in betas.items()}
            loss = -metric_b.sum()
        else:
            metric = metric_b.mean()
            if best is None or float(metric.detach()) > best[0]:
                best = [float(metric.detach()), lower.detach().clone(), upper.detach().clone(), snap(alphas), snap(betas)]
            loss = -metric
        if step == int(steps):
            break
        if not loss.requires_grad:
            break
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        with torch.no_grad():
            for a in alphas.values():
                a.clamp_(0.0, 1.0)
            for b in betas.values():
                b.clamp_(0.0)
    return best[1], best[2], best[3], best[4]


def concrete_forward_graph(module: Any, x: torch.Tensor, *, input_name: str = "input", record_pre: bool = False):
    """Plain forward pass of the graph at concrete points x (any dtype / device); with `record_pre` also returns the
    inputs of every ReLU (name -> tensor), which the soundness tests use to keep the samples that satisfy a split."""
    P = {k: torch.as_tensor(v).to(dtype=x.dtype, device=x.device) for k, v in module.bindings.get("params", {}).items()}
    env = {input_name: x}
    pre = {}
    B = x.shape[0]
    get = lambda n: env[n] if n in env else P[n]  # noqa: E731
    for op in _task(module).ops:
        t, out = op.op_type, op.outputs[0]
        if t == "linear":
            y = get(op.inputs[0]).reshape(B, -1).matmul(P[op.inputs[1]].t())
            env[out] = y + P[op.inputs[2]] if len(op.inputs) == 3 else y
        elif t == "conv2d":
            b = P[op.inputs[2]] if len(op.inputs) == 3 else None
            env[out] = F.conv2d(get(op.inputs[0]), P[op.inputs[1]], b, _pair(op.attrs.get("stride", 1)), _pair(op.attrs.get("padding", 0)),
                                _pair(op.attrs.get("dilation", 1)), int(op.attrs.get("groups", 1)))
        elif t == "relu":
            pre[op.inputs[0]] = get(op.inputs[0])
            env[out] = torch.relu(get(op.inputs[0]))
        elif t == "add":
            env[out] = get(op.inputs[0]) + get(op.inputs[1])
        elif t in ("flatten", "reshape"):
            v = get(op.inputs[0])
            env[out] = v.reshape(B, -1) if t == "flatten" else v.reshape((B,) + tuple(int(d) for d in op.attrs.get("shape", ()))[1:])
        elif t == "concat":
            env[out] = torch.cat([get(n) for n in op.inputs], dim=1)
        else:
            raise NotImplementedError(t)
    y = env[_task(module).output_values[0]]
    return (y, pre) if record_pre else y
