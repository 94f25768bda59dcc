"""Executor-step boundary: `CudaTaskExecutor` and `CudaIntervalDomain`.

`CudaTaskExecutor` offers the two methods the reference's schedulers call on an
executor -- `run_ibp(module, input_spec, output_value=None)`
(runtime/task_executor.py:108-115, implemented by PythonTaskExecutor at 127-358
and TVMTaskExecutor runtime/tvm_executor.py:730-1034) and
`run_ibp_task(task, env=, params=, storage_plan=)` (runtime/scheduler.py:21-30,
PythonTaskExecutor 360-563) -- and `CudaIntervalDomain` the transformer methods
of `AbstractDomain` (domains/base.py:5-36, IntervalDomain domains/interval.py:27-114).
Affine and ReLU work runs in libbf_b200.so; pure data-movement ops (flatten,
reshape, permute, concat) stay views.  Unsupported ops raise NotImplementedError
exactly like the reference executors.
"""
from __future__ import annotations

from typing import Any, Dict, Optional

import torch

from . import _lib
from .crown import _cuda_device, _f32, _stream_ptr, ibp_trace, needs_graph_path
from .ir import IntervalState, input_mid_rad, lp_ball_of, normalize_input_spec
from .network import _pair, dense_conv_weight


def _is_interval_kind(kind: Any) -> bool:
    return getattr(kind, "value", kind) == "interval_ibp"


def _state_like(state_in: Any, lower: torch.Tensor, upper: torch.Tensor) -> Any:
    """Interval state of the same class as `state_in`, so that a caller which checks types with isinstance (the
    reference's PythonTaskExecutor does, task_executor.py:166-176) gets its own IntervalState back."""
    cls = type(state_in)
    if cls is not IntervalState:
        try:
            return cls(lower=lower, upper=upper)
        except TypeError:
            pass
    return IntervalState(lower=lower, upper=upper)


class CudaIntervalDomain:
    """Interval transformers on the device (centre/radius arithmetic).  Results have the class of the input state."""

    @property
    def domain_id(self) -> str:
        return "interval"

    def affine_transformer(self, state_in: Any, weight: Any, bias: Any, **attrs: Any) -> IntervalState:
        if not (hasattr(state_in, "lower") and hasattr(state_in, "upper")):
            raise TypeError(f"IntervalDomain expects IntervalState, got {type(state_in)}")
        lib = _lib.load()
        x_l, x_u = state_in.lower, state_in.upper
        device = _cuda_device(x_l)
        w = weight if torch.is_tensor(weight) else torch.as_tensor(weight)
        w = _f32(w, device)
        b = None
        if bias is not None:
            b = bias if torch.is_tensor(bias) else torch.as_tensor(bias)
            b = _f32(b, device)
        op = attrs.get("op")
        relu_in = 1 if attrs.get("relu_in", False) else 0
        xl, xu = _f32(x_l, device), _f32(x_u, device)
        B = int(xl.shape[0])
        if op == "conv2d" or (op is None and xl.dim() == 4 and w.dim() == 4):
            st, pd = _pair(attrs.get("stride", 1)), _pair(attrs.get("padding", 0))
            w = dense_conv_weight(w, attrs)   # grouped / dilated: the equal dense convolution
            Ci, Hi, Wi = (int(d) for d in xl.shape[1:])
            Co, _, kh, kw = (int(d) for d in w.shape)
            Ho = (Hi + 2 * pd[0] - kh) // st[0] + 1
            Wo = (Wi + 2 * pd[1] - kw) // st[1] + 1
            y_l = torch.empty(B, Co, Ho, Wo, dtype=torch.float32, device=device)
            y_u = torch.empty_like(y_l)
            _lib.check(lib.bf_ibp_conv2d(
                _lib.ptr(xl), _lib.ptr(xu), _lib.IN_LOWER_UPPER, relu_in, _lib.ptr(w), _lib.ptr(b), None, 0, None, None,
                _lib.ptr(y_l), _lib.ptr(y_u), None, B, Ci, Hi, Wi, Co, kh, kw, st[0], st[1], pd[0], pd[1], _stream_ptr(device)))
            return _state_like(state_in, y_l.to(x_l.device), y_u.to(x_l.device))
        if op not in (None, "linear"):
            raise NotImplementedError(f"unsupported affine op for IntervalDomain: {op}")
        if w.dim() == 3:
            # one weight matrix per batch element [B,S,I] (spec merged into the last layer, task_executor.py:231-245)
            S, n_in = int(w.shape[1]), int(w.shape[2])
            if xl.dim() != 2 or int(w.shape[0]) != B or int(xl.shape[1]) != n_in:
                raise ValueError(f"batched linear mismatch: x={tuple(xl.shape)} w={tuple(w.shape)}")
            if b is not None and tuple(b.shape) != (B, S):
                b = b.expand(B, S).contiguous()
            y_l = torch.empty(B, S, dtype=torch.float32, device=device)
            y_u = torch.empty_like(y_l)
            _lib.check(lib.bf_ibp_linear_batched(_lib.ptr(xl), _lib.ptr(xu), relu_in, _lib.ptr(w), _lib.ptr(b), _lib.ptr(y_l), _lib.ptr(y_u),
                                                 B, S, n_in, _stream_ptr(device)))
            return _state_like(state_in, y_l.to(x_l.device), y_u.to(x_l.device))
        lead = tuple(xl.shape[:-1])
        n_in, n_out = int(w.shape[1]), int(w.shape[0])
        x2l, x2u = xl.reshape(-1, n_in), xu.reshape(-1, n_in)
        rows = int(x2l.shape[0])
        y_l = torch.empty(rows, n_out, dtype=torch.float32, device=device)
        y_u = torch.empty_like(y_l)
        _lib.check(lib.bf_ibp_linear(
            _lib.ptr(x2l), _lib.ptr(x2u), _lib.IN_LOWER_UPPER, relu_in, _lib.ptr(w), _lib.ptr(b), None, 0, None, None,
            _lib.ptr(y_l), _lib.ptr(y_u), None, rows, n_in, n_out, _stream_ptr(device)))
        return _state_like(state_in, y_l.reshape(lead + (n_out,)).to(x_l.device), y_u.reshape(lead + (n_out,)).to(x_l.device))

    def relu_transformer(self, state_in: Any) -> IntervalState:
        if not (hasattr(state_in, "lower") and hasattr(state_in, "upper")):
            raise TypeError(f"IntervalDomain expects IntervalState, got {type(state_in)}")
        # In chains the clamp is fused into the consuming affine kernel (relu_in); stand-alone it is one elementwise kernel.
        lib = _lib.load()
        device = _cuda_device(state_in.lower)
        l, u = _f32(state_in.lower, device), _f32(state_in.upper, device)
        ol, ou = torch.empty_like(l), torch.empty_like(u)
        _lib.check(lib.bf_interval_relu(_lib.ptr(l), _lib.ptr(u), _lib.ptr(ol), _lib.ptr(ou), l.numel(), _stream_ptr(device)))
        return _state_like(state_in, ol.to(state_in.lower.device), ou.to(state_in.lower.device))

    def elementwise_transformer(self, states_in, op: str) -> IntervalState:
        if len(states_in) != 2:
            raise ValueError(f"elementwise '{op}' expects 2 inputs, got {len(states_in)}")
        a, b = states_in
        if op == "add":
            if tuple(a.lower.shape) != tuple(b.lower.shape):
                raise NotImplementedError("elementwise add supports exact same-shape inputs only")
            lib = _lib.load()
            device = _cuda_device(a.lower)
            al, au, bl, bu = (_f32(t, device) for t in (a.lower, a.upper, b.lower, b.upper))
            ol, ou = torch.empty_like(al), torch.empty_like(au)
            _lib.check(lib.bf_interval_add(_lib.ptr(al), _lib.ptr(au), _lib.ptr(bl), _lib.ptr(bu), _lib.ptr(ol), _lib.ptr(ou), al.numel(),
                                           _stream_ptr(device)))
            return _state_like(a, ol.to(a.lower.device), ou.to(a.lower.device))
        if op == "mul":  # corner products; operands broadcast like torch's `*` (domains/interval.py:102-112)
            lib = _lib.load()
            device = _cuda_device(a.lower)
            shape = torch.broadcast_shapes(tuple(a.lower.shape), tuple(b.lower.shape))
            al, au, bl, bu = (_f32(t, device).expand(shape).contiguous() for t in (a.lower, a.upper, b.lower, b.upper))
            ol, ou = torch.empty_like(al), torch.empty_like(au)
            _lib.check(lib.bf_interval_mul(_lib.ptr(al), _lib.ptr(au), _lib.ptr(bl), _lib.ptr(bu), _lib.ptr(ol), _lib.ptr(ou), al.numel(),
                                           _stream_ptr(device)))
            return _state_like(a, ol.to(a.lower.device), ou.to(a.lower.device))
        raise NotImplementedError(f"unsupported elementwise op: {op}")


class CudaTaskExecutor:
    """Drop-in for PythonTaskExecutor / TVMTaskExecutor on INTERVAL_IBP tasks."""

    def __init__(self, domain: Optional[CudaIntervalDomain] = None):
        self.domain = domain or CudaIntervalDomain()

    # ---- whole-module IBP -------------------------------------------------
    def run_ibp(self, module: Any, input_spec: Any, *, output_value: Optional[str] = None) -> IntervalState:
        module.validate()
        task = module.get_entry_task()
        if not _is_interval_kind(task.kind):
            raise NotImplementedError(f"CudaTaskExecutor only supports INTERVAL_IBP, got {task.kind}")
        spec = normalize_input_spec(input_spec)
        if spec.value_name not in task.input_values:
            raise ValueError(f"input_spec.value_name '{spec.value_name}' not in task.input_values: {task.input_values}")
        if output_value is None:
            if len(task.output_values) != 1:
                raise ValueError(f"task has {len(task.output_values)} outputs; specify output_value explicitly")
            output_value = task.output_values[0]
        params = module.bindings.get("params", {})
        last = task.ops[-1]
        w_last = params.get(last.inputs[1]) if (last.op_type == "linear" and len(last.inputs) >= 2 and isinstance(params, dict)) else None
        if torch.is_tensor(w_last) and w_last.dim() == 3:
            return self._run_ibp_spec_fused(module, task, spec, output_value)
        walkers = {"linear", "conv2d", "relu", "add", "concat", "flatten", "reshape"}
        if any(op.op_type not in walkers for op in task.ops):
            return self._run_ibp_generic(module, task, spec, output_value)
        if needs_graph_path(module):
            from .dag import run_ibp_dag

            return run_ibp_dag(module, spec, output_value=output_value)
        trace = ibp_trace(module, spec)
        chain = trace.chain
        dev = spec.center.device
        B = trace.B
        if output_value == chain.output_name:
            shape = (B,) + tuple(chain.output_shape)
            return IntervalState(lower=trace.out_l.reshape(shape).to(dev), upper=trace.out_u.reshape(shape).to(dev))
        for r, name in enumerate(chain.relu_input_names):
            shape = (B,) + tuple(chain.relu_shapes[r])
            if output_value == name:
                return IntervalState(lower=trace.pre_l[r].reshape(shape).to(dev), upper=trace.pre_u[r].reshape(shape).to(dev))
            if output_value == chain.layers[chain.relu_layer_ids[r]].out_name:
                return IntervalState(lower=trace.pre_l[r].reshape(shape).clamp_min(0).to(dev), upper=trace.pre_u[r].reshape(shape).clamp_min(0).to(dev))
        raise KeyError(f"missing value in env/params: {output_value}")

    def _run_ibp_spec_fused(self, module: Any, task: Any, spec: Any, output_value: str) -> IntervalState:
        """Module whose last Linear carries the merged output spec (weight [B,S,I], bias [B,S];
        planner/interval_v1.py:85-163): the layers below run as a chain, the last one as the batched-W kernel."""
        from .ir import BFTaskModule, BoundTask

        last = task.ops[-1]
        params = module.bindings["params"]
        if output_value != last.outputs[0]:
            raise KeyError(f"missing value in env/params: {output_value}")
        body = list(task.ops[:-1])
        relu_in = bool(body) and body[-1].op_type == "relu"
        if relu_in:
            body = body[:-1]
        w, b = params[last.inputs[1]], (params[last.inputs[2]] if len(last.inputs) == 3 else None)
        if not body:  # the fused layer reads the input set itself
            _mid, _rad, lo, up = input_mid_rad(spec)
            x = IntervalState(lower=lo.flatten(1), upper=up.flatten(1))
        else:
            sub_task = BoundTask(task_id=task.task_id, kind=task.kind, ops=body, input_values=list(task.input_values),
                                 output_values=[body[-1].outputs[0]])
            sub = BFTaskModule(tasks=[sub_task], entry_task_id=task.task_id, bindings=module.bindings)
            x = self.run_ibp(sub, spec)
            x = IntervalState(lower=x.lower.flatten(1), upper=x.upper.flatten(1))
        return self.domain.affine_transformer(x, w, b, op="linear", relu_in=relu_in)

    # ---- op-by-op interpretation over the domain ---------------------------
    def _interpret(self, ops, get_interval, put, get_tensor, linear_on_input=None) -> None:
        """The op loop of the reference's executors (task_executor.py:184-350) over `self.domain`: linear / conv2d
        (affine_transformer; a rank-3 weight is the batched form, 229-246), relu, add, mul, concat, flatten, reshape,
        permute / transpose and spec_linear (185-213).  `linear_on_input(op)` may return the result of a Linear op that
        reads the input set directly (an Lp ball needs its dual norms there), or None."""
        for op in ops:
            t = op.op_type
            if t in ("linear", "conv2d"):
                done = linear_on_input(op) if (t == "linear" and linear_on_input is not None) else None
                if done is not None:
                    put(op.outputs[0], done)
                    continue
                x = get_interval(op.inputs[0])
                w = get_tensor(op.inputs[1])
                b = get_tensor(op.inputs[2]) if len(op.inputs) == 3 else None
                attrs = dict(op.attrs)
                attrs["op"] = t
                put(op.outputs[0], self.domain.affine_transformer(x, w, b, **attrs))
            elif t == "spec_linear":
                x = get_interval(op.inputs[0])
                Cm = get_tensor(op.inputs[1])
                Cm = Cm if torch.is_tensor(Cm) else torch.as_tensor(Cm)
                if Cm.dim() != 3:
                    raise ValueError(f"spec_linear expects C rank-3 [B,S,O], got {tuple(Cm.shape)}")
                if x.lower.dim() != 2:
                    raise ValueError(f"spec_linear expects logits rank-2 [B,O], got {tuple(x.lower.shape)}")
                if Cm.shape[0] != x.lower.shape[0] or Cm.shape[2] != x.lower.shape[1]:
                    raise ValueError(f"spec_linear shape mismatch: C={tuple(Cm.shape)} logits={tuple(x.lower.shape)}")
                put(op.outputs[0], self.domain.affine_transformer(x, Cm, None, op="linear"))
            elif t == "relu":
                put(op.outputs[0], self.domain.relu_transformer(get_interval(op.inputs[0])))
            elif t == "add":
                a, b2 = get_interval(op.inputs[0]), get_interval(op.inputs[1])
                if tuple(a.lower.shape) != tuple(b2.lower.shape):
                    raise NotImplementedError("CudaTaskExecutor only supports add with exact same-shape inputs")
                put(op.outputs[0], self.domain.elementwise_transformer([a, b2], op="add"))
            elif t == "mul":
                put(op.outputs[0], self.domain.elementwise_transformer([get_interval(op.inputs[0]), get_interval(op.inputs[1])], op="mul"))
            elif t == "flatten":
                x = get_interval(op.inputs[0])
                sd, ed = int(op.attrs.get("start_dim", 0)), int(op.attrs.get("end_dim", -1))
                put(op.outputs[0], IntervalState(lower=torch.flatten(x.lower, sd, ed), upper=torch.flatten(x.upper, sd, ed)))
            elif t == "reshape":
                x = get_interval(op.inputs[0])
                shape = op.attrs.get("shape")
                put(op.outputs[0], x if shape is None else IntervalState(lower=x.lower.reshape(shape), upper=x.upper.reshape(shape)))
            elif t in ("permute", "transpose"):
                x = get_interval(op.inputs[0])
                dims = [int(d) for d in op.attrs.get("dims")]
                put(op.outputs[0], IntervalState(lower=x.lower.permute(*dims), upper=x.upper.permute(*dims)))
            elif t == "concat":
                parts = [get_interval(n) for n in op.inputs]
                axis = int(op.attrs.get("axis", 1))
                put(op.outputs[0], IntervalState(lower=torch.cat([p.lower for p in parts], dim=axis), upper=torch.cat([p.upper for p in parts], dim=axis)))
            else:
                raise NotImplementedError(f"unsupported op_type in task executor: {t}")

    def _run_ibp_generic(self, module: Any, task: Any, spec: Any, output_value: str) -> IntervalState:
        """Whole-module IBP for op lists outside the chain / graph walkers (mul, permute / transpose, spec_linear):
        every op through the domain's kernels, values kept in their own shapes."""
        params = module.bindings.get("params", {})
        ball = lp_ball_of(spec)
        device = _cuda_device(spec.center)
        if ball is not None:
            center = _f32(spec.center, device)
            lo, up = center - float(ball[1]), center + float(ball[1])   # the bounding box every non-Linear consumer sees
        else:
            _mid, _rad, lo, up = input_mid_rad(spec)
        env: Dict[str, IntervalState] = {spec.value_name: IntervalState(lower=_f32(lo, device), upper=_f32(up, device))}
        views = {spec.value_name}

        def get_interval(name: str) -> IntervalState:
            if name in env:
                return env[name]
            if name in params:
                t = params[name]
                t = _f32(t if torch.is_tensor(t) else torch.as_tensor(t), device)
                return IntervalState(lower=t, upper=t)
            raise KeyError(f"missing value in env/params: {name}")

        def get_tensor(name: str) -> Any:
            if name in params:
                return params[name]
            raise KeyError(f"missing param tensor: {name}")

        def put(name: str, st: IntervalState) -> None:
            env[name] = st

        def linear_on_input(op):
            if ball is None or op.inputs[0] not in views:
                return None
            lib = _lib.load()
            W = _f32(get_tensor(op.inputs[1]), device)
            if W.dim() != 2:
                return None
            b = _f32(get_tensor(op.inputs[2]), device) if len(op.inputs) == 3 else None
            c = _f32(spec.center, device).reshape(int(spec.center.shape[0]), -1).contiguous()
            n_out, n_in, Bc, s = int(W.shape[0]), int(W.shape[1]), int(c.shape[0]), _stream_ptr(device)
            row_dev = torch.empty(n_out, dtype=torch.float32, device=device)
            yl, yu = torch.empty(Bc, n_out, device=device), torch.empty(Bc, n_out, device=device)
            _lib.check(lib.bf_row_dual_norms(_lib.ptr(W), n_out, n_in, int(ball[0]), float(ball[1]), _lib.ptr(row_dev), s))
            _lib.check(lib.bf_ibp_linear_lp(_lib.ptr(c), _lib.ptr(row_dev), _lib.ptr(W), _lib.ptr(b), None, 0, None, None, _lib.ptr(yl), _lib.ptr(yu),
                                            None, Bc, n_in, n_out, s))
            return IntervalState(lower=yl, upper=yu)

        for op in task.ops:   # one op at a time so that flatten / reshape views of the input stay known
            self._interpret([op], get_interval, put, get_tensor, linear_on_input)
            if op.op_type in ("flatten", "reshape") and op.inputs[0] in views:
                views.add(op.outputs[0])
        if output_value not in env:
            raise KeyError(f"missing value in env/params: {output_value}")
        out = env[output_value]
        dev = spec.center.device
        return IntervalState(lower=out.lower.to(dev), upper=out.upper.to(dev))

    # ---- one task of a scheduled task graph -------------------------------
    def run_ibp_task(self, task: Any, *, env: Dict[str, IntervalState], params: Dict[str, Any], storage_plan: Any) -> None:
        if not _is_interval_kind(task.kind):
            raise NotImplementedError(f"CudaTaskExecutor only supports INTERVAL_IBP, got {task.kind}")

        def buf(value_name: str) -> str:
            logical = storage_plan.value_to_buffer.get(value_name)
            if logical is None:
                raise KeyError(f"value not found in storage_plan: {value_name}")
            return storage_plan.to_physical(logical)

        def get_interval(value_name: str) -> IntervalState:
            bid = buf(value_name)
            if bid in env:
                return env[bid]
            if value_name in params:
                t = params[value_name]
                t = t if torch.is_tensor(t) else torch.as_tensor(t)
                st = IntervalState(lower=t, upper=t)
                env[bid] = st
                return st
            raise KeyError(f"missing value in env/params: {value_name}")

        def get_tensor(value_name: str) -> Any:
            if value_name in params:
                return params[value_name]
            raise KeyError(f"missing param tensor: {value_name}")

        self._interpret(task.ops, get_interval, lambda name, st: env.__setitem__(buf(name), st), get_tensor)
