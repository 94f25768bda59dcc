"""Chain compilation: a single-task `BFTaskModule` -> device-resident layer list.

The reference interprets `task.ops` op by op on every call
(runtime/crown_ibp.py:146-336, runtime/task_executor.py:184-350).  Here the op
list is validated once, its parameters are made contiguous fp32 device tensors
and handed to the C library as a `bf_chain`; every later call only passes
pointers.  Supported ops are the ones the bound-propagation configurations use:
linear, conv2d, relu, flatten(start_dim=1); anything else raises NotImplementedError
like the reference executors do for unknown ops.  A grouped or dilated Conv2d is handed
to the kernels as the equal dense convolution (`dense_conv_weight`).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

from . import _lib


def _pair(v: Any) -> Tuple[int, int]:
    if isinstance(v, int):
        return (int(v), int(v))
    v = tuple(int(x) for x in v)
    return (v[0], v[0]) if len(v) == 1 else (v[0], v[1])


class _DenseConvWeights:
    """Dense equivalents of grouped / dilated Conv2d weights, one per (weight tensor, groups, dilation).  Keyed by
    storage address, shape, device, in-place version counter and the two attributes; an entry keeps the original
    tensor alive so its address cannot be reused while the entry exists; least recently used entries are dropped."""

    def __init__(self, capacity: int = 32):
        self.capacity = int(capacity)
        self._entries: Dict[Tuple, Tuple[torch.Tensor, torch.Tensor]] = {}

    def get(self, W: torch.Tensor, groups: int, dilation: Tuple[int, int]) -> torch.Tensor:
        key = (W.data_ptr(), tuple(W.shape), str(W.device), int(W._version), int(groups), tuple(dilation))
        hit = self._entries.pop(key, None)
        if hit is None:
            Co, Cig, kh, kw = (int(d) for d in W.shape)
            if Co % groups != 0:
                raise ValueError(f"conv2d: {Co} output channels are not divisible by groups={groups}")
            cog, (dh, dw) = Co // groups, dilation
            dense = torch.zeros(Co, Cig * groups, dh * (kh - 1) + 1, dw * (kw - 1) + 1, dtype=W.dtype, device=W.device)
            for g in range(groups):
                dense[g * cog:(g + 1) * cog, g * Cig:(g + 1) * Cig, ::dh, ::dw] = W[g * cog:(g + 1) * cog]
            hit = (W, dense.contiguous())
            while len(self._entries) >= self.capacity:
                self._entries.pop(next(iter(self._entries)))
        self._entries[key] = hit  # most recently used last
        return hit[1]


_DENSE_CONV = _DenseConvWeights()


def dense_conv_weight(W: torch.Tensor, attrs: Any) -> torch.Tensor:
    """The weight of the dense, undilated convolution that equals conv2d(x, W, groups=g, dilation=d): output channel
    block k sees only input channel block k (zeros elsewhere) and the taps sit d apart in a kernel of d*(k-1)+1 (zeros
    between them).  Products with the inserted zeros add exact zeros, so every kernel of the library applies unchanged
    (`F.conv2d(..., dilation, groups)` in the reference: domains/interval.py:57-74, crown_ibp.py:1127-1170).  Returns W
    itself for groups = 1, dilation = 1."""
    attrs = attrs or {}
    groups, dilation = int(attrs.get("groups", 1)), _pair(attrs.get("dilation", 1))
    if groups == 1 and dilation == (1, 1):
        return W
    if groups < 1 or dilation[0] < 1 or dilation[1] < 1 or W.dim() != 4:
        raise ValueError(f"conv2d: bad groups={groups} / dilation={dilation} for a weight of shape {tuple(W.shape)}")
    return _DENSE_CONV.get(W, groups, dilation)


@dataclass
class ChainLayer:
    op: str
    name: str
    in_name: str
    out_name: str
    in_shape: Tuple[int, ...]
    out_shape: Tuple[int, ...]
    W: Optional[torch.Tensor] = None
    b: Optional[torch.Tensor] = None
    stride: Tuple[int, int] = (1, 1)
    padding: Tuple[int, int] = (0, 0)


def _numel(shape: Sequence[int]) -> int:
    n = 1
    for d in shape:
        n *= int(d)
    return n


class CudaChain:
    """Validated chain with device parameters and its `bf_chain` handle."""

    def __init__(self, module: Any, input_shape: Sequence[int], device: torch.device, *, input_name: Optional[str] = None):
        self.lib = _lib.load()
        self._module = module  # pins the module so that its id() stays unique while cached
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("the B200 backend needs a CUDA device; there is no CPU path")
        task = module.get_entry_task()
        if getattr(module, "task_graph", None) is not None or len(module.tasks) != 1:
            raise NotImplementedError("chain compilation supports single-task modules only")
        raw = module.bindings.get("params", {})
        params: Dict[str, Any] = dict(raw) if isinstance(raw, dict) else {}
        self.input_name = input_name or task.input_values[0]
        self.output_name = task.output_values[0]
        self.input_shape = tuple(int(d) for d in input_shape)

        def dev(t: Any) -> torch.Tensor:
            if not torch.is_tensor(t):
                t = torch.as_tensor(t)
            return t.detach().to(device=self.device, dtype=torch.float32).contiguous()

        layers: List[ChainLayer] = []
        shape = self.input_shape
        cur = self.input_name
        for op in task.ops:
            if len(op.outputs) != 1 or op.inputs[0] != cur:
                raise NotImplementedError(f"op '{op.name}' does not continue the chain at value '{cur}'")
            t = op.op_type
            if t == "linear":
                W = dev(params[op.inputs[1]])
                b = dev(params[op.inputs[2]]) if len(op.inputs) == 3 else None
                if W.dim() != 2 or len(shape) != 1 or W.shape[1] != shape[0]:
                    raise ValueError(f"linear '{op.name}': weight {tuple(W.shape)} does not match input shape {shape}")
                out_shape = (int(W.shape[0]),)
                layers.append(ChainLayer("linear", op.name, cur, op.outputs[0], shape, out_shape, W, b))
            elif t == "conv2d":
                W = dense_conv_weight(dev(params[op.inputs[1]]), op.attrs)
                b = dev(params[op.inputs[2]]) if len(op.inputs) == 3 else None
                st, pd = _pair(op.attrs.get("stride", 1)), _pair(op.attrs.get("padding", 0))
                if len(shape) != 3 or W.dim() != 4 or W.shape[1] != shape[0]:
                    raise ValueError(f"conv2d '{op.name}': weight {tuple(W.shape)} does not match input shape {shape}")
                ho = (shape[1] + 2 * pd[0] - W.shape[2]) // st[0] + 1
                wo = (shape[2] + 2 * pd[1] - W.shape[3]) // st[1] + 1
                out_shape = (int(W.shape[0]), int(ho), int(wo))
                layers.append(ChainLayer("conv2d", op.name, cur, op.outputs[0], shape, out_shape, W, b, st, pd))
            elif t == "relu":
                layers.append(ChainLayer("relu", op.name, cur, op.outputs[0], shape, shape))
                out_shape = shape
            elif t in ("flatten", "reshape"):
                if t == "flatten" and (int(op.attrs.get("start_dim", 1)) != 1 or int(op.attrs.get("end_dim", -1)) != -1):
                    raise NotImplementedError("only flatten(start_dim=1, end_dim=-1) is supported")
                out_shape = (_numel(shape),)
                if t == "reshape":
                    tgt = tuple(int(d) for d in op.attrs.get("shape", ()))
                    if len(tgt) < 2 or _numel(tgt[1:]) != _numel(shape):
                        raise NotImplementedError("reshape must keep the batch axis and the element count")
                    out_shape = tgt[1:]
                layers.append(ChainLayer("flatten", op.name, cur, op.outputs[0], shape, out_shape))
            else:
                raise NotImplementedError(f"unsupported op_type in the CUDA chain backend: {t}")
            cur = op.outputs[0]
            shape = out_shape
        self.layers = layers
        self.output_shape = shape
        self.relu_layer_ids = [i for i, l in enumerate(layers) if l.op == "relu"]
        self.relu_input_names = [layers[i].in_name for i in self.relu_layer_ids]
        self.relu_shapes = [layers[i].in_shape for i in self.relu_layer_ids]
        self.relu_widths = [_numel(s) for s in self.relu_shapes]
        self.n0 = _numel(self.input_shape)
        self.value_shapes: Dict[str, Tuple[int, ...]] = {self.input_name: self.input_shape}
        for l in layers:
            self.value_shapes[l.out_name] = l.out_shape
        self.max_width = max([self.n0] + [_numel(l.out_shape) for l in layers])

        descs = (_lib.LayerDesc * len(layers))()
        opmap = {"linear": _lib.OP_LINEAR, "conv2d": _lib.OP_CONV2D, "relu": _lib.OP_RELU, "flatten": _lib.OP_FLATTEN}
        for k, l in enumerate(layers):
            d = descs[k]
            d.op = opmap[l.op]
            d.W = l.W.data_ptr() if l.W is not None else None
            d.bias = l.b.data_ptr() if l.b is not None else None
            d.n_in, d.n_out = _numel(l.in_shape), _numel(l.out_shape)
            if l.op == "conv2d":
                d.Ci, d.Hi, d.Wi = l.in_shape
                d.Co, d.Ho, d.Wo = l.out_shape
                d.kh, d.kw = int(l.W.shape[2]), int(l.W.shape[3])
                d.sh, d.sw = l.stride
                d.ph, d.pw = l.padding
        handle = C.c_void_p()
        _lib.check(self.lib.bf_chain_create(descs, len(layers), C.byref(handle)))
        self.handle = handle
        # tensor-core path: split + pack the static weights once (buffer owned here, freed with the chain)
        nbytes = int(self.lib.bf_chain_tc_bytes(handle))
        self._tc_buffer = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        _lib.check(self.lib.bf_chain_tc_prepare(handle, self._tc_buffer.data_ptr(), nbytes, torch.cuda.current_stream(self.device).cuda_stream))

    def tc_status(self) -> int:
        """Synchronous read of the tensor-core kernels' status word (non-zero: a bounded wait expired)."""
        st = C.c_int(0)
        _lib.check(self.lib.bf_chain_tc_status(self.handle, C.byref(st)))
        return int(st.value)

    def __del__(self):
        h = getattr(self, "handle", None)
        if h:
            try:
                self.lib.bf_chain_destroy(h)
            except Exception:
                pass
            self.handle = None

    # layer count that produces `value_name` (for intermediate-value bounds)
    def layers_upto(self, value_name: Optional[str]) -> int:
        if value_name is None or value_name == self.output_name:
            return len(self.layers)
        for k, l in enumerate(self.layers):
            if l.out_name == value_name:
                return k + 1
        raise KeyError(f"value '{value_name}' is not produced by this chain")

    @property
    def is_linear_relu_chain(self) -> bool:
        ops = [l.op for l in self.layers]
        return len(ops) % 2 == 1 and all(o == ("linear" if k % 2 == 0 else "relu") for k, o in enumerate(ops))


_CHAIN_CACHE: Dict[Tuple, CudaChain] = {}


def compile_chain(module: Any, input_shape: Sequence[int], device: torch.device) -> CudaChain:
    """Cached by module identity, parameter storage and device (a module whose
    parameter tensors are replaced gets a fresh chain)."""
    raw = module.bindings.get("params", {})
    key = (
        id(module),
        tuple(int(d) for d in input_shape),
        str(device),
        tuple((k, v.data_ptr() if torch.is_tensor(v) else id(v)) for k, v in raw.items()) if isinstance(raw, dict) else (),
    )
    chain = _CHAIN_CACHE.get(key)
    if chain is None:
        if len(_CHAIN_CACHE) > 64:
            _CHAIN_CACHE.clear()
        chain = CudaChain(module, input_shape, device)
        _CHAIN_CACHE[key] = chain
    return chain
