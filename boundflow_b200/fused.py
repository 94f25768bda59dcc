"""Fused ReLU -> affine backward region executor (`FusedCrownExecutor` protocol).

Implements `supports_descriptor`, `supports` and `run(request, stream=)` of the
reference's fused-region contract (runtime/fused_crown.py:97-123) over
bf_crown_relu_linear_bwd / bf_crown_relu_conv2d_bwd, with the same legality
rules as the reference's compiled executors (`_plain_static_cuda_fp32`,
fused_crown.py:279-304): plain CROWN only, contiguous fp32 CUDA tensors without
grad.  Returning False from `supports*` makes the reference runtime fall back to
its eager step, exactly as for its own TVM executor.  Unlike the TVM v1 kernels
(backends/tvm/fused_crown_conv2d.py:75-84) any kernel size / stride / padding is
accepted for conv2d; groups and dilation run as the equal dense convolution
(`network.dense_conv_weight`).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

import torch

from . import _lib
from .network import _pair, dense_conv_weight


@dataclass(frozen=True)
class FusedReluAffineRequest:
    kind: str
    A_u: torch.Tensor
    A_l: torch.Tensor
    alpha_u: torch.Tensor
    alpha_l: torch.Tensor
    beta_u: torch.Tensor
    beta_l: torch.Tensor
    weight: torch.Tensor
    bias: Optional[torch.Tensor]
    input_shape: Tuple[int, ...]
    output_shape: Tuple[int, ...]
    attrs: Mapping[str, object]


@dataclass(frozen=True)
class FusedReluAffineResult:
    A_prev_u: torch.Tensor
    A_prev_l: torch.Tensor
    bias_delta_u: torch.Tensor
    bias_delta_l: torch.Tensor


def _context_ok(context: Any) -> bool:
    return bool(
        getattr(context, "plain_crown", True)
        and not getattr(context, "requires_grad", False)
        and not getattr(context, "alpha_enabled", False)
        and not getattr(context, "beta_enabled", False)
        and not getattr(context, "split_state_present", False)
    )


class CudaFusedCrownExecutor:
    backend = "b200_cuda"

    def __init__(self) -> None:
        self.lib = _lib.load()

    def supports_descriptor(self, descriptor: Any, context: Any) -> bool:
        if not _context_ok(context) or descriptor.kind not in ("linear", "conv2d"):
            return False
        dev = getattr(descriptor, "device", None)
        if dev is not None and torch.device(dev).type != "cuda":
            return False
        if getattr(descriptor, "dtype", torch.float32) != torch.float32:
            return False
        return True

    def supports(self, request: Any, context: Any) -> bool:
        if not _context_ok(context) or request.kind not in ("linear", "conv2d"):
            return False
        tensors = [request.A_u, request.A_l, request.alpha_u, request.alpha_l, request.beta_u, request.beta_l, request.weight]
        if request.bias is not None:
            tensors.append(request.bias)
        ok = all(t.device.type == "cuda" and t.dtype == torch.float32 and t.is_contiguous() and not t.requires_grad for t in tensors)
        return bool(ok)

    def run(self, request: Any, *, stream: Optional[torch.cuda.Stream] = None) -> FusedReluAffineResult:
        device = request.A_u.device
        if device.type != "cuda":
            raise RuntimeError("CudaFusedCrownExecutor needs CUDA tensors")
        st = stream if stream is not None else torch.cuda.current_stream(device)
        sp = st.cuda_stream
        D, S = int(request.A_u.shape[0]), int(request.A_u.shape[1])
        n_prev = 1
        for d in request.input_shape:
            n_prev *= int(d)
        with torch.cuda.stream(st):
            outs = []
            for side, A in ((_lib.SIDE_UPPER, request.A_u), (_lib.SIDE_LOWER, request.A_l)):
                A_prev = torch.empty((D, S) + tuple(request.input_shape), dtype=torch.float32, device=device)
                delta = torch.empty(D, S, dtype=torch.float32, device=device)
                if request.kind == "linear":
                    n_cur = int(request.weight.shape[0])
                    # large regions run the tcgen05 kernel on a packed copy of the weight (cached per weight tensor)
                    pack = _lib.LINEAR_PACKS.get(request.weight, D * S, sp)
                    _lib.check(self.lib.bf_crown_relu_linear_bwd_packed(
                        _lib.ptr(A), side, _lib.ptr(request.alpha_u), _lib.ptr(request.alpha_l), _lib.ptr(request.beta_u),
                        _lib.ptr(request.beta_l), None, _lib.ptr(request.weight), _lib.ptr(request.bias), _lib.ptr(pack),
                        _lib.ptr(A_prev), _lib.ptr(delta), 0, D, S, n_cur, n_prev, sp))
                else:
                    Co, Ho, Wo = (int(d) for d in request.output_shape)
                    Ci, Hi, Wi = (int(d) for d in request.input_shape)
                    weight = dense_conv_weight(request.weight, request.attrs)   # grouped / dilated: the equal dense convolution
                    kh, kw = int(weight.shape[2]), int(weight.shape[3])
                    sh, sw = _pair(request.attrs.get("stride", 1))
                    ph, pw = _pair(request.attrs.get("padding", 0))
                    nbytes = int(self.lib.bf_crown_relu_conv2d_bwd_scratch_bytes(D, S, Co, Ho, Wo))
                    scratch = torch.empty(nbytes, dtype=torch.uint8, device=device)
                    _lib.check(self.lib.bf_crown_relu_conv2d_bwd(
                        _lib.ptr(A), side, _lib.ptr(request.alpha_u), _lib.ptr(request.alpha_l), _lib.ptr(request.beta_u),
                        _lib.ptr(request.beta_l), _lib.ptr(weight), _lib.ptr(request.bias), _lib.ptr(A_prev),
                        _lib.ptr(delta), 0, _lib.ptr(scratch), nbytes, D, S, Ci, Hi, Wi, Co, Ho, Wo, kh, kw, sh, sw, ph, pw, sp))
                outs.append((A_prev, delta))
        return FusedReluAffineResult(A_prev_u=outs[0][0], A_prev_l=outs[1][0], bias_delta_u=outs[0][1], bias_delta_l=outs[1][1])
