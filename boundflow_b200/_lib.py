"""ctypes binding of libbf_b200.so (the C ABI declared in include/bf_b200.h).

There is no fallback: if the shared library is missing the import of any
compute entry point raises, and every non-zero return code becomes a Python
exception carrying bf_last_error_string().
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional, Sequence

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libbf_b200.so")

BF_OK = 0
BF_E_INVALID, BF_E_UNSUPPORTED, BF_E_WORKSPACE, BF_E_CUDA = -1, -2, -3, -4
SIDE_LOWER, SIDE_UPPER = 0, 1
IN_LOWER_UPPER, IN_MID_RAD, IN_CENTER_DEV = 0, 1, 2
NORM_BOX, NORM_L1, NORM_L2, NORM_INF = 0, 1, 2, 3
OP_LINEAR, OP_CONV2D, OP_RELU, OP_FLATTEN = 1, 2, 3, 4
REDUCE_MEAN, REDUCE_SUM, REDUCE_MIN, REDUCE_SOFTMIN = 0, 1, 2, 3
OBJECTIVE_GAP, OBJECTIVE_BOTH = 2, 3

_p = C.c_void_p
_i = C.c_int
_f = C.c_float
_sz = C.c_size_t


class LayerDesc(C.Structure):
    _fields_ = [("op", _i), ("W", _p), ("bias", _p), ("n_in", _i), ("n_out", _i)] + [
        (k, _i) for k in ("Ci", "Hi", "Wi", "Co", "Ho", "Wo", "kh", "kw", "sh", "sw", "ph", "pw")
    ]


# name -> (restype, argtypes); mirrors include/bf_b200.h one to one
SIGNATURES = {
    "bf_version": (_i, []),
    "bf_last_error_string": (C.c_char_p, []),
    "bf_launch_count": (C.c_ulonglong, []),
    "bf_tc_launch_count": (C.c_ulonglong, []),
    "bf_kernel_timing_enable": (None, [_i]),
    "bf_kernel_timing_read": (_i, [_i, C.POINTER(_i), C.POINTER(_f)]),
    "bf_kernel_timing_slots": (_i, []),
    "bf_kernel_timing_slot_name": (C.c_char_p, [_i]),
    "bf_kernel_timing_read_work": (_i, [_i, C.POINTER(_i), C.POINTER(_f), C.POINTER(C.c_double), C.POINTER(C.c_double)]),
    "bf_ibp_linear": (_i, [_p, _p, _i, _i, _p, _p, _p, _i, _p, _p, _p, _p, _p, _i, _i, _i, _p]),
    "bf_ibp_conv2d": (_i, [_p, _p, _i, _i, _p, _p, _p, _i, _p, _p, _p, _p, _p] + [_i] * 11 + [_p]),
    "bf_relu_relax": (_i, [_p, _p, _p, _i, _p, _p, _p, _i, _i, _p]),
    "bf_alpha_adaptive_init": (_i, [_p, _p, _p, _i, _i, _p]),
    "bf_crown_relu_linear_bwd": (_i, [_p, _i, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _p]),
    "bf_linear_pack_bytes": (_sz, [_i, _i]),
    "bf_linear_pack": (_i, [_p, _i, _i, _p, _sz, _p]),
    "bf_linear_pack_status": (_i, [_p, C.POINTER(_i)]),
    "bf_crown_relu_linear_bwd_packed": (_i, [_p, _i, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _p]),
    "bf_crown_relu_conv2d_bwd_scratch_bytes": (_sz, [_i] * 5),
    "bf_crown_relu_conv2d_bwd": (_i, [_p, _i, _p, _p, _p, _p, _p, _p, _p, _p, _i, _p, _sz] + [_i] * 14 + [_p]),
    "bf_crown_relu_conv2d_bwd_noalloc_max_bytes": (_sz, []),
    "bf_crown_relu_conv2d_bwd_noalloc": (_i, [_p, _i, _p, _p, _p, _p, _p, _p, _p, _p, _i] + [_i] * 14 + [_p]),
    "bf_concretize": (_i, [_p, _p, _p, _p, _p, _i, _i, _i, _i, _p]),
    "bf_verdict": (_i, [_p, _f, _f, _p, _p, _i, _i, _p]),
    "bf_verdict_masked": (_i, [_p, _f, _f, _p, _p, _p, _i, _i, _p]),
    "bf_chain_create": (_i, [C.POINTER(LayerDesc), _i, C.POINTER(_p)]),
    "bf_chain_destroy": (None, [_p]),
    "bf_chain_num_relu": (_i, [_p]),
    "bf_chain_tc_bytes": (_sz, [_p]),
    "bf_chain_tc_prepare": (_i, [_p, _p, _sz, _p]),
    "bf_chain_tc_status": (_i, [_p, C.POINTER(_i)]),
    "bf_chain_ibp": (_i, [_p, _p, _p, _i, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _sz, _i, _p]),
    "bf_chain_crown_workspace_bytes": (_sz, [_p, _i, _i, _i]),
    "bf_crown_relu_bwd_scratch_bytes": (_sz, [_i, _i, _i]),
    "bf_crown_relu_bwd": (_i, [_p, _i, _p, _p, _p, _p, _p, _p, _i, _p, _sz, _i, _i, _i, _p]),
    "bf_accumulate": (_i, [_p, _p, C.c_longlong, _p]),
    "bf_interval_relu": (_i, [_p, _p, _p, _p, C.c_longlong, _p]),
    "bf_interval_add": (_i, [_p, _p, _p, _p, _p, _p, C.c_longlong, _p]),
    "bf_interval_mul": (_i, [_p, _p, _p, _p, _p, _p, C.c_longlong, _p]),
    "bf_first_layer_certificate_max_halfspaces": (_i, []),
    "bf_first_layer_certificate": (_i, [_p, _i, _p, _p, _p, _p, _p, _p, _p, _i, _f, _f, _i, _i, _i, _p]),
    "bf_first_layer_certificate_lp": (_i, [_p, _i, _p, _p, _p, _f, _i, _p, _p, _p, _i, _f, _f, _i, _i, _i, _p]),
    "bf_ibp_linear_batched": (_i, [_p, _p, _i, _p, _p, _p, _p, _i, _i, _i, _p]),
    "bf_chain_crown": (_i, [_p, _i, _i, _p, _p, _p, _p, _p, _p, _p, _i, _f, _p, _p, _sz, _i, _i, _p]),
    "bf_chain_crown_influence": (_i, [_p, _i, _i, _p, _p, _p, _p, _p, _p, _p, _i, _f, _p, _p, _p, _sz, _i, _i, _p]),
    "bf_chain_crown_onehot": (_i, [_p, _i, _i, _i, _p, _p, _p, _p, _p, _p, _i, _f, _p, _p, _sz, _i, _i, _p]),
    "bf_row_dual_norms": (_i, [_p, _i, _i, _i, _f, _p, _p]),
    "bf_ibp_linear_lp": (_i, [_p, _p, _p, _p, _p, _i, _p, _p, _p, _p, _p, _i, _i, _i, _p]),
    "bf_concretize_lp": (_i, [_p, _p, _f, _i, _p, _p, _i, _i, _i, _i, _p]),
    "bf_chain_alpha_workspace_bytes": (_sz, [_p, _i, _i]),
    "bf_chain_alpha_crown": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _i, _f, _p, _p, _p, _i, _f, _i, _p, _sz, _i, _i, _p]),
    "bf_chain_alpha_beta_workspace_bytes": (_sz, [_p, _i, _i]),
    "bf_chain_alpha_beta_crown": (_i, [_p] * 12 + [_i, _f, _p, _p, _p, _i, _f, _i, _p, _sz, _i, _i, _p]),
    "bf_chain_alpha_beta_crown_reduce": (_i, [_p] * 12 + [_i, _f, _p, _p, _p, _i, _f, _i, _f, _p, _sz, _i, _i, _p]),
    "bf_chain_alpha_crown_objective": (_i, [_p] * 8 + [_i, _f, _p, _p, _i, _f, _i, _i, _f, _f, _f, _p, _sz, _i, _i, _p]),
    "bf_conv2d_dense_rows": (_i, [_p, _p, _p, _i, _p, _p] + [_i] * 12 + [_p]),
    "bf_relu_split_apply": (_i, [_p, _p, _p, _i, _p, _i, _i, _p]),
    "bf_interval_intersect": (_i, [_p, _p, _p, _p, _p, _i, _i, _p]),
    "bf_rows_add_broadcast": (_i, [_p, _p, _i, _i, _i, _i, _p]),
    "bf_adjoint_start_box": (_i, [_p, _p, _p, _i, _i, _i, _p]),
    "bf_adjoint_start_lp": (_i, [_p, _p, _f, _i, _i, _i, _i, _p]),
    "bf_rows_conv2d_fwd": (_i, [_p, _p, _p, _p] + [_i] * 13 + [_p]),
    "bf_relu_adjoint_rows": (_i, [_p] * 10 + [_i, _i, _i, _p]),
    "bf_alpha_select_best": (_i, [_p, _p, _p, _p, _i, _i, _f, _p, _i, _i, _p]),
    "bf_alpha_adam_step": (_i, [_p] * 9 + [_i, _f, _i, _i, _i, _i, _i, _p]),
    "bf_beta_adam_step": (_i, [_p, _p, _p, _p, _p, _i, _p, _p, _p, _i, _f, _i, _i, _i, _i, _i, _p]),
    "bf_alpha_select_best_paired": (_i, [_p, _p, _p, _p, _i, _i, _i, _f, _f, _f, _p, _i, _i, _p]),
    "bf_rows_scale": (_i, [_p, _p, C.c_longlong, _i, _p]),
    "bf_rows_colmax_abs": (_i, [_p, _p, _i, _i, _i, _p]),
    "bf_shared_metric": (_i, [_p, C.c_longlong, _p, _p, _i, _p]),
    "bf_copy_if": (_i, [_p, _p, C.c_longlong, _p, _p]),
    "bf_shared_adam_scratch_floats": (_sz, [_i, _i]),
    "bf_shared_adam_step": (_i, [_p, _p, _p, _p, _p, _i, _p, _p, _p, _i, _f, _f, _i, _i, _i, _i, _p]),
    "bf_shared_beta_add": (_i, [_p, _p, _i, _p, _i, _i, _p]),
    "bf_chain_alpha_crown_shared_objective": (_i, [_p] * 8 + [_i, _f, _p, _p, _p, _i, _f, _i, _i, _f, _f, _f, _p, _sz, _i, _i, _p]),
    "bf_branch_scores": (_i, [_p, _p, _p, _i, _p, _p, _p, _i, _p]),
    "bf_chain_alpha_grad": (_i, [_p, _p, _p, _p, _p, _p, _p, _i, _f, _p, _p, _i, _p, _sz, _i, _i, _p]),
    "bf_chain_alpha_shared_workspace_bytes": (_sz, [_p, _i, _i, _i]),
    "bf_chain_alpha_crown_shared": (_i, [_p] * 12 + [_i, _f, _p, _p, _p, _i, _f, _p, _sz, _i, _i, _p]),
    "bf_chain_alpha_beta_crown_shared_reduce": (_i, [_p] * 12 + [_i, _f, _p, _p, _p, _i, _f, _i, _f, _p, _sz, _i, _i, _p]),
}

_lib: Optional[C.CDLL] = None


class BackendError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"libbf_b200 error {code}: {message}")
        self.code = code


def load() -> C.CDLL:
    """Load the shared library (once) and set every prototype."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m boundflow_b200.csrc.build` "
            "(the CUDA backend has no CPU or PyTorch fallback)"
        )
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
        setattr(lib, name, _exact_arity(fn, len(args), name))
    _lib = lib
    return lib


def _exact_arity(fn, n_args: int, name: str):
    """ctypes refuses a call with too FEW arguments but passes surplus ones on, which silently shifts every later argument of
    a call written against an older signature (sizes, strides, the stream).  Every entry point is therefore called through
    this check: exactly the declared number of arguments, or TypeError."""

    def call(*args):
        if len(args) != n_args:
            raise TypeError(f"{name} takes exactly {n_args} arguments ({len(args)} given)")
        return fn(*args)

    call.__name__ = name
    call.restype, call.argtypes = fn.restype, fn.argtypes
    return call


def check(code: int) -> None:
    if code != BF_OK:
        msg = load().bf_last_error_string().decode("utf-8", "replace")
        if code == BF_E_UNSUPPORTED:
            raise NotImplementedError(f"libbf_b200: {msg}")
        if code == BF_E_INVALID:
            raise ValueError(f"libbf_b200: {msg}")
        raise BackendError(code, msg)


def ptr(t) -> Optional[int]:
    """Device pointer of a torch tensor (None -> NULL)."""
    return None if t is None else t.data_ptr()


def ptr_array(ts: Optional[Sequence]) -> Optional[C.Array]:
    """Host array of device pointers (entries may be None)."""
    if ts is None:
        return None
    arr = (_p * len(ts))()
    for k, t in enumerate(ts):
        arr[k] = None if t is None else t.data_ptr()
    return arr


def int_array(vals: Optional[Sequence[int]]):
    if vals is None:
        return None
    return (_i * len(vals))(*[int(v) for v in vals])


def launch_count() -> int:
    return int(load().bf_launch_count())


def tc_launch_count() -> int:
    """Launches of the tcgen05 contraction kernels since the library was loaded."""
    return int(load().bf_tc_launch_count())


class LinearPackCache:
    """Packed tensor-core images of Linear weights for the layer-level entry point
    `bf_crown_relu_linear_bwd_packed`, built once per weight tensor.

    An entry is keyed by the weight's storage address, shape, device and in-place version counter and
    keeps the weight tensor itself alive, so an address can never be reused by another tensor while its
    pack is cached.  Least recently used entries are dropped beyond `capacity`."""

    MIN_ROWS, MIN_WIDTH = 256, 32  # below these sizes the library uses the FFMA tiles and needs no pack

    def __init__(self, capacity: int = 32):
        self.capacity = int(capacity)
        self._entries: "dict[tuple, tuple]" = {}

    def get(self, W, rows: int, stream_ptr: int):
        """Device pack for weight `W` ([n_cur, n_prev], fp32, contiguous, CUDA), or None when the problem is too small."""
        n_cur, n_prev = int(W.shape[0]), int(W.shape[1])
        if rows < self.MIN_ROWS or n_cur < self.MIN_WIDTH or n_prev < self.MIN_WIDTH:
            return None
        key = (W.data_ptr(), n_cur, n_prev, W.device.index, W._version)
        hit = self._entries.pop(key, None)
        if hit is None:
            import torch

            lib = load()
            nbytes = int(lib.bf_linear_pack_bytes(n_cur, n_prev))
            pack = torch.empty(nbytes, dtype=torch.uint8, device=W.device)
            check(lib.bf_linear_pack(W.data_ptr(), n_cur, n_prev, pack.data_ptr(), nbytes, stream_ptr))
            hit = (W, pack)
            while len(self._entries) >= self.capacity:
                self._entries.pop(next(iter(self._entries)))
        self._entries[key] = hit  # most recently used last
        return hit[1]


LINEAR_PACKS = LinearPackCache()
