"""Host-side mirror of the reference types that cross the executor boundary.

The backend is duck-typed: it only reads the attributes listed here, so objects
built by the reference itself (boundflow/ir/task.py:119-240 `TaskOp`,
`BoundTask`, `BFTaskModule`, `StoragePlan`; boundflow/domains/interval.py:13-24
`IntervalState`; boundflow/runtime/task_executor.py:24-71 `InputSpec`,
`LinfInputSpec`; boundflow/runtime/perturbation.py:73-359 `LpBallPerturbation`,
`BoxPerturbation`; boundflow/ir/spec.py:10 `LinearSpec`) can be handed to it
unchanged.  These light-weight equivalents exist so that the backend, its tests
and its benchmark run where the reference package is not installed.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Dict, List, Optional

import torch


class TaskKind(Enum):
    INTERVAL_IBP = "interval_ibp"


@dataclass
class TaskOp:
    op_type: str
    name: str
    inputs: List[str]
    outputs: List[str]
    attrs: Dict[str, Any] = field(default_factory=dict)


@dataclass
class BoundTask:
    task_id: str
    kind: Any
    ops: List[TaskOp]
    input_values: List[str]
    output_values: List[str]
    input_buffers: List[str] = field(default_factory=list)
    output_buffers: List[str] = field(default_factory=list)
    params: List[str] = field(default_factory=list)


@dataclass
class StoragePlan:
    """value name -> logical buffer -> physical buffer (identity when empty)."""

    buffers: Dict[str, Any] = field(default_factory=dict)
    value_to_buffer: Dict[str, str] = field(default_factory=dict)
    physical_buffers: Dict[str, Any] = field(default_factory=dict)
    logical_to_physical: Dict[str, str] = field(default_factory=dict)

    def to_physical(self, logical_buffer_id: str) -> str:
        return self.logical_to_physical.get(logical_buffer_id, logical_buffer_id)


@dataclass
class BFTaskModule:
    tasks: List[BoundTask]
    entry_task_id: str
    bindings: Dict[str, Any] = field(default_factory=dict)
    storage_plan: StoragePlan = field(default_factory=StoragePlan)
    task_graph: Optional[Any] = None

    def get_task(self, task_id: str) -> BoundTask:
        for t in self.tasks:
            if t.task_id == task_id:
                return t
        raise KeyError(f"task_id not found: {task_id}")

    def get_entry_task(self) -> BoundTask:
        return self.get_task(self.entry_task_id)

    def validate(self) -> None:
        if not self.tasks:
            raise ValueError("BFTaskModule.tasks must be non-empty")
        self.get_entry_task()
        for t in self.tasks:
            if not t.ops:
                raise ValueError(f"task '{t.task_id}' has no ops")


@dataclass
class IntervalState:
    lower: torch.Tensor
    upper: torch.Tensor


@dataclass(frozen=True)
class LpBallPerturbation:
    p: Any
    eps: float

    def norm(self) -> str:
        p = self.p
        if isinstance(p, str):
            if p.strip().lower() in {"inf", "l_inf", "linf"}:
                return "inf"
            raise ValueError(f"unsupported p string for LpBallPerturbation: {p!r}")
        if float(p) == float("inf"):
            return "inf"
        if int(p) == p and int(p) in (1, 2):
            return str(int(p))
        raise ValueError(f"unsupported p for LpBallPerturbation: {p!r}")


@dataclass(frozen=True)
class BoxPerturbation:
    lower: torch.Tensor
    upper: torch.Tensor

    def __post_init__(self) -> None:
        if self.lower.shape != self.upper.shape:
            raise ValueError("BoxPerturbation shape mismatch")
        if not torch.is_floating_point(self.lower) or self.lower.dtype != self.upper.dtype:
            raise TypeError("BoxPerturbation bounds must be floating point of one dtype")


@dataclass(frozen=True)
class LinfInputSpec:
    value_name: str
    center: torch.Tensor
    eps: float


@dataclass(frozen=True)
class InputSpec:
    value_name: str
    center: torch.Tensor
    perturbation: Any

    @staticmethod
    def linf(*, value_name: str, center: torch.Tensor, eps: float) -> "InputSpec":
        return InputSpec(value_name, center, LpBallPerturbation(p="inf", eps=float(eps)))

    @staticmethod
    def l2(*, value_name: str, center: torch.Tensor, eps: float) -> "InputSpec":
        return InputSpec(value_name, center, LpBallPerturbation(p=2, eps=float(eps)))

    @staticmethod
    def l1(*, value_name: str, center: torch.Tensor, eps: float) -> "InputSpec":
        return InputSpec(value_name, center, LpBallPerturbation(p=1, eps=float(eps)))

    @staticmethod
    def box(*, value_name: str, lower: torch.Tensor, upper: torch.Tensor) -> "InputSpec":
        return InputSpec(value_name, (lower + upper) / 2.0, BoxPerturbation(lower=lower, upper=upper))


@dataclass(frozen=True)
class LinearSpec:
    C: torch.Tensor
    name: str = "linear_spec"


def normalize_input_spec(spec: Any) -> InputSpec:
    """`LinfInputSpec` -> `InputSpec` (task_executor.py:566-571 in the reference)."""
    if hasattr(spec, "perturbation"):
        return spec
    return InputSpec.linf(value_name=spec.value_name, center=spec.center, eps=float(spec.eps))


def input_mid_rad(spec: Any):
    """Midpoint/radius tensors of an input spec's perturbation set.

    Box: midpoint (lo+up)/2 and radius (up-lo)/2 (perturbation.py:297-298);
    L-inf ball: the centre itself and eps (perturbation.py:201-215).
    Other norms are not accelerated by this backend.
    """
    spec = normalize_input_spec(spec)
    pert = spec.perturbation
    if hasattr(pert, "lower") and hasattr(pert, "upper"):
        lo, up = pert.lower, pert.upper
        return (lo + up) / 2.0, (up - lo) / 2.0, lo, up
    if hasattr(pert, "eps"):
        p = pert.norm() if hasattr(pert, "norm") else pert._normalize_p()
        if p != "inf":
            raise NotImplementedError("midpoint/radius form exists for boxes and L-inf balls only; see lp_ball_of()")
        eps = float(pert.eps)
        c = spec.center
        return c, torch.full_like(c, eps), c - eps, c + eps
    raise TypeError(f"unsupported perturbation: {type(pert)}")


def lp_ball_of(spec: Any):
    """(p, eps) with p in {1, 2} when the input set is an L1 / L2 ball, else None.
    (`LpBallPerturbation`, runtime/perturbation.py:73-222; L-inf balls are handled as boxes.)"""
    spec = normalize_input_spec(spec)
    pert = spec.perturbation
    if hasattr(pert, "lower") and hasattr(pert, "upper"):
        return None
    if hasattr(pert, "eps"):
        p = pert.norm() if hasattr(pert, "norm") else pert._normalize_p()
        if p in ("1", "2"):
            return int(p), float(pert.eps)
    return None
