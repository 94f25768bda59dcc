"""boundflow_b200: B200 (sm_100a) CUDA backend for BoundFlow's bound-propagation hot path.

Importing the package never touches CUDA; the first compute call loads
libbf_b200.so (built by `python -m boundflow_b200.csrc.build`) and fails loudly
if it is missing -- there is no CPU or PyTorch fallback.
"""
from .ir import (  # noqa: F401
    BFTaskModule,
    BoundTask,
    BoxPerturbation,
    InputSpec,
    IntervalState,
    LinearSpec,
    LinfInputSpec,
    LpBallPerturbation,
    StoragePlan,
    TaskKind,
    TaskOp,
)

__all__ = [
    "BFTaskModule", "BoundTask", "BoxPerturbation", "InputSpec", "IntervalState", "LinearSpec", "LinfInputSpec",
    "LpBallPerturbation", "StoragePlan", "TaskKind", "TaskOp",
]
