"""Typed Task-IR registry that runs fused ReLU->Affine backward tasks on the CUDA backend.

The reference dispatches typed Task IR units through registries with one method,
`dispatch(task, key, *, session, template)` (boundflow/runtime/task_backend_dispatch.py:
`PyTorchTaskBackendRegistry` 279-360, `TVMTaskBackendRegistry` 420-497, composite
`TypedTaskBackendRegistry` 500-540).  `TVMTaskBackendRegistry` turns a fused task (two ops:
relu_relaxation then linear_backward / conv2d_backward) into
`session.execute_fused_relu_affine_task(op_ids, output_value_ids=, executor=TVMFusedCrownExecutor())`
(bound_ir_interpreter.py:617-756).  `CudaTypedTaskBackendRegistry` is that registry with
`CudaFusedCrownExecutor` as the executor: it serves the backend kinds the plan marks as fused
(`tvm_fused_tir`, `tvm_tir_unfused`, `pytorch_chunked` by default) and hands every other
candidate to the registry given as `fallback` (normally the reference's
`TypedTaskBackendRegistry`).  Objects are read by attribute only, so the reference's own
`TaskIRUnit`, `BackendDispatchKey`, `PlanTemplate` and session are passed unchanged.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Iterable, Optional, Tuple

from .fused import CudaFusedCrownExecutor

FUSED_KINDS = ("tvm_fused_tir", "tvm_tir_unfused", "pytorch_chunked")


@dataclass(frozen=True)
class _PreparedTask:
    backend: str
    task_id: str
    op_ids: Tuple[str, ...]
    output_value_ids: Tuple[str, ...]
    capability_id: str


def _kind_value(x: Any) -> str:
    return str(getattr(x, "value", x))


class CudaTypedTaskBackendRegistry:
    def __init__(self, *, fallback: Optional[Any] = None, fused_kinds: Iterable[str] = FUSED_KINDS, executor: Optional[Any] = None):
        self.fallback = fallback
        self.fused_kinds = frozenset(fused_kinds)
        self.executor = executor if executor is not None else CudaFusedCrownExecutor()
        self._prepared: Dict[str, _PreparedTask] = {}
        self.cache_hits = 0
        self.cache_misses = 0
        self.cuda_dispatches = 0

    def dispatch(self, task: Any, key: Any, *, session: Any, template: Any) -> Any:
        candidates = {c.candidate_id: c for c in template.backend_candidates}
        candidate = candidates.get(key.backend_candidate_id)
        if candidate is None:
            raise ValueError("typed registry dispatch references unknown backend")
        backend = _kind_value(candidate.backend)
        if backend not in self.fused_kinds:
            if self.fallback is None:
                raise ValueError(f"CUDA registry rejects backend: {backend}")
            return self.fallback.dispatch(task, key, session=session, template=template)
        if key.task_id != task.task_id or key.backend_candidate_id != task.backend.backend_candidate_id or \
                key.capability_id != task.backend.capability_id:
            raise ValueError("backend dispatch key does not match typed task")
        if not getattr(candidate, "static_legal", True) or candidate.capability_id != task.backend.capability_id:
            raise ValueError("typed backend registry rejects selected capability")
        refs = tuple(task.op_refs)
        if not (len(refs) == 2 and _kind_value(refs[0].kind) == "relu_relaxation"
                and _kind_value(refs[1].kind) in ("linear_backward", "conv2d_backward")):
            raise ValueError("CUDA CROWN backend requires fused ReLU->Affine Task IR")
        prepared = _PreparedTask(backend=backend, task_id=task.task_id, op_ids=tuple(r.op_id for r in refs),
                                 output_value_ids=tuple(task.output_value_ids), capability_id=candidate.capability_id)
        digest = key.stable_hash()
        cached = self._prepared.get(digest)
        if cached is None:
            self._prepared[digest] = prepared
            self.cache_misses += 1
        elif cached != prepared:
            raise ValueError("CUDA backend cache key collision or stale task")
        else:
            self.cache_hits += 1
        self.cuda_dispatches += 1
        return session.execute_fused_relu_affine_task(prepared.op_ids, output_value_ids=prepared.output_value_ids, executor=self.executor)
