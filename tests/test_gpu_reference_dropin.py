"""The reference's OWN objects and callers driven through the CUDA adapters.

These tests need the reference package as built by `oracle/make_ref.py` (byte-compiled into the
git-ignored `oracle/_ref/`); they skip when it is absent.  Each test runs the reference's caller
twice -- once on its stock PyTorch path, once with a CUDA adapter plugged into the hook the
reference provides for it -- and compares:

  * `solve_bab_mlp(..., query_runtime=CudaQueryRuntime())`       bab.py:631-639, 1005, 1197
  * `run_ibp_scheduled(module, spec, executor=CudaTaskExecutor())` scheduler.py:160-255 on a module
    that `plan_interval_ibp_v2` split into several tasks
  * `PythonTaskExecutor(domain=CudaIntervalDomain())`               task_executor.py:127, domains/base.py:5-36
  * `run_crown_ibp_mlp(fused_crown_executor=CudaFusedCrownExecutor(),
                       fused_crown_steps=plan_fused_crown_regions(ops))`   crown_ibp.py:2054-2068
  * `PlainCrownBoundIRSession.execute_fused_relu_affine_task(..., executor=)` bound_ir_interpreter.py:617-756
    through `CudaTypedTaskBackendRegistry.dispatch`
  * the whole-query functions of `boundflow_b200.crown` fed the reference's `BFTaskModule` / `InputSpec`.
"""
import sys
from types import SimpleNamespace

import pytest
import torch

from oracle.make_ref import ref_path
from tests.helpers import assert_close

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(ref_path() is None, reason="oracle/_ref not built (python oracle/make_ref.py <checkout>)")]


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available()
    from boundflow_b200.csrc import build

    build.build()
    if ref_path() not in sys.path:
        sys.path.insert(0, ref_path())
    return torch.device("cuda", 0)


def _ref_mlp(seed, widths, device="cpu"):
    """Random ReLU MLP as the reference's BFTaskModule (plain tensors, no grad), one input point and its clean logits."""
    from boundflow.ir.task import BFTaskModule, BoundTask, TaskKind, TaskOp

    g = torch.Generator().manual_seed(seed)
    ops, params, cur = [], {}, "input"
    for k in range(len(widths) - 1):
        params[f"W{k}"] = (torch.randn(widths[k + 1], widths[k], generator=g) * (2.0 / widths[k]) ** 0.5).to(device)
        params[f"b{k}"] = (torch.randn(widths[k + 1], generator=g) * 0.1).to(device)
        out = "out" if k == len(widths) - 2 else f"h{k + 1}"
        ops.append(TaskOp(op_type="linear", name=f"lin{k}", inputs=[cur, f"W{k}", f"b{k}"], outputs=[out]))
        cur = out
        if k < len(widths) - 2:
            ops.append(TaskOp(op_type="relu", name=f"relu{k}", inputs=[cur], outputs=[f"r{k + 1}"]))
            cur = f"r{k + 1}"
    task = BoundTask(task_id="t0", kind=TaskKind.INTERVAL_IBP, ops=ops, input_values=["input"], output_values=["out"])
    x = torch.rand(1, widths[0], generator=g).to(device)
    h = x
    for k in range(len(widths) - 1):
        h = h @ params[f"W{k}"].t() + params[f"b{k}"]
        if k < len(widths) - 2:
            h = h.relu()
    return BFTaskModule(tasks=[task], entry_task_id="t0", bindings={"params": params}), x, h


@pytest.mark.parametrize("seed,eps", [(24, 0.3), (25, 0.1), (26, 0.1), (27, 0.2)])
@pytest.mark.parametrize("node_batch", [1, 4])
def test_solve_bab_mlp_through_cuda_query_runtime(dev, seed, eps, node_batch):
    """The reference's BaB driver with the CUDA query runtime reaches the reference's own verdict in the
    same number of nodes (cases found by running the reference: 7 to 21 nodes, proven and unsafe)."""
    from boundflow.runtime.bab import BabConfig, solve_bab_mlp
    from boundflow.runtime.task_executor import InputSpec

    from boundflow_b200.query_runtime import CudaQueryRuntime

    module, x, logits = _ref_mlp(seed, (4, 8, 8, 2))
    y = int(logits.argmax())
    C = torch.zeros(1, 1, 2)
    C[0, 0, y], C[0, 0, 1 - y] = 1.0, -1.0
    spec = InputSpec.linf(value_name="input", center=x, eps=eps)
    cfg = BabConfig(max_nodes=64, oracle="alpha_beta", node_batch_size=node_batch, alpha_steps=5, alpha_lr=0.2, alpha_init=0.5,
                    beta_init=0.0, threshold=0.0, tol=1e-8)
    want = solve_bab_mlp(module, spec, linear_spec_C=C, config=cfg)
    rt = CudaQueryRuntime()
    got = solve_bab_mlp(module, spec, linear_spec_C=C, config=cfg, query_runtime=rt)
    assert got.status == want.status
    assert got.nodes_visited == want.nodes_visited
    assert abs(float(got.best_lower) - float(want.best_lower)) <= 1e-4 + 1e-5 * abs(float(want.best_lower))
    assert rt.audit()["queries"] >= 1


def test_toy_property_through_cuda_query_runtime(dev):
    """The 1-D toy of the reference's own BaB tests (identity-ReLU-identity on [-1, 1]): once with alpha fixed at 0.5
    and no optimisation steps (the root bound is negative, the driver has to split), once with 40 steps and node
    batches of 4; status, node count and best lower bound equal the reference's own run."""
    from boundflow.ir.task import BFTaskModule, BoundTask, TaskKind, TaskOp
    from boundflow.runtime.bab import BabConfig, solve_bab_mlp
    from boundflow.runtime.task_executor import InputSpec

    from boundflow_b200.query_runtime import CudaQueryRuntime

    one, zero = torch.tensor([[1.0]]), torch.tensor([0.0])
    task = BoundTask(task_id="t0", kind=TaskKind.INTERVAL_IBP, input_values=["input"], output_values=["out"], ops=[
        TaskOp(op_type="linear", name="linear1", inputs=["input", "W1", "b1"], outputs=["h1"]),
        TaskOp(op_type="relu", name="relu1", inputs=["h1"], outputs=["r1"]),
        TaskOp(op_type="linear", name="linear2", inputs=["r1", "W2", "b2"], outputs=["out"])])
    module = BFTaskModule(tasks=[task], entry_task_id="t0", bindings={"params": {"W1": one, "b1": zero, "W2": one.clone(), "b2": zero.clone()}})
    spec = InputSpec.linf(value_name="input", center=torch.tensor([[0.0]]), eps=1.0)
    for cfg in (BabConfig(max_nodes=16, oracle="alpha_beta", node_batch_size=1, alpha_steps=0, alpha_lr=0.2, alpha_init=0.5, beta_init=0.0, threshold=0.0, tol=1e-8),
                BabConfig(max_nodes=32, oracle="alpha_beta", node_batch_size=4, alpha_steps=40, alpha_lr=0.2, alpha_init=0.5, beta_init=0.0, threshold=0.0, tol=1e-8)):
        want = solve_bab_mlp(module, spec, config=cfg)
        got = solve_bab_mlp(module, spec, config=cfg, query_runtime=CudaQueryRuntime())
        assert got.status == want.status
        assert got.nodes_visited == want.nodes_visited
        assert abs(float(got.best_lower) - float(want.best_lower)) <= 1e-6


def test_run_ibp_scheduled_multitask_module_with_cuda_executor(dev):
    """A module the reference's planner split into tasks, walked by the reference's scheduler with the CUDA
    executor as its step executor (env of physical buffers mutated in place)."""
    import torch.nn as nn
    from boundflow.frontends.pytorch.frontend import import_torch
    from boundflow.planner import plan_interval_ibp_v0, plan_interval_ibp_v2
    from boundflow.planner.interval_v2 import IntervalV2PartitionConfig
    from boundflow.runtime.scheduler import run_ibp_scheduled
    from boundflow.runtime.task_executor import LinfInputSpec, PythonTaskExecutor

    from boundflow_b200.executor import CudaIntervalDomain, CudaTaskExecutor

    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(16, 32), nn.ReLU(), nn.Linear(32, 24), nn.ReLU(), nn.Linear(24, 8))
    x0 = torch.randn(4, 16)
    program = import_torch(model, (x0,), export_mode="export", normalize=True)
    m0 = plan_interval_ibp_v0(program)
    out_name = m0.get_entry_task().output_values[0]
    m2 = plan_interval_ibp_v2(program, config=IntervalV2PartitionConfig(min_tasks=2))
    assert m2.task_graph is not None and len(m2.tasks) >= 2
    spec = LinfInputSpec(value_name="input", center=x0, eps=0.05)
    want = run_ibp_scheduled(m2, spec, executor=PythonTaskExecutor(), output_value=out_name)
    got = run_ibp_scheduled(m2, spec, executor=CudaTaskExecutor(), output_value=out_name)
    assert_close(got.lower, want.lower, "scheduled IBP lower")
    assert_close(got.upper, want.upper, "scheduled IBP upper")
    # whole-module entry point on the single-task plan, and the CUDA domain inside the reference's own executor
    got0 = CudaTaskExecutor().run_ibp(m0, spec)
    assert_close(got0.lower, want.lower, "run_ibp lower")
    got_dom = PythonTaskExecutor(domain=CudaIntervalDomain()).run_ibp(m0, spec)
    assert_close(got_dom.lower, want.lower, "CUDA domain lower")
    assert_close(got_dom.upper, want.upper, "CUDA domain upper")


@pytest.mark.parametrize("widths,B", [((12, 20, 16, 5), 3), ((64, 512, 512, 10), 40)])
def test_reference_crown_with_cuda_fused_executor(dev, widths, B, tc_from_256_rows):
    """The reference's CROWN sweep (torch on the GPU) with every planned ReLU->affine region handed to the CUDA
    executor; the second case (360 coefficient rows, 512-wide layers) must reach the tcgen05 kernel."""
    from boundflow.runtime.crown_ibp import run_crown_ibp_mlp
    from boundflow.runtime.fused_crown import plan_fused_crown_regions
    from boundflow.runtime.task_executor import InputSpec

    from boundflow_b200 import _lib
    from boundflow_b200.fused import CudaFusedCrownExecutor

    module, _x, _h = _ref_mlp(5, widths, device=dev)
    g = torch.Generator().manual_seed(9)
    x = torch.rand(B, widths[0], generator=g).to(dev)
    S = 9
    C = torch.randn(B, S, widths[-1], generator=g).to(dev)
    spec = InputSpec.linf(value_name="input", center=x, eps=0.02)
    want = run_crown_ibp_mlp(module, spec, linear_spec_C=C)
    steps = plan_fused_crown_regions(module.get_entry_task().ops)
    assert len(steps) >= 1
    tc0 = _lib.tc_launch_count()
    got = run_crown_ibp_mlp(module, spec, linear_spec_C=C, fused_crown_executor=CudaFusedCrownExecutor(), fused_crown_steps=steps)
    assert_close(got.lower, want.lower, "fused-executor CROWN lower")
    assert_close(got.upper, want.upper, "fused-executor CROWN upper")
    if B * S >= 256:
        assert _lib.tc_launch_count() > tc0, "the large fused region did not run on the tensor-core kernel"


def test_typed_ir_session_with_cuda_registry(dev):
    """A real PlainCrownBoundIRSession of the reference: the fused ReLU->Linear Bound-IR pair goes through
    CudaTypedTaskBackendRegistry.dispatch into session.execute_fused_relu_affine_task(executor=CUDA), every other op
    through the session's own reference step; the result equals the whole-graph reference interpreter."""
    from boundflow.frontends.plain_crown_bound_ir import build_plain_crown_bound_ir
    from boundflow.runtime.bound_ir_interpreter import PlainCrownBoundIRSession, execute_plain_crown_bound_ir
    from boundflow.runtime.crown_ibp import _forward_ibp_trace_mlp
    from boundflow.runtime.task_executor import InputSpec

    from boundflow_b200.typed_backend import CudaTypedTaskBackendRegistry

    module, _x, _h = _ref_mlp(11, (6, 40, 36, 4), device=dev)
    x = torch.rand(3, 6, generator=torch.Generator().manual_seed(3)).to(dev)
    spec = InputSpec.linf(value_name="input", center=x, eps=0.1)
    interval_env, relu_pre = _forward_ibp_trace_mlp(module, spec)
    bound_module = build_plain_crown_bound_ir(module, spec, interval_env=interval_env, relu_pre=relu_pre).module
    want = execute_plain_crown_bound_ir(bound_module, task_module=module, input_spec=spec, relu_pre=relu_pre)
    session = PlainCrownBoundIRSession(bound_module, task_module=module, input_spec=spec, relu_pre=relu_pre)
    registry = CudaTypedTaskBackendRegistry()
    ops = bound_module.graph.ops
    i, fused = 0, 0
    while i < len(ops):
        op = ops[i]
        nxt = ops[i + 1] if i + 1 < len(ops) else None
        if op.kind.value == "relu_relaxation" and nxt is not None and nxt.kind.value in ("linear_backward", "conv2d_backward"):
            # the typed task / key / template as the registry reads them (attributes only)
            cand = SimpleNamespace(candidate_id=f"cand{i}", backend=SimpleNamespace(value="tvm_fused_tir"), capability_id="cap", static_legal=True)
            task = SimpleNamespace(task_id=f"task{i}", backend=SimpleNamespace(backend_candidate_id=cand.candidate_id, capability_id="cap"),
                                   op_refs=(SimpleNamespace(op_id=op.op_id, kind=op.kind), SimpleNamespace(op_id=nxt.op_id, kind=nxt.kind)),
                                   output_value_ids=tuple(nxt.outputs))
            key = SimpleNamespace(task_id=task.task_id, backend_candidate_id=cand.candidate_id, capability_id="cap", stable_hash=lambda t=task: t.task_id)
            registry.dispatch(task, key, session=session, template=SimpleNamespace(backend_candidates=(cand,)))
            fused += 1
            i += 2
        else:
            session.execute_task((op.op_id,), output_value_ids=tuple(op.outputs))
            i += 1
    got = session.result()
    assert fused == 2 and registry.cuda_dispatches == 2
    assert_close(got.lower, want.lower, "typed-IR session lower")
    assert_close(got.upper, want.upper, "typed-IR session upper")


def test_whole_query_functions_accept_reference_objects(dev):
    """`boundflow_b200.crown` called with the reference's BFTaskModule / InputSpec / AlphaState instead of the mirrors."""
    from boundflow.runtime.alpha_beta_crown import run_alpha_beta_crown_mlp as ref_ab
    from boundflow.runtime.alpha_crown import AlphaState
    from boundflow.runtime.crown_ibp import _forward_ibp_trace_mlp, run_crown_ibp_mlp as ref_crown
    from boundflow.runtime.task_executor import InputSpec

    from boundflow_b200.crown import forward_ibp_trace_mlp, run_alpha_beta_crown_mlp, run_crown_ibp_mlp

    module, _x, _h = _ref_mlp(21, (10, 32, 32, 6))
    g = torch.Generator().manual_seed(4)
    x = torch.rand(5, 10, generator=g)
    C = torch.randn(5, 4, 6, generator=g)
    spec = InputSpec.box(value_name="input", lower=(x - 0.05).clamp(0, 1), upper=(x + 0.05).clamp(0, 1))
    want = ref_crown(module, spec, linear_spec_C=C)
    got = run_crown_ibp_mlp(module, spec, linear_spec_C=C)
    assert_close(got.lower, want.lower, "CROWN lower")
    assert_close(got.upper, want.upper, "CROWN upper")
    # the reference's execution-strategy keywords are accepted (no effect on the bounds)
    got = run_crown_ibp_mlp(module, spec, linear_spec_C=C, materialization_plan=None, materialization_placement_plan=None,
                            fused_crown_executor=None, fused_crown_steps=())
    assert_close(got.lower, want.lower, "CROWN lower, strategy keywords given")
    env_w, pre_w = _forward_ibp_trace_mlp(module, spec)
    env_g, pre_g = forward_ibp_trace_mlp(module, spec)
    for name in pre_w:
        assert_close(pre_g[name].lower, pre_w[name].lower, f"pre {name} lower")
        assert_close(pre_g[name].upper, pre_w[name].upper, f"pre {name} upper")
    a0 = {n: torch.full_like(p.lower, 0.5) for n, p in pre_w.items()}
    bw, aw, _bw, _sw = ref_ab(module, spec, linear_spec_C=C, steps=1, lr=0.1, warm_start_alpha=AlphaState(alpha_by_relu_input=a0), per_batch_params=True)
    bg, ag, _bg, _sg = run_alpha_beta_crown_mlp(module, spec, linear_spec_C=C, steps=1, lr=0.1, warm_start_alpha=AlphaState(alpha_by_relu_input=a0), per_batch_params=True)
    assert_close(bg.lower, bw.lower, "alpha-CROWN (1 step) lower")
    assert_close(bg.upper, bw.upper, "alpha-CROWN (1 step) upper")
