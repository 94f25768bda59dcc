"""CPU-side checks: the C-ABI library loads and exports every declared symbol, host
logic (IR mirrors, workload generators, sharding) behaves, and argument validation in
the library works without touching a GPU."""
import ctypes
import os
import re
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from boundflow_b200.csrc import build

    build.build()
    from boundflow_b200 import _lib

    return _lib.load()


def test_library_exports_every_declared_symbol(lib):
    from boundflow_b200 import _lib

    header = open(os.path.join(ROOT, "include", "bf_b200.h")).read()
    declared = set(re.findall(r"\b(bf_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations parsed"
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in include/bf_b200.h but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes prototype"
    assert set(_lib.SIGNATURES) == declared
    assert lib.bf_version() >= 100


def test_argument_validation_needs_no_gpu(lib):
    from boundflow_b200 import _lib

    assert lib.bf_ibp_linear(None, None, 0, 0, None, None, None, 0, None, None, None, None, None, 1, 1, 1, None) == _lib.BF_E_INVALID
    assert b"null" in lib.bf_last_error_string()
    assert lib.bf_concretize(None, None, None, None, None, 0, 1, 1, 1, None) == _lib.BF_E_INVALID
    descs = (_lib.LayerDesc * 2)()
    descs[0].op, descs[0].n_in, descs[0].n_out = _lib.OP_RELU, 4, 4
    descs[1].op, descs[1].n_in, descs[1].n_out = _lib.OP_RELU, 5, 5   # width mismatch
    h = ctypes.c_void_p()
    assert lib.bf_chain_create(descs, 2, ctypes.byref(h)) == _lib.BF_E_INVALID
    with pytest.raises(ValueError):
        _lib.check(_lib.BF_E_INVALID)
    with pytest.raises(NotImplementedError):
        _lib.check(_lib.BF_E_UNSUPPORTED)
    # a surplus argument (a call written against an older signature) is refused instead of shifting the later ones
    with pytest.raises(TypeError):
        lib.bf_concretize(None, None, None, None, None, 0, 1, 1, 1, 1, None)
    with pytest.raises(TypeError):
        lib.bf_concretize(None, None, None, None, None, 0, 1, 1, 1)


def test_chain_workspace_queries(lib):
    from boundflow_b200 import _lib

    descs = (_lib.LayerDesc * 3)()
    dummy = ctypes.c_void_p(256)  # never dereferenced on the host
    descs[0].op, descs[0].n_in, descs[0].n_out, descs[0].W = _lib.OP_LINEAR, 784, 100, dummy
    descs[1].op, descs[1].n_in, descs[1].n_out = _lib.OP_RELU, 100, 100
    descs[2].op, descs[2].n_in, descs[2].n_out, descs[2].W = _lib.OP_LINEAR, 100, 10, dummy
    h = ctypes.c_void_p()
    assert lib.bf_chain_create(descs, 3, ctypes.byref(h)) == 0
    assert lib.bf_chain_num_relu(h) == 1
    B, S = 64, 9
    a = lib.bf_chain_alpha_workspace_bytes(h, B, S)
    c = lib.bf_chain_crown_workspace_bytes(h, B, S, 3)
    assert a >= B * S * (784 + 100) * 4 and c >= 2 * B * S * 784 * 4
    assert lib.bf_chain_alpha_workspace_bytes(h, 2 * B, S) > a
    lib.bf_chain_destroy(h)


def test_missing_library_fails_loudly(tmp_path, monkeypatch):
    from boundflow_b200 import _lib

    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(ImportError):
        _lib.load()


def test_no_cuda_means_error_not_fallback():
    if torch.cuda.is_available():
        pytest.skip("CUDA present")
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import run_crown_ibp_mlp
    from boundflow_b200.ir import InputSpec

    wl = W.make_workload("c1", batch=2)
    with pytest.raises(RuntimeError):
        run_crown_ibp_mlp(wl.module, InputSpec.box(value_name="input", lower=wl.lo, upper=wl.up), linear_spec_C=wl.C)


def test_workloads_are_seeded_and_prefix_stable():
    from boundflow_b200 import workloads as W

    a = W.make_workload("c3", batch=4)
    b = W.make_workload("c3", batch=8)
    assert torch.equal(a.x, b.x[:4]) and torch.equal(a.C, b.C[:4])
    assert torch.equal(a.module.bindings["params"]["W1"], b.module.bindings["params"]["W1"])
    assert a.C.shape == (4, 9, 10) and (a.C.sum(dim=2) == 0).all()
    c5 = W.make_workload("c5", batch=1)
    assert [l["op"] for l in c5.layers].count("conv2d") == 4 and c5.relu_names == ["h1", "h2", "h3", "h4", "h5"]


def test_split_domains_pick_unstable_neurons():
    from boundflow_b200 import workloads as W
    from oracle import crown_oracle as O

    wl = W.make_workload("c4")
    root = O.forward_ibp_trace(wl.layers, O.box_input(wl.lo, wl.up))
    splits = W.make_split_domains(wl, root.pre, n_domains=6)
    total = sum(s.abs().to(torch.int64).sum(dim=1) for s in splits)
    assert (total == 10).all()
    for s, (l, u) in zip(splits, root.pre):
        amb = ((l < 0) & (u > 0)).expand_as(s)
        assert ((s != 0) <= amb).all()


def test_ir_mirrors_and_input_sets():
    from boundflow_b200.ir import InputSpec, LinfInputSpec, input_mid_rad, normalize_input_spec

    x = torch.rand(3, 5)
    mid, rad, lo, up = input_mid_rad(LinfInputSpec("input", x, 0.1))
    assert torch.equal(mid, x) and torch.allclose(rad, torch.full_like(x, 0.1))
    spec = InputSpec.box(value_name="input", lower=x - 0.2, upper=x + 0.1)
    mid, rad, lo, up = input_mid_rad(spec)
    assert torch.allclose(mid, x - 0.05) and torch.allclose(rad, torch.full_like(x, 0.15))
    assert normalize_input_spec(spec) is spec
    with pytest.raises(NotImplementedError):
        input_mid_rad(InputSpec("input", x, __import__("boundflow_b200").LpBallPerturbation(p=2, eps=0.1)))


def test_shard_ranges_cover_everything():
    from boundflow_b200.dist import shard_range, shard_sizes

    for n in (0, 1, 7, 64, 8192, 8193):
        for world in (1, 2, 3, 8):
            spans = [shard_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            assert max(shard_sizes(n, world)) - min(shard_sizes(n, world)) <= 1


_GLOO_WORKER = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from boundflow_b200.dist import shard_range, gather_domain_results
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo", rank=rank, world_size=world)
n, S = 11, 9
full = torch.arange(n * S, dtype=torch.float32).reshape(n, S)
verd = (torch.arange(n) % 3 == 0).to(torch.int8)
a, b = shard_range(n, rank, world)
lo, v = gather_domain_results(full[a:b].clone(), verd[a:b].clone(), n)
assert torch.equal(lo, full) and torch.equal(v, verd), (rank, lo, v)
dist.barrier(); dist.destroy_process_group()
print("ok", rank)
"""


def test_gather_world_size_2_gloo(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(_GLOO_WORKER)
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT="29631")
        procs.append(subprocess.Popen([sys.executable, str(script), ROOT], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT))
    for p in procs:
        out, _ = p.communicate(timeout=120)
        assert p.returncode == 0, out.decode()


def test_typed_registry_routes_fused_tasks_to_the_cuda_executor():
    """Typed Task-IR dispatch (no GPU needed: the session and the executor are fakes)."""
    from types import SimpleNamespace as NS

    from boundflow_b200.typed_backend import CudaTypedTaskBackendRegistry

    calls = []

    class Session:
        def execute_fused_relu_affine_task(self, op_ids, *, output_value_ids, executor):
            calls.append((op_ids, output_value_ids, executor))
            return "step-result"

    class Fallback:
        def dispatch(self, task, key, *, session, template):
            return "fallback-result"

    def make(kind, second="linear_backward", n_ops=2):
        cand = NS(candidate_id="cand0", backend=NS(value=kind), capability_id="cap0", static_legal=True)
        refs = [NS(op_id="op_relu", kind=NS(value="relu_relaxation")), NS(op_id="op_aff", kind=NS(value=second))][:n_ops]
        task = NS(task_id="t0", backend=NS(backend_candidate_id="cand0", capability_id="cap0"), op_refs=refs, output_value_ids=("v1", "v2"))
        key = NS(task_id="t0", backend_candidate_id="cand0", capability_id="cap0", stable_hash=lambda: "h-" + kind + second)
        return task, key, NS(backend_candidates=[cand])

    executor = object()
    reg = CudaTypedTaskBackendRegistry(fallback=Fallback(), executor=executor)
    task, key, template = make("tvm_fused_tir")
    assert reg.dispatch(task, key, session=Session(), template=template) == "step-result"
    assert calls[-1] == (("op_relu", "op_aff"), ("v1", "v2"), executor)
    assert reg.dispatch(task, key, session=Session(), template=template) == "step-result"
    assert (reg.cache_misses, reg.cache_hits, reg.cuda_dispatches) == (1, 1, 2)
    task, key, template = make("pytorch_chunked", second="conv2d_backward")
    assert reg.dispatch(task, key, session=Session(), template=template) == "step-result"
    task, key, template = make("reference")
    assert reg.dispatch(task, key, session=Session(), template=template) == "fallback-result"
    with pytest.raises(ValueError):
        CudaTypedTaskBackendRegistry(executor=executor).dispatch(task, key, session=Session(), template=template)
    task, key, template = make("tvm_fused_tir", n_ops=1)
    with pytest.raises(ValueError):
        reg.dispatch(task, key, session=Session(), template=template)
    task, key, template = make("tvm_fused_tir")
    key.capability_id = "other"
    with pytest.raises(ValueError):
        reg.dispatch(task, key, session=Session(), template=template)


def test_query_runtime_groups_chunks_and_keeps_request_order(monkeypatch):
    """Host logic of CudaQueryRuntime.execute (no GPU: the batch executor is replaced)."""
    from types import SimpleNamespace as NS

    import torch

    from boundflow_b200.ir import InputSpec
    from boundflow_b200.query_runtime import CudaQueryRuntime

    def req(qid, method, steps):
        spec = InputSpec.box(value_name="input", lower=torch.zeros(1, 4), upper=torch.ones(1, 4))
        payload = NS(input_spec=spec, linear_spec_c=torch.zeros(2, 3), split_by_relu_input={"h": torch.zeros(5, dtype=torch.int8)},
                     warm_alpha_by_relu_input={}, warm_beta_by_relu_input={})
        return NS(query=NS(query_id=qid, bound_method=NS(value=method), execution_options={"alpha_steps": steps}), payload=payload)

    batches = []

    def fake_batch(self, module, reqs, method):
        batches.append((method, [r.query.query_id for r in reqs]))
        return [f"res-{r.query.query_id}" for r in reqs]

    monkeypatch.setattr(CudaQueryRuntime, "_execute_batch", fake_batch)
    rt = CudaQueryRuntime(max_batch_size=2)
    reqs = [req("a0", "alpha-beta-CROWN", 5), req("b0", "alpha-CROWN", 5), req("a1", "alpha-beta-CROWN", 5),
            req("c0", "alpha-beta-CROWN", 7), req("a2", "alpha-beta-CROWN", 5)]
    out = rt.execute(None, reqs)
    assert out == [(r.query.query_id, f"res-{r.query.query_id}") for r in reqs]
    # same method + options + shapes share a batch, chunked by max_batch_size; different options or methods do not mix
    assert ("alpha-beta-CROWN", ["a0", "a1"]) in batches and ("alpha-beta-CROWN", ["a2"]) in batches
    assert ("alpha-CROWN", ["b0"]) in batches and ("alpha-beta-CROWN", ["c0"]) in batches
    assert rt.execute(None, []) == []
    with pytest.raises(ValueError):
        CudaQueryRuntime(max_batch_size=0)


def test_capability_query_graph_detection_and_dense_conv_weights():
    """Host logic that needs no GPU: `get_crown_ibp_mlp_stats` (same conditions as the reference, crown_ibp.py:2279-2349),
    `needs_graph_path`, and the dense equivalent of a grouped, dilated Conv2d weight."""
    import torch

    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import get_crown_ibp_mlp_stats, needs_graph_path
    from boundflow_b200.ir import BFTaskModule, BoundTask, TaskKind, TaskOp
    from boundflow_b200.network import dense_conv_weight

    chain = W.make_workload("c2", batch=1).module
    st = get_crown_ibp_mlp_stats(chain)
    assert st.supported and st.ops_seen[0] == "conv2d" and not needs_graph_path(chain)
    for name, module in ((k, v[0]) for k, v in W.make_graph_cases().items()):
        assert needs_graph_path(module), name
        assert get_crown_ibp_mlp_stats(module).supported, name
    for name, (module, *_rest) in W.make_executor_op_cases().items():
        assert not get_crown_ibp_mlp_stats(module).supported, name

    def one_op(op):
        task = BoundTask(task_id="t", kind=TaskKind.INTERVAL_IBP, ops=[op], input_values=["input"], output_values=[op.outputs[0]])
        return BFTaskModule(tasks=[task], entry_task_id="t", bindings={"params": {}})

    assert "flatten" in get_crown_ibp_mlp_stats(one_op(TaskOp("flatten", "f", ["input"], ["y"], {"start_dim": 0, "end_dim": -1}))).reason
    assert "add expects 2 inputs" in get_crown_ibp_mlp_stats(one_op(TaskOp("add", "a", ["input"], ["y"]))).reason
    assert "concat axis" in get_crown_ibp_mlp_stats(one_op(TaskOp("concat", "c", ["input", "input"], ["y"], {"axis": 2}))).reason
    # dense equivalents: groups only, dilation only, both, and the identity case
    g = torch.Generator().manual_seed(0)
    x = torch.randn(2, 6, 9, 9, generator=g)
    for groups, dil, k in ((3, 1, 3), (1, 2, 3), (2, 3, 2), (6, 1, 1)):
        Wg = torch.randn(6, 6 // groups, k, k, generator=g)
        attrs = {"groups": groups, "dilation": (dil, dil)}
        ref = torch.nn.functional.conv2d(x, Wg, None, 1, 2, dil, groups)
        got = torch.nn.functional.conv2d(x, dense_conv_weight(Wg, attrs), None, 1, 2)
        assert torch.allclose(got, ref, atol=1e-5), (groups, dil)
        assert dense_conv_weight(Wg, attrs) is dense_conv_weight(Wg, attrs)   # cached per weight tensor
    W1 = torch.randn(4, 6, 3, 3, generator=g)
    assert dense_conv_weight(W1, {"groups": 1, "dilation": 1}) is W1
    with pytest.raises(ValueError):
        dense_conv_weight(torch.randn(5, 3, 3, 3), {"groups": 2})
