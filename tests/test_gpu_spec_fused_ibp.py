"""IBP with the output spec merged into the last Linear layer (batched-W linear kernel)."""
import copy

import pytest
import torch

from tests.helpers import assert_close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available()
    from boundflow_b200.csrc import build

    build.build()
    return torch.device("cuda", 0)


def _fused_module(wl, dev):
    """What `_fuse_linear_spec_into_last_linear` makes of the module: W' = C @ W, b' = C @ b on the last op."""
    from boundflow_b200.ir import BFTaskModule, BoundTask, TaskOp

    src = wl.module.get_entry_task()
    ops = [TaskOp(o.op_type, o.name, list(o.inputs), list(o.outputs), dict(o.attrs)) for o in src.ops]
    params = dict(wl.module.bindings["params"])
    last = ops[-1]
    params["spec_W"] = torch.matmul(wl.C, params[last.inputs[1]]).to(dev)
    params["spec_b"] = torch.matmul(wl.C, params[last.inputs[2]]).to(dev)
    last.inputs = [last.inputs[0], "spec_W", "spec_b"]
    last.outputs = ["spec_out"]
    task = BoundTask(task_id="t0", kind=src.kind, ops=ops, input_values=list(src.input_values), output_values=["spec_out"])
    return BFTaskModule(tasks=[task], entry_task_id="t0", bindings={"params": params})


@pytest.mark.parametrize("tag", ["c1", "c3"])
def test_matches_reference_golden(dev, golden, tag):
    from boundflow_b200 import workloads as W
    from boundflow_b200.executor import CudaTaskExecutor
    from boundflow_b200.ir import InputSpec

    g = golden("spec_fused_ibp.npz")
    wl = W.make_workload(tag) if tag == "c1" else W.make_workload(tag, batch=8)
    spec = InputSpec.box(value_name="input", lower=wl.lo.to(dev), upper=wl.up.to(dev))
    out = CudaTaskExecutor().run_ibp(_fused_module(wl, dev), spec)
    assert tuple(out.lower.shape) == tuple(g[f"{tag}_lower"].shape)
    assert_close(out.lower, g[f"{tag}_lower"], "lower")
    assert_close(out.upper, g[f"{tag}_upper"], "upper")


def test_batched_linear_entry_point_against_torch(dev):
    from boundflow_b200 import _lib

    lib = _lib.load()
    g = torch.Generator("cpu").manual_seed(3)
    B, S, n = 5, 7, 301
    l = torch.randn(B, n, generator=g) - 0.3
    u = l + torch.rand(B, n, generator=g)
    Wb = torch.randn(B, S, n, generator=g)
    bias = torch.randn(B, S, generator=g)
    s = torch.cuda.current_stream(dev).cuda_stream
    for relu_in in (0, 1):
        xl, xu = (torch.relu(l), torch.relu(u)) if relu_in else (l, u)
        mid, rad = (xl + xu) / 2, (xu - xl) / 2
        c = torch.einsum("bi,bsi->bs", mid, Wb)
        d = torch.einsum("bi,bsi->bs", rad, Wb.abs())
        for bb in (bias, None):
            ol, ou = torch.empty(B, S, device=dev), torch.empty(B, S, device=dev)
            args = [t.to(dev).contiguous() for t in (l, u, Wb)]
            bd = None if bb is None else bb.to(dev)
            _lib.check(lib.bf_ibp_linear_batched(args[0].data_ptr(), args[1].data_ptr(), relu_in, args[2].data_ptr(), _lib.ptr(bd),
                                                 ol.data_ptr(), ou.data_ptr(), B, S, n, s))
            add = 0 if bb is None else bb
            assert_close(ol, c - d + add, "lower")
            assert_close(ou, c + d + add, "upper")
