"""IBP and CROWN on graphs that are not chains (residual add, fan-out), against the reference's outputs."""
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


@pytest.mark.parametrize("name", ["residual_s1", "residual_s2", "fanout_mlp", "mini_resnet", "concat_cnn", "concat_mlp"])
def test_graph_matches_reference_golden(dev, golden, name):
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import needs_graph_path, run_crown_ibp_mlp
    from boundflow_b200.executor import CudaTaskExecutor
    from boundflow_b200.ir import InputSpec

    g = golden("graph_cases.npz")
    module, _x, lo, up, C = W.make_graph_cases()[name]
    assert needs_graph_path(module)
    spec = InputSpec.box(value_name="input", lower=lo.to(dev), upper=up.to(dev))
    ibp = CudaTaskExecutor().run_ibp(module, spec)
    assert_close(ibp.lower, g[f"{name}_ibp_lower"], "ibp lower")
    assert_close(ibp.upper, g[f"{name}_ibp_upper"], "ibp upper")
    crown = run_crown_ibp_mlp(module, spec, linear_spec_C=None if C is None else C.to(dev))
    assert_close(crown.lower, g[f"{name}_crown_lower"], "crown lower")
    assert_close(crown.upper, g[f"{name}_crown_upper"], "crown upper")
    # CROWN is never looser than IBP here by more than rounding, and the bounds are ordered
    assert bool((crown.lower <= crown.upper + 1e-5).all())


def test_chain_modules_keep_the_fused_path_and_unsupported_inputs_are_refused(dev):
    from boundflow_b200 import workloads as W
    from boundflow_b200.crown import needs_graph_path, run_crown_ibp_mlp
    from boundflow_b200.ir import InputSpec

    assert not needs_graph_path(W.make_workload("c1").module)
    assert not needs_graph_path(W.make_workload("c2", batch=1).module)
    module, _x, lo, up, _C = W.make_graph_cases()["fanout_mlp"]
    spec = InputSpec.box(value_name="input", lower=lo.to(dev), upper=up.to(dev))
    with pytest.raises(NotImplementedError):
        run_crown_ibp_mlp(module, spec, relu_split_state={"h": torch.zeros(5, 24, dtype=torch.int8, device=dev)})


def test_building_blocks_against_torch(dev):
    """bf_crown_relu_bwd (incl. rows wider than one chunk) and bf_accumulate."""
    from boundflow_b200 import _lib

    lib = _lib.load()
    g = torch.Generator("cpu").manual_seed(11)
    s = torch.cuda.current_stream(dev).cuda_stream
    for B, S, n in ((3, 5, 37), (2, 3, 9001)):
        A = torch.randn(B, S, n, generator=g)
        au, al, bu = (torch.rand(B, n, generator=g) for _ in range(3))
        bl = torch.zeros(B, n)
        d0 = torch.randn(B, S, generator=g)
        Ad, aud, ald, bud, bld = (t.to(dev).contiguous() for t in (A, au, al, bu, bl))
        nb = int(lib.bf_crown_relu_bwd_scratch_bytes(B, S, n))
        scratch = torch.empty(max(nb, 16), dtype=torch.uint8, device=dev)
        for side in (0, 1):
            pos = A >= 0
            if side == 0:
                slope, icpt = torch.where(pos, al.unsqueeze(1), au.unsqueeze(1)), torch.where(pos, bl.unsqueeze(1), bu.unsqueeze(1))
            else:
                slope, icpt = torch.where(pos, au.unsqueeze(1), al.unsqueeze(1)), torch.where(pos, bu.unsqueeze(1), bl.unsqueeze(1))
            out, dd = torch.empty(B, S, n, device=dev), d0.to(dev).clone()
            _lib.check(lib.bf_crown_relu_bwd(Ad.data_ptr(), side, aud.data_ptr(), ald.data_ptr(), bud.data_ptr(), bld.data_ptr(), out.data_ptr(),
                                             dd.data_ptr(), 1, scratch.data_ptr(), scratch.numel(), B, S, n, s))
            assert_close(out, A * slope, f"A_prev side {side}")
            assert_close(dd, d0 + (A * icpt).sum(dim=2), f"delta side {side}", rtol=1e-4)
    x, y = torch.randn(1000, generator=g), torch.randn(1000, generator=g)
    xd = x.to(dev)
    _lib.check(lib.bf_accumulate(xd.data_ptr(), y.to(dev).data_ptr(), 1000, s))
    assert_close(xd, x + y, "accumulate")
