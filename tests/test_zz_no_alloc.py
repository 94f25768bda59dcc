"""The allocation-free conv backward entry point against the caller-scratch one.

Collected last on purpose (file name), so that a run that stops at the first failure has
already exercised everything else.  The entry point serves callers that cannot allocate
device memory when they call (device pools frozen after start-up, plugins inside a process
that owns all device memory, runtimes that forbid cudaMalloc on the request path); its scratch is a 16 MiB array inside the library,
shared by all calls and never cleared, so the second call below deliberately uses different
inputs and a smaller problem: stale contents of the first call must not leak into it."""
import pytest
import torch

from tests.helpers import assert_close

pytestmark = pytest.mark.gpu


def _case(seed, D, S, Co, Ho, Ci, k, st, pd, dev):
    from oracle import crown_oracle as O

    g = torch.Generator("cpu").manual_seed(seed)
    Hi = (Ho - 1) * st - 2 * pd + k
    A = torch.randn(D, S, Co * Ho * Ho, generator=g)
    l = torch.randn(D, Co * Ho * Ho, generator=g) - 0.2
    u = l + torch.rand(D, Co * Ho * Ho, generator=g) * 2.0
    au, bu, al, _ = O.relu_relax(l, u)
    W = torch.randn(Co, Ci, k, k, generator=g)
    b = torch.randn(Co, generator=g)
    t = lambda x: x.to(dev).contiguous()
    return dict(A=t(A), au=t(au), bu=t(bu), al=t(al), W=t(W), b=t(b), D=D, S=S, Co=Co, Ho=Ho, Ci=Ci, Hi=Hi, k=k, st=st, pd=pd)


def _run(lib, _lib, c, dev, noalloc, side):
    A_prev = torch.full((c["D"], c["S"], c["Ci"] * c["Hi"] * c["Hi"]), float("nan"), device=dev)
    delta = torch.full((c["D"], c["S"]), float("nan"), device=dev)
    geom = (c["D"], c["S"], c["Ci"], c["Hi"], c["Hi"], c["Co"], c["Ho"], c["Ho"], c["k"], c["k"], c["st"], c["st"], c["pd"], c["pd"])
    stream = torch.cuda.current_stream().cuda_stream
    head = (c["A"].data_ptr(), side, c["au"].data_ptr(), c["al"].data_ptr(), c["bu"].data_ptr(), None, c["W"].data_ptr(), c["b"].data_ptr(),
            A_prev.data_ptr(), delta.data_ptr(), 0)
    if noalloc:
        _lib.check(lib.bf_crown_relu_conv2d_bwd_noalloc(*head, *geom, stream))
    else:
        nbytes = int(lib.bf_crown_relu_conv2d_bwd_scratch_bytes(c["D"], c["S"], c["Co"], c["Ho"], c["Ho"]))
        scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        _lib.check(lib.bf_crown_relu_conv2d_bwd(*head, scratch.data_ptr(), nbytes, *geom, stream))
    torch.cuda.synchronize()
    return A_prev, delta


def test_noalloc_conv_backward_matches_scratch_variant_twice():
    assert torch.cuda.is_available()
    from boundflow_b200.csrc import build

    build.build()
    from boundflow_b200 import _lib

    lib = _lib.load()
    dev = torch.device("cuda", 0)
    assert lib.bf_crown_relu_conv2d_bwd_noalloc_max_bytes() == 16 * 1024 * 1024
    first = _case(1, 6, 9, 16, 7, 8, 4, 2, 1, dev)     # 6*9*16*49 floats of scratch
    second = _case(2, 3, 5, 6, 5, 3, 3, 1, 1, dev)     # smaller: reuses the front of the same array
    for case in (first, second):
        for side in (_lib.SIDE_LOWER, _lib.SIDE_UPPER):
            ref_A, ref_d = _run(lib, _lib, case, dev, noalloc=False, side=side)
            got_A, got_d = _run(lib, _lib, case, dev, noalloc=True, side=side)
            assert torch.isfinite(got_A).all() and torch.isfinite(got_d).all()
            assert_close(got_A, ref_A, "A_prev")
            assert_close(got_d, ref_d, "delta")
            assert torch.equal(got_A, ref_A) and torch.equal(got_d, ref_d)  # same kernels, same order: bit-equal
            # and against the CPU oracle, so that this file stands on its own: ReLU backward of this side's rows
            # (crown_ibp.py:1262-1298) followed by the transposed convolution and its bias term (crown_ibp.py:1106-1173)
            from oracle import crown_oracle as O

            c = case
            A, au, bu, al = (c[k].cpu() for k in ("A", "au", "bu", "al"))
            zero_b, zeros = torch.zeros(c["D"], c["S"]), torch.zeros_like(bu)
            A_u, A_l, b_u, b_l = O.relu_backward(A, A, zero_b, zero_b, au, bu, al, zeros)
            lam, icpt = (A_l, b_l) if side == _lib.SIDE_LOWER else (A_u, b_u)
            want_A, want_d = O.conv2d_backward(lam, icpt, c["W"].cpu(), c["b"].cpu(), (c["st"], c["st"]), (c["pd"], c["pd"]),
                                               (c["Ci"], c["Hi"], c["Hi"]), (c["Co"], c["Ho"], c["Ho"]))
            assert_close(got_A, want_A, "A_prev vs oracle")
            assert_close(got_d, want_d, "delta vs oracle")


def test_noalloc_rejects_oversized_requests():
    from boundflow_b200.csrc import build

    build.build()
    from boundflow_b200 import _lib

    lib = _lib.load()
    x = torch.zeros(8, device="cuda")
    # 4096 * 9 * 64 * 16 * 16 floats = 2.4 GB of scratch: far beyond the built-in 16 MiB
    rc = lib.bf_crown_relu_conv2d_bwd_noalloc(x.data_ptr(), 0, x.data_ptr(), x.data_ptr(), x.data_ptr(), None, x.data_ptr(), None,
                                              x.data_ptr(), x.data_ptr(), 0, 4096, 9, 32, 32, 32, 64, 16, 16, 4, 4, 2, 2, 1, 1, None)
    assert rc == _lib.BF_E_WORKSPACE
    assert b"exceeds the built-in scratch" in lib.bf_last_error_string()
