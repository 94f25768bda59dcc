"""Shared checks for the parity tests."""
import os

import numpy as np
import torch

ATOL = 1e-4   # absolute tolerance on every bound
RTOL = 1e-5   # relative tolerance on every bound


def close(got, ref, atol=ATOL, rtol=RTOL):
    got = torch.as_tensor(np.asarray(got.detach().cpu() if torch.is_tensor(got) else got), dtype=torch.float64)
    ref = torch.as_tensor(np.asarray(ref.detach().cpu() if torch.is_tensor(ref) else ref), dtype=torch.float64)
    err = (got - ref).abs()
    tol = atol + rtol * ref.abs()
    return bool((err <= tol).all()), float((err - tol).max()), float(err.max())


def assert_close(got, ref, what="", atol=ATOL, rtol=RTOL):
    ok, excess, worst = close(got, ref, atol, rtol)
    report = os.environ.get("BF_TOLERANCE_REPORT")
    if report and (atol != ATOL or rtol != RTOL):
        # measurement aid: how far a comparison with a widened tolerance is from the strict one
        g64 = torch.as_tensor(np.asarray(got.detach().cpu() if torch.is_tensor(got) else got), dtype=torch.float64)
        r64 = torch.as_tensor(np.asarray(ref.detach().cpu() if torch.is_tensor(ref) else ref), dtype=torch.float64)
        ratio = float(((g64 - r64).abs() / (ATOL + RTOL * r64.abs())).max())
        with open(report, "a") as fh:
            fh.write(f"{os.environ.get('PYTEST_CURRENT_TEST', '?')} | {what} | atol={atol:g} rtol={rtol:g} | err/strict={ratio:.3f}\n")
    assert ok, f"{what}: max |err| {worst:.3e}, exceeds atol {atol} + rtol {rtol}*|ref| by {excess:.3e}"


def checksum(*tensors):
    return np.array([float(t.double().sum()) for t in tensors] + [float(t.double().abs().sum()) for t in tensors])


def workload_checksum(wl):
    return checksum(wl.x, wl.C, *[p for p in wl.module.bindings["params"].values()])
