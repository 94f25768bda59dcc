"""Layer-level timing of the fused ReLU + Conv2d backward (`bf_crown_relu_conv2d_bwd`).

    python -m boundflow_b200.convbench [--rows 2048] [--layers c5conv2T,c5conv3T] [--reps 10]

Times one call per layer shape (ReLU scaling pass + transposed convolution, one side) with
CUDA events and prints multiply-accumulates per second; the shapes are the transposed
convolutions of the MNIST- and CIFAR-shaped CNN workloads (`workloads.py`, c2 and c5).
"""
from __future__ import annotations

import argparse

import torch

from . import _lib

# name: (Co, Ho, Wo, Ci, Hi, Wi, kernel, stride, padding) of the forward layer whose transpose is applied
LAYERS = {
    "c5conv2T": (32, 16, 16, 32, 32, 32, 4, 2, 1),
    "c5conv3T": (64, 16, 16, 32, 16, 16, 3, 1, 1),
    "c5conv4T": (64, 8, 8, 64, 16, 16, 4, 2, 1),
    "c5conv1T": (32, 32, 32, 3, 32, 32, 3, 1, 1),
    "c2conv2T": (32, 7, 7, 16, 14, 14, 4, 2, 1),
    "c2conv1T": (16, 14, 14, 1, 28, 28, 4, 2, 1),
}


def time_layer(name: str, rows: int, reps: int, dev: torch.device) -> dict:
    lib = _lib.load()
    Co, Ho, Wo, Ci, Hi, Wi, k, st, pd = LAYERS[name]
    S = 8
    B = max(1, rows // S)
    M = B * S
    g = torch.Generator("cpu").manual_seed(7)
    n = Co * Ho * Wo
    A = torch.randn(B, S, n, generator=g).to(dev)
    au, al, bu = (torch.rand(B, n, generator=g).to(dev) for _ in range(3))
    bl = torch.zeros(B, n, device=dev)
    W = torch.randn(Co, Ci, k, k, generator=g).to(dev)
    bias = torch.randn(Co, generator=g).to(dev)
    out = torch.empty(B, S, Ci * Hi * Wi, device=dev)
    delta = torch.empty(B, S, device=dev)
    nbytes = int(lib.bf_crown_relu_conv2d_bwd_scratch_bytes(B, S, Co, Ho, Wo))
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream

    def run() -> None:
        _lib.check(lib.bf_crown_relu_conv2d_bwd(
            A.data_ptr(), _lib.SIDE_LOWER, au.data_ptr(), al.data_ptr(), bu.data_ptr(), bl.data_ptr(), W.data_ptr(), bias.data_ptr(),
            out.data_ptr(), delta.data_ptr(), 0, scratch.data_ptr(), nbytes, B, S, Ci, Hi, Wi, Co, Ho, Wo, k, k, st, st, pd, pd, stream))

    for _ in range(3):
        run()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        run()
    e1.record()
    torch.cuda.synchronize(dev)
    ms = e0.elapsed_time(e1) / reps
    macs = M * n * Ci * k * k
    return {"layer": name, "rows": M, "ms": ms, "tmac_per_s": macs / ms / 1e9}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=2048)
    ap.add_argument("--layers", default=",".join(LAYERS))
    ap.add_argument("--reps", type=int, default=10)
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("convbench needs a CUDA device")
    dev = torch.device("cuda", 0)
    for name in args.layers.split(","):
        r = time_layer(name, args.rows, args.reps, dev)
        print(f"{r['layer']:10s} rows={r['rows']} {r['ms']:8.3f} ms  {r['tmac_per_s']:7.2f} TMAC/s", flush=True)


if __name__ == "__main__":
    main()
