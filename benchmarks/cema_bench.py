"""Micro-benchmark of the CEMA scan kernels (forward and backward) on the
Megalodon-7B layer shape: one 4096-token chunk, 4096 features, 16 states.

    python benchmarks/cema_bench.py [--tokens 4096] [--dim 4096] [--ndim 16] [--pass fwd|bwd|both]

The op is bound by the fp32 FMA pipes, not by memory: per element and state it
costs about 10 FMAs forward and 32 backward, so the printed "FMA floor" is
elements * states * that count / (148 SMs * 128 lanes * SM clock), with the SM
clock taken from `nvidia-smi` at start.  Timing: CUDA events, 3 warm-up + 10
timed calls, a 256 MiB buffer rewritten between calls (cold L2).
"""
import argparse
import os
import subprocess
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from megalodon_b200.ops._ext import require  # noqa: E402


def time_it(fn, flush):
    for _ in range(3):
        fn()
    ts = []
    for _ in range(10):
        flush.add_(1.0)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--dim", type=int, default=4096)
    ap.add_argument("--ndim", type=int, default=16)
    ap.add_argument("--pass", dest="which", default="both", choices=["fwd", "bwd", "both"])
    args = ap.parse_args()
    ext = require()
    dev = torch.device("cuda")
    L, D, N = args.tokens, args.dim, args.ndim
    flush = torch.zeros(64 * 1024 * 1024, device=dev)
    x = torch.randn(1, L, D, device=dev).bfloat16()
    dy = torch.randn(1, L, D, device=dev).bfloat16()
    p = torch.rand(D, N, device=dev) * 0.5 + 0.1
    mag = 1.0 - p * (torch.rand(D, N, device=dev) * 0.5 + 0.1)
    q = torch.view_as_real(torch.polar(mag, torch.rand(D, N, device=dev) * 3.0)).contiguous()
    gamma = (torch.randn(D, N, 2, device=dev) * 0.25).contiguous()
    omega = torch.randn(D, device=dev)
    hx = torch.randn(1, D, N, 2, device=dev)
    dh = torch.randn(1, D, N, 2, device=dev)
    try:
        mhz = float(subprocess.check_output(["nvidia-smi", "--query-gpu=clocks.max.sm", "--format=csv,noheader,nounits",
                                             "-i", str(torch.cuda.current_device())]).decode().split()[0])
    except Exception:  # noqa: BLE001
        mhz = 1965.0
    lanes_per_s = 148 * 128 * mhz * 1e6
    elems = L * D * N
    if args.which in ("fwd", "both"):
        ms = time_it(lambda: ext.cema_fwd(x, p, q, gamma, omega, hx, True), flush)
        floor = elems * 10 / lanes_per_s * 1e3
        print(f"cema fwd  L={L} D={D} N={N}: {ms * 1e3:8.1f} us   FMA floor {floor * 1e3:7.1f} us "
              f"({floor / ms:.2f} of the floor rate at {mhz:.0f} MHz)   HBM bytes {(2 * L * D * 2 * 2) / 1e6:.0f} MB")
    if args.which in ("bwd", "both"):
        ms = time_it(lambda: ext.cema_bwd(dy, x, p, q, gamma, omega, hx, dh), flush)
        floor = elems * 32 / lanes_per_s * 1e3
        print(f"cema bwd  L={L} D={D} N={N}: {ms * 1e3:8.1f} us   FMA floor {floor * 1e3:7.1f} us "
              f"({floor / ms:.2f} of the floor rate at {mhz:.0f} MHz)")


if __name__ == "__main__":
    main()
