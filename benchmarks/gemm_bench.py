"""Micro-benchmark of the tcgen05 GEMM against torch.matmul (cuBLAS) on the
projection shapes of Megalodon-7B (4096 tokens per call).

    python benchmarks/gemm_bench.py [--tokens 4096]

Timing: CUDA events, 3 warm-up + 10 timed launches, a 256 MiB buffer is
rewritten between launches so operands come from HBM / a cold L2.
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from megalodon_b200.ops import cuda_ops  # noqa: E402


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
    ap.add_argument("--only", default=None, help="run a single projection, e.g. wv/wr (for profiler captures)")
    ap.add_argument("--no-cublas", action="store_true", help="skip the torch.matmul comparison")
    args = ap.parse_args()
    T = args.tokens
    dev = torch.device("cuda")
    flush = torch.zeros(64 * 1024 * 1024, device=dev)
    shapes = [("wz", 1024, 4096), ("wv/wr", 8192, 4096), ("wh1", 4096, 4096), ("wh2", 4096, 8192),
              ("fc1/fc3", 11264, 4096), ("fc2", 4096, 11264), ("vocab", 32000, 4096)]
    print(f"{'layer':8s} {'pass':6s} {'M':>6s} {'N':>6s} {'K':>6s} {'tcgen05 ms':>11s} {'TFLOP/s':>8s} "
          f"{'cuBLAS ms':>10s} {'TFLOP/s':>8s} {'ratio':>6s}")
    for name, n_out, k_in in shapes:
        if args.only is not None and name != args.only:
            continue
        x = torch.randn(T, k_in, device=dev).bfloat16()
        w = torch.randn(n_out, k_in, device=dev).bfloat16()
        dy = torch.randn(T, n_out, device=dev).bfloat16()
        cases = [
            ("fwd", T, n_out, k_in, lambda: cuda_ops.gemm(x, w), lambda: torch.matmul(x, w.t())),
            ("dgrad", T, k_in, n_out, lambda: cuda_ops.gemm(dy, w, b_mn=True), lambda: torch.matmul(dy, w)),
            ("wgrad", n_out, k_in, T, lambda: cuda_ops.gemm(dy, x, a_mn=True, b_mn=True),
             lambda: torch.matmul(dy.t(), x)),
        ]
        for pname, M, N, K, mine, ref in cases:
            t0 = time_it(mine, flush)
            t1 = t0 if args.no_cublas else time_it(ref, flush)
            fl = 2.0 * M * N * K / 1e9
            print(f"{name:8s} {pname:6s} {M:6d} {N:6d} {K:6d} {t0:11.3f} {fl / t0:8.1f} {t1:10.3f} {fl / t1:8.1f} "
                  f"{t1 / t0:6.2f}")
    cuda_ops.check_kernel_errors()


if __name__ == "__main__":
    main()
