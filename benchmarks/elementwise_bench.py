"""Bandwidth check of the memory-bound kernels on Megalodon-7B shapes (4096 tokens x 4096 features,
64 norm groups, SwiGLU width 11264, 4 heads x 4096 x 4096 attention scores).

    python benchmarks/elementwise_bench.py

For each op: time (CUDA events, 3 warm-up + 10 timed calls, a 256 MiB buffer rewritten between
calls so inputs come from HBM), algorithmic bytes, and achieved bytes/s as a fraction of the measured
copy bandwidth in MEASURED_PEAKS.json (fallback 6.65 TB/s if the file is absent).
"""
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from megalodon_b200.ops import cuda_ops  # noqa: E402


def peak_gbs():
    try:
        return float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"]), "measured"
    except Exception:  # noqa: BLE001
        return 6650.0, "fallback"


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
    dev = torch.device("cuda")
    peak, kind = peak_gbs()
    flush = torch.zeros(64 * 1024 * 1024, device=dev)
    T, D, G, F = 4096, 4096, 64, 11264
    bf = torch.bfloat16
    x = torch.randn(1, T, D, device=dev).to(bf)
    g = torch.randn(1, T, D, device=dev).to(bf)
    w = torch.zeros(D, device=dev, dtype=bf)
    b = torch.zeros(D, device=dev, dtype=bf)
    rows = []

    def add(name, fn, nbytes):
        ms = time_it(fn, flush)
        rows.append((name, ms * 1e3, nbytes / 1e6, nbytes / (ms * 1e-3) / 1e9))

    ext = cuda_ops._C()
    e2 = 2 * T * D          # bytes of one bf16 activation
    y, rstd = ext.rms_norm_fwd(x, w, 1.0, 1e-5)
    add("rms_norm fwd", lambda: ext.rms_norm_fwd(x, w, 1.0, 1e-5), 2 * e2)
    add("rms_norm bwd (+dw)", lambda: ext.rms_norm_bwd(g, x, w, 1.0, rstd), 3 * e2)
    add("rms_norm bwd (no dw)", lambda: ext.rms_norm_bwd(g, x, None, 1.0, rstd), 3 * e2)
    yl, mean, rstdl = ext.layer_norm_fwd(x, w, b, 1.0, 1e-5)
    add("layer_norm fwd", lambda: ext.layer_norm_fwd(x, w, b, 1.0, 1e-5), 2 * e2)
    add("layer_norm bwd", lambda: ext.layer_norm_bwd(g, x, w, 1.0, mean, rstdl), 3 * e2)
    cnt = torch.zeros(1, dtype=torch.long, device=dev)
    pm = torch.zeros(1, G, device=dev).to(bf)
    pv = torch.ones(1, G, device=dev).to(bf)
    xs = x.clone().requires_grad_()
    add("timestep_norm fwd", lambda: cuda_ops.timestep_norm(x, cnt, pm, pv, w, b, None, G, 1e-5), 3 * e2)
    out = cuda_ops.timestep_norm(xs, cnt, pm, pv, w.clone().requires_grad_(), b.clone().requires_grad_(), None, G, 1e-5)
    add("timestep_norm bwd", lambda: torch.autograd.grad(out[0], xs, g, retain_graph=True), 5 * e2)
    a1 = torch.randn(T, F, device=dev).to(bf)
    a2 = torch.randn(T, F, device=dev).to(bf)
    g3 = torch.randn(T, F, device=dev).to(bf)
    ef = 2 * T * F
    add("swiglu fwd", lambda: ext.swiglu_fwd(a1, a2), 3 * ef)
    add("swiglu bwd", lambda: ext.swiglu_bwd(g3, a1, a2), 5 * ef)
    s = torch.randn(4, T, T, device=dev).to(bf)
    es = 2 * 4 * T * T
    add("causal softmax fwd (in place)", lambda: ext.attn_softmax_fwd(s, T, T, True, 0.0, 0, 0), es)   # reads + writes the lower triangle
    ds = torch.randn(4, T, T, device=dev).to(bf)
    add("causal softmax bwd (in place)", lambda: ext.attn_softmax_bwd(s, ds, T, T, True), es * 3 // 2)
    print(f"{'op':32s} {'us':>9s} {'MB':>9s} {'GB/s':>9s}  of {kind} {peak:.0f} GB/s")
    for name, us, mb, gbs in rows:
        print(f"{name:32s} {us:9.1f} {mb:9.1f} {gbs:9.0f}  {gbs / peak:5.2f}")


if __name__ == "__main__":
    main()
