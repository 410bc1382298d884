"""Chunk attention of the 7B model, product by product (one 4096-token chunk, 4 heads, d_qk = 256 and
d_v = 2048 per head, causal, bf16), against the tensor-core roofline.

    python benchmarks/attention_bench.py [--iters 20]

CUDA events after warm-up; 256 MiB are rewritten between calls so that nothing stays in the 126 MB L2.
Every product of `_Attention` is timed on its own through the same `cuda_ops.gemm` call the op makes
(causal tile structure, soft-max epilogues), then the whole forward and backward.  FLOPs count the lower
triangle only (what the causal modes compute); the roofline is the measured sustained cuBLAS throughput.
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--only", default=None, help="substring of the product names to run (for a profiler capture)")
    args = ap.parse_args()
    import torch
    from megalodon_b200.ops import cuda_ops
    from megalodon_b200.utils.profiling import measured_peaks
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    peak = measured_peaks()["bf16_tflops_sustained"] * 1e12
    B, L, H, dk, dv = 1, args.tokens, 4, 256, 2048
    torch.manual_seed(0)
    q = (torch.randn(B, L, H, dk, device=dev) / dk ** 0.5).bfloat16()
    k = torch.randn(B, L, H, dk, device=dev).bfloat16()
    v = torch.randn(B, L, H, dv, device=dev).bfloat16()
    do = torch.randn(B, L, H, dv, device=dev).bfloat16()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed(fn, name=None):
        if args.only and (name is None or args.only not in name):
            return None
        for _ in range(3):
            fn()
        tot = 0.0
        for _ in range(args.iters):
            flush.fill_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            tot += e0.elapsed_time(e1)
        return tot / args.iters

    hv = cuda_ops._heads_view
    P = torch.empty(B, H, L, L, dtype=torch.bfloat16, device=dev)
    out = torch.empty(B, L, H, dv, dtype=torch.bfloat16, device=dev)
    rmax = torch.full((B, H, L), float("-inf"), device=dev)
    rsum = torch.zeros((B, H, L), device=dev)
    qb, kb, vb, ob, dob, Pb = hv(q, 0), hv(k, 0), hv(v, 0), hv(out, 0), hv(do, 0), P[0]
    tri = 0.5 * (1 + 1.0 / (L // 256))           # fraction of the 256 x 256 tiles on or below the diagonal
    f_qk = 2.0 * L * L * dk * H * tri
    f_pv = 2.0 * L * L * dv * H * tri
    rows = []

    def row(name, ms, flops):
        if ms is None:
            return
        rows.append({"product": name, "ms": round(ms, 4), "gflop": round(flops / 1e9, 1),
                     "tflops": round(flops / ms / 1e9, 1), "fraction_of_sustained_cublas": round(flops / (ms / 1e3) / peak, 3)})

    row("Q K^T pass 1 (row maxima only)", timed(lambda: cuda_ops.gemm(qb, kb, out=Pb, mode=1, alpha=1.0, softmax=dict(epi_kind=1, row_out=rmax[0])), "Q K^T pass 1 (row maxima only)"), f_qk)
    row("Q K^T pass 2 (exp, row sums, P written)", timed(lambda: cuda_ops.gemm(qb, kb, out=Pb, mode=1, alpha=1.0, softmax=dict(epi_kind=2, row_in=rmax[0], row_out=rsum[0])), "Q K^T pass 2 (exp, row sums, P written)"), f_qk)
    row("P V (scaled by 1 / row sum)", timed(lambda: cuda_ops.gemm(Pb, vb, b_mn=True, out=ob, mode=2, softmax=dict(epi_kind=3, row_in=rsum[0])), "P V (scaled by 1 / row sum)"), f_pv)
    dos, delta = cuda_ops._C().attn_bwd_prep(do, out, rsum)
    row("attn_bwd_prep (delta, dO / row sum)", timed(lambda: cuda_ops._C().attn_bwd_prep(do, out, rsum), "attn_bwd_prep (delta, dO / row sum)"), 0.0)
    dvb = hv(torch.empty_like(v), 0)
    dqb = hv(torch.empty_like(q), 0)
    dkb = hv(torch.empty_like(k), 0)
    row("dV = P^T dO'", timed(lambda: cuda_ops.gemm(Pb, hv(dos, 0), a_mn=True, b_mn=True, out=dvb, mode=3), "dV = P^T dO'"), f_pv)
    P2 = P.clone()
    row("dS from dO V^T (epilogue over P)", timed(lambda: cuda_ops.gemm(dob, vb, out=P2[0], mode=1, softmax=dict(epi_kind=4, row_in=rsum[0], row_in2=delta[0], aux=P2[0])), "dS from dO V^T (epilogue over P)"), f_pv)
    row("dQ = dS K", timed(lambda: cuda_ops.gemm(Pb, kb, b_mn=True, out=dqb, mode=2, alpha=1.0), "dQ = dS K"), f_qk)
    row("dK = dS^T Q", timed(lambda: cuda_ops.gemm(Pb, qb, a_mn=True, b_mn=True, out=dkb, mode=3, alpha=1.0), "dK = dS^T Q"), f_qk)

    qr, kr, vr = (t.clone().requires_grad_() for t in (q, k, v))
    row("forward (op)", timed(lambda: cuda_ops.attention(qr, kr, vr, 1.0, 0.0, True, True), "forward (op)"), 2 * f_qk + f_pv)

    def fwd_bwd():
        o = cuda_ops.attention(qr, kr, vr, 1.0, 0.0, True, True)
        o.backward(do)
        qr.grad = kr.grad = vr.grad = None
    row("forward + backward (op)", timed(fwd_bwd, "forward + backward (op)"), 4 * f_qk + 3 * f_pv)
    cuda_ops.check_kernel_errors()
    print(json.dumps({"bench": "attention", "tokens": L, "heads": H, "d_qk": dk, "d_v": dv, "dtype": "bf16",
                      "peak_tflops_sustained": peak / 1e12, "rows": rows}))
    for r in rows:
        print(f"{r['product']:44s} {r['ms']:8.4f} ms {r['gflop']:8.1f} GFLOP {r['tflops']:8.1f} TFLOP/s "
              f"{r['fraction_of_sustained_cublas']:6.3f} of sustained cuBLAS", file=sys.stderr)


if __name__ == "__main__":
    main()
