"""The parameter all-gather fused into the consuming GEMM, measured on its own.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        benchmarks/gather_gemm_bench.py [--tokens 4096]

For each forward projection of the 7B block (weight [N, K] row-sharded over the N ranks, activations
[tokens, K] local) four ways to get y = x w^T are timed, CUDA events after warm-up, max over ranks:

    gemm only            the weight already complete in local memory (what the fused kernel must approach)
    fused                copy warps of the GEMM pull the row blocks from their owners while it computes
    pull, then gemm      stand-alone pull kernel over peer memory, then the plain GEMM
    NCCL, then gemm      all_gather_into_tensor, then the plain GEMM (what the reference's FSDP does)

    python benchmarks/gather_gemm_bench.py --local 8 [--only wv] [--iters 3]

runs the fused kernel alone on ONE GPU with the 8 "ranks" as local buffers (no link traffic): the form a
profiler can capture (one process, one kernel, a few launches).

The fused kernel's roofline fraction is printed: the target time is the slower of FLOPs over the
measured cuBLAS throughput and remote bytes over the measured per-direction link bandwidth (770 GB/s).
The weight is re-sharded between iterations only logically: every iteration pulls the same shards again,
so the remote bytes are real each time; the operands of one projection (weight + activations + output)
exceed what stays resident across the other projections' iterations in the 126 MB L2.
"""
import argparse
import json
import os
import sys

os.environ.setdefault("CUDA_MODULE_LOADING", "EAGER")
os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "32")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

SHAPES = [("wz", 1024, 4096), ("wv", 8192, 4096), ("wr", 8192, 4096), ("wh1", 4096, 4096), ("wh2", 4096, 8192),
          ("fc1", 11264, 4096), ("fc2", 4096, 11264)]
LINK_GBS = 770.0


def local_mode(args):
    import torch
    from megalodon_b200.ops import cuda_ops
    from megalodon_b200.ops._ext import require
    ext = require()
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    world, M = args.local, args.tokens
    out = []
    for name, N, K in SHAPES:
        if (args.only and name != args.only) or not ext.gemm_gather_supported(M, N, K, world):
            continue
        w = (torch.randn(N, K, device=dev) / K ** 0.5).bfloat16()
        blocks = [w[r * (N // world):(r + 1) * (N // world)].clone() for r in range(world)]
        x = torch.randn(M, K, device=dev).bfloat16()
        full = torch.empty(N, K, device=dev, dtype=torch.bfloat16)
        ptrs = [b.data_ptr() for b in blocks]

        def run():
            return cuda_ops.gemm(x, full, b_gather=(ptrs, 1))[0]
        for _ in range(2):
            run()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.iters):
            y = run()
        e1.record()
        torch.cuda.synchronize()
        plain0, plain1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        plain0.record()
        for _ in range(args.iters):
            ref = cuda_ops.gemm(x, w)[0]
        plain1.record()
        torch.cuda.synchronize()
        out.append({"weight": name, "N": N, "K": K, "fused_local_ms": round(e0.elapsed_time(e1) / args.iters, 4),
                    "gemm_only_ms": round(plain0.elapsed_time(plain1) / args.iters, 4),
                    "max_abs_diff": (y.float() - ref.float()).abs().max().item()})
    cuda_ops.check_kernel_errors()
    print(json.dumps({"bench": "gather_gemm_local", "ranks_emulated": world, "tokens": M, "rows": out}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--local", type=int, default=0, help="emulate this many ranks with local buffers on one GPU")
    ap.add_argument("--only", default=None, help="one projection by name (wz, wv, wr, wh1, wh2, fc1, fc2)")
    args = ap.parse_args()
    if args.local:
        return local_mode(args)
    import torch
    import torch.distributed as dist
    from megalodon_b200.ops import cuda_ops
    from megalodon_b200.ops._ext import require
    from megalodon_b200.parallel import init_torch_distributed
    from megalodon_b200.parallel.symm import AbortRecord, SymmetricRegion
    from megalodon_b200.utils.profiling import measured_peaks
    ext = require()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    assert world > 1, "launch with torchrun on 2 or more GPUs"
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    rank = init_torch_distributed(timeout=300).global_rank
    dev = torch.device("cuda", local)
    peak = measured_peaks()["bf16_tflops_sustained"] * 1e12
    M = args.tokens
    biggest = max(n * k for _, n, k in SHAPES) // world
    region = SymmetricRegion(biggest * 2 + 256, None, dev)
    abort = AbortRecord.get(dev)
    rows_out = []

    def timed(fn):
        for _ in range(3):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / args.iters], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for name, N, K in SHAPES:
        if not ext.gemm_gather_supported(M, N, K, world):
            continue
        torch.manual_seed(rank)
        shard = region.view(0, (N // world) * K * 2, torch.bfloat16).view(N // world, K)
        shard.copy_((torch.randn(N // world, K, device=dev) / K ** 0.5).bfloat16())
        x = torch.randn(M, K, device=dev).bfloat16()
        full = torch.empty(N, K, device=dev, dtype=torch.bfloat16)
        ptrs = [region.peer_ptr(r, 0) for r in range(world)]
        ptr_t = torch.tensor(ptrs, dtype=torch.int64, device=dev)
        table = torch.tensor([[0, (N // world) * K, 0]], dtype=torch.int64, device=dev)
        torch.cuda.synchronize()
        dist.barrier()
        ms_nccl = timed(lambda: (dist.all_gather_into_tensor(full.view(-1), shard.reshape(-1)), cuda_ops.gemm(x, full)))
        ref = cuda_ops.gemm(x, full)[0].float()
        ms_plain = timed(lambda: cuda_ops.gemm(x, full))
        ms_pull = timed(lambda: (ext.gather_pull(full, ptr_t, table, N * K, abort.dev, (N // world) * K),
                                 cuda_ops.gemm(x, full)))
        full.fill_(float("nan"))
        ms_fused = timed(lambda: cuda_ops.gemm(x, full, b_gather=(ptrs, rank)))
        err = (cuda_ops.gemm(x, full, b_gather=(ptrs, rank))[0].float() - ref).abs().max().item()
        flops = 2.0 * M * N * K
        remote = N * K * 2 * (world - 1) / world
        target_ms = max(flops / peak, remote / (LINK_GBS * 1e9)) * 1e3
        rows_out.append({"weight": name, "N": N, "K": K, "gemm_only_ms": round(ms_plain, 4), "fused_ms": round(ms_fused, 4),
                         "pull_then_gemm_ms": round(ms_pull, 4), "nccl_then_gemm_ms": round(ms_nccl, 4),
                         "roofline_target_ms": round(target_ms, 4), "fused_fraction_of_roofline": round(target_ms / ms_fused, 3),
                         "bound": "compute" if flops / peak > remote / (LINK_GBS * 1e9) else "link",
                         "max_abs_diff_vs_plain": err})
        torch.cuda.synchronize()
        dist.barrier()
    cuda_ops.check_kernel_errors()
    abort.check()
    if rank == 0:
        print(json.dumps({"bench": "gather_gemm", "n_gpus": world, "tokens": M, "dtype": "bf16",
                          "peaks": {"bf16_tflops_sustained": peak / 1e12, "link_gbs": LINK_GBS}, "rows": rows_out}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
