"""The peer-memory collectives in isolation (no GEMM running beside them), against NCCL.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        benchmarks/collective_bench.py [--mib 512]

Timed with CUDA events after warm-up, max over ranks, buffers larger than L2:
    reduce-scatter   SymmetricReduceScatter (stage copy + flag barrier + pull / sum / scale / cast / sum of
                     squares in one kernel)            vs  dist.reduce_scatter_tensor
    all-gather       gather_pull_kernel (pull into the natural layout)   vs  dist.all_gather_into_tensor
    all-reduce       SymmetricAllReduce (copy-in, reduce + sum of squares + push, copy-out)  vs  dist.all_reduce
    hand-off         PeerMailbox send + receive of one 512.5 KiB state along the line, per hop
Bandwidths are bytes that must cross NVLink per GPU and direction, (N - 1) / N of the buffer, over the time,
and their fraction of the measured 770 GB/s per direction.
"""
import argparse
import json
import os
import sys

os.environ.setdefault("CUDA_MODULE_LOADING", "EAGER")
os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "32")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
LINK_GBS = 770.0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mib", type=int, default=512, help="size of the full (unsharded) bf16 buffer")
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    import torch
    import torch.distributed as dist
    from megalodon_b200.ops._ext import require
    from megalodon_b200.parallel import init_torch_distributed
    from megalodon_b200.parallel.symm import (AbortRecord, PeerMailbox, SymmetricAllReduce, SymmetricReduceScatter,
                                              SymmetricRegion)
    ext = require()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    assert world > 1
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    rank = init_torch_distributed(timeout=300).global_rank
    dev = torch.device("cuda", local)
    abort = AbortRecord.get(dev)
    n = (args.mib << 20) // 2
    n -= n % (world * 64)
    shard_n = n // world
    cross = n * 2 * (world - 1) / world            # bytes per GPU and direction

    def timed(fn, iters=args.iters):
        for _ in range(3):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def row(name, ms, nbytes):
        gbs = nbytes / (ms / 1e3) / 1e9
        return {"op": name, "ms": round(ms, 4), "gb_per_s": round(gbs, 1), "fraction_of_link": round(gbs / LINK_GBS, 3)}

    out = []
    grad = torch.randn(n, device=dev).bfloat16()
    shard = torch.empty(shard_n, device=dev, dtype=torch.bfloat16)
    sumsq = torch.zeros((), device=dev, dtype=torch.float64)
    rs = SymmetricReduceScatter(None, dev, n, torch.bfloat16, timeout_s=10.0)
    out.append(row("reduce-scatter, peer memory (copy + barrier + fused kernel)",
                   timed(lambda: rs.reduce_scatter(grad, shard, 1.0 / world, sumsq)), cross))
    out.append(row("reduce-scatter, NCCL", timed(lambda: dist.reduce_scatter_tensor(shard, grad)), cross))

    region = SymmetricRegion(shard_n * 2 + 256, None, dev)
    mine = region.view(0, shard_n * 2, torch.bfloat16)
    mine.copy_(torch.randn(shard_n, device=dev).bfloat16())
    full = torch.empty(n, device=dev, dtype=torch.bfloat16)
    ptrs = region.ptr_table_at(0).contiguous()
    table = torch.tensor([[0, shard_n, 0]], dtype=torch.int64, device=dev)
    torch.cuda.synchronize()
    dist.barrier()
    out.append(row("all-gather, pull kernel", timed(lambda: ext.gather_pull(full, ptrs, table, n, abort.dev, shard_n)), cross))
    out.append(row("all-gather, NCCL", timed(lambda: dist.all_gather_into_tensor(full, mine)), cross))

    bucket = 256 << 20
    ar_region = SymmetricRegion(SymmetricAllReduce.bytes_needed(bucket, world), None, dev)
    ar = SymmetricAllReduce(ar_region, bucket, timeout_s=10.0)
    buf = torch.randn(n, device=dev).bfloat16()
    out.append(row("all-reduce + sum of squares, peer memory (copy-in, kernel, copy-out)",
                   timed(lambda: ar.all_reduce_([buf], sumsq=sumsq, scale=1.0 / world), iters=5), 2 * cross))
    out.append(row("all-reduce, NCCL", timed(lambda: dist.all_reduce(buf), iters=5), 2 * cross))

    # hand-off along the line: every rank but the first receives, every rank but the last sends
    slot = (2 * 64 + 2 * 4096 * 16) * 4
    mregion = SymmetricRegion(PeerMailbox.bytes_needed(slot, 8), None, dev)
    box = PeerMailbox(mregion, rank - 1 if rank > 0 else None, rank + 1 if rank + 1 < world else None, slot,
                      n_slots=8, timeout_s=10.0)
    state = torch.randn(slot // 4, device=dev)

    def handoff():
        if rank > 0:
            box.recv(state, "fwd")
        if rank + 1 < world:
            box.send(state, "fwd")
    ms = timed(handoff, iters=50)
    out.append({"op": "state hand-off along the line (512.5 KiB per hop)", "ms_per_round": round(ms, 4),
                "us_per_hop": round(ms * 1e3 / (world - 1), 2)})
    torch.cuda.synchronize()
    abort.check()
    if rank == 0:
        print(json.dumps({"bench": "collectives", "n_gpus": world, "buffer_mib": args.mib, "link_gbs": LINK_GBS, "rows": out}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
