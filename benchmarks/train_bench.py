"""Training-step benchmark for the parallel layouts other than the headline one.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        benchmarks/train_bench.py --mp M --cp C [--seq-len S] [--micro-batch B] [--model mega7B_32k]

data parallel size = N / (M * C).  Presets for the configurations of the 7B study:
    FSDP only:             --mp 1 --cp 1 --seq-len 4096 --micro-batch 4       (8 GPUs in the study)
    tensor x data:         --mp 4 --cp 1 --seq-len 8192 --micro-batch 2       (mp 4 x dp 2)
Tensor-parallel linears run through the fused all-gather->GEMM / GEMM->reduce-scatter kernels, chunk
parallelism through the peer mailbox, gradients through the peer-memory reduce-scatter, parameters
through the gathering GEMM.

`--composition library` runs the same model and step as a composition of library calls instead: cuBLAS
for every matrix product, matmul + softmax attention with the scores materialised, NCCL send/recv for
the chunk hand-off, NCCL all-gather / reduce-scatter for FSDP and the tensor-parallel collectives.  That
is the sequence of calls the reference issues (README.md:138-150, model/mega.py:251-262,
modules/chunk_parallel/mappings.py:25-89), run inside THIS framework - it is not the reference, whose
own kernels for CEMA, TimestepNorm and the norms cannot be built here.  It gives the fused paths a
number to beat besides a roofline.  Timing as in
bench.py: W warm-up steps, K timed steps between barrier + synchronize, CUDA events, max over ranks;
synthetic tokens, random-init weights.  Rank 0 prints one JSON line.
"""
import argparse
import dataclasses
import json
import os
import sys

os.environ.setdefault("CUDA_MODULE_LOADING", "EAGER")
os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "32")    # one hardware queue per stream in use
# growable segments: the step allocates 154 GB of 180; fixed-size segments left 17 GB reserved but unusable
os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mp", type=int, default=1)
    ap.add_argument("--cp", type=int, default=1)
    ap.add_argument("--seq-len", type=int, default=4096)
    ap.add_argument("--micro-batch", type=int, default=4, help="sequences per data-parallel rank")
    ap.add_argument("--model", default="mega7B_32k")
    ap.add_argument("--layers", type=int, default=None, help="debug: fewer layers (not a valid result)")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--ckpt", type=int, default=1, help="layer-wise activation checkpointing (1/0)")
    ap.add_argument("--reshard", type=int, default=0, help="free gathered parameters after forward (ZeRO-3 memory)")
    ap.add_argument("--no-fused-tp", action="store_true")
    ap.add_argument("--composition", default="fused", choices=["fused", "library"],
                    help="fused: this framework's kernels and peer-memory collectives; library: cuBLAS + NCCL + "
                         "materialised attention (context baseline, see the module docstring)")
    ap.add_argument("--step-timeout-s", type=float, default=150.0)
    args = ap.parse_args()

    import torch
    import torch.distributed as dist
    from megalodon_b200.config import OptimConf
    from megalodon_b200.models.mega import ModelStore, build_model
    from megalodon_b200.optim import build_optimizer
    from megalodon_b200.ops import cuda_ops
    from megalodon_b200.parallel import init_torch_distributed, initialize_model_parallel
    from megalodon_b200.parallel.initialize import get_data_parallel_rank, get_data_parallel_world_size
    from megalodon_b200.utils import clip_grad_norm_, set_random_seed

    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    rank = 0
    if world > 1:
        rank = init_torch_distributed(timeout=300).global_rank
    assert world % (args.mp * args.cp) == 0
    if world > 1:
        initialize_model_parallel(args.mp, args.cp)
    dp = get_data_parallel_world_size() if world > 1 else 1
    dp_rank = get_data_parallel_rank() if world > 1 else 0

    cfg = dataclasses.replace(ModelStore[args.model])
    if args.layers is not None:
        cfg.num_layers = args.layers
    cfg.layerwise_ckpt = bool(args.ckpt)
    library = args.composition == "library"
    if library:
        cuda_ops.set_gemm_backend("cublas")
        cfg.efficient_attn = None
    set_random_seed(1234)
    model = build_model(cfg, "bf16", fp32_reduce_scatter=False, reshard_after_forward=bool(args.reshard),
                        shard_over_chunk_group=args.cp > 1)
    model.defer_grad_clip = True
    local_len = args.seq_len // args.cp
    abort_record = None
    if library:
        pass                                  # NCCL hand-off, NCCL FSDP and tensor-parallel collectives
    elif args.cp > 1:
        from megalodon_b200.parallel.symm import enable_peer_transport
        enable_peer_transport(model, max_batch=args.micro_batch, n_slots=8, timeout_s=10.0)
    elif world > 1 and dp > 1:
        from megalodon_b200.parallel.symm import enable_peer_gather, enable_peer_reduce_scatter
        enable_peer_reduce_scatter(model, timeout_s=10.0)
        enable_peer_gather(model, timeout_s=10.0)
    if args.mp > 1 and not args.no_fused_tp and not library:
        from megalodon_b200.parallel.tp_comm import enable_tp_fused
        enable_tp_fused(model, max_tokens=args.micro_batch * local_len)
    if world > 1 and not library:
        from megalodon_b200.parallel.symm import AbortRecord
        abort_record = AbortRecord.get(torch.device("cuda", local_rank))
    from bench import StepWatchdog
    dog = StepWatchdog(rank, args.step_timeout_s, abort_record)
    opt, sched = build_optimizer(model, OptimConf(lr=1e-4, warmup=10, clip=1.0), 1000, "bf16")

    g = torch.Generator().manual_seed(100 + dp_rank)       # model- and chunk-parallel ranks see the same batch
    toks = torch.randint(0, cfg.vocab_size, (args.micro_batch, args.seq_len + 1), generator=g).cuda()
    x, y = toks[:, :-1].contiguous(), toks[:, 1:].contiguous()

    def step():
        tok_loss, _ = model(x, targets=y)
        loss = tok_loss.mean()
        loss.backward()
        model.grad_all_reduce()
        clip_grad_norm_(model, 1.0)
        opt.step()
        sched.step()
        opt.zero_grad()
        return loss

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        last = step()
        torch.cuda.synchronize()
        if abort_record is not None:
            abort_record.check()
        dog.progress(f"warm-up step {i} done")
    cuda_ops.check_kernel_errors()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        last = step()
        dog.progress(f"timed step {i} enqueued")
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    cuda_ops.check_kernel_errors()
    if abort_record is not None:
        abort_record.check()
    if world > 1:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    tokens = args.micro_batch * dp * args.seq_len * args.steps
    if rank == 0:
        out = {"metric": "train tokens/s", "value": tokens / (ms / 1e3), "unit": "tokens/s", "n_gpus": world,
               "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "dtype": "bf16",
               "data": "synthetic",
               "config": {"model": f"{args.model} L{cfg.num_layers}", "parallelism": f"dp{dp}xcp{args.cp}xmp{args.mp}",
                          "seq_len": args.seq_len, "micro_batch_per_dp_rank": args.micro_batch,
                          "global_batch": args.micro_batch * dp, "activation_checkpointing": bool(args.ckpt),
                          "reshard_after_forward": bool(args.reshard),
                          "composition": ("cuBLAS + NCCL + materialised attention inside this framework (not the reference)"
                                          if library else "this framework's kernels and peer-memory collectives"),
                          "fused_tp": args.mp > 1 and not args.no_fused_tp and not library,
                          "final_loss": float(last.item())}}
        if args.layers is not None:
            out["invalid"] = "reduced depth (debug run)"
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    dog.stop()


if __name__ == "__main__":
    main()
