"""Drives the UNMODIFIED reference (installed under baseline/_ref) through its own public API for the
headline benchmark: Megalodon-7B, one 32768-token sequence per step, chunk parallel over the N ranks,
bf16, AdamW with clipping.  Nothing of this framework is on the path: model, layers, kernels, FSDP
wrapper, loss, optimiser and clipping are the reference's (megalodon/model/mega.py:245 build_model,
megalodon/modules/losses.py:12 cross_entropy, megalodon/optim/optimizer.py:24 build_optimizer,
megalodon/utils.py:118 clip_grad_norm_, megalodon/distributed/initialize.py:31).

The timing rules are the ones of the framework's own arm: W untimed steps, K steps between CUDA events
with a barrier and a synchronize on both sides, max over ranks, and a second region that includes the
pinned host->device copy of the tokens and the device->host read of the loss every step.

`run(args)` returns the result dictionary on rank 0 (None elsewhere) or raises; the caller turns an
exception into the arm's `unavailable` line.
"""
import os
import sys
import time


def _conf_7b_32k(ModelConf, chunks_per_rank: int):
    # the 7B shape of the reference's model store (32 layers, width 4096, 4 heads, z 1024, v 8192, SwiGLU FFN
    # of 11264) with 4096-token chunks and its fused attention path; layer checkpointing where one rank holds
    # more than two chunks, as in the framework's own arm (the reference checkpoints all layers or none)
    return ModelConf(num_layers=32, model_dim=4096, num_heads=4, z_dim=1024, value_dim=8192, ffn_hidden_dim=11264,
                     chunk_size=4096, norm_num_groups=64, swiglu=True, efficient_attn="fused",
                     vocab_size=32000, layerwise_ckpt=chunks_per_rank > 2)


def run(args, ref_root: str):
    sys.path.insert(0, ref_root)
    import torch
    import torch.distributed as dist
    from megalodon.config import ModelConf, OptimConf
    from megalodon.distributed import init_torch_distributed, initialize_model_parallel
    from megalodon.model.mega import build_model
    from megalodon.modules.losses import cross_entropy
    from megalodon.optim import build_optimizer
    from megalodon.utils import clip_grad_norm_, set_random_seed

    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("LOCAL_RANK", "0")
    _, rank, _ = init_torch_distributed()
    initialize_model_parallel(1, world)          # model parallel 1, chunk parallel over every rank
    set_random_seed(1234)
    cfg = _conf_7b_32k(ModelConf, args.seq_len // world // 4096)
    model = build_model(cfg, "bf16", False, False)
    opt, sched = build_optimizer(model, OptimConf(lr=1e-4, warmup=10, clip=1.0), 1000, "bf16")
    gen = torch.Generator().manual_seed(0)

    def batch():
        toks = torch.randint(0, cfg.vocab_size, (1, args.seq_len + 1), generator=gen)
        return toks[:, :-1].contiguous().pin_memory(), toks[:, 1:].contiguous().pin_memory()

    def step(x, y):
        logits, _ = model(x)
        loss = cross_entropy(logits, y).mean()
        loss.backward()
        clip_grad_norm_(model, 1.0)
        opt.step()
        sched.step()
        opt.zero_grad()
        return loss

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        x, y = batch()
        step(x.cuda(non_blocking=True), y.cuda(non_blocking=True)).item()
    x, y = batch()
    xd, yd = x.cuda(), y.cuda()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step(xd, yd)
    e1.record()
    barrier()
    dev_ms = e0.elapsed_time(e1)
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e2.record()
    last = float("nan")
    for _ in range(args.steps):
        x, y = batch()
        last = step(x.cuda(non_blocking=True), y.cuda(non_blocking=True)).item()
    e3.record()
    barrier()
    e2e_ms = e2.elapsed_time(e3)
    wall_ms = (time.perf_counter() - t0) * 1e3
    if world > 1:
        t = torch.tensor([dev_ms, e2e_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dev_ms, e2e_ms = t.tolist()
    tokens = args.seq_len * args.steps
    out = None
    if rank == 0:
        out = {"impl": "reference", "value": tokens / (dev_ms / 1e3), "unit": "tokens/s", "n_gpus": world,
               "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms / args.steps,
               "higher_is_better": True, "scaling": "strong", "dtype": "bf16", "data": "synthetic",
               "config": {"model": "mega 7B (L32 D4096 H4 z1024 v8192 ffn11264 swiglu chunk4096 V32000)",
                          "global_batch": 1, "seq_len": args.seq_len, "parallelism": f"cp{world}",
                          "activation_checkpointing": "all layers" if cfg.layerwise_ckpt else False,
                          "final_loss": last},
               "e2e": {"value": tokens / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                       "wall_ms_per_step": wall_ms / args.steps, "h2d_bytes_per_step": 2 * args.seq_len * 8,
                       "d2h_bytes_per_step": 4}}
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return out
