"""Inference benchmark: chunk-parallel prefill throughput and per-token decode latency.

    # prefill: the prompt is split over N chunk-parallel GPUs, CEMA / TimestepNorm state handed on
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        benchmarks/infer_bench.py --phase prefill [--prompt-len 131072]
    # decode: model parallel over N GPUs (N <= number of heads), recurrent cache, greedy
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        benchmarks/infer_bench.py --phase decode [--batches 1,4,16] [--gen-len 256]

    # both: prefill with chunk parallelism over all N GPUs, hand weights and state over to a
    # tensor-parallel layout over the same N GPUs (N may exceed the number of heads), decode there
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        benchmarks/infer_bench.py --phase both [--prompt-len 131072] [--batches 1,4,16] [--gen-len 256]

`prefill` and `decode` alone use one process-group layout each; the decode phase then fills its cache by
prefilling a short prompt (one full chunk plus a remainder) through the cache path.  `both` switches
layouts inside the process: the tensor-parallel model receives the prefill model's weights (sliced on
the GPU from its gathered buffers) and the prefill's final state re-sharded by features and heads.
Random-init bf16 weights, uniform random prompt.  Timing: CUDA events after warm-up, max over ranks.
Rank 0 prints one JSON line per phase.
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
    ap.add_argument("--phase", choices=["prefill", "decode", "both"], required=True)
    ap.add_argument("--model", default="mega7B_32k")
    ap.add_argument("--layers", type=int, default=None, help="debug: fewer layers (not a valid result)")
    ap.add_argument("--prompt-len", type=int, default=None, help="prefill: total prompt tokens (default 16384 per GPU)")
    ap.add_argument("--batches", default="1,4,16")
    ap.add_argument("--gen-len", type=int, default=256)
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--kernel-profile", default=None,
                    help="decode: also run one eager fixed-shape step per batch size under torch.profiler and write "
                         "the per-kernel summary to this path (never part of a reported number)")
    ap.add_argument("--stall-dump-s", type=float, default=240.0,
                    help="a phase that makes no progress for this long dumps every thread's Python stack to stderr "
                         "and ends the process (0: off)")
    ap.add_argument("--eager", action="store_true", help="decode through the regular cache path instead of the "
                                                         "graph-replayed fixed-shape session")
    args = ap.parse_args()

    import torch
    import torch.distributed as dist
    from megalodon_b200.models.mega import ModelStore, build_model
    from megalodon_b200.ops import cuda_ops
    from megalodon_b200.parallel import init_torch_distributed, initialize_model_parallel
    from megalodon_b200.utils import init_cache, set_random_seed

    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    rank = 0
    if world > 1:
        rank = init_torch_distributed().global_rank
    cfg = dataclasses.replace(ModelStore[args.model])
    if args.layers is not None:
        cfg.num_layers = args.layers
    cfg.layerwise_ckpt = False
    cfg.dropout = cfg.hidden_dropout = cfg.attention_dropout = 0.0
    set_random_seed(1234)

    def maxed(ms):
        if world > 1:
            t = torch.tensor([ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
        return ms

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if args.phase == "both":
        from megalodon_b200.decoding import DecodeSession
        from megalodon_b200.parallel import destroy_model_parallel, get_model_parallel_rank
        from megalodon_b200.parallel.chunk_parallel import set_handoff_transport
        from megalodon_b200.reloading import shard_state_dict_for_model_parallel
        from megalodon_b200.utils import expand_cache, reshard_cache
        assert world > 1, "--phase both needs several GPUs"
        # ---- phase 1: chunk-parallel prefill
        initialize_model_parallel(1, world)
        model = build_model(cfg, "bf16", reshard_after_forward=False, shard_over_chunk_group=True)
        model.eval()
        model._wrapped.seq_microbatch_chunks = 1
        from megalodon_b200.parallel.symm import enable_peer_transport
        enable_peer_transport(model, max_batch=1, n_slots=8, timeout_s=10.0)
        P = args.prompt_len or 16384 * world
        assert P % (world * cfg.chunk_size) == 0
        toks = torch.randint(0, cfg.vocab_size, (1, P), generator=torch.Generator().manual_seed(0)).cuda()
        with torch.no_grad():
            logits, cache = model(toks, prefill=True)            # warm-up
            del logits, cache
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            logits, cache = model(toks, prefill=True)
            e1.record()
            barrier()
        prefill_ms = maxed(e0.elapsed_time(e1))
        cuda_ops.check_kernel_errors()
        first_tok = logits.argmax(-1, keepdim=True)               # [1, 1]
        # ---- hand-over: weights sliced on the GPU, state re-sharded, process groups re-made
        full_sd = model.gathered_state_dict()
        destroy_model_parallel()
        set_handoff_transport("nccl")
        initialize_model_parallel(world, 1)
        mp_rank = get_model_parallel_rank()
        barrier()
        t_switch = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t_switch[0].record()
        decoder = build_model(cfg, "bf16", reshard_after_forward=False)
        decoder.eval()
        decoder.load_state_dict(shard_state_dict_for_model_parallel(full_sd, cfg.num_heads, mp_rank, world), strict=False)
        state = reshard_cache(cache, mp_rank, world)
        del model, full_sd, cache
        torch.cuda.empty_cache()
        t_switch[1].record()
        barrier()
        switch_ms = maxed(t_switch[0].elapsed_time(t_switch[1]))
        # ---- phase 2: tensor-parallel decode from the prefilled state
        results = {}
        with torch.inference_mode():
            for B in [int(b) for b in args.batches.split(",")]:
                sess = DecodeSession(decoder, B, torch.bfloat16)
                sess.load_cache(expand_cache(state, B))
                tok = first_tok.expand(B, 1).contiguous()
                for _ in range(8):
                    tok = sess.step(tok).argmax(-1, keepdim=True)
                barrier()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(args.gen_len):
                    tok = sess.step(tok).argmax(-1, keepdim=True)
                e1.record()
                barrier()
                results[B] = maxed(e0.elapsed_time(e1) / args.gen_len)
                del sess
        cuda_ops.check_kernel_errors()
        if rank == 0:
            out = {"metric": "prefill tokens/s and decode ms/token", "value": P / (prefill_ms / 1e3), "unit": "tokens/s",
                   "decode_ms_per_token": results, "layout_switch_ms": switch_ms, "n_gpus": world, "dtype": "bf16",
                   "data": "synthetic",
                   "config": {"model": f"{args.model} L{cfg.num_layers}", "prompt_len": P,
                              "prefill": f"cp{world}, peer-memory hand-off", "decode": f"mp{world}"
                              + (f" ({world // cfg.num_heads} ranks per head)" if world > cfg.num_heads else ""),
                              "gen_len": args.gen_len, "sampling": "greedy", "chunk": cfg.chunk_size}}
            if args.layers is not None:
                out["invalid"] = "reduced depth (debug run)"
            print(json.dumps(out))
    elif args.phase == "prefill":
        if world > 1:
            initialize_model_parallel(1, world)
        model = build_model(cfg, "bf16", reshard_after_forward=False, shard_over_chunk_group=True)
        model.eval()
        model._wrapped.seq_microbatch_chunks = 1
        if world > 1:
            from megalodon_b200.parallel.symm import enable_peer_transport
            enable_peer_transport(model, max_batch=1, n_slots=8, timeout_s=30.0)
        P = args.prompt_len or 16384 * world
        assert P % (world * cfg.chunk_size) == 0
        g = torch.Generator().manual_seed(0)
        toks = torch.randint(0, cfg.vocab_size, (1, P), generator=g).cuda()
        with torch.no_grad():
            for _ in range(2):
                logits, cache = model(toks, prefill=True)
            del logits, cache
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.reps):
                logits, cache = model(toks, prefill=True)     # last-position logits + the cache a decoder takes over
                nxt = logits.argmax(-1)
                del logits, cache
            e1.record()
            barrier()
        ms = maxed(e0.elapsed_time(e1) / args.reps)
        cuda_ops.check_kernel_errors()
        if rank == 0:
            out = {"metric": "prefill tokens/s", "value": P / (ms / 1e3), "unit": "tokens/s", "n_gpus": world,
                   "ms": ms, "dtype": "bf16", "data": "synthetic",
                   "config": {"model": f"{args.model} L{cfg.num_layers}", "prompt_len": P, "parallelism": f"cp{world}",
                              "chunk": cfg.chunk_size}}
            if args.layers is not None:
                out["invalid"] = "reduced depth (debug run)"
            print(json.dumps(out))
    else:
        if world > 1:
            initialize_model_parallel(world, 1)
        model = build_model(cfg, "bf16", reshard_after_forward=False)
        model.eval()
        inner = model
        while hasattr(inner, "_wrapped"):
            inner = inner._wrapped
        c = cfg.chunk_size
        results = {}
        import faulthandler
        with torch.inference_mode():
            for B in [int(b) for b in args.batches.split(",")]:
                if args.stall_dump_s > 0:
                    faulthandler.dump_traceback_later(args.stall_dump_s, exit=True)     # re-armed per batch size
                g = torch.Generator().manual_seed(B)
                prompt = torch.randint(0, cfg.vocab_size, (B, c + 17), generator=g).cuda()
                cache = init_cache(B, inner, torch.bfloat16, device=prompt.device)
                _, cache = model(prompt[:, :c], cache=cache)            # one whole chunk
                logits, cache = model(prompt[:, c:], cache=cache)       # remainder of the prompt
                tok = logits[:, -1].argmax(-1, keepdim=True)
                if args.eager:
                    state = {"cache": cache}

                    def step(tok):
                        lg, state["cache"] = model(tok, cache=state["cache"])
                        return lg[:, -1].argmax(-1, keepdim=True)
                else:
                    from megalodon_b200.decoding import DecodeSession
                    sess = DecodeSession(model, B, torch.bfloat16)
                    sess.load_cache(cache)

                    def step(tok):
                        return sess.step(tok).argmax(-1, keepdim=True)
                for _ in range(8):                                       # warm-up decode steps (and graph capture)
                    tok = step(tok)
                barrier()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(args.gen_len):
                    tok = step(tok)
                e1.record()
                barrier()
                results[B] = maxed(e0.elapsed_time(e1) / args.gen_len)
                faulthandler.cancel_dump_traceback_later()
                print(f"[rank {rank}] batch {B}: {results[B]:.2f} ms/token", file=sys.stderr, flush=True)
                if not args.eager and not args.kernel_profile:
                    del sess, step
                if args.kernel_profile and rank == 0:
                    import collections
                    from torch.profiler import ProfilerActivity, profile
                    from megalodon_b200.decoding import DecodeSession
                    eager = DecodeSession(model, B, torch.bfloat16, use_graph=False)
                    eager.load_cache(cache)          # the state right after the prompt is as good as any for a profile
                    for _ in range(3):
                        tok = eager.step(tok).argmax(-1, keepdim=True)
                    torch.cuda.synchronize()
                    with profile(activities=[ProfilerActivity.CUDA]) as prof:
                        tok = eager.step(tok).argmax(-1, keepdim=True)
                        torch.cuda.synchronize()
                    agg = collections.defaultdict(lambda: [0.0, 0])
                    for e in prof.events():
                        if e.device_type == torch.autograd.DeviceType.CUDA:
                            agg[e.name][0] += e.device_time
                            agg[e.name][1] += 1
                    tot = sum(v[0] for v in agg.values())
                    with open(f"{args.kernel_profile}.batch{B}", "w") as f:
                        f.write(f"batch {B}: kernel time {tot / 1e3:.2f} ms, {sum(v[1] for v in agg.values())} launches\n")
                        for name, (t, n) in sorted(agg.items(), key=lambda kv: -kv[1][0])[:25]:
                            f.write(f"{t / 1e3:8.3f} ms {100 * t / tot:5.1f}% {n:5d}x {t / n:8.1f} us  {name[:110]}\n")
        cuda_ops.check_kernel_errors()
        if rank == 0:
            out = {"metric": "decode ms/token", "value": results, "unit": "ms", "n_gpus": world,
                   "higher_is_better": False, "dtype": "bf16", "data": "synthetic",
                   "config": {"model": f"{args.model} L{cfg.num_layers}", "parallelism": f"mp{world}",
                              "gen_len": args.gen_len, "prompt_len": c + 17, "sampling": "greedy",
                              "path": "eager cache path" if args.eager else "CUDA-graph decode session"}}
            if args.layers is not None:
                out["invalid"] = "reduced depth (debug run)"
            print(json.dumps(out))
    if world > 1:
        import faulthandler
        import gc
        # sessions (captured graphs, peer-memory regions of their collectives) go before the process group
        from megalodon_b200.parallel.model_parallel import mappings
        mappings.use_small_collective(None)
        sess = None  # noqa: F841
        gc.collect()
        torch.cuda.synchronize()
        if args.stall_dump_s > 0:
            faulthandler.dump_traceback_later(min(args.stall_dump_s, 90.0), exit=True)
        dist.barrier()
        dist.destroy_process_group()
        faulthandler.cancel_dump_traceback_later()


if __name__ == "__main__":
    main()
