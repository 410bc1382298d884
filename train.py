"""Pre-training entry point: the training loop the reference only sketches in its
README (README.md:82-151), made runnable.

    torchrun --nproc-per-node 8 train.py --model mega7B_32k --seq_len 32768 \
        --chunk_parallel_size 8 --steps 100 --dump_dir runs/x [--data_path data.jsonl --tokenizer_path tok.model]

Without `--data_path` it trains on synthetic uniform-random tokens.  Checkpoints
are sharded `model.ckpt.RRRRR.pth` files (`--save_every`); `--resume` continues
from them; `--consolidate_to DIR` writes `consolidated[.NN].pth` at the end.
"""
import argparse
import dataclasses
import logging
import os
import sys

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from megalodon_b200 import reloading  # noqa: E402
from megalodon_b200.config import ModelConf, OptimConf, TokenizerConf, TrainerConf  # noqa: E402
from megalodon_b200.data.dataloader import DataLoader, SyntheticTokens  # noqa: E402
from megalodon_b200.logger import add_logger_file_handler, initialize_logger  # noqa: E402
from megalodon_b200.models.mega import ModelStore, build_model  # noqa: E402
from megalodon_b200.optim import build_optimizer  # noqa: E402
from megalodon_b200.parallel import (  # noqa: E402
    get_chunk_parallel_rank, get_data_parallel_rank, get_data_parallel_world_size, get_model_parallel_rank,
    init_signal_handler, init_torch_distributed, initialize_model_parallel)
from megalodon_b200.utils import clip_grad_norm_, log_host, set_random_seed, setup_env  # noqa: E402
from megalodon_b200.utils.profiling import MetricsWriter, StepTimer, model_flops_per_token, nvtx_range  # noqa: E402

logger = logging.getLogger()


def parse() -> TrainerConf:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="mega200M", help="preset name from ModelStore")
    for f in dataclasses.fields(TrainerConf):
        if f.name in ("model", "optim", "tokenizer"):
            continue
        typ = f.type if isinstance(f.type, type) else str
        if f.type in ("bool", bool):
            ap.add_argument(f"--{f.name}", type=lambda s: s.lower() == "true", default=f.default)
        elif f.type in ("int", int):
            ap.add_argument(f"--{f.name}", type=int, default=f.default)
        else:
            ap.add_argument(f"--{f.name}", type=str, default=f.default)
    for f in dataclasses.fields(OptimConf):
        ap.add_argument(f"--{f.name}", type=type(f.default), default=f.default)
    ap.add_argument("--tokenizer_path", default=None)
    ap.add_argument("--vocab_size", type=int, default=32000)
    ap.add_argument("--layerwise_ckpt", type=lambda s: s.lower() == "true", default=True)
    ap.add_argument("--ckpt_layers", type=int, default=None,
                    help="with --layerwise_ckpt: checkpoint only the first K blocks (default: all)")
    ap.add_argument("--seq_microbatch_chunks", type=int, default=1)
    ap.add_argument("--shard_over_chunk_group", type=lambda s: s.lower() == "true", default=True)
    ap.add_argument("--peer_transport", type=lambda s: s.lower() == "true", default=True)
    ap.add_argument("--consolidate_to", default=None)
    a = ap.parse_args()
    model = dataclasses.replace(ModelStore[a.model])
    if model.vocab_size <= 0:
        model.vocab_size = a.vocab_size
    model.layerwise_ckpt = a.layerwise_ckpt
    model.ckpt_layers = a.ckpt_layers
    model.efficient_attn = model.efficient_attn or "fused"
    optim = OptimConf(**{f.name: getattr(a, f.name) for f in dataclasses.fields(OptimConf)})
    cfg = TrainerConf(model=model, optim=optim, tokenizer=TokenizerConf(path=a.tokenizer_path))
    for f in dataclasses.fields(TrainerConf):
        if f.name not in ("model", "optim", "tokenizer"):
            setattr(cfg, f.name, getattr(a, f.name))
    cfg.extra = a
    return cfg


def main() -> None:
    cfg = parse()
    initialize_logger()
    setup_env()
    log_host()
    init_signal_handler()
    info = init_torch_distributed()
    initialize_model_parallel(cfg.model_parallel_size, cfg.chunk_parallel_size)
    if cfg.dump_dir and info.global_rank == 0:
        os.makedirs(cfg.dump_dir, exist_ok=True)
        add_logger_file_handler(os.path.join(cfg.dump_dir, "train.log"))
    logger.info(f"Global rank: {info.global_rank} -- model parallel rank: {get_model_parallel_rank()}/"
                f"{cfg.model_parallel_size} -- chunk parallel rank: {get_chunk_parallel_rank()}/"
                f"{cfg.chunk_parallel_size} -- data parallel rank: {get_data_parallel_rank()}/"
                f"{get_data_parallel_world_size()}")
    set_random_seed(cfg.seed)
    model = build_model(cfg.model, cfg.dtype, cfg.fp32_reduce_scatter, cfg.reshard_after_forward,
                        shard_over_chunk_group=cfg.extra.shard_over_chunk_group)
    model._wrapped.seq_microbatch_chunks = cfg.extra.seq_microbatch_chunks or None
    model.defer_grad_clip = torch.cuda.is_available()
    if cfg.extra.peer_transport and torch.cuda.is_available() and cfg.chunk_parallel_size > 1:
        from megalodon_b200.parallel.symm import enable_peer_transport
        enable_peer_transport(model, max_batch=cfg.batch_size)
    elif (cfg.extra.peer_transport and torch.cuda.is_available() and get_data_parallel_world_size() > 1
          and cfg.dtype != "fp32"):
        # plain data parallelism: gradient reduce-scatter and parameter gathers through peer memory
        from megalodon_b200.parallel.symm import enable_peer_gather, enable_peer_reduce_scatter
        enable_peer_reduce_scatter(model)
        enable_peer_gather(model)
    if (cfg.extra.peer_transport and torch.cuda.is_available() and cfg.model_parallel_size > 1
            and cfg.dtype != "fp32"):
        # collectives of the tensor-parallel projections inside their GEMMs
        from megalodon_b200.parallel.tp_comm import enable_tp_fused
        local_len = cfg.seq_len // max(1, cfg.chunk_parallel_size)
        if cfg.extra.seq_microbatch_chunks:
            local_len = min(local_len, cfg.model.chunk_size * cfg.extra.seq_microbatch_chunks)
        enable_tp_fused(model, max_tokens=cfg.batch_size * local_len)
    logger.info(model)
    optimizer, scheduler = build_optimizer(model, cfg.optim, cfg.steps, cfg.dtype)
    step = 0
    if cfg.resume and cfg.dump_dir and os.path.exists(os.path.join(cfg.dump_dir, reloading.model_ckpt_name(info.global_rank))):
        step = reloading.load_sharded(model, optimizer, scheduler, cfg.dump_dir)
        logger.info(f"resumed from step {step}")

    if cfg.data_path:
        from megalodon_b200.data.tokenizer import Tokenizer
        tok = Tokenizer(cfg.tokenizer)
        assert tok.n_words == cfg.model.vocab_size, (tok.n_words, cfg.model.vocab_size)

        def batches():
            while True:
                dl = DataLoader(tok, cfg.data_path, cfg.batch_size, get_data_parallel_rank(), get_data_parallel_world_size())
                for b in dl:
                    x, y = b["x"][:, :cfg.seq_len], b["y"][:, :cfg.seq_len]
                    if x.size(1) == cfg.seq_len:
                        yield x, y
                dl.close()
        data = batches()
    else:
        data = iter(SyntheticTokens(cfg.model.vocab_size, cfg.batch_size, cfg.seq_len,
                                    seed=cfg.seed + get_data_parallel_rank()))
    metrics = MetricsWriter(os.path.join(cfg.dump_dir, "metrics.jsonl") if cfg.dump_dir else None)
    timer = StepTimer()
    device = next(model.parameters()).device
    tokens_per_step = cfg.batch_size * cfg.seq_len * get_data_parallel_world_size()
    flops_tok = model_flops_per_token(cfg.model, with_recompute=cfg.model.layerwise_ckpt)
    while step < cfg.steps:
        x, y = next(data)
        timer.start()
        with nvtx_range("step"):
            x, y = x.to(device, non_blocking=True), y.to(device, non_blocking=True)
            tok_loss, _ = model(x, targets=y)
            loss = tok_loss.mean()
            loss.backward()
            model.grad_all_reduce()
            norm = clip_grad_norm_(model, cfg.optim.clip)
            optimizer.step()
            scheduler.step()
            optimizer.zero_grad()
        ms = timer.stop()
        step += 1
        if step % cfg.log_every == 0:
            lv, nv = float(loss), float(norm)
            tps = tokens_per_step / (ms / 1e3)
            logger.info(f"step {step} loss {lv:.4f} gnorm {nv:.3f} lr {scheduler.get_last_lr()[0]:.3e} "
                        f"{ms:.1f} ms {tps:.0f} tok/s {tps * flops_tok / 1e12:.1f} TFLOP/s")
            metrics.write(step=step, loss=lv, grad_norm=nv, ms=ms, tokens_per_s=tps,
                          tflops=tps * flops_tok / 1e12, lr=scheduler.get_last_lr()[0])
        if cfg.save_every and cfg.dump_dir and step % cfg.save_every == 0:
            reloading.save_sharded(model, optimizer, scheduler, step, cfg.dump_dir, cfg.model, cfg.tokenizer)
    if cfg.dump_dir:
        reloading.save_sharded(model, optimizer, scheduler, step, cfg.dump_dir, cfg.model, cfg.tokenizer)
    if cfg.extra.consolidate_to:
        reloading.save_consolidated(model, cfg.extra.consolidate_to, cfg.model, cfg.tokenizer, dtype=cfg.dtype)
    logger.info("===== Finished training.")


if __name__ == "__main__":
    main()
