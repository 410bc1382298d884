"""Evaluation entry point with the flags of the reference's eval.py (eval.py:160-258):
perplexity over jsonl files and greedy / sampled generation from a prompt file.

    torchrun --nproc-per-node N eval.py --model_parallel_size 1 --checkpoint_dir CKPT --dump_dir OUT \
        --dtype bf16 --ppl_files_str a.jsonl,b.jsonl --prompt_path prompts.jsonl --batch_size 1

Flags arrive as strings and are converted here (no `fire` dependency).  Unlike the
reference, `--model_parallel_size` may be omitted (the checkpoint's value is used)
and `--top_k/--top_p` are forwarded to generation.
"""
import argparse
import json
import logging
import math
import os
import sys
from dataclasses import dataclass
from pathlib import Path
from typing import List, Optional

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from megalodon_b200.config import ValidConf  # noqa: E402
from megalodon_b200.data.dataloader import DataLoader  # noqa: E402
from megalodon_b200.generation import generate  # noqa: E402
from megalodon_b200.inference import inference  # noqa: E402
from megalodon_b200.logger import initialize_logger  # noqa: E402
from megalodon_b200.parallel import (  # noqa: E402
    get_chunk_parallel_rank, get_chunk_parallel_world_size, get_data_parallel_group, get_data_parallel_rank,
    get_data_parallel_world_size, get_model_parallel_rank)
from megalodon_b200.parallel.setup import get_global_rank  # noqa: E402
from megalodon_b200.parallel.utils import reduce_scalar  # noqa: E402
from megalodon_b200.reloading import reload_model  # noqa: E402
from megalodon_b200.utils import get_default_half, log_host, parse_bool_flag, set_random_seed, setup_env  # noqa: E402

logger = logging.getLogger()


@dataclass
class EvalConf:
    valid: ValidConf
    checkpoint_dir: str
    dump_dir: str
    tokenizer_path: Optional[str] = None
    master_logging_only: bool = True
    dtype: str = get_default_half()
    model_parallel_size: Optional[int] = None
    seed: int = 42

    def __post_init__(self):
        assert Path(self.checkpoint_dir).is_dir(), self.checkpoint_dir
        os.makedirs(self.dump_dir, exist_ok=True)


@torch.no_grad()
def eval_ppl(model, dtype: str, path: str, tokenizer, batch_size: int, world_rank: int, world_size: int):
    model.eval()
    assert get_chunk_parallel_world_size() == 1, "task evaluation does not support chunk parallel"
    loader = DataLoader(tokenizer=tokenizer, path=path, batch_size=batch_size, world_rank=world_rank,
                        world_size=world_size)
    batches = list(iter(loader))
    loader.close()
    real = len(batches)
    # every rank must run the same number of forwards: pad with repeats of the first batch
    most = int(reduce_scalar(real, op="max"))
    if real == 0 and most > 0:
        raise RuntimeError(f"rank {world_rank} received no data from {path}")
    batches += [batches[0]] * (most - real)
    device = next(model.parameters()).device
    loss, ntokens = 0.0, 0
    for i, batch in enumerate(batches):
        x, y = batch["x"].to(device), batch["y"].to(device)
        nll = inference(model, x, y, dtype)
        if i < real:
            loss += nll.sum().item()
            ntokens += int((y != -100).sum().item())
    tot_loss = reduce_scalar(loss, op="sum", group=get_data_parallel_group())
    tot_toks = reduce_scalar(ntokens, op="sum", group=get_data_parallel_group())
    return math.exp(tot_loss / max(tot_toks, 1)), tot_toks


@torch.no_grad()
def run_generation(model, dtype: str, tokenizer, cfg: ValidConf, dump_dir: str, world_rank: int, world_size: int):
    assert get_chunk_parallel_world_size() == 1, "generation does not support chunk parallel"
    logger.info(f"Evaluating generation on {cfg.prompt_path} ...")
    with open(cfg.prompt_path) as f:
        lines = [json.loads(line) for line in f if line.strip()]
    logger.info(f"Reloaded {len(lines)} lines from {cfg.prompt_path}")
    n_prompts = len(lines)
    per = math.ceil(n_prompts / world_size)
    prompts = [x["text"] for x in lines] + ["FAKE"] * (per * world_size - n_prompts)
    mine = prompts[per * world_rank:per * (world_rank + 1)]
    out = None
    if get_model_parallel_rank() == 0 and get_chunk_parallel_rank() == 0:
        gen_dir = Path(dump_dir) / "generations"
        gen_dir.mkdir(parents=True, exist_ok=True)
        out = open(gen_dir / f"{world_rank}.jsonl", "a")
    for i, prompt in enumerate(mine):
        res: List[List[int]] = generate(model, dtype, tokenizer, prompt=[prompt], use_sampling=cfg.use_sampling,
                                        temp=cfg.temperature, top_k=cfg.top_k, top_p=cfg.top_p,
                                        max_gen_len=cfg.gen_seq_len, remove_prompts=True)
        text = tokenizer.decode(res[0], cut_at_eos=True)
        is_real = per * world_rank + i < n_prompts
        if out is not None and is_real:
            out.write(json.dumps({"prompt": prompt, "generation": text}, ensure_ascii=False) + "\n")
    if out is not None:
        out.close()


def main(checkpoint_dir: str, dump_dir: str, tokenizer_path: Optional[str] = None, master_logging_only: str = "true",
         dtype: str = get_default_half(), model_parallel_size: Optional[str] = None, ppl_files_str: str = "",
         prompt_path: str = "", batch_size: str = "1", use_sampling: str = "false", temperature: str = "1.0",
         top_k: str = "0", top_p: str = "0.0", gen_seq_len: str = "512", seed: str = "42"):
    valid = ValidConf(ppl_files_str=ppl_files_str, prompt_path=prompt_path, batch_size=int(batch_size),
                      use_sampling=parse_bool_flag(use_sampling), temperature=float(temperature), top_k=int(top_k),
                      top_p=float(top_p), gen_seq_len=int(gen_seq_len))
    cfg = EvalConf(valid=valid, checkpoint_dir=checkpoint_dir, dump_dir=dump_dir, tokenizer_path=tokenizer_path,
                   master_logging_only=parse_bool_flag(master_logging_only), dtype=dtype,
                   model_parallel_size=None if model_parallel_size in (None, "", "None") else int(model_parallel_size),
                   seed=int(seed))
    initialize_logger()
    setup_env()
    log_host()
    if get_global_rank() > 0 and cfg.master_logging_only:
        logger.info(f"No print for worker {get_global_rank()}")
        logger.disabled = True
    model, tokenizer, ckpt_cfg = reload_model(checkpoint_dir=cfg.checkpoint_dir, model_parallel_size=cfg.model_parallel_size,
                                              chunk_parallel_size=1, dtype=cfg.dtype, tokenizer_path=cfg.tokenizer_path)
    logger.info(f"checkpoint config: {ckpt_cfg}")
    logger.info(model)
    world_rank, world_size = get_data_parallel_rank(), get_data_parallel_world_size()
    torch_seed = cfg.seed + int(os.environ.get("SLURM_ARRAY_TASK_ID", 0)) + world_rank
    logger.info(f"Setting torch seed to {torch_seed}")
    set_random_seed(torch_seed)
    torch.backends.cuda.matmul.allow_tf32 = True
    logger.info("Running PPL evaluations ...")
    for path in cfg.valid.ppl_files:
        logger.info(f"Evaluating PPL on {path} ...")
        ppl, n_tokens = eval_ppl(model, cfg.dtype, path, tokenizer, cfg.valid.batch_size, world_rank, world_size)
        logger.info(f"PPL on {path}: {ppl}, w. {n_tokens} tokens.")
        if torch.cuda.is_available():
            torch.cuda.empty_cache()
    if cfg.valid.prompt_path:
        run_generation(model, cfg.dtype, tokenizer, cfg.valid, cfg.dump_dir, world_rank, world_size)
    logger.info("===== Finished all evaluations.")


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    for name, default in (("checkpoint_dir", None), ("dump_dir", None), ("tokenizer_path", None),
                          ("master_logging_only", "true"), ("dtype", get_default_half()), ("model_parallel_size", None),
                          ("ppl_files_str", ""), ("prompt_path", ""), ("batch_size", "1"), ("use_sampling", "false"),
                          ("temperature", "1.0"), ("top_k", "0"), ("top_p", "0.0"), ("gen_seq_len", "512"),
                          ("seed", "42")):
        ap.add_argument(f"--{name}", default=default, required=default is None and name in ("checkpoint_dir", "dump_dir"))
    main(**vars(ap.parse_args()))
