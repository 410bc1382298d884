"""Autoregressive generation with the recurrent cache: whole chunks of the
prompt are prefilled `MAX_CHUNKS_PER_BATCH` at a time, the remainder of the
prompt goes through in one call, then one forward per new token.  Greedy,
temperature, top-k and top-p (nucleus) sampling (reference:
megalodon/generation.py:23-185)."""
from __future__ import annotations

import logging
from typing import List, Optional, Tuple

import torch

from .parallel import get_data_parallel_world_size, get_model_parallel_group, model_parallel_is_initialized
from .parallel.utils import reduce_scalar
from .utils import check_same_in_process_group, get_torch_dtype, init_cache, truncate_cache

logger = logging.getLogger()

MAX_CHUNKS_PER_BATCH = 2
TRUNCATE_CHUNKS = 8


def _dist_on() -> bool:
    return torch.distributed.is_available() and torch.distributed.is_initialized()


def get_min_length(input_tokens: Optional[List[List[int]]]) -> int:
    n = int(1e9) if input_tokens is None else min(len(t) for t in input_tokens)
    return int(reduce_scalar(n, op="min")) if _dist_on() else n


def get_max_length(input_tokens: Optional[List[List[int]]]) -> int:
    n = 0 if input_tokens is None else max(len(t) for t in input_tokens)
    return int(reduce_scalar(n, op="max")) if _dist_on() else n


def get_generation_range(prompt_tokens: Optional[List[List[int]]], max_gen_len: int) -> Tuple[int, int]:
    return get_min_length(prompt_tokens), get_max_length(prompt_tokens) + max_gen_len


def sample_top_k(probs: torch.Tensor, k: int) -> torch.Tensor:
    kth = torch.topk(probs, k).values[:, [-1]]
    probs = probs.masked_fill(probs < kth, 0.0)
    probs = probs / probs.sum(dim=-1, keepdim=True)
    return torch.multinomial(probs, num_samples=1)


def sample_top_p(probs: torch.Tensor, p: float) -> torch.Tensor:
    sorted_p, order = torch.sort(probs, dim=-1, descending=True)
    before = torch.cumsum(sorted_p, dim=-1) - sorted_p
    sorted_p = sorted_p.masked_fill(before > p, 0.0)
    sorted_p = sorted_p / sorted_p.sum(dim=-1, keepdim=True)
    pick = torch.multinomial(sorted_p, num_samples=1)
    return torch.gather(order, -1, pick)


@torch.inference_mode()
def generate(model, dtype: str, tokenizer, prompt: Optional[List[str]] = None, max_prompt_len: int = 256,
             max_gen_len: int = 256, use_sampling: bool = False, temp: float = 1.0, top_k: int = 0,
             top_p: float = 0.0, remove_prompts: bool = True,
             truncate_chunks: Optional[int] = None,
             use_decode_session: Optional[bool] = None) -> List[List[int]]:
    """`use_decode_session`: run the one-token steps through `decoding.DecodeSession` (fixed-shape
    state, replayed from a CUDA graph on a single GPU) instead of the growing-cache path; same tokens,
    a fraction of the per-token cost.  Default: on for CUDA models without tensor parallelism."""
    model.eval()
    device = next(model.parameters()).device
    if prompt is not None:
        prompt_tokens = [tokenizer.encode(t, bos=True, eos=False) for t in prompt]
        n_truncated = sum(max_prompt_len < len(t) for t in prompt_tokens)
    else:
        prompt_tokens, n_truncated = None, 0
    total_truncated = reduce_scalar(n_truncated, op="sum") if _dist_on() else n_truncated
    if total_truncated > 0:
        logger.info(f"There are {total_truncated} prompts that are truncated on the left, length greater "
                    f"than max_prompt_len = {max_prompt_len}, maximum prompt length = "
                    f"{get_max_length(prompt_tokens)} across all gpus.")
    if prompt_tokens is not None:
        prompt_tokens = [t if len(t) < max_prompt_len else t[len(t) - max_prompt_len:] for t in prompt_tokens]

    start_pos, end_pos = get_generation_range(prompt_tokens, max_gen_len)
    if prompt_tokens is None:       # padding example so every rank runs the same number of steps
        prompt_tokens = [[tokenizer.bos_id] * end_pos]
    bsz = len(prompt_tokens)
    if truncate_chunks is not None:
        assert bsz == 1 and get_data_parallel_world_size() == 1 and truncate_chunks > 0 and remove_prompts

    tokens = torch.full((bsz, end_pos), tokenizer.pad_id, dtype=torch.long, device=device)
    for k, t in enumerate(prompt_tokens):
        tokens[k, :len(t)] = torch.tensor(t, dtype=torch.long, device=device)
    prompt_mask = tokens != tokenizer.pad_id
    if model_parallel_is_initialized():
        check_same_in_process_group(tokens, name="prompt_tokens", group_name="model",
                                    group=get_model_parallel_group())

    c = model.chunk_size
    remainder = 0
    if truncate_chunks is not None and end_pos > truncate_chunks * c:
        remainder = end_pos % c
        tokens, prompt_mask = tokens[:, remainder:], prompt_mask[:, remainder:]
        start_pos, end_pos = start_pos - remainder, end_pos - remainder

    compute_dtype = get_torch_dtype(dtype)
    cache = init_cache(bsz, model, compute_dtype, device=device)
    n_chunks = (start_pos - 1) // c
    prev_pos = n_chunks * c
    for first in range(0, n_chunks, MAX_CHUNKS_PER_BATCH):
        s, e = first * c, min(first + MAX_CHUNKS_PER_BATCH, n_chunks) * c
        _, cache = model(tokens[:, s:e], cache=cache)
        if TRUNCATE_CHUNKS * c <= e:
            ss = e - (TRUNCATE_CHUNKS - MAX_CHUNKS_PER_BATCH) * c
            fresh = init_cache(bsz, model, compute_dtype, truncate=True, device=device)
            _, stats_only = model(tokens[:, ss:e], cache=fresh)
            cache = truncate_cache(cache, stats_only)

    logger.debug(f"prev_pos={prev_pos}, start_pos={start_pos}, end_pos={end_pos}")
    if use_decode_session is None:
        tensor_parallel = model_parallel_is_initialized() and \
            torch.distributed.get_world_size(get_model_parallel_group()) > 1
        use_decode_session = device.type == "cuda" and not tensor_parallel
    session = None
    for cur in range(start_pos, end_pos):
        if session is not None:
            logits = session.step(tokens[:, prev_pos])
        else:
            logits, cache = model(tokens[:, prev_pos:cur], cache=cache)
            logits = logits[:, -1]
            if use_decode_session:
                # from here on every call feeds exactly one token: switch to the fixed-shape state
                from .decoding import DecodeSession
                session = DecodeSession(model, bsz, compute_dtype)
                session.load_cache(cache)
        if use_sampling:
            probs = torch.softmax(logits / temp, dim=-1)
            if top_p > 0.0:
                nxt = sample_top_p(probs, top_p)
            elif top_k > 0:
                nxt = sample_top_k(probs, top_k)
            else:
                nxt = torch.multinomial(probs, num_samples=1)
            nxt = nxt.reshape(-1)
        else:
            nxt = torch.argmax(logits, dim=-1)
        # inside the prompt the given token wins
        tokens[:, cur] = torch.where(prompt_mask[:, cur], tokens[:, cur], nxt)
        prev_pos = cur

    out = []
    for i, row in enumerate(tokens):
        n = len(prompt_tokens[i]) - remainder
        out.append(row[n:n + max_gen_len].tolist() if remove_prompts else row[:n + max_gen_len].tolist())
    return out
