"""JSONL data loading.

`DataLoader` is the evaluation reader of the reference
(megalodon/data/dataloader.py:13-73): line i of the file belongs to rank
`i % world_size`; each example gives `x = tokens[:-1]`, `y = tokens[1:]`;
batches are right-padded (x with 0, y with -100) and over-long rows keep their
tail.  `SyntheticTokens` yields uniform-random token batches from pinned host
memory for benchmarks and smoke runs.
"""
from __future__ import annotations

import json
import logging
from typing import Dict, Iterator, List

import torch

from ..utils import pad

logger = logging.getLogger()


class DataLoader:
    def __init__(self, tokenizer, path: str, batch_size: int, world_rank: int, world_size: int):
        self.tokenizer = tokenizer
        self.world_rank = world_rank
        self.world_size = world_size
        self.path = path
        self.batch_size = batch_size
        self.jsonl_file = open(path, "r", encoding="utf-8")
        self.line_num = 0

    def __iter__(self) -> Iterator[Dict[str, torch.Tensor]]:
        xs: List[List[int]] = []
        ys: List[List[int]] = []
        for line in self.jsonl_file:
            self.line_num += 1
            if (self.line_num - 1) % self.world_size != self.world_rank:
                continue
            try:
                toks = self.tokenizer.encode(json.loads(line)["text"], bos=True, eos=True)
            except Exception:  # noqa: BLE001 - a bad line must not end the evaluation
                logger.error(f"Error when trying to load line {self.line_num} in {self.path}")
                continue
            xs.append(toks[:-1])
            ys.append(toks[1:])
            if len(xs) == self.batch_size:
                yield self.build_batch({"x": xs, "y": ys})
                xs, ys = [], []
        if xs:
            yield self.build_batch({"x": xs, "y": ys})

    def build_batch(self, batch: Dict[str, List[List[int]]]) -> Dict[str, torch.Tensor]:
        return {"x": self.to_tensor(batch["x"], 0), "y": self.to_tensor(batch["y"], -100)}

    @staticmethod
    def to_tensor(rows: List[List[int]], pad_value: int) -> torch.Tensor:
        width = max(len(r) for r in rows)
        return torch.tensor([pad(r, max_length=width, value=pad_value, truncating="pre") for r in rows],
                            dtype=torch.long)

    def close(self) -> None:
        self.jsonl_file.close()


class SyntheticTokens:
    """Endless stream of (x, y) next-token batches of uniform-random ids held in
    pinned host memory (when CUDA is present), `batch_size x seq_len` each."""

    def __init__(self, vocab_size: int, batch_size: int, seq_len: int, seed: int = 0, n_buffers: int = 4):
        g = torch.Generator().manual_seed(seed)
        self.buffers = []
        for _ in range(n_buffers):
            t = torch.randint(0, vocab_size, (batch_size, seq_len + 1), generator=g, dtype=torch.long)
            if torch.cuda.is_available():
                t = t.pin_memory()
            self.buffers.append(t)
        self._i = 0

    def __iter__(self):
        return self

    def __next__(self):
        t = self.buffers[self._i % len(self.buffers)]
        self._i += 1
        return t[:, :-1], t[:, 1:]
