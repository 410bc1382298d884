"""SentencePiece tokenizer with an optional block of extra ids appended after
the model's own vocabulary (a multiple of 256) from which BOS / EOS / PAD are
taken when the SentencePiece model does not define them (reference:
megalodon/data/tokenizer.py:11-101)."""
from __future__ import annotations

import logging
import os
from typing import List, Optional, Union

from ..config import TokenizerConf

logger = logging.getLogger()


class Tokenizer:
    def __init__(self, tokenizer_cfg: TokenizerConf):
        from sentencepiece import SentencePieceProcessor
        path = tokenizer_cfg.tokenizer_path
        assert os.path.isfile(path), path
        self.sp_model = SentencePieceProcessor(model_file=path)
        logger.info(f"Reloaded SentencePiece model from {path}")
        extra = tokenizer_cfg.additional_vocab_size
        assert extra % 256 == 0, f"additional vocab size is not multiple of 256: {extra}"
        self.additional_vocab_size = extra
        self.sp_model_vocab_size = self.sp_model.vocab_size()
        assert self.sp_model_vocab_size == self.sp_model.get_piece_size()
        self.already_tokenized_data = tokenizer_cfg.data_tokenized
        self.n_words: int = self.sp_model_vocab_size + extra
        self.used_special_tokens = 0
        # resolved in this order, so extra ids are handed out BOS, EOS, PAD
        self._bos_id = self._special(self.sp_model.bos_id())
        self._eos_id = self._special(self.sp_model.eos_id())
        self._pad_id = self._special(self.sp_model.pad_id())
        logger.info(f"#words: {self.n_words} - BOS ID: {self.bos_id} - EOS ID: {self.eos_id} "
                    f"- PAD ID: {self.pad_id}")

    def _special(self, sp_id: int) -> int:
        if sp_id != -1 or self.additional_vocab_size == 0:
            return sp_id
        new_id = self.sp_model_vocab_size + self.used_special_tokens
        self.used_special_tokens += 1
        return new_id

    @property
    def bos_id(self) -> int:
        return self._bos_id

    @property
    def eos_id(self) -> int:
        return self._eos_id

    @property
    def pad_id(self) -> int:
        return self._pad_id

    def encode(self, s: Union[str, List[int]], bos: bool, eos: bool) -> List[int]:
        if self.already_tokenized_data:
            t = list(s)
        else:
            assert isinstance(s, str)
            t = self.sp_model.encode(s)
        if bos:
            t.insert(0, self.bos_id)
        if eos:
            t.append(self.eos_id)
        return t

    def encode_str(self, s: str) -> List[str]:
        assert isinstance(s, str)
        return self.sp_model.encode(s, out_type=str)

    def decode(self, tokens: List[int], cut_at_eos: bool = True) -> str:
        if cut_at_eos and self.eos_id in tokens:
            tokens = tokens[:tokens.index(self.eos_id) + 1]
        tokens = [t for t in tokens if 0 <= t < self.sp_model_vocab_size]
        return self.sp_model.decode(tokens)
