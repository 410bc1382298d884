"""Configuration dataclasses.

Field names and defaults follow the reference (megalodon/config.py:12-118) so
that a `config.json` written next to a reference checkpoint can be splatted
into these classes unchanged.  `TrainerConf` is new: the reference README only
sketches it (README.md:106); it is the config consumed by `train.py`.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field, asdict
from pathlib import Path
from typing import List, Optional

_ATTN_IMPLS = (None, "swift", "fused")


@dataclass
class TokenizerConf:
    path: Optional[str] = None
    additional_vocab_size: int = 0
    data_tokenized: bool = False

    @property
    def tokenizer_path(self) -> str:
        if self.path is None or not os.path.isfile(self.path):
            raise FileNotFoundError(f"tokenizer model not found: {self.path}")
        return self.path


@dataclass
class OptimConf:
    # AdamW on the fp32 master shards
    lr: float = 1e-3                 # peak learning rate, reached after `warmup` steps
    warmup: int = 2000               # linear warm-up steps starting from lr * lr_init_ratio
    weight_decay: float = 0.1        # decoupled
    epsilon: float = 1e-8
    beta1: float = 0.9
    beta2: float = 0.98
    clip: float = 1.0                # global-norm clipping threshold; 0 disables clipping
    # schedule after warm-up: "linear" | "cosine" | "constant"
    scheduler: str = "linear"
    lr_init_ratio: float = 1e-4
    lr_end_ratio: float = 0.01       # final lr as a fraction of the peak
    cycles: float = 1.0              # cosine cycles over the decay phase


@dataclass
class ModelConf:
    # ---- sizes
    num_layers: int = 8
    model_dim: int = 1024            # residual stream D
    z_dim: int = 256                 # shared query/key width S (all heads together)
    value_dim: int = 2048            # value / gate width E (all heads together)
    num_heads: int = 1
    ffn_hidden_dim: int = 2048
    cema_ndim: int = 16              # complex EMA states per feature
    chunk_size: int = 2048           # attention never crosses a chunk
    vocab_size: int = -1             # -1: filled in from the tokenizer
    output_size: int = -1            # -1: same as vocab_size
    # ---- attention implementation: None = unfused (post-softmax dropout), "swift" / "fused" = kernels (DropKey)
    efficient_attn: Optional[str] = None
    init_mode: str = "he"            # none | bert | he | gaussian | xavier
    # ---- normalisation
    norm_num_groups: int = 32        # TimestepNorm groups
    norm_affine: bool = True
    norm_eps: float = 1e-5
    rope_base: Optional[float] = None
    # ---- regularisation
    dropout: float = 0.0
    hidden_dropout: float = 0.0
    attention_dropout: float = 0.0
    # ---- variants
    swiglu: bool = False             # SiLU(fc1 x) * fc3 x instead of SiLU(fc1 x)
    rescale_nffn: bool = False       # learnable per-layer scale 0.1 * 0.5^layer on the FFN branch
    scale_emb: bool = False          # multiply embeddings by sqrt(D)
    share_emb: bool = False          # tie output projection and embedding
    layerwise_ckpt: bool = False     # activation checkpointing per block
    # with layerwise_ckpt: checkpoint only the first `ckpt_layers` blocks (None = all of them); the
    # rest keep their activations, which trades spare memory for less recomputation
    ckpt_layers: Optional[int] = None

    def __post_init__(self):
        # The reference checks `z_dim % z_dim` (always true, config.py:73); the
        # intended constraint is divisibility by the head count.
        if self.z_dim % self.num_heads or self.value_dim % self.num_heads:
            raise ValueError("z_dim and value_dim must be divisible by num_heads")
        for name in ("dropout", "hidden_dropout", "attention_dropout"):
            p = getattr(self, name)
            if not 0.0 <= p < 1.0:
                raise ValueError(f"{name}={p} outside [0, 1)")
        if self.efficient_attn not in _ATTN_IMPLS:
            raise ValueError(f"efficient_attn must be one of {_ATTN_IMPLS}")

    def to_dict(self):
        return asdict(self)


@dataclass
class ValidConf:
    ppl_files_str: str = ""
    prompt_path: str = ""
    batch_size: int = 1
    use_sampling: bool = False
    temperature: float = 1.0
    top_k: int = 0
    top_p: float = 0.0
    gen_seq_len: int = 8192

    @property
    def ppl_files(self) -> List[str]:
        return [p for p in self.ppl_files_str.split(",") if p]

    def __post_init__(self):
        if self.temperature < 0 or self.top_k < 0 or not 0 <= self.top_p < 1:
            raise ValueError("invalid decoding parameters")
        files = self.ppl_files
        if files:
            if len(set(files)) != len(files):
                raise ValueError("duplicate PPL files")
            for p in files:
                if not p.endswith(".jsonl") or not Path(p).is_file():
                    raise FileNotFoundError(p)
        if self.prompt_path:
            if not self.prompt_path.endswith(".jsonl") or not os.path.isfile(self.prompt_path):
                raise FileNotFoundError(self.prompt_path)


@dataclass
class TrainerConf:
    """Everything `train.py` needs: the README loop's implied fields."""
    model: ModelConf = field(default_factory=ModelConf)
    optim: OptimConf = field(default_factory=OptimConf)
    tokenizer: TokenizerConf = field(default_factory=TokenizerConf)
    steps: int = 100
    dtype: str = "bf16"
    model_parallel_size: int = 1
    chunk_parallel_size: int = 1
    fp32_reduce_scatter: bool = False
    reshard_after_forward: bool = True
    batch_size: int = 1            # sequences per data-parallel rank
    seq_len: int = 4096            # full sequence length (before chunk-parallel split)
    seed: int = 0
    data_path: Optional[str] = None  # jsonl; synthetic tokens when None
    dump_dir: Optional[str] = None
    save_every: int = 0
    log_every: int = 1
    resume: bool = False
