"""Checkpoints.

Reading follows the reference layout (megalodon/reloading.py:66-245):

    <dir>/config.json              {"tokenizer": {...}, "model": {...}, [training run:
                                    "model_parallel_size", "chunk_parallel_size", "slurm": {"world_size"}]}
    <dir>/consolidate_config.json  {"model_parallel_size": int, "dtype": str}   (marks "consolidated")
    <dir>/consolidated.pth         mp == 1
    <dir>/consolidated.NN.pth      mp  > 1, one file per model-parallel rank
    <dir>/model.ckpt.RRRRR.pth     sharded training checkpoint, one file per global rank

The reference can only *load consolidated* checkpoints.  This module also
writes both kinds (`save_consolidated`, `save_sharded`) and reloads sharded
ones including optimiser state, step counter and RNG state
(`load_sharded`), which is what `train.py --resume` uses.
"""
from __future__ import annotations

import json
import logging
import os
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Any, Dict, Optional, Tuple

import torch
import torch.distributed as dist

from .config import ModelConf, TokenizerConf
from .models.mega import Mega, build_model  # noqa: F401  (re-exported like the reference)
from .parallel import (
    get_chunk_parallel_world_size,
    get_data_parallel_rank,
    get_data_parallel_world_size,
    get_model_parallel_rank,
    get_model_parallel_world_size,
    init_signal_handler,
    init_torch_distributed,
    initialize_model_parallel,
    model_parallel_is_initialized,
)
from .utils import default_device, get_default_half, get_torch_dtype

logger = logging.getLogger()


@dataclass
class ReloadedConf:
    world_size: int
    dp_world_size: int
    mp_world_size: int
    cp_world_size: int
    dtype: str
    is_fsdp: bool
    cfg: Dict[str, Any]

    def new_mp_world_size(self, model_parallel_size: Optional[int]) -> int:
        return self.mp_world_size if model_parallel_size is None else model_parallel_size

    def new_cp_world_size(self, chunk_parallel_size: Optional[int]) -> int:
        return self.cp_world_size if chunk_parallel_size is None else chunk_parallel_size

    def __post_init__(self):
        if self.is_fsdp:
            assert self.dtype == "fp32"
        else:
            assert self.mp_world_size == self.world_size // self.cp_world_size
            assert self.dp_world_size == 1


def model_ckpt_name(rank: int) -> str:
    return f"model.ckpt.{rank:05d}.pth"


def get_consolidated_ckpt_path(ckpt_dir: Path, mp_rank: int = 0, mp_size: int = 1) -> Path:
    if mp_size == 1:
        assert mp_rank == 0
        return Path(ckpt_dir) / "consolidated.pth"
    return Path(ckpt_dir) / f"consolidated.{mp_rank:02d}.pth"


def _is_consolidated_ckpt(ckpt_dir: Path) -> bool:
    return (Path(ckpt_dir) / "consolidate_config.json").exists()


def reload_config(ckpt_dir: Path) -> ReloadedConf:
    ckpt_dir = Path(ckpt_dir)
    with (ckpt_dir / "config.json").open() as fp:
        cfg = json.load(fp)
    if _is_consolidated_ckpt(ckpt_dir):
        with (ckpt_dir / "consolidate_config.json").open() as fp:
            ccfg = json.load(fp)
        mp = int(ccfg["model_parallel_size"])
        return ReloadedConf(world_size=mp, dp_world_size=1, mp_world_size=mp, cp_world_size=1,
                            dtype=ccfg["dtype"], is_fsdp=False, cfg=cfg)
    mp = int(cfg["model_parallel_size"])
    cp = int(cfg.get("chunk_parallel_size", 1))
    world = int(cfg["slurm"]["world_size"])
    assert 0 < mp <= world and world % mp == 0
    return ReloadedConf(world_size=world, dp_world_size=world // mp // cp, mp_world_size=mp,
                        cp_world_size=cp, dtype="fp32", is_fsdp=True, cfg=cfg)


def reload_config_and_tokenizer(ckpt_dir: Path, tokenizer_path: Optional[str] = None):
    from .data.tokenizer import Tokenizer
    reloaded = reload_config(ckpt_dir)
    cfg = reloaded.cfg
    tok_cfg = TokenizerConf(**cfg["tokenizer"])
    if tokenizer_path is not None:
        tok_cfg.path = tokenizer_path
    assert tok_cfg.path is not None and Path(tok_cfg.path).exists(), tok_cfg.path
    tokenizer = Tokenizer(tokenizer_cfg=tok_cfg)
    known = {f for f in ModelConf.__dataclass_fields__}
    model_cfg = ModelConf(**{k: v for k, v in cfg["model"].items() if k in known})
    model_cfg.init_mode = "none"
    # training-time memory settings have no place in the evaluation model
    model_cfg.layerwise_ckpt = False
    model_cfg.ckpt_layers = None
    if model_cfg.vocab_size == -1:          # old checkpoints do not record it
        model_cfg.vocab_size = tokenizer.n_words
    assert model_cfg.vocab_size == tokenizer.n_words, (tokenizer.n_words, model_cfg.vocab_size)
    return reloaded, tokenizer, model_cfg


def init_distributed_mode(model_parallel_size: int, chunk_parallel_size: int) -> None:
    init_signal_handler()
    logger.info("Starting init of torch.distributed...")
    info = init_torch_distributed()
    logger.info("Done init of torch.distributed.")
    logger.info("Starting init of model parallel...")
    if not model_parallel_is_initialized():
        initialize_model_parallel(model_parallel_size, chunk_parallel_size)
    logger.info("Done init of model parallel.")
    if info.is_slurm:
        logger.info(f"ENV: {os.environ}")
        logger.info(f"CUDA version: {torch.version.cuda}")


def build_consolidated_model(model_cfg: ModelConf, dtype: str) -> Mega:
    """Un-sharded inference model in `dtype` on the default device."""
    logger.info("Start: building consolidated model...")
    model = Mega(model_cfg).to(get_torch_dtype(dtype)).to(default_device())
    logger.info("Done: building consolidated model.")
    return model


def load_state_dict(model: Mega, state_dict: Dict, strict: bool) -> None:
    """Missing or unexpected *buffers* are logged (older checkpoints lack some); a missing
    *parameter* is an error even with `strict=False` - the model is built with `init_mode='none'`,
    so a weight that is not in the file would stay uninitialised memory."""
    missing, unexpected = model.load_state_dict(state_dict, strict=strict)
    if missing:
        logger.warning(f"Missing keys when reloading: {missing}")
    if unexpected:
        logger.warning(f"Unexpected keys when reloading: {unexpected}")
    params = {name for name, _ in model.named_parameters()}
    lost = [k for k in missing if k in params]
    if lost:
        raise RuntimeError(f"checkpoint has no value for {len(lost)} parameter(s), e.g. {lost[:4]}; "
                           f"keys it has that the model does not: {list(unexpected)[:4]}")


def load_consolidated_weights(ckpt_dir: Path, model: Mega, reloaded: ReloadedConf, dtype: str) -> None:
    assert not reloaded.is_fsdp
    if dtype != reloaded.dtype:
        logger.warning(f"Asking dtype: {dtype} when consolidated ckpt has dtype: {reloaded.dtype}")
    mp = get_model_parallel_world_size()
    if mp != reloaded.mp_world_size:
        raise ValueError(f"Asking model_parallel_size: {mp} when checkpoint was consolidated with "
                         f"model_parallel_size: {reloaded.mp_world_size}")
    path = get_consolidated_ckpt_path(Path(ckpt_dir), get_model_parallel_rank(), mp)
    logger.info("Loading consolidated ckpt...")
    state = torch.load(path, map_location="cpu", weights_only=True)
    logger.info("Done loading consolidated ckpt")
    load_state_dict(model, state, strict=False)
    logger.info("Done with state-dict reloading.")


def reload_model(checkpoint_dir: str, init_distributed: bool = True,
                 model_parallel_size: Optional[int] = None, chunk_parallel_size: Optional[int] = None,
                 dtype: str = get_default_half(), tokenizer_path: Optional[str] = None):
    ckpt_dir = Path(checkpoint_dir)
    reloaded, tokenizer, model_cfg = reload_config_and_tokenizer(ckpt_dir, tokenizer_path)
    new_mp = reloaded.new_mp_world_size(model_parallel_size)
    new_cp = reloaded.new_cp_world_size(chunk_parallel_size)
    if init_distributed:
        init_distributed_mode(new_mp, new_cp)
    assert new_mp == get_model_parallel_world_size(), f"{new_mp} != {get_model_parallel_world_size()}"
    assert new_cp == get_chunk_parallel_world_size(), f"{new_cp} != {get_chunk_parallel_world_size()}"
    assert _is_consolidated_ckpt(ckpt_dir), \
        "only consolidated checkpoints can be reloaded for evaluation; run `consolidate` first"
    logger.info(f"Reloading consolidated model -- Path={ckpt_dir} -- MP={new_mp}")
    model = build_consolidated_model(model_cfg, dtype)
    load_consolidated_weights(ckpt_dir, model, reloaded, dtype)
    return model, tokenizer, reloaded


# ---------------------------------------------------------------------------- re-slicing for tensor parallelism
def shard_state_dict_for_model_parallel(state: Dict[str, torch.Tensor], num_heads: int, mp_rank: int,
                                        mp_size: int) -> Dict[str, torch.Tensor]:
    """Slice a full (model_parallel_size = 1) state dict down to what tensor-parallel rank `mp_rank` of
    `mp_size` holds, following how each layer partitions itself:

      output features (rows)   wv, wr, wh1, fc1, fc3 (+ biases), TimestepNorm weight / bias / priors,
                               CEMA parameters, the layer scale `nffn.alpha`
      input features (columns) wh2, fc2, the vocabulary projection, the embedding table
      by head                  wz (+ bias) rows and gamma / beta columns; with more ranks than heads
                               each head's slice is replicated on the mp_size / num_heads ranks that
                               share the head
      replicated               RMSNorm and LayerNorm weights (they act on gathered features), rope

    The reference can only load a consolidated checkpoint at the tensor-parallel size it was written
    with (reloading.py:117-122); this makes an mp = 1 file usable at any size, including sizes above
    the number of heads."""
    if mp_size == 1:
        return dict(state)

    def cut(t: torch.Tensor, dim: int, index: int = mp_rank, count: int = mp_size) -> torch.Tensor:
        n = t.size(dim) // count
        assert n * count == t.size(dim), (tuple(t.shape), dim, count)
        return t.narrow(dim, index * n, n).contiguous()

    head_split = max(1, mp_size // num_heads)
    by_head = (mp_rank // head_split, num_heads) if mp_size > num_heads else (mp_rank, mp_size)
    out: Dict[str, torch.Tensor] = {}
    for key, t in state.items():
        leaf = key.rsplit(".", 2)[-2:] if key.count(".") else [key]
        mod, name = (leaf[0], leaf[1]) if len(leaf) == 2 else ("", leaf[0])
        if mod in ("rmsnorm", "norm", "rope") or t.dim() == 0:
            out[key] = t
        elif mod == "wz":
            out[key] = cut(t, 0, *by_head)
        elif name in ("gamma", "beta") and mod == "mega":
            out[key] = cut(t, 1, *by_head)
        elif mod in ("wv", "wr", "wh1", "fc1", "fc3", "timenorm", "final_norm", "cema") or key.endswith("nffn.alpha"):
            out[key] = cut(t, 0)
        elif mod in ("wh2", "fc2", "output", "embed"):
            out[key] = cut(t, 1) if t.dim() == 2 else t
        else:
            raise KeyError(f"no tensor-parallel slicing rule for {key!r} of shape {tuple(t.shape)}")
    return out


# ---------------------------------------------------------------------------- writing
def _write_config(ckpt_dir: Path, model_cfg: ModelConf, tokenizer_cfg: Optional[TokenizerConf],
                  extra: Optional[Dict[str, Any]] = None) -> None:
    cfg: Dict[str, Any] = {
        "tokenizer": asdict(tokenizer_cfg) if tokenizer_cfg is not None else asdict(TokenizerConf()),
        "model": asdict(model_cfg),
    }
    cfg.update(extra or {})
    with (ckpt_dir / "config.json").open("w") as fp:
        json.dump(cfg, fp, indent=2)


def _is_writer() -> bool:
    return not (dist.is_available() and dist.is_initialized()) or dist.get_rank() == 0


def save_consolidated(model, ckpt_dir: str, model_cfg: ModelConf,
                      tokenizer_cfg: Optional[TokenizerConf] = None, dtype: str = "bf16") -> None:
    """Write `consolidated[.NN].pth` (+ both json files) from an FSDP-wrapped or a
    plain model.  Every rank of the sharding group must call this."""
    ckpt_dir = Path(ckpt_dir)
    ckpt_dir.mkdir(parents=True, exist_ok=True)
    state = model.state_dict()
    tdtype = get_torch_dtype(dtype)
    state = {k: (v.to(tdtype) if v.is_floating_point() else v).cpu() for k, v in state.items()}
    mp = get_model_parallel_world_size()
    first_replica = get_data_parallel_rank() == 0
    if model_parallel_is_initialized():
        from .parallel import get_chunk_parallel_rank
        first_replica = first_replica and get_chunk_parallel_rank() == 0
    if first_replica:
        torch.save(state, get_consolidated_ckpt_path(ckpt_dir, get_model_parallel_rank(), mp))
    if _is_writer():
        _write_config(ckpt_dir, model_cfg, tokenizer_cfg)
        with (ckpt_dir / "consolidate_config.json").open("w") as fp:
            json.dump({"model_parallel_size": mp, "dtype": dtype}, fp)
    if dist.is_available() and dist.is_initialized():
        dist.barrier()


def save_sharded(model, optimizer, scheduler, step: int, ckpt_dir: str, model_cfg: ModelConf,
                 tokenizer_cfg: Optional[TokenizerConf] = None) -> None:
    """One `model.ckpt.RRRRR.pth` per global rank: this rank's fp32 shards,
    optimiser state, scheduler state, step and RNG state."""
    ckpt_dir = Path(ckpt_dir)
    ckpt_dir.mkdir(parents=True, exist_ok=True)
    rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
    world = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
    payload = {
        "model": model.local_state_dict(),
        "optimizer": optimizer.state_dict() if optimizer is not None else None,
        "scheduler": scheduler.state_dict() if scheduler is not None else None,
        "step": int(step),
        "rng": {"cpu": torch.get_rng_state(),
                "cuda": torch.cuda.get_rng_state() if torch.cuda.is_available() else None},
    }
    tmp = ckpt_dir / (model_ckpt_name(rank) + ".tmp")
    torch.save(payload, tmp)
    os.replace(tmp, ckpt_dir / model_ckpt_name(rank))
    if _is_writer():
        _write_config(ckpt_dir, model_cfg, tokenizer_cfg, {
            "model_parallel_size": get_model_parallel_world_size(),
            "chunk_parallel_size": get_chunk_parallel_world_size(),
            "slurm": {"world_size": world},
            "step": int(step),
        })
    if world > 1:
        dist.barrier()


def load_sharded(model, optimizer, scheduler, ckpt_dir: str) -> int:
    """Inverse of `save_sharded` (same world size and parallel layout). Returns the step."""
    rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
    payload = torch.load(Path(ckpt_dir) / model_ckpt_name(rank), map_location="cpu", weights_only=False)
    model.load_local_state_dict(payload["model"])
    if optimizer is not None and payload["optimizer"] is not None:
        optimizer.load_state_dict(payload["optimizer"])
    if scheduler is not None and payload["scheduler"] is not None:
        scheduler.load_state_dict(payload["scheduler"])
    torch.set_rng_state(payload["rng"]["cpu"])
    if payload["rng"]["cuda"] is not None and torch.cuda.is_available():
        torch.cuda.set_rng_state(payload["rng"]["cuda"])
    return int(payload["step"])


def consolidate(sharded_dir: str, out_dir: str, dtype: str = "bf16") -> None:
    """Offline: merge the `model.ckpt.*.pth` files of a training run into
    `consolidated[.NN].pth` files (one per model-parallel rank), on the CPU."""
    src, dst = Path(sharded_dir), Path(out_dir)
    dst.mkdir(parents=True, exist_ok=True)
    with (src / "config.json").open() as fp:
        cfg = json.load(fp)
    mp = int(cfg["model_parallel_size"])
    cp = int(cfg.get("chunk_parallel_size", 1))
    world = int(cfg["slurm"]["world_size"])
    tdtype = get_torch_dtype(dtype)
    for mp_rank in range(mp):
        # global ranks that share this model-parallel slice, in sharding-group order
        members = [r for r in range(world) if r % mp == mp_rank]
        payloads = {r: torch.load(src / model_ckpt_name(r), map_location="cpu", weights_only=False)["model"]
                    for r in members}
        first = payloads[members[0]]
        state: Dict[str, torch.Tensor] = {}
        for unit, meta in first["meta"].items():
            shard_world = meta["world_size"]
            by_rank = {payloads[r]["meta"][unit]["rank"]: payloads[r]["shards"][unit] for r in members}
            prefix = "" if unit == "_root" else unit + "."
            # rank r's shard holds piece r of every parameter at the same shard offset
            for name, shape, _offset, piece, shard_offset in meta["params"]:
                n = 1
                for s in shape:
                    n *= s
                whole = torch.cat([by_rank[i][shard_offset:shard_offset + piece] for i in range(shard_world)])
                state[prefix + name] = whole[:n].view(shape).to(tdtype).clone()
        for name, buf in first["buffers"].items():
            state[name] = buf.to(tdtype) if buf.is_floating_point() else buf
        # tied embedding: expose the shared tensor under both names
        if cfg["model"].get("share_emb") and "embed.weight" in state:
            state["output.output.weight"] = state["embed.weight"]
        torch.save(state, get_consolidated_ckpt_path(dst, mp_rank, mp))
    out_cfg = {"tokenizer": cfg["tokenizer"], "model": cfg["model"]}
    with (dst / "config.json").open("w") as fp:
        json.dump(out_cfg, fp, indent=2)
    with (dst / "consolidate_config.json").open("w") as fp:
        json.dump({"model_parallel_size": mp, "dtype": dtype}, fp)
    del cp
