"""Tracing and metrics (the reference has none; its requirements.txt lists
wandb/tqdm but never imports them).

* `nvtx_range(name)` - NVTX ranges around layers / ops when `MEGALODON_B200_NVTX=1`.
* `StepTimer` - device-side step timing with CUDA events, max over ranks.
* `MetricsWriter` - one JSON line per step (loss, grad-norm, tokens/s, step ms,
  bytes moved by collectives) appended to a file by rank 0.
* `model_flops_per_token` / `roofline_fraction` - achieved versus the measured
  peaks of the machine (`MEASURED_PEAKS.json` written by the benchmark driver).
"""
from __future__ import annotations

import contextlib
import json
import os
import time
from typing import Any, Dict, Optional

import torch
import torch.distributed as dist

_NVTX = os.environ.get("MEGALODON_B200_NVTX", "0") == "1"


@contextlib.contextmanager
def nvtx_range(name: str):
    if _NVTX and torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


class StepTimer:
    """Times consecutive steps on the device; `stop()` returns milliseconds, maximum over ranks."""

    def __init__(self, group: Optional[dist.ProcessGroup] = None):
        self.group = group
        self.cuda = torch.cuda.is_available()
        self._t0 = None
        if self.cuda:
            self._e0 = torch.cuda.Event(enable_timing=True)
            self._e1 = torch.cuda.Event(enable_timing=True)

    def start(self) -> None:
        if self.cuda:
            self._e0.record()
        else:
            self._t0 = time.perf_counter()

    def stop(self) -> float:
        if self.cuda:
            self._e1.record()
            self._e1.synchronize()
            ms = self._e0.elapsed_time(self._e1)
        else:
            ms = (time.perf_counter() - self._t0) * 1e3
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(self.group) > 1:
            from ..parallel.utils import comm_device
            t = torch.tensor(ms, dtype=torch.float64, device=comm_device(self.group))
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
            ms = float(t.item())
        return ms


class MetricsWriter:
    def __init__(self, path: Optional[str]):
        self.path = path
        self.enabled = path is not None and (not dist.is_initialized() or dist.get_rank() == 0)
        if self.enabled:
            os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)

    def write(self, **fields: Any) -> None:
        if not self.enabled:
            return
        with open(self.path, "a") as fp:
            fp.write(json.dumps(fields) + "\n")


def model_flops_per_token(cfg, seq_chunk: Optional[int] = None, with_recompute: bool = False) -> float:
    """Forward + backward FLOPs per token of a Megalodon model (matrix products only):
    6 x (projection parameters) + causal chunk attention."""
    d, s, e, f = cfg.model_dim, cfg.z_dim, cfg.value_dim, cfg.ffn_hidden_dim
    per_layer = d * s + 2 * d * e + d * d + e * d + (3 if cfg.swiglu else 2) * d * f
    c = seq_chunk or cfg.chunk_size
    attn = (s + e) * c / 2.0                    # MACs per token per layer, causal half of the chunk
    macs = cfg.num_layers * (per_layer + attn) + d * (cfg.vocab_size if cfg.output_size == -1 else cfg.output_size)
    mult = 4.0 if with_recompute else 3.0       # fwd + bwd (2x) [+ recomputed fwd]
    return 2.0 * macs * mult


def measured_peaks(path: Optional[str] = None) -> Dict[str, float]:
    """Copy bandwidth (GB/s) and cuBLAS bf16 throughput (TFLOP/s) measured on this pool; falls back
    to an earlier measurement when the driver-written file is absent."""
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = path or os.path.join(here, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fp:
            d = json.load(fp)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def roofline_fraction(flops: float, bytes_moved: float, seconds: float, sustained: bool = True) -> Dict[str, float]:
    pk = measured_peaks()
    tf = pk["bf16_tflops_sustained" if sustained else "bf16_tflops"] * 1e12
    t_min = max(flops / tf, bytes_moved / (pk["hbm_gbs"] * 1e9))
    return {"fraction": t_min / seconds if seconds > 0 else 0.0, "of": pk["source"]}
