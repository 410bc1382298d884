"""Token-by-token decoding against a fixed-shape state, replayed from a CUDA graph.

The regular cache path (`Mega.forward(tokens, cache)`, reference:
megalodon/model/mega.py:190-233 and generation.py:105-125) grows the key/value
tail by concatenation and tracks lengths in Python, so every token costs a few
hundred eager kernel launches: the 7B model spends about 40 ms of host time per
token.  A `DecodeSession` keeps the whole recurrent state in buffers whose
shapes never change -

    per layer   k, v [B, H, chunk, d]   chunk-local keys / values (entries past `pos` are masked)
                count [B], mean, var [B, G]   TimestepNorm running statistics
                hx [B, D, N] complex          CEMA state
    output norm count, mean, var
    pos [1]     position of the next token inside its chunk (device tensor)

- runs one step through the model's own layers, and after two eager steps
captures the step in a CUDA graph; from then on a token is one graph launch.
On CPU, with tensor-parallel ranks, or with `use_graph=False` the same code
runs eagerly, which is what the tests compare against the regular cache path.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
from torch import Tensor


def _unwrap(model):
    while hasattr(model, "_wrapped"):
        model = model._wrapped
    return model


class DecodeSession:
    def __init__(self, model, batch_size: int, dtype: torch.dtype = torch.bfloat16, use_graph: Optional[bool] = None):
        self.model = model
        self.mega = _unwrap(model)
        m = self.mega
        if hasattr(model, "materialize_views"):
            model.materialize_views()         # the step calls sub-modules directly, not the FSDP wrapper
        self.B = batch_size
        self.dtype = dtype
        self.device = next(model.parameters()).device
        # Graph capture is the default on a GPU.  With tensor-parallel ranks the collectives of the step
        # (all-reduce after the row-parallel projections, gathers of feature-sharded activations and of
        # the logits) go through `SmallCollective`: one peer-memory kernel each, whose epoch lives in
        # device memory, so the captured step replays correctly (NCCL inside the capture did not complete).
        self._small = None
        from .parallel.initialize import (get_model_parallel_group, get_model_parallel_world_size,
                                          model_parallel_is_initialized)
        mp = get_model_parallel_world_size() if model_parallel_is_initialized() else 1
        if mp > 1 and self.device.type == "cuda" and use_graph is not False:
            from .parallel.model_parallel import mappings
            from .parallel.symm import SmallCollective
            self._small = SmallCollective(get_model_parallel_group(), self.device, max_bytes=2 << 20)
            mappings.use_small_collective(self._small)
        self.use_graph = (self.device.type == "cuda") if use_graph is None else use_graph
        c = m.chunk_size
        first = _unwrap(m.layers[0]).mega
        H, dk, dv = first.local_heads, first.z_head_dim, first.local_v_head_dim
        G = first.timenorm.groups_per_partition
        D, N = first.local_mdim, first.cema.ndim
        dev = self.device
        stat_dtype = dtype

        def norm_state(groups):
            return [torch.zeros(batch_size, dtype=torch.int64, device=dev),
                    torch.zeros(batch_size, groups, dtype=stat_dtype, device=dev),
                    torch.ones(batch_size, groups, dtype=stat_dtype, device=dev)]

        self.layers: List[dict] = []
        for _ in range(m.num_layers):
            self.layers.append({
                "k": torch.zeros(batch_size, H, c, dk, dtype=dtype, device=dev),
                "v": torch.zeros(batch_size, H, c, dv, dtype=dtype, device=dev),
                "norm": norm_state(G),
                "hx": torch.zeros(batch_size, D, N, dtype=torch.complex64, device=dev),
            })
        self.out_norm = norm_state(m.output.final_norm.groups_per_partition)
        self.pos = torch.zeros(1, dtype=torch.int64, device=dev)
        self.tok = torch.zeros(batch_size, 1, dtype=torch.int64, device=dev)
        self.logits: Optional[Tensor] = None
        self._graph = None
        self._eager_steps = 0
        self._fresh = True           # no statistics yet: the norms start from their priors

    # ------------------------------------------------------------------ state import
    @torch.no_grad()
    def load_cache(self, cache) -> None:
        """Take over the state of a regular cache (e.g. after prefilling the prompt)."""
        layers, out_norm = cache
        for st, (kv, norm, hx) in zip(self.layers, layers):
            st["k"].zero_()
            st["v"].zero_()
            n = 0
            if kv is not None and kv[0] is not None:
                n = int(kv[2])
                if n > 0:
                    st["k"][:, :, :n].copy_(kv[0][:, -n:].transpose(1, 2))
                    st["v"][:, :, :n].copy_(kv[1][:, -n:].transpose(1, 2))
            for dst, src in zip(st["norm"], norm):
                dst.copy_(src)
            st["hx"].copy_(hx)
        for dst, src in zip(self.out_norm, out_norm):
            dst.copy_(src)
        self.pos.fill_(n)
        self._fresh = False

    # ------------------------------------------------------------------ one token
    def _step_body(self) -> Tensor:
        m = self.mega
        from . import ops
        x = m.embed(self.tok)
        if m.emb_scale is not None:
            x = x * m.emb_scale
        freqs = m.rope.get_freqs_cis(0, m.chunk_size).index_select(0, self.pos)
        for layer, st in zip(m.layers, self.layers):
            norm = tuple(st["norm"]) if not self._fresh else (None, None, None)
            hx = st["hx"] if not self._fresh else None
            x, (_, new_norm, new_hx) = layer(x, freqs, None, ((st["k"], st["v"], self.pos), norm, hx))
            for dst, src in zip(st["norm"], new_norm):
                dst.copy_(src)
            st["hx"].copy_(new_hx)
        out_norm = tuple(self.out_norm) if not self._fresh else (None, None, None)
        logits, new_out = m.output(x, out_norm)
        for dst, src in zip(self.out_norm, new_out):
            dst.copy_(src)
        self.pos.add_(1).remainder_(m.chunk_size)
        return logits[:, -1].float()

    @torch.no_grad()
    def step(self, tokens: Tensor) -> Tensor:
        """tokens [B] or [B, 1] -> logits [B, V] (fp32) of the next position."""
        self.tok.copy_(tokens.reshape(self.B, 1))
        if self._graph is not None:
            self._graph.replay()
            return self.logits
        was_training = self.model.training
        if was_training:            # eval() drops the cached CEMA coefficients, so only when needed
            self.model.eval()
        try:
            if self._fresh or not self.use_graph or self._eager_steps < 2:
                self.logits = self._step_body()
                self._fresh = False
                self._eager_steps += 1
                return self.logits
            # capture: the step reads and writes only the session's buffers
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            # with a process group alive its watchdog thread makes CUDA calls of its own; in the default
            # (global) capture mode those would invalidate the capture, so other threads are exempted
            dist_on = torch.distributed.is_available() and torch.distributed.is_initialized()
            mode = {"capture_error_mode": "thread_local"} if dist_on else {}
            try:
                if self._small is not None:
                    from .parallel.model_parallel import mappings
                    mappings.small_collective_strict(True)
                try:
                    with torch.cuda.graph(graph, **mode):
                        captured = self._step_body()
                finally:
                    if self._small is not None:
                        mappings.small_collective_strict(False)
            except Exception as e:  # noqa: BLE001 - an op that cannot be captured: stay on the eager step
                import logging
                logging.getLogger().warning(f"decode step could not be captured in a CUDA graph ({e}); "
                                            "continuing with eager fixed-shape steps")
                torch.cuda.synchronize()
                self.use_graph = False
                self.logits = self._step_body()
                return self.logits
            self.logits = captured
            self._graph = graph
            # capturing does not execute: run this token now (the state was not advanced yet)
            graph.replay()
            return self.logits
        finally:
            if was_training:
                self.model.train()

    @torch.no_grad()
    def greedy(self, first_token: Tensor, n_tokens: int) -> Tensor:
        """Generate `n_tokens` greedily starting from `first_token` [B]; returns [B, n_tokens]."""
        out = []
        tok = first_token.reshape(self.B)
        for _ in range(n_tokens):
            tok = self.step(tok).argmax(-1)
            out.append(tok.clone())
        return torch.stack(out, dim=1)
