"""The Megalodon language model: embedding -> N x (MEGA layer + normalised
FFN) -> TimestepNorm -> vocabulary projection (reference:
megalodon/model/mega.py:43-288).

`Mega.forward(tokens [B, L], cache=None)` returns `(logits fp32 [B, L/cp, V],
cache)`.  Without a cache every chunk-parallel rank receives the full token
matrix and processes its own contiguous slice.  With a cache (prefill/decode)
the per-layer KV tail, normalisation statistics and CEMA state are carried
between calls.

`build_model` wraps every block and the root in this framework's own FSDP and
places the model on the GPU when there is one (on the CPU otherwise).
"""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch
from torch import Tensor, nn

from .. import ops
from ..config import ModelConf
from ..modules import (
    MovingAverageGatedAttention,
    NormalizedFeedForwardNetwork,
    RotaryEmbedding,
    TimestepNorm,
)
from ..parallel import (
    FullyShardedDataParallel,
    checkpoint_wrapper,
    enable_wrap,
    get_chunk_parallel_group,
    get_chunk_parallel_rank,
    get_chunk_parallel_world_size,
    get_data_parallel_group,
    get_data_parallel_world_size,
    get_model_parallel_group,
    get_model_parallel_world_size,
    model_parallel_is_initialized,
    wrap,
)
from ..parallel.chunk_parallel import (
    attach_to_graph,
    recv_from_prev_chunk_parallel_region,
    send_to_next_chunk_parallel_region,
    should_recv_from_prev,
    should_send_to_next,
)
from ..parallel.model_parallel import ParallelEmbedding, RowParallelLinear
from ..utils import create_on_gpu, get_init_fn, get_torch_dtype


class MegaBlock(nn.Module):
    def __init__(self, cfg: ModelConf, layer_id: int):
        super().__init__()
        self.layer_id = layer_id
        self.mega = MovingAverageGatedAttention(
            mdim=cfg.model_dim, zdim=cfg.z_dim, hdim=cfg.value_dim, num_heads=cfg.num_heads,
            ndim=cfg.cema_ndim, chunk_size=cfg.chunk_size, efficient_attn=cfg.efficient_attn,
            dropout=cfg.dropout, attention_dropout=cfg.attention_dropout,
            hidden_dropout=cfg.hidden_dropout, norm_num_groups=cfg.norm_num_groups,
            norm_affine=cfg.norm_affine, norm_eps=cfg.norm_eps, init_mode=cfg.init_mode)
        rescale = 0.1 * (0.5 ** layer_id) if cfg.rescale_nffn else None
        self.nffn = NormalizedFeedForwardNetwork(
            model_dim=cfg.model_dim, ffn_hidden_dim=cfg.ffn_hidden_dim, swiglu=cfg.swiglu,
            dropout=cfg.dropout, hidden_dropout=cfg.hidden_dropout, norm_affine=cfg.norm_affine,
            norm_eps=cfg.norm_eps, rescale=rescale, init_mode=cfg.init_mode)

    def forward(self, x: Tensor, freqs_cis: Tensor, mask: Optional[Tensor] = None, cache=None,
                carry=None, piece=None):
        y, state = self.mega(x, freqs_cis, mask, cache, carry, piece)
        # two-hop residual: the FFN adds the block input, not the attention output
        return self.nffn(y, x), state


class MegaOutputLayer(nn.Module):
    def __init__(self, cfg: ModelConf, embed_weight: nn.Parameter):
        super().__init__()
        self.model_dim = cfg.model_dim
        self.output_size = cfg.vocab_size if cfg.output_size == -1 else cfg.output_size
        self.final_norm = TimestepNorm(cfg.model_dim, cfg.norm_num_groups, eps=cfg.norm_eps)
        self.output = RowParallelLinear(cfg.model_dim, self.output_size, bias=False,
                                        input_is_parallel=True, parallel_output=False,
                                        init_method=get_init_fn("gaussian", dim=cfg.model_dim))
        self.share_emb = cfg.share_emb
        if self.share_emb:
            self.output.weight = embed_weight

    def normalize(self, x: Tensor, cache=None, carry=None, piece=None):
        """Final TimestepNorm with the same cache / carry / piece protocol as the
        MEGA layer.  Returns (normalised x, cache or carry)."""
        prev_count = prev_mean = prev_var = None
        streaming = piece is not None
        first_piece = piece is None or piece[0] == 0
        last_piece = piece is None or piece[0] == piece[1] - 1
        emit = piece is not None and len(piece) > 3 and bool(piece[3])
        if cache is not None:
            prev_count, prev_mean, prev_var = cache
        elif carry is not None:
            prev_count, prev_mean, prev_var = carry
        elif first_piece and should_recv_from_prev():
            bsz = x.size(0)
            local_len = x.size(1) if piece is None else piece[2]
            g = self.final_norm.groups_per_partition
            prev_count = torch.full((bsz,), local_len * get_chunk_parallel_rank(), dtype=torch.int64,
                                    device=x.device)
            buf = torch.empty((bsz, 2 * g), dtype=x.dtype, device=x.device,
                              requires_grad=self.training and torch.is_grad_enabled())
            packed = recv_from_prev_chunk_parallel_region(buf)
            prev_mean, prev_var = torch.split(packed, [g, g], dim=-1)

        x, prev_count, prev_mean, prev_var = self.final_norm(x, prev_count, prev_mean, prev_var)

        if cache is not None:
            return x, (prev_count.detach(), prev_mean.detach(), prev_var.detach())
        if last_piece and should_send_to_next():
            packed = send_to_next_chunk_parallel_region(torch.cat([prev_mean, prev_var], dim=-1))
            x = attach_to_graph(x, packed)
        if streaming and not last_piece:
            return x, (prev_count, prev_mean, prev_var)
        if emit:
            return x, (prev_count.detach(), prev_mean.detach(), prev_var.detach())
        return x, None

    def forward(self, x: Tensor, cache: Optional[Tuple[Tensor, Tensor, Tensor]] = None, carry=None,
                piece=None):
        x, state = self.normalize(x, cache, carry, piece)
        return self.output(x), state


class Mega(nn.Module):
    def __init__(self, cfg: ModelConf):
        super().__init__()
        assert cfg.vocab_size > 0
        self.cfg = cfg
        self.vocab_size = cfg.vocab_size
        self.num_layers = cfg.num_layers
        self.model_dim = cfg.model_dim
        self.num_heads = cfg.num_heads
        self.chunk_size = cfg.chunk_size
        self.output_size = self.vocab_size if cfg.output_size == -1 else cfg.output_size
        self.dropout = cfg.dropout
        self.efficient_attn = cfg.efficient_attn
        self.emb_scale = math.sqrt(cfg.model_dim) if cfg.scale_emb else None
        self.share_emb = cfg.share_emb
        self.chunk_parallel_size = get_chunk_parallel_world_size()
        self.chunk_parallel_rank = get_chunk_parallel_rank()

        self.embed = ParallelEmbedding(self.vocab_size, self.model_dim, gather_output=False,
                                       init_method=get_init_fn("gaussian", dim=self.model_dim))
        self.z_head_dim = cfg.z_dim // cfg.num_heads
        self.v_head_dim = cfg.value_dim // cfg.num_heads
        mp = get_model_parallel_world_size()
        # more ranks than heads: one head per rank, its value columns split over mp / num_heads ranks
        self.local_heads = max(1, self.num_heads // mp)
        self.local_v_head_dim = self.v_head_dim // max(1, mp // self.num_heads)
        self.rope = RotaryEmbedding(self.z_head_dim, cfg.chunk_size, base=cfg.rope_base)
        self.layers = nn.ModuleList()
        for layer_id in range(self.num_layers):
            block = MegaBlock(cfg, layer_id)
            n_ckpt = self.num_layers if getattr(cfg, "ckpt_layers", None) is None else cfg.ckpt_layers
            layer = checkpoint_wrapper(block) if (cfg.layerwise_ckpt and layer_id < n_ckpt) else block
            self.layers.append(wrap(layer))
        self.output = MegaOutputLayer(cfg, self.embed.weight)

    def forward(self, tokens: Tensor, cache=None, targets: Optional[Tensor] = None, prefill: bool = False):
        """tokens [B, L].  Returns `(logits fp32 [B, L/cp, V], cache)`.

        `prefill=True` runs `self.prefill(tokens)` instead (chunk-parallel prefill that returns the
        last position's logits and a cache); it goes through `forward` so that a wrapping FSDP unit
        has gathered the parameters.

        With `targets` [B, L] (training only) the vocabulary projection and the
        cross-entropy are evaluated piece by piece and the first return value is
        the vector of per-token losses gathered over the chunk group (what
        `modules.losses.cross_entropy(logits, targets)` returns), so the fp32
        logits of the whole sequence are never materialised.

        `self.seq_microbatch_chunks = k` feeds the local sequence through every
        layer in pieces of k chunks, carrying the TimestepNorm statistics and
        CEMA state from piece to piece: same math, bounded activation memory."""
        if prefill:
            assert cache is None and targets is None
            return self.prefill(tokens)
        bsz, seq_len = tokens.shape
        c = self.chunk_size
        if cache is None:
            cache_layers = cache_output = None
            cache_len = 0
            assert seq_len % self.chunk_parallel_size == 0
            seq_len //= self.chunk_parallel_size
            lo = self.chunk_parallel_rank * seq_len
            tokens = tokens[:, lo:lo + seq_len]
            if targets is not None:
                targets = targets[:, lo:lo + seq_len]
        else:
            assert targets is None
            cache_layers, cache_output = cache
            first_kv = cache_layers[0][0]
            cache_len = 0 if first_kv is None else first_kv[-1]
            # With a cache the tokens are not split and nothing is handed between ranks: on a
            # chunk-parallel group every rank runs the same step on the same state (replicated decode,
            # e.g. after `prefill`), which keeps the sharded parameters' collectives in lockstep.
            if cache_len > 0:
                assert cache_len + seq_len <= c
        assert seq_len < c or seq_len % c == 0, f"{seq_len}/{c}"

        x = self.embed(tokens)
        if self.emb_scale is not None:
            x = x * self.emb_scale
        x = ops.memory_efficient_dropout(x, self.dropout, self.training)

        if self.efficient_attn:
            mask = None
        else:
            m = min(seq_len, c)
            mask = torch.full((1, 1, m, m + cache_len), float("-inf"), device=tokens.device)
            mask = torch.triu(mask, diagonal=cache_len + 1).to(x.dtype)
        freqs_cis = self.rope.get_freqs_cis(cache_len, min(cache_len + seq_len, c))

        piece_len = None
        k = getattr(self, "seq_microbatch_chunks", None)
        if cache is None and k and seq_len > k * c:
            piece_len = k * c
        if piece_len is None:
            for i, layer in enumerate(self.layers):
                x, layer_cache = layer(x, freqs_cis, mask, cache_layers[i] if cache is not None else None)
                if cache is not None:
                    cache_layers[i] = layer_cache
            if targets is not None:
                xn, _ = self.output.normalize(x)
                return self._gather_losses([self._piece_loss(xn, targets)]), None
            out, cache_output = self.output(x, cache_output)
            if cache is not None:
                cache = (cache_layers, cache_output)
            return out.float(), cache

        # ---- sequence micro-batching (training / scoring without cache)
        pieces = list(torch.split(x, piece_len, dim=1))
        n = len(pieces)
        for layer in self.layers:
            carry = None
            for i in range(n):
                pieces[i], carry = layer(pieces[i], freqs_cis, mask, None, carry, (i, n, seq_len))
        outs, carry = [], None
        tgt = None if targets is None else torch.split(targets, piece_len, dim=1)
        for i in range(n):
            xn, carry = self.output.normalize(pieces[i], None, carry, (i, n, seq_len))
            pieces[i] = None
            outs.append(self._piece_loss(xn, tgt[i]) if targets is not None else self.output.output(xn).float())
        if targets is not None:
            return self._gather_losses(outs), None
        return torch.cat(outs, dim=1), None

    @torch.no_grad()
    def prefill(self, tokens: Tensor):
        """Chunk-parallel prefill: tokens [B, L] with L a multiple of chunk_size x chunk-parallel size.
        Every rank runs its slice (the CEMA / TimestepNorm state is handed from rank to rank as in
        training), the last rank's final state is broadcast, and every rank returns
        `(logits of the last position [B, V] fp32, cache)` where `cache` has the structure of
        `utils.init_cache` with an empty key/value tail - ready for `forward(tokens, cache)` or
        `decoding.DecodeSession.load_cache`.  The reference cannot combine a cache with chunk
        parallelism (model/mega.py:210)."""
        import torch.distributed as dist
        from ..parallel import get_chunk_parallel_group, get_chunk_parallel_ranks
        bsz, total = tokens.shape
        c, cp = self.chunk_size, self.chunk_parallel_size
        assert total % (c * cp) == 0, "prefill length must be a multiple of chunk_size x chunk-parallel size"
        seq_len = total // cp
        lo = self.chunk_parallel_rank * seq_len
        x = self.embed(tokens[:, lo:lo + seq_len])
        if self.emb_scale is not None:
            x = x * self.emb_scale
        k = getattr(self, "seq_microbatch_chunks", None) or (seq_len // c)
        piece_len = min(seq_len, k * c)
        n = seq_len // piece_len
        mask = None
        if not self.efficient_attn:
            mask = torch.triu(torch.full((1, 1, c, c), float("-inf"), device=tokens.device), diagonal=1).to(x.dtype)
        freqs_cis = self.rope.get_freqs_cis(0, c)
        pieces = list(torch.split(x, piece_len, dim=1))
        layer_states = []
        for layer in self.layers:
            carry = None
            for i in range(n):
                pieces[i], carry = layer(pieces[i], freqs_cis, mask, None, carry, (i, n, seq_len, True))
            layer_states.append(carry)
        carry = None
        for i in range(n):
            xn, carry = self.output.normalize(pieces[i], None, carry, (i, n, seq_len, True))
        logits = self.output.output(xn[:, -1:]).float()[:, 0]
        out_state = carry
        if cp > 1:
            src = get_chunk_parallel_ranks()[-1]
            group = get_chunk_parallel_group()
            flat = [logits] + [t for st in layer_states for t in (st[0], st[1], st[2], torch.view_as_real(st[3]))] \
                + list(out_state)
            for t in flat:
                dist.broadcast(t, src=src, group=group)
        first = self.layers[0]
        while hasattr(first, "_wrapped"):
            first = first._wrapped
        dt = x.dtype
        cache_layers = []
        for count, mean, var, hx in layer_states:
            kv = (torch.empty((bsz, 0, self.local_heads, self.z_head_dim), dtype=dt, device=x.device),
                  torch.empty((bsz, 0, self.local_heads, self.local_v_head_dim), dtype=dt, device=x.device), 0)
            cache_layers.append((kv, (count, mean, var), hx))
        return logits, (cache_layers, tuple(out_state))

    def _piece_loss(self, xn: Tensor, targets: Tensor) -> Tensor:
        logits = self.output.output(xn)
        return ops.cross_entropy(logits.flatten(0, 1), targets.flatten(0, 1)).view(targets.shape)

    @staticmethod
    def _gather_losses(parts: List[Tensor]) -> Tensor:
        from ..parallel.chunk_parallel import gather_from_chunk_parallel_region
        local = parts[0] if len(parts) == 1 else torch.cat(parts, dim=1)
        return gather_from_chunk_parallel_region(local.flatten())


def build_model(model_cfg: ModelConf, dtype: str, fp32_reduce_scatter: bool = False,
                reshard_after_forward: bool = True, *, shard_over_chunk_group: bool = False,
                materialize_fp32_grads: bool = False, device: Optional[torch.device] = None) -> Mega:
    """Build the FSDP-wrapped model in training mode.

    With `shard_over_chunk_group` the parameters, gradients and optimiser state
    are sharded over the combined data x chunk group instead of being
    replicated across the chunk group."""
    if model_parallel_is_initialized():
        dp_group, mp_group, cp_group = (get_data_parallel_group(), get_model_parallel_group(),
                                        get_chunk_parallel_group())
    else:
        dp_group = mp_group = cp_group = None
    shard_group, divide = dp_group, None
    if shard_over_chunk_group and model_parallel_is_initialized() and get_chunk_parallel_world_size() > 1:
        from ..parallel.initialize import get_shard_parallel_group
        shard_group = get_shard_parallel_group()
        divide = float(get_data_parallel_world_size())
    fsdp_cfg = dict(
        process_group=shard_group,
        process_group_reduce_scatter=shard_group,
        model_parallel_process_group=mp_group,
        chunk_parallel_process_group=cp_group,
        compute_dtype=get_torch_dtype(dtype),
        state_dict_device=torch.device("cpu"),
        mixed_precision=dtype != "fp32",
        flatten_parameters=True,
        fp32_reduce_scatter=fp32_reduce_scatter,
        reshard_after_forward=reshard_after_forward,
        gradient_divide_factor=divide,
        chunk_group_is_sharded=shard_group is not dp_group,
        materialize_fp32_grads=materialize_fp32_grads,
    )
    ctx = torch.device(device) if device is not None else create_on_gpu()
    with ctx:
        with enable_wrap(wrapper_cls=FullyShardedDataParallel, **fsdp_cfg):
            model = wrap(Mega(model_cfg))
    model.train()
    return model


ModelStore = {
    "mega200M": ModelConf(num_layers=12, model_dim=1024, num_heads=1, z_dim=256, value_dim=2048,
                          ffn_hidden_dim=2560, chunk_size=2048, norm_num_groups=32),
    "mega1.3B": ModelConf(num_layers=24, model_dim=2048, num_heads=2, z_dim=512, value_dim=4096,
                          ffn_hidden_dim=4864, chunk_size=2048, norm_num_groups=64),
    "mega1.3B_pg19": ModelConf(num_layers=24, model_dim=2048, num_heads=2, z_dim=512, value_dim=4096,
                               ffn_hidden_dim=3584, chunk_size=2048, norm_num_groups=64, swiglu=True,
                               scale_emb=True, share_emb=True),
    "mega7.1B": ModelConf(num_layers=32, model_dim=4096, num_heads=4, z_dim=1024, value_dim=8192,
                          ffn_hidden_dim=11264, chunk_size=2048, norm_num_groups=64),
    "mega7.3B": ModelConf(num_layers=32, model_dim=4096, num_heads=4, z_dim=1024, value_dim=8192,
                          ffn_hidden_dim=8192, chunk_size=2048, norm_num_groups=64, swiglu=True),
    # small shape for plumbing / correctness runs on CPU
    "mega_tiny": ModelConf(num_layers=2, model_dim=128, num_heads=1, z_dim=32, value_dim=256, ffn_hidden_dim=256,
                           cema_ndim=4, chunk_size=64, norm_num_groups=32, swiglu=True),
    # the 7B shape used for the long-context throughput benchmark
    "mega7B_32k": ModelConf(num_layers=32, model_dim=4096, num_heads=4, z_dim=1024, value_dim=8192,
                            ffn_hidden_dim=11264, chunk_size=4096, norm_num_groups=64, swiglu=True,
                            vocab_size=32000, efficient_attn="fused"),
}
