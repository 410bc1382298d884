"""In-house fully-sharded data parallelism (ZeRO-3) - no fairscale.

Public surface follows the reference's subclass of fairscale's FSDP
(megalodon/distributed/fairscale_fsdp.py:15-219) and the way the model uses it
(megalodon/model/mega.py:245-269): nested wrapping (one unit per block plus a
root unit), `parameters()` yielding the fp32 flat shards that the optimiser
updates, `clip_grad_norm_`, `grad_all_reduce`, and full / local state dicts.

Design of one unit
------------------
* All parameters of the unit live in ONE flat buffer in their natural order.
  Sharding is PER PARAMETER: every parameter is padded to `world` pieces of
  the same length (a multiple of 64 elements = 128 B in bf16, so TMA tiles and
  vector loads stay aligned) and rank r holds piece r of every parameter; a
  rank's shard is the concatenation of its pieces.  For a weight matrix
  [N, K] with N divisible by `world`, piece r is the row block
  [r N / world, (r + 1) N / world): every rank owns an equal slice of every
  matrix, which is what lets a kernel pull the rows it needs from their owner
  with balanced traffic (`symm.SymmetricParamGather`, the gathering GEMM).
  Mapping (element j of parameter p, piece length `piece`, natural offset
  `offset`, `shard_offset = offset / world`):
      full[offset + j]  <->  shard of rank j // piece, index shard_offset + j % piece
  A cut of the flat buffer into `world` contiguous ranges (fairscale's layout)
  would put a whole matrix on one or two ranks.
* The fp32 shard is an `nn.Parameter` (`flat_param`): the master weights.
  A compute-dtype copy of the shard (`flat_param._lowp_shard`) feeds the
  all-gather; the fused AdamW kernel refreshes it in the same pass that
  updates the master weights.
* Forward: all-gather the compute-dtype shards into the full buffer, hand the
  wrapped module *views* of it, run, optionally free the full buffer
  (`reshard_after_forward`).  The storage is resized in place so views and
  tensors saved for backward stay valid once it is re-gathered.
* Backward: a hook on the unit's outputs re-gathers the parameters if needed.
  The parameter views are the outputs of one autograd node per iteration
  (`_FlatViews`); its backward runs once every parameter gradient of a forward
  call is known, writes them into the unit's flat gradient buffer and, after
  the last call, launches the reduce-scatter (on a side stream on GPUs).
  Weights consumed by the native linear op skip even that copy: their view
  carries a handle to the matching slice of the flat gradient and the weight-
  gradient GEMM accumulates straight into it.
* The gradient shard stays in the reduction dtype (`_grad_shard`).  The fused
  optimiser reads it directly; for generic optimisers an fp32 `.grad` is
  materialised (`materialize_fp32_grads`).

Sharding group
--------------
`process_group` is the group the parameters are sharded over.  The reference
shards over the data-parallel group only and replicates across the chunk
group, summing gradients there in a separate `grad_all_reduce()` call.  Chunk
ranks process different tokens with the same weights, exactly like
data-parallel ranks, so this implementation can also shard over the combined
data x chunk group (`gradient_divide_factor` = data-parallel size keeps the
reference's scaling: mean over data ranks, sum over chunk ranks); then
`grad_all_reduce()` has nothing left to do.
"""
from __future__ import annotations

import math
from collections import OrderedDict
from enum import Enum, auto
from typing import Any, Dict, Iterator, List, Optional, Tuple, Union


import torch
import torch.distributed as dist
import torch.nn as nn

from contextlib import nullcontext as _nullcontext

from .utils import all_gather_flat, reduce_scatter_flat

ALIGN = 64


class TrainingState(Enum):
    IDLE = auto()
    FORWARD = auto()
    BACKWARD_PRE = auto()
    BACKWARD_POST = auto()


class _ParamInfo:
    """`offset`: start in the natural-order buffer; `piece`: elements of this parameter held by each
    rank (world * piece >= numel); `shard_offset`: start of the piece inside every rank's shard."""
    __slots__ = ("name", "shape", "numel", "offset", "owners", "piece", "shard_offset")

    def __init__(self, name, shape, numel, offset, owners, piece=0, shard_offset=0):
        self.name, self.shape, self.numel, self.offset, self.owners = name, shape, numel, offset, owners
        self.piece, self.shard_offset = piece, shard_offset


def _group_size(group) -> int:
    if group is None or not (dist.is_available() and dist.is_initialized()):
        return 1
    return dist.get_world_size(group)


def _group_rank(group) -> int:
    if group is None or not (dist.is_available() and dist.is_initialized()):
        return 0
    return dist.get_rank(group)


def calc_grad_norm(grads: List[torch.Tensor], norm_type: float) -> torch.Tensor:
    """Norm of a list of gradient tensors viewed as one vector (fp32 accumulate)."""
    grads = [g for g in grads if g is not None]
    if not grads:
        return torch.tensor(0.0)
    if norm_type == math.inf:
        return torch.stack([g.detach().abs().max().float() for g in grads]).max()
    parts = torch.stack([torch.linalg.vector_norm(g.detach().float(), norm_type) for g in grads])
    return torch.linalg.vector_norm(parts, norm_type)


class _FlatViews(torch.autograd.Function):
    """leaf -> one view per parameter of the unit.  Backward receives every parameter gradient of one
    forward call at once: the point where the unit knows that call's gradients are complete."""

    @staticmethod
    def forward(ctx, leaf: torch.Tensor, unit: "FullyShardedDataParallel"):
        ctx.unit = unit
        ctx.set_materialize_grads(False)
        base = leaf.detach()
        return tuple(base[info.offset:info.offset + info.numel].view(info.shape) for info in unit._infos)

    @staticmethod
    def backward(ctx, *grads):
        ctx.unit._collect_grads(grads)
        return None, None


class FullyShardedDataParallel(nn.Module):
    _is_wrapper = True

    def __init__(
        self,
        module: nn.Module,
        process_group: Optional[dist.ProcessGroup] = None,
        process_group_reduce_scatter: Any = None,
        model_parallel_process_group: Optional[dist.ProcessGroup] = None,
        chunk_parallel_process_group: Optional[dist.ProcessGroup] = None,
        *,
        compute_dtype: Optional[torch.dtype] = None,
        mixed_precision: bool = False,
        flatten_parameters: bool = True,
        fp32_reduce_scatter: bool = False,
        reshard_after_forward: bool = True,
        state_dict_device: Optional[torch.device] = None,
        bucket_cap_mb: int = 25,
        buffer_dtype: Optional[torch.dtype] = None,
        compute_device: Optional[torch.device] = None,
        move_params_to_cpu: bool = False,
        move_grads_to_cpu: bool = False,
        clear_autocast_cache: bool = False,
        force_input_to_fp32: bool = False,
        verbose: bool = False,
        gradient_divide_factor: Optional[float] = None,
        chunk_group_is_sharded: bool = False,
        materialize_fp32_grads: bool = True,
    ):
        super().__init__()
        assert flatten_parameters, "only flattened parameters are supported"
        assert not move_params_to_cpu and not move_grads_to_cpu, "CPU offload is not supported"
        self.process_group = process_group
        self.process_group_reduce_scatter = process_group_reduce_scatter or process_group
        self.model_parallel_process_group = model_parallel_process_group
        self.model_parallel_world_size = _group_size(model_parallel_process_group)
        self.chunk_parallel_process_group = chunk_parallel_process_group
        self.chunk_parallel_world_size = _group_size(chunk_parallel_process_group)
        self.chunk_group_is_sharded = chunk_group_is_sharded
        self.world_size = _group_size(process_group)
        self.rank = _group_rank(process_group)
        self.mixed_precision = mixed_precision
        self.compute_dtype = (compute_dtype or torch.float32) if mixed_precision else torch.float32
        self.buffer_dtype = buffer_dtype or self.compute_dtype
        self.fp32_reduce_scatter = fp32_reduce_scatter
        self.reshard_after_forward = reshard_after_forward and self.world_size > 1
        self.flatten_parameters = True
        self.state_dict_device = state_dict_device
        self.bucket_cap_mb = bucket_cap_mb
        self.move_params_to_cpu = False
        self.move_grads_to_cpu = False
        self.clear_autocast_cache = clear_autocast_cache
        self.force_input_to_fp32 = force_input_to_fp32
        self.verbose = verbose
        self.materialize_fp32_grads = materialize_fp32_grads
        # When True, `clip_grad_norm_` leaves the gradients untouched and hands its clipping
        # coefficient (a device scalar) to `FusedAdamW`, which applies it while reading the
        # gradients: one pass over gradient memory saved.  Gradients inspected between the two
        # calls are then unclipped.
        self.defer_grad_clip = False
        self._clip_coef = None
        self.gradient_divide_factor = float(gradient_divide_factor if gradient_divide_factor is not None
                                            else self.world_size)
        self.training_state = TrainingState.IDLE
        self._is_root: Optional[bool] = None
        self._wrapped = module
        self._comm_stream = None
        self._gather_stream = None
        self._gather_event = None
        self._pending: List[Any] = []

        self._flatten(module, compute_device)
        self.compute_device = self.flat_param.device
        self._full: Optional[torch.Tensor] = None          # gathered compute-dtype buffer
        self._full_leaf: Optional[torch.Tensor] = None
        self._flat_grad: Optional[torch.Tensor] = None     # this iteration's gradients, compute dtype
        self._full_version = -1
        self._bwd_hook_armed = False
        self._calls = 0
        self._fires = 0

    # ------------------------------------------------------------------ construction
    def _flatten(self, module: nn.Module, device: Optional[torch.device]) -> None:
        infos: List[_ParamInfo] = []
        by_id: Dict[int, _ParamInfo] = {}
        offset = 0
        datas: List[torch.Tensor] = []
        for mod_name, mod in module.named_modules():
            if isinstance(mod, FullyShardedDataParallel):
                continue
            if self._inside_child_unit(module, mod_name):
                continue
            for pname, p in list(mod._parameters.items()):
                if p is None:
                    continue
                full_name = _clean_name(f"{mod_name}.{pname}" if mod_name else pname)
                if id(p) in by_id:
                    by_id[id(p)].owners.append((mod, pname, full_name))
                    continue
                piece = -(-p.numel() // (self.world_size * ALIGN)) * ALIGN
                info = _ParamInfo(full_name, tuple(p.shape), p.numel(), offset, [(mod, pname, full_name)],
                                  piece, offset // self.world_size)
                by_id[id(p)] = info
                infos.append(info)
                datas.append(p.detach())
                offset += piece * self.world_size
        self._infos = infos
        world = self.world_size
        self._numel_padded = max(world * ALIGN, offset)
        self._shard_numel = self._numel_padded // world
        self._piece_tables: Dict[Any, torch.Tensor] = {}
        if device is None:
            device = datas[0].device if datas else torch.device("cpu")
        shard = torch.zeros(self._shard_numel, dtype=torch.float32, device=device)
        for info, d in zip(infos, datas):
            self._write_piece(shard, info, d.reshape(-1))
        self.flat_param = nn.Parameter(shard)
        self.flat_param._fsdp_unit = self
        self.flat_param._grad_shard = None
        self.flat_param._lowp_shard = None
        self.flat_param._lowp_version = -1
        # the wrapped modules give up their Parameters; they get views each forward
        for info in infos:
            for mod, pname, _ in info.owners:
                del mod._parameters[pname]
                setattr(mod, pname, None)
        if self.mixed_precision:
            # buffers follow the compute dtype like the reference's `model.to(dtype)` path
            for b_name, buf in list(module.named_buffers()):
                if buf.is_floating_point() and not self._inside_child_unit(module, b_name.rpartition(".")[0]):
                    buf.data = buf.data.to(self.buffer_dtype)

    @staticmethod
    def _inside_child_unit(root: nn.Module, mod_name: str) -> bool:
        if not mod_name:
            return False
        cur = root
        for part in mod_name.split("."):
            cur = cur._modules[part]
            if isinstance(cur, FullyShardedDataParallel):
                return True
        return False

    # ------------------------------------------------------------------ layout (see the module docstring)
    def _write_piece(self, shard: torch.Tensor, info: _ParamInfo, flat_param: torch.Tensor) -> None:
        """Copy this rank's piece of one (unpadded, flattened) parameter into `shard`."""
        a = self.rank * info.piece
        b = min(a + info.piece, info.numel)
        if a < b:
            shard[info.shard_offset:info.shard_offset + (b - a)].copy_(flat_param[a:b])

    def piece_table(self, device, infos=None, key=None) -> torch.Tensor:
        """int64 [P, 3] rows (shard_offset, piece, offset) on `device`: what the native kernels that
        move data between the shard and the natural layouts need.  `infos` restricts the table to
        some parameters (cached under `key`)."""
        key = (str(device), key)
        t = self._piece_tables.get(key)
        if t is None:
            rows = [[i.shard_offset, i.piece, i.offset] for i in (self._infos if infos is None else infos)]
            if infos is None and not rows:
                rows = [[0, self._shard_numel, 0]]
            t = self._piece_tables[key] = torch.tensor(rows, dtype=torch.int64, device=device).reshape(-1, 3)
        return t

    def _unshard(self, rank_major: torch.Tensor, full: torch.Tensor) -> None:
        """[shard of rank 0 | shard of rank 1 | ...] -> natural order."""
        W, S = self.world_size, self._shard_numel
        src = rank_major.view(W, S)
        for i in self._infos:
            full[i.offset:i.offset + W * i.piece].view(W, i.piece).copy_(src[:, i.shard_offset:i.shard_offset + i.piece])

    def _to_rank_major(self, full: torch.Tensor, rank_major: torch.Tensor) -> None:
        """natural order -> [what rank 0 owns | what rank 1 owns | ...] (input of a reduce-scatter)."""
        W, S = self.world_size, self._shard_numel
        dst = rank_major.view(W, S)
        for i in self._infos:
            dst[:, i.shard_offset:i.shard_offset + i.piece].copy_(full[i.offset:i.offset + W * i.piece].view(W, i.piece))

    def _scratch(self, numel: int, dtype: torch.dtype, device) -> torch.Tensor:
        """Root-owned scratch for the rank-major side of a collective, one per (stream, dtype): uses on
        one stream are ordered, so one buffer per stream is enough however many units are in flight."""
        root = getattr(self, "_root", self)
        pool = root.__dict__.setdefault("_scratch_pool", {})
        sid = torch.cuda.current_stream(device).cuda_stream if torch.device(device).type == "cuda" else 0
        key = (sid, dtype)
        buf = pool.get(key)
        if buf is None or buf.numel() < numel:
            buf = pool[key] = torch.empty(numel, dtype=dtype, device=device)
        return buf[:numel]

    def _all_gather_natural(self, full: torch.Tensor, shard: torch.Tensor) -> None:
        """full (natural order) <- every rank's shard."""
        tmp = self._scratch(self._numel_padded, shard.dtype, shard.device)
        all_gather_flat(tmp, shard, self.process_group)
        self._unshard(tmp, full)

    def __getattr__(self, name: str) -> Any:
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(self._modules["_wrapped"], name)

    @property
    def module(self) -> nn.Module:
        return self._wrapped

    # ------------------------------------------------------------------ unit tree
    def _units(self) -> List["FullyShardedDataParallel"]:
        return [m for m in self.modules() if isinstance(m, FullyShardedDataParallel)]

    def _lazy_init(self) -> None:
        if self._is_root is not None:
            return
        self._is_root = True
        # plain attributes, not sub-modules: registering the root as a child of its units would make
        # the module tree cyclic (train() / eval() would never return)
        for u in self._units():
            if u is not self:
                u._is_root = False
                object.__setattr__(u, "_root", self)
        object.__setattr__(self, "_root", self)
        if self.compute_device.type == "cuda" and self.world_size > 1:
            # high priority: the flag barriers and reductions on this stream are what peers wait for;
            # their few CTAs should be placed ahead of the compute stream's pending ones
            self._comm_stream = torch.cuda.Stream(self.compute_device, priority=-1)

    @property
    def children_share_process_group(self) -> bool:
        return all(u.process_group is self.process_group for u in self._units())

    def assert_state(self, state: TrainingState) -> None:
        if self.training_state != state:
            raise AssertionError(f"expected FSDP state {state}, got {self.training_state}")

    @property
    def params_with_grad(self) -> List[nn.Parameter]:
        out = []
        for u in self._units():
            p = u.flat_param
            if p.grad is not None or p._grad_shard is not None:
                out.append(p)
        return out

    # ------------------------------------------------------------------ gather / free
    def _lowp_shard(self) -> torch.Tensor:
        p = self.flat_param
        if not self.mixed_precision:
            return p.data
        if p._lowp_shard is None:
            p._lowp_shard = torch.empty(self._shard_numel, dtype=self.compute_dtype, device=p.device)
            p._lowp_version = -1
        if p._lowp_version != _ver(p):
            p._lowp_shard.copy_(p.data)
            p._lowp_version = _ver(p)
        return p._lowp_shard

    def _full_is_valid(self) -> bool:
        return (self._full is not None and self._full.untyped_storage().size() > 0
                and self._full_version == _ver(self.flat_param))

    def _gather_full(self) -> None:
        """Make `self._full` hold every parameter of the unit in compute dtype."""
        shard = self._lowp_shard()
        if self.world_size == 1:
            if self._full is None or self._full.data_ptr() != shard.data_ptr():
                self._full = shard
            self._full_version = _ver(self.flat_param)
            return
        if self._full is None:
            self._full = torch.empty(self._numel_padded, dtype=shard.dtype, device=shard.device)
        elif self._full.untyped_storage().size() == 0:
            self._full.untyped_storage().resize_(self._numel_padded * self._full.element_size())
        # write through `.data`: the re-gather before backward must not bump the
        # autograd version counter shared with the views handed to the module
        puller = getattr(getattr(self, "_root", self), "_symm_gather", None)
        if puller is not None and shard.is_cuda:
            puller.shards_written()
            puller.pull(self, self._full.data)
        else:
            self._all_gather_natural(self._full.data, shard)
        self._full_version = _ver(self.flat_param)

    def _prefetch_gathers(self) -> None:
        """Root only: all-gather every unit whose full buffer stays resident
        between forward and backward, on a side stream, as soon as the step starts.

        With the all-gathers on the compute stream the ranks of a chunk-parallel
        group advance in lockstep layer by layer (a collective completes only when
        every rank has reached it), while the state handoff makes rank r start a
        layer only after rank r-1 finished it: together that serialises the ranks.
        Issued up front on their own stream the gathers depend on nothing but the
        optimizer step, and each unit's forward waits only for its own event."""
        if self.compute_device.type != "cuda":
            return
        stale = [u for u in self._units()
                 if u.world_size > 1 and (u._is_root or not u.reshard_after_forward) and not u._full_is_valid()]
        if not stale:
            return
        shards = [u._lowp_shard() for u in stale]          # casts (if any) run on the compute stream
        for u, shard in zip(stale, shards):
            if u._full is None:
                u._full = torch.empty(u._numel_padded, dtype=shard.dtype, device=shard.device)
        if self._gather_stream is None:
            self._gather_stream = torch.cuda.Stream(self.compute_device, priority=-1)
        gs = self._gather_stream
        gs.wait_stream(torch.cuda.current_stream())
        puller = getattr(self, "_symm_gather", None)
        with torch.cuda.stream(gs):
            if puller is not None:
                puller.shards_written()        # flag barrier: every rank's shards of this step are in place
            for u, shard in zip(stale, shards):
                if puller is not None:
                    puller.pull(u, u._full.data)
                else:
                    u._all_gather_natural(u._full.data, shard)
                u._full_version = _ver(u.flat_param)
                ev = torch.cuda.Event()
                ev.record(gs)
                u._gather_event = ev

    def _pull_pending(self) -> None:
        puller = getattr(getattr(self, "_root", self), "_symm_gather", None)
        for info in list(self._fused_infos):
            if info.name in self._fused_pending:
                puller.pull_one(self, info, self._full.data)

    def _free_full(self) -> None:
        if self.world_size > 1 and self._full is not None:
            self._full.untyped_storage().resize_(0)

    def _set_views(self, leaf: torch.Tensor, track: bool = False) -> None:
        """Hand the wrapped modules views of `leaf`.  With `track` the views come out of `_FlatViews`
        so their gradients flow back into the unit's flat gradient buffer."""
        if track:
            views = _FlatViews.apply(leaf, self)
        else:
            views = [leaf[info.offset:info.offset + info.numel].view(info.shape) for info in self._infos]
        direct = track and leaf.is_cuda and leaf.dtype in (torch.bfloat16, torch.float16)
        fused = {i.name for i in getattr(self, "_fused_infos", ())}
        for info, v in zip(self._infos, views):
            if direct and len(info.shape) == 2:
                v._wgrad_sink = _WgradSink(self, info)
            if info.name in fused:
                v._gather_spec = _GatherSpec(self, info)
            for mod, pname, _ in info.owners:
                mod.__dict__[pname] = v

    def _grad_buffer(self) -> torch.Tensor:
        """Flat gradient of this iteration in compute dtype.  Nothing is zero-filled up front: the first
        contribution to a parameter's range is written (the weight-gradient GEMM runs without its
        accumulating epilogue, other gradients are copied), later ones are added, and what received
        nothing is zeroed when the unit's gradients leave (`_zero_unwritten`).  Only the gaps between
        parameters and the padding at the end are cleared here."""
        if self._flat_grad is None:
            arena = getattr(self, "_grad_arena", None)
            if arena is not None and self.flat_param._grad_shard is None and self.flat_param.grad is None:
                # peer-mapped home of this unit's gradient (chunk-group all-reduce in place); a second
                # backward before the optimiser step finds the first gradient still there and takes
                # ordinary memory instead
                region, off, nbytes = arena
                self._flat_grad = region.view(off, nbytes, self._full.dtype)[:self._numel_padded]
            else:
                self._flat_grad = torch.empty(self._numel_padded, dtype=self._full.dtype, device=self._full.device)
            self._grad_unwritten = {id(info) for info in self._infos}
            for a, b in self._grad_gaps():
                self._flat_grad[a:b].zero_()
        return self._flat_grad

    def _full_dtype_size(self) -> int:
        return torch.empty(0, dtype=self.compute_dtype if self.mixed_precision else torch.float32).element_size()

    def _grad_gaps(self):
        gaps = getattr(self, "_grad_gap_list", None)
        if gaps is None:
            gaps, pos = [], 0
            for info in sorted(self._infos, key=lambda i: i.offset):
                if info.offset > pos:
                    gaps.append((pos, info.offset))
                pos = max(pos, info.offset + info.numel)
            if pos < self._numel_padded:
                gaps.append((pos, self._numel_padded))
            self._grad_gap_list = gaps
        return gaps

    def _grad_view(self, info: "_ParamInfo") -> torch.Tensor:
        return self._grad_buffer()[info.offset:info.offset + info.numel].view(info.shape)

    def _claim_first_write(self, info: "_ParamInfo") -> bool:
        """True once per parameter and iteration: the caller must overwrite the range, not add to it."""
        self._grad_buffer()
        if id(info) in self._grad_unwritten:
            self._grad_unwritten.discard(id(info))
            return True
        return False

    def _zero_unwritten(self) -> None:
        buf = self._grad_buffer()
        for info in self._infos:
            if id(info) in self._grad_unwritten:
                buf[info.offset:info.offset + info.numel].zero_()
        self._grad_unwritten = set()

    def _collect_grads(self, grads) -> None:
        """Backward of `_FlatViews`: add the gradients autograd produced (everything except weights
        whose GEMM already accumulated into the buffer), then see whether the unit is complete."""
        buf = self._grad_buffer()
        dsts, srcs, cdst, csrc = [], [], [], []
        for info, g in zip(self._infos, grads):
            if g is not None:
                dst = buf[info.offset:info.offset + info.numel]
                src = g.reshape(-1) if g.dtype == buf.dtype else g.reshape(-1).to(buf.dtype)
                if self._claim_first_write(info):
                    cdst.append(dst)
                    csrc.append(src)
                else:
                    dsts.append(dst)
                    srcs.append(src)
        if cdst:
            torch._foreach_copy_(cdst, csrc)
        if dsts:
            torch._foreach_add_(dsts, srcs)      # a couple of multi-tensor launches instead of one per parameter
        self._post_backward()

    # ------------------------------------------------------------------ forward / backward
    def forward(self, *args, **kwargs):
        self._lazy_init()
        p = self.flat_param
        if self._is_root and self.world_size > 1:
            self._prefetch_gathers()
        if self._gather_event is not None:
            torch.cuda.current_stream().wait_event(self._gather_event)
            self._gather_event = None
        if not self._full_is_valid():
            self._gather_full()
        want_grad = torch.is_grad_enabled() and p.requires_grad
        if want_grad:
            # One leaf per iteration: when the unit is called several times before
            # backward (sequence micro-batching) every call shares it, so the
            # gradients of all calls accumulate into one flat buffer.
            if self._full_leaf is None:
                leaf = self._full.detach().requires_grad_(True)
                self._full_leaf = leaf
                self._calls = 0
                self._fires = 0
                self._set_views(leaf, track=True)
            self._calls += 1
        else:
            self._set_views(self._full)
        self.training_state = TrainingState.FORWARD
        out = self._wrapped(*args, **kwargs)
        self.training_state = TrainingState.IDLE
        if getattr(self, "_fused_pending", None):
            self._pull_pending()           # matrices that no gathering GEMM consumed in this call
        if self.reshard_after_forward and not self._is_root:
            self._free_full()
            if want_grad:
                out = self._arm_pre_backward(out)
        return out

    def _arm_pre_backward(self, out):
        self._bwd_hook_armed = True

        def pre_backward(grad):
            if self._bwd_hook_armed:
                self._bwd_hook_armed = False
                if not self._full_is_valid():
                    self._gather_full()
            return grad

        def visit(o):
            if isinstance(o, torch.Tensor) and o.requires_grad:
                o.register_hook(pre_backward)
            elif isinstance(o, (tuple, list)):
                for x in o:
                    visit(x)
        visit(out)
        return out

    def _post_backward(self, force: bool = False):
        """Runs whenever the gradients of one forward call have been collected.  With an
        activation-checkpointed block that is once per forward call of this iteration (each
        recomputation runs its own backward); otherwise once."""
        from .checkpoint import CheckpointWrapper
        self._fires += 1
        expected = self._calls if isinstance(self._wrapped, CheckpointWrapper) else 1
        if self._fires < expected and not force:
            return None          # keep accumulating in the flat gradient buffer
        self._zero_unwritten()
        flat_grad = self._grad_buffer()
        self._flat_grad = None
        self._full_leaf = None
        p = self.flat_param
        red_dtype = torch.float32 if (self.fp32_reduce_scatter or not self.mixed_precision) else self.compute_dtype
        g = flat_grad if flat_grad.dtype == red_dtype else flat_grad.to(red_dtype)
        root = self._root
        fused_rs = getattr(root, "_symm_rs", None)
        if self.world_size > 1 and fused_rs is not None and flat_grad.dtype == fused_rs.dtype:
            # peer-memory reduce-scatter: sum + 1/dp scale + cast + |g|^2 partial in one kernel
            accumulate = p._grad_shard is not None
            if accumulate and p._grad_shard.dtype != torch.float32:
                # second backward pass before an optimiser step: the running sum moves to fp32
                self._sync_comm()
                p._grad_shard = p._grad_shard.float()
            shard = p._grad_shard if accumulate else torch.empty(self._shard_numel, dtype=red_dtype, device=g.device)
            if getattr(root, "_fused_sumsq", None) is None:
                root._fused_sumsq = torch.zeros((), dtype=torch.float64, device=g.device)
                root._fused_sumsq_complete = True
                root._fused_sumsq_kind = "reduce_scatter"
            if accumulate:
                root._fused_sumsq_complete = False     # norm of a sum is not the sum of norms
            stream = root._comm_stream
            if stream is not None:
                stream.wait_stream(torch.cuda.current_stream())
            update = getattr(p, "_update_in_backward", None)
            if update is not None and not accumulate:
                # no clipping in this run: the optimiser's update of the shard rides in the same kernel
                with (torch.cuda.stream(stream) if stream is not None else _nullcontext()):
                    update(fused_rs, flat_grad, 1.0 / self.gradient_divide_factor, root._fused_sumsq,
                           self.piece_table(flat_grad.device))
                if stream is not None:
                    flat_grad.record_stream(stream)
                    root._pending.append(True)
                if self.reshard_after_forward and not self._is_root:
                    self._free_full()
                return None
            with (torch.cuda.stream(stream) if stream is not None else _nullcontext()):
                fused_rs.reduce_scatter(flat_grad, shard, 1.0 / self.gradient_divide_factor,
                                        root._fused_sumsq, accumulate, table=self.piece_table(flat_grad.device))
            if stream is not None:
                flat_grad.record_stream(stream)
                shard.record_stream(stream)
                root._pending.append(True)
            p._grad_shard = shard
            if self.reshard_after_forward and not self._is_root:
                self._free_full()
            return None
        if self.world_size > 1:
            if self.gradient_divide_factor != 1.0:
                g = g / self.gradient_divide_factor
            shard = torch.empty(self._shard_numel, dtype=red_dtype, device=g.device)

            def scatter():
                # the collective wants [what rank 0 owns | what rank 1 owns | ...]
                ordered = self._scratch(self._numel_padded, g.dtype, g.device)
                self._to_rank_major(g, ordered)
                reduce_scatter_flat(shard, ordered, self.process_group_reduce_scatter)

            if root._comm_stream is not None:
                root._comm_stream.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(root._comm_stream):
                    scatter()
                g.record_stream(root._comm_stream)
                shard.record_stream(root._comm_stream)
                root._pending.append(True)
            else:
                scatter()
        else:
            shard = g
            if self.gradient_divide_factor != 1.0:
                shard = shard / self.gradient_divide_factor
        if p._grad_shard is None:
            p._grad_shard = shard
        else:
            # several backward passes before one optimiser step: accumulate in fp32 like the
            # reference's FSDP (a bf16 running sum loses the small micro-batch contributions)
            self._sync_comm()
            p._grad_shard = p._grad_shard.float().add_(shard)
        if self.reshard_after_forward and not self._is_root:
            self._free_full()
        return None

    def _sync_comm(self) -> None:
        root = getattr(self, "_root", self)
        if root._comm_stream is not None and root._pending:
            torch.cuda.current_stream().wait_stream(root._comm_stream)
            root._pending.clear()

    def finish_backward(self) -> None:
        """Wait for outstanding reduce-scatters and (optionally) expose fp32
        `.grad` on the flat parameters.  Called by every public method that
        reads gradients; safe to call more than once."""
        self._lazy_init()
        from .checkpoint import CheckpointWrapper
        for u in self._units():
            if u._full_leaf is None:
                continue
            if u._flat_grad is not None:   # backward ended before every expected collection arrived
                u._post_backward(force=True)
            else:
                u._full_leaf = None
        self._sync_comm()
        if self.materialize_fp32_grads:
            for u in self._units():
                p = u.flat_param
                if p._grad_shard is not None:
                    g32 = p._grad_shard.float()
                    p.grad = g32 if p.grad is None else p.grad + g32
                    p._grad_shard = None

    def _grad_tensors(self) -> List[torch.Tensor]:
        out = []
        for u in self._units():
            p = u.flat_param
            if p._grad_shard is not None:
                out.append(p._grad_shard)
            if p.grad is not None:
                out.append(p.grad)
        return out

    # ------------------------------------------------------------------ public gradient API
    @torch.no_grad()
    def grad_all_reduce(self) -> None:
        """Sum gradients over the chunk-parallel group.  Must be called after
        backward when the chunk group holds replicas (reference semantics).  A
        no-op when the chunk group is part of the sharding group."""
        self._lazy_init()
        assert self._is_root, "grad_all_reduce should only be called on the root (parent) instance"
        self.assert_state(TrainingState.IDLE)
        self.finish_backward()
        if self.chunk_parallel_world_size == 1 or self.chunk_group_is_sharded:
            return
        fused = getattr(self, "_symm_allreduce", None)
        if fused is not None:
            # one pass over peer memory: sum over the chunk group + this rank's share of |g|^2
            acc = torch.zeros((), dtype=torch.float64, device=self.compute_device)
            rest = []
            for u in self._units():
                p = u.flat_param
                g, arena = p._grad_shard, getattr(u, "_grad_arena", None)
                if g is not None and arena is not None and g.data_ptr() == arena[0].local.data_ptr() + arena[1]:
                    # the gradient already lives in peer-mapped memory: reduced where it is (the slot's
                    # padding beyond the unit was zeroed when the region was made and nothing writes it)
                    fused.all_reduce_arena_(arena[1], arena[2], g.dtype, sumsq=acc)
                elif g is not None:
                    rest.append(g)
                if p.grad is not None:
                    rest.append(p.grad)
            if rest:
                fused.all_reduce_(rest, sumsq=acc)
            self._fused_sumsq = acc
            self._fused_sumsq_kind = "allreduce"
            return
        for g in self._grad_tensors():
            dist.all_reduce(g, group=self.chunk_parallel_process_group)
        # the squared norm a fused reduce-scatter accumulated describes the gradients BEFORE this sum
        self._fused_sumsq = None

    @torch.no_grad()
    def clip_grad_norm_(self, max_norm: Union[float, int], norm_type: Union[float, int] = 2.0) -> torch.Tensor:
        """Clip the global gradient norm (over the sharding group and the
        model-parallel group) to `max_norm`; returns the norm before clipping."""
        self._lazy_init()
        assert self._is_root, "clip_grad_norm should only be called on the root (parent) instance"
        self.assert_state(TrainingState.IDLE)
        self.finish_backward()
        max_norm, norm_type = float(max_norm), float(norm_type)
        grads = self._grad_tensors()
        dev = self.compute_device
        if dev.type == "cuda" and norm_type == 2.0:
            return self._clip_l2_on_device(grads, max_norm)
        local = calc_grad_norm(grads, norm_type).to(dev)
        if norm_type == math.inf:
            total = local
            if self.world_size > 1:
                dist.all_reduce(total, op=dist.ReduceOp.MAX, group=self.process_group)
            if self.model_parallel_world_size > 1:
                dist.all_reduce(total, op=dist.ReduceOp.MAX, group=self.model_parallel_process_group)
        else:
            total = local ** norm_type
            if self.world_size > 1:
                dist.all_reduce(total, group=self.process_group)
            if self.model_parallel_world_size > 1:
                dist.all_reduce(total, group=self.model_parallel_process_group)
            total = total ** (1.0 / norm_type)
        coef = max_norm / (total + 1e-6)
        if coef < 1:
            for g in grads:
                g.mul_(coef.to(g.dtype))
        return total

    def _clip_l2_on_device(self, grads: List[torch.Tensor], max_norm: float) -> torch.Tensor:
        """L2 clipping without a host round trip: sum-of-squares kernels into one
        fp64 scalar, scalar all-reduces, then every gradient is scaled by a
        coefficient that stays on the device (a no-op kernel when it is 1)."""
        from .. import ops
        from ..ops import cuda_ops
        acc = getattr(self, "_fused_sumsq", None)
        if acc is not None and getattr(self, "_fused_sumsq_kind", "") == "reduce_scatter":
            # the fused reduce-scatter already accumulated |shard|^2 (valid unless micro-batches were summed)
            self._fused_sumsq = None
            if not getattr(self, "_fused_sumsq_complete", True):
                acc = torch.zeros((), dtype=torch.float64, device=self.compute_device)
                for g in grads:
                    ops.sum_squares(g, acc)
        elif acc is not None:
            # the fused chunk-group all-reduce already produced per-rank partial sums of squares
            self._fused_sumsq = None
            dist.all_reduce(acc, group=self.chunk_parallel_process_group)
        else:
            acc = torch.zeros((), dtype=torch.float64, device=self.compute_device)
            for g in grads:
                ops.sum_squares(g, acc)
        if self.world_size > 1:
            dist.all_reduce(acc, group=self.process_group)
        if self.model_parallel_world_size > 1:
            dist.all_reduce(acc, group=self.model_parallel_process_group)
        norm, coef = cuda_ops.clip_coef(acc, max_norm)
        if getattr(self, "defer_grad_clip", False):
            # the fused optimiser multiplies by `coef` while it reads the gradients
            self._clip_coef = coef
        else:
            for g in grads:
                cuda_ops.scale_by_ptr(g, coef)
        return norm

    def zero_grad(self, set_to_none: bool = True) -> None:
        self._clip_coef = None
        self._fused_sumsq = None
        for u in self._units():
            u.flat_param.grad = None
            u.flat_param._grad_shard = None

    # ------------------------------------------------------------------ state dicts
    def _unit_prefixes(self) -> List[Tuple[str, "FullyShardedDataParallel"]]:
        out = []
        for name, m in self.named_modules():
            if isinstance(m, FullyShardedDataParallel):
                out.append((_clean_name(name), m))
        return out

    @torch.no_grad()
    def _full_fp32(self) -> torch.Tensor:
        shard = self.flat_param.data
        if self.world_size == 1:
            return shard
        full = torch.empty(self._numel_padded, dtype=shard.dtype, device=shard.device)
        tmp = torch.empty_like(full)
        all_gather_flat(tmp, shard.contiguous(), self.process_group)
        self._unshard(tmp, full)
        return full

    @torch.no_grad()
    def state_dict(self, *args, **kwargs) -> "OrderedDict[str, torch.Tensor]":
        """Full (unsharded, unflattened) fp32 state dict under the wrapped
        model's own parameter names; every rank of the sharding group must call
        it.  Tensors are moved to `state_dict_device` when that is set."""
        self._lazy_init()
        sd: "OrderedDict[str, torch.Tensor]" = OrderedDict()
        dev = self.state_dict_device
        for prefix, unit in self._unit_prefixes():
            full = unit._full_fp32()
            for info in unit._infos:
                t = full[info.offset:info.offset + info.numel].view(info.shape).clone()
                t = t.to(dev) if dev is not None else t
                for _, _, name in info.owners:
                    sd[f"{prefix}.{name}" if prefix else name] = t
        for name, buf in self._wrapped.named_buffers():
            owner = self._wrapped
            parts = name.split(".")
            for part in parts[:-1]:
                owner = owner._modules[part]
            if parts[-1] in owner._non_persistent_buffers_set:
                continue
            sd[_clean_name(name)] = buf.detach().clone().to(dev) if dev is not None else buf.detach().clone()
        return sd

    @torch.no_grad()
    def materialize_views(self) -> None:
        """Gather every unit (if it is not current) and hand the wrapped modules plain views of the
        parameters, without running a forward pass.  For code that calls sub-modules of the wrapped
        model directly (the fixed-shape decode session) right after construction or loading."""
        self._lazy_init()
        for unit in self._units():
            if unit._gather_event is not None:
                torch.cuda.current_stream().wait_event(unit._gather_event)
                unit._gather_event = None
            if not unit._full_is_valid():
                unit._gather_full()
            if getattr(unit, "_fused_pending", None):
                unit._pull_pending()
            unit._set_views(unit._full)

    @torch.no_grad()
    def gathered_state_dict(self) -> "OrderedDict[str, torch.Tensor]":
        """The compute-dtype parameters as they sit in the units' gathered buffers, under the wrapped
        model's names (views, no copy, no communication).  Needs every unit's buffer to be resident
        and current - i.e. a forward pass since the last optimiser step with
        `reshard_after_forward=False`.  Used to hand the weights of one parallel layout to another
        inside one process (chunk-parallel prefill, then tensor-parallel decode)."""
        self._lazy_init()
        sd: "OrderedDict[str, torch.Tensor]" = OrderedDict()
        for prefix, unit in self._unit_prefixes():
            if not unit._full_is_valid():
                raise RuntimeError(f"unit {prefix or '<root>'} holds no current gathered parameters")
            for info in unit._infos:
                t = unit._full[info.offset:info.offset + info.numel].view(info.shape)
                for _, _, name in info.owners:
                    sd[f"{prefix}.{name}" if prefix else name] = t
        for name, buf in self._wrapped.named_buffers():
            owner = self._wrapped
            parts = name.split(".")
            for part in parts[:-1]:
                owner = owner._modules[part]
            if parts[-1] not in owner._non_persistent_buffers_set:
                sd[_clean_name(name)] = buf.detach()
        return sd

    @torch.no_grad()
    def load_state_dict(self, state_dict: Dict[str, torch.Tensor], strict: bool = True):
        """Load a full state dict (every rank passes the same dict)."""
        self._lazy_init()
        missing, used = [], set()
        for prefix, unit in self._unit_prefixes():
            for info in unit._infos:
                src = None
                for _, _, name in info.owners:
                    key = f"{prefix}.{name}" if prefix else name
                    if key in state_dict:
                        src = state_dict[key]
                        used.add(key)
                if src is None:
                    missing.append(f"{prefix}.{info.name}" if prefix else info.name)
                    continue
                assert tuple(src.shape) == info.shape, (info.name, tuple(src.shape), info.shape)
                unit._write_piece(unit.flat_param.data, info, src.reshape(-1).to(unit.flat_param.device))
            unit.flat_param._master_version = getattr(unit.flat_param, "_master_version", 0) + 1
        bufs = dict(self._wrapped.named_buffers())
        for name, buf in bufs.items():
            key = _clean_name(name)
            if key in state_dict:
                buf.copy_(state_dict[key].to(buf.device))
                used.add(key)
        unexpected = [k for k in state_dict if k not in used]
        if strict and (missing or unexpected):
            raise RuntimeError(f"load_state_dict: missing={missing} unexpected={unexpected}")
        return nn.modules.module._IncompatibleKeys(missing, unexpected)

    @torch.no_grad()
    def local_state_dict(self) -> Dict[str, Any]:
        """This rank's shards only (no communication): the sharded-checkpoint payload."""
        self._lazy_init()
        out: Dict[str, Any] = {"shards": OrderedDict(), "meta": OrderedDict(), "buffers": OrderedDict()}
        for prefix, unit in self._unit_prefixes():
            key = prefix or "_root"
            out["shards"][key] = unit.flat_param.detach().cpu().clone()
            out["meta"][key] = {
                "world_size": unit.world_size, "rank": unit.rank, "numel_padded": unit._numel_padded,
                "layout": "per_parameter",      # rank r holds piece r of every parameter (see the module docstring)
                "params": [(i.name, list(i.shape), i.offset, i.piece, i.shard_offset) for i in unit._infos],
            }
        for name, buf in self._wrapped.named_buffers():
            out["buffers"][_clean_name(name)] = buf.detach().cpu().clone()
        return out

    @torch.no_grad()
    def load_local_state_dict(self, payload: Dict[str, Any]) -> None:
        self._lazy_init()
        for prefix, unit in self._unit_prefixes():
            key = prefix or "_root"
            meta = payload["meta"][key]
            assert (meta["world_size"] == unit.world_size and meta["rank"] == unit.rank
                    and meta.get("layout", "flat_cut" if unit.world_size > 1 else "per_parameter") == "per_parameter"), \
                "sharded checkpoint was written with a different sharding layout"
            unit.flat_param.data.copy_(payload["shards"][key].to(unit.flat_param.device))
            unit.flat_param._master_version = getattr(unit.flat_param, "_master_version", 0) + 1
        bufs = dict(self._wrapped.named_buffers())
        for name, buf in bufs.items():
            key = _clean_name(name)
            if key in payload["buffers"]:
                buf.copy_(payload["buffers"][key].to(buf.device))

    def extra_repr(self) -> str:
        return (f"world_size=({self.world_size}, {self.chunk_parallel_world_size}, "
                f"{self.model_parallel_world_size}), flatten_parameters={self.flatten_parameters}, "
                f"mixed_precision={self.mixed_precision}, compute_dtype={self.compute_dtype}, "
                f"fp32_reduce_scatter={self.fp32_reduce_scatter}, "
                f"reshard_after_forward={self.reshard_after_forward}")


class _WgradSink:
    """Carried by a 2-D weight view: where its gradient goes.  Calling it returns the matching view of the
    unit's flat gradient and whether the product has to be ADDED to what is there (False the first time in
    an iteration: the range is still uninitialised memory and the GEMM writes it)."""

    __slots__ = ("unit", "info")

    def __init__(self, unit, info):
        self.unit, self.info = unit, info

    def __call__(self):
        first = self.unit._claim_first_write(self.info)
        return self.unit._grad_view(self.info), not first


class _GatherSpec:
    """Carried by the view of a weight matrix whose all-gather is left to the first GEMM that consumes
    it (`ops.cuda_ops._Linear`): where every rank's row block lives, and whether it is still missing
    from the unit's gathered buffer."""
    __slots__ = ("unit", "info")

    def __init__(self, unit: "FullyShardedDataParallel", info: _ParamInfo):
        self.unit, self.info = unit, info

    @property
    def pending(self) -> bool:
        return self.info.name in self.unit._fused_pending

    def sources(self):
        """(address of every rank's row block, this rank)."""
        esize = self.unit._full.element_size()
        return [a + self.info.shard_offset * esize for a in self.unit._shard_peer_addr], self.unit.rank

    def done(self) -> None:
        self.unit._fused_pending.discard(self.info.name)

    def pull_now(self) -> None:
        root = getattr(self.unit, "_root", self.unit)
        root._symm_gather.pull_one(self.unit, self.info, self.unit._full.data)


def _ver(p: torch.Tensor):
    """Version of the master shard: autograd's counter (in-place updates by
    ordinary optimisers) plus a counter bumped by writers that go through
    `.data` (the fused optimiser, checkpoint loading)."""
    return (p._version, getattr(p, "_master_version", 0))


def _clean_name(name: str) -> str:
    """Drop wrapper path segments so names match the unwrapped model's."""
    return ".".join(p for p in name.split(".") if p not in ("_wrapped",))


# ---------------------------------------------------------------------- auto-wrap context
_WRAP_STATE: Dict[str, Any] = {"cls": None, "kwargs": None}


class enable_wrap:
    """Inside this context `wrap(module)` wraps with the given class/kwargs;
    outside it `wrap` is the identity (same contract as fairscale's)."""

    def __init__(self, wrapper_cls=FullyShardedDataParallel, **kwargs):
        self.cls, self.kwargs = wrapper_cls, kwargs

    def __enter__(self):
        self.prev = dict(_WRAP_STATE)
        _WRAP_STATE["cls"], _WRAP_STATE["kwargs"] = self.cls, self.kwargs
        return self

    def __exit__(self, *exc):
        _WRAP_STATE.update(self.prev)
        return False


def wrap(module: nn.Module, **overrides) -> nn.Module:
    if _WRAP_STATE["cls"] is None:
        return module
    kwargs = dict(_WRAP_STATE["kwargs"])
    kwargs.update(overrides)
    return _WRAP_STATE["cls"](module, **kwargs)
