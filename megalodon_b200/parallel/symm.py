"""Peer-mapped ("symmetric") memory and the communication objects built on it.

`SymmetricRegion` gives every rank of a process group a buffer of the same size
and the device address of every peer's copy (allocation and the handle
exchange go through `torch.distributed._symmetric_memory`; the data path is
this framework's own kernels in `csrc/comm_kernels.cu`).

On top of it:

* `PeerMailbox` - the chunk-parallel state handoff.  A message is stored
  straight into the neighbour's mailbox slot and announced with a
  sequence-numbered flag; the receiver acknowledges into the sender's memory so
  a slot is never overwritten before it was read.  Drop-in transport for
  `chunk_parallel.mappings` (`set_handoff_transport("p2p", mailbox)`).
* `SymmetricAllReduce` - sum of gradient buffers over the group fused with the
  squared-norm partial sums needed for clipping.

Both also run over `HostFabric`, an in-process emulation of the peer memory of
all ranks, which is how the slot / sequence / acknowledgement protocol and the
timeout paths are tested without GPUs.

Failure handling
----------------
Waiting never blocks forever, and one lost signal costs one timeout for the
whole job, not one per wait:

* every wait is bounded by `timeout_s`;
* all communication objects of a device share one `AbortRecord`.  The first
  wait that runs out writes who it was there (rank, kind of wait, direction,
  sequence number wanted and seen); every later wait on that GPU returns at
  once;
* a kernel that gave up still signals its peers, with a poison value instead
  of a sequence number, so their waits return at once too and they poison
  their own neighbours in turn;
* the record is mirrored into pinned host memory: `AbortRecord.tripped()` is a
  plain host read (no device synchronisation) that a training loop can poll
  between steps; `check()` raises `PeerTimeout` with the recorded details.

After a failure the flags stay poisoned; `reset()` (collective) clears them.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.distributed as dist


class PeerTimeout(RuntimeError):
    """A bounded wait on a peer's flag ran out (or a peer that gave up released it)."""


POISON = 0xFFFFFFFF          # flag value written by a kernel that gave up
_BAD_INDEX_WHERE = {1: "gather: shard index", 2: "gather: natural index", 3: "reduce-scatter: natural index",
                    4: "reduce-scatter + AdamW: natural index"}
_WAIT_KINDS = {1: "send (waiting for the receiver to acknowledge the slot)", 2: "receive (waiting for the message)",
               3: "flag barrier", 4: "staged-buffer wait"}
_DIRS = {0: "forward", 1: "backward"}


def describe_abort(words) -> str:
    """Readable form of an abort record (sequence of >= 8 ints, word 0 = code)."""
    code, kind, where, want, seen, rank, tag, poisoned = (int(w) for w in list(words)[:8])
    if code == 30:
        idx = (where << 32) | (seen & 0xFFFFFFFF)
        return (f"{_BAD_INDEX_WHERE.get(kind, 'kernel')} {idx} outside a buffer of {want} elements: "
                f"the access was skipped (wrong piece table?) (code 30)")
    want &= 0xFFFFFFFF
    seen &= 0xFFFFFFFF
    what = _WAIT_KINDS.get(kind, f"wait of kind {kind}")
    loc = f"direction {_DIRS.get(where, where)}" if kind in (1, 2) else f"peer {where}"
    why = ("released by a poisoned flag: a peer gave up first" if poisoned
           else f"timed out: wanted {want}, flag shows {'POISON' if seen == POISON else seen}")
    return f"rank {rank}: {what}, {loc}, message/epoch {tag}: {why} (code {code})"


class AbortRecord:
    """The failure record shared by every communication object of one device (see the module docstring).
    `dev` is the int32[16] device tensor handed to the kernels, `host` its pinned mirror."""

    WORDS = 16
    _by_device: Dict[int, "AbortRecord"] = {}

    @classmethod
    def get(cls, device) -> "AbortRecord":
        device = torch.device(device)
        idx = device.index if device.index is not None else torch.cuda.current_device()
        rec = cls._by_device.get(idx)
        if rec is None:
            rec = cls._by_device[idx] = cls(torch.device("cuda", idx))
        return rec

    def __init__(self, device: torch.device):
        from ..ops._ext import require
        self.device = device
        self.host = torch.zeros(self.WORDS, dtype=torch.int32).pin_memory()
        words = [0] * self.WORDS
        addr = int(require().pinned_device_ptr(self.host))      # 0 if the mirror cannot be mapped
        for i, w in ((8, addr & 0xFFFFFFFF), (9, addr >> 32)):
            words[i] = w - (1 << 32) if w >= (1 << 31) else w
        self.dev = torch.tensor(words, dtype=torch.int32, device=device)

    def tripped(self) -> bool:
        """Host-only look at the pinned mirror: True once a kernel on this device gave up."""
        return int(self.host[0]) != 0

    def read(self) -> Optional[List[int]]:
        """The record (synchronises the device), or None when healthy."""
        words = self.dev.tolist()
        return words if words[0] != 0 else None

    def clear(self) -> None:
        self.dev[:8].zero_()
        self.host[:8].zero_()

    def check(self) -> None:
        words = self.read()
        if words is not None:
            raise PeerTimeout(describe_abort(words))


def _round_up(x: int, m: int) -> int:
    return -(-x // m) * m


# ----------------------------------------------------------------------------- memory
class SymmetricRegion:
    """`nbytes` of device memory on every rank of `group`, each rank knowing all addresses."""

    def __init__(self, nbytes: int, group: Optional[dist.ProcessGroup], device: torch.device):
        import torch.distributed._symmetric_memory as symm_mem
        self.nbytes = _round_up(nbytes, 256)
        self.group = group if group is not None else dist.group.WORLD
        self.device = torch.device(device)
        self.local = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=self.device)
        self.local.zero_()
        torch.cuda.synchronize(self.device)
        self.handle = symm_mem.rendezvous(self.local, self.group)
        self.rank = int(self.handle.rank)
        self.world = int(self.handle.world_size)
        self.ptrs: List[int] = [int(p) for p in self.handle.buffer_ptrs]
        self.ptr_table = torch.tensor(self.ptrs, dtype=torch.int64, device=self.device)
        dist.barrier(group=self.group)          # every rank has zeroed its copy

    def check_range(self, offset: int, nbytes: int = 0, rank: Optional[int] = None, align: int = 4) -> None:
        """Host-side validation of every address handed to a kernel: inside the region, aligned
        (4 bytes for flags, 16 for payload), existing rank.  A bad offset is an exception here,
        never a fault on a peer GPU."""
        if rank is not None and not 0 <= rank < self.world:
            raise ValueError(f"rank {rank} outside the region's group of {self.world}")
        if offset < 0 or nbytes < 0 or offset + nbytes > self.nbytes:
            raise ValueError(f"range [{offset}, {offset + nbytes}) outside the {self.nbytes}-byte region")
        if offset % align != 0:
            raise ValueError(f"offset {offset} is not {align}-byte aligned")

    def view(self, offset: int, nbytes: int, dtype: torch.dtype) -> torch.Tensor:
        self.check_range(offset, nbytes, align=16)
        return self.local[offset:offset + nbytes].view(dtype)

    def peer_ptr(self, rank: int, offset: int = 0, nbytes: int = 0) -> int:
        self.check_range(offset, nbytes, rank)
        return self.ptrs[rank] + offset

    def ptr_table_at(self, offset: int, nbytes: int = 0) -> torch.Tensor:
        self.check_range(offset, nbytes)
        return self.ptr_table + offset


class HostFabric:
    """In-process stand-in for the peer memory of `world` ranks (CPU tensors).
    Used by the tests of the host-side protocol logic."""

    def __init__(self, world: int, nbytes: int):
        self.world = world
        self.nbytes = _round_up(nbytes, 256)
        self.mem = [torch.zeros(self.nbytes, dtype=torch.uint8) for _ in range(world)]
        self.dropped_flags = 0        # fault injection: number of upcoming flag writes to lose
        self.abort: List[Optional[str]] = [None] * world     # per rank: why its "device" gave up
        self.timeouts = 0             # waits that ran their full time (a poisoned flag does not count)

    def region(self, rank: int) -> "HostRegion":
        return HostRegion(self, rank)


class HostRegion:
    def __init__(self, fabric: HostFabric, rank: int):
        self.fabric, self.rank, self.world, self.nbytes = fabric, rank, fabric.world, fabric.nbytes
        self.local = fabric.mem[rank]
        self.device = torch.device("cpu")

    def u32(self, rank: int, offset: int) -> torch.Tensor:
        return self.fabric.mem[rank][offset:offset + 4].view(torch.int32)

    def read_u32(self, rank: int, offset: int) -> int:
        return int(self.u32(rank, offset).item()) & 0xFFFFFFFF

    def write_u32(self, rank: int, offset: int, value: int) -> None:
        self.u32(rank, offset).fill_(value - (1 << 32) if value >= (1 << 31) else value)

    def bytes_of(self, rank: int, offset: int, nbytes: int) -> torch.Tensor:
        return self.fabric.mem[rank][offset:offset + nbytes]


# ----------------------------------------------------------------------------- mailbox
class PeerMailbox:
    """Line-topology mailbox between chunk-parallel neighbours.

    Memory layout of every rank's region (identical everywhere):
        [2 directions][n_slots] payload slots of slot_bytes
        [2][n_slots] uint32 arrival flags     (written by the sender)
        [2][n_slots] uint32 acknowledgements  (written by the receiver, into the sender's memory)
    Direction 0 = forward activations (from the previous rank), 1 = backward gradients (from the
    next rank).  Message k of a direction uses slot (k - 1) % n_slots with sequence number k.
    """

    FWD, BWD = 0, 1

    def __init__(self, region, prev_rank: Optional[int], next_rank: Optional[int], slot_bytes: int,
                 n_slots: int = 8, timeout_s: float = 30.0):
        self.region = region
        self.prev, self.next = prev_rank, next_rank       # ranks within the region's group
        self.slot_bytes = _round_up(slot_bytes, 256)
        self.n_slots = n_slots
        self.timeout_ns = int(timeout_s * 1e9)
        need = self.bytes_needed(slot_bytes, n_slots)
        assert region.nbytes >= need, f"region of {region.nbytes} B is too small for the mailbox ({need} B)"
        self.send_seq = [0, 0]
        self.recv_seq = [0, 0]
        self._is_host = isinstance(region, HostRegion)
        # Debug aid (MEGALODON_B200_POISON_SLOTS=1): a slot is overwritten with NaN patterns once it has
        # been read, so reading a slot that was not refilled shows up as NaNs downstream instead of the
        # plausible values of an older message ("poison, then verify" with `verify_received`).
        import os
        self.poison_slots = os.environ.get("MEGALODON_B200_POISON_SLOTS", "0") == "1"
        if not self._is_host:
            dev = region.device
            self._counters = torch.zeros(4, dtype=torch.int32, device=dev)
            self._abort = AbortRecord.get(dev)
            self._stage: Dict[int, torch.Tensor] = {}

    @staticmethod
    def bytes_needed(slot_bytes: int, n_slots: int = 8) -> int:
        return 2 * n_slots * _round_up(slot_bytes, 256) + 2 * 2 * n_slots * 4 + 256

    # ---- layout
    def _slot_off(self, direction: int, slot: int) -> int:
        return (direction * self.n_slots + slot) * self.slot_bytes

    def _flag_off(self, direction: int, slot: int) -> int:
        return 2 * self.n_slots * self.slot_bytes + (direction * self.n_slots + slot) * 4

    def _ack_off(self, direction: int, slot: int) -> int:
        return self._flag_off(0, 0) + 2 * self.n_slots * 4 + (direction * self.n_slots + slot) * 4

    @staticmethod
    def _dir(direction) -> int:
        return {"fwd": 0, "bwd": 1, 0: 0, 1: 1}[direction]

    # ---- transport API used by chunk_parallel.mappings
    def send(self, t: torch.Tensor, direction) -> None:
        d = self._dir(direction)
        peer = self.next if d == self.FWD else self.prev
        assert peer is not None, "no neighbour in that direction"
        nbytes = t.numel() * t.element_size()
        assert nbytes <= self.slot_bytes, f"message of {nbytes} B exceeds the slot size {self.slot_bytes} B"
        self.send_seq[d] += 1
        seq = self.send_seq[d]
        slot = (seq - 1) % self.n_slots
        need_ack = max(0, seq - self.n_slots)       # the previous message in this slot must have been read
        if self._is_host:
            self._host_send(t, d, peer, slot, seq, need_ack, nbytes)
        else:
            src, padded = self._padded(t, nbytes)
            from ..ops._ext import require
            require().p2p_send(src, self.region.peer_ptr(peer, self._slot_off(d, slot)), padded,
                               self.region.peer_ptr(peer, self._flag_off(d, slot)), seq,
                               self.region.peer_ptr(self.region.rank, self._ack_off(d, slot)), need_ack,
                               self._counters[d:d + 1], self.timeout_ns, self._abort.dev, self.region.rank, d)

    def recv(self, buf: torch.Tensor, direction) -> torch.Tensor:
        d = self._dir(direction)
        peer = self.prev if d == self.FWD else self.next
        assert peer is not None, "no neighbour in that direction"
        nbytes = buf.numel() * buf.element_size()
        assert nbytes <= self.slot_bytes
        self.recv_seq[d] += 1
        seq = self.recv_seq[d]
        slot = (seq - 1) % self.n_slots
        if self._is_host:
            self._host_recv(buf, d, peer, slot, seq, nbytes)
        else:
            dst, padded = self._padded(buf, nbytes, for_write=True)
            from ..ops._ext import require
            me = self.region.rank
            require().p2p_recv(dst, self.region.peer_ptr(me, self._slot_off(d, slot)), padded,
                               self.region.peer_ptr(me, self._flag_off(d, slot)), seq,
                               self.region.peer_ptr(peer, self._ack_off(d, slot)), self._counters[2 + d:3 + d],
                               self.timeout_ns, self._abort.dev, self.region.rank, d, self.poison_slots)
            if dst.data_ptr() != buf.data_ptr():
                buf.view(-1).view(torch.uint8).copy_(dst.view(torch.uint8)[:nbytes])
        return buf

    @staticmethod
    def verify_received(buf: torch.Tensor) -> None:
        """With slot poisoning on: a received tensor must not contain poison (synchronises)."""
        if buf.is_floating_point() and bool(torch.isnan(buf).any()):
            raise RuntimeError("received message contains poisoned words: the slot was read before it was refilled")

    def check(self) -> None:
        """Raise `PeerTimeout` if a kernel on this device gave up waiting (synchronises the device)."""
        if self._is_host:
            why = self.region.fabric.abort[self.region.rank]
            if why:
                raise PeerTimeout(why)
            return
        self._abort.check()

    def reset(self, group: Optional[dist.ProcessGroup] = None) -> None:
        """Back to the initial state after a failure: flags, acknowledgements, sequence numbers and the
        abort record are cleared.  Collective over the mailbox's group (every rank must call it with
        nothing in flight); on the host fabric it clears this rank's side only."""
        lo = self._flag_off(0, 0)
        n = 2 * 2 * self.n_slots * 4
        self.send_seq, self.recv_seq = [0, 0], [0, 0]
        if self._is_host:
            self.region.local[lo:lo + n].zero_()
            self.region.fabric.abort[self.region.rank] = None
            return
        torch.cuda.synchronize(self.region.device)
        self.region.local[lo:lo + n].zero_()
        self._counters.zero_()
        self._abort.clear()
        torch.cuda.synchronize(self.region.device)
        dist.barrier(group=group if group is not None else self.region.group)

    # ---- CUDA helpers
    def _padded(self, t: torch.Tensor, nbytes: int, for_write: bool = False):
        """The kernels move whole 16-byte words from 16-byte aligned addresses."""
        padded = _round_up(nbytes, 16)
        tc = t if t.is_contiguous() else t.contiguous()
        if padded == nbytes and tc.data_ptr() % 16 == 0 and (tc is t or not for_write):
            return tc, padded
        stage = self._stage.get(padded)
        if stage is None:
            stage = torch.zeros(padded, dtype=torch.uint8, device=self.region.device)
            self._stage[padded] = stage
        if not for_write:
            stage[:nbytes].copy_(tc.view(-1).view(torch.uint8))
        return stage, padded

    # ---- host emulation (same protocol as the kernels, CPU tensors; a wait that is not already
    # satisfied counts as one that ran its full time)
    def _host_wait(self, rank_of_flag: int, off: int, want: int, what: str) -> None:
        r = self.region
        fab = r.fabric
        if fab.abort[r.rank]:
            raise PeerTimeout(f"rank {r.rank}: gave up earlier ({fab.abort[r.rank]})")
        seen = r.read_u32(rank_of_flag, off)
        if seen == POISON:
            fab.abort[r.rank] = f"rank {r.rank}: {what}: released by a poisoned flag: a peer gave up first"
        elif seen < want:
            fab.timeouts += 1
            fab.abort[r.rank] = f"rank {r.rank}: {what}: timed out: wanted {want}, flag shows {seen}"
        else:
            return
        raise PeerTimeout(fab.abort[r.rank])

    def _host_send(self, t, d, peer, slot, seq, need_ack, nbytes):
        r = self.region
        try:
            if r.fabric.abort[r.rank] or need_ack:
                self._host_wait(r.rank, self._ack_off(d, slot), need_ack,
                                f"send (waiting for the receiver to acknowledge the slot), direction {_DIRS[d]}")
        except PeerTimeout:
            r.write_u32(peer, self._flag_off(d, slot), POISON)       # releases the receiver at once
            raise
        r.bytes_of(peer, self._slot_off(d, slot), nbytes).copy_(t.detach().contiguous().view(-1).view(torch.uint8))
        if r.fabric.dropped_flags > 0:
            r.fabric.dropped_flags -= 1          # injected fault: the flag write is lost
            return
        r.write_u32(peer, self._flag_off(d, slot), seq)

    def _host_recv(self, buf, d, peer, slot, seq, nbytes):
        r = self.region
        try:
            self._host_wait(r.rank, self._flag_off(d, slot), seq,
                            f"receive (waiting for the message), direction {_DIRS[d]}")
        except PeerTimeout:
            r.write_u32(peer, self._ack_off(d, slot), POISON)        # releases a sender waiting for this slot
            raise
        buf.view(-1).view(torch.uint8).copy_(r.bytes_of(r.rank, self._slot_off(d, slot), nbytes))
        r.write_u32(peer, self._ack_off(d, slot), seq)


# ----------------------------------------------------------------------------- all-reduce + grad norm
class SymmetricAllReduce:
    """In-place sum over the group of tensors staged through a symmetric bucket,
    returning the squared L2 norm of the reduced values (this rank's slice:
    summing the returned partials over the group gives the full norm)."""

    def __init__(self, region: SymmetricRegion, bucket_bytes: int, timeout_s: float = 30.0):
        self.region = region
        self.bucket_bytes = (bucket_bytes // 256) * 256
        assert region.nbytes >= self.bytes_needed(bucket_bytes, region.world)
        self.pad_off = self.bucket_bytes
        self.timeout_ns = int(timeout_s * 1e9)
        self.epoch = 0
        dev = region.device
        self._abort = AbortRecord.get(dev)
        self._bufs = region.ptr_table_at(0).contiguous()
        self._pads = region.ptr_table_at(self.pad_off).contiguous()

    @staticmethod
    def bytes_needed(bucket_bytes: int, world: int) -> int:
        return (bucket_bytes // 256) * 256 + _round_up(4 * world, 256)

    def _barrier(self) -> None:
        from ..ops._ext import require
        self.epoch += 1
        require().peer_barrier(self._pads, self.region.rank, self.epoch, self.timeout_ns, self._abort.dev, self.epoch)

    @torch.no_grad()
    def all_reduce_(self, tensors: List[torch.Tensor], sumsq: Optional[torch.Tensor] = None,
                    scale: float = 1.0) -> None:
        """Sum every tensor over the group in place; `sumsq` (fp64 scalar) accumulates
        this rank's share of the squared norm of the results."""
        from ..ops._ext import require
        from ..ops.cuda_ops import _DT
        ext = require()
        for t in tensors:
            flat = t.view(-1)
            esize = flat.element_size()
            per = self.bucket_bytes // esize
            for lo in range(0, flat.numel(), per):
                part = flat[lo:lo + per]
                nbytes = part.numel() * esize
                padded = _round_up(nbytes, 16 * self.region.world)
                stage = self.region.view(0, padded, t.dtype)
                stage[:part.numel()].copy_(part)
                if padded != nbytes:
                    stage[part.numel():].zero_()
                self._barrier()                      # every rank has staged its bucket
                ext.allreduce_sumsq(self._bufs, self.region.rank, padded, scale, sumsq, _DT[t.dtype], self._abort.dev)
                self._barrier()                      # every rank has pushed its reduced slice
                part.copy_(stage[:part.numel()])

    # ---- gradients that already live in peer-mapped memory (no copy-in / copy-out)
    def attach_arena(self, arena: SymmetricRegion) -> None:
        """`arena`: a region in which the caller keeps its gradient buffers at the same offsets on every
        rank; `all_reduce_arena_` then reduces them where they are."""
        self.arena = arena

    @torch.no_grad()
    def all_reduce_arena_(self, offset: int, nbytes: int, dtype: torch.dtype,
                          sumsq: Optional[torch.Tensor] = None, scale: float = 1.0) -> None:
        """Sum bytes [offset, offset + nbytes) of the arena over the group in place (every rank reduces one
        slice from all peers and pushes the result to all of them), with this rank's share of the squared
        norm added to `sumsq`.  `nbytes` must be a multiple of 16 * world.  Two barriers, no copies."""
        from ..ops._ext import require
        from ..ops.cuda_ops import _DT
        assert nbytes % (16 * self.region.world) == 0 and offset % 16 == 0
        self.arena.check_range(offset, nbytes, align=16)
        bufs = self.arena.ptr_table_at(offset, nbytes)
        self._barrier()                      # every rank's backward has written this range
        require().allreduce_sumsq(bufs, self.region.rank, nbytes, scale, sumsq, _DT[dtype], self._abort.dev)
        self._barrier()                      # every rank has pushed its reduced slice

    def check(self) -> None:
        self._abort.check()

    def reset(self) -> None:
        """Collective: clear the signal pad, the epoch and the abort record after a failure."""
        _reset_pads(self, self.region, self.pad_off)


class SmallCollective:
    """All-reduce and last-dimension all-gather of small 16-bit tensors (the activations of a decode step)
    over peer memory, one kernel each, with the epoch kept in device memory: the calls carry no
    per-launch sequence number, so a step that contains them can be captured in a CUDA graph and replayed.
    Every rank must issue the same sequence of calls.  Results are bitwise identical on all ranks (the
    slots are summed in rank order)."""

    def __init__(self, group: Optional[dist.ProcessGroup], device: torch.device, max_bytes: int = 1 << 18,
                 timeout_s: float = 10.0):
        self.slot_bytes = _round_up(max_bytes, 256)
        world = dist.get_world_size(group)
        self.buf_bytes = 2 * world * self.slot_bytes
        self.region = SymmetricRegion(self.buf_bytes + _round_up(4 * world, 256), group, device)
        self.rank, self.world = self.region.rank, world
        self.timeout_ns = int(timeout_s * 1e9)
        self._abort = AbortRecord.get(self.region.device)
        self._bufs = self.region.ptr_table_at(0).contiguous()
        self._pads = self.region.ptr_table_at(self.buf_bytes).contiguous()
        self._counter = torch.zeros(1, dtype=torch.int32, device=self.region.device)
        torch.cuda.synchronize(self.region.device)
        dist.barrier(group=self.region.group)          # every pad is zero before the first flag arrives

    def fits(self, x: torch.Tensor) -> bool:
        nbytes = x.numel() * x.element_size()
        return (x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and 0 < nbytes <= self.slot_bytes
                and nbytes % 16 == 0 and (x.shape[-1] * 2) % 16 == 0)

    def _call(self, x: torch.Tensor, gather: bool) -> torch.Tensor:
        from ..ops._ext import require
        return require().small_collective(x.contiguous(), self._bufs, self._pads, self._counter, self.rank,
                                          self.slot_bytes, gather, self.timeout_ns, self._abort.dev)

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        return self._call(x, False)

    def all_gather_last_dim(self, x: torch.Tensor) -> torch.Tensor:
        return self._call(x, True)

    def check(self) -> None:
        self._abort.check()


class SymmetricReduceScatter:
    """Gradient reduce-scatter of an FSDP unit by pulling from peer memory, fused with the averaging
    scale, the cast to the shard dtype and the squared-norm partial sum used for clipping.  Two staging
    buffers alternate, so one flag barrier per unit is enough (see `reduce_scatter`)."""

    def __init__(self, group, device, max_numel: int, dtype: torch.dtype, timeout_s: float = 60.0):
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.dtype = dtype
        esize = torch.empty(0, dtype=dtype).element_size()
        self.stage_bytes = _round_up(max_numel * esize, 256)
        self.pad_off = 2 * self.stage_bytes
        self.region = SymmetricRegion(self.pad_off + _round_up(4 * self.world, 256), group, device)
        self._pads = self.region.ptr_table_at(self.pad_off).contiguous()
        self._bufs = [self.region.ptr_table_at(0).contiguous(), self.region.ptr_table_at(self.stage_bytes).contiguous()]
        self._abort = AbortRecord.get(device)
        self.timeout_ns = int(timeout_s * 1e9)
        self.epoch = 0
        self._toggle = 0

    @torch.no_grad()
    def reduce_scatter(self, flat_grad: torch.Tensor, out_shard: torch.Tensor, scale: float,
                       sumsq: Optional[torch.Tensor], accumulate: bool = False,
                       table: Optional[torch.Tensor] = None) -> None:
        """out_shard (+)= scale * (this rank's slice of the sum over ranks of flat_grad).  With `table`
        (the unit's `piece_table`) `flat_grad` is in natural parameter order and the slice of rank r is
        piece r of every parameter; without it the slice is the contiguous range r.

        Staging buffer t is rewritten two calls later; by then every peer has passed the barrier of
        the call in between, which its stream reaches only after its own read of buffer t finished."""
        from ..ops._ext import require
        from ..ops.cuda_ops import _DT
        ext = require()
        n = flat_grad.numel()
        assert n * flat_grad.element_size() <= self.stage_bytes and flat_grad.dtype == self.dtype
        assert n == out_shard.numel() * self.world
        t = self._toggle
        self._toggle ^= 1
        stage = self.region.view(t * self.stage_bytes, n * flat_grad.element_size(), flat_grad.dtype)
        stage.copy_(flat_grad.view(-1))
        self.epoch += 1
        ext.peer_barrier(self._pads, self.rank, self.epoch, self.timeout_ns, self._abort.dev, self.epoch)
        ext.reduce_scatter_sumsq(self._bufs[t], self.rank, _DT[flat_grad.dtype], scale, out_shard, sumsq, accumulate,
                                 self._abort.dev, table)

    @torch.no_grad()
    def reduce_scatter_adamw(self, flat_grad: torch.Tensor, master: torch.Tensor, exp_avg: torch.Tensor,
                             exp_avg_sq: torch.Tensor, low: Optional[torch.Tensor], scale: float,
                             sumsq: Optional[torch.Tensor], *, lr: float, beta1: float, beta2: float, eps: float,
                             weight_decay: float, step: int, table: Optional[torch.Tensor] = None) -> None:
        """Reduce-scatter fused with the AdamW update of this rank's shard (see
        `reduce_scatter_adamw_kernel`): the reduced gradient is consumed in registers, `master`,
        `exp_avg`, `exp_avg_sq` (fp32 shards) are updated in place and `low` receives the
        compute-dtype copy of the new weights."""
        from ..ops._ext import require
        from ..ops.cuda_ops import _DT
        ext = require()
        n = flat_grad.numel()
        assert n * flat_grad.element_size() <= self.stage_bytes and flat_grad.dtype == self.dtype
        assert n == master.numel() * self.world
        t = self._toggle
        self._toggle ^= 1
        stage = self.region.view(t * self.stage_bytes, n * flat_grad.element_size(), flat_grad.dtype)
        stage.copy_(flat_grad.view(-1))
        self.epoch += 1
        ext.peer_barrier(self._pads, self.rank, self.epoch, self.timeout_ns, self._abort.dev, self.epoch)
        ext.reduce_scatter_adamw(self._bufs[t], self.rank, _DT[flat_grad.dtype], scale, master, exp_avg, exp_avg_sq,
                                 low, sumsq, lr, beta1, beta2, eps, weight_decay, step, self._abort.dev, table)

    def check(self) -> None:
        self._abort.check()

    def reset(self) -> None:
        """Collective: clear the signal pad, the epoch and the abort record after a failure."""
        _reset_pads(self, self.region, self.pad_off)
        self._toggle = 0


class SymmetricParamGather:
    """Parameter all-gather of FSDP units by pulling from peer memory (replaces the NCCL all-gather
    that fairscale issues before every block, reference model/mega.py:251-262).

    The compute-dtype shard of every unit lives in one peer-mapped region.  `pull(unit, full)` runs
    one kernel that reads piece r of every parameter from rank r's shard and writes it to its place
    in the natural-order buffer `full` - no rank-major staging copy, no reordering pass.  Before the
    first pull after an optimiser step, `shards_written()` runs a flag barrier: every rank has
    finished writing its shards (the fused AdamW kernel writes them).  Overwriting a shard that a
    slower rank is still reading cannot happen: a rank updates its shards only after the gradient
    reductions of the step, which need every rank's backward pass and therefore every rank's pulls."""

    def __init__(self, model, timeout_s: float = 30.0, fuse_into_gemm: bool = True):
        from ..ops._ext import require
        self.model = model
        # With `fuse_into_gemm` the weight matrices of the blocks are not pulled by `pull` at all: the
        # forward GEMM that first consumes a weight gathers it itself, its copy warps pulling the row
        # blocks from their owners while the tensor cores work on the rows already there
        # (`GemmGatherSpec` in csrc/kernels.h).  `pull` then moves only the small parameters.
        self.fuse_into_gemm = fuse_into_gemm
        units = model._units()
        self.group = model.process_group
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        device = next(model.parameters()).device
        esize = torch.empty(0, dtype=model.compute_dtype).element_size()
        offs, total = [], 0
        for u in units:
            assert u.process_group is self.group, "all units must share the sharding group"
            assert len(u._infos) <= require().piece_table_limit(), "too many parameters in one unit"
            offs.append(total)
            total += _round_up(u._shard_numel * esize, 256)
        self.pad_off = total
        self.region = SymmetricRegion(total + _round_up(4 * self.world, 256), self.group, device)
        self._pads = self.region.ptr_table_at(self.pad_off).contiguous()
        self._abort = AbortRecord.get(device)
        self.timeout_ns = int(timeout_s * 1e9)
        self.epoch = 0
        self._token = None
        self._peer_ptrs: Dict[int, torch.Tensor] = {}
        for u, off in zip(units, offs):
            shard = self.region.view(off, u._shard_numel * esize, model.compute_dtype)
            p = u.flat_param
            shard.copy_(p.data)
            p._lowp_shard = shard
            p._lowp_version = (p._version, getattr(p, "_master_version", 0))
            self._peer_ptrs[id(u)] = self.region.ptr_table_at(off).contiguous()
            u._shard_peer_addr = [self.region.peer_ptr(r, off) for r in range(self.world)]
            u._fused_infos = self._fusable(u) if fuse_into_gemm and not u._is_root else []
            u._fused_pending = set()
        torch.cuda.synchronize(device)
        dist.barrier(group=self.group)

    def _fusable(self, unit) -> list:
        """Parameters of `unit` that the gathering GEMM can take: matrices [N, K] whose row blocks are
        whole 128-row chunks without padding."""
        out = []
        for i in unit._infos:
            if (len(i.shape) == 2 and i.shape[0] % (self.world * 128) == 0 and i.shape[1] % 64 == 0
                    and i.piece * self.world == i.numel):
                out.append(i)
        return out

    def shards_written(self) -> None:
        """Flag barrier on the current stream, once per version of the master weights."""
        from ..ops._ext import require
        root = self.model
        token = tuple((u.flat_param._version, getattr(u.flat_param, "_master_version", 0)) for u in root._units())
        if token == self._token:
            return
        self._token = token
        for u in root._units():
            u._lowp_shard()                  # a no-op unless the master weights changed behind the optimiser
        self.epoch += 1
        require().peer_barrier(self._pads, self.rank, self.epoch, self.timeout_ns, self._abort.dev, self.epoch)

    def pull(self, unit, full: torch.Tensor) -> None:
        """Gather `unit` into `full`, except the matrices left to the gathering GEMMs (they are marked
        pending on the unit; `FullyShardedDataParallel.forward` pulls whatever no GEMM took)."""
        from ..ops._ext import require
        skip = unit._fused_infos
        if skip:
            names = {i.name for i in skip}
            rest = [i for i in unit._infos if i.name not in names]
            table = unit.piece_table(full.device, rest, key="unfused")
            listed = self.world * sum(i.piece for i in rest)
            unit._fused_pending = set(names)
        else:
            table = unit.piece_table(full.device)
            listed = unit._numel_padded
        if listed:
            require().gather_pull(full, self._peer_ptrs[id(unit)], table, listed, self._abort.dev, unit._shard_numel)

    def pull_one(self, unit, info, full: torch.Tensor) -> None:
        """Gather a single parameter (a matrix whose first use was not a gathering GEMM)."""
        from ..ops._ext import require
        table = unit.piece_table(full.device, [info], key=("one", info.name))
        require().gather_pull(full, self._peer_ptrs[id(unit)], table, self.world * info.piece, self._abort.dev,
                              unit._shard_numel)
        unit._fused_pending.discard(info.name)

    def check(self) -> None:
        self._abort.check()

    def reset(self) -> None:
        _reset_pads(self, self.region, self.pad_off)
        self._token = None


def enable_peer_gather(model, timeout_s: float = 30.0,
                       fuse_into_gemm: Optional[bool] = None) -> Optional[SymmetricParamGather]:
    """Replace the NCCL parameter all-gather of every FSDP unit of `model` by pulls from peer memory;
    with `fuse_into_gemm` (default on, MEGALODON_B200_FUSED_AG=0 turns it off) the weight matrices are
    gathered inside the GEMM that first consumes them."""
    import os
    if getattr(model, "world_size", 1) <= 1 or not getattr(model, "mixed_precision", False):
        return None
    if fuse_into_gemm is None:
        fuse_into_gemm = os.environ.get("MEGALODON_B200_FUSED_AG", "1") == "1"
    model._lazy_init()
    sg = SymmetricParamGather(model, timeout_s=timeout_s, fuse_into_gemm=fuse_into_gemm)
    model._symm_gather = sg
    return sg


def _reset_pads(obj, region: SymmetricRegion, pad_off: int) -> None:
    torch.cuda.synchronize(region.device)
    region.local[pad_off:pad_off + _round_up(4 * region.world, 256)].zero_()
    obj.epoch = 0
    obj._abort.clear()
    torch.cuda.synchronize(region.device)
    dist.barrier(group=region.group)


# ----------------------------------------------------------------------------- wiring
def enable_peer_transport(model, max_batch: int, *, n_slots: int = 8, allreduce_bucket_mb: int = 256,
                          timeout_s: float = 30.0):
    """Switch a built (FSDP-wrapped) model to the peer-memory data paths of its
    chunk-parallel group: the state handoff between neighbouring ranks goes
    through a `PeerMailbox`, and (when gradients are replicated over the chunk
    group) `grad_all_reduce()` uses `SymmetricAllReduce`.  Call on every rank of
    the chunk group after `build_model`.  Returns (mailbox, allreduce | None)."""
    from .chunk_parallel.mappings import set_handoff_transport
    from .initialize import get_chunk_parallel_group, get_chunk_parallel_rank, get_chunk_parallel_world_size
    cp = get_chunk_parallel_world_size()
    if cp == 1:
        return None, None
    import os
    import warnings
    if os.environ.get("CUDA_MODULE_LOADING", "").upper() != "EAGER":
        warnings.warn("CUDA_MODULE_LOADING is not EAGER: a lazy kernel load behind a kernel that waits for a peer "
                      "can stall both ranks until the bounded waits time out")
    inner = model
    while hasattr(inner, "_wrapped"):
        inner = inner._wrapped
    mega = inner.layers[0]
    while hasattr(mega, "_wrapped"):
        mega = mega._wrapped
    mega = mega.mega
    width = 2 * mega.timenorm.groups_per_partition + 2 * mega.local_mdim * mega.cema.ndim
    slot_bytes = max_batch * width * 4
    device = next(model.parameters()).device
    group = get_chunk_parallel_group()
    r = get_chunk_parallel_rank()
    region = SymmetricRegion(PeerMailbox.bytes_needed(slot_bytes, n_slots), group, device)
    mailbox = PeerMailbox(region, r - 1 if r > 0 else None, r + 1 if r + 1 < cp else None, slot_bytes,
                          n_slots=n_slots, timeout_s=timeout_s)
    set_handoff_transport("p2p", mailbox)
    if (getattr(model, "world_size", 1) > 1 and getattr(model, "mixed_precision", False)
            and os.environ.get("MEGALODON_B200_PEER_RS", "1") == "1"):
        enable_peer_reduce_scatter(model, timeout_s=timeout_s)
    if os.environ.get("MEGALODON_B200_PEER_AG", "1") == "1":
        enable_peer_gather(model, timeout_s=timeout_s)
    reducer = None
    if not getattr(model, "chunk_group_is_sharded", False):
        bucket = allreduce_bucket_mb << 20
        ar_region = SymmetricRegion(SymmetricAllReduce.bytes_needed(bucket, cp), group, device)
        reducer = SymmetricAllReduce(ar_region, bucket, timeout_s=timeout_s)
        model._symm_allreduce = reducer
        if (getattr(model, "world_size", 1) == 1 and hasattr(model, "_units")
                and getattr(model, "mixed_precision", False)
                and os.environ.get("MEGALODON_B200_GRAD_ARENA", "1") == "1"):
            # no data parallelism inside the chunk group: the flat gradient of every unit IS what gets
            # all-reduced, so it is kept in peer-mapped memory and reduced where it is
            model._lazy_init()
            units = list(model._units())
            step = 16 * cp
            sizes = [_round_up(u._numel_padded * u._full_dtype_size(), max(256, step)) for u in units]
            arena = SymmetricRegion(sum(sizes), group, device)
            off = 0
            for u, nb in zip(units, sizes):
                u._grad_arena = (arena, off, nb)
                off += nb
            reducer.attach_arena(arena)
    return mailbox, reducer


def enable_peer_reduce_scatter(model, timeout_s: float = 60.0) -> Optional[SymmetricReduceScatter]:
    """Replace the NCCL reduce-scatter of every FSDP unit of `model` by the fused peer-memory kernel
    (reduce + scale + cast + gradient-norm partial sums)."""
    if getattr(model, "world_size", 1) <= 1:
        return None
    units = model._units()
    biggest = max(u._numel_padded for u in units)
    device = next(model.parameters()).device
    rs = SymmetricReduceScatter(model.process_group, device, biggest, model.compute_dtype, timeout_s=timeout_s)
    model._lazy_init()
    model._symm_rs = rs
    return rs
