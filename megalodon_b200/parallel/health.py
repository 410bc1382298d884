"""Failure detection between steps (the reference relies on the NCCL watchdog and
SLURM requeue only, distributed/setup.py:17-40).

Every rank publishes a heartbeat (step number + wall-clock time) to a key-value
store between steps and looks at its peers' heartbeats before it launches the
next step.  A peer whose heartbeat is older than `timeout_s`, or that announced
its departure, makes `check()` raise `PeerLost` *on the host, before any kernel
or collective of the next step is enqueued* - so the survivors neither hang in
a collective nor leave work in flight.  Device-side waits (mailbox flags, peer
barriers, mbarriers) are bounded separately and report through error words
(`PeerMailbox.check`, `cuda_ops.check_kernel_errors`); `StepGuard` polls all of
them at one place.
"""
from __future__ import annotations

import json
import time
from typing import Callable, Iterable, List, Optional

import torch.distributed as dist


class PeerLost(RuntimeError):
    def __init__(self, rank: int, why: str):
        super().__init__(f"rank {rank} {why}")
        self.rank = rank


class Heartbeat:
    def __init__(self, store, rank: int, world: int, timeout_s: float = 60.0, prefix: str = "hb"):
        self.store, self.rank, self.world = store, rank, world
        self.timeout_s = timeout_s
        self.prefix = prefix
        self.beat(step=-1)

    @classmethod
    def over_tcp(cls, host: str, port: int, rank: int, world: int, timeout_s: float = 60.0) -> "Heartbeat":
        import datetime
        store = dist.TCPStore(host, port, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=30),
                              wait_for_workers=False)
        return cls(store, rank, world, timeout_s)

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def beat(self, step: int, leaving: bool = False) -> None:
        self.store.set(self._key(self.rank), json.dumps({"step": step, "t": time.time(), "leaving": leaving}))

    def leave(self, step: int) -> None:
        """Announce an orderly exit (call between steps, with nothing in flight)."""
        self.beat(step, leaving=True)

    def peers(self) -> List[Optional[dict]]:
        out: List[Optional[dict]] = []
        for r in range(self.world):
            try:
                out.append(json.loads(self.store.get(self._key(r)).decode()) if self.store.check([self._key(r)]) else None)
            except Exception:  # noqa: BLE001 - an unreachable store counts as "no news"
                out.append(None)
        return out

    def check(self, now: Optional[float] = None) -> None:
        now = time.time() if now is None else now
        for r, hb in enumerate(self.peers()):
            if r == self.rank:
                continue
            if hb is None:
                continue                      # has not started yet
            if hb.get("leaving"):
                raise PeerLost(r, f"left the job at step {hb['step']}")
            if now - hb["t"] > self.timeout_s:
                raise PeerLost(r, f"sent no heartbeat for {now - hb['t']:.1f} s (last step {hb['step']})")


class StepGuard:
    """Call `before_step(step)` at the top of every training step: publishes this rank's heartbeat, checks
    the peers' and polls the device-side error words collected from the previous step."""

    def __init__(self, heartbeat: Optional[Heartbeat] = None, checks: Iterable[Callable[[], None]] = ()):
        self.heartbeat = heartbeat
        self.checks = list(checks)

    def before_step(self, step: int) -> None:
        for fn in self.checks:
            fn()
        if self.heartbeat is not None:
            self.heartbeat.beat(step)
            self.heartbeat.check()
