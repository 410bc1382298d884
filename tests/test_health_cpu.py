"""Failure detection on CPU ranks (gloo): a rank that leaves, a rank that goes
silent, and a collective that would otherwise hang ends with an error."""
import datetime
import os
import time

import pytest
import torch

from dist_utils import _free_port, run_ranks


def _leaver(rank, world, port):
    from megalodon_b200.parallel.health import Heartbeat, PeerLost, StepGuard
    import torch.distributed as dist
    hb = Heartbeat.over_tcp("127.0.0.1", port, rank, world, timeout_s=1.0)
    guard = StepGuard(hb)
    log = []
    dist.barrier()                      # both ranks are up and have published their first heartbeat
    for step in range(30):
        try:
            guard.before_step(step)
        except PeerLost as e:
            log.append(("lost", e.rank, step))
            break
        if rank == 1 and step == 2:
            hb.leave(step)              # orderly exit between steps
            log.append(("left", rank, step))
            break
        time.sleep(0.1)
        log.append(("ok", rank, step))
    dist.barrier()                      # keep the store (hosted by rank 0) alive until everyone is done
    return log


def test_rank_that_leaves_is_noticed_before_the_next_step():
    port = _free_port()
    res = run_ranks(_leaver, 2, port)
    assert ("left", 1, 2) in res[1]
    assert any(e[0] == "lost" and e[1] == 1 for e in res[0]), res[0]


def _silent(rank, world, port):
    from megalodon_b200.parallel.health import Heartbeat, PeerLost
    hb = Heartbeat.over_tcp("127.0.0.1", port, rank, world, timeout_s=0.5)
    import torch.distributed as dist
    dist.barrier()
    out = "not detected"
    if rank == 1:
        time.sleep(2.0)                 # stops beating (stuck on the host)
        out = "silent"
    else:
        t0 = time.time()
        while time.time() - t0 < 3.0:
            hb.beat(0)
            try:
                hb.check()
            except PeerLost as e:
                out = ("lost", e.rank, round(time.time() - t0, 1))
                break
            time.sleep(0.1)
    dist.barrier()
    return out


def test_silent_rank_times_out():
    port = _free_port()
    res = run_ranks(_silent, 2, port)
    assert res[0][0] == "lost" and res[0][1] == 1 and res[0][2] < 2.5, res[0]


def test_heartbeat_logic_with_fake_clock():
    from megalodon_b200.parallel.health import Heartbeat, PeerLost

    class FakeStore(dict):
        def set(self, k, v):
            self[k] = v.encode()

        def get(self, k):
            return self[k]

        def check(self, keys):
            return all(k in self for k in keys)

    store = FakeStore()
    a = Heartbeat(store, 0, 2, timeout_s=10.0)
    a.check()                                       # peer not started: fine
    b = Heartbeat(store, 1, 2, timeout_s=10.0)
    a.check()
    with pytest.raises(PeerLost):
        a.check(now=time.time() + 11.0)             # peer's heartbeat is stale
    b.leave(7)
    with pytest.raises(PeerLost) as ei:
        a.check()
    assert "left the job at step 7" in str(ei.value)
