"""Host-side logic of the peer mailbox (slots, sequence numbers,
acknowledgements, timeouts) on the in-process fabric - no GPU involved."""
import pytest
import torch

from megalodon_b200.parallel.symm import HostFabric, PeerMailbox, PeerTimeout


def _pair(n_slots=2, slot_bytes=64):
    fabric = HostFabric(2, PeerMailbox.bytes_needed(slot_bytes, n_slots))
    a = PeerMailbox(fabric.region(0), None, 1, slot_bytes, n_slots=n_slots)
    b = PeerMailbox(fabric.region(1), 0, None, slot_bytes, n_slots=n_slots)
    return fabric, a, b


def test_messages_arrive_in_order_and_slots_are_reused():
    _, a, b = _pair(n_slots=2)
    for k in range(7):                      # more messages than slots: acknowledgements recycle them
        msg = torch.full((12,), float(k))
        a.send(msg, "fwd")
        out = torch.empty(12)
        b.recv(out, "fwd")
        assert torch.equal(out, msg)
        grad = torch.full((5,), -float(k))
        b.send(grad, "bwd")
        back = torch.empty(5)
        a.recv(back, "bwd")
        assert torch.equal(back, grad)


def test_receive_without_send_times_out_and_reset_recovers():
    fabric, a, b = _pair()
    out = torch.empty(4)
    with pytest.raises(PeerTimeout):
        b.recv(out, "fwd")
    assert fabric.timeouts == 1
    with pytest.raises(PeerTimeout):         # the failure is sticky: no second full-length wait
        b.recv(out, "fwd")
    assert fabric.timeouts == 1
    with pytest.raises(PeerTimeout):
        b.check()
    a.reset()
    b.reset()
    a.send(torch.arange(4.0), "fwd")
    b.recv(out, "fwd")
    assert torch.equal(out, torch.arange(4.0))
    b.check()


def test_sender_may_not_lap_the_receiver():
    _, a, b = _pair(n_slots=2)
    a.send(torch.zeros(4), "fwd")
    a.send(torch.ones(4), "fwd")
    with pytest.raises(PeerTimeout):         # third message would overwrite an unread slot
        a.send(torch.ones(4) * 2, "fwd")


def test_dropped_flag_is_detected_by_the_receiver():
    fabric, a, b = _pair()
    fabric.dropped_flags = 1                 # host-side fault injection: the announcement is lost
    a.send(torch.ones(4), "fwd")
    with pytest.raises(PeerTimeout):
        b.recv(torch.empty(4), "fwd")


def _line(world, n_slots=2, slot_bytes=64):
    fabric = HostFabric(world, PeerMailbox.bytes_needed(slot_bytes, n_slots))
    boxes = [PeerMailbox(fabric.region(r), r - 1 if r > 0 else None, r + 1 if r + 1 < world else None, slot_bytes,
                         n_slots=n_slots) for r in range(world)]
    return fabric, boxes


def _try(fn, *args):
    """On the GPU a kernel that gave up does not stop the host: the next operation is still launched
    (and, under the abort record, releases its peer with a poisoned flag)."""
    try:
        fn(*args)
        return True
    except PeerTimeout:
        return False


def _forward(boxes, k, log=None):
    """One layer's handoff along the line: rank r receives from r - 1, then sends to r + 1."""
    world = len(boxes)
    for r in range(world):
        val, ok = float(k), True
        if r > 0:
            got = torch.zeros(3)
            ok = _try(boxes[r].recv, got, "fwd")
            val = float(got[0]) + 1.0
        if r + 1 < world:
            ok = _try(boxes[r].send, torch.full((3,), val), "fwd") and ok
        if log is not None and ok:
            log[r].append(val)


def _backward(boxes, k, log=None):
    world = len(boxes)
    for r in reversed(range(world)):
        val, ok = -float(k), True
        if r + 1 < world:
            got = torch.zeros(5)
            ok = _try(boxes[r].recv, got, "bwd")
            val = float(got[0]) - 1.0
        if r > 0:
            ok = _try(boxes[r].send, torch.full((5,), val), "bwd") and ok
        if log is not None and ok:
            log[r].append(val)


def test_four_rank_line_middle_ranks_both_directions_beyond_the_slot_count():
    """Ranks 1 and 2 have both neighbours: they receive and send in both directions, and with two
    slots and seven rounds every slot, flag and acknowledgement is reused several times."""
    fabric, boxes = _line(4, n_slots=2)
    for k in range(7):
        log = [[] for _ in range(4)]
        _forward(boxes, k, log)
        assert [v[0] for v in log] == [k, k + 1, k + 2, k + 3]
        log = [[] for _ in range(4)]
        _backward(boxes, k, log)
        assert [v[0] for v in log] == [-k - 3, -k - 2, -k - 1, -k]
    assert fabric.timeouts == 0
    for b in boxes:
        b.check()


def test_one_dropped_flag_takes_all_four_ranks_out_within_one_timeout():
    fabric, boxes = _line(4, n_slots=2)
    _forward(boxes, 0)
    _backward(boxes, 0)
    fabric.dropped_flags = 1                 # rank 0's next announcement to rank 1 is lost
    _forward(boxes, 1)                       # rank 1 times out; ranks 2 and 3 are released by poison
    assert fabric.timeouts == 1
    assert [a is not None for a in fabric.abort] == [False, True, True, True]
    _backward(boxes, 1)                      # rank 0 learns of it from rank 1's poisoned gradient flag
    assert fabric.timeouts == 1, "only the first wait may run its full time"
    assert all(a is not None for a in fabric.abort)
    assert "timed out" in fabric.abort[1] and "direction forward" in fabric.abort[1]
    assert "wanted 2" in fabric.abort[1] and "flag shows 0" in fabric.abort[1]     # slot 1 was never written
    for r in (0, 2, 3):
        assert "poisoned" in fabric.abort[r]
    for b in boxes:
        with pytest.raises(PeerTimeout):
            b.check()
    for b in boxes:
        b.reset()
    log = [[] for _ in range(4)]
    _forward(boxes, 5, log)
    assert [v[0] for v in log] == [5, 6, 7, 8]


def test_abort_record_is_readable():
    from megalodon_b200.parallel.symm import POISON, describe_abort
    msg = describe_abort([12, 2, 1, 133, 132, 5, 133, 0])
    assert "rank 5" in msg and "receive" in msg and "backward" in msg and "wanted 133" in msg and "132" in msg
    assert "poisoned" in describe_abort([13, 3, 2, 7, POISON - (1 << 32), 1, 7, 1])


def test_oversized_message_is_rejected():
    _, a, _ = _pair(slot_bytes=64)
    with pytest.raises(AssertionError):
        a.send(torch.zeros(1000), "fwd")


def test_region_rejects_bad_ranges():
    """Offsets handed to kernels are validated on the host (no GPU needed for the check itself)."""
    import pytest
    from megalodon_b200.parallel.symm import SymmetricRegion
    r = SymmetricRegion.__new__(SymmetricRegion)
    r.nbytes, r.world = 4096, 2
    r.check_range(0, 4096)
    r.check_range(4092, 4, rank=1)
    for bad in [dict(offset=-4), dict(offset=4096, nbytes=4), dict(offset=2, nbytes=4),
                dict(offset=0, nbytes=16, rank=2), dict(offset=8, nbytes=16, align=16)]:
        with pytest.raises(ValueError):
            r.check_range(**bad)
