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


def test_receive_without_send_times_out_and_can_be_retried():
    _, a, b = _pair()
    out = torch.empty(4)
    with pytest.raises(PeerTimeout):
        b.recv(out, "fwd")
    a.send(torch.arange(4.0), "fwd")         # the late message is still delivered
    b.recv(out, "fwd")
    assert torch.equal(out, torch.arange(4.0))


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
