from .mappings import (
    send_to_next_chunk_parallel_region,
    recv_from_prev_chunk_parallel_region,
    gather_from_chunk_parallel_region,
    should_send_to_next,
    should_recv_from_prev,
    attach_to_graph,
    set_handoff_transport,
    get_handoff_transport,
    HandoffTape,
    use_tape,
    current_tape,
)
