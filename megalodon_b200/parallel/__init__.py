"""Parallel runtime: process-group topology, bootstrap, FSDP, tensor- and
chunk-parallel layers.  Exposes the reference's `megalodon.distributed` API
(distributed/__init__.py:1-21)."""
from .initialize import (
    initialize_model_parallel,
    destroy_model_parallel,
    get_chunk_parallel_group,
    get_chunk_parallel_world_size,
    get_chunk_parallel_rank,
    get_chunk_parallel_ranks,
    get_chunk_parallel_next_rank,
    get_chunk_parallel_prev_rank,
    get_data_parallel_group,
    get_data_parallel_world_size,
    get_data_parallel_rank,
    get_data_parallel_ranks,
    get_model_parallel_group,
    get_model_parallel_rank,
    get_model_parallel_ranks,
    get_model_parallel_src_rank,
    get_model_parallel_world_size,
    model_parallel_is_initialized,
)
from .fsdp import FullyShardedDataParallel, TrainingState, enable_wrap, wrap, calc_grad_norm
from .checkpoint import checkpoint_wrapper, CheckpointWrapper
from .setup import init_torch_distributed, init_signal_handler, DistInfo
