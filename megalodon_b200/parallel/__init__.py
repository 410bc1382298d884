"""Parallel runtime: process-group topology, bootstrap, FSDP, tensor- and
chunk-parallel layers.  The public names are those of the reference's
`megalodon.distributed` package (distributed/__init__.py:1-21) plus this
framework's FSDP / checkpointing entry points; each is imported from its
sub-module on first use."""
import importlib

_EXPORTS = {
    "initialize": (
        "initialize_model_parallel destroy_model_parallel model_parallel_is_initialized "
        "get_model_parallel_group get_model_parallel_world_size get_model_parallel_rank "
        "get_model_parallel_ranks get_model_parallel_src_rank "
        "get_data_parallel_group get_data_parallel_world_size get_data_parallel_rank get_data_parallel_ranks "
        "get_chunk_parallel_group get_chunk_parallel_world_size get_chunk_parallel_rank get_chunk_parallel_ranks "
        "get_chunk_parallel_next_rank get_chunk_parallel_prev_rank"
    ),
    "fsdp": "FullyShardedDataParallel TrainingState enable_wrap wrap calc_grad_norm",
    "checkpoint": "checkpoint_wrapper CheckpointWrapper",
    "setup": "init_torch_distributed init_signal_handler DistInfo",
}
_WHERE = {name: mod for mod, names in _EXPORTS.items() for name in names.split()}
__all__ = sorted(_WHERE)


def __getattr__(name):
    if name in _WHERE:
        value = getattr(importlib.import_module(f"{__name__}.{_WHERE[name]}"), name)
        globals()[name] = value
        return value
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


def __dir__():
    return sorted(list(globals()) + __all__)
