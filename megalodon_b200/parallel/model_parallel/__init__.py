"""Tensor-parallel layers and the autograd mappings between replicated and feature-sharded
activations (reference: modules/model_parallel/__init__.py)."""
import importlib

_WHERE = {}
for _mod, _names in {
    "layers": "ColumnParallelLinear RowParallelLinear ParallelEmbedding",
    "mappings": ("copy_to_model_parallel_region reduce_from_model_parallel_region "
                 "scatter_to_model_parallel_region gather_from_model_parallel_region "
                 "gather_copy_model_parallel_region reduce_scatter_model_parallel_region"),
}.items():
    for _n in _names.split():
        _WHERE[_n] = _mod
__all__ = sorted(_WHERE)


def __getattr__(name):
    if name in _WHERE:
        value = getattr(importlib.import_module(f"{__name__}.{_WHERE[name]}"), name)
        globals()[name] = value
        return value
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
