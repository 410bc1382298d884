from .layers import ColumnParallelLinear, RowParallelLinear, ParallelEmbedding
from .mappings import (
    copy_to_model_parallel_region,
    gather_from_model_parallel_region,
    reduce_from_model_parallel_region,
    scatter_to_model_parallel_region,
    gather_copy_model_parallel_region,
    reduce_scatter_model_parallel_region,
)
