from ..parallel.utils import *  # noqa: F401,F403
from ..parallel.utils import (  # noqa: F401
    ensure_divisibility, divide_and_check_no_remainder, split_tensor_along_specific_dim,
    reduce_scalar, ReduceOpMap, comm_device,
)
