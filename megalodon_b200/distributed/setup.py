from ..parallel.setup import *  # noqa: F401,F403
from ..parallel.setup import (  # noqa: F401
    get_global_rank, get_local_rank, get_world_size, is_master, is_slurm_job, is_torch_run,
    get_master_addr, get_master_port, init_torch_distributed, init_signal_handler,
    init_distributed_process_group,
)
