"""megalodon_b200: a Blackwell-native (sm_100a) Megalodon training and
inference framework."""
import os as _os

# Kernels of this package wait on flags that another rank's kernels write (the
# peer mailbox, the flag barriers of the symmetric collectives).  With CUDA's
# default lazy module loading, the first launch of any not-yet-loaded kernel may
# have to wait for running kernels to drain; if the running kernel is one of
# those waits, and the peer it waits for is in turn waiting for the kernel being
# loaded, both ranks stall until the bounded waits give up.  Loading every
# kernel when its module is registered removes that dependency.  The variable
# is read when CUDA initialises, so it is set at import time, before the first
# CUDA call; an explicit setting by the user is left alone.
_os.environ.setdefault("CUDA_MODULE_LOADING", "EAGER")
# For the same reason no two streams of this package may share a hardware work queue: work queued
# behind a waiting kernel of ANOTHER stream in the same queue cannot start, although nothing orders
# the two.  The default of 8 queues is fewer than the streams in use (compute, parameter gather,
# gradient reduction, one internal stream per NCCL communicator); 32 gives each its own.  Also read
# when CUDA initialises.
_os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "32")
# The kernels of this package reach peer memory with plain loads and stores only (no `multimem`), so the
# symmetric-memory allocator is asked not to bind its buffers to an NVLink multicast object: a rank that
# leaves (a failed step, the benchmark's restart on another transport) while its memory is bound to one
# can raise NVLink faults on the GPUs of the ranks that stay.
_os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")

__version__ = "0.1.0"
