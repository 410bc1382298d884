"""Alias of `megalodon_b200.parallel` under the reference's package name
(`megalodon.distributed`)."""
from ..parallel import *  # noqa: F401,F403
from ..parallel import initialize, setup, utils, fsdp  # noqa: F401
