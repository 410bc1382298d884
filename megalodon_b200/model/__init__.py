"""Alias of `megalodon_b200.models` under the reference's package name."""
from ..models import *  # noqa: F401,F403
