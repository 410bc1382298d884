from ..parallel.initialize import *  # noqa: F401,F403
