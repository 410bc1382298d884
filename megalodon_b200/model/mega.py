from ..models.mega import *  # noqa: F401,F403
from ..models.mega import Mega, MegaBlock, MegaOutputLayer, build_model, ModelStore  # noqa: F401
