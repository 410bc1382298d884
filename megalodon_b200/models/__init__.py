from .mega import Mega, MegaBlock, MegaOutputLayer, build_model, ModelStore
