from .optimizer import rescale_grads, build_optimizer, FusedAdamW
from .lr_scheduler import build_lr_scheduler, build_lr_fn
