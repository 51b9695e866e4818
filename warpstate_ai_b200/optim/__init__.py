from .adamw import ArenaAdamW, cosine_lr, linear_warmup_decay_lr, warmup_ratio_cosine_lr
from .arena import ParamArena

__all__ = ["ArenaAdamW", "ParamArena", "cosine_lr", "linear_warmup_decay_lr", "warmup_ratio_cosine_lr"]
