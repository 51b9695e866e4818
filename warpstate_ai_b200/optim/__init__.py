from .adamw import ArenaAdamW, cosine_lr
from .arena import ParamArena

__all__ = ["ArenaAdamW", "ParamArena", "cosine_lr"]
