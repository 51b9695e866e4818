"""Drop-in `warpstate` package: the reference's public import surface
(``from warpstate import WarpStateConfig, WarpStateLM``) served by warpstate_ai_b200."""
from .config import WarpStateConfig
from .model import WarpStateLM

__all__ = ["WarpStateConfig", "WarpStateLM"]
