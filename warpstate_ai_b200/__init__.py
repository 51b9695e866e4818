"""WarpState-B200: a Blackwell-native training and inference framework for the WarpState LM."""
from .config import WarpStateConfig, warpstate_2b, warpstate_smoke
from .models.warpstate import WarpStateLM

__all__ = ["WarpStateConfig", "WarpStateLM", "warpstate_2b", "warpstate_smoke"]
__version__ = "0.1.0"
