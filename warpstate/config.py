from warpstate_ai_b200.config import WarpStateConfig

__all__ = ["WarpStateConfig"]
