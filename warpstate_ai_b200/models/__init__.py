from .warpstate import (LayerCache, RMSNorm, SwiGLU, WarpStateCore, WarpStateLM, apply_rope,
                        rope_cos_sin, rotate_half)

__all__ = ["LayerCache", "RMSNorm", "SwiGLU", "WarpStateCore", "WarpStateLM", "apply_rope",
           "rope_cos_sin", "rotate_half"]
