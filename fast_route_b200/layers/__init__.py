from .stable_route import fused_moe

__all__ = ["fused_moe"]
