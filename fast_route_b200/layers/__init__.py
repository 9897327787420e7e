from .stable_route import fused_moe
from .host import fused_moe_host

__all__ = ["fused_moe", "fused_moe_host"]
