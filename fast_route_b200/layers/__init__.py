from .stable_route import fused_moe, fused_experts
from .host import fused_moe_host

__all__ = ["fused_moe", "fused_experts", "fused_moe_host"]
