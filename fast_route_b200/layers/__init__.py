from .stable_route import fused_moe, fused_experts
from .host import fused_moe_host
from .block import moe_block, add_rmsnorm

__all__ = ["fused_moe", "fused_experts", "fused_moe_host", "moe_block", "add_rmsnorm"]
