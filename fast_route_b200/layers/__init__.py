from .stable_route import fused_moe, fused_experts
from .host import fused_moe_host, fused_moe_host_wait
from .block import moe_block, add_rmsnorm
from .fp8 import fused_moe_fp8, quantize_experts_fp8

__all__ = ["fused_moe", "fused_experts", "fused_moe_host", "fused_moe_host_wait", "moe_block", "add_rmsnorm", "fused_moe_fp8",
           "quantize_experts_fp8"]
