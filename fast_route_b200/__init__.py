"""fast_route_b200: the fused-routing Mixture-of-Experts layer of hgl71964/fast-route,
rebuilt for NVIDIA B200 (sm_100a) as hand-written CUDA behind a C ABI.

``ops`` and ``layers`` mirror the reference's ``fast_route.ops`` / ``fast_route.layers``
operator surface; ``parallel`` adds expert parallelism over NCCL.
"""

from . import _lib
from .layers.stable_route import fused_moe, fused_experts
from .layers.host import fused_moe_host, fused_moe_host_wait
from .layers.block import moe_block, add_rmsnorm
from .layers.fp8 import fused_moe_fp8, quantize_experts_fp8
from .ops.stable_route import fused_route, route_from_logits
from .ops.fused_moe import moe_align_block_size, invoke_fused_moe_kernel

__all__ = ["fused_moe", "fused_experts", "fused_moe_host", "fused_moe_host_wait", "moe_block", "add_rmsnorm", "fused_moe_fp8", "quantize_experts_fp8", "fused_route", "route_from_logits", "moe_align_block_size",
           "invoke_fused_moe_kernel", "_lib"]
