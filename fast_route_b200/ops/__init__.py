from .stable_route import fused_route, route_from_logits
from .vllm_route import topk_softmax
from .fused_moe import moe_align_block_size, invoke_fused_moe_kernel, gemm1_silu, gemm2, permute_rows, combine

__all__ = ["fused_route", "route_from_logits", "topk_softmax", "moe_align_block_size", "invoke_fused_moe_kernel",
           "gemm1_silu", "gemm2", "permute_rows", "combine"]
