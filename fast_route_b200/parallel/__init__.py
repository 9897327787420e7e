from .ep import ExpertParallelGroup, fused_moe_ep

__all__ = ["ExpertParallelGroup", "fused_moe_ep"]
