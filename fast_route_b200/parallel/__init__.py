from .ep import ExpertParallelGroup, fused_moe_ep, fused_moe_ep_p2p, fused_moe_ep_host

__all__ = ["ExpertParallelGroup", "fused_moe_ep", "fused_moe_ep_p2p", "fused_moe_ep_host"]
