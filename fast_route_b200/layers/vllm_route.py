"""The reference's baseline layer (routing as in vLLM: softmax over all experts, then top-k) with
the same signature as ``fast_route/fast_route/layers/vllm_route.py:17-25``."""

from __future__ import annotations

import torch

from .. import _lib
from ..ops.stable_route import fused_route
from ..ops.vllm_route import topk_softmax
from .stable_route import fused_experts


def fused_moe(hidden_states: torch.Tensor, gate: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, topk: int,
              renormalize: bool = True, inplace: bool = False) -> torch.Tensor:
    """``gating_output = hidden_states @ gate`` rounded to the input dtype as a matmul would
    (``layers/vllm_route.py:78``), softmax over all E experts in fp32, top-k on the probabilities,
    optional renormalisation, then the expert GEMMs of the fused layer.  The logits come from this
    library's own tensor-core gate kernel (fp32 accumulation)."""
    assert hidden_states.shape[1] == w1.shape[2], "Incompatible dimensions"
    assert hidden_states.is_contiguous(), "Hidden_states must be contiguous"
    assert w1.is_contiguous(), "Expert weights1 must be contiguous"
    assert w2.is_contiguous(), "Expert weights2 must be contiguous"
    assert hidden_states.dtype in [torch.float16, torch.bfloat16]
    _lib.require_cuda(hidden_states, gate, w1, w2)
    M, _ = hidden_states.shape
    dev = hidden_states.device
    if M == 0:
        return hidden_states if inplace else torch.empty_like(hidden_states)
    _, _, logits = fused_route(hidden_states, gate, topk, return_logits=True)
    gating_output = logits.to(hidden_states.dtype)
    topk_weights = torch.empty(M, topk, dtype=torch.float32, device=dev)
    topk_ids = torch.empty(M, topk, dtype=torch.int32, device=dev)
    topk_softmax(topk_weights, topk_ids, None, gating_output, renormalize=renormalize)
    return fused_experts(hidden_states, w1, w2, topk_weights, topk_ids, inplace=inplace)


__all__ = ["fused_moe"]
