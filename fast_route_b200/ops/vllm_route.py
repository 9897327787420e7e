"""The routing op of the reference's baseline layer: softmax over all experts, then top-k.

``topk_softmax`` has the argument order of ``vllm._moe_C.topk_softmax`` as the reference calls it
(``fast_route/fast_route/layers/vllm_route.py:79-84``): three caller-allocated ``[M, topk]`` outputs
and the fp32 (or fp16 / bf16) gating output ``[M, E]``.
"""

from __future__ import annotations

import torch

from .. import _lib


def topk_softmax(topk_weights: torch.Tensor, topk_ids: torch.Tensor, token_expert_indicies: torch.Tensor,
                 gating_output: torch.Tensor, renormalize: bool = False) -> None:
    """Fills ``topk_weights`` (fp32 softmax probabilities of the selected experts), ``topk_ids``
    (int32, equal probabilities go to the lower expert id) and ``token_expert_indicies``
    (int32, entry ``[t, j] = j*M + t``; may be ``None``).  ``renormalize`` folds the division by the
    sum of the k probabilities (``layers/vllm_route.py:83-84``) into the same kernel."""
    _lib.require_cuda(topk_weights, topk_ids, gating_output)
    M, E = gating_output.shape
    topk = topk_weights.shape[1]
    assert topk_weights.shape == (M, topk) and topk_ids.shape == (M, topk)
    assert topk_weights.dtype == torch.float32 and topk_ids.dtype == torch.int32
    assert topk_weights.stride(1) == 1 and topk_ids.stride(1) == 1
    assert 0 < topk <= E
    src_stride = 0
    if token_expert_indicies is not None:
        assert token_expert_indicies.shape == (M, topk) and token_expert_indicies.dtype == torch.int32
        assert token_expert_indicies.is_cuda and token_expert_indicies.stride(1) == 1
        src_stride = token_expert_indicies.stride(0)
    rc = _lib.load().fr_softmax_topk(_lib.ptr(gating_output), _lib.dtype_code(gating_output.dtype), M, E,
                                     gating_output.stride(0), gating_output.stride(1), topk,
                                     1 if renormalize else 0, _lib.ptr(topk_weights), topk_weights.stride(0),
                                     _lib.ptr(topk_ids), topk_ids.stride(0), _lib.ptr(token_expert_indicies),
                                     src_stride, _lib.stream_ptr(gating_output.device))
    _lib.check(rc, "fr_softmax_topk")


__all__ = ["topk_softmax"]
