"""The MoE layer with the reference's signature
(``fast_route/fast_route/layers/stable_route.py:10-102`` of the reference).
"""

from __future__ import annotations

import torch

from .. import _lib


def fused_moe(hidden_states: torch.Tensor, gate: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, topk: int,
              renormalize: bool = True, inplace: bool = False, return_routing: bool = False):
    """Mixture-of-Experts layer: route -> align -> grouped GEMM (+SiLU*mul) -> grouped GEMM
    (x routed weight) -> sum over the k experts of each token.

    ``hidden_states[M,H]`` fp16/bf16 contiguous, ``gate[H,E]`` (any strides; ``W_g[E,H].t()`` is
    the fast layout), ``w1[E,2I,H]`` (rows ``:I`` feed SiLU, rows ``I:`` multiply), ``w2[E,H,I]``.
    Returns ``[M,H]`` in the input dtype; with ``inplace`` the result is written into
    ``hidden_states`` as in the reference (``:97-102``).  One C call launches the whole
    sequence on the current stream with no host synchronisation.
    """
    assert hidden_states.shape[1] == w1.shape[2], "Incompatible dimensions"
    assert hidden_states.is_contiguous(), "Hidden_states must be contiguous"
    assert w1.is_contiguous(), "Expert weights1 must be contiguous"
    assert w2.is_contiguous(), "Expert weights2 must be contiguous"
    assert hidden_states.dtype in [torch.float16, torch.bfloat16]
    assert w1.dtype == hidden_states.dtype and w2.dtype == hidden_states.dtype and gate.dtype == hidden_states.dtype
    _lib.require_cuda(hidden_states, gate, w1, w2)
    M, H = hidden_states.shape
    E, N, _ = w1.shape
    I = N // 2
    assert w2.shape == (E, H, I) and gate.shape == (H, E)
    lib = _lib.load()
    dev = hidden_states.device
    out = hidden_states if inplace else torch.empty_like(hidden_states)
    tw = ti = None
    if return_routing:
        tw = torch.empty(M, topk, dtype=torch.float32, device=dev)
        ti = torch.empty(M, topk, dtype=torch.int32, device=dev)
    if M == 0:
        return (out, tw, ti) if return_routing else out
    nbytes = lib.fr_moe_workspace_bytes(M, H, I, E, topk)
    ws = _lib.workspace(nbytes, dev, "layer")
    rc = lib.fr_moe_layer(_lib.ptr(hidden_states), _lib.ptr(gate), gate.stride(0), gate.stride(1), _lib.ptr(w1),
                          _lib.ptr(w2), _lib.dtype_code(hidden_states.dtype), M, H, I, E, topk,
                          1 if renormalize else 0, _lib.ptr(out), _lib.ptr(tw), _lib.ptr(ti), _lib.ptr(ws),
                          ws.numel(), _lib.stream_ptr(dev))
    _lib.check(rc, "fr_moe_layer")
    return (out, tw, ti) if return_routing else out


def fused_experts(hidden_states: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, topk_weights: torch.Tensor,
                  topk_ids: torch.Tensor, inplace: bool = False) -> torch.Tensor:
    """The expert part of the layer for a routing computed elsewhere, with the argument order of the
    vLLM-style ``fused_moe(hidden_states, w1, w2, topk_weights, topk_ids, inplace)`` that the reference
    benchmarks against (``benchmarks/swizzle_moe/v0_moe_fused.py:219-224``).  ``topk_weights`` /
    ``topk_ids`` are ``[M, topk]`` of any float / integer dtype and any strides (they are compacted to
    fp32 / int32 here, which also removes the reference's strided-view pitfall)."""
    assert hidden_states.shape[1] == w1.shape[2], "Incompatible dimensions"
    assert hidden_states.is_contiguous() and w1.is_contiguous() and w2.is_contiguous()
    assert hidden_states.dtype in [torch.float16, torch.bfloat16]
    assert topk_weights.shape == topk_ids.shape
    _lib.require_cuda(hidden_states, w1, w2, topk_weights, topk_ids)
    M, H = hidden_states.shape
    E, N, _ = w1.shape
    I = N // 2
    topk = topk_ids.shape[1]
    tw = topk_weights.to(torch.float32).contiguous()
    ti = topk_ids.to(torch.int32).contiguous()
    out = hidden_states if inplace else torch.empty_like(hidden_states)
    if M == 0:
        return out
    lib = _lib.load()
    dev = hidden_states.device
    ws = _lib.workspace(lib.fr_moe_workspace_bytes(M, H, I, E, topk), dev, "layer")
    rc = lib.fr_moe_layer_routed(_lib.ptr(hidden_states), _lib.ptr(ti), _lib.ptr(tw), _lib.ptr(w1), _lib.ptr(w2),
                                 _lib.dtype_code(hidden_states.dtype), M, H, I, E, topk, _lib.ptr(out), _lib.ptr(ws),
                                 ws.numel(), _lib.stream_ptr(dev))
    _lib.check(rc, "fr_moe_layer_routed")
    return out
