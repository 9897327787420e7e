"""Router operators with the reference's signatures.

``fused_route`` mirrors ``fast_route/fast_route/ops/stable_route.py:123-178`` of the
reference: same arguments, same return (first-k columns of the caller's buffers), same
assertions.  Underneath, one tcgen05 gate-GEMM kernel computes the logits and selects the
stable top-k / softmax in its epilogue.
"""

from __future__ import annotations

import torch

from .. import _lib


def _route_compact(hidden_state, gate, topk, renormalize, want_logits=False):
    M, K = hidden_state.shape
    Kg, E = gate.shape
    assert K == Kg, "Incompatible dimensions"
    lib = _lib.load()
    dev = hidden_state.device
    w = torch.empty(M, topk, dtype=torch.float32, device=dev)
    ids = torch.empty(M, topk, dtype=torch.int32, device=dev)
    logits = torch.empty(M, E, dtype=torch.float32, device=dev) if want_logits else None
    nbytes = lib.fr_route_fused_workspace_bytes(M, K, E, topk)
    ws = _lib.workspace(nbytes, dev, "route")
    rc = lib.fr_route_fused(_lib.ptr(hidden_state), _lib.dtype_code(hidden_state.dtype), M, K,
                            hidden_state.stride(0), _lib.ptr(gate), gate.stride(0), gate.stride(1), E, topk,
                            1 if renormalize else 0, _lib.ptr(w), _lib.ptr(ids), _lib.ptr(logits), _lib.ptr(ws),
                            ws.numel(), _lib.stream_ptr(dev))
    _lib.check(rc, "fr_route_fused")
    return w, ids, logits


def fused_route(hidden_state: torch.Tensor, gate: torch.Tensor, topk: int, topk_weights: torch.Tensor = None,
                topk_ids: torch.Tensor = None, renormalize=True, return_logits: bool = False):
    """``hidden_state[M,K]``, ``gate[K,E]`` -> (weights[:, :topk], ids[:, :topk]).

    ``topk_weights`` / ``topk_ids`` are the caller's ``[M,E]`` buffers as in the reference
    (any float / integer dtype); the first ``topk`` columns receive the result, the remaining
    columns what the reference leaves there (the rest of the stable argsort / zeros), and the
    returned tensors are views of the first ``topk`` columns.  Passing ``None`` returns fresh compact
    contiguous ``[M,topk]`` fp32 / int32 tensors, the layout the expert kernels take.
    The reference only supports ``renormalize=True`` (``ops/stable_route.py:130``);
    ``False`` divides by the softmax denominator over all experts instead.
    """
    _lib.require_cuda(hidden_state, gate)
    assert hidden_state.dim() == 2 and gate.dim() == 2
    M, K = hidden_state.shape
    _, N = gate.shape
    assert N <= 256, f"{N} number of experts should be small enough for one MMA tile"
    assert 0 < topk <= N
    assert hidden_state.dtype in (torch.float16, torch.bfloat16) and gate.dtype == hidden_state.dtype
    assert hidden_state.stride(1) == 1, "hidden_state rows must be contiguous"
    if topk_weights is None:
        w, ids, logits = _route_compact(hidden_state, gate, topk, renormalize, return_logits)
        return (w, ids, logits) if return_logits else (w, ids)
    # The reference's kernel stores all E columns of the caller's buffers (ops/stable_route.py:110-121): the ids
    # of the complete stable descending argsort and zeros after the first k weights.  Same here: the gate GEMM
    # leaves its fp32 logits, the ranking kernel fills the full width from them.
    assert topk_ids is not None and topk_weights.shape == (M, N) and topk_ids.shape == (M, N)
    _, _, logits = _route_compact(hidden_state, gate, topk, renormalize, True)
    direct = (topk_weights.dtype == torch.float32 and topk_ids.dtype == torch.int32 and
              topk_weights.stride(1) == 1 and topk_ids.stride(1) == 1)
    if direct:
        route_from_logits(logits, topk, renormalize, fill_rest=True, topk_weights=topk_weights, topk_ids=topk_ids)
    else:
        fw, fi = route_from_logits(logits, topk, renormalize, fill_rest=True)
        topk_weights.copy_(fw)
        topk_ids.copy_(fi)
    w, ids = topk_weights[:, :topk], topk_ids[:, :topk]
    return (w, ids, logits) if return_logits else (w, ids)


def route_from_logits(logits: torch.Tensor, topk: int, renormalize: bool = True, fill_rest: bool = False,
                      topk_weights: torch.Tensor = None, topk_ids: torch.Tensor = None):
    """Stable top-k + softmax over the selected k from router logits ``[M,E]`` (fp16, bf16, fp32).

    ``fill_rest=True`` returns ``[M,E]`` tensors holding what the reference's kernel leaves in
    its full-width buffers (``ops/stable_route.py:110-121``): the complete stable descending
    argsort, and zeros after the first k weights.
    """
    _lib.require_cuda(logits)
    M, E = logits.shape
    assert 0 < topk <= E
    cols = E if fill_rest else topk
    dev = logits.device
    if topk_weights is None:
        topk_weights = torch.empty(M, cols, dtype=torch.float32, device=dev)
        topk_ids = torch.empty(M, cols, dtype=torch.int32, device=dev)
    assert topk_weights.dtype == torch.float32 and topk_ids.dtype == torch.int32
    assert topk_weights.stride(1) == 1 and topk_ids.stride(1) == 1
    rc = _lib.load().fr_topk_softmax(_lib.ptr(logits), _lib.dtype_code(logits.dtype), M, E, logits.stride(0),
                                     logits.stride(1), topk, 1 if renormalize else 0, _lib.ptr(topk_weights),
                                     topk_weights.stride(0), _lib.ptr(topk_ids), topk_ids.stride(0),
                                     1 if fill_rest else 0, _lib.stream_ptr(dev))
    _lib.check(rc, "fr_topk_softmax")
    return topk_weights, topk_ids
