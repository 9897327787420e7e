"""CPU oracle for the MoE layer (test infrastructure only; CPU torch, fp32).

Restates the reference's naive layer ``torch_moe``
(``benchmarks/swizzle_moe/perf_test_moe.py:17-31``) with the activation of
``benchmarks/swizzle_moe/activation.py:27-30``:  every (token, slot) assignment
is pushed through its expert ``w2[e] . (silu(w1[e][:I] x) * (w1[e][I:] x))`` and
the k results of a token are summed with the routing weights.  The stacked
``w1[E, 2I, H]`` keeps the SiLU branch in rows ``0..I-1`` and the linear branch
in rows ``I..2I-1``; ``w2`` is ``[E, H, I]``.
"""

from __future__ import annotations

import numpy as np
import torch
import torch.nn.functional as F

from . import route as _route


def silu_and_mul(x: torch.Tensor) -> torch.Tensor:
    """``silu(x[..., :d]) * x[..., d:]`` (``activation.py:27-30``)."""
    d = x.shape[-1] // 2
    return F.silu(x[..., :d]) * x[..., d:]


def torch_moe(a: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor,
              topk_weight: torch.Tensor, topk_ids: torch.Tensor) -> torch.Tensor:
    """Layer output given the routing; all math in the dtype of ``a`` (use fp32).

    Follows ``perf_test_moe.py:17-31`` step by step: replicate each token k
    times, run each expert on the rows routed to it, weight and sum.
    """
    M, H = a.shape
    k = topk_ids.shape[1]
    rep = a.view(M, 1, H).expand(M, k, H).reshape(-1, H)
    out = torch.zeros(M * k, w2.shape[1], dtype=a.dtype)
    flat_ids = topk_ids.reshape(-1)
    for e in range(w1.shape[0]):
        rows = (flat_ids == e).nonzero().flatten()
        if rows.numel():
            h = silu_and_mul(rep[rows] @ w1[e].t())
            out[rows] = h @ w2[e].t()
    return (out.view(M, k, -1) * topk_weight.reshape(M, k, 1).to(a.dtype)).sum(dim=1)


def moe_layer(x: torch.Tensor, gate: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor,
              topk: int, renormalize: bool = True, routing=None):
    """Whole layer in fp32 on the given (already rounded) inputs.

    ``gate`` is ``[H, E]`` as in ``layers/stable_route.py:10-18``.  If ``routing``
    = (weights, ids) is given it replaces the oracle router, so that a device
    path can be compared on identical assignments.  Returns (out, weights, ids).
    """
    xf, w1f, w2f = x.float().cpu(), w1.float().cpu(), w2.float().cpu()
    if routing is None:
        w, ids, _ = _route.route_from_hidden(x, gate, topk, renormalize)
    else:
        w, ids = routing
        w = w.detach().cpu().numpy() if hasattr(w, "detach") else np.asarray(w)
        ids = ids.detach().cpu().numpy() if hasattr(ids, "detach") else np.asarray(ids)
    wt = torch.from_numpy(np.ascontiguousarray(w, dtype=np.float32))
    it = torch.from_numpy(np.ascontiguousarray(ids).astype(np.int64))
    out = torch_moe(xf, w1f, w2f, wt, it)
    return out, w, ids
