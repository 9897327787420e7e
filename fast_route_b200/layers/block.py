"""Transformer-block glue around the MoE layer.

The reference's transformer-layer benchmark computes ``h = attn(x) + x`` and feeds ``h`` to its MoE
layer (``benchmarks/fused_route/transformerLayer_bench.py:66-79``); a Mixtral block additionally
normalises ``h`` (RMSNorm) before the experts and adds ``h`` back afterwards.  ``moe_block`` runs
all of that as one C call: the residual add and the norm are one kernel, the trailing residual is
added inside the combine kernel.
"""

from __future__ import annotations

import torch

from .. import _lib


def add_rmsnorm(a: torch.Tensor, b: torch.Tensor = None, gamma: torch.Tensor = None, eps: float = 1e-5,
                want_h: bool = True):
    """``h = a (+ b)``; ``x = h * rsqrt(mean(h^2) + eps) * gamma``.  Returns ``(h, x)``
    (``h`` is None when not requested, ``x`` is ``h`` when there is no ``gamma``)."""
    _lib.require_cuda(a, b, gamma)
    assert a.dim() == 2 and a.is_contiguous() and a.dtype in (torch.float16, torch.bfloat16)
    M, H = a.shape
    h = torch.empty_like(a) if (want_h or gamma is None) else None
    x = torch.empty_like(a) if gamma is not None else None
    rc = _lib.load().fr_add_rmsnorm(_lib.ptr(a), H, _lib.ptr(b), H, _lib.ptr(gamma), float(eps),
                                    _lib.dtype_code(a.dtype), M, H, _lib.ptr(h), H, _lib.ptr(x), H,
                                    _lib.stream_ptr(a.device))
    _lib.check(rc, "fr_add_rmsnorm")
    return h, (x if gamma is not None else h)


def moe_block(attn_out: torch.Tensor, x: torch.Tensor, gate: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor,
              topk: int, gamma: torch.Tensor = None, eps: float = 1e-5, add_residual: bool = False,
              renormalize: bool = True, out: torch.Tensor = None) -> torch.Tensor:
    """``h = attn_out (+ x)``; ``u = rmsnorm(h) * gamma`` if ``gamma`` is given else ``h``;
    returns ``(h if add_residual else 0) + fused_moe(u)``.

    With ``x`` given, ``gamma=None`` and ``add_residual=False`` this is the reference's block.
    ``out`` may alias ``attn_out`` or ``x``.
    """
    assert attn_out.is_contiguous() and attn_out.dtype in (torch.float16, torch.bfloat16)
    assert x is None or (x.shape == attn_out.shape and x.dtype == attn_out.dtype and x.is_contiguous())
    assert w1.is_contiguous() and w2.is_contiguous()
    _lib.require_cuda(attn_out, x, gate, w1, w2, gamma)
    M, H = attn_out.shape
    E, N, _ = w1.shape
    I = N // 2
    assert gate.shape == (H, E) and w2.shape == (E, H, I)
    assert gamma is None or (gamma.shape == (H,) and gamma.dtype == attn_out.dtype and gamma.is_contiguous())
    if out is None:
        out = torch.empty_like(attn_out)
    if M == 0:
        return out
    lib = _lib.load()
    dev = attn_out.device
    ws = _lib.workspace(lib.fr_moe_block_workspace_bytes(M, H, I, E, topk), dev, "layer")
    rc = lib.fr_moe_block(_lib.ptr(attn_out), _lib.ptr(x), _lib.ptr(gamma), float(eps), _lib.ptr(gate), gate.stride(0),
                          gate.stride(1), _lib.ptr(w1), _lib.ptr(w2), _lib.dtype_code(attn_out.dtype), M, H, I, E, topk,
                          1 if renormalize else 0, 1 if add_residual else 0, _lib.ptr(out), _lib.ptr(ws), ws.numel(),
                          _lib.stream_ptr(dev))
    _lib.check(rc, "fr_moe_block")
    return out
