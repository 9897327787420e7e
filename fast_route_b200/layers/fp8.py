"""The MoE layer with 8-bit floating-point (E4M3) expert weights.

``quantize_experts_fp8`` turns ``w1[E,2I,H]`` / ``w2[E,H,I]`` into E4M3 bytes plus one fp32 scale per
weight row; ``fused_moe_fp8`` runs the layer on them.  Activations stay fp16/bf16 at the interface and are
quantised row by row inside the layer.  The reference does not have this mode (it only carries
commented-out fp8 autotune entries, ``fast_route/fast_route/ops/stable_route.py:20-28``).
"""

from __future__ import annotations

import torch

from .. import _lib

E4M3_MAX = 448.0


def quantize_rows_e4m3(t: torch.Tensor):
    """Per-row symmetric quantisation: returns (bytes as float8_e4m3fn, fp32 scale per row) with
    ``t ~= q.float() * scale[..., None]``."""
    amax = t.abs().amax(dim=-1, keepdim=True).float()
    scale = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    q = (t.float() / scale).to(torch.float8_e4m3fn)
    return q, scale.squeeze(-1).contiguous()


def quantize_experts_fp8(w1: torch.Tensor, w2: torch.Tensor):
    """``(w1_q, w1_scale[E,2I], w2_q, w2_scale[E,H])`` for ``fused_moe_fp8`` (one expert at a time, so
    no fp32 copy of all experts is ever alive)."""
    def one(w):
        q = torch.empty(w.shape, dtype=torch.float8_e4m3fn, device=w.device)
        s = torch.empty(w.shape[:2], dtype=torch.float32, device=w.device)
        for e in range(w.shape[0]):
            q[e], s[e] = quantize_rows_e4m3(w[e])
        return q, s
    w1_q, s1 = one(w1)
    w2_q, s2 = one(w2)
    return w1_q, s1, w2_q, s2


def fused_moe_fp8(hidden_states: torch.Tensor, gate: torch.Tensor, w1_q: torch.Tensor, w1_scale: torch.Tensor,
                  w2_q: torch.Tensor, w2_scale: torch.Tensor, topk: int, renormalize: bool = True,
                  inplace: bool = False, return_routing: bool = False):
    """Same contract as ``fused_moe`` with quantised expert weights."""
    assert hidden_states.is_contiguous() and hidden_states.dtype in (torch.float16, torch.bfloat16)
    assert w1_q.dtype == torch.float8_e4m3fn and w2_q.dtype == torch.float8_e4m3fn
    assert w1_q.is_contiguous() and w2_q.is_contiguous()
    _lib.require_cuda(hidden_states, gate, w1_q, w2_q, w1_scale, w2_scale)
    M, H = hidden_states.shape
    E, N, _ = w1_q.shape
    I = N // 2
    assert w1_q.shape == (E, 2 * I, H) and w2_q.shape == (E, H, I) and gate.shape == (H, E)
    assert w1_scale.shape == (E, 2 * I) and w2_scale.shape == (E, H)
    assert w1_scale.dtype == torch.float32 and w2_scale.dtype == torch.float32
    assert w1_scale.is_contiguous() and w2_scale.is_contiguous()
    lib = _lib.load()
    dev = hidden_states.device
    out = hidden_states if inplace else torch.empty_like(hidden_states)
    tw = ti = None
    if return_routing:
        tw = torch.empty(M, topk, dtype=torch.float32, device=dev)
        ti = torch.empty(M, topk, dtype=torch.int32, device=dev)
    if M == 0:
        return (out, tw, ti) if return_routing else out
    ws = _lib.workspace(lib.fr_moe_fp8_workspace_bytes(M, H, I, E, topk), dev, "layer")
    rc = lib.fr_moe_layer_fp8(_lib.ptr(hidden_states), _lib.ptr(gate), gate.stride(0), gate.stride(1), _lib.ptr(w1_q),
                              _lib.ptr(w1_scale), _lib.ptr(w2_q), _lib.ptr(w2_scale),
                              _lib.dtype_code(hidden_states.dtype), M, H, I, E, topk, 1 if renormalize else 0,
                              _lib.ptr(out), _lib.ptr(tw), _lib.ptr(ti), _lib.ptr(ws), ws.numel(), _lib.stream_ptr(dev))
    _lib.check(rc, "fr_moe_layer_fp8")
    return (out, tw, ti) if return_routing else out
