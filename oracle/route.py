"""CPU oracle for the router (test infrastructure, never imported by the product).

Restates ``route_kernel`` of the reference
(``fast_route/fast_route/ops/stable_route.py:32-121``):

* logits = X . G accumulated in fp32 (``:66-80``);
* stable descending argsort over all E columns, equal values ordered by the
  lower expert id (``:97-98``; tie rule ``ops/stable_argsort.py:37-50``, asserted
  bit-exact against ``torch.sort(stable=True)`` by the reference's
  ``tests/test_argsort.py:134-145``);
* softmax over the first ``topk`` sorted logits only (``:101-107``), which equals
  softmax-over-E followed by renormalisation of the selected k.

The softmax weights follow a fixed recipe made only of single IEEE-754 fp32
operations (no fused multiply-add, no library ``exp``) so that a GPU kernel can
reproduce every bit:  e_j = exp_recipe(l_j - l_0),  s = ((e_0 + e_1) + e_2) ...,
w_j = e_j / s.
"""

from __future__ import annotations

import numpy as np

_F = np.float32
_LOG2E = _F(1.4426950408889634)
_LN2_HI = _F(0.693359375)            # 355/512, few mantissa bits: n*LN2_HI is exact
_LN2_LO = _F(-2.12194440e-4)         # ln(2) - LN2_HI
_EXP_CLAMP = _F(-87.0)
# coefficients are fp32 quotients (1.0f / 5040.0f ...), the way a C compiler folds them
_C = [_F(1.0) / _F(5040.0), _F(1.0) / _F(720.0), _F(1.0) / _F(120.0), _F(1.0) / _F(24.0),
      _F(1.0) / _F(6.0), _F(0.5), _F(1.0), _F(1.0)]


def exp_recipe(x: np.ndarray) -> np.ndarray:
    """exp(x) for x <= 0 in fp32 from mul/add/sub/rint only (each rounded once).

    n = rint(x*log2e); r = (x - n*LN2_HI) - n*LN2_LO; degree-7 Horner polynomial
    evaluated with separate multiply and add; result scaled by 2^n through the
    exponent bits.  Inputs below -87 are clamped to -87 (result stays normal).
    """
    x = np.asarray(x, dtype=_F)
    x = np.maximum(x, _EXP_CLAMP)
    t = x * _LOG2E
    n = np.rint(t).astype(_F)
    r = (x - n * _LN2_HI).astype(_F)
    r = (r - n * _LN2_LO).astype(_F)
    p = np.full_like(r, _C[0])
    for c in _C[1:]:
        p = (p * r).astype(_F)
        p = (p + c).astype(_F)
    scale = ((n.astype(np.int32) + 127) << 23).astype(np.int32).view(_F)
    return (p * scale).astype(_F)


def _as_f32(a) -> np.ndarray:
    """fp16 / bf16 / fp32 array-like (numpy or torch) -> float32 numpy (exact)."""
    if hasattr(a, "detach"):
        a = a.detach().cpu().float().numpy()
    a = np.asarray(a)
    return a.astype(_F)


def stable_topk(logits, k: int):
    """Stable descending order of each row; returns (values[M,k], ids[M,k] int32).

    Equal values keep ascending expert id (``ops/stable_argsort.py:46-50``).
    -0.0 and +0.0 compare equal, as in ``torch.sort``.  NaN is outside the
    contract (the reference's generators never produce it).
    """
    l = _as_f32(logits)
    order = np.argsort(-l, axis=1, kind="stable")
    # -l maps +0/-0 to -0/+0 which compare equal, so stability is preserved.
    ids = order[:, :k].astype(np.int32)
    vals = np.take_along_axis(l, order[:, :k], axis=1)
    return vals, ids


def topk_softmax(logits, k: int, renormalize: bool = True):
    """Router from logits: (weights fp32 [M,k], ids int32 [M,k]).

    ``renormalize=True`` is the reference's only mode
    (``ops/stable_route.py:130``).  ``False`` divides by the sum over all E
    columns instead (vLLM-style weights, ``layers/vllm_route.py:79-84``); that
    mode is specified to a tolerance only, because its sum order is free.
    """
    l = _as_f32(logits)
    vals, ids = stable_topk(l, k)
    d = (vals - vals[:, :1]).astype(_F)
    e = exp_recipe(d)
    if renormalize:
        s = e[:, 0].copy()
        for j in range(1, k):
            s = (s + e[:, j]).astype(_F)
    else:
        s = np.zeros(l.shape[0], dtype=_F)
        full = exp_recipe((l - vals[:, :1]).astype(_F))
        for j in range(l.shape[1]):
            s = (s + full[:, j]).astype(_F)
    w = (e / s[:, None]).astype(_F)
    return w, ids


def softmax_topk(logits, k: int, renormalize: bool = False):
    """Softmax over all E columns, then top-k on the probabilities: the routing of the
    reference's baseline layer (``fast_route/fast_route/layers/vllm_route.py:72-84``).

    The op it calls, ``vllm._moe_C.topk_softmax``, belongs to vLLM 0.4.0.post1
    (``requirements.txt:1``; not vendored): fp32 softmax, then k rounds of arg-max in which
    equal probabilities go to the lower expert id, ``token_expert_indicies[t,j] = j*M + t``.
    Parity of the weights is unpinned beyond the reference's own tolerance for this op
    (``tests/test_route.py:136-143``, atol 1e-2); the bit recipe below is this build's:
    e = exp_recipe(l - max), s = sums of 8 consecutive columns in ascending order combined by
    a balanced binary tree over adjacent blocks (E padded with zeros to a power of two >= 8),
    p = e * (1/s); renormalize: w_j = p_j / ((p_0 + p_1) + ...).

    Returns (weights fp32 [M,k], ids int32 [M,k], source_rows int32 [M,k]).
    """
    l = _as_f32(logits)
    M, E = l.shape
    Ep = 8
    while Ep < E:
        Ep *= 2
    mx = l.max(axis=1, keepdims=True)
    e = np.zeros((M, Ep), dtype=_F)
    e[:, :E] = exp_recipe((l - mx).astype(_F))
    blocks = e.reshape(M, Ep // 8, 8)
    part = blocks[:, :, 0].copy()
    for i in range(1, 8):
        part = (part + blocks[:, :, i]).astype(_F)
    while part.shape[1] > 1:
        part = (part[:, 0::2] + part[:, 1::2]).astype(_F)
    inv = (_F(1.0) / part[:, 0]).astype(_F)
    p = (e[:, :E] * inv[:, None]).astype(_F)
    order = np.argsort(-p, axis=1, kind="stable")[:, :k]
    ids = order.astype(np.int32)
    w = np.take_along_axis(p, order, axis=1)
    if renormalize:
        s = w[:, 0].copy()
        for j in range(1, k):
            s = (s + w[:, j]).astype(_F)
        w = (w / s[:, None]).astype(_F)
    src = (np.arange(k, dtype=np.int64)[None, :] * M + np.arange(M, dtype=np.int64)[:, None]).astype(np.int32)
    return w, ids, src


def full_argsort_fill(logits, k: int):
    """What the reference leaves in caller-provided ``[M,E]`` buffers.

    ``route_kernel`` stores all E columns (``ops/stable_route.py:110-121``): the
    ids buffer holds the full stable descending argsort, the weights buffer the k
    softmax weights followed by zeros (exp(-inf) = 0).
    """
    l = _as_f32(logits)
    M, E = l.shape
    w, _ = topk_softmax(l, k)
    _, ids = stable_topk(l, E)
    wfull = np.zeros((M, E), dtype=_F)
    wfull[:, :k] = w
    return wfull, ids


def gate_logits(x, gate) -> np.ndarray:
    """fp32 logits  X[M,H] . G[H,E]  computed with CPU torch in fp32."""
    import torch
    xt = x.detach().cpu().float() if hasattr(x, "detach") else torch.from_numpy(_as_f32(x))
    gt = gate.detach().cpu().float() if hasattr(gate, "detach") else torch.from_numpy(_as_f32(gate))
    return (xt @ gt).numpy().astype(_F)


def route_from_hidden(x, gate, k: int, renormalize: bool = True):
    """Router from hidden states: returns (weights, ids, logits_fp32)."""
    l = gate_logits(x, gate)
    w, ids = topk_softmax(l, k, renormalize)
    return w, ids, l
