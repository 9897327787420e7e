"""Seeded synthetic inputs with the shapes and value distributions of the
reference's benchmarks (``benchmarks/fused_route/moe_bench.py:83-88`` draws
random normal tensors; no dataset is involved).

Every tensor is drawn in fp32 on the CPU from its own ``torch.Generator`` seeded
``seed*1000 + tensor_index`` and then cast / moved, so a CPU checker and the GPU
see identical bits.
"""

from __future__ import annotations

import torch


def _gen(seed: int, index: int) -> torch.Generator:
    return torch.Generator(device="cpu").manual_seed(seed * 1000 + index)


def randn(shape, seed: int, index: int, std: float = 1.0) -> torch.Tensor:
    t = torch.randn(*shape, generator=_gen(seed, index), dtype=torch.float32)
    return t * std if std != 1.0 else t


def moe_inputs(M: int, H: int, I: int, E: int, seed: int = 0, dtype=torch.bfloat16,
               device="cpu", weight_std: float = 0.02, gate_bias=None):
    """x[M,H]~N(0,1); W_g[E,H], w1[E,2I,H], w2[E,H,I] ~ N(0, weight_std^2).

    Returns (x, gate, w1, w2) with ``gate`` the ``[H,E]`` strided view ``W_g.t()``
    that the layer interface takes.  Weights are generated expert by expert so
    very large layers never hold an fp32 copy of all experts.
    ``gate_bias`` (length-E tensor) is folded in by appending one constant
    column to x and one row to the gate (H grows by 8 to keep 16-byte rows):
    the reference has no bias argument, a bias is just one more input feature.
    """
    x = randn((M, H), seed, 0)
    wg = randn((E, H), seed, 1, weight_std)
    if gate_bias is not None:
        pad = 8
        xb = torch.zeros(M, H + pad)
        xb[:, :H] = x
        xb[:, H] = 1.0
        wgb = torch.zeros(E, H + pad)
        wgb[:, :H] = wg
        wgb[:, H] = gate_bias.float()
        x, wg = xb, wgb
    Hx = x.shape[1]
    w1 = torch.empty(E, 2 * I, Hx, dtype=dtype, device=device)
    w2 = torch.empty(E, Hx, I, dtype=dtype, device=device)
    for e in range(E):
        a = randn((2 * I, H), seed, 100 + e, weight_std)
        b = randn((H, I), seed, 10000 + e, weight_std)
        if Hx != H:
            a = torch.cat([a, torch.zeros(2 * I, Hx - H)], 1)
            b = torch.cat([b, torch.zeros(Hx - H, I)], 0)
        w1[e].copy_(a)
        w2[e].copy_(b)
    x = x.to(dtype).to(device)
    gate = wg.to(dtype).to(device).t()
    return x, gate, w1, w2


def zipf_gate_bias(E: int, s: float = 1.2, scale: float = 1.0, seed: int = 0) -> torch.Tensor:
    """log of a Zipf(s) pmf over a seeded permutation of the experts, times ``scale``."""
    ranks = torch.arange(1, E + 1, dtype=torch.float64)
    pmf = ranks.pow(-s)
    pmf = pmf / pmf.sum()
    perm = torch.randperm(E, generator=_gen(seed, 7))
    bias = torch.empty(E, dtype=torch.float64)
    bias[perm] = pmf.log()
    return (bias * scale).float()


def routing_logits(M: int, E: int, k: int, seed: int = 0, dtype=torch.float16,
                   dup_frac: float = 0.05) -> torch.Tensor:
    """logits[M,E] ~ N(0,1) in ``dtype``; ``dup_frac`` of the rows get exact
    duplicate values copied across at least k columns, so ties straddle the k-th
    rank and exercise the stable tie-break."""
    g = _gen(seed, 3)
    x = torch.randn(M, E, generator=g, dtype=torch.float32).to(dtype)
    dup = torch.rand(M, generator=g) < dup_frac
    ncopy = max(k, 2)
    src = torch.randint(0, E, (M, ncopy), generator=g)
    dst = torch.randint(0, E, (M, ncopy), generator=g)
    rows = dup.nonzero().flatten()
    if rows.numel():
        vals = x[rows].gather(1, src[rows])
        x[rows] = x[rows].scatter(1, dst[rows], vals)
    return x


def layer_flops(M: int, H: int, I: int, E: int, k: int) -> float:
    """Algorithmic FLOPs of one layer call: gate GEMM + the three expert GEMMs."""
    return 2.0 * M * H * E + 6.0 * M * k * H * I


def layer_bytes(active_experts: int, M: int, H: int, I: int, E: int, elt: int = 2) -> float:
    """Algorithmic HBM bytes: active experts' weights once + x in + out + gate."""
    return active_experts * 3.0 * H * I * elt + 2.0 * M * H * elt + H * E * elt


__all__ = ["randn", "moe_inputs", "zipf_gate_bias", "routing_logits", "layer_flops", "layer_bytes"]
