"""The layer with E4M3 expert weights against an fp32 evaluation that applies the same quantisation
steps (weights per row, activations per token row before each GEMM, the intermediate rounded to the
16-bit type in between).  The quantisation itself costs a few percent against the unquantised layer;
that is a property of the format, checked separately with a loose bound."""

import numpy as np
import pytest
import torch

import fast_route_b200 as fr
import oracle
from fast_route_b200 import synth
from fast_route_b200.layers.fp8 import quantize_rows_e4m3

pytestmark = pytest.mark.gpu


def fp8_layer_reference(x, w1_q, s1, w2_q, s2, tw, ti, dt):
    """fp32 math on exactly the values the device multiplies."""
    M, H = x.shape
    k = ti.shape[1]
    w1 = w1_q.float() * s1[..., None]
    w2 = w2_q.float() * s2[..., None]
    xq, xs = quantize_rows_e4m3(x)
    xd = xq.float() * xs[:, None]
    out = torch.zeros(M, H)
    for j in range(k):
        for e in range(w1.shape[0]):
            rows = (ti[:, j] == e).nonzero().flatten()
            if rows.numel() == 0:
                continue
            h = oracle.silu_and_mul(xd[rows] @ w1[e].t()).to(dt)          # intermediate stored in 16 bits
            hq, hs = quantize_rows_e4m3(h)
            y = ((hq.float() * hs[:, None]) @ w2[e].t()) * tw[rows, j:j + 1]
            out[rows] += y.to(dt).float()                                  # per-slot result stored in 16 bits
    return out


@pytest.mark.parametrize("M,H,I,E,k,dt", [(64, 256, 256, 4, 2, torch.bfloat16), (300, 512, 384, 8, 2, torch.bfloat16),
                                          (1000, 256, 640, 16, 4, torch.float16), (5, 512, 1024, 8, 2, torch.bfloat16),
                                          (1, 512, 1024, 8, 2, torch.bfloat16), (2048, 512, 256, 64, 6, torch.bfloat16),
                                          (4000, 1024, 512, 8, 2, torch.bfloat16)])
def test_fp8_layer_vs_quantised_reference(dev, M, H, I, E, k, dt):
    x, gate, w1, w2 = synth.moe_inputs(M, H, I, E, seed=21, dtype=dt, weight_std=0.05)
    w1_q, s1, w2_q, s2 = fr.quantize_experts_fp8(w1.to(dev), w2.to(dev))
    out, tw, ti = fr.fused_moe_fp8(x.to(dev), gate.to(dev), w1_q, s1, w2_q, s2, k, return_routing=True)
    # routing is the 16-bit router: identical to the unquantised layer's
    tw0, ti0 = fr.fused_route(x.to(dev), gate.to(dev), k)
    assert torch.equal(ti, ti0) and torch.equal(tw, tw0)
    ref = fp8_layer_reference(x, w1_q.cpu(), s1.cpu(), w2_q.cpu(), s2.cpu(), tw.cpu(), ti.cpu(), dt)
    diff = (out.float().cpu() - ref).abs()
    scale = max(1.0, ref.abs().max().item())
    # a 16-bit rounding boundary of the intermediate can fall differently (accumulation order), which
    # moves one fp8 code of one element: bounded by a few 16-bit ulps of the output
    assert diff.max().item() <= 3e-2 * scale, diff.max().item()
    assert (diff.mean() / ref.abs().mean()).item() <= 5e-3
    # against the unquantised fp32 layer: the cost of the format
    full, _, _ = oracle.moe_layer(x, gate, w1, w2, k, routing=(tw.cpu(), ti.cpu()))
    rel = ((out.float().cpu() - full).abs().mean() / full.abs().mean()).item()
    assert rel <= 1e-1, rel
    out2 = fr.fused_moe_fp8(x.to(dev), gate.to(dev), w1_q, s1, w2_q, s2, k)
    assert torch.equal(out, out2)


def test_quantize_rows_roundtrip(dev):
    t = synth.randn((33, 512), 5, 0).to(dev)
    q, s = quantize_rows_e4m3(t)
    back = q.float() * s[:, None]
    assert (back - t).abs().max().item() <= t.abs().max().item() * 2.0 ** -4
    z, sz = quantize_rows_e4m3(torch.zeros(2, 16, device=dev))
    assert (z.float() == 0).all() and (sz == 1).all()
