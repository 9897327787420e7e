"""Seeded random shapes through the layer, the W4A16 GEMM and the softmax-then-top-k router: odd expert counts,
hidden sizes that are not multiples of the tile sizes, batch sizes on both sides of every kernel-selection
threshold.  Same checks as the fixed cases: routing bit-exact from the device's logits, layer within the stated
tolerance of the fp32 oracle on the same routing, calls repeatable bit for bit, device status clean."""

import random

import numpy as np
import pytest
import torch

import fast_route_b200 as fr
import oracle
from fast_route_b200 import _lib, synth
from fast_route_b200.ops import splitk_gemm as sk
from fast_route_b200.ops.vllm_route import topk_softmax

pytestmark = pytest.mark.gpu


def bits(a):
    return np.ascontiguousarray(a).view(np.int32)


@pytest.mark.parametrize("seed", [1, 2])
def test_layer_random_shapes(dev, seed):
    rnd = random.Random(seed)
    done = 0
    while done < 40:
        E = rnd.choice([1, 2, 3, 4, 7, 8, 16, 24, 64, 100, 128, 256])
        k = rnd.choice([kk for kk in (1, 2, 3, 4, 6, 8) if kk <= E])
        M = rnd.choice([1, 2, 3, 7, 8, 9, 16, 17, 31, 33, 64, 100, 128, 200, 257, 400, 700, 1024, 1500])
        H = rnd.choice([64, 72, 128, 200, 256, 520, 1024])
        I = rnd.choice([64, 72, 136, 256, 520, 1024])
        dt = rnd.choice([torch.bfloat16, torch.float16])
        if M * k * max(H, I) * E > 1.5e9:
            continue
        done += 1
        x, gate, w1, w2 = synth.moe_inputs(M, H, I, E, seed=seed * 1000 + done, dtype=dt, weight_std=0.05)
        xd, gd, w1d, w2d = x.to(dev), gate.to(dev), w1.to(dev), w2.to(dev)
        out, tw, ti = fr.fused_moe(xd, gd, w1d, w2d, k, return_routing=True)
        case = dict(M=M, H=H, I=I, E=E, k=k, dt=dt)
        assert torch.equal(out, fr.fused_moe(xd, gd, w1d, w2d, k)), case
        _, _, lg = fr.fused_route(xd, gd, k, return_logits=True)
        ow, oi = oracle.topk_softmax(lg.cpu().numpy(), k)
        assert np.array_equal(ti.cpu().numpy(), oi), case
        assert np.array_equal(bits(tw.cpu().numpy()), bits(ow)), case
        ref, _, _ = oracle.moe_layer(x, gate, w1, w2, k, routing=(tw.cpu(), ti.cpu()))
        diff = (out.float().cpu() - ref).abs()
        assert diff.max().item() <= 2e-2 + ref.abs().max().item() * 2.0 ** -7, case
        assert (diff.mean() / ref.abs().mean().clamp_min(1e-9)).item() <= 1e-2, case
    assert _lib.device_status()[0] == 0


def test_w4a16_random_shapes(dev):
    rnd = random.Random(7)
    for it in range(60):
        m = rnd.choice([1, 2, 5, 16, 17, 33, 48, 64, 65, 100, 128, 129, 200, 300])   # 64 / 65: the two GEMM kernels
        gs = rnd.choice([64, 128, 192, 256])       # 64 and 192: a pair of K steps spans two quantisation groups
        k = gs * rnd.choice([1, 2, 3, 4, 8, 16])
        n = 8 * rnd.choice([1, 3, 8, 16, 17, 33, 64, 100, 129])
        g = torch.Generator().manual_seed(it)
        a = (torch.randn(m, k, generator=g) * 0.5).half()
        b = torch.randint(-2**31, 2**31 - 1, (k // 8, n), generator=g, dtype=torch.int64).to(torch.int32)
        z = torch.randint(-2**31, 2**31 - 1, (k // gs, n // 8), generator=g, dtype=torch.int64).to(torch.int32)
        s = (torch.randn(k // gs, n, generator=g) * rnd.choice([0.5, 0.5, 0.05, 1e-3])).half()
        split = rnd.choice([0, 0, 1, 2, 4, 8])
        c = sk.matmul_split_k(a.to(dev), b.to(dev), s.to(dev), z.to(dev), gs, split_k=split)
        case = dict(m=m, k=k, n=n, gs=gs, split=split)
        assert torch.equal(c, sk.matmul_split_k(a.to(dev), b.to(dev), s.to(dev), z.to(dev), gs, split_k=split)), case
        w = oracle.w4a16.dequant(b, s, z, gs).astype(np.float64)
        a64 = a.numpy().astype(np.float64)
        ref = a64 @ w
        bound = 2.0 ** -11 * np.abs(ref) + 2e-6 * (np.abs(a64) @ np.abs(w)) + 1e-7
        assert (np.abs(c.cpu().numpy().astype(np.float64) - ref) <= bound).all(), case
    assert _lib.device_status()[0] == 0


def test_softmax_then_topk_random_shapes(dev):
    rnd = random.Random(11)
    for it in range(40):
        E = rnd.choice([1, 2, 3, 5, 8, 9, 16, 31, 64, 100, 128, 200, 256])
        k = rnd.choice([kk for kk in (1, 2, 3, 4, 6, 8) if kk <= E])
        M = rnd.choice([1, 2, 33, 257, 1000, 5000])
        dt = rnd.choice([torch.float16, torch.bfloat16, torch.float32])
        renorm = rnd.choice([False, True])
        lg = synth.routing_logits(M, E, k, seed=it, dtype=dt, dup_frac=0.3)
        w = torch.empty(M, k, dtype=torch.float32, device=dev)
        ids = torch.empty(M, k, dtype=torch.int32, device=dev)
        src = torch.empty(M, k, dtype=torch.int32, device=dev)
        topk_softmax(w, ids, src, lg.to(dev), renormalize=renorm)
        ow, oi, osrc = oracle.softmax_topk(lg, k, renormalize=renorm)
        case = dict(M=M, E=E, k=k, dt=dt, renorm=renorm)
        assert np.array_equal(ids.cpu().numpy(), oi), case
        assert np.array_equal(bits(w.cpu().numpy()), bits(ow)), case
        assert np.array_equal(src.cpu().numpy(), osrc), case
