"""W4A16 split-K GEMM on the GPU against the CPU oracle and the reference kernel's own outputs
(benchmarks/splitk_gemm/splitk.py:26-103, 178-216; its driver case is m=16, k=n=4096, group 128).

Tolerances: the dequantised fp16 weights are bit-exact.  The GEMM accumulates in fp32 and rounds once
to fp16, so |c - ref| <= 2^-11 |ref| (final rounding) + 2e-6 * (|a| . |w|) (fp32 accumulation in any
order); the reference's own output carries four more fp16 roundings from its atomics."""

import os

import numpy as np
import pytest
import torch

import oracle
from fast_route_b200 import _lib
from fast_route_b200.ops import splitk_gemm as sk

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def inputs(m, k, n, groupsize, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    a = (torch.randn(m, k, generator=g) * 0.5).half()
    b = torch.randint(-2**31, 2**31 - 1, (k // 8, n), generator=g, dtype=torch.int64).to(torch.int32)
    zeros = torch.randint(-2**31, 2**31 - 1, (k // groupsize, n // 8), generator=g, dtype=torch.int64).to(torch.int32)
    scales = (torch.randn(k // groupsize, n, generator=g) * 0.5).half()
    return a, b, scales, zeros


def check(c, a, b, scales, zeros, groupsize):
    w = oracle.w4a16.dequant(b, scales, zeros, groupsize).astype(np.float64)
    a64 = a.numpy().astype(np.float64)
    ref = a64 @ w
    bound = 2.0 ** -11 * np.abs(ref) + 2e-6 * (np.abs(a64) @ np.abs(w)) + 1e-7
    err = np.abs(c.cpu().numpy().astype(np.float64) - ref)
    assert (err <= bound).all(), (err.max(), (err / bound).max())


def test_reference_kernel_golden_vectors(dev):
    g = np.load(os.path.join(GOLD, "w4a16.npz"))
    for ci in range(3):
        a, b, s, z = (torch.from_numpy(g[f"{n}_{ci}"]) for n in ("a", "b", "scales", "zeros"))
        c = sk.matmul_split_k(a.to(dev), b.to(dev), s.to(dev), z.to(dev))
        gold = g[f"c_{ci}"]
        if ci == 2:     # one-hot activations: rows of the dequantised matrix, exact in both implementations
            assert np.array_equal(c.cpu().numpy().view(np.uint16), gold.view(np.uint16))
        else:
            check(c, a, b, s, z, 128)
            ref = oracle.w4a16.matmul_split_k(a, b, s, z)
            assert (np.abs(c.cpu().numpy().astype(np.float64) - gold.astype(np.float64))
                    <= 9 * 2.0 ** -11 * np.maximum(np.abs(ref), 64.0)).all()


@pytest.mark.parametrize("k,n,gs", [(128, 8, 64), (512, 64, 128), (1024, 200, 256), (4096, 4096, 128)])
def test_dequantised_weights_bit_exact(dev, k, n, gs):
    _, b, s, z = inputs(1, k, n, gs, seed=k + n)
    w = sk.dequantize(b.to(dev), s.to(dev), z.to(dev), gs)
    assert np.array_equal(w.cpu().numpy().view(np.uint16), oracle.w4a16.dequant(b, s, z, gs).view(np.uint16))
    # the GEMM's in-kernel dequantisation: one-hot activations return weight rows exactly
    m = min(256, k)
    rows = torch.randperm(k, generator=torch.Generator().manual_seed(1))[:m]
    if k == 1024:
        for factor in (200.0, 1e-3, 0.0):     # scales >= 32, < 2^-9 and zero take the un-fused product path
            s = (s.float() * factor).half()
            w = sk.dequantize(b.to(dev), s.to(dev), z.to(dev), gs)
            assert np.array_equal(w.cpu().numpy().view(np.uint16), oracle.w4a16.dequant(b, s, z, gs).view(np.uint16))
        _, _, s, _ = inputs(1, k, n, gs, seed=k + n)
        s = s * 40                            # a mix of both paths inside one matrix
        w = sk.dequantize(b.to(dev), s.to(dev), z.to(dev), gs)
        assert np.array_equal(w.cpu().numpy().view(np.uint16), oracle.w4a16.dequant(b, s, z, gs).view(np.uint16))
    a = torch.zeros(m, k, dtype=torch.float16)
    a[torch.arange(m), rows] = 1.0
    c = sk.matmul_split_k(a.to(dev), b.to(dev), s.to(dev), z.to(dev), gs)
    assert torch.equal(c.cpu(), w.cpu()[rows])
    # up to 64 rows the kernel keeps the dequantised operand in tensor memory, with k interleaved inside every packed
    # word and the activation tile reordered to match: the same exactness must hold there
    for msmall in (1, 16, 48, 64):
        msmall = min(msmall, m)
        c = sk.matmul_split_k(a[:msmall].to(dev), b.to(dev), s.to(dev), z.to(dev), gs)
        assert torch.equal(c.cpu(), w.cpu()[rows[:msmall]]), msmall


@pytest.mark.parametrize("m", [1, 5, 16, 17, 100, 256, 300])
@pytest.mark.parametrize("k,n,gs", [(512, 64, 128), (1024, 328, 64), (2048, 1024, 256)])
def test_shapes(dev, m, k, n, gs):
    a, b, s, z = inputs(m, k, n, gs, seed=m * 3 + n)
    c = sk.matmul_split_k(a.to(dev), b.to(dev), s.to(dev), z.to(dev), gs)
    check(c, a, b, s, z, gs)


def test_reference_driver_case_all_split_factors_and_determinism(dev):
    m, k, n, gs = 16, 4096, 4096, 128           # benchmarks/splitk_gemm/splitk.py:279-283
    a, b, s, z = inputs(m, k, n, gs, seed=0)
    ad, bd, sd, zd = a.to(dev), b.to(dev), s.to(dev), z.to(dev)
    outs = {}
    for split in (0, 1, 2, 4, 8):
        outs[split] = sk.matmul_split_k(ad, bd, sd, zd, gs, split_k=split)
        check(outs[split], a, b, s, z, gs)
        again = sk.matmul_split_k(ad, bd, sd, zd, gs, split_k=split)
        assert torch.equal(outs[split], again)
    # strided activations and output
    abig = torch.zeros(m, k + 64, dtype=torch.float16, device=dev)
    abig[:, :k] = ad
    cbig = torch.zeros(m, n + 8, dtype=torch.float16, device=dev)
    sk.matmul_split_k(abig[:, :k], bd, sd, zd, gs, out=cbig[:, :n])
    assert torch.equal(cbig[:, :n], outs[0]) and float(cbig[:, n:].abs().sum()) == 0.0
    assert _lib.device_status()[0] == 0


def test_argument_errors(dev):
    a, b, s, z = inputs(4, 512, 64, 128, seed=1)
    ad, bd, sd, zd = a.to(dev), b.to(dev), s.to(dev), z.to(dev)
    lib = _lib.load()
    c = torch.empty(4, 64, dtype=torch.float16, device=dev)
    st = _lib.stream_ptr(dev)
    args = lambda **kw: [kw.get("a", _lib.ptr(ad)), 512, _lib.ptr(bd), _lib.ptr(sd), _lib.ptr(zd), kw.get("m", 4),
                         kw.get("n", 64), kw.get("k", 512), kw.get("gs", 128), _lib.ptr(c), 64, kw.get("split", 0), st]
    assert lib.fr_w4a16_gemm(*args(a=None)) == -1
    assert lib.fr_w4a16_gemm(*args(n=60)) == -3
    assert lib.fr_w4a16_gemm(*args(k=448)) == -3
    assert lib.fr_w4a16_gemm(*args(gs=32)) == -3
    assert lib.fr_w4a16_gemm(*args(split=3)) == -1
    assert lib.fr_w4a16_gemm(*args(m=0)) == 0
