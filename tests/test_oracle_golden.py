"""The CPU oracle against the golden vectors produced by the reference's own code
(see tests/golden/make_golden.py for how they were made)."""

import os

import numpy as np
import pytest
import torch

import oracle

GOLD = os.path.join(os.path.dirname(__file__), "golden")


@pytest.mark.parametrize("E", [8, 16, 64, 128])
@pytest.mark.parametrize("name", ["f16", "f32"])
def test_stable_argsort_matches_reference_kernel(E, name):
    g = np.load(os.path.join(GOLD, "stable_argsort.npz"))
    x = g[f"x_{E}_{name}"]
    vals, ids = oracle.stable_topk(x, E)
    assert np.array_equal(ids, g[f"ids_{E}_{name}"])
    assert np.array_equal(vals, g[f"sorted_{E}_{name}"])
    # the vectors contain ties, otherwise the tie rule is not exercised
    assert (np.diff(np.sort(x, axis=1), axis=1) == 0).any()


@pytest.mark.parametrize("case", range(5))
def test_route_matches_reference_kernel(case):
    g = np.load(os.path.join(GOLD, "route_kernel.npz"))
    M, K, E, k = (int(v) for v in g[f"meta_{case}"])
    h = torch.from_numpy(g[f"h_{case}"])
    gate = torch.from_numpy(g[f"g_{case}"])
    w, ids, logits = oracle.route_from_hidden(h, gate, k)
    assert np.array_equal(ids, g[f"ids_{case}"][:, :k])
    # reference tolerance for the weights: atol 1e-2 (fast_route/tests/test_route.py:67-74);
    # the restatement is far inside it
    np.testing.assert_allclose(w, g[f"w_{case}"][:, :k], atol=2e-7, rtol=0)
    wfull, idfull = oracle.full_argsort_fill(logits, k)
    assert np.array_equal(idfull, g[f"ids_{case}"])
    np.testing.assert_allclose(wfull, g[f"w_{case}"], atol=2e-7, rtol=0)


def test_torch_moe_small_matches_reference_function():
    g = np.load(os.path.join(GOLD, "torch_moe.npz"))
    x, gate, w1, w2 = (torch.from_numpy(g[f"small_{n}"]) for n in ("x", "gate", "w1", "w2"))
    out, w, ids = oracle.moe_layer(x, gate, w1, w2, 2)
    assert np.array_equal(ids, g["small_ti"])
    np.testing.assert_allclose(w, g["small_tw"], atol=2e-7, rtol=0)
    np.testing.assert_allclose(out.numpy(), g["small_out"], atol=1e-6, rtol=1e-5)


def test_torch_moe_reference_cpu_case():
    """fp32, M=256, H=1024, I=2048, E=8, top-2, seed 0: the reference's CPU-runnable case."""
    from fast_route_b200 import synth
    g = np.load(os.path.join(GOLD, "torch_moe.npz"))
    x, gate, w1, w2 = synth.moe_inputs(256, 1024, 2048, 8, seed=0, dtype=torch.float32)
    sums = np.array([x.double().sum().item(), w1.double().sum().item(), w2.double().sum().item()])
    np.testing.assert_allclose(sums, g["c1_x_sum"], rtol=1e-9, err_msg="seeded inputs differ from the ones the golden output was made from")
    out, w, ids = oracle.moe_layer(x, gate, w1, w2, 2)
    assert np.array_equal(ids, g["c1_ti"])
    np.testing.assert_allclose(w, g["c1_tw"], atol=2e-7, rtol=0)
    np.testing.assert_allclose(out[::8, ::16].numpy(), g["c1_out_sample"], atol=2e-5, rtol=1e-4)


def test_align_docstring_example():
    """Known answer from fast_route/fast_route/ops/fused_moe.py:151-159 (1-based experts there)."""
    ids = np.array([[2, 3, 4], [1, 2, 4], [1, 3, 4], [1, 2, 3]]) - 1
    s, e, n, c = oracle.moe_align_block_size(ids, 4, 4)
    assert s[:16].tolist() == [3, 6, 9, 12, 0, 4, 10, 12, 1, 7, 11, 12, 2, 5, 8, 12]
    assert e[:4].tolist() == [0, 1, 2, 3] and int(n[0]) == 16 and c.tolist() == [3, 3, 3, 3]


def test_align_properties():
    rng = np.random.default_rng(0)
    for (n, E, bs) in [(0, 4, 16), (1, 8, 128), (1000, 64, 64), (777, 5, 7)]:
        ids = rng.integers(0, E, size=n)
        if E == 64:
            ids[ids == 3] = 2          # an expert without tokens
        s, e, npost, c = oracle.moe_align_block_size(ids, bs, E)
        npost = int(npost[0])
        assert npost % bs == 0 and npost == sum((int(x) + bs - 1) // bs * bs for x in c)
        valid = s[:npost]
        real = valid[valid < n]
        assert sorted(real.tolist()) == list(range(n))
        blocks = valid.reshape(-1, bs)
        for b, row in enumerate(blocks):
            r = row[row < n]
            assert (ids[r] == e[b]).all() and (np.diff(r) > 0).all()
        assert (s[npost:] == n).all()


def test_exp_recipe_accuracy_and_tie_rule():
    xs = np.linspace(-87, 0, 100001).astype(np.float32)
    rel = np.abs(oracle.exp_recipe(xs) - np.exp(xs.astype(np.float64))) / np.exp(xs.astype(np.float64))
    assert rel.max() < 2e-7
    assert oracle.exp_recipe(np.float32(0.0)) == np.float32(1.0)
    logits = np.array([[1.0, 2.0, 2.0, 0.5, 2.0, -0.0, 0.0, -1.0]], dtype=np.float32)
    w, ids = oracle.topk_softmax(logits, 4)
    assert ids.tolist() == [[1, 2, 4, 0]]
    np.testing.assert_allclose(w.sum(), 1.0, atol=1e-6)
    _, full = oracle.stable_topk(logits, 8)
    assert full.tolist() == [[1, 2, 4, 0, 3, 5, 6, 7]]   # -0.0 and +0.0 tie -> lower id first
    wt = torch.softmax(torch.sort(torch.from_numpy(logits), descending=True, stable=True)[0][:, :4], -1)
    np.testing.assert_allclose(w, wt.numpy(), atol=1e-6)


def test_softmax_topk_order_rule_and_source_rows():
    """Baseline-layer routing (softmax over all experts, then top-k): equal probabilities go to the
    lower expert id, weights are the plain softmax, source rows are j*M + t
    (fast_route/fast_route/layers/vllm_route.py:72-84 and the vLLM 0.4.0 op it calls)."""
    rng = np.random.default_rng(5)
    for E, k in ((8, 2), (60, 6), (64, 6), (128, 8), (256, 4)):
        logits = rng.standard_normal((257, E)).astype(np.float32)
        logits[::5, 1] = logits[::5, 0]                       # exact ties
        logits[::7] = 0.25                                    # all-equal rows
        w, ids, src = oracle.softmax_topk(logits, k)
        p64 = torch.softmax(torch.from_numpy(logits).double(), -1).numpy()
        assert np.abs(w - np.take_along_axis(p64, ids.astype(np.int64), 1)).max() < 2e-7
        assert np.array_equal(ids[::7], np.tile(np.arange(k, dtype=np.int32), (len(ids[::7]), 1)))
        # selection is a valid stable top-k of the probabilities
        order = np.argsort(-p64, axis=1, kind="stable")[:, :k]
        agree = (order == ids).all(1)
        assert agree.mean() > 0.99          # fp32 vs fp64 may order near-equal probabilities differently
        assert np.array_equal(src, np.arange(k)[None, :] * 257 + np.arange(257)[:, None])
        wr, ids2, _ = oracle.softmax_topk(logits, k, renormalize=True)
        assert np.array_equal(ids, ids2)
        assert np.abs(wr.sum(1) - 1).max() < 1e-6
        assert np.abs(wr - w / w.sum(1, keepdims=True)).max() < 2e-7


def test_w4a16_oracle_matches_reference_kernel():
    """Outputs of the reference's W4A16 split-K Triton kernel (benchmarks/splitk_gemm/splitk.py:26-103)
    run on CPU.  One-hot activations make output rows equal single dequantised weight rows, which pins
    the fp16 dequantisation bit for bit; the random cases agree to the fp16 roundings of the reference's
    four atomically added K slices."""
    g = np.load(os.path.join(GOLD, "w4a16.npz"))
    w = oracle.w4a16.dequant(g["b_2"], g["scales_2"], g["zeros_2"])
    assert np.array_equal(w[g["onehot_rows"]].view(np.uint16), g["c_2"].view(np.uint16))
    for ci in range(2):
        ref = oracle.w4a16.matmul_split_k(g[f"a_{ci}"], g[f"b_{ci}"], g[f"scales_{ci}"], g[f"zeros_{ci}"])
        c = g[f"c_{ci}"].astype(np.float64)
        # 4 partial sums each rounded to fp16 (2^-11 relative) plus the roundings of the running sum
        assert (np.abs(c - ref) <= 8 * 2.0 ** -11 * np.maximum(np.abs(ref), 64.0)).all()


def test_w4a16_dequant_known_answers():
    """Hand-computed nibble order: word 0x76543210 holds q = 0..7 for rows k = 0..7 (:62, :70, :86);
    zero-point word 0x00000021 gives z = 1 for column 0 and z = 2 for column 1 (:65, :71, :83)."""
    b = np.full((8, 8), 0x76543210, dtype=np.int64).astype(np.int32)          # k = 64
    scales = np.full((1, 8), 0.5, dtype=np.float16)
    zeros = np.array([[0x00000021]], dtype=np.int32)
    w = oracle.w4a16.dequant(b, scales, zeros, groupsize=64).astype(np.float64)
    q = np.tile(np.arange(8), 8)
    z = np.array([1, 2, 0, 0, 0, 0, 0, 0])
    assert np.array_equal(w, (q[:, None] - (z[None, :] + 1)) * 0.5)
