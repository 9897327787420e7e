"""Router from logits and the align stage on the GPU, bit-exact against the CPU oracle.
Shapes follow the reference's tests (fast_route/tests/test_argsort.py:101-145,
test_route.py:12-77) and the routing microbenchmark (16384 tokens, E in {8,64,128},
top-k in {2,6,8}, block 64, 5 % rows with exact duplicates)."""

import os

import numpy as np
import pytest
import torch

import oracle
from fast_route_b200 import synth
from fast_route_b200.ops import fused_moe as fm
from fast_route_b200.ops import stable_route as sr

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def bits(a):
    return np.ascontiguousarray(a).view(np.int32)


@pytest.mark.parametrize("E,k", [(8, 2), (8, 6), (8, 8), (64, 2), (64, 6), (64, 8), (128, 2), (128, 6), (128, 8)])
def test_routing_microbench_bit_exact(dev, E, k):
    M, bs = 16384, 64
    logits = synth.routing_logits(M, E, k, seed=0, dtype=torch.float16, dup_frac=0.05)
    w, ids = sr.route_from_logits(logits.to(dev), k)
    s, e, npost = fm.moe_align_block_size(ids, bs, E)
    ow, oi = oracle.topk_softmax(logits, k)
    os_, oe, on, _ = oracle.moe_align_block_size(oi, bs, E)
    assert np.array_equal(ids.cpu().numpy(), oi)
    assert np.array_equal(bits(w.cpu().numpy()), bits(ow))
    assert int(npost.item()) == int(on[0])
    assert np.array_equal(s.cpu().numpy(), os_)
    nb = int(on[0]) // bs
    assert np.array_equal(e.cpu().numpy()[:nb], oe[:nb])
    # softmax weights are also close to the library softmax (report-level check)
    wt = torch.softmax(torch.sort(logits.float(), descending=True, stable=True)[0][:, :k], -1).numpy()
    assert np.abs(w.cpu().numpy() - wt).max() < 5e-7


@pytest.mark.parametrize("E", [1, 2, 3, 5, 8, 9, 16, 31, 64, 100, 128, 200, 256, 300])
@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16, torch.float32])
def test_topk_shapes_and_dtypes(dev, E, dt):
    for k in sorted({1, min(2, E), min(8, E), min(12, E), E if E <= 16 else 1}):
        for M in (1, 33, 1000):
            logits = synth.routing_logits(M, E, k, seed=E * 7 + k, dtype=dt, dup_frac=0.3)
            w, ids = sr.route_from_logits(logits.to(dev), k)
            ow, oi = oracle.topk_softmax(logits, k)
            assert np.array_equal(ids.cpu().numpy(), oi), (E, k, M)
            assert np.array_equal(bits(w.cpu().numpy()), bits(ow)), (E, k, M)


def test_stable_argsort_golden_vectors(dev):
    """The reference's own bitonic argsort outputs (ties included) for full-width ordering."""
    g = np.load(os.path.join(GOLD, "stable_argsort.npz"))
    for E in (8, 16, 64, 128):
        for name, dt in (("f16", torch.float16), ("f32", torch.float32)):
            x = torch.from_numpy(g[f"x_{E}_{name}"]).to(dt)
            w, ids = sr.route_from_logits(x.to(dev), min(4, E), fill_rest=True)
            assert np.array_equal(ids.cpu().numpy(), g[f"ids_{E}_{name}"]), (E, name)
            assert (w[:, min(4, E):] == 0).all()


def test_fill_rest_matches_reference_buffers(dev):
    for E, k in ((8, 2), (64, 6), (128, 8), (300, 12)):
        logits = synth.routing_logits(500, E, k, seed=3, dtype=torch.float16, dup_frac=0.2)
        w, ids = sr.route_from_logits(logits.to(dev), k, fill_rest=True)
        ow, oi = oracle.full_argsort_fill(logits, k)
        assert np.array_equal(ids.cpu().numpy(), oi)
        assert np.array_equal(bits(w.cpu().numpy()), bits(ow))


def test_strided_logits_and_all_equal_rows(dev):
    base = synth.routing_logits(257, 64, 4, seed=5, dtype=torch.float16).to(dev)
    view = base.t().contiguous().t()          # column-major storage
    assert view.stride(1) != 1
    w, ids = sr.route_from_logits(view, 4)
    ow, oi = oracle.topk_softmax(base.cpu(), 4)
    assert np.array_equal(ids.cpu().numpy(), oi) and np.array_equal(bits(w.cpu().numpy()), bits(ow))
    flat = torch.zeros(10, 16, dtype=torch.float16, device=dev)   # every value ties: ids 0..k-1
    w, ids = sr.route_from_logits(flat, 3)
    assert ids.cpu().tolist() == [[0, 1, 2]] * 10
    assert np.array_equal(bits(w.cpu().numpy()), bits(oracle.topk_softmax(flat.cpu(), 3)[0]))


def test_no_renormalize_matches_softmax_over_all_experts(dev):
    logits = synth.routing_logits(300, 64, 6, seed=9, dtype=torch.float32)
    w, ids = sr.route_from_logits(logits.to(dev), 6, renormalize=False)
    p = torch.softmax(logits, -1)
    so, si = torch.sort(logits, descending=True, stable=True)
    assert np.array_equal(ids.cpu().numpy(), si[:, :6].numpy().astype(np.int32))
    np.testing.assert_allclose(w.cpu().numpy(), p.gather(1, si[:, :6]).numpy(), atol=1e-6)


def test_align_docstring_example(dev):
    ids = torch.tensor([[2, 3, 4], [1, 2, 4], [1, 3, 4], [1, 2, 3]], dtype=torch.int32) - 1
    s, e, n = fm.moe_align_block_size(ids.to(dev), 4, 4)
    assert s.cpu().tolist()[:16] == [3, 6, 9, 12, 0, 4, 10, 12, 1, 7, 11, 12, 2, 5, 8, 12]
    assert e.cpu().tolist()[:4] == [0, 1, 2, 3] and int(n.item()) == 16


@pytest.mark.parametrize("M,k,E,bs", [(1, 1, 1, 1), (1, 2, 8, 128), (3, 2, 8, 128), (100, 2, 8, 128),
                                      (4096, 2, 8, 128), (16384, 2, 8, 64), (16384, 8, 128, 64),
                                      (16384, 6, 64, 64), (8192, 6, 64, 128), (33, 1, 600, 16),
                                      (70000, 2, 8, 128), (1000, 4, 1500, 8), (0, 2, 8, 128)])
def test_align_matches_oracle(dev, M, k, E, bs):
    g = torch.Generator().manual_seed(M + E)
    ids = torch.randint(0, E, (M, k), generator=g, dtype=torch.int32)
    if E >= 8:
        ids[ids == 5] = 2      # an expert that receives nothing
    for _ in range(2):         # twice: the result must not depend on scheduling
        s, e, npost, cnt, inv = fm.moe_align_block_size(ids.to(dev), bs, E, return_extra=True)
        os_, oe, on, oc = oracle.moe_align_block_size(ids, bs, E)
        nb = int(on[0]) // bs
        assert int(npost.item()) == int(on[0])
        assert np.array_equal(s.cpu().numpy(), os_)
        assert np.array_equal(e.cpu().numpy()[:nb], oe[:nb])
        assert (e.cpu().numpy()[nb:] == -1).all()
        assert np.array_equal(cnt.cpu().numpy(), oc)
        if M:
            assert np.array_equal(os_[inv.cpu().numpy()], np.arange(M * k))


def test_align_skewed_and_single_expert(dev):
    M, k, E = 8192, 6, 64
    bias = synth.zipf_gate_bias(E, 1.2, 3.0)
    logits = torch.randn(M, E, generator=torch.Generator().manual_seed(1)) + bias
    _, ids = sr.route_from_logits(logits.to(dev), k)
    s, e, npost, cnt, _ = fm.moe_align_block_size(ids, 128, E, return_extra=True)
    os_, oe, on, oc = oracle.moe_align_block_size(ids.cpu(), 128, E)
    assert np.array_equal(s.cpu().numpy(), os_) and np.array_equal(cnt.cpu().numpy(), oc)
    assert (oc == 0).any() and oc.max() > 8 * oc.mean()
    one = torch.full((5000, 1), 3, dtype=torch.int32)
    s, e, npost = fm.moe_align_block_size(one.to(dev), 128, 8)
    assert np.array_equal(s.cpu().numpy(), oracle.moe_align_block_size(one, 128, 8)[0])


@pytest.mark.reads_status
def test_out_of_range_expert_id_is_reported_not_trapped(dev):
    from fast_route_b200 import _lib
    _lib.device_status()
    ids = torch.tensor([[0, 1], [9, 1], [2, -1]], dtype=torch.int32, device=dev)
    s, e, npost = fm.moe_align_block_size(ids, 4, 4)
    code, detail, _, count = _lib.device_status()
    assert code == 2 and count == 2
    assert int(npost.item()) == 12         # the three valid experts 0,1,2 still get their blocks
    assert _lib.device_status()[0] == 0    # reading clears


@pytest.mark.reads_status
def test_rejected_ids_contribute_zero_to_the_layer(dev):
    """An id outside [0, E) (for instance -1 for "expert held elsewhere") is reported and its slot adds nothing:
    the align stage marks its position -1, so the combine can never pick up a position an earlier call left in
    the reused workspace.  Checked with the cooperative and the cluster align kernel, on the row-block, the
    token-N and the split-K path, twice each."""
    import fast_route_b200 as fr
    from fast_route_b200 import _lib
    _lib.device_status()
    for M, H, I, E, k in ((5000, 256, 384, 8, 2), (3000, 256, 384, 8, 2), (200, 256, 384, 8, 2), (6, 512, 1024, 8, 2)):
        x, gate, w1, w2 = synth.moe_inputs(M, H, I, E, seed=17, dtype=torch.bfloat16, weight_std=0.05)
        xd, w1d, w2d = x.to(dev), w1.to(dev), w2.to(dev)
        tw, ti = fr.fused_route(xd, gate.to(dev), k)
        fr.fused_experts(xd, w1d, w2d, tw, ti)                      # fills the workspace with valid positions
        bad = ti.clone()
        bad[::3, 1] = -1
        bad[1::7, 0] = E + 3
        tw_masked = tw.clone()
        tw_masked[::3, 1] = 0.0
        tw_masked[1::7, 0] = 0.0
        good = torch.where((bad < 0) | (bad >= E), torch.zeros_like(ti), bad)
        want = fr.fused_experts(xd, w1d, w2d, tw_masked, good)      # same layer with the bad slots weighted zero
        assert _lib.device_status()[0] == 0
        for _ in range(2):
            got = fr.fused_experts(xd, w1d, w2d, tw, bad)
            code, _, _, count = _lib.device_status()
            assert code == 2 and count >= int(((bad < 0) | (bad >= E)).sum())
            assert torch.isfinite(got.float()).all()
            assert (got.float() - want.float()).abs().max().item() <= 2e-2


@pytest.mark.reads_status
def test_grid_barrier_wait_runs_out_and_is_reported(dev):
    """A bounded wait that expires: the count word of the align workspace's grid barrier is pre-set so that no
    arrival can complete it, and the poll budget word next to it is set to a few thousand polls (milliseconds).
    Every block must give up, the kernel must return, the status block must say 'wait expired', and after the
    workspace has been zeroed again the next call must be bit-exact.  Nothing traps and nothing waits without
    a limit."""
    from fast_route_b200 import _lib
    lib = _lib.load()
    _lib.device_status()
    M, k, E, bs = 16384, 2, 8, 64
    n = M * k
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, E, (M, k), generator=g, dtype=torch.int32)
    idd = ids.to(dev)
    s = torch.empty(n + E * (bs - 1), dtype=torch.int32, device=dev)
    e = torch.empty(n + E, dtype=torch.int32, device=dev)
    npost = torch.zeros(1, dtype=torch.int32, device=dev)
    ws = torch.zeros(lib.fr_align_workspace_bytes(E), dtype=torch.uint8, device=dev)

    def call():
        rc = lib.fr_align(_lib.ptr(idd), n, E, bs, _lib.ptr(s), s.numel(), _lib.ptr(e), e.numel(), _lib.ptr(npost),
                          None, None, _lib.ptr(ws), ws.numel(), _lib.stream_ptr(dev))
        assert rc == 0
    words = ws[:16].view(torch.int32)
    words[0] = 0x40000000           # arrivals can never reach "number of blocks - 1"
    words[3] = 5000                 # polls before a block gives up
    call()
    code, detail, _, count = _lib.device_status()      # synchronises: the kernel returned
    assert code == 1 and detail == 0x500 and count >= 1
    ws.zero_()
    call()
    os_, oe, on, _ = oracle.moe_align_block_size(ids, bs, E)
    assert _lib.device_status()[0] == 0
    assert int(npost.item()) == int(on[0]) and np.array_equal(s.cpu().numpy(), os_)


def _route_align_c_abi(dev, logits, k, bs, with_ws):
    """fr_route_align through the C ABI; with a workspace it is the single cooperative kernel."""
    from fast_route_b200 import _lib
    lib = _lib.load()
    M, E = logits.shape
    n = M * k
    lg = logits.to(dev)
    w = torch.empty(M, k, dtype=torch.float32, device=dev)
    ids = torch.empty(M, k, dtype=torch.int32, device=dev)
    s = torch.empty(n + E * (bs - 1), dtype=torch.int32, device=dev)
    e = torch.empty(n + E, dtype=torch.int32, device=dev)
    npost = torch.empty(1, dtype=torch.int32, device=dev)
    ws = torch.zeros(lib.fr_align_workspace_bytes(E), dtype=torch.uint8, device=dev) if with_ws else None
    for _ in range(3):      # the workspace must stay reusable call after call
        rc = lib.fr_route_align(_lib.ptr(lg), _lib.dtype_code(lg.dtype), M, E, lg.stride(0), lg.stride(1), k,
                                _lib.ptr(w), _lib.ptr(ids), bs, _lib.ptr(s), s.numel(), _lib.ptr(e), e.numel(),
                                _lib.ptr(npost), _lib.ptr(ws), ws.numel() if with_ws else 0, _lib.stream_ptr(dev))
        assert rc == 0
    return w.cpu().numpy(), ids.cpu().numpy(), s.cpu().numpy(), e.cpu().numpy(), int(npost.item())


@pytest.mark.parametrize("E,k,M,dt", [(8, 2, 16384, torch.float16), (64, 6, 16384, torch.float16),
                                      (128, 8, 16384, torch.float16), (128, 8, 16384, torch.bfloat16),
                                      (64, 6, 5000, torch.float16), (100, 4, 9000, torch.bfloat16),
                                      (256, 8, 3000, torch.float16), (8, 2, 300000, torch.float16),
                                      (16, 1, 20000, torch.float16)])
@pytest.mark.parametrize("with_ws", [True, False])
def test_route_align_fused_entry_point(dev, E, k, M, dt, with_ws):
    bs = 64
    logits = synth.routing_logits(M, E, k, seed=21, dtype=dt, dup_frac=0.05)
    w, ids, s, e, npost = _route_align_c_abi(dev, logits, k, bs, with_ws)
    ow, oi = oracle.topk_softmax(logits, k)
    os_, oe, on, _ = oracle.moe_align_block_size(oi, bs, E)
    assert np.array_equal(ids, oi) and np.array_equal(bits(w), bits(ow))
    assert npost == int(on[0]) and np.array_equal(s, os_)
    assert np.array_equal(e[:npost // bs], oe[:npost // bs]) and (e[npost // bs:] == -1).all()


@pytest.mark.parametrize("E,k", [(1, 1), (4, 2), (8, 2), (16, 4), (60, 6), (64, 6), (100, 3), (128, 8), (256, 8)])
@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16, torch.float32])
def test_softmax_then_topk_baseline_routing(dev, E, k, dt):
    """Routing of the reference's baseline layer (fast_route/fast_route/layers/vllm_route.py:72-84):
    bit-exact against the oracle recipe, with and without renormalisation, ties included."""
    from fast_route_b200.ops.vllm_route import topk_softmax
    for M in (1, 37, 4096):
        logits = synth.routing_logits(M, E, k, seed=E + k, dtype=dt, dup_frac=0.3)
        lg = logits.to(dev)
        for renorm in (False, True):
            w = torch.empty(M, k, dtype=torch.float32, device=dev)
            ids = torch.empty(M, k, dtype=torch.int32, device=dev)
            src = torch.empty(M, k, dtype=torch.int32, device=dev)
            topk_softmax(w, ids, src, lg, renormalize=renorm)
            ow, oi, osrc = oracle.softmax_topk(logits, k, renormalize=renorm)
            assert np.array_equal(ids.cpu().numpy(), oi), (E, k, M, renorm)
            assert np.array_equal(bits(w.cpu().numpy()), bits(ow)), (E, k, M, renorm)
            assert np.array_equal(src.cpu().numpy(), osrc)
        if M > 1:
            # the reference's tolerance for this op (tests/test_route.py:136-143) against library softmax
            p = torch.softmax(logits.float(), -1)
            ref = torch.gather(p, 1, torch.from_numpy(oi.astype(np.int64)))
            w = torch.empty(M, k, dtype=torch.float32, device=dev)
            ids = torch.empty(M, k, dtype=torch.int32, device=dev)
            topk_softmax(w, ids, None, lg)
            assert (w.cpu() - ref).abs().max() < 1e-6


def test_softmax_then_topk_strided_and_limits(dev):
    from fast_route_b200 import _lib
    from fast_route_b200.ops.vllm_route import topk_softmax
    base = synth.routing_logits(300, 128, 4, seed=9, dtype=torch.float32)
    view = base.to(dev)[:, ::2]                                 # element stride 2
    w = torch.empty(300, 4, dtype=torch.float32, device=dev)
    ids = torch.empty(300, 4, dtype=torch.int32, device=dev)
    topk_softmax(w, ids, None, view)
    ow, oi, _ = oracle.softmax_topk(base[:, ::2], 4)
    assert np.array_equal(ids.cpu().numpy(), oi) and np.array_equal(bits(w.cpu().numpy()), bits(ow))
    big = torch.zeros(4, 512, device=dev)
    with pytest.raises(_lib.FastRouteError):
        topk_softmax(torch.empty(4, 2, device=dev), torch.empty(4, 2, dtype=torch.int32, device=dev), None, big)
