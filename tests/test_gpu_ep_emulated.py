"""The expert-parallel kernels (plan, NVLink gather, grouped GEMMs, combine; fr_ep_experts / fr_ep_combine)
on ONE GPU: W ranks are emulated by W peer regions in the same device memory that share one pointer
table, and the stages run rank after rank in one process (no kernel ever waits for another).  The result
must equal the single-GPU layer on the concatenated batch, bit for bit when both run the same GEMM kernel.
The real multi-GPU run (symmetric memory + NCCL) is in test_gpu_ep.py."""

import numpy as np
import pytest
import torch

import fast_route_b200 as fr
from fast_route_b200 import _lib, synth
from fast_route_b200.parallel import ep

pytestmark = pytest.mark.gpu


def _run_emulated(dev, W, M, H, I, E, k, skew, seed=7):
    bias = synth.zipf_gate_bias(E, 1.2, 3.0) if skew else None
    x_all, gate, w1, w2 = synth.moe_inputs(M * W, H, I, E, seed=seed, dtype=torch.bfloat16, weight_std=0.05,
                                           gate_bias=bias)
    Hx = x_all.shape[1]
    x_all, gate, w1, w2 = x_all.to(dev), gate.to(dev), w1.to(dev), w2.to(dev)
    El = E // W
    regions = ep.PeerRegion.emulated(W, E, M, Hx, k, torch.bfloat16, dev)
    states = [ep.ep_route_stage(regions[r], x_all[r * M:(r + 1) * M], gate, k, E) for r in range(W)]
    all_counts = torch.stack([s.counts for s in states]).contiguous()
    for r in range(W):
        ep.ep_experts_stage(regions[r], r, all_counts, w1[r * El:(r + 1) * El], w2[r * El:(r + 1) * El], E)
    outs = [ep.ep_combine_stage(regions[r], states[r], E) for r in range(W)]
    torch.cuda.synchronize()
    _lib.raise_on_device_error()
    ref, tw, ti = fr.fused_moe(x_all, gate, w1, w2, k, return_routing=True)
    return torch.cat(outs), ref, regions, states, all_counts, ti


@pytest.mark.parametrize("W,M,H,I,E,k,skew,exact", [(2, 4096, 2048, 1024, 8, 2, False, True),
                                                    (4, 2048, 4096, 512, 8, 2, False, True),
                                                    (2, 8192, 4096, 512, 8, 2, False, True),
                                                    (8, 1024, 512, 768, 8, 2, False, False),
                                                    (4, 300, 256, 384, 16, 4, True, False),
                                                    (2, 3, 512, 1024, 8, 2, False, False),
                                                    (8, 512, 512, 256, 64, 6, True, False)])
def test_ep_kernels_on_emulated_ranks_match_single_gpu_layer(dev, W, M, H, I, E, k, skew, exact):
    """`exact` cases give every expert enough rows that neither side uses split-K or the token-N kernel, and both
    batch sizes select the tensor-core router: the same kernels see the same rows and the outputs are
    bit-identical.  The others are held to the layer tolerance (different fp32 summation order)."""
    out, ref, regions, states, all_counts, ti = _run_emulated(dev, W, M, H, I, E, k, skew)
    if exact:
        assert torch.equal(out, ref)
    else:
        err = (out.float() - ref.float()).abs().max().item()
        assert err <= 2e-2 + ref.float().abs().max().item() * 2.0 ** -7, err
    # routing of the sharded run is the single-GPU routing of the same tokens (the router kernel is picked by the
    # batch size and the two kernels add in different orders, so outside the exact cases a near tie may flip)
    same = (torch.cat([s.ids for s in states]) == ti).all(dim=1).float().mean().item()
    assert same == 1.0 if exact else same > 0.995
    # the device plan equals its host mirror
    for r in range(W):
        plan = ep.plan_tables(all_counts.cpu().numpy(), r)
        assert np.array_equal(regions[r].comb_base.cpu().numpy(), plan["comb_base"])


def test_ep_emulated_twice_and_smaller_batch_in_same_regions(dev):
    """Regions are reused call after call and may hold fewer tokens than they were sized for."""
    W, M, H, I, E, k = 2, 2048, 4096, 512, 8, 2
    x_all, gate, w1, w2 = synth.moe_inputs(M * W, H, I, E, seed=3, dtype=torch.bfloat16, weight_std=0.05)
    x_all, gate, w1, w2 = x_all.to(dev), gate.to(dev), w1.to(dev), w2.to(dev)
    El = E // W
    regions = ep.PeerRegion.emulated(W, E, M, H, k, torch.bfloat16, dev)
    for m in (M, 1000, M):
        xs = [x_all[r * M:r * M + m] for r in range(W)]
        states = [ep.ep_route_stage(regions[r], xs[r], gate, k, E) for r in range(W)]
        all_counts = torch.stack([s.counts for s in states]).contiguous()
        for r in range(W):
            ep.ep_experts_stage(regions[r], r, all_counts, w1[r * El:(r + 1) * El], w2[r * El:(r + 1) * El], E)
        out = torch.cat([ep.ep_combine_stage(regions[r], states[r], E) for r in range(W)])
        ref = fr.fused_moe(torch.cat(xs), gate, w1, w2, k)
        if m == M:
            assert torch.equal(out, ref)
        else:    # the small batch takes split-K on the single GPU: same values up to the fp32 summation order
            assert (out.float() - ref.float()).abs().max().item() <= 2e-2 + ref.float().abs().max().item() * 2.0 ** -7


@pytest.mark.reads_status
def test_ep_receive_capacity_overflow_is_reported_not_written(dev):
    """A y buffer smaller than what arrives: the plan clamps to the capacity, reports status 4 and nothing is
    written past the buffer (the rows that did not fit contribute zero)."""
    lib = _lib.load()
    _lib.device_status()
    W, M, H, I, E, k = 2, 512, 256, 128, 2, 1
    regions = ep.PeerRegion.emulated(W, E, M, H, k, torch.bfloat16, dev)
    x_all, gate, w1, w2 = synth.moe_inputs(M * W, H, I, E, seed=1, dtype=torch.bfloat16, weight_std=0.05)
    gate = gate.clone()
    gate[:, 1] = -gate[:, 0]
    x_all, gate, w1, w2 = x_all.to(dev), gate.to(dev), w1.to(dev), w2.to(dev)
    states = [ep.ep_route_stage(regions[r], x_all[r * M:(r + 1) * M], gate, k, E) for r in range(W)]
    all_counts = torch.stack([s.counts for s in states]).contiguous()
    r = 0
    small_rows = 256                                   # capacity: two blocks, far fewer than the ~512 rows that arrive
    guard = regions[r].y[small_rows:small_rows + 8].clone()
    ws = _lib.workspace(lib.fr_ep_workspace_bytes(small_rows, H, I, E), dev, "ep_small")
    comb = torch.empty(E, dtype=torch.int32, device=dev)
    rc = lib.fr_ep_experts(ep.ctypes_ptr(regions[r].base_ptrs), W, r, regions[r].x_off, H, M, regions[r].sorted_off,
                           regions[r].tw_off, M * k, k, _lib.ptr(all_counts), _lib.ptr(w1[:1]), _lib.ptr(w2[:1]), 1, H,
                           I, E, _lib.ptr(regions[r].y), small_rows, _lib.ptr(comb), 7, _lib.ptr(ws), ws.numel(),
                           _lib.stream_ptr(dev))
    assert rc == 0
    code, detail, _, _ = _lib.device_status()
    assert code == 4 and detail > small_rows
    assert torch.equal(regions[r].y[small_rows:small_rows + 8], guard)
