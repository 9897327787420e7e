"""Expert-parallel bookkeeping on CPU ranks (gloo, world size 2 and 4): the split sizes,
the count exchange, the order of received rows and the return path of
fast_route_b200.parallel.ep, with the CPU oracle standing in for the device kernels.
The result must equal the single-process oracle layer on the concatenated batch.
Also here: the plan of the peer-memory path (every rank derives all positions from the gathered
histograms alone) and what the surviving rank sees when a peer leaves or never joins."""

import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, M, H, I, E, k, skew, out_q, fail_rank):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    try:
        import oracle
        from fast_route_b200 import synth
        from fast_route_b200.parallel import ep

        group = ep.ExpertParallelGroup(dist.group.WORLD, E)
        bias = synth.zipf_gate_bias(E, 1.2, 3.0) if skew else None
        x_all, gate, w1, w2 = synth.moe_inputs(M * world, H, I, E, seed=5, dtype=torch.float32, weight_std=0.1,
                                               gate_bias=bias)
        x = x_all[rank * M:(rank + 1) * M]
        lo, hi = group.local_expert_range()
        tw, ti, _ = oracle.route_from_hidden(x, gate, k)
        n = M * k
        sorted_ids, _, _, counts = oracle.moe_align_block_size(ti, 1, E)
        counts = torch.from_numpy(counts)
        if fail_rank == rank:
            counts = counts.clone()
            counts[0] += 1                      # an inconsistent histogram must be rejected locally
        recv_counts = ep.exchange_counts(counts, group)
        try:
            ep.validate_counts(counts, n, recv_counts)
        except RuntimeError as err:
            out_q.put((rank, "rejected", str(err)))
            return
        if fail_rank is not None:
            out_q.put((rank, "ok-peer", None))
            return
        in_splits = ep.send_splits(counts, world)
        out_splits = recv_counts.sum(dim=1).tolist()
        order = torch.from_numpy(sorted_ids[:n].astype(np.int64))
        send_rows = x[order // k].contiguous()
        send_w = torch.from_numpy(tw).reshape(-1)[order].contiguous()
        recv_rows = ep.all_to_all_rows(send_rows, in_splits, out_splits, group)
        recv_w = ep.all_to_all_rows(send_w, in_splits, out_splits, group)
        row_expert = ep.recv_row_experts(recv_counts)
        assert row_expert.numel() == recv_rows.shape[0]
        y = torch.zeros(recv_rows.shape[0], x.shape[1])
        for e in range(hi - lo):
            rows = (row_expert == e).nonzero().flatten()
            if rows.numel():
                h = oracle.silu_and_mul(recv_rows[rows] @ w1[lo + e].t())
                y[rows] = (h @ w2[lo + e].t()) * recv_w[rows, None]
        back = ep.all_to_all_rows(y, out_splits, in_splits, group)
        inv = np.empty(n, dtype=np.int64)
        inv[sorted_ids[:n]] = np.arange(n)
        out = back[torch.from_numpy(inv)].view(M, k, -1).sum(dim=1)
        ref, _, _ = oracle.moe_layer(x_all, gate, w1, w2, k)
        err = (out - ref[rank * M:(rank + 1) * M]).abs().max().item()
        out_q.put((rank, "done", err, in_splits, out_splits))
    finally:
        dist.destroy_process_group()


def _run(world, M, H, I, E, k, skew=False, fail_rank=None):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, M, H, I, E, k, skew, q, fail_rank))
             for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    return sorted(results)


@pytest.mark.parametrize("world,E,k,skew", [(2, 8, 2, False), (4, 8, 2, False), (2, 16, 4, True)])
def test_ep_exchange_reproduces_single_process_layer(world, E, k, skew):
    results = _run(world, M=24, H=32, I=48, E=E, k=k, skew=skew)
    total_in = total_out = 0
    for rank, tag, err, in_splits, out_splits in results:
        assert tag == "done" and err < 1e-5, (rank, err)
        assert sum(in_splits) == 24 * k
        total_in += sum(in_splits)
        total_out += sum(out_splits)
    assert total_in == total_out == world * 24 * k


def test_ep_inconsistent_counts_rejected_before_payload():
    results = _run(2, M=8, H=32, I=16, E=4, k=2, fail_rank=1)
    tags = {r[0]: r[1] for r in results}
    assert tags[1] == "rejected" and tags[0] == "ok-peer"


def _reject_together_main(rank, world, port, out_q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import datetime
    sys.path.insert(0, ROOT)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    try:
        from fast_route_b200.parallel import ep
        group = ep.ExpertParallelGroup(dist.group.WORLD, 4)
        counts = torch.tensor([2, 2, 2, 2], dtype=torch.int32)
        if rank == 1:
            counts[0] += 1                               # only rank 1's histogram is inconsistent
        allc = ep.gather_counts(counts, group)
        try:
            ep.validate_all_counts(allc, 8)
            out_q.put((rank, "accepted"))
        except RuntimeError as err:
            out_q.put((rank, "rejected: " + str(err)))
    finally:
        dist.destroy_process_group()


def test_ep_inconsistent_counts_rejected_by_every_rank_together():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_reject_together_main, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=60) for _ in range(world))
    for p in procs:
        p.join(timeout=30)
        assert p.exitcode == 0
    assert all(v.startswith("rejected") and "rank 1" in v for v in results.values()), results


def test_ep_helpers():
    from fast_route_b200.parallel import ep
    rc = torch.tensor([[2, 0], [1, 3]], dtype=torch.int32)
    assert ep.recv_row_experts(rc).tolist() == [0, 0, 0, 1, 1, 1]
    assert ep.send_splits(torch.tensor([1, 2, 3, 4]), 2) == [3, 7]
    with pytest.raises(RuntimeError):
        ep.validate_counts(torch.tensor([1, 2]), 4, torch.tensor([[0]]))
    ep.validate_all_counts(torch.tensor([[1, 3], [2, 2]]), 4)
    with pytest.raises(RuntimeError, match="rank 1"):
        ep.validate_all_counts(torch.tensor([[1, 3], [2, 3]]), 4)
    with pytest.raises(RuntimeError):
        ep.validate_all_counts(torch.tensor([[5, -1], [2, 2]]), 4)


# ------------------------------------------------------------------------------------
# peer-memory path: positions derived from the all-gathered histograms (ep.plan_tables)
# ------------------------------------------------------------------------------------
def _plan_rank_main(rank, world, port, M, H, I, E, k, skew, out_q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=30))
    try:
        import oracle
        from fast_route_b200 import synth
        from fast_route_b200.parallel import ep

        group = ep.ExpertParallelGroup(dist.group.WORLD, E)
        El = group.experts_per_rank
        bias = synth.zipf_gate_bias(E, 1.2, 3.0) if skew else None
        x_all, gate, w1, w2 = synth.moe_inputs(M * world, H, I, E, seed=5, dtype=torch.float32, weight_std=0.1,
                                               gate_bias=bias)
        x = x_all[rank * M:(rank + 1) * M].contiguous()
        lo, hi = group.local_expert_range()
        tw, ti, _ = oracle.route_from_hidden(x, gate, k)
        n = M * k
        sorted_ids, _, _, counts = oracle.moe_align_block_size(ti, 1, E)
        inv = np.empty(n, dtype=np.int64)
        inv[sorted_ids[:n]] = np.arange(n)
        # the one metadata collective: everybody's histogram
        all_counts = torch.empty(world, E, dtype=torch.int32)
        dist.all_gather_into_tensor(all_counts.view(-1), torch.from_numpy(counts.astype(np.int32)))
        plan = ep.plan_tables(all_counts.numpy(), rank)
        # "peer memory": what the kernels would read from the other ranks' regions
        xs = [torch.empty_like(x) for _ in range(world)]
        sorts = [torch.empty(n, dtype=torch.int64) for _ in range(world)]
        tws = [torch.empty(n) for _ in range(world)]
        dist.all_gather(xs, x)
        dist.all_gather(sorts, torch.from_numpy(sorted_ids[:n].astype(np.int64)))
        dist.all_gather(tws, torch.from_numpy(np.ascontiguousarray(tw)).reshape(-1).float())
        num_post = plan["num_post"]
        y = torch.zeros(max(num_post, 1), x.shape[1])
        filled = np.zeros(max(num_post, 1), dtype=bool)
        for i in range(El * world):
            j, s_ = divmod(i, world)
            for off in range(int(plan["seg_count"][i])):
                row = int(plan["seg_start"][i]) + off
                sid = int(sorts[s_][int(plan["seg_src_off"][i]) + off])
                assert int(plan["expert_ids"][row // 128]) == j and not filled[row]
                filled[row] = True
                h = oracle.silu_and_mul(xs[s_][sid // k][None] @ w1[lo + j].t())
                y[row] = (h @ w2[lo + j].t())[0] * tws[s_][sid]
        ys = [torch.empty(0)] * world
        sizes = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(sizes, torch.tensor([y.shape[0]]))
        ys = [torch.empty(int(sz), x.shape[1]) for sz in sizes]
        for src in range(world):                      # variable sizes: one broadcast per owner
            buf = y if src == rank else ys[src]
            dist.broadcast(buf, src=src)
            ys[src] = buf
        out = torch.zeros(M, x.shape[1])
        for t in range(M):
            for jj in range(k):
                e = int(ti[t, jj])
                out[t] += ys[e // El][int(plan["comb_base"][e]) + int(inv[t * k + jj])]
        ref, _, _ = oracle.moe_layer(x_all, gate, w1, w2, k)
        err = (out - ref[rank * M:(rank + 1) * M]).abs().max().item()
        out_q.put((rank, err, int(filled.sum()), int(all_counts[:, lo:hi].sum())))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,E,k,skew", [(2, 8, 2, False), (4, 8, 2, False), (2, 16, 4, True), (4, 4, 1, False)])
def test_ep_plan_from_gathered_histograms_reproduces_single_process_layer(world, E, k, skew):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_plan_rank_main, args=(r, world, port, 24, 32, 48, E, k, skew, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err, rows_filled, rows_expected in sorted(results):
        assert err < 1e-5, (rank, err)
        assert rows_filled == rows_expected


def test_plan_tables_small_example():
    from fast_route_b200.parallel import ep
    c = np.array([[3, 0, 5, 2], [1, 4, 0, 130]])
    p0, p1 = ep.plan_tables(c, 0), ep.plan_tables(c, 1)
    assert p0["seg_start"].tolist() == [0, 3, 128, 128, 256] and p0["seg_count"].tolist() == [3, 1, 0, 4]
    assert p0["seg_src_off"].tolist() == [0, 0, 3, 1] and p0["comb_base"].tolist() == [0, 125, -3, 120]
    assert p1["num_post"] == 384 and p1["expert_ids"].tolist() == [0, 1, 1]
    assert p1["seg_start"].tolist() == [0, 5, 128, 130, 384] and p1["comb_base"].tolist() == [3, 127, 0, 125]


def test_plan_tables_agree_between_token_owner_and_expert_owner():
    """The invariant the peer-memory path rests on: from the same histogram matrix, the token owner's `comb_base`
    and the expert owner's segment table name the same row for every assignment; segments of one owner are
    disjoint, ordered and inside the padded extent of their expert."""
    from fast_route_b200.parallel import ep
    rng = np.random.default_rng(7)
    for world, E in ((2, 8), (4, 8), (8, 8), (8, 64), (4, 12), (1, 4)):
        for trial in range(6):
            c = rng.integers(0, 400, size=(world, E))
            c[rng.random((world, E)) < 0.2] = 0                     # experts a rank sends nothing to
            if trial == 0:
                c[:, 0] = 0                                          # an expert nobody uses
            El = E // world
            plans = [ep.plan_tables(c, r) for r in range(world)]
            for owner in range(world):
                po = plans[owner]
                end_prev = 0
                for j in range(El):
                    e = owner * El + j
                    tot = int(c[:, e].sum())
                    first = int(po["seg_start"][j * world])
                    assert first % 128 == 0 and first >= end_prev
                    for s_ in range(world):
                        i = j * world + s_
                        assert int(po["seg_count"][i]) == c[s_, e]
                        assert int(po["seg_src_off"][i]) == int(c[s_, :e].sum())
                        assert int(po["seg_start"][i]) == first + int(c[:s_, e].sum())
                        # the token owner s_ finds its assignments to e exactly there
                        selfpre = int(c[s_, :e].sum())
                        assert int(plans[s_]["comb_base"][e]) + selfpre == int(po["seg_start"][i])
                    end_prev = first + (tot + 127) // 128 * 128
                    assert (po["expert_ids"][first // 128:end_prev // 128] == j).all()
                assert po["num_post"] == end_prev == int(po["seg_start"][El * world])


# ------------------------------------------------------------------------------------
# a peer that leaves between steps, a peer that never joins: the survivor gets an exception
# ------------------------------------------------------------------------------------
def _leaver_main(rank, world, port, mode, out_q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import datetime
    import time
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    counts = torch.full((4,), rank + 1, dtype=torch.int32)
    allc = torch.empty(world, 4, dtype=torch.int32)
    dist.all_gather_into_tensor(allc.view(-1), counts)          # step 1: everybody is there
    assert allc[:, 0].tolist() == list(range(1, world + 1))
    if rank == world - 1:
        if mode == "exit":
            dist.destroy_process_group()                       # leaves between steps, nothing in flight
            out_q.put((rank, "left"))
            return
        time.sleep(8)                                          # never joins step 2 within the group's timeout
        out_q.put((rank, "late"))
        return
    try:
        dist.all_gather_into_tensor(allc.view(-1), counts)      # step 2
        out_q.put((rank, "completed"))
    except Exception as err:                                   # noqa: BLE001 - any exception is the point
        out_q.put((rank, "raised:" + type(err).__name__))


@pytest.mark.parametrize("mode", ["exit", "timeout"])
def test_ep_peer_leaves_or_never_joins(mode):
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_leaver_main, args=(r, world, port, mode, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=60) for _ in range(world))
    for p in procs:
        p.join(timeout=30)
    assert results[0].startswith("raised:"), results
    assert results[1] in ("left", "late")
