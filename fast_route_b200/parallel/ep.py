"""Expert parallelism for the MoE layer: one process per GPU, experts sharded evenly,
tokens data-parallel, NCCL all-to-all dispatch and combine over NVLink.

The reference is single-GPU (it has no collective call site); this module adds the
sharded form of its layer ``fast_route/fast_route/layers/stable_route.py:10-102``.
Rank r of W owns experts ``[r*E/W, (r+1)*E/W)`` and brings its own batch of tokens.

Per call, on every rank:
  1. local fused router (global expert ids);
  2. local align with block size 1: a stable sort of the assignments by expert.  Experts
     are contiguous per rank, so the sorted order is already grouped by destination rank
     and the per-expert histogram gives the all-to-all split sizes;
  3. a small all-gather of the per-expert counts (every rank validates the same matrix);
  4. the permute kernel gathers token rows straight into the send buffer; NCCL all-to-all
     moves rows (and their routing weights) to the expert owners;
  5. the owner runs the expert pipeline on the received rows (align by local expert,
     grouped GEMMs, routed weight applied in the second GEMM's epilogue) and leaves the
     results in arrival order, which is the send order of the return all-to-all;
  6. the source rank sums the k returned rows of every token in slot order.
Row results do not depend on where a row is computed, and the final sum keeps the slot
order of the single-GPU layer.
"""

from __future__ import annotations

from typing import List, Tuple

import torch
import torch.distributed as dist


class ExpertParallelGroup:
    """A process group plus the even expert partition over its ranks."""

    def __init__(self, pg, num_experts: int):
        self.pg = pg
        self.world = dist.get_world_size(pg)
        self.rank = dist.get_rank(pg)
        if num_experts % self.world != 0:
            raise ValueError(f"{num_experts} experts do not divide over {self.world} ranks")
        self.num_experts = num_experts
        self.experts_per_rank = num_experts // self.world

    def local_expert_range(self) -> Tuple[int, int]:
        lo = self.rank * self.experts_per_rank
        return lo, lo + self.experts_per_rank


# ------------------------------------------------------------------------------------
# host-side bookkeeping (plain tensors; shared by the GPU path and the CPU-rank tests)
# ------------------------------------------------------------------------------------
def send_splits(counts: torch.Tensor, world: int) -> List[int]:
    """Rows this rank sends to each rank, from its per-expert histogram ``counts[E]``."""
    return counts.view(world, -1).sum(dim=1).tolist()


def exchange_counts(counts: torch.Tensor, group: ExpertParallelGroup) -> torch.Tensor:
    """All-to-all of the histograms: returns ``recv_counts[W, E/W]`` where row s holds how
    many rows source rank s sends for each of this rank's experts."""
    send = counts.view(group.world, group.experts_per_rank).contiguous()
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group.pg)
    return recv


def gather_counts(counts: torch.Tensor, group: ExpertParallelGroup) -> torch.Tensor:
    """All-gather of the histograms: ``all_counts[W, E]``, identical on every rank, so that every rank validates the
    same data and all of them accept or reject a step together (a rank that raised alone would leave its peers in
    a collective that never completes)."""
    out = torch.empty(group.world * counts.numel(), dtype=counts.dtype, device=counts.device)
    dist.all_gather_into_tensor(out, counts.contiguous(), group=group.pg)
    return out.view(group.world, -1)


def validate_all_counts(all_counts: torch.Tensor, n_assignments: int) -> None:
    """Rejects inconsistent histograms before any payload collective; same verdict on every rank."""
    if int(all_counts.min()) < 0:
        raise RuntimeError("negative row count in the gathered expert histograms")
    sums = all_counts.sum(dim=1)
    if int((sums != n_assignments).sum()):
        bad = int((sums != n_assignments).nonzero()[0])
        raise RuntimeError(f"expert histogram of rank {bad} sums to {int(sums[bad])}, expected {n_assignments}")


def validate_counts(counts: torch.Tensor, n_assignments: int, recv_counts: torch.Tensor) -> None:
    """Rejects inconsistent split sizes before any payload collective is issued."""
    if int(counts.sum()) != n_assignments or int(counts.min()) < 0:
        raise RuntimeError(f"expert histogram sums to {int(counts.sum())}, expected {n_assignments}")
    if int(recv_counts.min()) < 0:
        raise RuntimeError("negative row count received from a peer")


def recv_row_experts(recv_counts: torch.Tensor, total: int = None) -> torch.Tensor:
    """Local expert id of every received row.  Rows arrive grouped by source rank and,
    inside a source's segment, by expert in ascending order.  ``total`` (the number of
    received rows, known on the host from the split sizes) avoids a device synchronisation."""
    world, epr = recv_counts.shape
    pattern = torch.arange(epr, dtype=torch.int32, device=recv_counts.device).repeat(world)
    return torch.repeat_interleave(pattern, recv_counts.reshape(-1).long(), output_size=total)


def all_to_all_rows(send: torch.Tensor, in_splits: List[int], out_splits: List[int], group: ExpertParallelGroup,
                    async_op: bool = False):
    """Variable-size all-to-all of rows.  With ``async_op`` returns (recv, work) and the caller
    waits on ``work`` before touching ``recv``."""
    recv = torch.empty((sum(out_splits),) + tuple(send.shape[1:]), dtype=send.dtype, device=send.device)
    work = dist.all_to_all_single(recv, send, output_split_sizes=out_splits, input_split_sizes=in_splits,
                                  group=group.pg, async_op=async_op)
    return (recv, work) if async_op else recv


def chunk_bounds(M: int, chunks: int) -> List[Tuple[int, int]]:
    chunks = max(1, min(chunks, M)) if M > 0 else 1
    step = (M + chunks - 1) // chunks
    return [(lo, min(M, lo + step)) for lo in range(0, max(M, 1), step)] if M > 0 else [(0, 0)]


# ------------------------------------------------------------------------------------
# the layer
# ------------------------------------------------------------------------------------
def fused_moe_ep(hidden_states: torch.Tensor, gate: torch.Tensor, w1_local: torch.Tensor, w2_local: torch.Tensor,
                 topk: int, group: ExpertParallelGroup, renormalize: bool = True, chunks: int = None) -> torch.Tensor:
    """Expert-parallel MoE layer.  ``hidden_states[M,H]`` is this rank's batch, ``gate[H,E]`` is
    replicated, ``w1_local[E/W,2I,H]`` / ``w2_local[E/W,H,I]`` are this rank's experts.
    Returns this rank's ``[M,H]`` output.

    ``chunks`` > 1 (every rank must use the same number) cuts the batch into token ranges that
    move through dispatch -> experts -> return as a pipeline with asynchronous all-to-alls.
    Tokens are independent, so chunking does not change any result.  The default is 1: measured
    on B200, NCCL's all-to-all kernels do not overlap the persistent expert GEMMs (those hold
    every SM's shared memory), so chunking only adds launches.
    """
    from .. import _lib
    from ..ops import fused_moe as fm
    from ..ops.stable_route import fused_route

    lib = _lib.load()
    dev = hidden_states.device
    M, H = hidden_states.shape
    El, N2, _ = w1_local.shape
    I = N2 // 2
    E = group.num_experts
    assert El == group.experts_per_rank and gate.shape == (H, E)
    if chunks is None:
        chunks = 1
    bounds = chunk_bounds(M, chunks)
    dt = _lib.dtype_code(hidden_states.dtype)
    out = torch.empty_like(hidden_states)

    # stage 1: routing and histograms of every chunk, then ONE host sync for all split sizes
    st = []
    for lo, hi in bounds:
        xc = hidden_states[lo:hi]
        tw, ti = fused_route(xc, gate, topk, renormalize=renormalize)
        sorted_ids, _, _, counts, inv_pos = fm.moe_align_block_size(ti, 1, E, return_extra=True)
        allc = gather_counts(counts, group)            # [W, E], the same on every rank
        elo, ehi = group.local_expert_range()
        st.append({"x": xc, "tw": tw, "sorted": sorted_ids, "inv": inv_pos, "counts": counts, "all_counts": allc,
                   "recv_counts": allc[:, elo:ehi].contiguous(), "n": (hi - lo) * topk})
    counts_h = torch.stack([c["counts"] for c in st]).cpu()
    recv_h = torch.stack([c["recv_counts"] for c in st]).cpu()
    all_h = torch.stack([c["all_counts"] for c in st]).cpu()

    # stage 2: pack rows in destination order straight into the send buffer, start the dispatch
    for i, c in enumerate(st):
        n = c["n"]
        validate_all_counts(all_h[i], n)               # every rank sees the same matrix: all raise or none
        c["in_splits"] = send_splits(counts_h[i], group.world)
        c["out_splits"] = recv_h[i].sum(dim=1).tolist()
        num_post = torch.tensor([n], dtype=torch.int32, device=dev)
        send_rows = torch.empty(n, H, dtype=hidden_states.dtype, device=dev)
        if n:
            rc = lib.fr_permute_rows(_lib.ptr(c["x"]), dt, H, c["x"].stride(0), _lib.ptr(c["sorted"]),
                                     _lib.ptr(num_post), n, topk, n, _lib.ptr(send_rows), H, _lib.stream_ptr(dev))
            _lib.check(rc, "fr_permute_rows")
        send_w = c["tw"].reshape(-1)[c["sorted"][:n].long()]
        c["recv_rows"], c["work_rows"] = all_to_all_rows(send_rows, c["in_splits"], c["out_splits"], group, True)
        c["recv_w"], c["work_w"] = all_to_all_rows(send_w, c["in_splits"], c["out_splits"], group, True)

    # stage 3: experts on the received rows (arrival order is kept), start the return
    for c in st:
        c["work_rows"].wait()
        c["work_w"].wait()
        R = c["recv_rows"].shape[0]
        y = torch.empty(R, H, dtype=hidden_states.dtype, device=dev)
        if R:
            row_expert = recv_row_experts(c["recv_counts"], R)
            nbytes = lib.fr_moe_experts_workspace_bytes(R, H, I, El)
            ws = _lib.workspace(nbytes, dev, "ep_experts")
            rc = lib.fr_moe_experts(_lib.ptr(c["recv_rows"]), _lib.ptr(row_expert), _lib.ptr(c["recv_w"]),
                                    _lib.ptr(w1_local), _lib.ptr(w2_local), dt, R, H, I, El, _lib.ptr(y), _lib.ptr(ws),
                                    ws.numel(), _lib.stream_ptr(dev))
            _lib.check(rc, "fr_moe_experts")
        c["back"], c["work_back"] = all_to_all_rows(y, c["out_splits"], c["in_splits"], group, True)

    # stage 4: rows are back in this rank's sorted order; sum the k rows of every token in slot order
    for (lo, hi), c in zip(bounds, st):
        c["work_back"].wait()
        if hi > lo:
            fm.combine(c["back"], c["inv"], hi - lo, topk, out=out[lo:hi])
    return out


# ------------------------------------------------------------------------------------
# the layer over peer memory: dispatch fused into the gather, return fused into the combine,
# no sizes on the host
# ------------------------------------------------------------------------------------
BLOCK_M = 128


def plan_tables(all_counts, rank: int, block: int = BLOCK_M):
    """Host mirror (numpy) of the device plan of ``fr_ep_experts``: from ``all_counts[W][E]`` (tokens of rank s
    for expert e) the tables of rank ``rank``.  Returns a dict with

    * ``seg_start[El*W+1]``, ``seg_count[El*W]``, ``seg_src_off[El*W]`` - as expert owner: segment (j, s) = the rows
      of source rank s for local expert j; first row in the expert-sorted operand (experts padded to ``block`` rows,
      sources in rank order inside an expert), length, and first entry in source s's expert-sorted list;
    * ``num_post`` - rows of the operand in use; ``expert_ids[num_post/block]``;
    * ``comb_base[E]`` - as token owner: this rank's assignment at position q of its own sorted list, going to
      expert e, lands in row ``comb_base[e] + q`` of the y buffer of rank ``e // El``.

    Used by the CPU-rank tests and to check the kernel; the GPU path never calls it."""
    import numpy as np
    c = np.maximum(np.asarray(all_counts, dtype=np.int64), 0)
    W, E = c.shape
    El = E // W
    tot = c.sum(0)
    padded = (tot + block - 1) // block * block
    start = np.zeros(E, dtype=np.int64)
    for o in range(W):
        start[o * El:(o + 1) * El] = np.concatenate([[0], np.cumsum(padded[o * El:(o + 1) * El])[:-1]])
    below = c[:rank].sum(0)
    selfpre = np.concatenate([[0], np.cumsum(c[rank])[:-1]])
    lo = rank * El
    num_post = int(padded[lo:lo + El].sum())
    seg_start = np.zeros(El * W + 1, dtype=np.int64)
    seg_count = np.zeros(El * W, dtype=np.int64)
    seg_src_off = np.zeros(El * W, dtype=np.int64)
    for j in range(El):
        for s_ in range(W):
            i = j * W + s_
            seg_start[i] = start[lo + j] + c[:s_, lo + j].sum()
            seg_count[i] = c[s_, lo + j]
            seg_src_off[i] = c[s_, :lo + j].sum()
    seg_start[El * W] = num_post
    expert_ids = np.repeat(np.arange(El), padded[lo:lo + El] // block)
    return {"seg_start": seg_start, "seg_count": seg_count, "seg_src_off": seg_src_off, "num_post": num_post,
            "expert_ids": expert_ids, "comb_base": start + below - selfpre}


def _round_up(a: int, b: int) -> int:
    return (a + b - 1) // b * b


class PeerRegion:
    """The peer-readable memory of one rank, one allocation with the same layout on every rank:
    ``x[rows,H]`` its tokens, ``y[y_rows,H]`` the results of its own experts in expert-sorted order,
    ``sorted[n]`` its assignments ordered by expert, ``tw[n]`` its routing weights (n = rows * topk).
    ``base_ptrs`` is the device address of the table of every rank's region base.

    ``PeerRegion(group, ...)`` allocates symmetric memory and is collective (every rank, same arguments).
    ``PeerRegion.emulated(world, ...)`` builds ``world`` regions in ordinary memory of ONE GPU that share a pointer
    table: the same kernels then run rank after rank in one process (tests on a single-GPU box)."""

    def __init__(self, group: ExpertParallelGroup, rows: int, H: int, topk: int, dtype, device, _buf=None,
                 _table=None, _world=None, _experts_per_rank=None):
        from .. import _lib
        lib = _lib.load()
        world = group.world if group is not None else _world
        epr = group.experts_per_rank if group is not None else _experts_per_rank
        self.group, self.rows, self.H, self.topk, self.dtype, self.world = group, rows, H, topk, dtype, world
        self.n = rows * topk
        esz = torch.empty(0, dtype=dtype).element_size()
        # worst case: every assignment of every rank lands on this rank
        self.y_rows = int(lib.fr_moe_experts_rows_cap(self.n * world, epr))
        self.x_off = 0
        self.y_off = _round_up(rows * H * esz, 1024)
        self.sorted_off = self.y_off + _round_up(self.y_rows * H * esz, 1024)
        self.tw_off = self.sorted_off + _round_up(self.n * 4, 1024)
        self.nbytes = self.tw_off + _round_up(self.n * 4, 1024)
        if _buf is None:
            import os
            # symmetric memory would otherwise bind the buffers to an NVLink multicast object, which nothing here
            # uses (peer memory is only read by plain loads) and which must not outlive a rank that dies
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            import torch.distributed._symmetric_memory as symm_mem
            self.buf = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=device)
            self.handle = symm_mem.rendezvous(self.buf, group.pg)
            self.base_ptrs = int(self.handle.buffer_ptrs_dev)
        else:
            self.buf, self.handle, self.base_ptrs = _buf, None, int(_table.data_ptr())
            self._table = _table
        b = self.buf
        self.x = b[self.x_off:self.x_off + rows * H * esz].view(dtype).view(rows, H)
        self.y = b[self.y_off:self.y_off + self.y_rows * H * esz].view(dtype).view(self.y_rows, H)
        self.sorted = b[self.sorted_off:self.sorted_off + self.n * 4].view(torch.int32)
        self.tw = b[self.tw_off:self.tw_off + self.n * 4].view(torch.float32)
        self.comb_base = None
        self.sync_word = torch.zeros(1, dtype=torch.int32, device=device)

    @classmethod
    def emulated(cls, world: int, num_experts: int, rows: int, H: int, topk: int, dtype, device):
        from .. import _lib
        epr = num_experts // world
        esz = torch.empty(0, dtype=dtype).element_size()
        n = rows * topk
        y_rows = int(_lib.load().fr_moe_experts_rows_cap(n * world, epr))
        nbytes = _round_up(rows * H * esz, 1024) + _round_up(y_rows * H * esz, 1024) + 2 * _round_up(n * 4, 1024)
        table = torch.zeros(world, dtype=torch.int64, device=device)
        regions = []
        for r in range(world):
            buf = torch.zeros(nbytes + 1024, dtype=torch.uint8, device=device)
            off = (-buf.data_ptr()) % 1024
            buf = buf[off:off + nbytes]
            table[r] = buf.data_ptr()
            regions.append(cls(None, rows, H, topk, dtype, device, _buf=buf, _table=table, _world=world,
                               _experts_per_rank=epr))
        return regions


def _mark(timers, name, fn):
    """Runs fn(); with a timers list, brackets it with CUDA events on the current stream and appends (name, start, end)."""
    if timers is None:
        return fn()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    r = fn()
    b.record()
    timers.append((name, a, b))
    return r


class RouteState:
    """What a rank keeps between the stages of one call."""
    __slots__ = ("M", "ids", "inv_pos", "counts")


def ep_route_stage(region: PeerRegion, hidden_states: torch.Tensor, gate: torch.Tensor, topk: int,
                   num_experts: int, renormalize: bool = True, timers=None, copy_in: bool = True) -> RouteState:
    """Stage 1 (local): tokens into the region, fused router with the weights written straight into the region,
    align with block size 1 whose sorted list lands in the region.  Returns ids, positions and the histogram."""
    from .. import _lib
    lib = _lib.load()
    dev = hidden_states.device
    M, H = hidden_states.shape
    E = num_experts
    assert M <= region.rows and H == region.H and topk == region.topk and hidden_states.dtype == region.dtype
    n = M * topk
    dt = _lib.dtype_code(hidden_states.dtype)
    if copy_in:
        region.x[:M].copy_(hidden_states)
    st = RouteState()
    st.M = M
    st.ids = torch.empty(M, topk, dtype=torch.int32, device=dev)
    st.inv_pos = torch.empty(max(n, 1), dtype=torch.int32, device=dev)
    st.counts = torch.empty(E, dtype=torch.int32, device=dev)
    ws = _lib.workspace(lib.fr_route_fused_workspace_bytes(M, H, E, topk), dev, "route")
    rc = _mark(timers, "route", lambda: lib.fr_route_fused(
        _lib.ptr(region.x), dt, M, H, region.x.stride(0), _lib.ptr(gate), gate.stride(0), gate.stride(1), E, topk,
        1 if renormalize else 0, _lib.ptr(region.tw), _lib.ptr(st.ids), None, _lib.ptr(ws), ws.numel(),
        _lib.stream_ptr(dev)))
    _lib.check(rc, "fr_route_fused")
    expert_of_row = _lib.workspace(4 * max(n, 1), dev, "ep_block1")      # block size 1: one entry per assignment
    num_post = torch.empty(1, dtype=torch.int32, device=dev)
    aws = _lib.workspace(lib.fr_align_workspace_bytes(E), dev, "align")
    rc = _mark(timers, "moe_align", lambda: lib.fr_align(
        _lib.ptr(st.ids), n, E, 1, _lib.ptr(region.sorted), n, _lib.ptr(expert_of_row), n, _lib.ptr(num_post),
        _lib.ptr(st.counts), _lib.ptr(st.inv_pos), _lib.ptr(aws), aws.numel(), _lib.stream_ptr(dev)))
    _lib.check(rc, "fr_align")
    return st


def ep_experts_stage(region: PeerRegion, rank: int, all_counts: torch.Tensor, w1_local: torch.Tensor,
                     w2_local: torch.Tensor, num_experts: int, stages: int = 7) -> None:
    """Stage 2 (after every rank's stage 1 is visible): plan from the gathered histograms, gather of the token rows
    from their owners, both grouped GEMMs; results stay in ``region.y``.  ``stages``: 1 = plan + gather, 2 = first
    GEMM, 4 = second GEMM (a caller that times the stages issues them one by one)."""
    from .. import _lib
    lib = _lib.load()
    dev = w1_local.device
    El, N2, H = w1_local.shape
    I = N2 // 2
    assert all_counts.dtype == torch.int32 and all_counts.is_contiguous()
    assert all_counts.shape == (region.world, num_experts) and El * region.world == num_experts
    if region.comb_base is None:
        region.comb_base = torch.empty(num_experts, dtype=torch.int32, device=dev)
    ws = _lib.workspace(lib.fr_ep_workspace_bytes(region.y_rows, H, I, num_experts), dev, "ep_experts")
    rc = lib.fr_ep_experts(ctypes_ptr(region.base_ptrs), region.world, rank, region.x_off, region.x.stride(0),
                           region.rows, region.sorted_off, region.tw_off, region.n, region.topk,
                           _lib.ptr(all_counts), _lib.ptr(w1_local), _lib.ptr(w2_local),
                           _lib.dtype_code(region.dtype), H, I, num_experts, _lib.ptr(region.y), region.y_rows,
                           _lib.ptr(region.comb_base), stages, _lib.ptr(ws), ws.numel(), _lib.stream_ptr(dev))
    _lib.check(rc, "fr_ep_experts")


def ep_combine_stage(region: PeerRegion, st: RouteState, num_experts: int, out: torch.Tensor = None) -> torch.Tensor:
    """Stage 3 (after every rank's stage 2 is visible): each token's k result rows summed straight out of the
    expert owners' memory."""
    from .. import _lib
    lib = _lib.load()
    dev = st.ids.device
    if out is None:
        out = torch.empty(st.M, region.H, dtype=region.dtype, device=dev)
    rc = lib.fr_ep_combine(ctypes_ptr(region.base_ptrs), region.world, region.y_off, region.y.stride(0), region.y_rows,
                           _lib.dtype_code(region.dtype), _lib.ptr(st.ids), _lib.ptr(st.inv_pos),
                           _lib.ptr(region.comb_base), st.M, region.topk, region.H, num_experts, _lib.ptr(out),
                           out.stride(0), _lib.stream_ptr(dev))
    _lib.check(rc, "fr_ep_combine")
    return out


_peer_state: dict = {}


def _peer_region(group, M, H, topk, dtype, device) -> PeerRegion:
    key = (id(group.pg), H, topk, dtype, device.index)
    pr = _peer_state.get(key)
    if pr is None or pr.rows < M:
        if pr is not None:
            # growing: no peer may still be reading the old region when it is released (collective, like the
            # allocation that follows)
            torch.cuda.synchronize(device)
            dist.barrier(group=group.pg)
        pr = PeerRegion(group, M, H, topk, dtype, device)
        _peer_state[key] = pr
    return pr


def peer_input(group: ExpertParallelGroup, M: int, H: int, topk: int, dtype, device) -> torch.Tensor:
    """The ``[M,H]`` token buffer inside this rank's peer region (collective on first use, like the layer itself).
    A caller that produces its tokens straight into it (the previous layer's output, a host-to-device copy) and
    passes it to ``fused_moe_ep_p2p`` saves the copy into the region.  Write the next batch into it only on the
    stream the layer calls are issued on: by then every peer has finished reading the previous one."""
    return _peer_region(group, M, H, topk, dtype, torch.device(device)).x[:M]


def fused_moe_ep_p2p(hidden_states: torch.Tensor, gate: torch.Tensor, w1_local: torch.Tensor,
                     w2_local: torch.Tensor, topk: int, group: ExpertParallelGroup,
                     renormalize: bool = True, timers=None) -> torch.Tensor:
    """Expert-parallel MoE layer in which token rows cross NVLink exactly once each way, are never packed into
    send / receive buffers, and no size ever reaches the host (no synchronisation, no allocation that depends on
    the routing):

    * the only metadata that travels is one all-gather of the per-expert histograms (E integers per rank);
      every rank derives from it, on the device, where each (expert, source rank) segment sits in the owner's
      operand and where each of its own assignments will be found in the owner's results;
    * the expert owner's gather kernel reads the token rows (and their 8 bytes of routing data) directly from
      the memory of the GPUs that hold them while it builds the expert-sorted GEMM operand;
    * the results stay on the expert owner; the source's combine kernel sums the k result rows of each token
      straight out of the owners' memory.

    The all-gather and one more tiny collective order the ranks: a peer's tokens and routing are complete
    before anyone gathers them, a peer's results before anyone combines them, and nobody overwrites a region a
    peer may still be reading (a rank reaches the next call's writes only after it has passed the collective
    that every reader entered after its reads).  ``timers`` (a list) receives (name, start, end) CUDA events of
    the stages.  Every rank must call with at most ``rows`` tokens of the region it first allocated (the first
    call's M; larger batches re-allocate collectively, so all ranks must grow together)."""
    dev = hidden_states.device
    M, H = hidden_states.shape
    E, W = group.num_experts, group.world
    assert w1_local.shape[0] == group.experts_per_rank and gate.shape == (H, E)
    region = _peer_region(group, M, H, topk, hidden_states.dtype, dev)

    def mark(name, fn):
        return _mark(timers, name, fn)

    if hidden_states.data_ptr() != region.x.data_ptr():       # tokens produced straight into the region need no copy
        mark("copy into region", lambda: region.x[:M].copy_(hidden_states))
    st = ep_route_stage(region, hidden_states, gate, topk, E, renormalize, timers, copy_in=False)
    all_counts = torch.empty(W, E, dtype=torch.int32, device=dev)
    mark("count all-gather", lambda: dist.all_gather_into_tensor(all_counts.view(-1), st.counts, group=group.pg))
    if timers is None:
        ep_experts_stage(region, group.rank, all_counts, w1_local, w2_local, E)
    else:
        mark("gather", lambda: ep_experts_stage(region, group.rank, all_counts, w1_local, w2_local, E, 1))
        mark("moe_1", lambda: ep_experts_stage(region, group.rank, all_counts, w1_local, w2_local, E, 2))
        mark("moe_2", lambda: ep_experts_stage(region, group.rank, all_counts, w1_local, w2_local, E, 4))
    mark("results-ready sync", lambda: dist.all_reduce(region.sync_word, group=group.pg))
    return mark("combine", lambda: ep_combine_stage(region, st, E))


def ctypes_ptr(addr: int):
    import ctypes
    return ctypes.c_void_p(int(addr))


def fused_moe_ep_host(x_host: torch.Tensor, gate: torch.Tensor, w1_local: torch.Tensor, w2_local: torch.Tensor,
                      topk: int, group: "ExpertParallelGroup", out_host: torch.Tensor = None, p2p: bool = True,
                      pipelined: bool = False) -> torch.Tensor:
    """The expert-parallel layer for a rank whose token batch lives in pinned host memory: copy-in, the layer
    (``fused_moe_ep_p2p`` or ``fused_moe_ep``) and copy-out on three streams, one chunk per call.  ``pipelined``
    as in ``layers.host.fused_moe_host``: consecutive calls overlap; ``fused_moe_host_wait()``, then a
    synchronisation, before reading."""
    from ..layers.host import host_pipeline
    assert not x_host.is_cuda and x_host.is_pinned() and x_host.dim() == 2 and x_host.is_contiguous()
    dev = w1_local.device
    if out_host is None:
        out_host = torch.empty_like(x_host).pin_memory()
    fn = (lambda buf: fused_moe_ep_p2p(buf, gate, w1_local, w2_local, topk, group)) if p2p else \
         (lambda buf: fused_moe_ep(buf, gate, w1_local, w2_local, topk, group))
    return host_pipeline(fn, x_host, out_host, dev, x_host.shape[0], pipelined, tag="ep")
