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
  3. a small all-to-all of the per-expert counts;
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
        st.append({"x": xc, "tw": tw, "sorted": sorted_ids, "inv": inv_pos, "counts": counts,
                   "recv_counts": exchange_counts(counts, group), "n": (hi - lo) * topk})
    counts_h = torch.stack([c["counts"] for c in st]).cpu()
    recv_h = torch.stack([c["recv_counts"] for c in st]).cpu()

    # stage 2: pack rows in destination order straight into the send buffer, start the dispatch
    for i, c in enumerate(st):
        n = c["n"]
        validate_counts(counts_h[i], n, recv_h[i])
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
# the layer over peer memory: dispatch fused into the gather, return fused into the combine
# ------------------------------------------------------------------------------------
class PeerBuffers:
    """Symmetric (peer-readable) staging memory of one rank: ``x[rows, H]`` holds this rank's
    tokens, ``y[y_rows, H]`` its experts' results in expert-sorted order.  Allocation and the
    rendezvous are collective: every rank must construct it with the same arguments."""

    def __init__(self, group: ExpertParallelGroup, rows: int, H: int, topk: int, dtype, device):
        import torch.distributed._symmetric_memory as symm_mem
        from .. import _lib
        self.group, self.rows, self.H, self.topk, self.dtype = group, rows, H, topk, dtype
        lib = _lib.load()
        # worst case: every assignment of every rank lands on this rank
        self.y_rows = int(lib.fr_moe_experts_rows_cap(rows * topk * group.world, group.experts_per_rank))
        self.x = symm_mem.empty((rows, H), dtype=dtype, device=device)
        self.y = symm_mem.empty((self.y_rows, H), dtype=dtype, device=device)
        self.hx = symm_mem.rendezvous(self.x, group.pg)
        self.hy = symm_mem.rendezvous(self.y, group.pg)
        self.x_ptrs = self.hx.buffer_ptrs_dev      # device address of the table of per-rank base pointers
        self.y_ptrs = self.hy.buffer_ptrs_dev


_peer_state: dict = {}


def _peer_buffers(group, M, H, topk, dtype, device) -> PeerBuffers:
    key = (id(group.pg), H, topk, dtype, device.index)
    pb = _peer_state.get(key)
    if pb is None or pb.rows < M:
        pb = PeerBuffers(group, M, H, topk, dtype, device)
        _peer_state[key] = pb
    return pb


def fused_moe_ep_p2p(hidden_states: torch.Tensor, gate: torch.Tensor, w1_local: torch.Tensor,
                     w2_local: torch.Tensor, topk: int, group: ExpertParallelGroup,
                     renormalize: bool = True) -> torch.Tensor:
    """Expert-parallel MoE layer in which token rows cross NVLink exactly once each way and are
    never packed into send / receive buffers:

    * only 8 bytes of metadata per assignment (token index, routing weight) travel through an
      NCCL all-to-all; the expert owner's gather kernel then reads the token rows directly from
      the memory of the GPUs that hold them while it builds the expert-sorted GEMM operand;
    * the results stay on the expert owner; 4 bytes per assignment (its row in that buffer) go
      back, and the source's combine kernel sums the k result rows of each token straight out
      of the owners' memory.

    The two small all-to-alls also order the ranks: a peer's tokens are complete before anyone
    gathers them, a peer's results before anyone combines them, and nobody overwrites a buffer
    a peer may still be reading.  Every rank must call with the same M (rows per rank).
    """
    from .. import _lib
    from ..ops import fused_moe as fm
    from ..ops.stable_route import fused_route

    lib = _lib.load()
    dev = hidden_states.device
    M, H = hidden_states.shape
    El, N2, _ = w1_local.shape
    I = N2 // 2
    E, W = group.num_experts, group.world
    assert El == group.experts_per_rank and gate.shape == (H, E)
    n = M * topk
    dt = _lib.dtype_code(hidden_states.dtype)
    pb = _peer_buffers(group, M, H, topk, hidden_states.dtype, dev)
    pb.x[:M].copy_(hidden_states)

    tw, ti = fused_route(hidden_states, gate, topk, renormalize=renormalize)
    sorted_ids, _, _, counts, inv_pos = fm.moe_align_block_size(ti, 1, E, return_extra=True)
    recv_counts = exchange_counts(counts, group)
    counts_h, recv_h = counts.cpu(), recv_counts.cpu()              # the one host sync: split sizes
    validate_counts(counts_h, n, recv_h)
    in_splits = send_splits(counts_h, W)
    out_splits = recv_h.sum(dim=1).tolist()

    # metadata in destination order: (token row on this rank, routing weight bits)
    order = sorted_ids[:n].long()
    meta = torch.stack([(order // topk).to(torch.int32), tw.reshape(-1)[order].view(torch.int32)], dim=1)
    recv_meta = all_to_all_rows(meta, in_splits, out_splits, group)
    R = recv_meta.shape[0]
    inv_out = torch.empty(max(R, 1), dtype=torch.int32, device=dev)
    if R:
        src_rank = torch.repeat_interleave(torch.arange(W, dtype=torch.int32, device=dev),
                                           recv_counts.sum(dim=1), output_size=R)
        src_row = recv_meta[:, 0].contiguous()
        row_w = recv_meta[:, 1].contiguous().view(torch.float32)
        row_expert = recv_row_experts(recv_counts, R)
        nbytes = lib.fr_moe_experts_workspace_bytes(R, H, I, El)
        ws = _lib.workspace(nbytes, dev, "ep_experts")
        rc = lib.fr_moe_experts_peer(ctypes_ptr(pb.x_ptrs), H, W, pb.rows, _lib.ptr(src_rank), _lib.ptr(src_row),
                                     _lib.ptr(row_expert), _lib.ptr(row_w), _lib.ptr(w1_local), _lib.ptr(w2_local),
                                     dt, R, H, I, El, _lib.ptr(pb.y), pb.y_rows, _lib.ptr(inv_out), _lib.ptr(ws),
                                     ws.numel(), _lib.stream_ptr(dev))
        _lib.check(rc, "fr_moe_experts_peer")
    back_pos = all_to_all_rows(inv_out[:R], out_splits, in_splits, group)      # in this rank's sorted order
    pos_of = back_pos[inv_pos.long()].contiguous()
    rank_of = (ti.reshape(-1) // group.experts_per_rank).to(torch.int32).contiguous()
    out = torch.empty_like(hidden_states)
    rc = lib.fr_combine_peer(ctypes_ptr(pb.y_ptrs), H, W, pb.y_rows, dt, _lib.ptr(rank_of), _lib.ptr(pos_of), M, topk,
                             H, _lib.ptr(out), H, _lib.stream_ptr(dev))
    _lib.check(rc, "fr_combine_peer")
    return out


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
