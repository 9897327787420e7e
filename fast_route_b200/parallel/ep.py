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


def recv_row_experts(recv_counts: torch.Tensor) -> torch.Tensor:
    """Local expert id of every received row.  Rows arrive grouped by source rank and,
    inside a source's segment, by expert in ascending order."""
    world, epr = recv_counts.shape
    pattern = torch.arange(epr, dtype=torch.int32, device=recv_counts.device).repeat(world)
    return torch.repeat_interleave(pattern, recv_counts.reshape(-1).long())


def all_to_all_rows(send: torch.Tensor, in_splits: List[int], out_splits: List[int], group: ExpertParallelGroup):
    recv = torch.empty((sum(out_splits),) + tuple(send.shape[1:]), dtype=send.dtype, device=send.device)
    dist.all_to_all_single(recv, send, output_split_sizes=out_splits, input_split_sizes=in_splits, group=group.pg)
    return recv


# ------------------------------------------------------------------------------------
# the layer
# ------------------------------------------------------------------------------------
def fused_moe_ep(hidden_states: torch.Tensor, gate: torch.Tensor, w1_local: torch.Tensor, w2_local: torch.Tensor,
                 topk: int, group: ExpertParallelGroup, renormalize: bool = True) -> torch.Tensor:
    """Expert-parallel MoE layer.  ``hidden_states[M,H]`` is this rank's batch, ``gate[H,E]`` is
    replicated, ``w1_local[E/W,2I,H]`` / ``w2_local[E/W,H,I]`` are this rank's experts.
    Returns this rank's ``[M,H]`` output."""
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
    n = M * topk

    tw, ti = fused_route(hidden_states, gate, topk, renormalize=renormalize)
    sorted_ids, _, _, counts, inv_pos = fm.moe_align_block_size(ti, 1, E, return_extra=True)
    recv_counts = exchange_counts(counts, group)
    counts_h, recv_h = counts.cpu(), recv_counts.cpu()          # the one host sync: split sizes
    validate_counts(counts_h, n, recv_h)
    in_splits = send_splits(counts_h, group.world)
    out_splits = recv_h.sum(dim=1).tolist()

    # pack: rows gathered in destination order straight into the send buffer
    num_post = torch.tensor([n], dtype=torch.int32, device=dev)
    send_rows = torch.empty(n, H, dtype=hidden_states.dtype, device=dev)
    rc = lib.fr_permute_rows(_lib.ptr(hidden_states), _lib.dtype_code(hidden_states.dtype), H,
                             hidden_states.stride(0), _lib.ptr(sorted_ids), _lib.ptr(num_post), n, topk, n,
                             _lib.ptr(send_rows), H, _lib.stream_ptr(dev))
    _lib.check(rc, "fr_permute_rows")
    send_w = tw.reshape(-1)[sorted_ids[:n].long()]

    recv_rows = all_to_all_rows(send_rows, in_splits, out_splits, group)
    recv_w = all_to_all_rows(send_w, in_splits, out_splits, group)
    R = recv_rows.shape[0]

    y = torch.empty(R, H, dtype=hidden_states.dtype, device=dev)
    if R:
        row_expert = recv_row_experts(recv_counts)
        nbytes = lib.fr_moe_experts_workspace_bytes(R, H, I, El)
        ws = _lib.workspace(nbytes, dev, "ep_experts")
        rc = lib.fr_moe_experts(_lib.ptr(recv_rows), _lib.ptr(row_expert), _lib.ptr(recv_w), _lib.ptr(w1_local),
                                _lib.ptr(w2_local), _lib.dtype_code(hidden_states.dtype), R, H, I, El, _lib.ptr(y),
                                _lib.ptr(ws), ws.numel(), _lib.stream_ptr(dev))
        _lib.check(rc, "fr_moe_experts")

    back = all_to_all_rows(y, out_splits, in_splits, group)      # arrives in this rank's sorted order
    return fm.combine(back, inv_pos, M, topk)
