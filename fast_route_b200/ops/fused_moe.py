"""Align and grouped-GEMM operators with the reference's signatures
(``fast_route/fast_route/ops/fused_moe.py`` of the reference).
"""

from __future__ import annotations

import torch

from .. import _lib

BLOCK_M = _lib.BLOCK_M


def moe_align_block_size(topk_ids: torch.Tensor, block_size: int, num_experts: int, return_extra: bool = False):
    """Same contract as ``ops/fused_moe.py:133-175`` of the reference: returns
    ``(sorted_ids, expert_ids, num_tokens_post_pad)`` as int32 tensors of
    ``numel + E*(block_size-1)``, ``numel + E`` and 1 entries; padding entries hold the
    sentinel ``numel``.  Entries past the valid prefix are ``numel`` / ``-1`` (the reference
    leaves the tail of ``expert_ids`` uninitialised).  ``return_extra`` adds
    ``(counts[E], inv_pos[numel])``.
    """
    _lib.require_cuda(topk_ids)
    ids = topk_ids
    if ids.dtype != torch.int32 or not ids.is_contiguous():
        ids = ids.to(torch.int32).contiguous()
    n = ids.numel()
    dev = ids.device
    sorted_ids = torch.empty(n + num_experts * (block_size - 1), dtype=torch.int32, device=dev)
    expert_ids = torch.empty(n + num_experts, dtype=torch.int32, device=dev)
    num_post = torch.empty(1, dtype=torch.int32, device=dev)
    counts = torch.empty(num_experts, dtype=torch.int32, device=dev) if return_extra else None
    inv = torch.empty(max(n, 1), dtype=torch.int32, device=dev) if return_extra else None
    lib = _lib.load()
    ws = _lib.workspace(lib.fr_align_workspace_bytes(num_experts), dev, "align")
    rc = lib.fr_align(_lib.ptr(ids), n, num_experts, block_size, _lib.ptr(sorted_ids), sorted_ids.numel(),
                      _lib.ptr(expert_ids), expert_ids.numel(), _lib.ptr(num_post), _lib.ptr(counts),
                      _lib.ptr(inv), _lib.ptr(ws), ws.numel(), _lib.stream_ptr(dev))
    _lib.check(rc, "fr_align")
    if return_extra:
        return sorted_ids, expert_ids, num_post, counts, inv[:n]
    return sorted_ids, expert_ids, num_post


def permute_rows(x: torch.Tensor, sorted_ids: torch.Tensor, num_post: torch.Tensor, topk: int,
                 max_rows: int = None) -> torch.Tensor:
    """Rows of ``x`` gathered into expert-sorted order (zeros for padding entries)."""
    _lib.require_cuda(x, sorted_ids)
    n_rows = sorted_ids.numel() // BLOCK_M * BLOCK_M if max_rows is None else max_rows
    out = torch.empty(n_rows, x.shape[1], dtype=x.dtype, device=x.device)
    rc = _lib.load().fr_permute_rows(_lib.ptr(x), _lib.dtype_code(x.dtype), x.shape[1], x.stride(0),
                                     _lib.ptr(sorted_ids), _lib.ptr(num_post), x.shape[0] * topk, topk, n_rows,
                                     _lib.ptr(out), out.stride(0), _lib.stream_ptr(x.device))
    _lib.check(rc, "fr_permute_rows")
    return out


def _split_ws(n, cols, split_k, dev):
    if split_k <= 1:
        return None, 0
    nbytes = _lib.load().fr_gemm_splitk_workspace_bytes(n, cols, split_k)
    ws = _lib.workspace(nbytes, dev, "splitk")
    return ws, ws.numel()


def gemm1_silu(a_sorted: torch.Tensor, w1: torch.Tensor, expert_ids: torch.Tensor, num_post: torch.Tensor,
               sorted_ids: torch.Tensor = None, n: int = 0, split_k: int = 1) -> torch.Tensor:
    """``act[p,:] = silu(a[p] . w1[e,:I].T) * (a[p] . w1[e,I:].T)`` on expert-sorted rows."""
    _lib.require_cuda(a_sorted, w1)
    E, N2, H = w1.shape
    I = N2 // 2
    assert w1.is_contiguous() and a_sorted.shape[1] == H and a_sorted.shape[0] % BLOCK_M == 0
    act = torch.empty(a_sorted.shape[0], I, dtype=a_sorted.dtype, device=a_sorted.device)
    ws, wsb = _split_ws(n, N2, split_k, a_sorted.device)
    rc = _lib.load().fr_gemm1_silu(_lib.ptr(a_sorted), a_sorted.stride(0), _lib.ptr(w1),
                                   _lib.dtype_code(a_sorted.dtype), a_sorted.shape[0], H, I, E, _lib.ptr(expert_ids),
                                   _lib.ptr(num_post), _lib.ptr(sorted_ids), n, _lib.ptr(act), act.stride(0), split_k,
                                   _lib.ptr(ws), wsb, _lib.stream_ptr(a_sorted.device))
    _lib.check(rc, "fr_gemm1_silu")
    return act


def gemm2(act: torch.Tensor, w2: torch.Tensor, expert_ids: torch.Tensor, num_post: torch.Tensor,
          sorted_ids: torch.Tensor, topk_weights: torch.Tensor, n: int, split_k: int = 1) -> torch.Tensor:
    """``y[p,:] = w[sorted_ids[p]] * (act[p] . w2[e].T)`` on expert-sorted rows."""
    _lib.require_cuda(act, w2)
    E, H, I = w2.shape
    assert w2.is_contiguous() and act.shape[1] == I and act.shape[0] % BLOCK_M == 0
    y = torch.empty(act.shape[0], H, dtype=act.dtype, device=act.device)
    tw = None
    if topk_weights is not None:
        tw = topk_weights.reshape(-1)
        assert tw.dtype == torch.float32 and tw.is_contiguous()
    ws, wsb = _split_ws(n, H, split_k, act.device)
    rc = _lib.load().fr_gemm2(_lib.ptr(act), act.stride(0), _lib.ptr(w2), _lib.dtype_code(act.dtype), act.shape[0],
                              H, I, E, _lib.ptr(expert_ids), _lib.ptr(num_post), _lib.ptr(sorted_ids), _lib.ptr(tw),
                              n, _lib.ptr(y), y.stride(0), split_k, _lib.ptr(ws), wsb, _lib.stream_ptr(act.device))
    _lib.check(rc, "fr_gemm2")
    return y


def combine(y_sorted: torch.Tensor, inv_pos: torch.Tensor, M: int, topk: int, out: torch.Tensor = None):
    """``out[t] = sum_j y_sorted[inv_pos[t*topk + j]]`` (fp32 accumulation, slot order)."""
    _lib.require_cuda(y_sorted, inv_pos)
    H = y_sorted.shape[1]
    if out is None:
        out = torch.empty(M, H, dtype=y_sorted.dtype, device=y_sorted.device)
    rc = _lib.load().fr_combine(_lib.ptr(y_sorted), y_sorted.stride(0), _lib.dtype_code(y_sorted.dtype),
                                _lib.ptr(inv_pos), M, topk, H, y_sorted.shape[0], _lib.ptr(out), out.stride(0),
                                _lib.stream_ptr(y_sorted.device))
    _lib.check(rc, "fr_combine")
    return out


def invoke_fused_moe_kernel(A: torch.Tensor, B: torch.Tensor, C: torch.Tensor, topk_weights: torch.Tensor,
                            topk_ids: torch.Tensor, sorted_token_ids: torch.Tensor, expert_ids: torch.Tensor,
                            num_tokens_post_padded: torch.Tensor, mul_routed_weight: bool, top_k: int,
                            config: dict = None):
    """Grouped GEMM with the reference's argument list (``ops/fused_moe.py:178-214``):
    ``C[flat id] = A[flat id // top_k] . B[expert]^T`` (times the routed weight when
    ``mul_routed_weight``), rows addressed by ``sorted_token_ids``.  ``C`` is ``[M, topk, N]``
    as in the reference.  The alignment block must be 128 (``config['BLOCK_SIZE_M']`` is
    checked if given).  This general form runs the plain grouped GEMM and scatters rows back;
    the layer itself uses the fused ``gemm1_silu`` / ``gemm2`` path instead.
    """
    if config is not None:
        assert config.get("BLOCK_SIZE_M", BLOCK_M) == BLOCK_M, "align with block_size=128 for the sm_100a GEMM"
    _lib.require_cuda(A, B, C)
    E, N, K = B.shape
    n = topk_ids.numel()
    a_sorted = permute_rows(A, sorted_token_ids, num_tokens_post_padded, top_k)
    tw = topk_weights.reshape(-1).float().contiguous() if mul_routed_weight else None
    y = gemm2(a_sorted, B, expert_ids, num_tokens_post_padded, sorted_token_ids, tw, n)
    valid = sorted_token_ids[:y.shape[0]].long()
    keep = valid < n
    C.view(-1, N)[valid[keep]] = y[keep]
    return C
