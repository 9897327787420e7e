"""CPU oracle for ``moe_align_block_size`` (test infrastructure only).

The reference wrapper (``fast_route/fast_route/ops/fused_moe.py:133-175``)
allocates the three outputs and calls the CUDA op of vLLM 0.4.0.post1
(``requirements.txt:1``), which is not part of the reference tree.  Its
published behaviour, restated here: a stable counting sort of the flattened
``topk_ids`` by expert; each expert's segment is padded to a multiple of
``block_size`` with the sentinel ``numel``; one expert id per block; the total
padded length.  Known answer: the docstring example at ``ops/fused_moe.py:151-159``.
Everything past the valid prefix is unspecified in the reference (``sorted_ids``
is pre-filled with the sentinel at ``:168``, ``expert_ids`` is left
uninitialised); this oracle fills those tails with ``numel`` / ``-1``.
"""

from __future__ import annotations

import numpy as np


def moe_align_block_size(topk_ids, block_size: int, num_experts: int):
    """Returns (sorted_ids, expert_ids, num_tokens_post_pad, counts) as numpy int32.

    sorted_ids has ``numel + E*(block_size-1)`` entries and expert_ids
    ``numel + E`` entries, the sizes the reference allocates (``:161-167``).
    """
    if hasattr(topk_ids, "detach"):
        topk_ids = topk_ids.detach().cpu().numpy()
    flat = np.asarray(topk_ids).reshape(-1).astype(np.int64)
    n = flat.size
    E, bs = int(num_experts), int(block_size)
    counts = np.bincount(flat, minlength=E)[:E] if n else np.zeros(E, dtype=np.int64)
    padded = (counts + bs - 1) // bs * bs
    starts = np.concatenate([[0], np.cumsum(padded)])
    sorted_ids = np.full(n + E * (bs - 1), n, dtype=np.int32)
    expert_ids = np.full(n + E, -1, dtype=np.int32)
    order = np.argsort(flat, kind="stable")
    pos = 0
    for e in range(E):
        c = int(counts[e])
        s = int(starts[e])
        sorted_ids[s:s + c] = order[pos:pos + c]
        pos += c
        expert_ids[s // bs:(s + int(padded[e])) // bs] = e
    num_post = np.array([starts[E]], dtype=np.int32)
    return sorted_ids, expert_ids, num_post, counts.astype(np.int32)
