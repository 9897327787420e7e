"""The MoE layer for callers whose activations live in host memory.

``fused_moe_host`` streams a pinned host batch through the GPU in chunks: while chunk i is
being computed, chunk i+1 is copied in and chunk i-1 is copied out, each on its own CUDA
stream.  The layer math is ``fused_moe`` of ``layers/stable_route.py`` unchanged (tokens are
independent, so chunking does not change any result).  The reference has no such entry
point; its benchmarks keep everything on the device (``benchmarks/fused_route/moe_bench.py:85-97``).
"""

from __future__ import annotations

import torch

from .stable_route import fused_moe

_state: dict = {}


def _plan(M: int, chunk: int):
    """Chunk boundaries: a short first and last chunk keep the un-overlapped copy-in of the
    first chunk and copy-out of the last one small; the middle chunks are `chunk` rows."""
    if M <= chunk:
        return [(0, M)]
    edge = max(256, chunk // 4)
    cuts = [0, min(edge, M)]
    while M - cuts[-1] > chunk + edge:
        cuts.append(cuts[-1] + chunk)
    if M - cuts[-1] > edge:
        cuts.append(M - edge)
    cuts.append(M)
    return [(a, b) for a, b in zip(cuts[:-1], cuts[1:]) if b > a]


def fused_moe_host(x_host: torch.Tensor, gate: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, topk: int,
                   out_host: torch.Tensor = None, renormalize: bool = True, chunk: int = 6144) -> torch.Tensor:
    """``x_host[M,H]`` (pinned CPU memory, fp16/bf16) -> ``out_host[M,H]`` (pinned CPU memory).

    Weights and gate are device tensors as for ``fused_moe``.  The copies are asynchronous:
    synchronise the current stream (or the device) before reading ``out_host``.
    """
    assert not x_host.is_cuda and x_host.is_pinned(), "x_host must be pinned host memory"
    assert x_host.dim() == 2 and x_host.is_contiguous()
    dev = w1.device
    M, H = x_host.shape
    if out_host is None:
        out_host = torch.empty_like(x_host).pin_memory()
    assert out_host.is_pinned() and out_host.shape == x_host.shape and out_host.dtype == x_host.dtype
    plan = _plan(M, chunk)
    rows = max(b - a for a, b in plan)
    key = (dev.index, H, x_host.dtype)
    st = _state.get(key)
    if st is None or st["bufs"][0].shape[0] < rows:
        st = {"s_in": torch.cuda.Stream(dev), "s_out": torch.cuda.Stream(dev),
              "bufs": [torch.empty(rows, H, dtype=x_host.dtype, device=dev) for _ in range(3)]}
        _state[key] = st
    s_in, s_out, bufs = st["s_in"], st["s_out"], st["bufs"]
    cur = torch.cuda.current_stream(dev)
    s_in.wait_stream(cur)
    s_out.wait_stream(cur)
    nb = len(bufs)
    ev_in, ev_out = [], []
    for i, (lo, hi) in enumerate(plan):
        buf = bufs[i % nb][:hi - lo]
        with torch.cuda.stream(s_in):
            if i >= nb:
                s_in.wait_event(ev_out[i - nb])          # the buffer's previous result has left the device
            buf.copy_(x_host[lo:hi], non_blocking=True)
            e = torch.cuda.Event()
            e.record(s_in)
            ev_in.append(e)
        cur.wait_event(ev_in[i])
        fused_moe(buf, gate, w1, w2, topk, renormalize=renormalize, inplace=True)
        done = torch.cuda.Event()
        done.record(cur)
        with torch.cuda.stream(s_out):
            s_out.wait_event(done)
            out_host[lo:hi].copy_(buf, non_blocking=True)
            e = torch.cuda.Event()
            e.record(s_out)
            ev_out.append(e)
    cur.wait_stream(s_out)
    return out_host
