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


def _copy_out(st, item):
    """Queues one deferred copy-out on the state's output stream and marks its device buffer free afterwards."""
    res, dst, done, b, own = item
    s_out = st["s_out"]
    with torch.cuda.stream(s_out):
        s_out.wait_event(done)
        dst.copy_(res, non_blocking=True)
        if not own:
            res.record_stream(s_out)                 # keep the result's memory until it has left the device
        e = torch.cuda.Event()
        e.record(s_out)
        st["free"][b] = e


def host_pipeline(fn, x_host: torch.Tensor, out_host: torch.Tensor, dev: torch.device, chunk: int,
                  pipelined: bool, tag: str = "layer") -> torch.Tensor:
    """Streams ``x_host`` through ``fn`` (device tensor ``[rows,H]`` -> device tensor ``[rows,H]``, possibly the same
    storage) chunk by chunk: copy-in, ``fn`` and copy-out run on three streams and meet through events only.

    Pipelined calls queue their copy-out one call late, after the next call's ``fn`` has been issued: a large
    device-to-host copy queued earlier would sit in the copy engine in front of the few bytes a layer may read back
    to the host on its way (the expert-parallel layer reads its split sizes), and stall that layer for the length
    of the copy (measured with two GPUs: 11.5 instead of 9.4 ms per step)."""
    M, H = x_host.shape
    plan = _plan(M, chunk)
    rows = max(b - a for a, b in plan)
    key = (dev.index, H, x_host.dtype, tag)
    st = _state.get(key)
    if st is None or st["bufs"][0].shape[0] < rows:
        if st is not None:
            if st["pending"] is not None:
                _copy_out(st, st["pending"])
            st["s_out"].synchronize()                # the old buffers may still be on their way out
        st = {"s_in": torch.cuda.Stream(dev), "s_out": torch.cuda.Stream(dev),
              "bufs": [torch.empty(rows, H, dtype=x_host.dtype, device=dev) for _ in range(3)],
              "free": [None, None, None], "next": 0, "pending": None}
        _state[key] = st
    s_in, s_out, bufs, free = st["s_in"], st["s_out"], st["bufs"], st["free"]
    cur = torch.cuda.current_stream(dev)
    if not pipelined:
        if st["pending"] is not None:
            _copy_out(st, st["pending"])
            st["pending"] = None
        s_in.wait_stream(cur)
    nb = len(bufs)
    for lo, hi in plan:
        b = st["next"] % nb
        st["next"] += 1
        buf = bufs[b][:hi - lo]
        with torch.cuda.stream(s_in):
            if free[b] is not None:
                s_in.wait_event(free[b])             # the buffer's previous result has left the device
            buf.copy_(x_host[lo:hi], non_blocking=True)
            ev_in = torch.cuda.Event()
            ev_in.record(s_in)
        cur.wait_event(ev_in)
        res = fn(buf)
        done = torch.cuda.Event()
        done.record(cur)
        item = (res, out_host[lo:hi], done, b, res.data_ptr() == buf.data_ptr())
        if pipelined:
            if st["pending"] is not None:
                _copy_out(st, st["pending"])
            st["pending"] = item
        else:
            _copy_out(st, item)
    if not pipelined:
        cur.wait_stream(s_out)
    return out_host


def fused_moe_host(x_host: torch.Tensor, gate: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, topk: int,
                   out_host: torch.Tensor = None, renormalize: bool = True, chunk: int = 6144,
                   pipelined: bool = False) -> torch.Tensor:
    """``x_host[M,H]`` (pinned CPU memory, fp16/bf16) -> ``out_host[M,H]`` (pinned CPU memory).

    Weights and gate are device tensors as for ``fused_moe``.  The copies are asynchronous:
    synchronise the current stream (or the device) before reading ``out_host``.

    ``pipelined=True`` lets consecutive calls overlap as a serving loop wants them to: the copy-in does not
    wait for earlier work on the current stream (``x_host`` must be ready when the call is made) and the current
    stream does not wait for the copy-out, so the next call's input travels while this call computes and this
    call's result travels while the next one computes (its copy-out is queued during the next call).  Call
    ``fused_moe_host_wait()`` and then synchronise before reading any ``out_host`` of such calls: it queues the last
    copy-out and makes the current stream wait for all of them.  With calls that overlap like this one chunk per call
    (``chunk >= M``) is fastest; chunking inside a call only pays when calls are isolated.
    """
    assert not x_host.is_cuda and x_host.is_pinned(), "x_host must be pinned host memory"
    assert x_host.dim() == 2 and x_host.is_contiguous()
    dev = w1.device
    if out_host is None:
        out_host = torch.empty_like(x_host).pin_memory()
    assert out_host.is_pinned() and out_host.shape == x_host.shape and out_host.dtype == x_host.dtype
    return host_pipeline(lambda buf: fused_moe(buf, gate, w1, w2, topk, renormalize=renormalize, inplace=True),
                         x_host, out_host, dev, chunk, pipelined)


def fused_moe_host_wait(device=None) -> None:
    """Makes the current stream wait for the copy-outs of all earlier ``fused_moe_host`` calls on ``device``."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    cur = torch.cuda.current_stream(dev)
    for key, st in _state.items():
        if key[0] == dev.index:
            if st["pending"] is not None:
                _copy_out(st, st["pending"])
                st["pending"] = None
            cur.wait_stream(st["s_out"])
