"""CPU oracle for the W4A16 split-K GEMM (test infrastructure, never imported by the product).

Restates ``hint_kernel`` / ``matmul_split_k`` of the reference
(``benchmarks/splitk_gemm/splitk.py:26-103`` and ``:178-216``):

* ``b[k/8, n]`` int32: nibble ``j`` of word ``[kk, n]`` is the 4-bit weight of row ``k = 8*kk + j``
  (``:62, 70, 86``);
* ``zeros[k/g, n/8]`` int32: nibble ``j`` of word ``[gi, nn]`` is the zero point of column
  ``n = 8*nn + j`` (``:65, 71, 83``); ``scales[k/g, n]`` fp16; group ``g = groupsize`` rows of k;
* ``w = b * scales - (zeros + 1) * scales`` (``:84-87``) with fp16 operands, i.e. three fp16
  operations each rounded once (the reference runs them un-fused under the Triton interpreter; a
  GPU compile may contract the last two into one fused multiply-add, which this recipe does not);
* ``c = a . w`` accumulated in fp32 (``:76, 89``) and stored as fp16; the reference adds its four K
  slices into ``c`` with fp16 atomics (``:103``), so its own result is only defined up to a few fp16
  roundings in arbitrary order.  The oracle returns the fp64 dot product of the exact fp16 weights;
  the test states the tolerance.

Pinned against the reference kernel itself executed on CPU (``TRITON_INTERPRET=1``):
``tests/golden/w4a16.npz`` with its generator ``tests/golden/make_golden.py``.
"""

from __future__ import annotations

import numpy as np


def _np(a):
    if hasattr(a, "detach"):
        a = a.detach().cpu().numpy()
    return np.asarray(a)


def _round_f16(x64: np.ndarray) -> np.ndarray:
    """float64 -> float16 with a single rounding (numpy converts directly)."""
    return x64.astype(np.float16)


def dequant(b, scales, zeros, groupsize: int = 128) -> np.ndarray:
    """fp16 weights ``w[k, n]`` bit for bit as the reference computes them un-fused."""
    b = _np(b).astype(np.int64) & 0xFFFFFFFF
    zeros = _np(zeros).astype(np.int64) & 0xFFFFFFFF
    scales = _np(scales).astype(np.float16)
    k8, n = b.shape
    k = k8 * 8
    shifts = (np.arange(8, dtype=np.int64) * 4)
    q = ((b[:, None, :] >> shifts[None, :, None]) & 0xF).reshape(k, n)              # [k, n]
    z = ((zeros[:, :, None] >> shifts[None, None, :]) & 0xF).reshape(zeros.shape[0], -1)[:, :n]
    g = np.arange(k) // groupsize
    s = scales[g].astype(np.float64)                                                 # [k, n]
    qs = _round_f16(q.astype(np.float64) * s)               # products of fp16 values are exact in fp64
    zs = _round_f16((z[g] + 1).astype(np.float64) * s)
    return _round_f16(qs.astype(np.float64) - zs.astype(np.float64))


def matmul_split_k(a, b, scales, zeros, groupsize: int = 128) -> np.ndarray:
    """``a[m,k] . dequant(b)`` in float64 (the caller rounds / applies its tolerance)."""
    w = dequant(b, scales, zeros, groupsize).astype(np.float64)
    return _np(a).astype(np.float64) @ w


__all__ = ["dequant", "matmul_split_k"]
