"""W4A16 small-batch GEMM with the reference's call shape
(``matmul_split_k(a, b, scales, zeros)``, ``benchmarks/splitk_gemm/splitk.py:178-216``)."""

from __future__ import annotations

import torch

from .. import _lib


def matmul_split_k(a: torch.Tensor, b: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor,
                   groupsize: int = 128, split_k: int = 0, out: torch.Tensor = None) -> torch.Tensor:
    """``a[m,k]`` fp16, ``b[k/8,n]`` int32 (GPTQ nibbles along k), ``scales[k/g,n]`` fp16,
    ``zeros[k/g,n/8]`` int32 (nibbles along n) -> ``c[m,n]`` fp16.  The reference fixes
    ``groupsize = 128`` and ``split_k = 4`` (``:183-190``); here ``split_k = 0`` lets the library choose
    and the K slices are reduced deterministically."""
    _lib.require_cuda(a, b, scales, zeros)
    m, k = a.shape
    k8, n = b.shape
    assert k8 * 8 == k, "Incompatible dimensions"
    assert a.dtype == torch.float16 and scales.dtype == torch.float16
    assert b.dtype == torch.int32 and zeros.dtype == torch.int32
    assert a.stride(1) == 1 and b.is_contiguous() and scales.is_contiguous() and zeros.is_contiguous()
    assert scales.shape == (k // groupsize, n) and zeros.shape == (k // groupsize, n // 8)
    if out is None:
        out = torch.empty(m, n, dtype=torch.float16, device=a.device)
    assert out.dtype == torch.float16 and out.stride(1) == 1 and out.shape == (m, n)
    rc = _lib.load().fr_w4a16_gemm(_lib.ptr(a), a.stride(0), _lib.ptr(b), _lib.ptr(scales), _lib.ptr(zeros), m, n, k,
                                   groupsize, _lib.ptr(out), out.stride(0), split_k, _lib.stream_ptr(a.device))
    _lib.check(rc, "fr_w4a16_gemm")
    return out


def dequantize(b: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor, groupsize: int = 128) -> torch.Tensor:
    """The dense fp16 matrix ``w[k,n]`` that ``matmul_split_k`` multiplies with."""
    _lib.require_cuda(b, scales, zeros)
    k8, n = b.shape
    assert b.dtype == torch.int32 and zeros.dtype == torch.int32 and scales.dtype == torch.float16
    assert b.is_contiguous() and scales.is_contiguous() and zeros.is_contiguous()
    w = torch.empty(k8 * 8, n, dtype=torch.float16, device=b.device)
    rc = _lib.load().fr_w4a16_dequant(_lib.ptr(b), _lib.ptr(scales), _lib.ptr(zeros), n, k8 * 8, groupsize,
                                      _lib.ptr(w), w.stride(0), _lib.stream_ptr(b.device))
    _lib.check(rc, "fr_w4a16_dequant")
    return w


__all__ = ["matmul_split_k", "dequantize"]
