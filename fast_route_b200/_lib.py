"""Loader and thin ctypes binding of ``libfastroute_sm100.so`` (the C ABI declared in
``include/fast_route_sm100.h``).

There is no fallback: if the shared library is missing or a call fails, an exception
is raised.  PyTorch only supplies device memory and the current stream.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_int, c_int64, c_size_t, c_void_p

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libfastroute_sm100.so")

FR_F16, FR_BF16, FR_F32 = 0, 1, 2
BLOCK_M = 128

_DTYPES = {torch.float16: FR_F16, torch.bfloat16: FR_BF16, torch.float32: FR_F32}

# name -> (restype, argtypes); mirrors include/fast_route_sm100.h declaration by declaration
_P, _I, _L, _Z = c_void_p, c_int, c_int64, c_size_t
SIGNATURES = {
    "fr_version": (_I, []),
    "fr_error_string": (c_char_p, [_I]),
    "fr_check_status": (_I, [_P]),
    "fr_topk_softmax": (_I, [_P, _I, _L, _I, _L, _L, _I, _I, _P, _L, _P, _L, _I, _P]),
    "fr_softmax_topk": (_I, [_P, _I, _L, _I, _L, _L, _I, _I, _P, _L, _P, _L, _P, _L, _P]),
    "fr_align_workspace_bytes": (_Z, [_I]),
    "fr_align": (_I, [_P, _L, _I, _I, _P, _L, _P, _L, _P, _P, _P, _P, _Z, _P]),
    "fr_align_noalloc": (_I, [_P, _L, _I, _I, _P, _L, _P, _L, _P, _P, _P, _P]),
    "fr_route_align": (_I, [_P, _I, _L, _I, _L, _L, _I, _P, _P, _I, _P, _L, _P, _L, _P, _P, _Z, _P]),
    "fr_route_fused_workspace_bytes": (_Z, [_L, _I, _I, _I]),
    "fr_route_fused": (_I, [_P, _I, _L, _I, _L, _P, _L, _L, _I, _I, _I, _P, _P, _P, _P, _Z, _P]),
    "fr_permute_rows": (_I, [_P, _I, _I, _L, _P, _P, _L, _I, _L, _P, _L, _P]),
    "fr_gemm_splitk_workspace_bytes": (_Z, [_L, _L, _I]),
    "fr_gemm1_silu": (_I, [_P, _L, _P, _I, _L, _I, _I, _I, _P, _P, _P, _L, _P, _L, _I, _P, _Z, _P]),
    "fr_gemm2": (_I, [_P, _L, _P, _I, _L, _I, _I, _I, _P, _P, _P, _P, _L, _P, _L, _I, _P, _Z, _P]),
    "fr_combine": (_I, [_P, _L, _I, _P, _L, _I, _I, _L, _P, _L, _P]),
    "fr_moe_workspace_bytes": (_Z, [_L, _I, _I, _I, _I]),
    "fr_moe_layer": (_I, [_P, _P, _L, _L, _P, _P, _I, _L, _I, _I, _I, _I, _I, _P, _P, _P, _P, _Z, _P]),
    "fr_add_rmsnorm": (_I, [_P, _L, _P, _L, _P, ctypes.c_float, _I, _L, _I, _P, _L, _P, _L, _P]),
    "fr_moe_block_workspace_bytes": (_Z, [_L, _I, _I, _I, _I]),
    "fr_moe_block": (_I, [_P, _P, _P, ctypes.c_float, _P, _L, _L, _P, _P, _I, _L, _I, _I, _I, _I, _I, _I, _P, _P, _Z, _P]),
    "fr_moe_fp8_workspace_bytes": (_Z, [_L, _I, _I, _I, _I]),
    "fr_moe_layer_fp8": (_I, [_P, _P, _L, _L, _P, _P, _P, _P, _I, _L, _I, _I, _I, _I, _I, _P, _P, _P, _P, _Z, _P]),
    "fr_moe_layer_routed": (_I, [_P, _P, _P, _P, _P, _I, _L, _I, _I, _I, _I, _P, _P, _Z, _P]),
    "fr_moe_experts_workspace_bytes": (_Z, [_L, _I, _I, _I]),
    "fr_moe_experts": (_I, [_P, _P, _P, _P, _P, _I, _L, _I, _I, _I, _P, _P, _Z, _P]),
    "fr_moe_experts_rows_cap": (_L, [_L, _I]),
    "fr_ep_workspace_bytes": (_Z, [_L, _I, _I, _I]),
    "fr_ep_experts": (_I, [_P, _I, _I, _L, _L, _L, _L, _L, _L, _I, _P, _P, _P, _I, _I, _I, _I, _P, _L, _P, _I, _P, _Z, _P]),
    "fr_ep_combine": (_I, [_P, _I, _L, _L, _L, _I, _P, _P, _P, _L, _I, _I, _I, _P, _L, _P]),
    "fr_gather_rows": (_I, [_P, _L, _P, _L, _I, _P, _L, _P]),
    "fr_w4a16_gemm": (_I, [_P, _L, _P, _P, _P, _L, _I, _I, _I, _P, _L, _I, _P]),
    "fr_w4a16_dequant": (_I, [_P, _P, _P, _I, _I, _I, _P, _L, _P]),
}

_lib = None


class FastRouteError(RuntimeError):
    pass


def load() -> ctypes.CDLL:
    """Loads the shared library once; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FastRouteError(
                f"{LIB_PATH} not found: build it with `python -m fast_route_b200.build` "
                "(there is no CPU or PyTorch fallback)")
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPES[dt]
    except KeyError:
        raise AssertionError(f"unsupported dtype {dt}") from None


def ptr(t):
    return None if t is None else c_void_p(t.data_ptr())


def stream_ptr(device=None):
    return c_void_p(torch.cuda.current_stream(device).cuda_stream)


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = load().fr_error_string(rc).decode()
        if rc == -1:
            raise AssertionError(f"{what}: {msg}")
        raise FastRouteError(f"{what} failed ({rc}): {msg}")


def require_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise FastRouteError("fast_route_b200 runs on CUDA tensors only; there is no CPU path")


def device_status():
    """Synchronises and returns (code, detail, block, count) of the device status block."""
    out = (ctypes.c_uint * 4)()
    check(load().fr_check_status(out), "fr_check_status")
    return tuple(int(v) for v in out)


def raise_on_device_error() -> None:
    code, detail, block, count = device_status()
    if code:
        names = {1: "bounded wait expired", 2: "expert id out of range", 3: "bad sorted id",
                 4: "expert-parallel receive capacity exceeded"}
        raise FastRouteError(f"device status: {names.get(code, code)} (detail {detail:#x}, block {block}, "
                             f"{count} reports)")


_workspaces: dict = {}


def workspace(nbytes: int, device, tag: str = "layer") -> torch.Tensor:
    """A cached, 1024-byte aligned byte buffer per (device, stream, tag); grows on demand.
    New buffers are zero-filled once (the align stage keeps its grid-barrier words there)."""
    key = (torch.device(device).index, torch.cuda.current_stream(device).cuda_stream, tag)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes + 1024:
        buf = torch.zeros(int(nbytes) + 1024, dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    off = (-buf.data_ptr()) % 1024
    return buf[off:off + max(nbytes, 1)]
