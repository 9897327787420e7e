"""The C-ABI library builds, loads without a GPU and exports every symbol the public header
declares; the ctypes table covers the header one to one; host-side argument checks work."""

import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "fast_route_sm100.h")


def header_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fr_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported(lib):
    names = header_functions()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"


def test_ctypes_table_matches_header(lib):
    from fast_route_b200 import _lib
    assert sorted(_lib.SIGNATURES) == header_functions()
    text = re.sub(r"/\*.*?\*/", "", open(HEADER).read(), flags=re.S)
    for name, (_, args) in _lib.SIGNATURES.items():
        m = re.search(r"\b" + name + r"\s*\(([^;]*?)\)\s*;", text, flags=re.S)
        assert m, name
        params = [p for p in m.group(1).split(",") if p.strip() and p.strip() != "void"]
        assert len(params) == len(args), f"{name}: header has {len(params)} parameters, ctypes table {len(args)}"


def test_version_and_error_strings(lib):
    assert lib.fr_version() >= 100
    assert b"argument" in lib.fr_error_string(-1)
    assert b"aligned" in lib.fr_error_string(-3)
    assert lib.fr_error_string(0) == b"ok"


def test_workspace_queries_need_no_gpu(lib):
    big = lib.fr_moe_workspace_bytes(16384, 4096, 14336, 8, 2)
    small = lib.fr_moe_workspace_bytes(1, 4096, 14336, 8, 2)
    assert 1 << 30 < big < 4 << 30
    assert 0 < small < big
    assert lib.fr_moe_workspace_bytes(0, 4096, 14336, 8, 2) == 0
    assert lib.fr_gemm_splitk_workspace_bytes(32, 4096, 1) == 0
    assert lib.fr_gemm_splitk_workspace_bytes(32, 4096, 4) == 4 * 32 * 4096 * 4


def test_argument_checks_reject_before_any_launch(lib):
    null = ctypes.c_void_p(None)
    assert lib.fr_topk_softmax(null, 0, 4, 8, 8, 1, 2, 1, null, 2, null, 2, 0, null) == -1
    assert lib.fr_align(null, 8, 4, 16, null, 100, null, 100, null, null, null, null, 0, null) == -1
    assert lib.fr_moe_layer(null, null, 1, 1, null, null, 1, 4, 64, 64, 4, 2, 1, null, null, null, null, 0, null) == -1
    assert lib.fr_combine(null, 8, 1, null, 4, 2, 64, 128, null, 8, null) == -1
    # expert-parallel entry points: null tables, experts that do not divide over the ranks, misaligned capacity
    assert lib.fr_ep_experts(null, 2, 0, 0, 64, 8, 0, 0, 16, 2, null, null, null, 1, 64, 64, 8, null, 128, null, 7,
                             null, 0, null) == -1
    assert lib.fr_ep_combine(null, 2, 0, 64, 128, 1, null, null, null, 4, 2, 64, 8, null, 64, null) == -1
    assert lib.fr_ep_workspace_bytes(0, 64, 64, 8) == 0
    small, big = lib.fr_ep_workspace_bytes(1024, 4096, 14336, 8), lib.fr_ep_workspace_bytes(262272, 4096, 14336, 8)
    assert 0 < small < big and big > 9 << 30      # the operand and the activations of 262272 rows: 9.7 GB
    assert lib.fr_moe_experts_rows_cap(8 * 32768, 1) == 262272


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "fast_route_b200")
    for d, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                src = open(os.path.join(d, f)).read()
                assert not re.search(r"^\s*(from|import)\s+oracle\b", src, flags=re.M), f
                assert "oracle/" not in src, f


def test_cpu_tensors_are_rejected_loudly():
    import torch
    import fast_route_b200 as fr
    x = torch.zeros(4, 64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        fr.route_from_logits(torch.zeros(4, 8), 2)
    with pytest.raises(RuntimeError):
        fr.fused_moe(x, torch.zeros(64, 4, dtype=torch.bfloat16), torch.zeros(4, 128, 64, dtype=torch.bfloat16),
                     torch.zeros(4, 64, 64, dtype=torch.bfloat16), 2)


def test_host_chunk_plan_covers_the_batch_exactly():
    """The chunk plan of the host-buffer entry point: contiguous, non-empty, no overlap, every row once; short first
    and last chunks when a batch is split."""
    from fast_route_b200.layers.host import _plan
    for M in (1, 5, 255, 256, 1000, 6144, 6145, 7000, 8192, 16384, 16385, 100000):
        for chunk in (256, 1024, 6144, 1 << 20):
            plan = _plan(M, chunk)
            assert plan[0][0] == 0 and plan[-1][1] == M
            assert all(a < b for a, b in plan)
            assert all(plan[i][1] == plan[i + 1][0] for i in range(len(plan) - 1))
            assert max(b - a for a, b in plan) <= chunk + max(256, chunk // 4)
            if M <= chunk:
                assert plan == [(0, M)]
