"""Generates the golden vectors under tests/golden from the reference's own code.

Run where the reference tree is mounted:

    python tests/golden/make_golden.py /path/to/reference

It executes, on the CPU:
  * the reference's stable bitonic argsort (``fast_route/fast_route/ops/stable_argsort.py:96-114``)
    inside a small Triton test kernel shaped like the one in the reference's
    ``fast_route/tests/test_argsort.py:11-48``, under ``TRITON_INTERPRET=1``;
  * the reference's router kernel (``ops/stable_route.py:32-121``) launched the way
    its host wrapper does (``:132-170``), except that the zero-padded gate's own
    strides are passed when E < 16 (the wrapper passes the unpadded gate's strides
    there, which the reference's author flags as broken at ``:88-90``);
  * the reference's naive layer ``torch_moe`` (``benchmarks/swizzle_moe/perf_test_moe.py:17-31``)
    and activation (``benchmarks/swizzle_moe/activation.py:27-30``), extracted from
    the source text because the modules import an absent vLLM build.

  * the reference's W4A16 split-K Triton kernel ``hint_kernel``
    (``benchmarks/splitk_gemm/splitk.py:26-103``) launched with the tile sizes of its host
    wrapper (``:183-190``; the wrapper itself is not called: it dumps compiler output next to
    the source), on inputs drawn like its ``make_tensor`` (``:267-275``).

Outputs are small ``.npz`` files.  The tests only read the ``.npz`` files; they
never need the reference tree.
"""

import ast
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np
import torch
import torch.nn.functional as F
import triton
import triton.language as tl

REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("FAST_ROUTE_REFERENCE", "")
if not os.path.isdir(os.path.join(REF, "fast_route")):
    sys.exit("usage: python tests/golden/make_golden.py /path/to/the/reference/checkout")
HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(REF, "fast_route"))
sys.path.insert(0, os.path.join(HERE, "..", ".."))

from fast_route.ops.stable_argsort import argsort as ref_stable_argsort  # noqa: E402
import fast_route.ops.stable_route as ref_route  # noqa: E402
from fast_route_b200 import synth  # noqa: E402


@triton.jit
def _sort_rows(x_ptr, o_ptr, id_ptr, stride_m, DESCEND: tl.constexpr,
               BLOCK_M: tl.constexpr, BLOCK_N: tl.constexpr):
    pid = tl.program_id(0)
    offs = pid * stride_m * BLOCK_M + tl.arange(0, BLOCK_M)[:, None] * stride_m + tl.arange(0, BLOCK_N)[None, :]
    x = tl.load(x_ptr + offs)
    ids = tl.broadcast_to(tl.arange(0, BLOCK_N)[None, :], (BLOCK_M, BLOCK_N))
    o, ids = ref_stable_argsort(x, ids, 1, DESCEND)
    tl.store(o_ptr + offs, o)
    tl.store(id_ptr + offs, ids)


def golden_argsort():
    out = {}
    for E in (8, 16, 64, 128):
        for dt, name in ((torch.float16, "f16"), (torch.float32, "f32")):
            M = 64
            x = synth.routing_logits(M, E, 4, seed=11 + E, dtype=dt, dup_frac=0.25)
            o = torch.empty_like(x)
            ids = torch.empty(M, E, dtype=torch.int32)
            _sort_rows[(M // 16,)](x, o, ids, x.stride(0), 1, 16, E)
            out[f"x_{E}_{name}"] = x.float().numpy()
            out[f"sorted_{E}_{name}"] = o.float().numpy()
            out[f"ids_{E}_{name}"] = ids.numpy()
    np.savez_compressed(os.path.join(HERE, "stable_argsort.npz"), **out)
    print("stable_argsort.npz", len(out), "arrays")


def _run_ref_route(h, g, topk, BM=32):
    M, K = h.shape
    _, E = g.shape
    if E < 16:
        diff = 16 - E
        pg = torch.cat([g, torch.zeros((K, diff), dtype=g.dtype)], 1)
    else:
        diff, pg = 0, g
    tw = torch.empty(M, E, dtype=torch.float32)
    ti = torch.empty(M, E, dtype=torch.int32)
    ref_route.route_kernel.fn[(triton.cdiv(M, BM),)](
        h, pg, tw, ti, M, E, K, h.stride(0), h.stride(1), pg.stride(0), pg.stride(1),
        tw.stride(0), tw.stride(1), TOPK=topk, DIFF=diff, BLOCK_SIZE_M=BM,
        BLOCK_SIZE_N=max(E, 16), BLOCK_SIZE_K=32)
    return tw, ti


def golden_route():
    out = {}
    cases = [(64, 256, 16, 2), (64, 256, 8, 2), (64, 256, 16, 4), (32, 128, 64, 6), (64, 128, 128, 8)]
    for ci, (M, K, E, k) in enumerate(cases):
        h = (synth.randn((M, K), 5, ci) / 10).half()
        g = (synth.randn((K, E), 6, ci) / 10).half()
        tw, ti = _run_ref_route(h, g, k)
        out[f"h_{ci}"] = h.numpy()
        out[f"g_{ci}"] = g.numpy()
        out[f"w_{ci}"] = tw.numpy()          # full [M,E] buffers as the kernel leaves them
        out[f"ids_{ci}"] = ti.numpy()
        out[f"meta_{ci}"] = np.array([M, K, E, k], dtype=np.int64)
    np.savez_compressed(os.path.join(HERE, "route_kernel.npz"), **out)
    print("route_kernel.npz", len(cases), "cases")


def _extract(path, name, kind):
    tree = ast.parse(open(path).read())
    for node in ast.walk(tree):
        if isinstance(node, kind) and node.name == name:
            return node
    raise KeyError(name)


def load_ref_torch_moe():
    act_cls = _extract(os.path.join(REF, "benchmarks/swizzle_moe/activation.py"), "SiluAndMul", ast.ClassDef)
    fwd = next(n for n in act_cls.body if isinstance(n, ast.FunctionDef) and n.name == "_forward")
    ns = {"torch": torch, "F": F}
    exec(compile(ast.Module(body=[fwd], type_ignores=[]), "activation._forward", "exec"), ns)
    native_forward = ns["_forward"]

    class SiluAndMul:
        def __call__(self, x):
            return native_forward(self, x)

    fn = _extract(os.path.join(REF, "benchmarks/swizzle_moe/perf_test_moe.py"), "torch_moe", ast.FunctionDef)
    ns2 = {"torch": torch, "SiluAndMul": SiluAndMul}
    exec(compile(ast.Module(body=[fn], type_ignores=[]), "perf_test_moe.torch_moe", "exec"), ns2)
    return ns2["torch_moe"]


def golden_layer():
    ref_moe = load_ref_torch_moe()
    out = {}
    # small case: inputs stored
    M, H, I, E, k = 48, 64, 96, 4, 2
    x, gate, w1, w2 = synth.moe_inputs(M, H, I, E, seed=3, dtype=torch.float32, weight_std=0.1)
    logits = x @ gate
    p = torch.softmax(logits, -1)
    so, si = torch.sort(p, dim=1, descending=True, stable=True)
    tw = (so[:, :k] / so[:, :k].sum(-1, keepdim=True)).contiguous()
    ti = si[:, :k].contiguous()
    y = ref_moe(x, w1, w2, tw, ti)
    out.update(small_x=x.numpy(), small_gate=gate.contiguous().numpy(), small_w1=w1.numpy(),
               small_w2=w2.numpy(), small_tw=tw.numpy(), small_ti=ti.numpy().astype(np.int32),
               small_out=y.numpy())
    # the reference's CPU-runnable benchmark case: fp32, M=256, H=1024, I=2048, E=8, top-2, seed 0.
    # Inputs are regenerated from the seed by the tests; a strided sample of the output is stored.
    M, H, I, E, k = 256, 1024, 2048, 8, 2
    x, gate, w1, w2 = synth.moe_inputs(M, H, I, E, seed=0, dtype=torch.float32)
    logits = x @ gate
    so, si = torch.sort(logits, dim=1, descending=True, stable=True)
    tw = torch.softmax(so[:, :k], -1).contiguous()
    ti = si[:, :k].contiguous()
    y = ref_moe(x, w1, w2, tw, ti)
    out.update(c1_x_sum=np.array([x.double().sum().item(), w1.double().sum().item(), w2.double().sum().item()]),
               c1_ti=ti.numpy().astype(np.int32), c1_tw=tw.numpy(),
               c1_out_sample=y[::8, ::16].contiguous().numpy())
    np.savez_compressed(os.path.join(HERE, "torch_moe.npz"), **out)
    print("torch_moe.npz")


def w4a16_inputs(m, k, n, groupsize, seed):
    """Seeded inputs distributed like the reference's make_tensor (normal std 0.5 / uniform int32)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    a = (torch.randn(m, k, generator=g) * 0.5).half()
    b = torch.randint(-2**31, 2**31 - 1, (k // 8, n), generator=g, dtype=torch.int64).to(torch.int32)
    zeros = torch.randint(-2**31, 2**31 - 1, (k // groupsize, n // 8), generator=g, dtype=torch.int64).to(torch.int32)
    scales = (torch.randn(k // groupsize, n, generator=g) * 0.5).half()
    return a, b, scales, zeros


def golden_w4a16():
    sys.path.insert(0, os.path.join(REF, "benchmarks", "splitk_gemm"))
    import splitk as ref_splitk
    out = {}
    # case 2 has one-hot activation rows, so its output rows are single dequantised weight rows, exactly
    cases = [(16, 512, 64), (32, 1024, 96), (64, 512, 64)]
    for ci, (m, k, n) in enumerate(cases):
        groupsize, block_m, block_n, block_k, group_m, split_k = 128, 16, 32, 128, 8, 4
        a, b, scales, zeros = w4a16_inputs(m, k, n, groupsize, 40 + ci)
        if ci == 2:
            rows = (torch.arange(m) * 8 + torch.arange(m) % 8) % k      # every nibble position, every group
            a = torch.zeros(m, k, dtype=torch.float16)
            a[torch.arange(m), rows] = 1.0
            out["onehot_rows"] = rows.numpy()
        c = torch.zeros((m, n), dtype=torch.float16)
        grid = (triton.cdiv(m, block_m) * triton.cdiv(n, block_n), split_k)
        ref_splitk.hint_kernel[grid](a, b, c, scales, zeros,
                                     a.stride(0), a.stride(1), b.stride(0), b.stride(1), c.stride(0), c.stride(1),
                                     scales.stride(0), scales.stride(1), zeros.stride(0), zeros.stride(1),
                                     groupsize, m, n, k, block_m, block_n, block_k, group_m, split_k)
        out[f"a_{ci}"] = a.numpy()
        out[f"b_{ci}"] = b.numpy()
        out[f"scales_{ci}"] = scales.numpy()
        out[f"zeros_{ci}"] = zeros.numpy()
        out[f"c_{ci}"] = c.numpy()
    np.savez_compressed(os.path.join(HERE, "w4a16.npz"), **out)
    print("w4a16.npz", len(cases), "cases")


if __name__ == "__main__":
    torch.set_num_threads(8)
    golden_argsort()
    golden_route()
    golden_layer()
    golden_w4a16()
