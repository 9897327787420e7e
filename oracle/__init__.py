"""CPU oracle for the fused-routing MoE layer.  TEST INFRASTRUCTURE ONLY.

This package restates, in numpy / CPU torch, the arithmetic of the reference's
hot path (router -> align -> grouped expert GEMMs -> combine).  It is the checker
the CUDA library is compared against; nothing in the product package imports it.
Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may
import it.

Pinning status (what each restatement has been checked against):

* route (stable top-k order + softmax over the selected k):  pinned against the
  reference's own Triton kernels executed on CPU with ``TRITON_INTERPRET=1``
  (``fast_route/fast_route/ops/stable_argsort.py`` and ``ops/stable_route.py``);
  the vectors are committed under ``tests/golden`` with the generating script.
* layer (naive per-expert torch MoE): pinned against the reference function
  ``torch_moe`` (``benchmarks/swizzle_moe/perf_test_moe.py:17-31``) extracted
  from the reference source and executed on CPU; vectors under ``tests/golden``.
* align (``moe_align_block_size``): the arithmetic lives in vLLM 0.4.0.post1
  (``requirements.txt:1``), whose source is not part of the reference tree.  The
  only known answer the reference carries is the docstring example at
  ``fast_route/fast_route/ops/fused_moe.py:151-159``; the restatement reproduces
  it.  Beyond that example: PARITY UNPINNED (no reference test covers it).
* W4A16 split-K GEMM (``w4a16``): pinned against the reference's Triton kernel
  (``benchmarks/splitk_gemm/splitk.py:26-103``) executed on CPU with
  ``TRITON_INTERPRET=1``; vectors under ``tests/golden``.
* softmax-then-top-k routing of the baseline layer (``softmax_topk``): the op is
  ``vllm._moe_C.topk_softmax`` of vLLM 0.4.0.post1, not part of the reference
  tree.  Order rule and source-row formula restate that op's published kernel; the
  weights are only held to the reference's tolerance for it
  (``fast_route/tests/test_route.py:136-143``).  PARITY UNPINNED.
"""

from .route import (exp_recipe, stable_topk, topk_softmax, route_from_hidden,
                    full_argsort_fill, softmax_topk)
from .align import moe_align_block_size
from .moe import silu_and_mul, torch_moe, moe_layer
from . import w4a16

__all__ = [
    "exp_recipe", "stable_topk", "topk_softmax", "route_from_hidden",
    "full_argsort_fill", "softmax_topk", "moe_align_block_size", "silu_and_mul", "torch_moe",
    "moe_layer", "w4a16",
]
