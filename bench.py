#!/usr/bin/env python
"""Benchmark of the fused-routing MoE layer (Mixtral-8x7B shape by default).

    python bench.py --gpus N --steps K --warmup W            # this library, N GPUs of one node
    python bench.py --impl reference --gpus N --steps K ...  # the reference's naive torch MoE on host cores

One JSON line is printed by rank 0.  A step is one pass of the layer over one batch of
synthetic tokens (x ~ N(0,1), weights ~ N(0, 0.02^2), bf16).  With N > 1 the experts are
sharded over the ranks (expert parallel; token rows move by peer-memory loads inside the gather
and combine kernels, or by NCCL all-to-all with --ep-mode nccl) and every rank brings its own
batch of M tokens (weak scaling in tokens).  Every line also carries `parity` (the timed layer's
output checked outside the timed region) and `config5` (Mixtral-8x22B shape, 32768 tokens per
box split over the ranks).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# DRAM bytes of one GEMM1 launch at 16384 tokens, Mixtral-8x7B shape (one-pass ncu capture: 3.20 GB read + 0.95 GB written)
GEMM1_DRAM_BYTES_M16384 = 4.15e9
WORKLOADS = {
    # name: (H, I, E, topk)
    "mixtral-8x7b": (4096, 14336, 8, 2),
    "mixtral-8x22b": (6144, 16384, 8, 2),
    "fine-grained-64e": (2048, 1408, 64, 6),
    # same layer with a Zipf(1.2) preference over experts: the last input feature is the constant 1
    # and carries a per-expert bias in the gate, so the hottest expert gets ~15x the mean load
    "fine-grained-64e-zipf": (2048, 1408, 64, 6),
}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        p["source"] = "measured"
        return p
    p = dict(FALLBACK_PEAKS)
    p["source"] = "fallback"
    return p


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 50 ms while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index=0):
        self.proc = None
        self.path = None
        try:
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            self.sel = ["-i", uuid]
        except Exception:
            self.sel = []

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "50"] + self.sel, stdout=open(self.path, "w"),
                                         stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 8:
                    continue
                try:
                    sm.append(float(parts[0]))
                    mx.append(float(parts[1]))
                    power.append(float(parts[2]))
                except ValueError:
                    continue
                for nm, val in zip(names, parts[4:8]):
                    if val.lower().startswith("active"):
                        reasons.add(nm)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm),
                       power_w_max=max(power))
        return out


def cuda_time_ms(fn, reps, warm=3):
    """Median and min device time of fn() over reps launches (CUDA events on the current stream)."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
    for a, b in evs:
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    ts = sorted(a.elapsed_time(b) for a, b in evs)
    return statistics.median(ts), ts[0]


def cuda_time_quantiles(fn, reps=100, warm=20):
    """(median, p20, p80) device time in ms of fn(), like the reference's do_bench(quantiles=[0.5, 0.2, 0.8])
    (benchmarks/fused_route/moe_bench.py:90-98)."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
    for a, b in evs:
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    ts = sorted(a.elapsed_time(b) for a, b in evs)
    q = lambda f: ts[min(len(ts) - 1, int(f * len(ts)))]
    return q(0.5), q(0.2), q(0.8)


def make_weights(H, I, E, device, seed=0, dtype=torch.bfloat16, experts=None):
    """Random-init weights of the layer (N(0, 0.02^2)), generated on `device`."""
    g = torch.Generator(device=device).manual_seed(seed)
    ne = E if experts is None else len(experts)
    w1 = torch.empty(ne, 2 * I, H, dtype=dtype, device=device)
    w2 = torch.empty(ne, H, I, dtype=dtype, device=device)
    for e in range(ne):
        w1[e].copy_(torch.randn(2 * I, H, generator=g, device=device, dtype=torch.float32) * 0.02)
        w2[e].copy_(torch.randn(H, I, generator=g, device=device, dtype=torch.float32) * 0.02)
    wg = (torch.randn(E, H, generator=g, device=device, dtype=torch.float32) * 0.02).to(dtype)
    return wg, w1, w2


# --------------------------------------------------------------------------------------
# CPU baseline: the reference's naive torch MoE (restated in oracle/), host cores
# --------------------------------------------------------------------------------------
def cpu_reference_rate(H, I, E, k, sample_tokens, reps, warm=1, weights=None, budget_s=None):
    """Tokens/s of the reference's naive layer on the host cores.  One pass = router (fp32 logits,
    stable top-k, softmax over the k) + per-expert masked matmuls, fp32, on `sample_tokens` tokens.
    With `budget_s` the sample is shrunk so that warm + reps passes fit the budget."""
    import oracle
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    if weights is None:
        gen_dev = "cuda" if torch.cuda.is_available() else "cpu"
        wg, w1, w2 = make_weights(H, I, E, gen_dev, seed=0)
    else:
        wg, w1, w2 = weights
    wg, w1, w2 = wg.cpu().float(), w1.cpu().float(), w2.cpu().float()
    gate = wg.t()
    gen = torch.Generator().manual_seed(1)
    probe = torch.randn(64, H, generator=gen)
    oracle.moe_layer(probe, gate, w1, w2, k)          # warms the thread pool
    t0 = time.perf_counter()
    oracle.moe_layer(probe, gate, w1, w2, k)
    per_token = (time.perf_counter() - t0) / 64
    if budget_s is not None:
        fit = int(budget_s / max(per_token, 1e-9) / max(1, warm + reps))
        sample_tokens = max(64, min(sample_tokens, fit // 64 * 64))
    x = torch.randn(sample_tokens, H, generator=gen)
    for _ in range(warm):
        oracle.moe_layer(x, gate, w1, w2, k)
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        oracle.moe_layer(x, gate, w1, w2, k)
        times.append(time.perf_counter() - t0)
    t = statistics.median(times)
    return {"value": sample_tokens / t, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{sample_tokens} tokens of the same layer shape per pass, fp32, median of {reps} passes "
                      f"({t * 1e3:.0f} ms each); router + per-expert masked matmuls as in the reference's torch_moe",
            "ms_per_sample": t * 1e3, "total_s": sum(times)}


def run_reference(args, rank, world):
    """The reference arm: the reference's own CPU path (its naive torch MoE, restated in oracle/
    because the reference tree is not present where the benchmark runs) on all host threads."""
    if rank != 0:
        return
    H, I, E, k = WORKLOADS[args.workload]
    r = cpu_reference_rate(H, I, E, k, args.cpu_tokens, max(1, args.steps), warm=min(args.warmup, 2),
                           budget_s=args.cpu_budget)
    line = {
        "impl": "reference", "metric": "moe_layer_tokens_per_s", "value": r["value"], "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_sample"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{args.workload} MoE layer H={H} I={I} E={E} top-{k}, M={args.tokens} tokens per GPU "
                               f"per step; each CPU step is a bounded sample of that batch (see cpu_baseline.sample)"},
        "cpu_baseline": {k_: r[k_] for k_ in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": r["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------
# this library
# --------------------------------------------------------------------------------------
def sweep_single_gpu(fr, synth, wg, w1, w2, H, I, E, k, peaks, Ms):
    """Layer time vs M.  `ms` is the eager call (Python + 6-8 launches per call); `ms_graph` replays
    the same call captured in a CUDA graph (no host work between kernels) - the number the
    roofline fractions use, since at small M the eager time is host launch overhead."""
    rows = []
    dev = w1.device
    for M in Ms:
        x = torch.randn(M, H, device=dev, dtype=w1.dtype)
        _, _, ti = fr.fused_moe(x, wg.t(), w1, w2, k, return_routing=True)
        active = int(torch.unique(ti).numel())
        # timing protocol of the reference's benches: >= 20 warm-up calls, 100 timed calls, median / p20 / p80
        reps = 100 if M <= 4096 else 40
        med, m20, m80 = cuda_time_quantiles(lambda: fr.fused_moe(x, wg.t(), w1, w2, k), reps, 20 if M <= 4096 else 5)
        out = torch.empty_like(x)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            out = fr.fused_moe(x, wg.t(), w1, w2, k)
        gmed, g20, g80 = cuda_time_quantiles(g.replay, reps, 20 if M <= 4096 else 5)
        flops = synth.layer_flops(M, H, I, E, k)
        nbytes = synth.layer_bytes(active, M, H, I, E)
        # rates from the faster of the two medians: at large M both run the same kernels and differ only by how
        # far the power cap had pulled the clock down when their 100 calls ran
        best = min(med, gmed)
        rows.append({"M": M, "ms": round(med, 4), "ms_p20_p80": [round(m20, 4), round(m80, 4)],
                     "ms_graph": round(gmed, 4), "ms_graph_p20_p80": [round(g20, 4), round(g80, 4)],
                     "tokens_per_s": M / best * 1e3,
                     "tflops": flops / best / 1e9, "frac_tensor_peak": flops / best / 1e9 / peaks["bf16_tflops"],
                     "active_experts": active, "hbm_gbs": nbytes / best / 1e6,
                     "frac_hbm_peak": nbytes / best / 1e6 / peaks["hbm_gbs"],
                     "ref_convention_tflops": 2.0 * M * I * H / best / 1e9})
        del g
    return rows


def transformer_block(fr, wg, w1, w2, M, H, k):
    """Mixtral-style block tail: h = attn_out + x; out = h + moe(rmsnorm(h) * gamma).  Fused (one C call:
    add+norm kernel, residual inside the combine kernel) against the same math with framework ops around
    the layer."""
    dev, dt = w1.device, w1.dtype
    attn = torch.randn(M, H, device=dev, dtype=dt) * 0.5
    x = torch.randn(M, H, device=dev, dtype=dt)
    gamma = torch.ones(H, device=dev, dtype=dt)

    def fused():
        return fr.moe_block(attn, x, wg.t(), w1, w2, k, gamma=gamma, add_residual=True)

    def unfused():
        h = attn + x
        u = torch.nn.functional.rms_norm(h, (H,), gamma, 1e-5)
        return h + fr.fused_moe(u, wg.t(), w1, w2, k)
    fs, us = [], []
    for _ in range(3):          # interleaved, so clock drift under the power cap hits both alike
        fs.append(cuda_time_ms(fused, 4, warm=1)[0])
        us.append(cuda_time_ms(unfused, 4, warm=1)[0])
    return {"tokens": M, "ms_fused_block": statistics.median(fs), "ms_layer_plus_framework_ops": statistics.median(us)}


def fp8_points(fr, synth, wg, w1, w2, H, I, E, k, peaks):
    """The optional E4M3-weight mode of the layer (not the headline: that stays bf16)."""
    w1_q, s1, w2_q, s2 = fr.quantize_experts_fp8(w1, w2)
    rows = []
    for M in (1, 16, 256, 4096, 16384):
        x = torch.randn(M, H, device=w1.device, dtype=w1.dtype)
        _, _, ti = fr.fused_moe_fp8(x, wg.t(), w1_q, s1, w2_q, s2, k, return_routing=True)
        active = int(torch.unique(ti).numel())
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fr.fused_moe_fp8(x, wg.t(), w1_q, s1, w2_q, s2, k)
        ms, _ = cuda_time_ms(g.replay, 20 if M <= 256 else 8)
        del g
        nbytes = active * 3.0 * H * I + 2.0 * M * H * 2 + H * E * 2          # weights are one byte each
        rows.append({"M": M, "ms_graph": round(ms, 4), "tokens_per_s": M / ms * 1e3,
                     "tflops": synth.layer_flops(M, H, I, E, k) / ms / 1e9, "hbm_gbs": nbytes / ms / 1e6,
                     "frac_hbm_peak": nbytes / ms / 1e6 / peaks["hbm_gbs"]})
    return rows


def routing_latency(fr, synth, dev):
    from fast_route_b200 import _lib
    lib = _lib.load()
    out = []
    for E, k in ((8, 2), (64, 6), (128, 8)):
        M, bs = 16384, 64
        lg = synth.routing_logits(M, E, k, seed=1, dtype=torch.float16).to(dev)
        n = M * k
        w = torch.empty(M, k, dtype=torch.float32, device=dev)
        ids = torch.empty(M, k, dtype=torch.int32, device=dev)
        s = torch.empty(n + E * (bs - 1), dtype=torch.int32, device=dev)
        e = torch.empty(n + E, dtype=torch.int32, device=dev)
        npost = torch.empty(1, dtype=torch.int32, device=dev)

        ws = torch.zeros(lib.fr_align_workspace_bytes(E), dtype=torch.uint8, device=dev)   # zeroed once

        def call():
            rc = lib.fr_route_align(_lib.ptr(lg), 0, M, E, lg.stride(0), 1, k, _lib.ptr(w), _lib.ptr(ids), bs,
                                    _lib.ptr(s), s.numel(), _lib.ptr(e), e.numel(), _lib.ptr(npost), _lib.ptr(ws),
                                    ws.numel(), _lib.stream_ptr(dev))
            assert rc == 0, rc
        med, _ = cuda_time_ms(call, 50, 5)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            call()
        gmed, _ = cuda_time_ms(g.replay, 50, 5)

        def call_topk():
            rc = lib.fr_topk_softmax(_lib.ptr(lg), 0, M, E, lg.stride(0), 1, k, 1, _lib.ptr(w), k, _lib.ptr(ids), k, 0,
                                     _lib.stream_ptr(dev))
            assert rc == 0, rc

        def call_align():
            rc = lib.fr_align(_lib.ptr(ids), n, E, bs, _lib.ptr(s), s.numel(), _lib.ptr(e), e.numel(), _lib.ptr(npost),
                              None, None, _lib.ptr(ws), ws.numel(), _lib.stream_ptr(dev))
            assert rc == 0, rc
        parts = []
        for fn in (call_topk, call_align):
            gg = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gg):
                for _ in range(10):
                    fn()
            parts.append(cuda_time_ms(gg.replay, 20, 3)[0] * 100.0)   # us per launch (10 launches per replay)
        nbytes = M * E * 2 + M * k * 8 + M * k * 4 + 4 * (int(npost.item()) + int(npost.item()) // bs + 1)
        out.append({"tokens": M, "E": E, "topk": k, "block": bs, "us": med * 1e3, "us_graph": gmed * 1e3,
                    "us_topk_kernel": parts[0], "us_align_kernel": parts[1], "algorithmic_bytes": nbytes})
    return out


def w4a16_splitk(dev, peaks):
    """The reference's W4A16 split-K GEMM (benchmarks/splitk_gemm/splitk.py: m=16, k=n=4096, group 128) and
    neighbours in m.  HBM-bound on the packed weights; 20 weight sets (173 MB > L2) are cycled inside one CUDA
    graph so every launch streams its weights from DRAM.  The dense fp16 matmul of the framework on the
    dequantised matrix is timed beside it for scale."""
    from fast_route_b200.ops import splitk_gemm as sk
    gs = 128
    g = torch.Generator(device=dev).manual_seed(3)
    rows = []
    # the reference's driver shape, and a large FFN-sized matrix (117 MB packed) where the kernel is in steady state
    for k, n, sets, ms in ((4096, 4096, 20, (1, 16, 64, 256)), (8192, 28672, 2, (16,))):
        bs = [torch.randint(-2**31, 2**31 - 1, (k // 8, n), generator=g, device=dev, dtype=torch.int64).to(torch.int32)
              for _ in range(sets)]
        zs = [torch.randint(-2**31, 2**31 - 1, (k // gs, n // 8), generator=g, device=dev, dtype=torch.int64)
              .to(torch.int32) for _ in range(sets)]
        ss = [(torch.randn(k // gs, n, generator=g, device=dev) * 0.5).half() for _ in range(sets)]
        dense = [sk.dequantize(bs[i], ss[i], zs[i], gs) for i in range(sets)]
        for m in ms:
            a = (torch.randn(m, k, generator=g, device=dev) * 0.5).half()
            c = torch.empty(m, n, dtype=torch.float16, device=dev)
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                for i in range(sets):
                    sk.matmul_split_k(a, bs[i], ss[i], zs[i], gs, out=c)
            us = cuda_time_ms(gr.replay, 20, 3)[0] * 1e3 / sets
            torch.matmul(a, dense[0], out=c)          # library handle and workspace exist before the capture
            torch.cuda.synchronize()
            gd = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gd):
                for i in range(sets):
                    torch.matmul(a, dense[i], out=c)
            us_dense = cuda_time_ms(gd.replay, 20, 3)[0] * 1e3 / sets
            gl = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gl):
                for i in range(sets):
                    sk.matmul_split_k(a, bs[0], ss[0], zs[0], gs, out=c)
            us_l2 = cuda_time_ms(gl.replay, 20, 3)[0] * 1e3 / sets
            del gr, gd, gl
            nbytes = k * n // 2 + (k // gs) * n * 2 + (k // gs) * (n // 8) * 4 + m * k * 2 + m * n * 2
            rows.append({"m": m, "k": k, "n": n, "groupsize": gs, "us": round(us, 3),
                         "us_same_weights_every_launch": round(us_l2, 3),
                         "us_dense_fp16_framework_matmul": round(us_dense, 3), "algorithmic_bytes": nbytes,
                         "hbm_gbs": nbytes / us / 1e3, "frac_hbm_peak": nbytes / us / 1e3 / peaks["hbm_gbs"],
                         "tflops": 2.0 * m * n * k / us / 1e6})
        del bs, zs, ss, dense
    return rows


def gemm1_roofline(fr, synth, wg, w1, w2, M, H, I, E, k, peaks, reps):
    """Times the dominant kernel (grouped GEMM 1 + SiLU*mul epilogue) alone through the C ABI."""
    from fast_route_b200.ops import fused_moe as fm
    dev = w1.device
    x = torch.randn(M, H, device=dev, dtype=w1.dtype)
    tw, ti = fr.fused_route(x, wg.t(), k)
    s, e, npost, cnt, inv = fm.moe_align_block_size(ti, 128, E, return_extra=True)
    n = M * k
    rows = (n + min(n, E) * 127 + 127) // 128 * 128
    a = fm.permute_rows(x, s, npost, k, max_rows=rows)
    med, mn = cuda_time_ms(lambda: fm.gemm1_silu(a, w1, e, npost, s, n), reps)
    flops = 4.0 * n * H * I
    # the framework's dense bf16 matmul with the same FLOPs ([n, H] x [H, 2I], one expert's weights), timed right after
    # on the same GPU: what the library reaches here and now, beside the figure from MEASURED_PEAKS.json
    lib_tflops = None
    try:
        c = torch.empty(n, 2 * I, dtype=a.dtype, device=dev)
        wt = w1[0].t()
        lib_ms, _ = cuda_time_ms(lambda: torch.matmul(a[:n], wt, out=c), reps)
        lib_tflops = flops / lib_ms / 1e9
        med2, _ = cuda_time_ms(lambda: fm.gemm1_silu(a, w1, e, npost, s, n), reps)     # ours again: clock drift shows
        med = min(med, med2)
        del c
    except Exception:
        pass
    extra = {}
    if lib_tflops:
        extra = {"library_matmul_same_flops_tflops": lib_tflops, "frac_of_library_matmul_same_run": flops / med / 1e9 / lib_tflops}
    return {**extra, "bound": "tensor", "kernel": "grouped_gemm_kernel<256,4,SILU,bf16> (GEMM1 + SiLU*mul)",
            "achieved": flops / med / 1e9, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
            "frac": flops / med / 1e9 / peaks["bf16_tflops"],
            "frac_of_sustained_peak": flops / med / 1e9 / peaks["bf16_tflops_sustained"],
            "frac_of_datasheet_peak": flops / med / 1e9 / 2250.0,
            "peak_source": peaks["source"] + " (burst cuBLAS bf16; kernel timed alone)",
            "ms_per_launch": med, "algorithmic_flops_per_launch": flops, "traffic": None}


def stage_times_single_gpu(fr, wg, w1, w2, M, H, I, E, k, reps=5):
    """CUDA-event time of every stage of the layer under the reference's stage names
    (fast_route/fast_route/layers/profile_fused_route.py:61-121: route, moe_align, moe_1, silu_and_mul, moe_2),
    each stage issued alone through the operator surface; silu_and_mul is part of moe_1 here and `gather` /
    `combine` are the two memory-bound passes around the GEMMs."""
    from fast_route_b200.ops import fused_moe as fm
    dev = w1.device
    x = torch.randn(M, H, device=dev, dtype=w1.dtype)
    n = M * k
    rows = (n + min(n, E) * 127 + 127) // 128 * 128
    tw, ti = fr.fused_route(x, wg.t(), k)
    s, e, npost, cnt, inv = fm.moe_align_block_size(ti, 128, E, return_extra=True)
    a = fm.permute_rows(x, s, npost, k, max_rows=rows)
    act = fm.gemm1_silu(a, w1, e, npost, s, n)
    y = fm.gemm2(act, w2, e, npost, s, tw, n)
    out = {}
    out["route"] = cuda_time_ms(lambda: fr.fused_route(x, wg.t(), k), reps, 2)[0]
    out["moe_align"] = cuda_time_ms(lambda: fm.moe_align_block_size(ti, 128, E, return_extra=True), reps, 2)[0]
    out["gather"] = cuda_time_ms(lambda: fm.permute_rows(x, s, npost, k, max_rows=rows), reps, 2)[0]
    out["moe_1+silu_and_mul"] = cuda_time_ms(lambda: fm.gemm1_silu(a, w1, e, npost, s, n), reps, 2)[0]
    out["moe_2"] = cuda_time_ms(lambda: fm.gemm2(act, w2, e, npost, s, tw, n), reps, 2)[0]
    out["combine"] = cuda_time_ms(lambda: fm.combine(y, inv, M, k), reps, 2)[0]
    return {k_: round(v, 4) for k_, v in out.items()}


def routing_latency_with_clocks(fr, synth, dev, device_index):
    sampler = ClockSampler(device_index)
    sampler.start()
    rows = routing_latency(fr, synth, dev)
    return {"rows": rows, "clocks": sampler.stop()}


def router_from_hidden_states(fr, dev, dtype):
    """The reference's router op bench (benchmarks/fused_route/op_bench.py:62-130): fused_route from hidden
    states [m, 4096] to the top-k weights / ids, swept over the batch and the expert count."""
    rows = []
    K = 4096
    g = torch.Generator(device=dev).manual_seed(11)
    for E, k in ((8, 2), (64, 6), (128, 8)):
        gate = (torch.randn(E, K, device=dev, generator=g) * 0.02).to(dtype)
        for m in (1, 64, 1024, 4096, 16384):
            x = torch.randn(m, K, device=dev, dtype=dtype, generator=g)
            gr = torch.cuda.CUDAGraph()
            fr.fused_route(x, gate.t(), k)
            torch.cuda.synchronize()
            with torch.cuda.graph(gr):
                fr.fused_route(x, gate.t(), k)
            us = cuda_time_ms(gr.replay, 30, 5)[0] * 1e3
            del gr
            nbytes = m * K * 2 + E * K * 2 + m * k * 8
            rows.append({"tokens": m, "E": E, "topk": k, "us": round(us, 2), "hbm_gbs": nbytes / us / 1e3})
    return rows


def bind_to_gpu_numa_node(index):
    """Pins this process to the CPUs of the NUMA node the GPU hangs off, so that the pinned host buffers it allocates
    next (first touch) and the copy threads sit next to the GPU's PCIe root.  Returns the node or None."""
    try:
        p = torch.cuda.get_device_properties(index)
        bdf = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        node = int(open(f"/sys/bus/pci/devices/{bdf}/numa_node").read())
        if node < 0:
            return None
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        cpus &= os.sched_getaffinity(0)
        if not cpus:
            return None
        os.sched_setaffinity(0, cpus)
        return node
    except Exception:
        return None


def fp32_rows(x, tw, ti, w1, w2, rows):
    """Direct fp32 evaluation of the layer for a few token rows on the device (full experts in w1 / w2)."""
    I = w1.shape[1] // 2
    ref = torch.zeros(len(rows), x.shape[1], device=x.device)
    term_max = torch.zeros_like(ref)          # largest per-expert term of every output element
    cache = {}
    for i, r in enumerate(rows):
        for j in range(ti.shape[1]):
            e = int(ti[r, j])
            if e not in cache:
                if len(cache) >= 3:
                    cache.clear()
                cache[e] = (w1[e].float(), w2[e].float())
            a1, a2 = cache[e]
            h1 = a1 @ x[r].float()
            term = tw[r, j] * (a2 @ (torch.nn.functional.silu(h1[:I]) * h1[I:]))
            ref[i] += term
            term_max[i] = torch.maximum(term_max[i], term.abs())
    return ref, term_max


def parity_report(fr, layer, x, wg, w1_full, w2_full, k, world, dist):
    """Outside every timed region: the timed layer's output against (a) a direct fp32 evaluation of sampled token
    rows and (b), with N > 1, the single-GPU layer on this rank's tokens with all experts loaded; routing ids
    against a stable descending sort of the device's own logits.  Maxima / minima are taken over the ranks."""
    dev = x.device
    M = x.shape[0]
    out = layer(x)
    tw, ti, logits = fr.fused_route(x, wg.t(), k, return_logits=True)
    order = torch.sort(logits, dim=1, descending=True, stable=True)
    ids_ok = bool(torch.equal(order[1][:, :k].to(torch.int32), ti))
    wt = torch.softmax(order[0][:, :k], dim=-1)
    rows = sorted(set(list(range(0, M, max(1, M // 8)))[:8] + [M - 1]))
    ref, term_max = fp32_rows(x, tw, ti, w1_full, w2_full, rows)
    diff = (out[rows].float() - ref).abs()
    big = torch.maximum(ref.abs(), term_max)
    ref_rms = float(ref.pow(2).mean().sqrt())
    rep = {"rows": len(rows), "max_abs": float(diff.max()), "mean_rel": float(diff.mean() / ref.abs().mean()),
           "ref_abs_max": float(ref.abs().max()), "ref_rms": ref_rms, "max_abs_over_ref_rms": float(diff.max()) / ref_rms,
           "frac_within_flat_2e-2": float((diff <= 2e-2).float().mean()),
           "within_2e-2_plus_one_bf16_spacing": bool((diff <= 2e-2 + ref.abs() * 2.0 ** -7).all()),
           "within_2e-2_plus_one_bf16_spacing_of_largest_term": bool((diff <= 2e-2 + big * 2.0 ** -7).all()),
           "ids_bit_exact": ids_ok, "weights_max_abs_vs_softmax": float((tw - wt).abs().max()),
           "note": "reference = direct fp32 evaluation of the sampled token rows on the device; the flat 2e-2 is stated "
                   "for outputs of order 0.2 (the reference's CPU case); here one bf16 spacing of an output is "
                   "|value| / 128, and the layer, like the reference, keeps each token's per-expert terms in bf16 "
                   "before it sums them (largest term = the larger of |output| and the per-expert terms)"}
    if world > 1:
        single = fr.fused_moe(x, wg.t(), w1_full, w2_full, k)
        d = (out.float() - single.float()).abs().max()
        stats = torch.tensor([rep["max_abs"], rep["mean_rel"], float(d), 0.0 if torch.equal(out, single) else 1.0,
                              0.0 if ids_ok else 1.0, 1.0 - rep["frac_within_flat_2e-2"],
                              0.0 if rep["within_2e-2_plus_one_bf16_spacing"] else 1.0,
                              0.0 if rep["within_2e-2_plus_one_bf16_spacing_of_largest_term"] else 1.0], device=dev)
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        v = stats.tolist()
        rep.update({"max_abs": v[0], "mean_rel": v[1], "ep_vs_single_gpu_max_abs": v[2],
                    "ep_vs_single_gpu_bit_equal": v[3] == 0.0, "ids_bit_exact": v[4] == 0.0,
                    "frac_within_flat_2e-2": 1.0 - v[5], "within_2e-2_plus_one_bf16_spacing": v[6] == 0.0,
                    "within_2e-2_plus_one_bf16_spacing_of_largest_term": v[7] == 0.0,
                    "over": "max over ranks"})
    return rep


def timed_layer_steps(layer, xs, steps, warmup, barrier, world, dist, dev):
    """W warm-up and K timed steps bracketed by barrier + synchronize; device time, max over ranks (ms per step)."""
    for i in range(warmup):
        layer(xs[i % len(xs)])
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for i in range(steps):
        layer(xs[i % len(xs)])
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms / steps


def make_layer(fr, ep, group, world, wg, w1_full, w2_full, k, ep_mode):
    """(layer(x) -> out, local expert weights, kernel launches per step) for this rank."""
    if world == 1:
        return (lambda xb: fr.fused_moe(xb, wg.t(), w1_full, w2_full, k)), w1_full, w2_full, 6
    lo, hi = group.local_expert_range()
    w1, w2 = w1_full[lo:hi], w2_full[lo:hi]          # contiguous slices of the full tensors
    if ep_mode == "p2p":
        return (lambda xb: ep.fused_moe_ep_p2p(xb, wg.t(), w1, w2, k, group)), w1, w2, 7
    return (lambda xb: ep.fused_moe_ep(xb, wg.t(), w1, w2, k, group)), w1, w2, 12


def config5_point(fr, ep, synth, group, world, rank, dev, dtype, peaks, steps, warmup, barrier, dist, ep_mode, single_ms):
    """Expert-parallel Mixtral-8x22B-shaped layer: 32768 tokens per box split evenly over the ranks, experts sharded
    E/W per rank, device-timed max over ranks, with the stages timed by CUDA events in a separate pass."""
    H, I, E, k = WORKLOADS["mixtral-8x22b"]
    box_tokens = 32768
    M = box_tokens // world
    wg, w1_full, w2_full = make_weights(H, I, E, dev, seed=5)
    layer, w1, w2, launches = make_layer(fr, ep, group, world, wg, w1_full, w2_full, k, ep_mode)
    g = torch.Generator(device=dev).manual_seed(500 + rank)
    xs = [torch.randn(M, H, device=dev, dtype=dtype, generator=g) for _ in range(2)]
    if world > 1 and ep_mode == "p2p":            # tokens resident in the rank's peer region (see run_ours)
        x0 = ep.peer_input(group, M, H, k, dtype, dev)
        x0.copy_(xs[0])
        xs = [x0, x0]
    ms = timed_layer_steps(layer, xs, steps, warmup, barrier, world, dist, dev)
    flops = synth.layer_flops(box_tokens, H, I, E, k)
    rep = {"workload": f"mixtral-8x22b MoE layer H={H} I={I} E={E} top-{k}, {box_tokens} tokens per box = {M} per rank, "
                       f"experts sharded {E // world} per rank", "n_gpus": world, "steps": steps, "warmup": warmup,
           "ms_per_step": ms, "tokens_per_s": box_tokens / ms * 1e3, "tflops": flops / ms / 1e9,
           "frac_of_n_x_sustained_peak": flops / ms / 1e9 / (peaks["bf16_tflops_sustained"] * world),
           "frac_of_n_x_burst_peak": flops / ms / 1e9 / (peaks["bf16_tflops"] * world),
           "scaling": "strong (total work fixed)", "timing": "CUDA events, max over ranks"}
    # stage times: a separate pass with events between the stages (max over ranks of each stage's median)
    if world > 1 and ep_mode == "p2p":
        acc = {}
        for i in range(4):
            timers = []
            ep.fused_moe_ep_p2p(xs[i % 2], wg.t(), w1, w2, k, group, timers=timers)
            torch.cuda.synchronize()
            if i:                      # first pass warms the event path
                for name, a, b in timers:
                    acc.setdefault(name, []).append(a.elapsed_time(b))
        names = list(acc)
        t = torch.tensor([statistics.median(acc[nm]) for nm in names], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        rep["stage_ms_max_over_ranks"] = {nm: round(v, 4) for nm, v in zip(names, t.tolist())}
    elif world == 1:
        rep["stage_ms"] = stage_times_single_gpu(fr, wg, w1_full, w2_full, M, H, I, E, k)
    rep["parity"] = parity_report(fr, layer, xs[0], wg, w1_full, w2_full, k, world, dist)
    del xs, w1_full, w2_full
    return rep


def host_copy_ceiling(M, H, dtype, dev, steps, barrier, world, dist):
    """What the host side alone sustains: every rank copies one batch in and one batch out per step, concurrently,
    with no compute.  ms per step, max over ranks."""
    hx = torch.randn(M, H, dtype=dtype).pin_memory()
    ho = torch.empty(M, H, dtype=dtype).pin_memory()
    dx = torch.empty(M, H, dtype=dtype, device=dev)
    dy = torch.empty(M, H, dtype=dtype, device=dev)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

    def step():
        with torch.cuda.stream(s_in):
            dx.copy_(hx, non_blocking=True)
        with torch.cuda.stream(s_out):
            ho.copy_(dy, non_blocking=True)
    step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    torch.cuda.synchronize()
    ms = (time.perf_counter() - t0) * 1e3 / steps
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def run_ours(args, rank, world, local_rank):
    import fast_route_b200 as fr
    from fast_route_b200 import synth, _lib
    import torch.distributed as dist

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    H, I, E, k = WORKLOADS[args.workload]
    M = args.tokens
    peaks = load_peaks()
    dtype = torch.bfloat16

    if args.routing_only:
        print(json.dumps({"routing_latency": routing_latency(fr, synth, dev)}), flush=True)
        return
    if args.w4a16_only:
        print(json.dumps({"w4a16_splitk_gemm": w4a16_splitk(dev, peaks)}), flush=True)
        return

    numa_node = None
    ep = group = None
    # every rank holds the full expert set (same seed): its own shard is a slice of it, and the parity check
    # outside the timed region runs the single-GPU layer on the rank's tokens against it
    wg, w1_full, w2_full = make_weights(H, I, E, dev, seed=0)
    if world > 1:
        # one process per GPU: keep each process (and the pinned buffers it allocates) on its GPU's NUMA node
        numa_node = bind_to_gpu_numa_node(local_rank)
        from fast_route_b200.parallel import ep
        assert E % world == 0, "experts must divide over the ranks"
        group = ep.ExpertParallelGroup(dist.group.WORLD, E)
        if args.ep_mode == "p2p":
            # symmetric memory needs peer access between all GPUs of the node; whether it works is decided by
            # ALL ranks together, so that nobody is left alone in a collective of the other mode
            ok = torch.ones(1, device=dev)
            try:
                lo, hi = group.local_expert_range()
                ep.fused_moe_ep_p2p(torch.zeros(M, H, device=dev, dtype=dtype), wg.t(), w1_full[lo:hi], w2_full[lo:hi],
                                    k, group)
                torch.cuda.synchronize()
            except Exception as err:
                ok.zero_()
                print(f"rank {rank}: peer-memory path unavailable ({err})", file=sys.stderr)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if ok.item() == 0:
                args.ep_mode = "nccl"
    layer, w1, w2, launches_per_step = make_layer(fr, ep, group, world, wg, w1_full, w2_full, k, args.ep_mode)

    # The routing microbenchmark is a latency measurement of two tiny kernels, so it scales with the SM clock and the
    # clock depends on what ran before: it is taken here, before the GEMM loops push the GPU into its power cap, and
    # once more after them (`routing_latency_after_load`), each with the clock sampled beside it.
    routing_first = None
    if world == 1 and not args.no_sweep and not args.profile and args.workload == "mixtral-8x7b":
        routing_first = routing_latency_with_clocks(fr, synth, dev, local_rank)

    g = torch.Generator(device=dev).manual_seed(100 + rank)
    xs = [torch.randn(M, H, device=dev, dtype=dtype, generator=g) for _ in range(3)]
    if world > 1 and args.ep_mode == "p2p":
        # device-resident tokens of an expert-parallel rank live where its peers can read them: the token buffer of
        # the rank's peer region (one buffer, so every step reads the same batch; the weights, not the tokens, are
        # what exceeds the L2)
        x0 = ep.peer_input(group, M, H, k, dtype, dev)
        x0.copy_(xs[0])
        xs = [x0, x0, x0]
    if args.workload.endswith("-zipf"):
        wg[:, H - 1] = synth.zipf_gate_bias(E, 1.2, 1.6).to(device=dev, dtype=dtype)
        for xb in xs:
            xb[:, H - 1] = 1.0

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident throughput -------------------------------------------------
    for i in range(args.warmup):
        layer(xs[i % 3])
    barrier()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for i in range(args.steps):
        layer(xs[i % 3])
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if sampler else None
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_per_step = ms / args.steps
    total_tokens = M * world
    value = total_tokens / ms_per_step * 1e3
    _lib.raise_on_device_error()
    if world == 1:
        _, _, ti0 = fr.fused_moe(xs[0], wg.t(), w1, w2, k, return_routing=True)
        load = torch.bincount(ti0.flatten().long(), minlength=E).float()
        expert_load = {"max_over_mean": float(load.max() / load.mean()), "experts_without_tokens": int((load == 0).sum())}
    else:
        expert_load = None

    if args.profile:
        if rank == 0:
            print(json.dumps({"profile_run": True, "ms_per_step": ms_per_step, "tokens_per_s": value}), flush=True)
        return

    # ---- parity of the very configuration that was timed (outside the timed region) ---
    parity = parity_report(fr, layer, xs[0], wg, w1_full, w2_full, k, world, dist)
    _lib.raise_on_device_error()

    # ---- end to end through the public API with host buffers ------------------------
    # Every step copies its own input batch from pinned host memory and its result back.  The calls are pipelined
    # the way a serving loop issues them: step i+1's input travels while step i computes, step i's result travels
    # while step i+1 computes; the timed region ends after the last result has arrived.
    hx = [torch.randn(M, H, dtype=dtype).pin_memory() for _ in range(2)]
    hout = [torch.empty(M, H, dtype=dtype).pin_memory() for _ in range(2)]

    def e2e_step(i):
        if world == 1:
            fr.fused_moe_host(hx[i % 2], wg.t(), w1, w2, k, out_host=hout[i % 2], chunk=M, pipelined=True)
        else:
            ep.fused_moe_ep_host(hx[i % 2], wg.t(), w1, w2, k, group, out_host=hout[i % 2],
                                 p2p=(args.ep_mode == "p2p"), pipelined=True)
    for i in range(max(1, min(args.warmup, 3))):
        e2e_step(i)
    fr.fused_moe_host_wait(dev)
    barrier()
    e0.record()
    for i in range(args.steps):
        e2e_step(i)
    fr.fused_moe_host_wait(dev)
    e1.record()
    barrier()
    ems = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ems], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ems = float(t.item())
    e2e = {"value": total_tokens / (ems / args.steps) * 1e3, "unit": "tokens/s",
           "h2d_bytes_per_step": M * H * 2 * world, "d2h_bytes_per_step": M * H * 2 * world,
           "ms_per_step": ems / args.steps, "mode": "pipelined calls (copies of neighbouring steps overlap the compute)"}
    if world == 1:
        # one isolated call at a time: copy in, layer, copy out, synchronise (copies chunked inside the call)
        def isolated():
            fr.fused_moe_host(hx[0], wg.t(), w1, w2, k, out_host=hout[0])
            torch.cuda.synchronize()
        isolated()
        ts = []
        for _ in range(5):
            t0 = time.perf_counter()
            isolated()
            ts.append((time.perf_counter() - t0) * 1e3)
        e2e["isolated_call_ms"] = statistics.median(ts)
        e2e["isolated_call_tokens_per_s"] = M / statistics.median(ts) * 1e3
    copy_ms = host_copy_ceiling(M, H, dtype, dev, max(3, args.steps // 2), barrier, world, dist)
    e2e["host_copies_alone_ms_per_step"] = copy_ms
    e2e["host_copy_ceiling_tokens_per_s"] = total_tokens / copy_ms * 1e3
    e2e["frac_of_min_of_device_and_copy_ceiling"] = e2e["value"] / min(value, total_tokens / copy_ms * 1e3)
    if numa_node is not None:
        e2e["host_numa_node_rank0"] = numa_node
    del hx, hout

    # ---- the expert-parallel configuration of the scaling study (every N, N = 1 included) ----
    config5 = None
    if args.workload == "mixtral-8x7b" and not args.no_config5 and 8 % world == 0:
        config5 = config5_point(fr, ep, synth, group, world, rank, dev, dtype, peaks, max(5, args.steps // 2),
                                3, barrier, dist, args.ep_mode, None)
        _lib.raise_on_device_error()

    if rank != 0:
        return
    flops = synth.layer_flops(total_tokens, H, I, E, k)
    line = {
        "metric": "moe_layer_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{args.workload} MoE layer H={H} I={I} E={E} top-{k}, M={M} tokens per GPU per step",
                   "parallelism": "single GPU" if world == 1 else
                   f"expert parallel ep{world} + token data parallel, rows moved by {args.ep_mode}",
                   "l2": f"expert weights ({3.0 * E * H * I * 2 / 1e9:.1f} GB) and activations far exceed the 126 MB L2; "
                         "no explicit flush",
                   "tokens_per_step_total": total_tokens},
        "tflops": flops / ms_per_step / 1e9,
        "frac_tensor_peak": flops / ms_per_step / 1e9 / (peaks["bf16_tflops_sustained"] * world),
        "frac_tensor_peak_note": f"of {peaks['source']} sustained cuBLAS bf16 ({peaks['bf16_tflops_sustained']} TF/GPU)",
        "clocks": clocks, "e2e": e2e, "gpu_launches": launches_per_step * args.steps, "expert_load": expert_load,
        "parity": parity,
    }
    if config5 is not None:
        line["config5"] = config5
    if world == 1:
        line["roofline"] = gemm1_roofline(fr, synth, wg, w1, w2, M, H, I, E, k, peaks, reps=max(5, args.steps))
        if args.workload == "mixtral-8x7b" and M == 16384:
            line["roofline"]["traffic"] = GEMM1_DRAM_BYTES_M16384
            line["roofline"]["traffic_note"] = ("dram__bytes_read.sum + dram__bytes_write.sum of one GEMM1 launch at "
                                                "this size from a one-pass ncu capture (not measured in this run); "
                                                "algorithmic bytes are 2.16 GB read (weights + A once) + 0.97 GB written")
        if not args.no_sweep and args.workload == "mixtral-8x7b":
            Ms = [2 ** i for i in range(15)]          # the reference's sweep, benchmarks/fused_route/moe_bench.py:53
            line["sweep"] = sweep_single_gpu(fr, synth, wg, w1, w2, H, I, E, k, peaks, Ms)
            line["stage_ms"] = stage_times_single_gpu(fr, wg, w1, w2, M, H, I, E, k)
            line["routing_latency"] = routing_first["rows"]
            line["routing_latency_clocks"] = routing_first["clocks"]
            after = routing_latency_with_clocks(fr, synth, dev, local_rank)
            line["routing_latency_after_load"] = [
                {k_: r[k_] for k_ in ("tokens", "E", "topk", "block", "us", "us_graph")} for r in after["rows"]]
            line["routing_latency_after_load_clocks"] = after["clocks"]
            line["router_from_hidden_states"] = router_from_hidden_states(fr, dev, dtype)
            line["transformer_block"] = transformer_block(fr, wg, w1, w2, M, H, k)
            line["fp8_weights_mode"] = fp8_points(fr, synth, wg, w1, w2, H, I, E, k, peaks)
            line["w4a16_splitk_gemm"] = w4a16_splitk(dev, peaks)
        if not args.no_cpu:
            cb = cpu_reference_rate(H, I, E, k, args.cpu_tokens, 3, warm=1, weights=(wg, w1, w2), budget_s=20.0)
            line["cpu_baseline"] = {k_: cb[k_] for k_ in ("value", "unit", "cores", "kind", "sample")}
            # the reference's own CPU-runnable case (fp32, 256 tokens, H=1024, I=2048, 8 experts, top-2)
            c1 = cpu_reference_rate(1024, 2048, 8, 2, 256, 10, warm=3)
            line["cpu_reference_small_case"] = {
                "value": c1["value"], "unit": "tokens/s", "cores": c1["cores"], "ms": c1["ms_per_sample"],
                "gflops": (2.0 * 1024 * 8 + 6.0 * 2 * 1024 * 2048) * c1["value"] / 1e9,
                "config": "M=256 H=1024 I=2048 E=8 top-2 fp32, 3 warm-up + 10 timed passes, median"}
    _lib.raise_on_device_error()
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="mixtral-8x7b", choices=sorted(WORKLOADS))
    ap.add_argument("--tokens", "-m", type=int, default=16384, help="tokens per GPU per step")
    ap.add_argument("--cpu-tokens", type=int, default=1024, help="tokens in the CPU baseline's sample")
    ap.add_argument("--cpu-budget", type=float, default=120.0,
                    help="seconds the reference arm may spend in its timed passes (the sample shrinks to fit)")
    ap.add_argument("--ep-mode", default="p2p", choices=["p2p", "nccl"],
                    help="N > 1: token rows move by peer-memory loads inside the gather / combine kernels (p2p) "
                         "or through NCCL all-to-all send/receive buffers (nccl)")
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-config5", action="store_true",
                    help="skip the Mixtral-8x22B expert-parallel point (32768 tokens per box) added to every line")
    ap.add_argument("--routing-only", action="store_true",
                    help="only the routing/align latency microbenchmark (16384 tokens, E in 8/64/128)")
    ap.add_argument("--w4a16-only", action="store_true",
                    help="only the W4A16 split-K GEMM microbenchmark (k = n = 4096, group 128, m in 1/16/64/256)")
    ap.add_argument("--profile", action="store_true",
                    help="only warm-up + timed layer steps (for ncu captures): no e2e, sweep, roofline or CPU legs")
    args = ap.parse_args()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # peer memory is only read by plain loads and the collectives are tiny: no NVLink multicast objects, in
        # NCCL or in symmetric memory, that a rank ending early could leave bound
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        run_ours(args, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
