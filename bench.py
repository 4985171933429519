#!/usr/bin/env python3
"""Benchmark of the NVFP4 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--batch B]

Headline line (one JSON object on stdout, printed by rank 0): NVFP4 MoE-layer tokens/s on the
sparse 2:4 MoE GEMV decode configuration -- 512 experts, hidden 2048, moe_intermediate 512, top-10
routing from softmax of N(0,1) logits, B tokens per GPU (default 32).  A step is one MoE layer over
one batch.  With N > 1 the layer is expert-parallel (512/N experts per GPU, all-to-all dispatch and
combine over NCCL) and every GPU brings its own batch (weak scaling).

  value      device-timed whole-job tokens/s, inputs resident in HBM
  e2e        the same through the public op with host buffers (H2D of activations/routing and D2H
             of the result inside the timed region)
  roofline   sparse GEMV kernel (both projections of the layer): algorithmic weight+activation bytes /
             CUDA-event duration of the two launches, against the measured HBM copy bandwidth;
             per-projection times alongside
  cpu_baseline  the reference's dequantize-to-bf16 emulation (oracle port, torch on the host cores)

`--impl reference` times that CPU emulation as the main measurement instead.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(1, os.path.join(ROOT, "tests"))     # synthetic-data generators shared with the tests

E_TOTAL, HIDDEN, INTER, TOPK = 512, 2048, 512, 10
BYTES_PER_EXPERT_GATE_UP = 2 * INTER * HIDDEN * 7 // 16          # comp 1/4 + meta 1/8 + scale 1/16 B per weight
BYTES_PER_EXPERT_DOWN = HIDDEN * INTER * 7 // 16
N_ROUTINGS = 8
# dram__bytes_read.sum + dram__bytes_write.sum of the gate_up and down GEMV launches of one layer, per routed expert,
# from the ncu capture whose summary is committed with the profiles (244 routed experts: 233.61 MB + 118.83 MB)
NCU_TRAFFIC_BYTES_PER_EXPERT = (323.90e6 + 4.31e6) / 244.0
NCU_TRAFFIC_SOURCE = "ncu capture of the one-launch GEMV kernel (batch 32, 244 routed experts), scaled by routed experts"


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi; only samples whose timestamp falls
    inside the window marked by begin()/end() (the timed regions) are reported."""
    Q = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.proc = None
        self.idx = gpu_index
        self.t0 = self.t1 = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "20", "-i", str(self.idx)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def begin(self):
        self.t0 = time.time()

    def end(self):
        self.t1 = time.time()

    def stop(self):
        import datetime
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons, power = [], [], set(), []
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                if self.t0 is not None and not (self.t0 - 0.02 <= ts <= (self.t1 or ts) + 0.02):
                    continue
                sm.append(float(f[1]))
                mx.append(float(f[2]))
                power.append(float(f[3]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "power_w_max": max(power) if power else None}


def build_case(dev, e_local: int, batch: int, rank: int):
    import torch
    import synth
    from dgx_vllm_b200 import scaled_fp4_quant

    def qfn(w, gs):
        c, s = scaled_fp4_quant(w, gs, is_sf_swizzled_layout=False)
        return c, s.view(torch.uint8)

    w13 = synth.make_sparse_experts(e_local, 2 * INTER, HIDDEN, 1000 + rank, dev, qfn)
    w2 = synth.make_sparse_experts(e_local, HIDDEN, INTER, 2000 + rank, dev, qfn)
    batches = []
    for i in range(N_ROUTINGS):
        tw, ids = synth.make_routing(batch, E_TOTAL, TOPK, 10 * rank + i, dev)
        hidden = synth.make_hidden(batch, HIDDEN, 100 + 10 * rank + i, dev)
        batches.append((hidden, tw, ids))
    return w13, w2, batches


def cpu_baseline(batch: int, max_seconds: float = 25.0, steps: int = 5, warmup: int = 1):
    """Times the reference's dequantize-to-bf16 emulation of the same MoE layer on the host cores (all of them: the
    thread count is set explicitly, a launcher's OMP_NUM_THREADS=1 would otherwise leave one).  A step is one batch:
    every routed expert (about 240 of 512 at batch 32) is dequantized and multiplied on its own; the weight values come
    from a 64-expert table kept on the host (expert id modulo 64), which changes no arithmetic cost.  If `steps` full
    batches would take longer than max_seconds, a step processes the first rows of the batch only and says so."""
    import torch
    import synth
    from oracle import emulation
    import oracle
    import numpy as np

    torch.set_num_threads(os.cpu_count() or 1)

    def qfn(w, gs):
        bits = w.contiguous().view(torch.int16).numpy().view(np.uint16)
        c, s = oracle.quantize_bf16(bits, float(gs[0]))
        return torch.from_numpy(c), torch.from_numpy(s)

    e_cpu = 64                                     # experts materialised on the host
    w13 = synth.make_sparse_experts(e_cpu, 2 * INTER, HIDDEN, 1, "cpu", qfn)
    w2 = synth.make_sparse_experts(e_cpu, HIDDEN, INTER, 2, "cpu", qfn)
    tw, ids = synth.make_routing(batch, E_TOTAL, TOPK, 3, "cpu")
    hidden = synth.make_hidden(batch, HIDDEN, 4, "cpu")
    t0 = time.perf_counter()
    emulation.moe_layer_emulation(hidden[:1], tw[:1], ids[:1], w13, w2, INTER, table_rows=e_cpu)        # warm-up, 10 experts
    per_expert = (time.perf_counter() - t0) / TOPK
    uniq_full = int(ids.unique().numel())
    rows = batch
    while rows > 1 and per_expert * int(ids[:rows].unique().numel()) * (steps + warmup) > max_seconds:
        rows = max(1, rows // 2)
    for _ in range(warmup):
        emulation.moe_layer_emulation(hidden[:rows], tw[:rows], ids[:rows], w13, w2, INTER, table_rows=e_cpu)
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        emulation.moe_layer_emulation(hidden[:rows], tw[:rows], ids[:rows], w13, w2, INTER, table_rows=e_cpu)
        times.append(time.perf_counter() - t0)
    t = statistics.mean(times)
    uniq = int(ids[:rows].unique().numel())
    return {"value": rows / t, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": (f"{steps} steps of {rows} of the batch's {batch} tokens, {uniq} routed experts per step "
                       f"({uniq_full} for the whole batch), each dequantized and multiplied per step; weight values from a "
                       f"{e_cpu}-expert host table (id modulo {e_cpu}); mean step {t * 1e3:.1f} ms")}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    cb = cpu_baseline(args.batch, max_seconds=150.0, steps=args.steps, warmup=args.warmup)
    ms = args.batch / cb["value"] * 1e3
    line = {"impl": "reference", "metric": "NVFP4 MoE-layer tokens/s", "value": cb["value"], "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": config_dict(args),
            "cpu_baseline": cb, "e2e": {"value": cb["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0,
                                        "d2h_bytes_per_step": 0},
            "gpu_launches": 0, "host_threads": torch.get_num_threads()}
    print(json.dumps(line), flush=True)


class L2Flush:
    """Cold-L2 state before a timed launch: a 256 MiB buffer is written (twice the 126 MB L2), then a second 256 MiB
    buffer is read.  The write replaces every line the previous launch left in L2; the read pass then pushes the dirty
    lines of the written buffer out to HBM, so that their write-back does not run during -- and is not charged to -- the
    timed kernel.  What stays in L2 is clean data of a buffer no kernel uses."""

    def __init__(self, dev):
        import torch
        self.wr = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        self.rd = torch.zeros(64 << 20, dtype=torch.int32, device=dev)
        self.sink = None

    def __call__(self):
        self.wr.zero_()
        self.sink = self.rd.sum()


def _vllm_fp4_mm_us(timed, xc, wc, xs, ws, alpha, out, steps):
    """Time vLLM's cutlass_scaled_fp4_mm on the same operands (same cold-L2 protocol); a string says why not."""
    import torch
    try:
        from vllm import _custom_ops as vops
        f8 = torch.float8_e4m3fn
        xs8, ws8 = xs.view(f8), ws.view(f8)
        ref = vops.cutlass_scaled_fp4_mm(xc, wc, xs8, ws8, alpha, torch.bfloat16)
        torch.cuda.synchronize()
        if tuple(ref.shape) != tuple(out.shape):
            return "unavailable: unexpected result shape"
        diff = float((ref.float() - out.float()).abs().max() / out.float().abs().max().clamp_min(1e-30))
        if not diff < 2e-2:
            return f"unavailable: result differs from this library's by {diff:.3g}"
        return timed(lambda: vops.cutlass_scaled_fp4_mm(xc, wc, xs8, ws8, alpha, torch.bfloat16), steps) * 1e6
    except Exception as e:          # not built for this GPU, symbol missing, import failure
        return f"unavailable: {type(e).__name__}: {str(e)[:120]}"


def bench_dense_parts(dev, flush, hbm_peak, steps: int = 10, library: bool = True):
    """Secondary measurements reported next to the headline: dense NVFP4 GEMM (BASELINE configs[1]:
    N=14336, K=4096, M in {128,1024,4096}, activation quantized on the fly) and the quantizer alone.
    Each iteration is timed on its own with CUDA events after rewriting a 256 MiB buffer (cold L2)."""
    import torch
    import synth
    from dgx_vllm_b200 import cutlass_scaled_fp4_mm, scaled_fp4_quant
    from dgx_vllm_b200.ops import nvfp4_linear

    def timed(fn, n):
        ts = []
        for _ in range(3):
            fn()
        for _ in range(n):
            flush()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) * 1e-3)
        return statistics.mean(ts)

    N, K = 14336, 4096
    gen = torch.Generator(device=dev).manual_seed(7)
    w = (0.02 * torch.randn(N, K, generator=gen, device=dev)).to(torch.bfloat16)
    gw = synth.global_scale_of(w)
    wc, ws = scaled_fp4_quant(w, gw)
    del w
    parts = {}
    fp4_nominal = 9000.0      # TFLOP/s, dense NVFP4 nominal (4 x 2.25 PF bf16); no measured FP4 peak is provided
    for M in (128, 1024, 4096):
        x = torch.randn(M, K, generator=gen, device=dev).to(torch.bfloat16)
        gx = synth.global_scale_of(x)
        alpha = (1.0 / (gx * gw)).to(torch.float32)
        out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        xc, xs = scaled_fp4_quant(x, gx)
        t_mm = timed(lambda: cutlass_scaled_fp4_mm(xc, wc, xs, ws, alpha, torch.bfloat16, out=out), steps)

        def both():      # what a quantized linear layer does per forward: one library call for quantizer + GEMM
            nvfp4_linear(x, gx, wc, ws, alpha, out=out)
        t_all = timed(both, steps)
        flops = 2.0 * M * N * K
        byt = N * K * 0.5625 + M * K * 0.5625 + 2.0 * M * N
        parts[f"dense_gemm_m{M}"] = {
            "gemm_us": t_mm * 1e6, "quant_plus_gemm_us": t_all * 1e6, "tflops": flops / t_mm / 1e12,
            "frac_of_nominal_fp4_peak": flops / t_mm / 1e12 / fp4_nominal,
            "hbm_GBps": byt / t_mm / 1e9, "frac_of_measured_hbm": byt / t_mm / 1e9 / hbm_peak,
            "bound": "hbm" if M < 316 else "tensor"}
        # the serving stack's own library kernel for the same op on the same tensors, when this image's vLLM build has it
        # (comparison only: nothing in this package calls it)
        if library:
            parts[f"dense_gemm_m{M}"]["vllm_cutlass_scaled_fp4_mm_us"] = _vllm_fp4_mm_us(timed, xc, wc, xs, ws, alpha, out, steps)
        if M == 4096:
            # the same GEMM back to back for about half a second, with the clocks sampled: what the part sustains
            # under its power limit, and at which SM clock
            n_loop = 4000
            sampler = ClockSampler(dev.index or 0)
            sampler.start()
            for _ in range(20):
                cutlass_scaled_fp4_mm(xc, wc, xs, ws, alpha, torch.bfloat16, out=out)
            torch.cuda.synchronize()
            time.sleep(0.05)
            sampler.begin()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(n_loop):
                cutlass_scaled_fp4_mm(xc, wc, xs, ws, alpha, torch.bfloat16, out=out)
            b.record()
            torch.cuda.synchronize()
            sampler.end()
            t_loop = a.elapsed_time(b) * 1e-3 / n_loop
            parts[f"dense_gemm_m{M}"]["back_to_back"] = {"gemm_us": t_loop * 1e6, "tflops": flops / t_loop / 1e12,
                                                         "launches": n_loop, "clocks": sampler.stop()}
    for M in (4096, 16384):
        x = torch.randn(M, K, generator=gen, device=dev).to(torch.bfloat16)
        gx = synth.global_scale_of(x)
        t_q = timed(lambda: scaled_fp4_quant(x, gx), steps)
        byt = M * K * 2.5625
        parts[f"quantizer_{M}x{K}"] = {"us": t_q * 1e6, "GBps": byt / t_q / 1e9, "frac_of_measured_hbm": byt / t_q / 1e9 / hbm_peak}
    return parts


def bench_dense_nshard(dev, flush, world: int, rank: int, steps: int = 10):
    """BASELINE configs[1] on G GPUs: the N=14336 weight split by output columns, activation replicated
    and quantized on every rank, no exchange for the matmul; the optional all-gather of the column
    blocks is timed separately.  Device time per call (CUDA events around 4 calls issued back to back
    after an L2 flush), max over ranks."""
    import torch
    import torch.distributed as dist
    import synth
    from dgx_vllm_b200.dense_shard import ColumnShardedNvfp4Linear, shard_rows

    N, K = 14336, 4096
    b, e = shard_rows(N, world, rank)
    gen = torch.Generator(device=dev).manual_seed(7)
    w = (0.02 * torch.randn(N, K, generator=gen, device=dev)).to(torch.bfloat16)    # same on every rank
    gw = synth.global_scale_of(w)
    layer = ColumnShardedNvfp4Linear(N, gw, weight_bf16=w[b:e].contiguous())
    del w
    out = {}
    reps = 4
    for M in (128, 1024, 4096):
        x = torch.randn(M, K, generator=gen, device=dev).to(torch.bfloat16)
        gx = synth.global_scale_of(x)
        res = {}
        for gather in (False, True):
            ts = []
            for it in range(3 + steps):
                flush()
                dist.barrier()
                a, c = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                for _ in range(reps):       # back to back, so that host launch latency is not what is timed
                    layer.forward(x, gx, gather=gather)
                c.record()
                torch.cuda.synchronize()
                if it >= 3:
                    ts.append(a.elapsed_time(c) * 1e-3 / reps)
            t = torch.tensor([statistics.mean(ts)], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            res["quant_gemm_allgather_us" if gather else "quant_gemm_us"] = float(t.item()) * 1e6
        res["tflops_all_gpus"] = 2.0 * M * N * K / (res["quant_gemm_us"] * 1e-6) / 1e12
        res["frac_of_nominal_fp4_peak"] = res["tflops_all_gpus"] / (9000.0 * world)
        out[f"dense_gemm_m{M}_nshard{world}"] = res
    return out


def _dense_experts(dev, gen, E, N, K):
    """E dense NVFP4 expert matrices [N,K]: (codes [E,N,K/2], swizzled scales, global scales [E])."""
    import torch
    import synth
    from dgx_vllm_b200 import scaled_fp4_quant
    codes = torch.empty(E, N, K // 2, dtype=torch.uint8, device=dev)
    sf = torch.empty(E, (N + 127) // 128 * 128, (K // 16 + 3) // 4 * 4, dtype=torch.uint8, device=dev)
    gs = torch.empty(E, dtype=torch.float32, device=dev)
    for e0 in range(0, E, 64):
        n = min(64, E - e0)
        w = (0.02 * torch.randn(n, N, K, generator=gen, device=dev)).to(torch.bfloat16)
        for i in range(n):
            g = synth.global_scale_of(w[i])
            c, s_ = scaled_fp4_quant(w[i], g)
            codes[e0 + i], sf[e0 + i], gs[e0 + i] = c, s_.view(torch.uint8), g[0]
    return codes, sf, gs


def bench_moe_prefill_ep(dev, flush, world: int, rank: int, steps: int = 5):
    """BASELINE configs[3] expert-parallel: 8192 tokens in blocks of 8192/G per rank, 512/G experts per
    rank; all-gather of the token blocks, grouped NVFP4 path over the local experts, reduce-scatter of
    the fp32 partial rows.  Device time per layer, max over ranks."""
    import torch
    import torch.distributed as dist
    import synth
    from dgx_vllm_b200.moe_ep import ExpertParallelMoEPrefill

    T, E, H, I, topk = 8192, 512, 2048, 512, 10
    El, Tl = E // world, T // world
    gen = torch.Generator(device=dev).manual_seed(11 + rank)
    w13c, w13s, w13g = _dense_experts(dev, gen, El, 2 * I, H)
    w2c, w2s, w2g = _dense_experts(dev, gen, El, H, I)
    hidden = synth.make_hidden(Tl, H, 5 + rank, dev)
    tw, ids = synth.make_routing(Tl, E, topk, 6 + rank, dev, zipf=1.1)
    a1 = torch.full((El,), 448.0 * 6.0 / 6.0, dtype=torch.float32, device=dev)      # |N(0,1)| < 6 for these inputs
    a2 = torch.full((El,), 448.0 * 6.0 / 2.0, dtype=torch.float32, device=dev)
    layer = ExpertParallelMoEPrefill(E, (w13c, w13s, w13g, w2c, w2s, w2g, a1, a2))
    ts = []
    for it in range(3 + steps):
        flush()
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        layer.forward(hidden, tw, ids)
        b.record()
        torch.cuda.synchronize()
        if it >= 3:
            ts.append(a.elapsed_time(b) * 1e-3)
    t = torch.tensor([statistics.mean(ts)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    t = float(t.item())
    return {"tokens_per_s": T / t, "ms": t * 1e3, "tflops_all_gpus": 2.0 * T * topk * (2 * I * H + H * I) / t / 1e12,
            "config": f"8192 tokens ({Tl} per rank), 512 experts ({El} per rank), Zipf(1.1) top-10, all-gather + grouped path + reduce-scatter"}


def bench_moe_prefill(dev, flush, hbm_peak, steps: int = 5):
    """BASELINE configs[3]: 8192 tokens x hidden 2048, 512 experts, Zipf(1.1)-skewed top-10 routing,
    dense NVFP4 experts (gate_up 1024x2048, down 2048x512) through the grouped path: routing metadata ->
    token-major per-expert quantize -> grouped GEMM with SiLU*up + quantize in its epilogue -> grouped GEMM ->
    un-permute + weighted sum."""
    import torch
    from dgx_vllm_b200 import grouped_moe as gm
    import synth
    from dgx_vllm_b200 import scaled_fp4_quant
    from dgx_vllm_b200.ops import last_gemm_status

    T, E, H, I, topk = 8192, 512, 2048, 512, 10
    gen = torch.Generator(device=dev).manual_seed(11)

    w13c, w13s, w13g = _dense_experts(dev, gen, E, 2 * I, H)
    w2c, w2s, w2g = _dense_experts(dev, gen, E, H, I)
    hidden = synth.make_hidden(T, H, 5, dev)
    tw, ids = synth.make_routing(T, E, topk, 6, dev, zipf=1.1)
    a1 = (448.0 * 6.0 / hidden.float().abs().max()).repeat(E).float()
    a2 = torch.full((E,), 448.0 * 6.0 / 2.0, dtype=torch.float32, device=dev)
    alphas = gm.nvfp4_moe_alphas(w13g, w2g, a1, a2)     # layer constants

    def run():
        return gm.nvfp4_moe_prefill(hidden, tw, ids, w13c, w13s, w13g, w2c, w2s, w2g, a1, a2, alphas=alphas)

    for _ in range(3):
        run()
    status = last_gemm_status(dev)
    ts = []
    for _ in range(steps):
        flush()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        run()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b) * 1e-3)
    t = statistics.mean(ts)
    flops = 2.0 * T * topk * (2 * I * H + H * I)
    wbytes = E * (2 * I * H + H * I) * 0.5625
    return {"tokens_per_s": T / t, "ms": t * 1e3, "tflops": flops / t / 1e12, "weight_GBps": wbytes / t / 1e9,
            "frac_of_measured_hbm_weights_only": wbytes / t / 1e9 / hbm_peak, "gemm_status": status,
            "config": "8192 tokens, 512 experts, Zipf(1.1) top-10, dense NVFP4 experts, grouped path, 10 kernel launches"}


def bench_decode_stack(dev, batches=(1, 32, 128), layers: int = 48, distinct_layers: int = 4, reps: int = 5):
    """BASELINE configs[4]: Qwen3-Next-80B-A3B-shaped NVFP4 linear stack for decode -- 48 layers of
    (512 routed 2:4-sparse experts, top-10) + 1 shared dense NVFP4 expert, mixers stubbed by a fixed
    bf16 input per layer.  Captured once per batch size in a CUDA graph and replayed.
    Weights: `distinct_layers` independent layer sets cycled over the 48 layers (each set is 704 MB of
    routed weights, far beyond L2, and every layer uses its own routing)."""
    import torch
    import synth
    from dgx_vllm_b200 import cutlass_scaled_fp4_mm, scaled_fp4_quant
    from dgx_vllm_b200 import grouped_moe as gm
    from dgx_vllm_b200 import sparse_fp4_v7 as sp7

    E, H, I, topk = E_TOTAL, HIDDEN, INTER, TOPK
    keys = ("comp_T", "meta_T", "scale_T", "g_scales")

    def qfn(w, gs):
        c, s_ = scaled_fp4_quant(w, gs, is_sf_swizzled_layout=False)
        return c, s_.view(torch.uint8)

    sets = []
    gen = torch.Generator(device=dev).manual_seed(99)
    for li in range(distinct_layers):
        w13 = synth.make_sparse_experts(E, 2 * I, H, 3000 + li, dev, qfn)
        w2 = synth.make_sparse_experts(E, H, I, 4000 + li, dev, qfn)
        sh = []
        for (N, K) in ((2 * I, H), (H, I)):
            w = (0.02 * torch.randn(N, K, generator=gen, device=dev)).to(torch.bfloat16)
            g = synth.global_scale_of(w)
            c, s_ = scaled_fp4_quant(w, g)
            lin = scaled_fp4_quant(w, g, is_sf_swizzled_layout=False)[1] if li == (layers - 1) % distinct_layers else None
            sh.append((c, s_, g, lin))        # linear scales of the last layer's set, for the check below
        sets.append((w13, w2, sh))
    emap = torch.empty(0, dtype=torch.int32, device=dev)
    eo1 = lambda B: (torch.tensor([0, B], dtype=torch.int32, device=dev), torch.tensor([0, (B + 127) // 128 * 128], dtype=torch.int32, device=dev))
    out = {}
    for B in batches:
        xs = [synth.make_hidden(B, H, 500 + l, dev) for l in range(layers)]
        routes = [synth.make_routing(B, E, topk, 700 + l, dev) for l in range(layers)]
        gx = torch.tensor([448.0 * 6.0 / 6.0], dtype=torch.float32, device=dev)
        ga = torch.tensor([448.0 * 6.0 / 4.0], dtype=torch.float32, device=dev)
        offs, bso = eo1(B)
        alphas = [((1.0 / (gx * sh[0][2])).float(), (1.0 / (ga * sh[1][2])).float()) for (_, _, sh) in sets]

        def stack():
            acc = y = z = None
            for l in range(layers):
                w13, w2, sh = sets[l % distinct_layers]
                x = xs[l]
                tw, ids = routes[l]
                y = sp7.fused_sparse_moe_v7(x, tw, ids, emap, *[w13[k] for k in keys], *[w2[k] for k in keys], I, False)
                # shared expert: quant -> GEMM -> SiLU*up + quant -> GEMM
                (c13, s13, g13, _), (c2, s2, g2, _) = sh
                xc, xsf = scaled_fp4_quant(x, gx)
                al13, al2 = alphas[l % distinct_layers]
                gu = cutlass_scaled_fp4_mm(xc, c13, xsf, s13, al13, torch.bfloat16)
                hc, hsf = gm.silu_and_mul_scaled_fp4_experts_quant(gu, ga, offs, bso)
                z = cutlass_scaled_fp4_mm(hc, c2, hsf, s2, al2, torch.bfloat16)
                acc = y + z if acc is None else acc + y + z
            return acc, y, z

        for _ in range(2):
            stack()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            res, y_last, z_last = stack()
        graph.replay()
        torch.cuda.synchronize()
        verified = _verify_stack_last_layer(sets[(layers - 1) % distinct_layers], xs[-1], routes[-1], y_last, z_last, gx, ga, I)
        ts = []
        for _ in range(reps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            graph.replay()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) * 1e-3)
        t = statistics.mean(ts)
        uniq = statistics.mean(int(r[1].unique().numel()) for r in routes)
        byt = layers * (uniq * (BYTES_PER_EXPERT_GATE_UP + BYTES_PER_EXPERT_DOWN) + (2 * I * H + H * I) * 0.5625)
        out[f"batch_{B}"] = {"tokens_per_s": B / t, "ms_per_token_step": t * 1e3, "us_per_layer": t / layers * 1e6,
                             "weight_GBps": byt / t / 1e9, "finite": bool(torch.isfinite(res.float()).all().item()),
                             "verified_last_layer": verified}
        del graph
    out["config"] = (f"{layers} layers, {distinct_layers} distinct weight sets cycled, routed 2:4 sparse experts + shared dense "
                     f"NVFP4 expert per layer, one CUDA graph per batch size")
    return out


def bench_decode_stack_ep(dev, world: int, rank: int, ep_mode: str, batches=(1, 32, 128), layers: int = 48,
                          distinct_layers: int = 4, reps: int = 5):
    """BASELINE configs[4] on G GPUs: the 48-layer stack with the routed experts expert-parallel (512/G per GPU, the same
    exchange as the headline layer) and the shared dense NVFP4 expert replicated; every GPU brings its own batch.  Eager
    launches (the peer-memory exchange numbers its steps on the host).  Device time per token step, max over ranks; the last
    layer's routed output on rank 0's first tokens is checked against the CPU oracle (each rank evaluates its own experts,
    one all-reduce adds the partial rows)."""
    import torch
    import torch.distributed as dist
    import synth
    from dgx_vllm_b200 import cutlass_scaled_fp4_mm, scaled_fp4_quant
    from dgx_vllm_b200 import grouped_moe as gm
    from dgx_vllm_b200.moe_ep import ExpertParallelMoE

    E, H, I, topk = E_TOTAL, HIDDEN, INTER, TOPK
    El = E // world

    def qfn(w, gs):
        c, s_ = scaled_fp4_quant(w, gs, is_sf_swizzled_layout=False)
        return c, s_.view(torch.uint8)

    sets = []
    gen = torch.Generator(device=dev).manual_seed(99)           # shared expert: the same on every rank
    for li in range(distinct_layers):
        w13 = synth.make_sparse_experts(El, 2 * I, H, 3000 + 10 * li + rank, dev, qfn)
        w2 = synth.make_sparse_experts(El, H, I, 4000 + 10 * li + rank, dev, qfn)
        sh = []
        for (N, K) in ((2 * I, H), (H, I)):
            w = (0.02 * torch.randn(N, K, generator=gen, device=dev)).to(torch.bfloat16)
            g = synth.global_scale_of(w)
            c, s_ = scaled_fp4_quant(w, g)
            sh.append((c, s_, g))
        sets.append((ExpertParallelMoE(E, I, w13, w2, mode=ep_mode), w13, w2, sh))
    out = {}
    for B in batches:
        xs = [synth.make_hidden(B, H, 500 + l + 100 * rank, dev) for l in range(layers)]
        routes = [synth.make_routing(B, E, topk, 700 + l + 100 * rank, dev) for l in range(layers)]
        gx = torch.tensor([448.0 * 6.0 / 6.0], dtype=torch.float32, device=dev)
        ga = torch.tensor([448.0 * 6.0 / 4.0], dtype=torch.float32, device=dev)
        offs = torch.tensor([0, B], dtype=torch.int32, device=dev)
        bso = torch.tensor([0, (B + 127) // 128 * 128], dtype=torch.int32, device=dev)
        alphas = [((1.0 / (gx * sh[0][2])).float(), (1.0 / (ga * sh[1][2])).float()) for (_, _, _, sh) in sets]

        def stack():
            acc = y = None
            for l in range(layers):
                layer, _, _, sh = sets[l % distinct_layers]
                x = xs[l]
                tw, ids = routes[l]
                y = layer.forward(x, tw, ids)
                (c13, s13, _), (c2, s2, _) = sh
                xc, xsf = scaled_fp4_quant(x, gx)
                al13, al2 = alphas[l % distinct_layers]
                gu = cutlass_scaled_fp4_mm(xc, c13, xsf, s13, al13, torch.bfloat16)
                hc, hsf = gm.silu_and_mul_scaled_fp4_experts_quant(gu, ga, offs, bso)
                z = cutlass_scaled_fp4_mm(hc, c2, hsf, s2, al2, torch.bfloat16)
                acc = y + z if acc is None else acc + y + z
            return acc, y

        for _ in range(2):
            stack()
        ts = []
        for _ in range(reps):
            dist.barrier()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            res, y_last = stack()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) * 1e-3)
        t = torch.tensor([statistics.mean(ts)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        t = float(t.item())
        layer, w13, w2, _ = sets[(layers - 1) % distinct_layers]
        ver = verify_layer_step(layer, (xs[-1], routes[-1][0], routes[-1][1]), w13, w2, world, rank, dev, n_tok=min(2, B))
        out[f"batch_{B}_per_gpu"] = {"tokens_per_s": B * world / t, "ms_per_token_step": t * 1e3, "us_per_layer": t / layers * 1e6,
                                     "finite": bool(torch.isfinite(res.float()).all().item()), "verified_last_layer": ver}
    out["config"] = (f"{layers} layers, {distinct_layers} distinct weight sets cycled, routed 2:4 sparse experts expert-parallel over "
                     f"{world} GPUs ({El} per GPU, exchange: {ep_mode}) + replicated shared dense NVFP4 expert; eager launches")
    return out


def _rel(got, ref):
    import numpy as np
    return float(np.max(np.abs(np.asarray(got, np.float64) - np.asarray(ref, np.float64))) / (np.max(np.abs(ref)) + 1e-30))


def _verify_stack_last_layer(wset, x, route, y, z, gx, ga, I, n_tok: int = 2):
    """The decode stack's last layer on its first tokens, as replayed from the CUDA graph, against the CPU oracle:
    routed-expert output (<= 1e-2) and shared-expert output (quantize -> GEMM -> SiLU*up + quantize -> GEMM; both GEMM
    inputs are re-quantized, where single E2M1 codes may flip on a 16-bit rounding, hence the looser figure)."""
    import numpy as np
    import oracle
    from util import bf16_bits, expert_fetch
    w13, w2, sh = wset
    tw, ids = route
    n = min(n_tok, x.shape[0])
    ref_y = oracle.fused_sparse_moe_by_expert(x[:n].float().cpu().numpy(), tw[:n].cpu().numpy(), ids[:n].cpu().numpy(),
                                              expert_fetch(w13, w2), I)
    (c13, _, g13, l13), (c2, _, g2, l2) = sh
    bf = lambda v: oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits(v))
    u8 = lambda t: t.view(__import__("torch").uint8).cpu().numpy()
    gu = bf(oracle.nvfp4_linear(bf16_bits(x[:n]), float(gx[0]), c13.cpu().numpy(), u8(l13), float(g13[0])))
    act = bf((gu[:, :I] / (1.0 + np.exp(-gu[:, :I].astype(np.float64))) * gu[:, I:]).astype(np.float32))
    ref_z = oracle.nvfp4_linear(oracle.f32_to_bf16_bits(act), float(ga[0]), c2.cpu().numpy(), u8(l2), float(g2[0]))
    return {"tokens": n, "routed_rel_err": _rel(y[:n].float().cpu().numpy(), ref_y),
            "shared_rel_err": _rel(z[:n].float().cpu().numpy(), ref_z)}


def verify_layer_step(layer, batch0, w13, w2, world, rank, dev, n_tok: int = 4):
    """One step of the benchmarked layer on rank 0's first tokens against the CPU oracle, outside every timed region.
    With several ranks every rank evaluates the oracle over its own experts for those tokens and one all-reduce
    adds the partial rows."""
    import numpy as np
    import torch
    import torch.distributed as dist
    import oracle
    from util import expert_fetch
    h, tw, ids = batch0
    out = layer.forward(h, tw, ids)
    torch.cuda.synchronize()
    sample = [h[:n_tok].clone(), tw[:n_tok].clone(), ids[:n_tok].clone()]
    if world > 1:
        for t in sample:
            dist.broadcast(t, src=0)
    hs, ws_, is_ = [t.cpu() for t in sample]
    emap = layer.expert_map(dev).cpu().numpy()
    part = oracle.fused_sparse_moe_by_expert(hs.float().numpy(), ws_.numpy(), emap[is_.numpy()], expert_fetch(w13, w2), INTER)
    ref = torch.from_numpy(part).to(dev)
    if world > 1:
        dist.all_reduce(ref)
    if rank != 0:
        return None
    return {"tokens": n_tok, "rel_err": _rel(out[:n_tok].float().cpu().numpy(), ref.cpu().numpy()),
            "against": "CPU oracle (fp32 dequantize-then-matmul per routed expert), max|diff|/max|ref|"}


def bench_ep_local_call(dev, flush, hbm_peak, ranks: int = 8, batch: int = 32, steps: int = 20):
    """What ONE rank of an expert-parallel group of `ranks` GPUs runs per step, on this GPU alone: the fused layer over
    the ranks*batch tokens of all ranks with only E_TOTAL/ranks experts resident (`expert_map` masks the others).  No
    exchange: this isolates the local layer, whose GEMV launch has few items per SM and takes the 8-warp x 8-stage
    shape of the warp-scheduled kernel.  Cold L2, CUDA events from the library's benchmark hook."""
    import torch
    import synth
    from dgx_vllm_b200 import _lib, scaled_fp4_quant, sparse_fp4_v7 as sp7
    from dgx_vllm_b200.moe_ep import expert_map_for_rank

    def qfn(w, gs):
        c, s_ = scaled_fp4_quant(w, gs, is_sf_swizzled_layout=False)
        return c, s_.view(torch.uint8)

    e_local = E_TOTAL // ranks
    w13 = synth.make_sparse_experts(e_local, 2 * INTER, HIDDEN, 4000, dev, qfn)
    w2 = synth.make_sparse_experts(e_local, HIDDEN, INTER, 5000, dev, qfn)
    k4 = ("comp_T", "meta_T", "scale_T", "g_scales")
    emap = expert_map_for_rank(E_TOTAL, ranks, 0, dev)
    layer = sp7.FusedSparseMoE(*[w13[x] for x in k4], *[w2[x] for x in k4], INTER, expert_map=emap)
    T = ranks * batch
    cases = []
    for i in range(N_ROUTINGS):
        tw, ids = synth.make_routing(T, E_TOTAL, TOPK, 700 + i, dev)
        cases.append((synth.make_hidden(T, HIDDEN, 800 + i, dev), tw, ids))
    L = _lib.lib()
    for i in range(3):
        layer(*cases[i % N_ROUTINGS])
    torch.cuda.synchronize()
    t_layer, t_gemv, byts = [], [], []
    for i in range(steps):
        h, tw, ids = cases[i % N_ROUTINGS]
        m = emap[ids.long()]
        uniq, pairs = int(m[m >= 0].unique().numel()), int((m >= 0).sum().item())
        flush()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        for e in ev:
            e.record()
        L.b200fp4_fused_moe_profile_events(ev[0].cuda_event, ev[1].cuda_event, ev[2].cuda_event)
        a.record()
        layer(h, tw, ids)
        b.record()
        L.b200fp4_fused_moe_profile_events(0, 0, 0)
        torch.cuda.synchronize()
        t_layer.append(a.elapsed_time(b) * 1e-3)
        t_gemv.append(ev[0].elapsed_time(ev[2]) * 1e-3)
        byts.append(uniq * (BYTES_PER_EXPERT_GATE_UP + BYTES_PER_EXPERT_DOWN) + pairs * (HIDDEN * 2 + INTER * 4 + HIDDEN * 4))
    gbps = sum(byts) / sum(t_gemv) / 1e9
    return {"layer_us": statistics.mean(t_layer) * 1e6, "gemv_launch_us": statistics.mean(t_gemv) * 1e6,
            "gemv_GBps": gbps, "frac_of_measured_hbm": gbps / hbm_peak,
            "config": f"{T} tokens ({ranks} ranks x {batch}), {e_local} local of {E_TOTAL} experts, top-{TOPK}, cold L2"}


def bench_reference_v7_gpu(dev, w13, w2, batches, flush, ours, steps: int = 20):
    """The reference's own CUDA extension (sparse_fp4_kernel/sparse_fp4_v7.cu compiled unmodified for sm_100 by
    oracle/build_ref_v7.py) on the same tensors, inside its contract (identity expert_map, N >= 512; its lazy table
    initialisation happens in the warm-up calls).  Cold: L2 flushed before every layer, CUDA events; loop: back to back."""
    import torch
    from oracle import build_ref_v7
    mod = build_ref_v7.load()
    if mod is None:
        return {"unavailable": "oracle/_ref/sparse_fp4_v7 not built (oracle/build_ref_v7.py needs a checkout of the reference)"}
    k = ("comp_T", "meta_T", "scale_T", "g_scales")
    emap = torch.empty(0, dtype=torch.int32, device=dev)
    wargs = [w13[x] for x in k] + [w2[x] for x in k]

    def run(i):
        h, tw, ids = batches[i % N_ROUTINGS]
        return mod.fused_sparse_moe_v7(h, tw, ids, emap, *wargs, INTER, False)

    for i in range(3):
        theirs = run(i)
    torch.cuda.synchronize()
    cold = []
    for i in range(steps):
        flush()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        run(i)
        b.record()
        torch.cuda.synchronize()
        cold.append(a.elapsed_time(b) * 1e-3)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(steps):
        run(i)
    b.record()
    torch.cuda.synchronize()
    loop = a.elapsed_time(b) * 1e-3 / steps
    B = batches[0][0].shape[0]
    theirs = run(0).float()
    mine = ours(*batches[0]).float()
    return {"us_per_layer_cold_l2": statistics.mean(cold) * 1e6, "us_per_layer_back_to_back": loop * 1e6,
            "tokens_per_s_back_to_back": B / loop, "rel_diff_to_this_library": _rel(mine.cpu().numpy(), theirs.cpu().numpy()),
            "kernel": "fused_sparse_moe_v7 of the reference (batched_sparse_v7_kernel x 2 + 5 glue kernels), built with -arch sm_100"}


def config_dict(args):
    return {"workload": "sparse 2:4 NVFP4 MoE GEMV decode layer (BASELINE configs[2])", "experts": E_TOTAL,
            "hidden": HIDDEN, "moe_intermediate": INTER, "topk": TOPK, "batch_per_gpu": args.batch,
            "parallelism": f"ep{args.gpus}" if args.gpus > 1 else "single",
            "l2": f"routed expert weights per step exceed the 126 MB L2 at batch>=16; routing rotates over "
                  f"{N_ROUTINGS} seeded batches; before every timed launch of the per-kernel (roofline) loop a "
                  f"256 MiB buffer is rewritten and a second 256 MiB buffer is read (cold L2, no dirty lines left "
                  f"to write back during the timed kernel)"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--ep-mode", default="p2p", choices=["gather", "a2a", "p2p"],
                    help="expert-parallel exchange: this library's own dispatch / combine kernels over peer memory (default), "
                         "NCCL all-gather + reduce-scatter, or NCCL all-to-all both ways")
    ap.add_argument("--no-parts", action="store_true", help="skip the dense GEMM / quantizer side measurements")
    ap.add_argument("--only-prefill", action="store_true",
                    help="run just the grouped prefill layer (the `moe_prefill_8192_tokens` part) and print its numbers; "
                         "a short command for profiling that path")
    ap.add_argument("--only-dense", action="store_true",
                    help="run just the dense GEMM / quantizer parts and print their numbers; a short command for "
                         "profiling those kernels (with --no-library-comparison the serving stack's kernel is not timed)")
    ap.add_argument("--no-library-comparison", action="store_true")
    ap.add_argument("--only-ep-local", action="store_true",
                    help="run just the `ep8_local_call` part (the layer one of eight expert-parallel ranks runs per step, "
                         "on this GPU alone); a short command for profiling that launch shape")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        return run_reference(args)
    if args.only_dense:
        import torch
        dev = torch.device("cuda", 0)
        torch.cuda.set_device(dev)
        hbm_peak, _ = measured_peaks()
        print(json.dumps(bench_dense_parts(dev, L2Flush(dev), hbm_peak, library=not args.no_library_comparison)))
        return 0
    if args.only_ep_local:
        import torch
        dev = torch.device("cuda", 0)
        torch.cuda.set_device(dev)
        hbm_peak, _ = measured_peaks()
        print(json.dumps({"ep8_local_call": bench_ep_local_call(dev, L2Flush(dev), hbm_peak)}))
        return 0
    if args.only_prefill:
        import torch
        dev = torch.device("cuda", 0)
        torch.cuda.set_device(dev)
        flush = L2Flush(dev)
        hbm_peak, _ = measured_peaks()
        print(json.dumps({"moe_prefill_8192_tokens": bench_moe_prefill(dev, flush, hbm_peak)}))
        return 0

    import torch
    import torch.distributed as dist
    from dgx_vllm_b200 import _lib, sparse_fp4_v7 as sp7
    from dgx_vllm_b200.moe_ep import ExpertParallelMoE

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback); use --impl reference for the CPU arm")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    L = _lib.lib()
    if L.b200fp4_has_hardware_acceleration() != 1:
        raise SystemExit("bench.py needs an sm_100 device")

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    e_local = E_TOTAL // world
    w13, w2, batches = build_case(dev, e_local, args.batch, rank)
    layer = ExpertParallelMoE(E_TOTAL, INTER, w13, w2, mode=args.ep_mode)
    B = args.batch
    hbm_peak, peak_kind = measured_peaks()
    flush = L2Flush(dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step(i):
        h, tw, ids = batches[i % N_ROUTINGS]
        return layer.forward(h, tw, ids)

    for i in range(args.warmup):
        step(i)
    barrier()
    ep_mode_used = args.ep_mode if world > 1 else None
    if world > 1 and args.ep_mode == "p2p":
        # the peer-memory exchange reports a bounded wait that ran out through a status word: if any rank saw one during
        # the warm-up, every rank switches to the NCCL exchange for the rest of the run and the line says so
        stt = torch.tensor([layer.p2p_status()], dtype=torch.int32, device=dev)
        dist.all_reduce(stt, op=dist.ReduceOp.MAX)
        if int(stt.item()) != 0:
            layer = ExpertParallelMoE(E_TOTAL, INTER, w13, w2, mode="gather")
            ep_mode_used = f"gather (the peer-memory exchange reported status {int(stt.item())} during warm-up)"
            for i in range(args.warmup):
                step(i)
            barrier()
    verified = verify_layer_step(layer, batches[0], w13, w2, world, rank, dev)
    barrier()

    # ---- value: K steps back to back, device-timed
    sampler.begin()
    n0 = L.b200fp4_launch_count()
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for i in range(args.steps):
        step(i)
    ev1.record()
    barrier()
    ms_total = ev0.elapsed_time(ev1)
    launches = int(L.b200fp4_launch_count() - n0)
    t = torch.tensor([ms_total], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / args.steps
    value = B * world / (ms_step * 1e-3)

    # ---- roofline: per-launch duration of the two GEMV kernels, cold L2 (flush between steps), measured on the
    # very call the step makes: with several ranks that is the local layer over the records of ALL ranks' tokens
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    pev = [[torch.cuda.Event(enable_timing=True) for _ in range(5)] for _ in range(args.steps)] if world > 1 else None
    uniq, local_pairs = [], []
    emap_all = layer.expert_map(dev)
    for r in range(N_ROUTINGS):
        ids = batches[r][2]
        if world > 1:
            all_ids = torch.empty((world * B, TOPK), dtype=torch.int32, device=dev)
            dist.all_gather_into_tensor(all_ids, ids.contiguous())
        else:
            all_ids = ids
        m = emap_all[all_ids.long()]
        uniq.append(int(m[m >= 0].unique().numel()))
        local_pairs.append(int((m >= 0).sum().item()))
    uniq = [uniq[i % N_ROUTINGS] for i in range(args.steps)]
    local_pairs = [local_pairs[i % N_ROUTINGS] for i in range(args.steps)]
    for i in range(args.steps):
        flush()
        if world > 1:
            dist.barrier()
        for e in evs[i]:
            e.record()      # creates the underlying CUDA events; the library re-records them
        L.b200fp4_fused_moe_profile_events(evs[i][0].cuda_event, evs[i][1].cuda_event, evs[i][2].cuda_event)
        if pev:
            layer.phase_events = pev[i]
        step(i)
        layer.phase_events = None
        L.b200fp4_fused_moe_profile_events(0, 0, 0)
    torch.cuda.synchronize()
    # events 0 -> 2 bracket the two projections of the layer's default path (two launches at this batch
    # size; one cooperative launch up to 256 pairs)
    t_both = [evs[i][0].elapsed_time(evs[i][2]) * 1e-3 for i in range(args.steps)]
    # per-projection times: the same layer with one launch per projection (a few steps, cold L2)
    k4 = ("comp_T", "meta_T", "scale_T", "g_scales")
    n_sep = min(args.steps, 16)
    evs2 = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(n_sep)]
    if world > 1:
        n_sep = 0          # the per-projection split is a one-GPU side measurement
    for i in range(n_sep):
        h, tw, ids = batches[i % N_ROUTINGS]
        flush()
        for e in evs2[i]:
            e.record()
        L.b200fp4_fused_moe_profile_events(evs2[i][0].cuda_event, evs2[i][1].cuda_event, evs2[i][2].cuda_event)
        sp7.fused_sparse_moe_v7(h, tw, ids, layer.expert_map(dev), *[w13[x] for x in k4], *[w2[x] for x in k4], INTER, False,
                                separate_launches=True)
        L.b200fp4_fused_moe_profile_events(0, 0, 0)
    torch.cuda.synchronize()
    t_gu = [evs2[i][0].elapsed_time(evs2[i][1]) * 1e-3 for i in range(n_sep)]
    t_dn = [evs2[i][1].elapsed_time(evs2[i][2]) * 1e-3 for i in range(n_sep)]
    # algorithmic bytes per launch: weights of the unique local experts + activations in/out per local pair
    b_gu = [u * BYTES_PER_EXPERT_GATE_UP + p * (HIDDEN * 2 + INTER * 2) for u, p in zip(uniq, local_pairs)]
    b_dn = [u * BYTES_PER_EXPERT_DOWN + p * (INTER * 2 + HIDDEN * 4) for u, p in zip(uniq, local_pairs)]
    ach = (sum(b_gu) + sum(b_dn)) / sum(t_both) / 1e9
    # DRAM traffic (dram__bytes_read + dram__bytes_write of the two projections) is not measurable inside this run; the
    # figure is the ratio of an ncu capture of the same two kernels on a smaller case of this workload (NCU_TRAFFIC below:
    # bytes per routed expert) scaled to this run's routed experts -- traffic grows in proportion to them.
    traffic = NCU_TRAFFIC_BYTES_PER_EXPERT * statistics.mean(uniq) if world == 1 else None
    roofline = {"bound": "hbm", "achieved": ach, "peak": hbm_peak, "unit": "GB/s", "frac": ach / hbm_peak,
                "traffic": traffic, "traffic_source": NCU_TRAFFIC_SOURCE if world == 1 else None,
                "peak_kind": f"{peak_kind} copy bandwidth",
                "kernel": "fused_moe_ws_kernel: gate_up+SiLU and down projections of one layer in one launch (tensor-core 2:4 GEMV)",
                "per_launch_us": {"both_projections": statistics.mean(t_both) * 1e6},
                "algorithmic_bytes_per_step": (sum(b_gu) + sum(b_dn)) / args.steps,
                "unique_experts_mean": statistics.mean(uniq), "local_pairs_mean": statistics.mean(local_pairs)}
    if n_sep:
        roofline["per_launch_us"].update({"gate_up_separate_launch": statistics.mean(t_gu) * 1e6,
                                          "down_separate_launch": statistics.mean(t_dn) * 1e6})
        roofline["gate_up_GBps_separate_launch"] = sum(b_gu[:n_sep]) / sum(t_gu) / 1e9
        roofline["down_GBps_separate_launch"] = sum(b_dn[:n_sep]) / sum(t_dn) / 1e9
    ep_phases = None
    if pev:
        # device time of the four phases of the expert-parallel step (cold L2, ranks released by a barrier), max over ranks
        ph = torch.tensor([[pev[i][j].elapsed_time(pev[i][j + 1]) * 1e3 for j in range(4)] for i in range(args.steps)],
                          dtype=torch.float64, device=dev).mean(0)
        dist.all_reduce(ph, op=dist.ReduceOp.MAX)
        ep_phases = dict(zip(("pack_us", "dispatch_us", "local_layer_us", "combine_us"), [float(x) for x in ph.tolist()]))
        ep_phases["mode"] = ep_mode_used

    # ---- e2e: host buffers in, host result out, through the public op
    host = []
    for h, tw, ids in batches:
        host.append((h.cpu().pin_memory(), tw.cpu().pin_memory(), ids.cpu().pin_memory()))
    E2E_RING = 4                  # steps in flight: each has its own pinned result buffer
    out_ring = [torch.empty(B, HIDDEN, dtype=torch.bfloat16).pin_memory() for _ in range(E2E_RING)]
    tickets = [None] * E2E_RING

    def e2e_step(i):
        # host buffers in, host result out, the way a serving loop keeps the GPU fed: the step is queued (H2D copies of
        # its inputs, the layer, the D2H copy of its result) and the host moves on; a result buffer is reused only after
        # the step that last wrote it has completed.  On one GPU this is one call of the library's queued host-buffer
        # entry point per step (inputs of step i+1 travel on a copy stream while step i computes).
        j = i % E2E_RING
        if tickets[j] is not None:
            tickets[j].synchronize()
        hh, hw, hi = host[i % N_ROUTINGS]
        tickets[j] = layer.submit_host(hh, hw, hi, out_ring[j], dev, slot=i % 2)

    def e2e_sync_step(i):
        # the same with a host wait after every step (latency of one isolated step)
        hh, hw, hi = host[i % N_ROUTINGS]
        layer.forward_host(hh, hw, hi, out_ring[0], dev)

    def timed(step_fn, drain):
        for i in range(args.warmup):
            step_fn(i)
        drain()
        barrier()
        t0 = time.perf_counter()
        for i in range(args.steps):
            step_fn(i)
        drain()
        barrier()
        dt = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        return B * world * args.steps / float(dt.item())

    e2e_val = timed(e2e_step, lambda: layer.wait_host(dev))
    e2e_sync_val = timed(e2e_sync_step, lambda: None)
    sampler.end()
    clocks = sampler.stop() if rank == 0 else None
    nshard_parts = None
    if world > 1 and not args.no_parts and (14336 // world) % 128 == 0:
        del w13, w2, layer
        torch.cuda.empty_cache()
        nshard_parts = bench_dense_nshard(dev, flush, world, rank)
        torch.cuda.empty_cache()
        nshard_parts[f"moe_prefill_8192_tokens_ep{world}"] = bench_moe_prefill_ep(dev, flush, world, rank)
        torch.cuda.empty_cache()
        nshard_parts[f"decode_stack_48_layers_ep{world}"] = bench_decode_stack_ep(dev, world, rank, "gather" if str(ep_mode_used).startswith("gather") else args.ep_mode)
    h2d = B * HIDDEN * 2 + B * TOPK * 8
    d2h = B * HIDDEN * 2

    if rank == 0:
        line = {"metric": "NVFP4 MoE-layer tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f16 products, f32 accumulate (NVFP4 weights, bf16 activations)",
                "data": "synthetic", "config": config_dict(args), "roofline": roofline,
                "e2e": {"value": e2e_val, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                        "steps_in_flight": E2E_RING, "value_with_host_wait_every_step": e2e_sync_val},
                "gpu_launches": launches, "clocks": clocks, "verified": verified}
        if ep_phases:
            line["ep_phases"] = ep_phases
        if ep_mode_used:
            line["config"]["ep_exchange"] = ep_mode_used
        ref_gpu = None
        if world == 1 and not args.no_parts:
            ref_gpu = bench_reference_v7_gpu(dev, w13, w2, batches, flush, layer.forward)
        if world == 1 and not args.no_parts:
            del w13, w2, layer
            torch.cuda.empty_cache()
            line["parts"] = bench_dense_parts(dev, flush, hbm_peak)
            line["parts"]["ep8_local_call"] = bench_ep_local_call(dev, flush, hbm_peak)
            line["parts"]["reference_v7_gpu"] = ref_gpu
            torch.cuda.empty_cache()
            line["parts"]["moe_prefill_8192_tokens"] = bench_moe_prefill(dev, flush, hbm_peak)
            torch.cuda.empty_cache()
            line["parts"]["decode_stack_48_layers"] = bench_decode_stack(dev)
        if nshard_parts is not None:
            line["parts"] = nshard_parts
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(B)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
