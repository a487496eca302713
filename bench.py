#!/usr/bin/env python
"""Benchmark of one denoising step of the 28 transformer blocks at 1024x1024.

A "step" is what the reference's sampler loop does per sigma of its 8-step Turbo schedule
(src/pipeline/mod.rs:343-366) for one image of 4096 image + 512 text tokens at the reference's
dimensions (d 6144, q|k|v|gate 15360, SwiGLU 16384), minus the bf16 models around the blocks:
`modulation` -> copy [text; image] into the session -> the session's graph of 28 blocks x eleven
launches (prepare_norm, gemm qkvg, QK-norm + RoPE, V transpose, fp16 attention, prepare_gated,
gemm wo + residual, prepare_norm, gemm gate|up + SwiGLU, prepare_plain, gemm down + residual)
-> copy the image rows back -> `euler`.  Weights are seeded synthetic int8 (12.2 GB, so every
step streams far more than L2 holds).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

`value` is the integer-op rate of the four GEMMs (2*M*N*K summed over the step) divided by the
device time of the WHOLE step, inputs resident in HBM.  `w8a8_chain` is the same 28 blocks with
the three launches that are not W8A8 products left out.  `e2e` is the full block chain through
krea2_session_run: host x and modulation tables in pinned memory, copied in and read back inside
the timed region.  With N > 1 every rank runs its own image on its own GPU (independent sessions,
replicated weights, no collective on the data path): weak scaling; after that timing, and outside
it, the ranks run ONE image together -- column-sharded weights (`tp`) and token-sharded rows (`sp`),
each checked bit for bit against the single-GPU session -- and one forward at 16896 tokens
(`config4`).

--impl reference times the CPU restatement of the reference's arithmetic (the oracle; the
reference's own kernels need an AMD GPU and a Rust toolchain) on the host cores, on a bounded
sample of the same step.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

DIMS = {  # hidden, kv_heads, head_dim, inter
    "reference": dict(hidden=6144, kv_heads=12, head_dim=128, inter=16384),  # src/session/mod.rs:35-45
}
NOMINAL_INT8_TOPS = 4500.0  # dense int8 tensor peak of a B200, vendor figure
TEXT_TOKENS = 512
TURBO_STEPS = 8
GEMM_LABELS = {"gemm qkvg": "qkvg", "gemm wo + residual": "wo", "gemm gate|up + swiglu": "gu", "gemm down + residual": "down"}


def gemm_shapes(dims, tokens):
    h, inter = dims["hidden"], dims["inter"]
    qkvg = 2 * h + 2 * dims["kv_heads"] * dims["head_dim"]
    return {"gemm qkvg": (tokens, qkvg, h), "gemm wo + residual": (tokens, h, h),
            "gemm gate|up + swiglu": (tokens, 2 * inter, h), "gemm down + residual": (tokens, h, inter)}


def gemm_algorithmic_bytes(label, m, n, k):
    """A + W + the output (+ the residual read), the figure DRAM traffic is held against."""
    out = m * (n // 2 if "swiglu" in label else n) * 2
    return m * k + n * k + out + (out if "residual" in label else 0)


def step_ops(dims, tokens, layers):
    return layers * sum(2.0 * m * n * k for m, n, k in gemm_shapes(dims, tokens).values())


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


def profiled_dram_bytes():
    """DRAM bytes per launch of the four GEMMs at 4608 tokens, from the committed ncu summary: table rows
    `| <stage label> | <read bytes> | <write bytes> |`.  Empty when the summary is absent."""
    path = os.path.join(ROOT, "profiles", "gemm_i8_dram_bytes_m4608.md")
    out = {}
    if os.path.exists(path):
        with open(path) as f:
            for line in f:
                row = re.fullmatch(r"\|\s*(.+?)\s*\|\s*([0-9]+)\s*\|\s*([0-9]+)\s*\|", line.strip())  # a label may hold a '|'
                if row and row.group(1) in GEMM_LABELS:
                    out[row.group(1)] = (int(row.group(2)), int(row.group(3)))
    return out, os.path.relpath(path, ROOT)


class ClockSampler:
    """nvidia-smi clocks, power and throttle reasons of one GPU while a timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,power.draw")

    def __init__(self, index):
        self.proc = None
        physical = os.environ.get("CUDA_VISIBLE_DEVICES", "").split(",")
        if physical != [""] and index < len(physical):
            index = physical[index]
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={index}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            pass

    def stop(self, skip_first=0.0):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        clocks, watts, peak, reasons = [], [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        lines = out.strip().splitlines()
        lines = lines[int(len(lines) * skip_first):]
        for line in lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                clocks.append(float(parts[0]))
                peak = float(parts[1])
                watts.append(float(parts[6]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": peak,
                "reasons": sorted(reasons), "samples": len(clocks),
                "watts": statistics.median(watts) if watts else None}


# ---------------------------------------------------------------------------------- CPU arm
class CpuChain:
    """One block of the W8A8 chain on the oracle (all host threads) at `tokens` rows.  The synthetic
    operands are built once; `seconds()` times one pass."""

    def __init__(self, dims, tokens):
        import numpy as np

        import oracle
        oracle.build()
        self.np, self.oracle, self.tokens = np, oracle, tokens
        h, inter = dims["hidden"], dims["inter"]
        self.h, self.inter = h, inter
        self.qkvg = 2 * h + 2 * dims["kv_heads"] * dims["head_dim"]
        self.ph = h + 64 if h % 8192 == 0 else h
        self.pi = inter + 64 if inter % 8192 == 0 else inter
        rng = np.random.default_rng(0)

        def rows(n, pitch):
            return rng.integers(-127, 128, size=(n, pitch), dtype=np.int16).astype(np.int8)

        self.w = {"qkvg": rows(self.qkvg, self.ph), "wo": rows(h, self.ph), "gu": rows(2 * inter, self.ph),
                  "down": rows(h, self.pi)}
        self.s = {k: rng.uniform(1e-3, 1e-2, size=v.shape[0]).astype(np.float32) for k, v in self.w.items()}
        self.vec = [(rng.standard_normal(h) * 0.1).astype(np.float32) for _ in range(8)]
        self.x = oracle.f32_to_bf16_bits(rng.standard_normal((tokens, h)).astype(np.float32))
        # Every host core, whatever OMP_NUM_THREADS the launcher exported (torchrun sets it to 1).
        oracle.set_threads(os.cpu_count() or 1)
        self.threads = oracle.threads()

    def seconds(self):
        o, np, w, s, vec = self.oracle, self.np, self.w, self.s, self.vec
        h, inter, qkvg, ph, pi = self.h, self.inter, self.qkvg, self.ph, self.pi
        start = time.perf_counter()
        a_q, a_s = o.prepare_norm_i8(self.x, vec[0], vec[1], vec[2], h, ph)
        fused = o.gemm_i8_256(a_q, w["qkvg"], s["qkvg"], a_s, h, ph, qkvg)
        attn = np.ascontiguousarray(fused[:, :h])
        a_q, a_s = o.prepare_gated_i8(attn, np.ascontiguousarray(fused[:, qkvg - h:]), h, ph, h)
        x1 = o.gemm_i8_resid_256(a_q, w["wo"], s["wo"], a_s, self.x, vec[3], h, ph, h)
        a_q, a_s = o.prepare_norm_i8(x1, vec[4], vec[5], vec[6], h, ph)
        gu = o.gemm_i8_swiglu_256(a_q, w["gu"], s["gu"], a_s, h, ph, 2 * inter)
        a_q, a_s = o.prepare_plain_i8(gu, inter, pi)
        o.gemm_i8_resid_256(a_q, w["down"], s["down"], a_s, x1, vec[7], inter, pi, h)
        return time.perf_counter() - start


def run_reference(args, dims, config):
    """The reference arm: the CPU port of the path's W8A8 chain, timed on this host's cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample_tokens = args.cpu_tokens
    block_ops = step_ops(dims, sample_tokens, 1)
    chain = CpuChain(dims, sample_tokens)
    threads = chain.threads
    for _ in range(args.warmup):
        chain.seconds()
    times = [chain.seconds() for _ in range(args.steps)]
    per = sum(times) / len(times)
    tops = block_ops / per / 1e12
    sample = (f"the W8A8 launches of one block at {sample_tokens} of {config['tokens']} tokens per step "
              f"(1/{config['layers']} of the layers)")
    line = {
        "impl": "reference", "metric": "w8a8_path_int8_tops", "value": tops, "unit": "TOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": per * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8 x int8 -> i32, f32/bf16 epilogue", "data": "synthetic",
        "config": config,
        "cpu_baseline": {"value": tops, "unit": "TOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tops, "unit": "TOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "ms_per_step is the time of the bounded sample, not of a whole step",
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------- GPU arm
def calibrate_int8(torch, local, m, n, k):
    """Calibration only, never a product path: the vendor library's int8 GEMM (`torch._int_mm`, raw i32 output,
    no epilogue) on the dominant GEMM's shape, as a 20-launch burst and as three seconds back to back under the
    power cap, with the SM clock sampled beside each."""
    gen = torch.Generator(device="cuda").manual_seed(7)
    a = torch.randint(-127, 128, (m, k), generator=gen, device="cuda", dtype=torch.int8)
    w = torch.randint(-127, 128, (n, k), generator=gen, device="cuda", dtype=torch.int8)
    ops_per_launch = 2.0 * m * n * k
    out = {}
    try:
        fn = lambda: torch._int_mm(a, w.t())
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        sampler = ClockSampler(local)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(20):
            fn()
        end.record()
        torch.cuda.synchronize()
        out["burst_tops"] = ops_per_launch / (start.elapsed_time(end) / 20 * 1e-3) / 1e12
        out["burst_clocks"] = sampler.stop()
        sampler = ClockSampler(local)
        launches, began = 0, time.time()
        start.record()
        while time.time() - began < 3.0:
            for _ in range(25):
                fn()
            launches += 25
            torch.cuda.synchronize()
        end.record()
        torch.cuda.synchronize()
        out["sustained_tops"] = ops_per_launch / (start.elapsed_time(end) / launches * 1e-3) / 1e12
        out["sustained_clocks"] = sampler.stop(skip_first=0.34)
        out["how"] = f"torch._int_mm {m}x{k} @ {k}x{n}, i32 output"
    except Exception as error:  # a build of torch without the int8 library path: report, do not fail the bench
        out["error"] = str(error)[:200]
    del a, w
    torch.cuda.empty_cache()
    return out


def timed_ms(torch, barrier, stream, fn, iters, warmup=2):
    for _ in range(warmup):
        fn()
    barrier()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(stream)
    for _ in range(iters):
        fn()
    end.record(stream)
    barrier()
    return start.elapsed_time(end) / iters


def max_over_ranks(torch, dist, world, values):
    t = torch.tensor(values, dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


def all_ranks_agree(torch, dist, world, ok):
    flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device="cuda")
    if world > 1:
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    return bool(flag.item())


def one_image_on_all_ranks(torch, dist, k, args, mdims, weights, rank, world, barrier, single, x_dev, mods_dev, cos, sin):
    """After the data-parallel timing: the N ranks run ONE image together.  `tp`: column-sharded weights (the
    W8A8 chain; the all-gather fused into the GEMM epilogues' peer stores, and the NCCL all-gather baseline);
    `sp`: token-sharded rows (the full block; K and V pushed by the RoPE launch, and the NCCL baseline).  All four
    under CUDA-graph replay, each checked bit for bit against this rank's single-GPU session."""
    from krea2_hrx_b200 import parallel
    stream = torch.cuda.current_stream()
    tokens, layers = single.tokens(), single.layers()
    if world > 1:  # ONE image: every rank works on rank 0's inputs
        x_dev, mods_dev, cos, sin = x_dev.clone(), mods_dev.clone(), cos.cuda(), sin.cuda()
        for t in (x_dev, mods_dev, cos, sin):
            dist.broadcast(t, src=0)
        cos, sin = cos.cpu(), sin.cpu()
    fabric = parallel.SymmetricFabric()
    out = {}
    iters = max(3, min(args.steps, 10))

    # -- column-sharded weights, the W8A8 chain
    single.set_attention(False)
    want = x_dev.clone()
    single.run_device(stream, want, mods_dev, cos, sin)
    single_chain_ms = timed_ms(torch, barrier, stream, lambda: single.run_device(stream, x_dev.clone(), mods_dev, cos, sin), iters)
    tp = parallel.TensorParallel(fabric, rank, mdims, parallel.shard_weights(weights, layers, world, rank), tokens)
    fabric.barrier()
    identical = True
    for collective in ("fused", "nccl"):
        got = tp.forward_graph(x_dev, mods_dev, collective)
        fabric.barrier()
        identical = all_ranks_agree(torch, dist, world, torch.equal(got.view(torch.int16), want.view(torch.int16))) and identical
    fused_ms = timed_ms(torch, fabric.barrier, stream, lambda: tp.forward_graph(x_dev, mods_dev, "fused"), iters)
    nccl_ms = timed_ms(torch, fabric.barrier, stream, lambda: tp.forward_graph(x_dev, mods_dev, "nccl"), iters)
    single_chain_ms, fused_ms, nccl_ms = max_over_ranks(torch, dist, world, [single_chain_ms, fused_ms, nccl_ms])
    d = mdims
    gathered = tokens * (d.qkvg + d.hidden + d.inter + d.hidden) * 2 * layers  # every GEMM output of the chain
    out["tp"] = {"what": "column-sharded weights within one image, W8A8 chain, CUDA-graph replay",
                 "bit_identical": identical, "layers": layers, "tokens": tokens, "single_gpu_ms": single_chain_ms,
                 "fused_ms": fused_ms, "nccl_ms": nccl_ms, "speedup": single_chain_ms / fused_ms,
                 "speedup_nccl": single_chain_ms / nccl_ms,
                 "received_mb_per_gpu": gathered * (world - 1) / world / 1e6,
                 "nvlink_floor_ms": gathered * (world - 1) / world / 770e9 * 1e3}
    del tp
    torch.cuda.empty_cache()

    # -- token-sharded rows, the full block
    single.set_attention(True)
    want = x_dev.clone()
    single.run_device(stream, want, mods_dev, cos, sin)
    single_full_ms = timed_ms(torch, barrier, stream, lambda: single.run_device(stream, x_dev.clone(), mods_dev, cos, sin), iters)
    sp = parallel.TokenParallel(fabric, rank, weights, tokens, layers)
    fabric.barrier()
    first, count = sp.rows
    identical = True
    for collective in ("push", "nccl"):
        got = sp.forward(x_dev, mods_dev, cos, sin, collective=collective, graph=True)
        fabric.barrier()
        same = torch.equal(got.view(torch.int16), want[first:first + count].view(torch.int16))
        identical = all_ranks_agree(torch, dist, world, same) and identical
    push_ms = timed_ms(torch, fabric.barrier, stream, lambda: sp.forward(x_dev, mods_dev, cos, sin, "push", graph=True), iters)
    sp_nccl_ms = timed_ms(torch, fabric.barrier, stream, lambda: sp.forward(x_dev, mods_dev, cos, sin, "nccl", graph=True), iters)
    single_full_ms, push_ms, sp_nccl_ms = max_over_ranks(torch, dist, world, [single_full_ms, push_ms, sp_nccl_ms])
    kv_bytes = 2 * tokens * d.kv_heads * d.head_dim * 2 * layers
    out["sp"] = {"what": "token-sharded rows within one image, full block with attention, CUDA-graph replay",
                 "bit_identical": identical, "layers": layers, "tokens": tokens, "rows_per_gpu": sp.share,
                 "single_gpu_ms": single_full_ms, "push_ms": push_ms, "nccl_ms": sp_nccl_ms,
                 "speedup": single_full_ms / push_ms, "speedup_nccl": single_full_ms / sp_nccl_ms,
                 "received_mb_per_gpu": kv_bytes * (world - 1) / world / 1e6,
                 "nvlink_floor_ms": kv_bytes * (world - 1) / world / 770e9 * 1e3}
    # -- the 8-step loop of ONE image on the token-sharded ranks, against the same loop on one GPU
    from krea2_hrx_b200 import pipeline
    gen = torch.Generator().manual_seed(77)  # the same prompt, noise and tables on every rank
    text_tokens = min(512, tokens // 2)
    text = torch.randn((text_tokens, d.hidden), generator=gen).to(torch.bfloat16).cuda()
    noise = torch.randn((tokens - text_tokens, d.hidden), generator=gen).to(torch.bfloat16).cuda()
    tables = (torch.randn((layers, 6, d.hidden), generator=gen) * 0.1).to(torch.bfloat16).cuda()
    vectors = [(torch.randn(6 * d.hidden, generator=gen) * 0.1).to(torch.bfloat16).cuda() for _ in range(8)]
    alone = pipeline.Denoiser(single, tables, cos, sin, text, steps=8)
    together = pipeline.ShardedDenoiser(sp, tables, cos, sin, text, steps=8, collective="push", graph=True)
    want = alone.generate(noise.clone(), vectors)
    got = together.gather(together.generate(noise.clone(), vectors))
    fabric.barrier()
    same = all_ranks_agree(torch, dist, world, torch.equal(got.view(torch.int16), want.view(torch.int16)))
    alone_ms = timed_ms(torch, barrier, stream, lambda: alone.generate(noise.clone(), vectors), 2, warmup=1)
    together_ms = timed_ms(torch, fabric.barrier, stream,
                           lambda: together.gather(together.generate(noise.clone(), vectors)), 2, warmup=1)
    alone_ms, together_ms = max_over_ranks(torch, dist, world, [alone_ms, together_ms])
    out["sp"]["image"] = {"what": "8 Turbo steps of one image, rows sharded over the ranks from the first step to the "
                                  "last, one gather of the sample at the end", "steps": 8, "bit_identical": same,
                          "single_gpu_ms": alone_ms, "sharded_ms": together_ms, "speedup": alone_ms / together_ms}
    out["device_status_after_sharded_runs"] = k.device_status()
    del sp, together
    torch.cuda.empty_cache()
    return out


def largest_sequence(torch, k, session, args, mdims, weights, barrier, dist, world, rank):
    """One forward per GPU at the largest sequence a session serves (2048 x 2048: 16384 image + 512 text tokens).
    Checked without a CPU: every token goes through the W8A8 chain on its own, so sampled rows of the W8A8-only
    forward must equal a small session's forward over just those rows, bit for bit."""
    tokens, layers = 16896, args.layers
    stream = torch.cuda.current_stream()
    gen = torch.Generator().manual_seed(100 + rank)
    x = torch.randn((tokens, mdims.hidden), generator=gen).to(torch.bfloat16)
    mods = torch.randn((layers, 6, mdims.hidden), generator=gen) * 0.1
    cos = torch.cos(torch.rand((tokens, mdims.head_dim), generator=gen) * 6.28).contiguous()
    sin = torch.sin(torch.rand((tokens, mdims.head_dim), generator=gen) * 6.28).contiguous()
    x_dev, mods_dev = x.cuda(), mods.cuda()
    big = session.Session(stream, weights, tokens, layers)
    big.set_attention(False)
    chain_out = x_dev.clone()
    big.run_device(stream, chain_out, mods_dev, cos, sin)
    rows = torch.tensor([0, 1, 255, 256, 4607, 8191, 8192, 12345, 16383, 16384, 16800, 16895] + list(range(5000, 5020)))
    small = session.Session(stream, weights, len(rows), layers)
    small.set_attention(False)
    sampled = x_dev[rows.cuda()].contiguous()
    small.run_device(stream, sampled, mods_dev, cos[: len(rows)].contiguous(), sin[: len(rows)].contiguous())
    torch.cuda.synchronize()
    match = torch.equal(sampled.view(torch.int16), chain_out[rows.cuda()].view(torch.int16))
    small.close()
    iters = 3
    chain_ms = timed_ms(torch, barrier, stream, lambda: big.run_device(stream, x_dev.clone(), mods_dev, cos, sin), iters, warmup=1)
    big.set_attention(True)
    full_ms = timed_ms(torch, barrier, stream, lambda: big.run_device(stream, x_dev.clone(), mods_dev, cos, sin), iters, warmup=1)
    big.close()
    status = k.device_status()
    chain_ms, full_ms = max_over_ranks(torch, dist, world, [chain_ms, full_ms])
    match = all_ranks_agree(torch, dist, world, match and status == 0)
    ops = step_ops(dict(hidden=mdims.hidden, kv_heads=mdims.kv_heads, head_dim=mdims.head_dim, inter=mdims.inter), tokens, layers)
    torch.cuda.empty_cache()
    return {"what": "one forward per GPU at 2048x2048 (16384 image + 512 text tokens), an image per GPU",
            "tokens": tokens, "layers": layers, "images": world, "ms_per_step": full_ms, "w8a8_chain_ms_per_step": chain_ms,
            "tops": world * ops / (full_ms * 1e-3) / 1e12, "w8a8_chain_tops": world * ops / (chain_ms * 1e-3) / 1e12,
            "sampled_rows_match_a_small_session": match}


def run_b200(args, dims, config):
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")  # plain peer stores and rings only: nothing is bound to a multicast object
    import torch
    import torch.distributed as dist

    import krea2_hrx_b200 as k
    from krea2_hrx_b200 import pipeline, session

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the W8A8 path has no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    tokens, layers = config["tokens"], config["layers"]
    image_tokens = tokens - TEXT_TOKENS
    mdims = session.ModelDims(**dims)
    stream = torch.cuda.current_stream()
    weights = session.Weights(mdims, layers)
    weights.fill_synthetic(1234, stream)  # replicated: the same seed on every rank
    s = session.Session(stream, weights, tokens, layers)
    s.set_attention(True)
    full_block = s.set_attention(True)  # the second call reports whether the first one took (head shape permitting)
    # consecutive seeds per image, as `--images N` does (src/main.rs:48-50)
    gen = torch.Generator().manual_seed(rank)
    x_host = torch.randn((tokens, mdims.hidden), generator=gen).to(torch.bfloat16).pin_memory()
    mods_host = (torch.randn((layers, 6, mdims.hidden), generator=gen) * 0.1).pin_memory()
    cos = torch.cos(torch.rand((tokens, mdims.head_dim), generator=gen) * 6.28).contiguous()
    sin = torch.sin(torch.rand((tokens, mdims.head_dim), generator=gen) * 6.28).contiguous()
    tables = (torch.randn((layers, 6, mdims.hidden), generator=gen) * 0.1).to(torch.bfloat16).cuda()
    vectors = [(torch.randn(6 * mdims.hidden, generator=gen) * 0.05).to(torch.bfloat16).cuda() for _ in range(TURBO_STEPS)]
    x_first = x_host.clone()
    x_dev = x_host.cuda()
    mods_dev = mods_host.cuda()
    text = x_dev[:TEXT_TOKENS].contiguous()
    sample = x_dev[TEXT_TOKENS:].contiguous()
    ops_per_step = step_ops(dims, tokens, layers)
    denoiser = pipeline.Denoiser(s, tables, cos, sin, text, steps=TURBO_STEPS)
    counter = [0]

    def device_step():
        index = counter[0] % TURBO_STEPS
        if index == 0:
            sample.copy_(x_dev[TEXT_TOKENS:], non_blocking=True)  # a new image's noise every eight steps
        denoiser.step(index, sample, vectors[index])
        counter[0] += 1

    for _ in range(args.warmup):
        device_step()
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(stream)
    for _ in range(args.steps):
        device_step()
    end.record(stream)
    barrier()
    elapsed_ms = start.elapsed_time(end)
    clocks = sampler.stop() if sampler else None
    launches_per_step = s.launches_per_forward() + 2  # the session's kernels, modulation and euler

    # The same step back to back for three seconds with board power sampled beside it (rank 0): the step is bound
    # by the 1 kW cap, so joules per step is the figure a kernel change has to move.  Not part of `value`.
    sustained = None
    if not args.no_sustained:
        barrier()
        power = ClockSampler(local) if rank == 0 else None
        s_start, s_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        count, began = 0, time.time()
        s_start.record(stream)
        while time.time() - began < 3.0:
            for _ in range(4):
                device_step()
            count += 4
            torch.cuda.synchronize()
        s_end.record(stream)
        barrier()
        sustained_ms = s_start.elapsed_time(s_end) / count
        if power:
            sampled = power.stop(skip_first=0.34)
            sustained = {"seconds": 3.0, "steps": count, "ms_per_step": sustained_ms, "sm_mhz": sampled["sm_mhz"],
                         "watts": sampled["watts"], "reasons": sampled["reasons"],
                         "joules_per_step": sampled["watts"] * sustained_ms * 1e-3 if sampled["watts"] else None}

    # The same 28 blocks without the three launches that are not W8A8 products.
    s.set_attention(False)
    chain_ms = timed_ms(torch, barrier, stream, lambda: s.run_device(stream, x_dev, mods_dev, cos, sin), args.steps)
    s.set_attention(True)

    # End to end: pinned host buffers in, residual stream back, every step, through Session.run.  Two sessions
    # over the same weights, each on a stream and a host thread of its own (the crate's sessions share an
    # Arc<Weights> the same way), so one step's copies overlap the other session's kernels; every step still
    # copies its inputs in and its result out inside the timed region.  `single_session_ms` is one session alone.
    import threading
    lanes = []
    for _ in range(2):
        lane_stream = torch.cuda.Stream()
        lane = session.Session(lane_stream, weights, tokens, layers)
        lane.set_attention(True)
        lanes.append((lane, lane_stream, x_first.clone().pin_memory()))

    def drive(index, count):
        torch.cuda.set_device(local)  # the current device is per host thread
        lane, lane_stream, x_pinned = lanes[index]
        for _ in range(count):
            lane.run(lane_stream, x_pinned, mods_host, cos, sin)

    def run_lanes(total):
        workers = [threading.Thread(target=drive, args=(i, (total + 1 - i) // 2)) for i in range(2)]
        for w in workers:
            w.start()
        for w in workers:
            w.join()

    run_lanes(2 * min(args.warmup, 2))
    barrier()
    e2e_start = time.perf_counter()
    e_start, e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e_start.record(stream)
    run_lanes(args.steps)
    torch.cuda.synchronize()
    e_end.record(stream)
    barrier()
    e2e_ms = max(e_start.elapsed_time(e_end), 0.0)
    e2e_wall_ms = (time.perf_counter() - e2e_start) * 1e3
    drive(0, 1)
    barrier()
    single_start = time.perf_counter()
    drive(0, max(3, args.steps // 2))
    single_session_ms = (time.perf_counter() - single_start) * 1e3 / max(3, args.steps // 2)
    for lane, _, _ in lanes:
        lane.close()
    del lanes

    elapsed_ms, chain_ms, e2e_ms, e2e_wall_ms, single_session_ms = max_over_ranks(
        torch, dist, world, [elapsed_ms, chain_ms, e2e_ms, e2e_wall_ms, single_session_ms])

    # per-stage device time of one forward (events between launches on the session's stream)
    s.set_profile(True)
    x_prof = x_first.clone().pin_memory()
    s.run(stream, x_prof, mods_host, cos, sin)
    stage_ms = dict(s.stage_profile())
    s.set_profile(False)
    status = k.device_status()

    # The legs after the headline: a failure that every rank meets alike (an allocation that does not fit, a
    # library call this torch build lacks) is reported in the line instead of costing the numbers above.
    extra = {}
    if world > 1 and not args.no_sharded:
        try:
            extra.update(one_image_on_all_ranks(torch, dist, k, args, mdims, weights, rank, world, barrier, s, x_dev, mods_dev,
                                                cos, sin))
        except Exception as error:  # noqa: BLE001
            extra["sharded_runs_error"] = f"{type(error).__name__}: {error}"[:300]
    if (world > 1 or args.config4) and not args.no_config4:
        try:
            extra["config4"] = largest_sequence(torch, k, session, args, mdims, weights, barrier, dist, world, rank)
        except Exception as error:  # noqa: BLE001
            extra["config4"] = {"error": f"{type(error).__name__}: {error}"[:300]}

    if rank == 0:
        peaks, peak_source = measured_peaks()
        ms_per_step = elapsed_ms / args.steps
        value = world * ops_per_step / (ms_per_step * 1e-3) / 1e12
        e2e_value = world * ops_per_step / (e2e_ms / args.steps * 1e-3) / 1e12
        shapes = gemm_shapes(dims, tokens)
        dram, dram_source = profiled_dram_bytes()
        kernels = {}
        for label, (m, n, kk) in shapes.items():
            per_launch_ms = stage_ms[label] / layers
            entry = {"m": m, "n": n, "k": kk, "ms_per_launch": per_launch_ms,
                     "tops": 2.0 * m * n * kk / (per_launch_ms * 1e-3) / 1e12,
                     "frac_of_nominal_4500": 2.0 * m * n * kk / (per_launch_ms * 1e-3) / 1e12 / NOMINAL_INT8_TOPS}
            if label in dram and tokens == 4608:
                algorithmic = gemm_algorithmic_bytes(label, m, n, kk)
                entry.update({"dram_bytes_per_launch": sum(dram[label]), "algorithmic_bytes_per_launch": algorithmic,
                              "dram_over_algorithmic": sum(dram[label]) / algorithmic})
            kernels[label] = entry
        # The prologues against the HBM roofline: algorithmic bytes = one read of each 16-bit input row, one
        # int8 row and one f32 scale per token (the f32 [K] vectors are amortised over the tokens).
        hidden, inter = mdims.hidden, mdims.inter
        prologue_bytes = {"prepare": (2 * layers, tokens * (2 * hidden + hidden + 4)),
                          "prepare gated": (layers, tokens * (4 * hidden + hidden + 4)),
                          "prepare swiglu": (layers, tokens * (2 * inter + inter + 4))}
        for label, (launches, nbytes) in prologue_bytes.items():
            ms = stage_ms.get(label, 0.0)
            gbs = nbytes / (ms / launches * 1e-3) / 1e9 if ms > 0 else 0.0
            kernels[label] = {"ms_per_forward": ms, "launches": launches, "algorithmic_mb_per_launch": nbytes / 1e6,
                              "gbs": gbs, "frac_of_hbm": gbs / peaks["hbm_gbs"]}
        if full_block:
            q_heads = mdims.hidden // mdims.head_dim
            attention_flop = 4.0 * tokens * tokens * mdims.head_dim * q_heads
            attention_ms = stage_ms.get("f16 attention", 0.0) / layers
            kernels["f16 attention"] = {"ms_per_launch": attention_ms,
                                        "tflops": attention_flop / (attention_ms * 1e-3) / 1e12 if attention_ms else None,
                                        "frac_of_bf16_sustained": (attention_flop / (attention_ms * 1e-3) / 1e12 /
                                                                   peaks["bf16_tflops_sustained"]) if attention_ms else None}
            kernels["qk norm + rope"] = {"ms_per_launch": stage_ms.get("qk norm + rope", 0.0) / layers}
            kernels["V transpose"] = {"ms_per_launch": stage_ms.get("V transpose", 0.0) / layers}
        gu = kernels["gemm gate|up + swiglu"]
        int8_peak = 2.0 * peaks["bf16_tflops_sustained"]
        roofline = {
            "bound": "tensor", "kernel": "gemm_i8_swiglu_256 (gate|up, M=%d N=%d K=%d)" % shapes["gemm gate|up + swiglu"],
            "achieved": gu["tops"], "peak": int8_peak, "unit": "TOP/s", "frac": gu["tops"] / int8_peak,
            "peak_source": f"2 x bf16_tflops_sustained of {peak_source} MEASURED_PEAKS (int8 issues at twice the bf16 rate; "
                           "the file has no int8 figure)",
            "frac_of_nominal_4500": gu["tops"] / NOMINAL_INT8_TOPS,
            "traffic": gu.get("dram_bytes_per_launch"),
            "traffic_source": f"{dram_source}: ncu dram__bytes_read.sum + dram__bytes_write.sum per launch" if dram else None,
        }
        if world == 1 and not args.no_calibration:
            m, n, kk = shapes["gemm gate|up + swiglu"]
            calibration = calibrate_int8(torch, local, m, n, kk)
            roofline["calibration"] = calibration
            if "sustained_tops" in calibration:
                roofline["peak_calibrated_burst"] = calibration["burst_tops"]
                roofline["peak_calibrated_sustained"] = calibration["sustained_tops"]
                roofline["frac_calibrated"] = gu["tops"] / calibration["sustained_tops"]
        gemm_ms = sum(stage_ms[label] for label in shapes)
        line = {
            "metric": "w8a8_path_int8_tops", "value": value, "unit": "TOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int8 x int8 -> i32, f32/bf16 epilogue; f16 attention", "data": "synthetic",
            "config": config,
            "e2e": {"value": e2e_value, "unit": "TOP/s", "ms_per_step": e2e_ms / args.steps,
                    "wall_ms_per_step": e2e_wall_ms / args.steps, "single_session_ms": single_session_ms,
                    "h2d_bytes_per_step": x_host.numel() * 2 + mods_host.numel() * 4,
                    "d2h_bytes_per_step": x_host.numel() * 2,
                    "how": "Session.run (full block) from pinned host buffers, two sessions over shared weights on two "
                           "streams and host threads, so a step's copies overlap the other session's kernels; "
                           "single_session_ms is one session alone, wall clock per call"},
            "gpu_launches": args.steps * launches_per_step,
            "clocks": clocks,
            "roofline": roofline,
            "kernels": kernels,
            "frac_of_nominal_int8_peak": value / world / NOMINAL_INT8_TOPS,
            "gemm_only": {"ms_per_forward": gemm_ms, "tops": ops_per_step / (gemm_ms * 1e-3) / 1e12,
                          "how": "sum of the four GEMM stages of a profiled forward (events between launches)"},
            "w8a8_chain": {"ms_per_step": chain_ms, "tops": world * ops_per_step / (chain_ms * 1e-3) / 1e12,
                           "launches_per_step": layers * 8,
                           "what": "the same 28 blocks without QK-norm + RoPE, V transpose and attention (the query "
                                   "columns in the attention output's place)"},
            "sustained": sustained,
            "device_status": status,
        }
        line.update(extra)
        if world == 1 and not args.no_cpu_baseline:
            rows = 4 * args.cpu_tokens
            chain = CpuChain(dims, rows)
            seconds = chain.seconds()
            line["cpu_baseline"] = {
                "value": step_ops(dims, rows, 1) / seconds / 1e12, "unit": "TOP/s", "cores": chain.threads,
                "kind": "port",
                "sample": f"the W8A8 launches of one block at {rows} of {tokens} tokens (1/{layers} of the layers), {seconds:.1f} s",
            }
        print(json.dumps(line), flush=True)
    s.close()
    if world > 1:
        barrier()
        dist.destroy_process_group()


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=10)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--tokens", type=int, default=4608)
    parser.add_argument("--layers", type=int, default=28)
    parser.add_argument("--cpu-tokens", type=int, default=512, help="rows of the CPU baseline's bounded sample")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-calibration", action="store_true", help="skip the vendor-library int8 calibration")
    parser.add_argument("--no-sustained", action="store_true", help="skip the three-second back-to-back run with power sampling")
    parser.add_argument("--no-sharded", action="store_true", help="N > 1: skip the one-image-on-all-ranks runs")
    parser.add_argument("--no-config4", action="store_true", help="N > 1: skip the 16896-token forward")
    parser.add_argument("--config4", action="store_true", help="N = 1: also run the 16896-token forward")
    args = parser.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    dims = DIMS["reference"]
    config = {
        "workload": "one denoising step at 1024x1024 of the 8-step Turbo loop: modulation, 28 blocks x eleven launches "
                    "(3 prologues, 4 int8 GEMMs, QK-norm + RoPE, V transpose, fp16 attention), Euler; reference dimensions",
        "tokens": args.tokens, "layers": args.layers, **dims,
        "images_per_step": int(os.environ.get("WORLD_SIZE", "1")) if args.impl == "b200" else 1,
        "parallelism": f"dp{args.gpus} over images" if args.gpus > 1 else "single GPU",
        "l2": "inputs larger than L2: each step streams 12.2 GB of int8 weights",
    }
    if args.impl == "reference":
        run_reference(args, dims, config)
    else:
        run_b200(args, dims, config)


if __name__ == "__main__":
    main()
