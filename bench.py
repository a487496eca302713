#!/usr/bin/env python
"""Benchmark of the W8A8 linear-layer path of one denoising step.

A "step" is the W8A8 chain of the 28 transformer blocks for one 1024x1024 image (4096 image +
512 text tokens) at the reference's dimensions (d 6144, q|k|v|gate 15360, SwiGLU 16384): per
block prepare_norm -> gemm qkvg -> [a copy in attention's place] -> prepare_gated -> gemm wo +
residual -> prepare_norm -> gemm gate|up + SwiGLU -> prepare_plain -> gemm down + residual, on
seeded synthetic int8 weights (12.2 GB, so every step streams far more than L2 holds).
`full_block_step` in the output is the same step with the session's attention on (QK-norm +
RoPE, V transpose, fp16 attention: the reference's eleven launches per block).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

`value` is the integer-op rate of the four GEMMs (2*M*N*K summed over the step) divided by the
device time of the WHOLE chain, inputs resident in HBM, replayed as one CUDA graph through
krea2_session_run_device.  `e2e` is the same through krea2_session_run (two sessions in flight): host x and modulation
tables in pinned memory, copied in and read back inside the timed region.  With N > 1 every
rank runs its own image on its own GPU (independent sessions, replicated weights, no
collective on the data path): weak scaling.

--impl reference times the CPU restatement of the reference's arithmetic (the oracle; the
reference's own kernels need an AMD GPU and a Rust toolchain) on the host cores, on a bounded
sample of the same step.
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

DIMS = {  # hidden, kv_heads, head_dim, inter
    "reference": dict(hidden=6144, kv_heads=12, head_dim=128, inter=16384),  # src/session/mod.rs:35-45
}
NOMINAL_INT8_TOPS = 4500.0  # dense int8 tensor peak of a B200, vendor figure

# DRAM bytes (read + write) of one gate|up GEMM launch at M=4608, from the ncu capture summarised
# in profiles/gemm_i8_pair_kernel_qkvg_gateup_m4608.md (algorithmic bytes A + W + C: 380.6 MB).
GU_GEMM_DRAM_BYTES_PER_LAUNCH = 371.6e6


def gemm_shapes(dims, tokens):
    h, inter = dims["hidden"], dims["inter"]
    qkvg = 2 * h + 2 * dims["kv_heads"] * dims["head_dim"]
    return {"gemm qkvg": (tokens, qkvg, h), "gemm wo + residual": (tokens, h, h),
            "gemm gate|up + swiglu": (tokens, 2 * inter, h), "gemm down + residual": (tokens, h, inter)}


def step_ops(dims, tokens, layers):
    return layers * sum(2.0 * m * n * k for m, n, k in gemm_shapes(dims, tokens).values())


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={index}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            pass

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        clocks, peak, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                clocks.append(float(parts[0]))
                peak = float(parts[1])
            except ValueError:
                continue
            for name, flag in zip(names, parts[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": peak,
                "reasons": sorted(reasons), "samples": len(clocks)}


# ---------------------------------------------------------------------------------- CPU arm
class CpuChain:
    """One block of the chain on the oracle (all host threads) at `tokens` rows.  The synthetic
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
    """The reference arm: the CPU port of the path, timed on this host's cores."""
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
    sample = f"one block of the chain at {sample_tokens} of {config['tokens']} tokens per step (1/{config['layers']} of the layers)"
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
def run_b200(args, dims, config):
    import torch
    import torch.distributed as dist

    import krea2_hrx_b200 as k
    from krea2_hrx_b200 import session

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
    mdims = session.ModelDims(**dims)
    stream = torch.cuda.current_stream()
    weights = session.Weights(mdims, layers)
    weights.fill_synthetic(1234, stream)  # replicated: the same seed on every rank
    s = session.Session(stream, weights, tokens, layers)
    s.set_attention(False)  # the headline is the W8A8 chain; the full block is measured further down
    # consecutive seeds per image, as `--images N` does (src/main.rs:48-50)
    gen = torch.Generator().manual_seed(rank)
    x_host = torch.randn((tokens, mdims.hidden), generator=gen).to(torch.bfloat16).pin_memory()
    mods_host = (torch.randn((layers, 6, mdims.hidden), generator=gen) * 0.1).pin_memory()
    cos = torch.cos(torch.rand((tokens, mdims.head_dim), generator=gen) * 6.28).contiguous()
    sin = torch.sin(torch.rand((tokens, mdims.head_dim), generator=gen) * 6.28).contiguous()
    x_first = x_host.clone()
    x_dev = x_host.cuda()
    mods_dev = mods_host.cuda()
    ops_per_step = step_ops(dims, tokens, layers)

    def device_step():
        s.run_device(stream, x_dev, mods_dev, cos, sin)

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

    # End to end: pinned host buffers in, residual stream back, every step, through Session.run.  Two sessions
    # over the same weights, each on a stream and a host thread of its own (the crate's sessions share an
    # Arc<Weights> the same way), so one step's copies overlap the other session's kernels; every step still
    # copies its inputs in and its result out inside the timed region.
    import threading
    lanes = []
    for _ in range(2):
        lane_stream = torch.cuda.Stream()
        lane = session.Session(lane_stream, weights, tokens, layers)
        lane.set_attention(False)
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
    for lane, _, _ in lanes:
        lane.close()

    times = torch.tensor([elapsed_ms, e2e_ms, e2e_wall_ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    elapsed_ms, e2e_ms, e2e_wall_ms = times.tolist()

    # per-stage device time of one forward (events between launches on the session's stream)
    s.set_profile(True)
    x_prof = x_first.clone().pin_memory()
    s.run(stream, x_prof, mods_host, cos, sin)
    stage_ms = dict(s.stage_profile())
    s.set_profile(False)

    # The full block chain (QK-norm + RoPE, V transpose and fp16 attention between the q|k|v|gate GEMM and
    # the gated prologue): what one denoising step of the 28 blocks costs, beside the W8A8 chain above.
    full = None
    s.set_attention(True)
    if s.set_attention(True):  # the second call reports whether the first one took (head shape permitting)
        for _ in range(2):
            device_step()
        barrier()
        f_start, f_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f_start.record(stream)
        for _ in range(args.steps):
            device_step()
        f_end.record(stream)
        barrier()
        full_ms = torch.tensor([f_start.elapsed_time(f_end) / args.steps], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(full_ms, op=dist.ReduceOp.MAX)
        s.set_profile(True)
        s.run(stream, x_prof, mods_host, cos, sin)
        full_stage_ms = dict(s.stage_profile())
        s.set_profile(False)
        q_heads = mdims.hidden // mdims.head_dim
        attention_flop = 4.0 * tokens * tokens * mdims.head_dim * q_heads
        attention_ms = full_stage_ms.get("f16 attention", 0.0) / layers
        full = {"ms_per_step": full_ms.item(), "launches_per_step": s.launches_per_forward(),
                "attention_ms_per_launch": attention_ms,
                "attention_tflops": attention_flop / (attention_ms * 1e-3) / 1e12 if attention_ms else None,
                "rope_ms_per_launch": full_stage_ms.get("qk norm + rope", 0.0) / layers,
                "v_transpose_ms_per_launch": full_stage_ms.get("V transpose", 0.0) / layers}
    s.set_attention(False)
    status = k.device_status()

    if rank == 0:
        peaks, peak_source = measured_peaks()
        ms_per_step = elapsed_ms / args.steps
        value = world * ops_per_step / (ms_per_step * 1e-3) / 1e12
        e2e_value = world * ops_per_step / (e2e_ms / args.steps * 1e-3) / 1e12
        shapes = gemm_shapes(dims, tokens)
        kernels = {}
        for label, (m, n, kk) in shapes.items():
            per_launch_ms = stage_ms[label] / layers
            kernels[label] = {"m": m, "n": n, "k": kk, "ms_per_launch": per_launch_ms,
                              "tops": 2.0 * m * n * kk / (per_launch_ms * 1e-3) / 1e12}
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
        gu = kernels["gemm gate|up + swiglu"]
        int8_peak = 2.0 * peaks["bf16_tflops_sustained"]
        roofline = {
            "bound": "tensor", "kernel": "gemm_i8_swiglu_256 (gate|up, M=%d N=%d K=%d)" % shapes["gemm gate|up + swiglu"],
            "achieved": gu["tops"], "peak": int8_peak, "unit": "TOP/s", "frac": gu["tops"] / int8_peak,
            "peak_source": f"2 x bf16_tflops_sustained of {peak_source} MEASURED_PEAKS (int8 issues at twice the bf16 rate)",
            "frac_of_nominal_4500": gu["tops"] / NOMINAL_INT8_TOPS,
            "traffic": GU_GEMM_DRAM_BYTES_PER_LAUNCH,
        }
        line = {
            "metric": "w8a8_path_int8_tops", "value": value, "unit": "TOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int8 x int8 -> i32, f32/bf16 epilogue", "data": "synthetic",
            "config": config,
            "e2e": {"value": e2e_value, "unit": "TOP/s", "ms_per_step": e2e_ms / args.steps,
                    "wall_ms_per_step": e2e_wall_ms / args.steps,
                    "h2d_bytes_per_step": x_host.numel() * 2 + mods_host.numel() * 4,
                    "d2h_bytes_per_step": x_host.numel() * 2,
                    "how": "Session.run from pinned host buffers, two sessions over shared weights on two streams and "
                           "host threads, so a step's copies overlap the other session's kernels"},
            "gpu_launches": args.steps * s.launches_per_forward(),
            "clocks": clocks,
            "roofline": roofline,
            "kernels": kernels,
            "frac_of_nominal_int8_peak": value / world / NOMINAL_INT8_TOPS,
            "full_block_step": full,
            "device_status": status,
        }
        if world == 1 and not args.no_cpu_baseline:
            rows = 4 * args.cpu_tokens
            chain = CpuChain(dims, rows)
            seconds = chain.seconds()
            line["cpu_baseline"] = {
                "value": step_ops(dims, rows, 1) / seconds / 1e12, "unit": "TOP/s", "cores": chain.threads,
                "kind": "port",
                "sample": f"one block of the chain at {rows} of {tokens} tokens (1/{layers} of the layers), {seconds:.1f} s",
            }
        print(json.dumps(line), flush=True)
    s.close()
    if world > 1:
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
    args = parser.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    dims = DIMS["reference"]
    config = {
        "workload": "W8A8 chain of one denoising step at 1024x1024: 28 blocks x (3 prologues + 4 int8 GEMMs), "
                    "reference dimensions",
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
