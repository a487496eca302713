"""Per-kernel timings of the W8A8 path, the counterpart of the reference's kernel bench
(benches/kernels.rs:56-193: the four GEMMs over M in {1043, 4095, 4096, 4109, 12301, 16397}).

    python -m krea2_hrx_b200.bench_kernels --kernel all --m 4608
    python -m krea2_hrx_b200.bench_kernels --kernel gu --m 4608 --dims baseline --iters 20

Each line of output is one JSON object: the kernel, its shape, the mean CUDA-event time of
`iters` back-to-back launches after `warmup` (a 256 MB buffer is rewritten between timed
launches when --flush-l2 is given; GEMM weights at these sizes exceed L2 anyway), and the
rate against its roofline: integer TOP/s for GEMMs (2*M*N*K), algorithmic GB/s for prologues
(one read of the 16-bit rows, one int8 row and one f32 scale written per token).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from krea2_hrx_b200 import ops, shape  # noqa: E402

DIMS = {
    # hidden, fused q|k|v|gate (or q|k|v) width, SwiGLU inner width
    "reference": dict(hidden=6144, qkv=15360, inter=16384),  # src/session/mod.rs:35-45
    "baseline": dict(hidden=3072, qkv=9216, inter=8192),     # the benchmark brief's literal dimensions (d 3072, QKV 9216, SwiGLU 8192)
}
REFERENCE_M = [1043, 4095, 4096, 4109, 12301, 16397]  # benches/kernels.rs:64


def gemm_case(kind, dims):
    h, qkv, inter = dims["hidden"], dims["qkv"], dims["inter"]
    return {"qkvg": ("gemm_i8_256", h, qkv), "wo": ("gemm_i8_resid_256", h, h), "gu": ("gemm_i8_swiglu_256", h, 2 * inter),
            "down": ("gemm_i8_resid_256x256", inter, h), "acc": ("gemm_i8_acc", h, qkv),
            "gurot": ("gemm_i8_swiglu_rotated_256", h, 2 * inter), "qkvgrope": ("gemm_i8_rope_256", h, qkv)}[kind]


SUSTAIN_SECONDS = 0.0   # --sustain: also run every timed kernel back to back this long, sampling power and clock
LAST_SUSTAINED = {}


def sustained_run(fn, seconds):
    """Back-to-back launches for `seconds` with nvidia-smi sampling beside them: the mean launch time under the
    power cap, the median board power and SM clock, and their product, the energy of one launch."""
    import subprocess
    import time
    index = str(torch.cuda.current_device())
    physical = os.environ.get("CUDA_VISIBLE_DEVICES", "").split(",")
    if physical != [""] and int(index) < len(physical):
        index = physical[int(index)]
    sampler = subprocess.Popen(["nvidia-smi", "-i", index, "--query-gpu=clocks.sm,power.draw", "--format=csv,noheader,nounits",
                                "-lms", "100"], stdout=subprocess.PIPE, text=True)
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches, began = 0, time.time()
    start.record()
    while time.time() - began < seconds:
        for _ in range(50):
            fn()
        launches += 50
        torch.cuda.synchronize()
    end.record()
    torch.cuda.synchronize()
    sampler.terminate()
    rows = [line.split(",") for line in sampler.communicate()[0].strip().splitlines() if "," in line]
    rows = rows[len(rows) // 3:]  # the part is still ramping during the first samples
    clocks = sorted(float(r[0]) for r in rows)
    watts = sorted(float(r[1]) for r in rows)
    ms = start.elapsed_time(end) / launches
    out = {"sustained_ms": ms}
    if rows:
        out.update({"sm_mhz": clocks[len(clocks) // 2], "watts": watts[len(watts) // 2],
                    "joules_per_launch": watts[len(watts) // 2] * ms * 1e-3})
    return out


def time_launches(fn, iters, warmup, flush):
    ms = burst_time(fn, iters, warmup, flush)
    if SUSTAIN_SECONDS > 0:
        LAST_SUSTAINED.clear()
        LAST_SUSTAINED.update(sustained_run(fn, SUSTAIN_SECONDS))
    return ms


def burst_time(fn, iters, warmup, flush):
    scratch = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    stream = torch.cuda.current_stream()
    if flush:
        total = 0.0
        for _ in range(iters):
            scratch.fill_(1)
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record(stream)
            fn()
            end.record(stream)
            torch.cuda.synchronize()
            total += start.elapsed_time(end)
        return total / iters
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(stream)
    for _ in range(iters):
        fn()
    end.record(stream)
    torch.cuda.synchronize()
    return start.elapsed_time(end) / iters


def run_gemm(kind, m, dims, iters, warmup, flush):
    name, k, n = gemm_case(kind, dims)
    pitch = shape.gemm_pitch(k)
    gen = torch.Generator(device="cuda").manual_seed(m + n)
    a = torch.randint(-127, 128, (m, pitch), generator=gen, device="cuda", dtype=torch.int8)
    w = torch.randint(-127, 128, (n, pitch), generator=gen, device="cuda", dtype=torch.int8)
    ws = torch.rand(n, generator=gen, device="cuda") * 9e-3 + 1e-3
    a_scale = torch.rand(m, generator=gen, device="cuda") * 0.05 + 1e-3
    gate = torch.randn(n, generator=gen, device="cuda") * 0.1
    if name == "gemm_i8_256":
        c = torch.empty((m, n), dtype=torch.float16, device="cuda")
        fn = lambda: ops.gemm_i8_256(m, a, w, ws, a_scale, c, k, pitch, n)
    elif name == "gemm_i8_rope_256":
        q_heads, kv_heads = dims["hidden"] // 128, max(1, (n - 2 * dims["hidden"]) // 256)
        c = torch.empty((m, n), dtype=torch.float16, device="cuda")
        q_out = torch.empty((m, q_heads * 128), dtype=torch.float16, device="cuda")
        k_out, v_out = (torch.empty((m, kv_heads * 128), dtype=torch.float16, device="cuda") for _ in range(2))
        norms = [torch.randn(128, generator=gen, device="cuda") * 0.1 for _ in range(2)]
        cos, sin = torch.rand((m, 128), generator=gen, device="cuda"), torch.rand((m, 128), generator=gen, device="cuda")
        fn = lambda: ops.gemm_i8_rope_256(m, a, w, ws, a_scale, c, norms[0], norms[1], cos, sin, q_out, k_out, v_out, k, pitch, n,
                                          q_heads, kv_heads)
    elif name == "gemm_i8_swiglu_256":
        c = torch.empty((m, n // 2), dtype=torch.float16, device="cuda")
        fn = lambda: ops.gemm_i8_swiglu_256(m, a, w, ws, a_scale, c, k, pitch, n)
    elif name == "gemm_i8_swiglu_rotated_256":
        c = torch.empty((m, n // 2), dtype=torch.float16, device="cuda")
        fn = lambda: ops.gemm_i8_swiglu_rotated_256(m, a, w, ws, a_scale, c, k, pitch, n)
    elif name == "gemm_i8_resid_256":
        c = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
        fn = lambda: ops.gemm_i8_resid_256(m, a, w, ws, a_scale, c, gate, k, pitch, n)
    elif name == "gemm_i8_resid_256x256":
        c = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
        fn = lambda: ops.gemm_i8_resid_256x256(m, a, w, ws, a_scale, c, gate, k, pitch, n, 4,
                                               int(shape.gemm_schedule_rows(m)))
    else:
        c = torch.empty((m, n), dtype=torch.int32, device="cuda")
        fn = lambda: ops.gemm_i8_acc(m, a, w, c, k, pitch, n)
    ms = time_launches(fn, iters, warmup, flush)
    gop = 2.0 * m * n * k / 1e9
    return {"kernel": name, "stem": kind, "m": m, "k": k, "n": n, "k_stride": pitch, "ms": ms, "gop": gop,
            "tops": gop / ms}


def run_prologue(kind, m, dims, iters, warmup, flush):
    h, qkv, inter = dims["hidden"], dims["qkv"], dims["inter"]
    gen = torch.Generator(device="cuda").manual_seed(m)
    if kind == "norm":
        width = h
        x = torch.randn((m, width), generator=gen, device="cuda").to(torch.bfloat16)
        vec = [torch.randn(width, generator=gen, device="cuda") * 0.1 for _ in range(3)]
        bytes_in = 2 * width
    elif kind == "gated":
        width = h
        x = torch.randn((m, width), generator=gen, device="cuda").to(torch.float16)
        gate_stride = qkv if qkv % 256 == 0 and qkv >= 2 * width else width
        gate = torch.randn((m, gate_stride), generator=gen, device="cuda").to(torch.float16)
        bytes_in = 4 * width
    else:
        width = inter
        x = torch.randn((m, width), generator=gen, device="cuda").to(torch.float16)
        bytes_in = 2 * width
    pitch = shape.gemm_pitch(width)
    q = torch.zeros((m, pitch), dtype=torch.int8, device="cuda")
    qs = torch.zeros(m, dtype=torch.float32, device="cuda")
    if kind == "norm":
        fn = lambda: ops.prepare_norm_i8(x, vec[0], vec[1], vec[2], q, qs, width, pitch, 1e-5)
    elif kind == "rotated":
        fn = lambda: ops.prepare_rotated_i8(x, q, qs, width, pitch)
    elif kind == "gated":
        offset = gate_stride - width
        view = gate.view(-1)[offset:]
        fn = lambda: ops.prepare_gated_i8(x, view, q, qs, width, pitch, gate_stride, tokens=m)
    else:
        fn = lambda: ops.prepare_plain_i8(x, q, qs, width, pitch)
    ms = time_launches(fn, iters, warmup, flush)
    nbytes = m * (bytes_in + width + 4)
    return {"kernel": f"prepare_{kind}_i8", "m": m, "width": width, "out_stride": pitch, "ms": ms,
            "algorithmic_mb": nbytes / 1e6, "gbs": nbytes / ms / 1e6}


def run_attention(kind, m, dims, iters, warmup, flush):
    """The non-W8A8 launches of a block: `rope` (QK-norm + RoPE), `vt` (V transpose), `attention`."""
    h, qkv = dims["hidden"], dims["qkv"]
    q_heads = h // 128
    kv_heads = max(1, (qkv - 2 * h) // 256) if qkv > 2 * h else q_heads  # q|k|v|gate, else q|k|v with equal heads
    if qkv == 3 * h:
        kv_heads = q_heads
    kv_width = kv_heads * 128
    cap = shape.capacity(m)
    gen = torch.Generator(device="cuda").manual_seed(m)
    q = torch.randn((m, h), generator=gen, device="cuda").to(torch.float16)
    k = torch.randn((m, kv_width), generator=gen, device="cuda").to(torch.float16)
    v = torch.randn((m, kv_width), generator=gen, device="cuda").to(torch.float16)
    vt = torch.zeros((kv_width, cap), dtype=torch.float16, device="cuda")
    out = torch.zeros((m, h), dtype=torch.float16, device="cuda")
    if kind == "rope":
        fused = torch.randn((m, qkv), generator=gen, device="cuda").to(torch.float16)
        scale = [torch.randn(128, generator=gen, device="cuda") * 0.1 for _ in range(2)]
        cos, sin = torch.rand((m, 128), generator=gen, device="cuda"), torch.rand((m, 128), generator=gen, device="cuda")
        fn = lambda: ops.rope_qknorm_f16(fused, scale[0], scale[1], cos, sin, q, k, v, qkv, q_heads, kv_heads, h, 1e-5)
        ms = time_launches(fn, iters, warmup, flush)
        nbytes = m * (h + 2 * kv_width) * 4
        return {"kernel": "rope_qknorm_f16", "m": m, "ms": ms, "algorithmic_mb": nbytes / 1e6, "gbs": nbytes / ms / 1e6}
    if kind == "vt":
        fn = lambda: ops.v_transpose(v, vt, kv_width, cap)
        ms = time_launches(fn, iters, warmup, flush)
        nbytes = m * kv_width * 4
        return {"kernel": "v_transpose", "m": m, "ms": ms, "algorithmic_mb": nbytes / 1e6, "gbs": nbytes / ms / 1e6}
    ops.v_transpose(v, vt, kv_width, cap)
    fn = lambda: ops.attention_gqa(m, kv_heads, q, k, vt, out, h, kv_width, h, cap, 0.08838834764831845)
    ms = time_launches(fn, iters, warmup, flush)
    gflop = 4.0 * m * m * 128 * q_heads / 1e9
    return {"kernel": "attention_gqa_lds_f16_wmma", "m": m, "q_heads": q_heads, "kv_heads": kv_heads, "ms": ms,
            "gflop": gflop, "tflops": gflop / ms}


def run_sampler(kind, m, dims, iters, warmup, flush):
    """The pointwise kernels around the chain: `euler` and `guidance` over m x hidden bf16 elements (inputs
    larger than L2 at the default m), `modulation` over the [28][6][hidden] tables."""
    h = dims["hidden"]
    gen = torch.Generator(device="cuda").manual_seed(m)
    if kind == "modulation":
        count = 28 * 6 * h
        vector = torch.randn(6 * h, generator=gen, device="cuda").to(torch.bfloat16)
        tables = torch.randn(count, generator=gen, device="cuda").to(torch.bfloat16)
        out = torch.empty(count, dtype=torch.float32, device="cuda")
        ms = time_launches(lambda: ops.modulation(vector, tables, out), iters, warmup, flush)
        nbytes = count * 6
    else:
        count = m * h
        a = torch.randn(count, generator=gen, device="cuda").to(torch.bfloat16)
        b = torch.randn(count, generator=gen, device="cuda").to(torch.bfloat16)
        fn = (lambda: ops.euler_step(a, b, -0.1234)) if kind == "euler" else (lambda: ops.guidance(a, b, 3.5))
        ms = time_launches(fn, iters, warmup, flush)
        nbytes = count * 6  # two bf16 reads and one bf16 write per element
    return {"kernel": kind, "elements": count, "ms": ms, "algorithmic_mb": nbytes / 1e6, "gbs": nbytes / ms / 1e6}


def run_library(kind, m, dims, iters, warmup, flush):
    """Calibration, not a product path: the vendor library's int8 GEMM (`torch._int_mm`, raw i32 output, no
    epilogue) on the q|k|v|gate shape beside this library's fused kernel, each as a short burst and as a
    3-second back-to-back loop under the power cap."""
    import time
    h, n = dims["hidden"], dims["qkv"]
    gen = torch.Generator(device="cuda").manual_seed(m)
    a = torch.randint(-127, 128, (m, h), generator=gen, device="cuda", dtype=torch.int8)
    w = torch.randint(-127, 128, (n, h), generator=gen, device="cuda", dtype=torch.int8)
    ws = torch.rand(n, generator=gen, device="cuda") * 1e-2
    a_s = torch.rand(m, generator=gen, device="cuda") * 1e-2
    c = torch.empty((m, n), dtype=torch.float16, device="cuda")
    calls = {"library": lambda: torch._int_mm(a, w.t()), "fused": lambda: ops.gemm_i8_256(m, a, w, ws, a_s, c, h, h, n)}
    out = {"kernel": "int8 GEMM calibration", "m": m, "n": n, "k": h}
    bursts = {name: burst_time(fn, iters, warmup, flush) for name, fn in calls.items()}  # before the long loops heat the part
    for name, fn in calls.items():
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches, began = 0, time.time()
        start.record()
        while time.time() - began < 3.0:
            for _ in range(50):
                fn()
            launches += 50
            torch.cuda.synchronize()
        end.record()
        torch.cuda.synchronize()
        sustained = start.elapsed_time(end) / launches
        out[name] = {"burst_tops": 2.0 * m * n * h / bursts[name] / 1e9, "sustained_tops": 2.0 * m * n * h / sustained / 1e9}
    return out


def run_energy(kind, m, dims, iters, warmup, flush):
    """What limits the GEMM's sustained rate: the same q|k|v|gate launch back to back for 2.5 s with all-zero
    operands (no bit toggles in the operand paths and multipliers), with uniform int8 codes and with
    Gaussian-shaped codes, sampling board power and SM clock beside each.  Zero operands hold the full clock;
    random ones sit at the power cap at a lower clock."""
    h, n = dims["hidden"], dims["qkv"]
    gen = torch.Generator(device="cuda").manual_seed(m)
    ws = torch.rand(n, generator=gen, device="cuda") * 1e-2
    a_s = torch.rand(m, generator=gen, device="cuda") * 1e-2
    c = torch.empty((m, n), dtype=torch.float16, device="cuda")
    fills = {
        "zero": lambda shape_: torch.zeros(shape_, dtype=torch.int8, device="cuda"),
        "uniform": lambda shape_: torch.randint(-127, 128, shape_, generator=gen, device="cuda", dtype=torch.int8),
        "gaussian": lambda shape_: (torch.randn(shape_, generator=gen, device="cuda") * 30).clamp(-127, 127).to(torch.int8),
    }
    out = {"kernel": "gemm_i8_256 energy by operand values", "m": m, "n": n, "k": h}
    for name, fill in fills.items():
        a, w = fill((m, h)), fill((n, h))
        fn = lambda: ops.gemm_i8_256(m, a, w, ws, a_s, c, h, h, n)
        burst = burst_time(fn, iters, warmup, flush)
        sustained = sustained_run(fn, 2.5)
        gop = 2.0 * m * n * h / 1e9
        out[name] = {"burst_tops": gop / burst, "sustained_tops": gop / sustained["sustained_ms"], **sustained}
    return out


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--kernel", default="all",
                        help="qkvg, wo, gu, gurot, down, acc, norm, gated, plain, rotated, rope, vt, attention, euler, guidance, modulation, calibration, "
                             "energy, gemms, prologues or all "
                             "(comma separated)")
    parser.add_argument("--m", default="4608", help="rows, comma separated; 'reference' = the reference's bench list")
    parser.add_argument("--dims", default="reference", choices=sorted(DIMS))
    parser.add_argument("--iters", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--flush-l2", action="store_true")
    parser.add_argument("--sustain", type=float, default=0.0,
                        help="seconds of back-to-back launches per kernel with power and clock sampling")
    args = parser.parse_args()
    global SUSTAIN_SECONDS
    SUSTAIN_SECONDS = args.sustain
    kinds = []
    for item in args.kernel.split(","):
        kinds += {"all": ["qkvg", "wo", "gu", "down", "norm", "gated", "plain"], "gemms": ["qkvg", "wo", "gu", "down"],
                  "prologues": ["norm", "gated", "plain"]}.get(item, [item])
    rows = REFERENCE_M if args.m == "reference" else [int(v) for v in args.m.split(",")]
    dims = DIMS[args.dims]
    for kind in kinds:
        for m in rows:
            runner = run_prologue if kind in ("norm", "gated", "plain", "rotated") else \
                run_energy if kind == "energy" else \
                run_attention if kind in ("rope", "vt", "attention") else \
                run_sampler if kind in ("euler", "guidance", "modulation") else \
                run_library if kind == "calibration" else run_gemm
            result = runner(kind, m, dims, args.iters, args.warmup, args.flush_l2)
            result["dims"] = args.dims
            if SUSTAIN_SECONDS > 0 and kind not in ("calibration", "energy"):
                result["sustained"] = dict(LAST_SUSTAINED)
            print(json.dumps(result), flush=True)


if __name__ == "__main__":
    main()
