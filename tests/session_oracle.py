"""The session's block chain restated on the CPU oracle (src/session/mod.rs:671-840), used by
the GPU session tests and by the smoke check to verify a resident session end to end."""
from __future__ import annotations

import numpy as np
import torch

import oracle

SMALL = dict(hidden=2048, kv_heads=2, head_dim=128, inter=4096)


def host_weights(weights, layers):
    """Reads every span the chain uses back from the device, at its device pitch."""
    d = weights.dims
    out = []
    for i in range(layers):
        p = f"blocks.{i}"
        block = {}
        for name, dtype in [("qkvg.q", torch.int8), ("wo.q", torch.int8), ("gu.q", torch.int8), ("down.q", torch.int8),
                            ("qkvg.s", torch.float32), ("wo.s", torch.float32), ("gu.s", torch.float32),
                            ("down.s", torch.float32), ("prenorm", torch.float32), ("postnorm", torch.float32),
                            ("qnorm", torch.float32), ("knorm", torch.float32)]:
            block[name] = weights.read(f"{p}.{name}", dtype).numpy()
        out.append(block)
    return out


def oracle_forward(dims, blocks, x_bits, mods, first=0, count=None, attention=False, cos=None, sin=None):
    """x_bits: bf16 bits [tokens][hidden]; mods f32 [layers][6][hidden].  Returns the new x bits
    and the intermediates of the last block.  With `attention` the three launches between the
    q|k|v|gate GEMM and the gated prologue are the oracle's RoPE (exact) and float64 attention
    (a tolerance reference) or, when `attention` is a function, whatever it returns for (q, k, v,
    q_heads, kv_heads); without, the query columns take the attention output's place, as in a
    session whose attention is switched off, which keeps the whole chain bit-exact."""
    from krea2_hrx_b200 import shape
    hidden, inter = dims.hidden, dims.inter
    qkvg, gate_offset = dims.qkvg, dims.gate_offset
    ph, pi = shape.gemm_pitch(hidden), shape.gemm_pitch(inter)
    x = np.array(x_bits, dtype=np.uint16, copy=True)
    tokens = x.shape[0]
    count = len(blocks) - first if count is None else count
    trace = {}
    for index in range(first, first + count):
        w, m = blocks[index], mods[index]
        a_q, a_s = oracle.prepare_norm_i8(x, w["prenorm"], m[0], m[1], hidden, ph)
        fused = oracle.gemm_i8_256(a_q, w["qkvg.q"].reshape(qkvg, ph), w["qkvg.s"], a_s, hidden, ph, qkvg)
        if attention:
            q_heads = hidden // dims.head_dim
            q, k, v = oracle.rope_qknorm_f16(fused, w["qnorm"], w["knorm"], cos, sin, qkvg, q_heads, dims.kv_heads, hidden)
            if callable(attention):  # e.g. the GPU attention kernel on the oracle's own q, k, v
                attn = attention(q, k, v, q_heads, dims.kv_heads)
            else:
                attn = oracle.f32_to_f16_bits(oracle.attention_gqa(q, k, v, q_heads, dims.kv_heads,
                                                                  0.08838834764831845).astype(np.float32))
            trace_qkv = (q, k, v)
        else:
            attn = np.ascontiguousarray(fused[:, :hidden])  # a copy of the q columns
            trace_qkv = None
        # the gate view starts gate_offset columns into the fused rows, pitch qkvg
        flat = fused.reshape(-1)
        view = np.zeros(tokens * qkvg, dtype=np.uint16)
        view[:flat.size - gate_offset] = flat[gate_offset:]
        a_q, a_s = oracle.prepare_gated_i8(attn, view.reshape(tokens, qkvg), hidden, ph, qkvg)
        x = oracle.gemm_i8_resid_256(a_q, w["wo.q"].reshape(hidden, ph), w["wo.s"], a_s, x, m[2], hidden, ph, hidden)
        a_q, a_s = oracle.prepare_norm_i8(x, w["postnorm"], m[3], m[4], hidden, ph)
        gu = oracle.gemm_i8_swiglu_256(a_q, w["gu.q"].reshape(2 * inter, ph), w["gu.s"], a_s, hidden, ph, 2 * inter)
        a_q, a_s = oracle.prepare_plain_i8(gu, inter, pi)
        x = oracle.gemm_i8_resid_256(a_q, w["down.q"].reshape(hidden, pi), w["down.s"], a_s, x, m[5], inter, pi, hidden)
        trace = dict(fused=fused, gu=gu, a_q=a_q, a_s=a_s, qkv=trace_qkv)
    return x, trace


def make_inputs(dims, tokens, layers, seed=0):
    rng = np.random.default_rng(seed)
    x = oracle.f32_to_bf16_bits(rng.standard_normal((tokens, dims.hidden)).astype(np.float32))
    mods = (rng.standard_normal((layers, 6, dims.hidden)) * 0.5).astype(np.float32)
    mods[:, [2, 5]] *= 0.2
    cos = np.cos(rng.uniform(0, 6.28, (tokens, dims.head_dim))).astype(np.float32)
    sin = np.sin(rng.uniform(0, 6.28, (tokens, dims.head_dim))).astype(np.float32)
    return x, mods, cos, sin


def check_session(tokens=48, layers=2, seed=1):
    """Builds a small session over synthetic weights, runs it from host buffers and checks the
    residual stream against the oracle chain bit for bit."""
    from krea2_hrx_b200 import session
    dims = session.ModelDims(**SMALL)
    stream = torch.cuda.current_stream()
    weights = session.Weights(dims, layers)
    weights.fill_synthetic(seed, stream)
    s = session.Session(stream, weights, tokens, layers)
    x, mods, cos, sin = make_inputs(dims, tokens, layers, seed)
    host = host_weights(weights, layers)
    # the W8A8 chain alone: bit for bit
    s.set_attention(False)
    x_t = torch.from_numpy(x.copy()).view(torch.bfloat16)
    s.run(stream, x_t, torch.from_numpy(mods), torch.from_numpy(cos), torch.from_numpy(sin))
    want, _ = oracle_forward(dims, host, x, mods)
    got = x_t.view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(got, want), f"session output differs in {(got != want).sum()} of {got.size} elements"
    # the full block, with attention: within tolerance of the float64 attention chain
    s.set_attention(True)
    x_t = torch.from_numpy(x.copy()).view(torch.bfloat16)
    s.run(stream, x_t, torch.from_numpy(mods), torch.from_numpy(cos), torch.from_numpy(sin))
    want, _ = oracle_forward(dims, host, x, mods, attention=gpu_attention(tokens), cos=cos, sin=sin)
    got = x_t.view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(got, want), "full-block session differs from the oracle chain around the attention kernel"
    s.close()
    return True


def gpu_attention(tokens):
    """The library's own attention kernel as a stage of the oracle chain: the kernel is
    deterministic, so a session forward must equal the oracle chain with this in attention's place
    bit for bit (its accuracy against float64 is a separate, tolerance test)."""
    from krea2_hrx_b200 import ops, shape

    def run(q, k, v, q_heads, kv_heads):
        capacity = shape.capacity(tokens)
        width = kv_heads * 128
        v_dev = torch.from_numpy(v.view(np.int16)).view(torch.float16).cuda()
        vt = torch.zeros((width, capacity), dtype=torch.float16, device="cuda")
        ops.v_transpose(v_dev, vt, width, capacity)
        out = torch.zeros((tokens, q_heads * 128), dtype=torch.float16, device="cuda")
        ops.attention_gqa(tokens, kv_heads, torch.from_numpy(q.view(np.int16)).view(torch.float16).cuda(),
                          torch.from_numpy(k.view(np.int16)).view(torch.float16).cuda(), vt, out, q_heads * 128, width,
                          q_heads * 128, capacity, 0.08838834764831845)
        torch.cuda.synchronize()
        return out.view(torch.int16).cpu().numpy().view(np.uint16)
    return run


def relative_l2(got_bits, want_bits):
    got = oracle.bf16_bits_to_f32(got_bits).astype(np.float64)
    want = oracle.bf16_bits_to_f32(want_bits).astype(np.float64)
    return float(np.linalg.norm(got - want) / np.linalg.norm(want))
