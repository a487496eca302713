"""Running the block chain on several GPUs.

Three ways the path spreads over devices, none of which exists in the reference (one APU):

* data parallel over images -- one ordinary `session.Session` per device, no communication
  (`bench.py --gpus N`); nothing here is needed for it;
* column-sharded weights within one image (`TensorParallel`, below): device r holds rows
  [r*N/g, (r+1)*N/g) of every weight, runs the prologues redundantly (they are cheap), computes its
  column slab of each GEMM and lets the epilogue store every finished vector into all devices'
  copies of the output through peer-mapped pointers (`krea2_gemm_i8_sharded`).  A flag per device
  and launch, waited on by `krea2_shard_wait`, tells each device when every slab has landed.  No
  arithmetic changes, so the result is bit-identical to the single-device session.
  `TensorParallel.forward(..., collective="nccl")` is the baseline the fused path is compared with:
  the same sharded GEMMs into local buffers, then an NCCL all-gather and a local repack;
* token-sharded rows within one image (`TokenParallel`): the weights are replicated and device r runs rows
  [r*T/g, (r+1)*T/g) of the sequence through the whole block alone -- every prologue, GEMM row and query
  row belongs to one token -- so the only exchange is the keys and values of each block, which the sharded
  QK-norm + RoPE launch stores into every device's K and V tensors itself
  (`krea2_rope_qknorm_f16_sharded`; `collective="nccl"` is the all-gather baseline).  Bit-identical to the
  single-device block, attention included, at 1/15 of the column-sharded chain's bytes.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Iterator, List, Optional, Sequence, Tuple

import torch

from . import shape
from ._lib import InvalidArgument, RowShard, Shard, check, lib
from .session import ModelDims, Weights

PLAIN, RESID, SWIGLU = 0, 1, 2


def shard_columns(n: int, world: int, multiple: int) -> List[Tuple[int, int]]:
    """(first row, rows) of each device's share of a weight with `n` rows; every share is the same
    whole number of `multiple`-row units (128 for the GEMM tile; 32 interleaved rows = 16 outputs
    keep a gate|up pair together, and 128 covers that too)."""
    if world < 1 or world > 8:
        raise InvalidArgument("world must be 1..8")
    if n % (world * multiple) != 0:
        raise InvalidArgument(f"{n} rows do not split into {world} shares of whole {multiple}-row units")
    size = n // world
    return [(r * size, size) for r in range(world)]


def column_slab(full: torch.Tensor, world: int, rank: int) -> torch.Tensor:
    """Rank's contiguous copy of its column slab of a row-major [rows][width] tensor."""
    size = full.shape[1] // world
    return full[:, rank * size:(rank + 1) * size].contiguous()


def assemble_columns(full: torch.Tensor, gathered: torch.Tensor) -> None:
    """Writes all-gathered slabs [world][rows][width/world] back as the columns of `full`."""
    world, rows, size = gathered.shape
    full.view(rows, world, size).copy_(gathered.permute(1, 0, 2))


class DeviceView:
    """A raw device pointer as something torch can wrap (for slicing spans of `Weights`)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


def span_tensor(weights: Weights, name: str, dtype: torch.dtype) -> torch.Tensor:
    ptr, nbytes = weights.locate(name)
    return torch.as_tensor(DeviceView(ptr, nbytes), device="cuda").view(dtype)


@dataclass
class BlockShard:
    """One device's share of a block's weights (rows of each operand and the matching scales)."""
    qkvg_q: torch.Tensor
    qkvg_s: torch.Tensor
    wo_q: torch.Tensor
    wo_s: torch.Tensor
    gu_q: torch.Tensor
    gu_s: torch.Tensor
    down_q: torch.Tensor
    down_s: torch.Tensor
    prenorm: torch.Tensor
    postnorm: torch.Tensor


def shard_weights(weights: Weights, layers: int, world: int, rank: int) -> List[BlockShard]:
    """Slices every operand of `weights` (the full plan layout) into rank's rows."""
    d = weights.dims
    ph, pi = shape.gemm_pitch(d.hidden), shape.gemm_pitch(d.inter)
    out = []
    for i in range(layers):
        p = f"blocks.{i}"

        def rows(name, n, pitch):
            first, count = shard_columns(n, world, 128)[rank]
            q = span_tensor(weights, f"{p}.{name}.q", torch.int8).view(n, pitch)[first:first + count].clone()
            s = span_tensor(weights, f"{p}.{name}.s", torch.float32)[first:first + count].clone()
            return q, s

        qkvg = rows("qkvg", d.qkvg, ph)
        wo = rows("wo", d.hidden, ph)
        gu = rows("gu", 2 * d.inter, ph)
        down = rows("down", d.hidden, pi)
        out.append(BlockShard(*qkvg, *wo, *gu, *down,
                              span_tensor(weights, f"{p}.prenorm", torch.float32).clone(),
                              span_tensor(weights, f"{p}.postnorm", torch.float32).clone()))
    return out


class LocalFabric:
    """All "devices" are buffers on the current GPU: the single-GPU stand-in used to test the
    sharded path (every rank's launches go to one stream, in stage order)."""

    def __init__(self, world: int):
        self.world = world
        self._buffers = {}

    def allocate(self, name: str, rank: int, shape_, dtype) -> torch.Tensor:
        t = torch.zeros(shape_, dtype=dtype, device="cuda")
        self._buffers.setdefault(name, {})[rank] = t
        return t

    def pointers(self, name: str, rank: int) -> List[int]:
        return [self._buffers[name][r].data_ptr() for r in range(self.world)]

    def barrier(self) -> None:
        torch.cuda.synchronize()


class SymmetricFabric:
    """One process per GPU: buffers come from torch's symmetric memory, whose rendezvous hands every
    rank the peer-mapped address of every other rank's buffer."""

    def __init__(self, group=None):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        self._dist, self._symm = dist, symm
        self.group = group or dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self._handles = {}

    def allocate(self, name: str, rank: int, shape_, dtype) -> torch.Tensor:
        t = self._symm.empty(shape_, dtype=dtype, device=torch.device("cuda", torch.cuda.current_device()))
        handle = self._symm.rendezvous(t, self.group)
        t.zero_()
        self._handles[name] = (t, handle)
        return t

    def pointers(self, name: str, rank: int) -> List[int]:
        return [int(p) for p in self._handles[name][1].buffer_ptrs]

    def barrier(self) -> None:
        torch.cuda.synchronize()
        self._dist.barrier(self.group)
        torch.cuda.synchronize()


def require_clean_status() -> None:
    """Reads the device status word (which synchronises the device) and raises `Runtime` when a bounded wait of a
    sharded chain ran out, i.e. when the forward went on without a peer's data."""
    from ._lib import Runtime, device_status
    status = device_status()
    if status != 0:
        raise Runtime(f"device status {status}: a bounded wait of the sharded chain ran out (bit 16: a peer's data "
                      "never arrived); the result is not valid")


class TensorParallel:
    """One device's part of a column-sharded run of `layers` blocks over `tokens` rows."""

    def __init__(self, fabric, rank: int, dims: ModelDims, shards: Sequence[BlockShard], tokens: int,
                 stream: Optional[torch.cuda.Stream] = None):
        self.fabric, self.rank, self.world = fabric, rank, fabric.world
        self.dims, self.shards, self.tokens = dims, list(shards), tokens
        self.stream = stream or torch.cuda.current_stream()
        cap = shape.capacity(tokens)
        d = dims
        self.ph, self.pi = shape.gemm_pitch(d.hidden), shape.gemm_pitch(d.inter)
        wide = max(d.hidden, d.inter)
        self.x = fabric.allocate("x", rank, (cap, d.hidden), torch.bfloat16)
        self.fused = fabric.allocate("fused", rank, (cap, d.qkvg), torch.float16)
        self.attn_gu = fabric.allocate("attn_gu", rank, (cap, wide), torch.float16)
        self.flags = fabric.allocate("flags", rank, (8,), torch.int32)
        self.counter = torch.zeros(1, dtype=torch.int32, device="cuda")
        self.epoch_base = torch.zeros(1, dtype=torch.int32, device="cuda")  # advanced once per forward
        self.graphs = {}  # collective -> recorded CUDA graph
        self.a_q = torch.zeros((cap, shape.gemm_pitch(wide)), dtype=torch.int8, device="cuda")
        self.a_s = torch.zeros(cap, dtype=torch.float32, device="cuda")
        self.epoch = 0
        self.launches = 0

    # -- launches ---------------------------------------------------------------------------
    def _sharded(self, kind, w, s, gate, k, pitch, n_total, out_name, out_pitch, collective) -> None:
        first, count = shard_columns(n_total, self.world, 128)[self.rank]
        out_first = first // 2 if kind == SWIGLU else first
        desc = Shard()
        if collective == "fused":
            desc.world, desc.rank = self.world, self.rank
            for r, ptr in enumerate(self.fabric.pointers(out_name, self.rank)):
                desc.dest[r] = ptr
            for r, ptr in enumerate(self.fabric.pointers("flags", self.rank)):
                desc.flags[r] = ptr
            self.epoch += 1
            desc.epoch = self.epoch
            desc.counter = self.counter.data_ptr()
            desc.epoch_base = self.epoch_base.data_ptr()
        else:  # the slab goes to the local copy only; a collective moves it afterwards
            desc.world, desc.rank = 1, 0
            desc.dest[0] = getattr(self, out_name).data_ptr()
        desc.pitch, desc.offset = out_pitch, out_first
        # the residual gate is indexed by output column: this shard's slice of it
        gate_ptr = gate[first:first + count].data_ptr() if gate is not None else None
        check(lib().krea2_gemm_i8_sharded(self.stream.cuda_stream, kind, self.tokens, self.a_q.data_ptr(), w.data_ptr(),
                                          s.data_ptr(), self.a_s.data_ptr(), gate_ptr, k, pitch, count,
                                          ctypes.byref(desc)))
        self.launches += 1

    def _wait(self) -> None:
        check(lib().krea2_shard_wait(self.stream.cuda_stream, self.flags.data_ptr(), self.world, self.epoch,
                                     self.epoch_base.data_ptr()))

    def _gather(self, out_name: str, n_total: int, swiglu: bool) -> None:
        """The NCCL baseline: all-gather of the column slabs, then a repack into row-major."""
        import torch.distributed as dist
        width = n_total // 2 if swiglu else n_total
        t = self.tokens
        full = getattr(self, out_name).view(-1)[: t * width].view(t, width)
        gathered = torch.empty((self.world, t, width // self.world), dtype=full.dtype, device=full.device)
        dist.all_gather_into_tensor(gathered, column_slab(full, self.world, self.rank), group=self.fabric.group)
        assemble_columns(full, gathered)

    # -- the chain --------------------------------------------------------------------------
    def stages(self, mods: torch.Tensor, collective: str = "fused") -> Iterator[None]:
        """The block chain as a sequence of steps; every `yield` is a point where, on a single GPU
        standing in for several, the other ranks' launches of the same step must be issued before
        this rank goes on (in one process per GPU the generator is simply run to its end)."""
        from . import ops
        d, t, st = self.dims, self.tokens, self.stream
        h, inter, qkvg = d.hidden, d.inter, d.qkvg
        # torch's own copies and collectives between the launches must be queued on the same stream as the
        # launches: the generator holds that stream current across its yields
        with torch.cuda.stream(st):
            yield from self._stages(mods, collective, ops, d, t, st, h, inter, qkvg)

    def _stages(self, mods, collective, ops, d, t, st, h, inter, qkvg) -> Iterator[None]:

        def after_gemm(name, n_total, swiglu=False):
            if collective == "fused":
                self._wait()
            elif self.world > 1:
                self._gather(name, n_total, swiglu)

        self.epoch = 0  # epochs are relative to *epoch_base, which moves on at the end of the forward
        for i, w in enumerate(self.shards):
            m = mods[i]
            ops.prepare_norm_i8(self.x[:t], w.prenorm, m[0], m[1], self.a_q, self.a_s, h, self.ph, 1e-5, st)
            self._sharded(PLAIN, w.qkvg_q, w.qkvg_s, None, h, self.ph, qkvg, "fused", qkvg, collective)
            yield
            after_gemm("fused", qkvg)
            self.attn_gu[:t].view(-1)[: t * h].view(t, h).copy_(self.fused[:t, :h])  # attention stand-in
            attn = self.attn_gu.view(-1)[: t * h].view(t, h)
            ops.prepare_gated_i8(attn, self.fused.view(-1)[d.gate_offset:], self.a_q, self.a_s, h, self.ph, qkvg, st,
                                 tokens=t)
            self._sharded(RESID, w.wo_q, w.wo_s, m[2], h, self.ph, h, "x", h, collective)
            yield
            after_gemm("x", h)
            ops.prepare_norm_i8(self.x[:t], w.postnorm, m[3], m[4], self.a_q, self.a_s, h, self.ph, 1e-5, st)
            self._sharded(SWIGLU, w.gu_q, w.gu_s, None, h, self.ph, 2 * inter, "attn_gu", inter, collective)
            yield
            after_gemm("attn_gu", 2 * inter, swiglu=True)
            gu = self.attn_gu.view(-1)[: t * inter].view(t, inter)
            ops.prepare_plain_i8(gu, self.a_q, self.a_s, inter, self.pi, st)
            self._sharded(RESID, w.down_q, w.down_s, m[5], inter, self.pi, h, "x", h, collective)
            yield
            after_gemm("x", h)
        if collective == "fused":
            check(lib().krea2_shard_advance(st.cuda_stream, self.epoch_base.data_ptr(), self.epoch))

    def _checked(self, check_status: bool) -> None:
        if check_status:
            require_clean_status()

    def forward(self, x: torch.Tensor, mods: torch.Tensor, collective: str = "fused", check: bool = False) -> torch.Tensor:
        """x: device bf16 [tokens][hidden] (the same on every rank); returns the new residual stream.

        The waits for the peers' slabs are bounded (two seconds): when one runs out -- a peer that died, or one
        that is merely slow, e.g. still loading its module or instantiating its graph -- the device status word is
        raised and the chain CONTINUES on whatever has arrived.  The result is therefore valid only if
        `krea2_hrx_b200.device_status()` reads 0 afterwards; `check=True` reads it here (which synchronises the
        device) and raises `Runtime` otherwise."""
        with torch.cuda.stream(self.stream):
            self.x[: self.tokens].copy_(x)
        for _ in self.stages(mods, collective):
            pass
        self._checked(check)
        return self.x[: self.tokens]

    def forward_graph(self, x: torch.Tensor, mods: torch.Tensor, collective: str = "fused", check: bool = False) -> torch.Tensor:
        """The forward replayed from a CUDA graph recorded on first use (the inputs are copied into fixed buffers,
        as Session.run_device does); one graph per `collective`.  Every rank must call it the same number of times:
        the flags count forwards.  As with `forward`, the result is valid only if the device status reads 0
        afterwards (`check=True` reads it, synchronising the device)."""
        if collective not in self.graphs:
            if not hasattr(self, "_mods"):
                self._mods = mods.clone()
            capture = torch.cuda.Stream()
            capture.wait_stream(self.stream)
            saved = self.stream
            self.stream = capture
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=capture):
                for _ in self.stages(self._mods, collective):
                    pass
            self.stream = saved
            self.graphs[collective] = graph
        with torch.cuda.stream(self.stream):
            self._mods.copy_(mods)
            self.x[: self.tokens].copy_(x)
            self.graphs[collective].replay()
        self._checked(check)
        return self.x[: self.tokens]


def shard_rows(tokens: int, world: int) -> List[Tuple[int, int]]:
    """(first row, rows) of each device's share of a sequence: equal shares of ceil(tokens / world) rows, the
    last one shorter when the count does not divide."""
    if world < 1 or world > 8:
        raise InvalidArgument("world must be 1..8")
    share = -(-tokens // world)
    out = [(min(r * share, tokens), max(0, min(share, tokens - r * share))) for r in range(world)]
    if any(count < 1 for _, count in out):
        raise InvalidArgument(f"{tokens} rows do not give each of {world} devices a row")
    return out


class TokenParallel:
    """One device's rows of a token-sharded run of `layers` full blocks (attention included) over `tokens` rows.

    Cross-device ordering.  A device that has passed the wait of block i knows every peer has finished the
    attention of block i - 1 (each peer's K/V stores of block i follow that attention in its stream), so K and V
    alternate between two buffers by block parity and a device can run at most one block ahead of what its
    peers still read.  A forward ends with a flag-only signal and wait, after which the next forward may reuse
    both buffers.  The waits are bounded; as with `TensorParallel`, a result is valid only if
    `krea2_hrx_b200.device_status()` reads 0 afterwards."""

    SCALE = 0.08838834764831845  # 1 / sqrt(128), src/session/mod.rs:752

    def __init__(self, fabric, rank: int, weights: Weights, tokens: int, layers: int,
                 stream: Optional[torch.cuda.Stream] = None):
        self.fabric, self.rank, self.world = fabric, rank, fabric.world
        self.weights, self.dims, self.tokens, self.layers = weights, weights.dims, tokens, layers
        self.stream = stream or torch.cuda.current_stream()
        d = self.dims
        if d.head_dim != 128:
            raise InvalidArgument("the attention kernel is built for 128 channels per head")
        self.rows = shard_rows(tokens, self.world)[rank]
        self.share = -(-tokens // self.world)
        first, count = self.rows
        cap_local = shape.capacity(count)
        self.cap = -(-max(shape.capacity(tokens), self.world * self.share) // 64) * 64
        self.ph, self.pi = shape.gemm_pitch(d.hidden), shape.gemm_pitch(d.inter)
        self.kv_width = d.kv_heads * d.head_dim
        wide = max(d.hidden, d.inter)
        dev = torch.device("cuda", torch.cuda.current_device())
        self.x = torch.zeros((cap_local, d.hidden), dtype=torch.bfloat16, device=dev)
        self.a_q = torch.zeros((cap_local, shape.gemm_pitch(wide)), dtype=torch.int8, device=dev)
        self.a_s = torch.zeros(cap_local, dtype=torch.float32, device=dev)
        self.fused = torch.zeros((cap_local, d.qkvg), dtype=torch.float16, device=dev)
        self.attn_gu = torch.zeros((cap_local, wide), dtype=torch.float16, device=dev)
        self.q = torch.zeros((cap_local, d.hidden), dtype=torch.float16, device=dev)
        self.k_local = torch.zeros((self.share, self.kv_width), dtype=torch.float16, device=dev)
        self.v_local = torch.zeros((self.share, self.kv_width), dtype=torch.float16, device=dev)
        self.vt = torch.zeros((self.kv_width, self.cap), dtype=torch.float16, device=dev)
        self.k = [fabric.allocate(f"sp.k{b}", rank, (self.cap, self.kv_width), torch.float16) for b in range(2)]
        self.v = [fabric.allocate(f"sp.v{b}", rank, (self.cap, self.kv_width), torch.float16) for b in range(2)]
        self.flags = fabric.allocate("sp.flags", rank, (8,), torch.int32)
        self.counter = torch.zeros(1, dtype=torch.int32, device=dev)
        self.epoch_base = torch.zeros(1, dtype=torch.int32, device=dev)
        self.cos = torch.zeros((count, d.head_dim), dtype=torch.float32, device=dev)
        self.sin = torch.zeros((count, d.head_dim), dtype=torch.float32, device=dev)
        self.mods = torch.zeros((layers, 6, d.hidden), dtype=torch.float32, device=dev)
        self.epoch = 0
        self.graphs = {}
        self.blocks = []
        for i in range(layers):
            p = f"blocks.{i}"
            block = {name: span_tensor(weights, f"{p}.{name}", torch.int8 if name.endswith(".q") else torch.float32)
                     for name in ("qkvg.q", "qkvg.s", "wo.q", "wo.s", "gu.q", "gu.s", "down.q", "down.s", "prenorm",
                                  "postnorm", "qnorm", "knorm")}
            self.blocks.append(block)

    def _shard(self, parity: Optional[int]) -> RowShard:
        desc = RowShard()
        desc.world, desc.rank, desc.first_row = self.world, self.rank, self.rows[0]
        if parity is not None:
            for r, ptr in enumerate(self.fabric.pointers(f"sp.k{parity}", self.rank)):
                desc.k_dest[r] = ptr
            for r, ptr in enumerate(self.fabric.pointers(f"sp.v{parity}", self.rank)):
                desc.v_dest[r] = ptr
        for r, ptr in enumerate(self.fabric.pointers("sp.flags", self.rank)):
            desc.flags[r] = ptr
        self.epoch += 1
        desc.epoch = self.epoch
        desc.counter = self.counter.data_ptr()
        desc.epoch_base = self.epoch_base.data_ptr()
        return desc

    def _wait(self) -> None:
        check(lib().krea2_shard_wait(self.stream.cuda_stream, self.flags.data_ptr(), self.world, self.epoch,
                                     self.epoch_base.data_ptr()))

    def stages(self, collective: str = "push") -> Iterator[None]:
        """The block chain on this device's rows; every `yield` is a point where, on a single GPU standing in for
        several, the other ranks' launches of the same step must be queued before this rank waits for them."""
        with torch.cuda.stream(self.stream):
            yield from self._stages(collective)

    def _stages(self, collective: str) -> Iterator[None]:
        from . import ops
        d, st, t = self.dims, self.stream, self.tokens
        first, count = self.rows
        h, inter, qkvg, kvw = d.hidden, d.inter, d.qkvg, self.kv_width
        q_heads = h // d.head_dim
        x, attn = self.x[:count], self.attn_gu.view(-1)[: count * h].view(count, h)
        gu = self.attn_gu.view(-1)[: count * inter].view(count, inter)
        self.epoch = 0
        for i, w in enumerate(self.blocks):
            m, b = self.mods[i], i % 2
            ops.prepare_norm_i8(x, w["prenorm"], m[0], m[1], self.a_q, self.a_s, h, self.ph, 1e-5, st)
            ops.gemm_i8_256(count, self.a_q, w["qkvg.q"], w["qkvg.s"], self.a_s, self.fused, h, self.ph, qkvg, stream=st)
            if collective == "push":
                ops.rope_qknorm_f16_sharded(count, self.fused, w["qnorm"], w["knorm"], self.cos, self.sin, self.q, qkvg,
                                            q_heads, d.kv_heads, h, self._shard(b), stream=st)
                yield
                self._wait()
            else:
                import torch.distributed as dist
                ops.rope_qknorm_f16(self.fused, w["qnorm"], w["knorm"], self.cos, self.sin, self.q, self.k_local,
                                    self.v_local, qkvg, q_heads, d.kv_heads, h, stream=st, tokens=count)
                rows = self.world * self.share
                dist.all_gather_into_tensor(self.k[b][:rows], self.k_local, group=self.fabric.group)
                dist.all_gather_into_tensor(self.v[b][:rows], self.v_local, group=self.fabric.group)
            ops.v_transpose(self.v[b], self.vt, kvw, self.cap, st, rows=t)
            ops.attention_gqa_rows(count, t, d.kv_heads, self.q, self.k[b], self.vt, attn, h, kvw, h, self.cap, self.SCALE, st)
            ops.prepare_gated_i8(attn, self.fused.view(-1)[d.gate_offset:], self.a_q, self.a_s, h, self.ph, qkvg, st,
                                 tokens=count)
            ops.gemm_i8_resid_256(count, self.a_q, w["wo.q"], w["wo.s"], self.a_s, x, m[2], h, self.ph, h, stream=st)
            ops.prepare_norm_i8(x, w["postnorm"], m[3], m[4], self.a_q, self.a_s, h, self.ph, 1e-5, st)
            ops.gemm_i8_swiglu_256(count, self.a_q, w["gu.q"], w["gu.s"], self.a_s, gu, h, self.ph, 2 * inter, stream=st)
            ops.prepare_plain_i8(gu, self.a_q, self.a_s, inter, self.pi, st)
            ops.gemm_i8_resid_256x256(count, self.a_q, w["down.q"], w["down.s"], self.a_s, x, m[5], inter, self.pi, h,
                                      schedule_rows=shape.gemm_schedule_rows(count), stream=st)
        if collective == "push":
            ops.shard_signal(self._shard(None), st)  # no peer still reads K or V once every device has signalled
            yield
            self._wait()
            check(lib().krea2_shard_advance(st.cuda_stream, self.epoch_base.data_ptr(), self.epoch))

    def load(self, x: torch.Tensor, mods: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> None:
        """Copies this device's rows of x (device bf16 [tokens][hidden]) and of the HOST or device RoPE tables, and
        the modulation tables, into the fixed buffers."""
        first, count = self.rows
        with torch.cuda.stream(self.stream):
            self.x[:count].copy_(x[first:first + count], non_blocking=True)
            self.mods.copy_(mods, non_blocking=True)
            self.cos.copy_(cos.view(self.tokens, -1)[first:first + count], non_blocking=True)
            self.sin.copy_(sin.view(self.tokens, -1)[first:first + count], non_blocking=True)

    def forward(self, x: torch.Tensor, mods: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, collective: str = "push",
                graph: bool = False, check: bool = False) -> torch.Tensor:
        """Returns this device's rows of the new residual stream (`self.rows`).  With `graph` the chain is replayed
        from a CUDA graph recorded on first use (one per `collective`); every rank must then call it the same
        number of times, since the flags count forwards."""
        self.load(x, mods, cos, sin)
        return self.replay(collective, graph, check)

    def replay(self, collective: str = "push", graph: bool = False, check: bool = False) -> torch.Tensor:
        """The chain on what the fixed buffers hold (`self.x[:count]`, `self.mods`, `self.cos`, `self.sin`): for a
        caller that fills them itself, as the denoising loop does between steps."""
        if graph:
            if collective not in self.graphs:
                capture = torch.cuda.Stream()
                capture.wait_stream(self.stream)
                saved, self.stream = self.stream, capture
                recorded = torch.cuda.CUDAGraph()
                with torch.cuda.graph(recorded, stream=capture):
                    for _ in self.stages(collective):
                        pass
                self.stream = saved
                self.graphs[collective] = recorded
            with torch.cuda.stream(self.stream):
                self.graphs[collective].replay()
        else:
            for _ in self.stages(collective):
                pass
        if check:
            require_clean_status()
        return self.x[: self.rows[1]]


def run_emulated_rows(ranks: Sequence[TokenParallel], x, mods, cos, sin) -> List[torch.Tensor]:
    """Drives every rank of a token-sharded `LocalFabric` run on one GPU, step by step."""
    for r in ranks:
        r.load(x, mods, cos, sin)
    generators = [r.stages("push") for r in ranks]
    while True:
        finished = 0
        for g in generators:
            try:
                next(g)
            except StopIteration:
                finished += 1
        if finished == len(generators):
            break
    return [r.x[: r.rows[1]] for r in ranks]


def run_emulated(ranks: Sequence[TensorParallel], x: torch.Tensor, mods: torch.Tensor) -> List[torch.Tensor]:
    """Drives every rank of a `LocalFabric` on one GPU, step by step, so that each step's launches
    of all ranks are queued before anything waits for them."""
    for r in ranks:
        r.x[: r.tokens].copy_(x)
    generators = [r.stages(mods, "fused") for r in ranks]
    while True:
        finished = 0
        for g in generators:
            try:
                next(g)
            except StopIteration:
                finished += 1
        if finished == len(generators):
            break
    return [r.x[: r.tokens] for r in ranks]
