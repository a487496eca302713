"""krea2::kernels (src/kernels/mod.rs, blocks.rs): Config, Scalars, grid and the per-sequence
kernel list.  The reference compiles a specialization per shape at run time; here every shape is
served by the ahead-of-time library, so `Shape.jobs()` is the same table with nothing to build."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Tuple

from . import shape
from ._lib import Internal, InvalidArgument

Config = Dict[str, object]  # kernels::Config: config key -> value (ints, and eps as a float)


def config(entries) -> Config:
    """kernels::config([("tokens", 4115), ...])."""
    return dict(entries)


def grid(stage: str, x: int, y: int) -> Tuple[int, int, int]:
    """kernels::grid (mod.rs:77-84): refuses counts that do not fit a u32."""
    for count in (x, y):
        if count < 0 or count > 0xFFFFFFFF:
            raise Internal(f"{stage}: {count} workgroups exceed the grid")
    return (x, y, 1)


BLOCK_SIZES = {"prepare_norm_i8": 256, "prepare_gated_i8": 256, "prepare_plain_i8": 256, "gemm_i8_256": 256,
               "gemm_i8_resid_256": 256, "gemm_i8_swiglu_256": 256, "gemm_i8_resid_256x256": 512,
               "lora_transport": 256}


def workgroup(stage: str, kernel: str, threads: int) -> Tuple[int, int, int]:
    """kernels::workgroup (mod.rs:91-98): the block a kernel is built for, checked against the host's."""
    compiled = BLOCK_SIZES.get(kernel)
    if compiled != threads:
        raise Internal(f"{stage}: compiled for workgroup [{compiled}, 1, 1] but the host asked for {threads}")
    return (threads, 1, 1)


@dataclass
class Scalars:
    """kernels::Scalars (mod.rs:106-166): up to four indices, then up to eight floats."""
    indices: List[int] = field(default_factory=list)
    floats: List[float] = field(default_factory=list)

    def index(self, value: int) -> "Scalars":
        assert len(self.indices) < 4, "a kernel takes at most four indices"
        return Scalars(self.indices + [int(value)], list(self.floats))

    def float(self, value: float) -> "Scalars":
        assert len(self.floats) < 8, "a kernel takes at most eight floats"
        return Scalars(list(self.indices), self.floats + [float(value)])


@dataclass(frozen=True)
class Job:
    source: str
    stem: str
    config: Dict[str, str]


@dataclass(frozen=True)
class Shape:
    """kernels::Shape (blocks.rs:17-36)."""
    tokens: int
    capacity: int

    @staticmethod
    def new(tokens: int) -> "Shape":
        allowed = shape.tokens_range()
        if tokens not in allowed:
            raise InvalidArgument(f"tokens must be {allowed.start}..{allowed.stop - 1}")
        return Shape(tokens, shape.capacity(tokens))

    def jobs(self, hidden: int = 6144, inter: int = 16384, qkvg: int = 15360) -> List[Job]:
        """The W8A8 rows of blocks.rs:38-107 (the rope and attention jobs are outside this path)."""
        pitch_hidden, pitch_inter = str(shape.gemm_pitch(hidden)), str(shape.gemm_pitch(inter))
        group = str(shape.gemm_m_group())

        def gemm(family, stem, k, stride, n):
            tile = shape.gemm_tile(stem)
            cfg = {"k_size": k, "k_stride": stride, "n_size": n, "m_group": group}
            if tile is shape.GemmTile.Wide:
                cfg["schedule_rows"] = str(int(shape.gemm_schedule_rows(self.tokens)))
            return Job(shape.gemm_source(family, tile), stem, cfg)

        return [
            Job("prepare_norm_i8", "prepare_norm_i8", {"width": str(hidden), "out_stride": pitch_hidden, "eps": "1e-5"}),
            Job("prepare_gated_i8", "prepare_gated_i8",
                {"width": str(hidden), "out_stride": pitch_hidden, "gate_stride": str(qkvg)}),
            Job("prepare_plain_i8", "prepare_plain_i8", {"width": str(inter), "out_stride": pitch_inter}),
            gemm("gemm_i8_256", "gemm_qkvg", str(hidden), pitch_hidden, str(qkvg)),
            gemm("gemm_i8_swiglu_256", "gemm_gu", str(hidden), pitch_hidden, str(2 * inter)),
            gemm("gemm_i8_resid_256", "gemm_wo", str(hidden), pitch_hidden, str(hidden)),
            gemm("gemm_i8_resid_256", "gemm_down", str(inter), pitch_inter, str(hidden)),
        ]
