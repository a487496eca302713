"""krea2::kernels::shape (src/kernels/shape.rs): the launch-shape rules, answered by the library."""
from __future__ import annotations

import enum

from ._lib import lib

GEMM_ROWS = 256  # shape.rs:36


def tokens_range() -> range:
    """shape::TOKENS, inclusive on both ends."""
    return range(lib().krea2_shape_tokens_min(), lib().krea2_shape_tokens_max() + 1)


def capacity(tokens: int) -> int:
    return lib().krea2_shape_capacity(tokens)


def attention_rows(tokens: int) -> int:
    return lib().krea2_shape_attention_rows(tokens)


class GemmTile(enum.Enum):
    """shape.rs:43-65."""
    Narrow = "narrow"
    Wide = "wide"

    def columns(self) -> int:
        return 128 if self is GemmTile.Narrow else 256

    def threads(self) -> int:
        return 256 if self is GemmTile.Narrow else 512


def gemm_tile(stem: str) -> GemmTile:
    return GemmTile.Wide if lib().krea2_shape_gemm_tile_columns(stem.encode()) == 256 else GemmTile.Narrow


def gemm_source(family: str, tile: GemmTile) -> str:
    stem = b"gemm_down" if tile is GemmTile.Wide else b"gemm_wo"
    return lib().krea2_shape_gemm_source(family.encode(), stem).decode()


def gemm_m_group() -> int:
    return lib().krea2_shape_gemm_m_group()


def gemm_schedule_rows(tokens: int) -> bool:
    return bool(lib().krea2_shape_gemm_schedule_rows(tokens))


def gemm_pitch(k: int) -> int:
    return lib().krea2_shape_gemm_pitch(k)


def gemm_grid_rows(tokens: int) -> int:
    return lib().krea2_shape_gemm_grid_rows(tokens)
