"""The sampler's sigma schedule (src/pipeline/schedule.rs), evaluated by the library's C entry points.

Turbo (the distilled checkpoint) uses the fixed shift `mu = 1.15`; Raw computes it from the image's
token count with `dynamic_mu`.
"""
from __future__ import annotations

from ._lib import lib

TURBO_MU = 1.15


def dynamic_mu(image_tokens: int) -> float:
    """Linear between 256 tokens at 0.5 and 6400 tokens at 1.15 (schedule.rs:11-14)."""
    return float(lib().krea2_schedule_dynamic_mu(image_tokens))


def sigma(step: int, steps: int, mu: float) -> float:
    """The sigma at `step` of `steps`; the last one is zero (schedule.rs:17-27)."""
    return float(lib().krea2_schedule_sigma(step, steps, mu))


def next_sigma(step: int, last: int, steps: int, mu: float) -> float:
    """Where `step` lands when the run ends after step `last` of `steps` (schedule.rs:33-35)."""
    return float(lib().krea2_schedule_next_sigma(step, last, steps, mu))
