"""The denoising loop of `Pipeline::generate` (src/pipeline/mod.rs:336-366) around one resident session.

Per step the reference does: `schedule::sigma` / `next_sigma`; `step_inputs` (time embedding, image
projection, `Models::modulation`); `forward` (text and image tokens through the 28 blocks, then the final
layer), twice and combined by `ops.guidance` when guidance is on; `ops.euler_step`.  The time, text, image
and final-layer models are bf16 networks outside the W8A8 path, so this helper takes what they produce as
inputs and keeps the rest of the loop as it is:

* `vectors[step]`: the time model's modulation vector for that step (bf16 `[6 * hidden]`), which
  `ops.modulation` adds to the per-block tables exactly as `Models::modulation` does
  (src/models/graph.rs:405-425);
* the sample is the image tokens in the transformer's width (bf16 `[image_tokens][hidden]`: the latents after
  the image projection), the text tokens a constant bf16 `[text_tokens][hidden]`;
* the velocity is the image rows of the session's output (what the final layer would project back).

A step copies `[text; image]` into the session, replays its graph, and copies the image rows back, as
`run_blocks` does (src/pipeline/shared.rs:80-150).
"""
from __future__ import annotations

from typing import Callable, Optional, Sequence

import numpy as np
import torch

from . import ops, schedule
from ._lib import Cancelled, InvalidArgument
from .session import Session

CONTINUE, FINISH, CANCEL = "continue", "finish", "cancel"  # pipeline::Control


class Denoiser:
    """One image's loop state: the session, the blocks' modulation tables and the schedule."""

    def __init__(self, session: Session, tables: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, text: torch.Tensor,
                 steps: int = 8, mu: Optional[float] = schedule.TURBO_MU, guidance: float = 0.0,
                 uncond_text: Optional[torch.Tensor] = None):
        dims = session.weights.dims
        layers, tokens = session.layers(), session.tokens()
        if not 1 <= steps <= 100 or not 0.0 <= guidance <= 100.0:
            raise InvalidArgument("invalid generation arguments")  # src/pipeline/mod.rs:309-314
        if tables.dtype != torch.bfloat16 or tables.numel() != layers * 6 * dims.hidden or not tables.is_cuda:
            raise InvalidArgument("tables must be device bf16 [layers][6][hidden]")
        if text.dtype != torch.bfloat16 or text.dim() != 2 or text.shape[1] != dims.hidden or text.shape[0] >= tokens:
            raise InvalidArgument("text must be device bf16 [text_tokens][hidden] with text_tokens < tokens")
        if guidance > 0.0 and (uncond_text is None or uncond_text.shape != text.shape):
            raise InvalidArgument("guidance needs the negative prompt's text tokens, shaped like the prompt's")
        self.session, self.tables, self.cos, self.sin = session, tables.contiguous(), cos, sin
        self.text, self.uncond_text = text.contiguous(), uncond_text
        self.steps, self.guidance = steps, guidance
        self.text_tokens, self.image_tokens = text.shape[0], tokens - text.shape[0]
        # Turbo's shift is fixed; Raw's follows the image's token count (src/pipeline/mod.rs:338-339).
        self.mu = schedule.dynamic_mu(self.image_tokens) if mu is None else mu
        device = text.device
        self.mods = torch.empty((layers, 6, dims.hidden), dtype=torch.float32, device=device)
        self.x = torch.empty((tokens, dims.hidden), dtype=torch.bfloat16, device=device)
        self.velocity = torch.empty((self.image_tokens, dims.hidden), dtype=torch.bfloat16, device=device)
        self.unguided = torch.empty_like(self.velocity) if guidance > 0.0 else None

    def _forward(self, sample: torch.Tensor, text: torch.Tensor, velocity: torch.Tensor) -> None:
        stream = self.session.stream
        self.x[: self.text_tokens].copy_(text, non_blocking=True)
        self.x[self.text_tokens:].copy_(sample, non_blocking=True)
        self.session.run_device(stream, self.x, self.mods, self.cos, self.sin)
        velocity.copy_(self.x[self.text_tokens:], non_blocking=True)

    def step(self, index: int, sample: torch.Tensor, vector: torch.Tensor, last: Optional[int] = None) -> float:
        """Step `index` of the schedule on `sample` (updated in place); returns the Euler delta it used."""
        last = self.steps if last is None else last
        stream = self.session.stream
        with torch.cuda.stream(stream):
            sigma = schedule.sigma(index, self.steps, self.mu)
            # `next - sigma` is an f32 subtraction in the reference (src/pipeline/mod.rs:356)
            delta = float(np.float32(schedule.next_sigma(index, last, self.steps, self.mu)) - np.float32(sigma))
            ops.modulation(vector, self.tables, self.mods, stream)
            self._forward(sample, self.text, self.velocity)
            if self.guidance > 0.0:
                self._forward(sample, self.uncond_text, self.unguided)
                ops.guidance(self.velocity, self.unguided, self.guidance, stream)
            ops.euler_step(sample, self.velocity, delta, stream)
        return delta

    def generate(self, sample: torch.Tensor, vectors: Sequence[torch.Tensor],
                 progress: Optional[Callable[[int, int], str]] = None) -> torch.Tensor:
        """All steps on `sample` (bf16 `[image_tokens][hidden]`, updated in place and returned).  `progress(step,
        last)` is called after each step and may answer FINISH (end after the next step, which then lands on sigma
        zero) or CANCEL, as the reference's progress callback does (src/pipeline/mod.rs:357-364)."""
        if len(vectors) < self.steps:
            raise InvalidArgument("one modulation vector per step is needed")
        last, index = self.steps, 0
        while index < last:
            self.step(index, sample, vectors[index], last)
            if progress is not None:
                self.session.stream.synchronize()
                answer = progress(index + 1, last)
                if answer == FINISH:
                    last = min(last, index + 2)
                elif answer == CANCEL:
                    raise Cancelled("generation cancelled")
            index += 1
        return sample
