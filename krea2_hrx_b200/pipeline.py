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


def share_of_image(first: int, count: int, text_tokens: int):
    """Rows [first, first + count) of `[text; image]` as (text rows held, first image row, image rows held)."""
    text_count = max(0, min(first + count, text_tokens) - first)
    return text_count, max(first, text_tokens) - text_tokens, count - text_count


class ShardedDenoiser:
    """The same loop on one device's rows of a token-sharded image (`parallel.TokenParallel`).

    Nothing between two steps crosses rows: the modulation tables are per block, and the Euler update of a
    sample row needs that row's velocity only.  So a device keeps to its rows of `[text; image]` from the
    first step to the last -- the keys and values inside each block are the only exchange -- and the caller
    gathers `image_rows` of every device's sample once at the end.  Each device passes the whole sample
    (bf16 `[image_tokens][hidden]`) and owns the rows `image_rows` of it; the others are left as they were.
    Bit-identical to `Denoiser` on one device, row for row.  Guidance (a second forward per step) is not
    offered here."""

    def __init__(self, runner, tables: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, text: torch.Tensor,
                 steps: int = 8, mu: Optional[float] = schedule.TURBO_MU, collective: str = "push", graph: bool = True):
        dims, layers, tokens = runner.dims, runner.layers, runner.tokens
        if not 1 <= steps <= 100:
            raise InvalidArgument("invalid generation arguments")
        if tables.dtype != torch.bfloat16 or tables.numel() != layers * 6 * dims.hidden or not tables.is_cuda:
            raise InvalidArgument("tables must be device bf16 [layers][6][hidden]")
        if text.dtype != torch.bfloat16 or text.dim() != 2 or text.shape[1] != dims.hidden or text.shape[0] >= tokens:
            raise InvalidArgument("text must be device bf16 [text_tokens][hidden] with text_tokens < tokens")
        self.runner, self.tables, self.steps = runner, tables.contiguous(), steps
        self.collective, self.graph = collective, graph
        self.text_tokens, self.image_tokens = text.shape[0], tokens - text.shape[0]
        self.mu = schedule.dynamic_mu(self.image_tokens) if mu is None else mu
        first, count = runner.rows
        self.text_count, image_first, image_count = share_of_image(first, count, self.text_tokens)
        self.image_rows = (image_first, image_count)
        self.text_local = text[first:first + self.text_count].contiguous()
        with torch.cuda.stream(runner.stream):
            runner.cos.copy_(cos.view(tokens, -1)[first:first + count], non_blocking=True)
            runner.sin.copy_(sin.view(tokens, -1)[first:first + count], non_blocking=True)
        self._delta = 0.0

    def _rows(self, sample: torch.Tensor) -> torch.Tensor:
        if sample.dtype != torch.bfloat16 or tuple(sample.shape) != (self.image_tokens, self.runner.dims.hidden):
            raise InvalidArgument("sample must be device bf16 [image_tokens][hidden]")
        first, count = self.image_rows
        return sample[first:first + count]

    def begin_step(self, index: int, sample: torch.Tensor, vector: torch.Tensor, last: Optional[int] = None) -> float:
        """What precedes the blocks: this step's modulation tables and this device's rows of `[text; image]`."""
        last = self.steps if last is None else last
        runner, mine = self.runner, self._rows(sample)
        sigma = schedule.sigma(index, self.steps, self.mu)
        self._delta = float(np.float32(schedule.next_sigma(index, last, self.steps, self.mu)) - np.float32(sigma))
        with torch.cuda.stream(runner.stream):
            ops.modulation(vector, self.tables, runner.mods, runner.stream)
            count = runner.rows[1]
            if self.text_count:
                runner.x[: self.text_count].copy_(self.text_local, non_blocking=True)
            if mine.shape[0]:
                runner.x[self.text_count:count].copy_(mine, non_blocking=True)
        return self._delta

    def finish_step(self, sample: torch.Tensor) -> None:
        """What follows the blocks: the Euler update of this device's sample rows from its velocity rows."""
        runner, mine = self.runner, self._rows(sample)
        if mine.shape[0]:
            with torch.cuda.stream(runner.stream):
                ops.euler_step(mine, runner.x[self.text_count:runner.rows[1]], self._delta, runner.stream)

    def step(self, index: int, sample: torch.Tensor, vector: torch.Tensor, last: Optional[int] = None) -> float:
        delta = self.begin_step(index, sample, vector, last)
        self.runner.replay(self.collective, self.graph)
        self.finish_step(sample)
        return delta

    def generate(self, sample: torch.Tensor, vectors: Sequence[torch.Tensor]) -> torch.Tensor:
        """All steps on this device's rows of `sample` (updated in place; the other rows are not touched)."""
        if len(vectors) < self.steps:
            raise InvalidArgument("one modulation vector per step is needed")
        for index in range(self.steps):
            self.step(index, sample, vectors[index])
        return sample

    def gather(self, sample: torch.Tensor) -> torch.Tensor:
        """Fills every device's `sample` with all devices' rows: one all-gather of the devices' equal, padded shares
        of `[text; image]` over the runner's process group (`torch.distributed`)."""
        import torch.distributed as dist
        runner, mine = self.runner, self._rows(sample)
        count = runner.rows[1]
        with torch.cuda.stream(runner.stream):
            local = torch.zeros((runner.share, sample.shape[1]), dtype=sample.dtype, device=sample.device)
            if mine.shape[0]:
                local[self.text_count:count].copy_(mine, non_blocking=True)
            full = torch.empty((runner.world * runner.share, sample.shape[1]), dtype=sample.dtype, device=sample.device)
            dist.all_gather_into_tensor(full, local, group=runner.fabric.group)
            sample.copy_(full[self.text_tokens:runner.tokens], non_blocking=True)
        return sample
