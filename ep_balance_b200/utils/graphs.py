"""Replaying a whole step from a CUDA graph.

The native layer never reads device data on the host (routing, group sizes and slot use stay on the GPU), so a
forward, or a full training step with a ``capturable`` optimizer, is a fixed sequence of launches that can be
captured once and replayed.  Replay removes the host's per-launch cost; with device-side cross-rank barriers
in every step that matters beyond launch latency: a host that falls behind stalls every other rank's GPU.

    step = GraphedStep(lambda x: train_step(x), example_batch)      # warms up, then captures
    loss = step(batch)                                               # copies the batch in, replays, returns the static output

Everything the step touches must live at fixed addresses: parameters, optimizer state (use
``FusedAdamW(capturable=True)`` / ``torch.optim.AdamW(capturable=True)``) and the input, which is copied into a
static buffer before each replay.  In a multi-rank group every rank must build and call its ``GraphedStep`` the same
number of times, as with eager steps.
"""

from __future__ import annotations

from typing import Callable

import torch


class GraphedStep:
    def __init__(self, step_fn: Callable[[torch.Tensor], torch.Tensor], example_input: torch.Tensor, *,
                 warmup: int = 3) -> None:
        self.static_in = example_input.detach().clone()
        cur = torch.cuda.current_stream()
        side = torch.cuda.Stream(device=example_input.device)
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            for _ in range(warmup):
                step_fn(self.static_in)
        cur.wait_stream(side)
        torch.cuda.synchronize(example_input.device)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.static_out = step_fn(self.static_in)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        self.static_in.copy_(x, non_blocking=True)
        self.graph.replay()
        return self.static_out
