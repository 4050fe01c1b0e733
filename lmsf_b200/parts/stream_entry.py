"""What a span of layers that runs several times with the same weights adds to the residual stream at the start of each
pass: the embedding's output again (every pass but the first) and a learned vector per pass."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels
from .base import StepContext, StreamEntry, WeightSpec, register_part


@register_part("stream_entry", "loop_entry")
class LoopEntry(StreamEntry):
    """res += first (passes 1, 2, ... when `readd_first`) ; res += step[n_pass].  float32, one kernel."""
    graph_safe = True

    def __init__(self, hidden_size: int, times: int, readd_first: bool = True, step_vector: bool = True):
        self.hidden_size, self.times = int(hidden_size), int(times)
        self.readd_first, self.step_vector = bool(readd_first), bool(step_vector)
        self.needs_first = self.readd_first and self.times > 1
        self.step: Optional[torch.Tensor] = None
        self._step32: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {"step": WeightSpec([(self.times, self.hidden_size)], keep_fp32=True)} if self.step_vector else {}

    def prepare(self, dtype, device) -> None:
        self._step32 = self.step.float().contiguous() if self.step_vector else None

    def forward(self, ctx: StepContext, res: torch.Tensor, first: Optional[torch.Tensor], n_pass: int) -> None:
        if not (0 <= n_pass < self.times):
            raise ValueError(f"pass {n_pass} of a span that runs {self.times} times")
        add_first = first if (self.readd_first and n_pass > 0) else None
        if self.readd_first and n_pass > 0 and first is None:
            raise ValueError("the embedding's output was not kept for the later passes")
        kernels.stream_norm(res, first=add_first, vec=self._step32[n_pass] if self.step_vector else None)
