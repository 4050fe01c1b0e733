"""A small branch that lets the token itself speak in every layer: each layer owns `dim` columns of a table with one row
per token id; the stream chooses how much of them passes.

  e = table[token][offset : offset + dim];  g = gelu_tanh(h Wgate^T) * e;  out = g Wproj^T

The table is one tensor for all layers (a layer reads its columns in place); the gate's activation and the product with
the table's row are one kernel.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels
from .base import FeedForward, StepContext, WeightSpec, register_part
from .linear import matmul_tn


@register_part("feed_forward", "token_gated_projection")
class TokenGatedProjection(FeedForward):
    graph_safe = True

    def __init__(self, hidden_size: int, vocab_size: int, dim: int, table_width: int, offset: int):
        if not (0 <= offset and offset + dim <= table_width):
            raise ValueError(f"columns {offset}..{offset + dim} are outside a table of {table_width} columns")
        self.hidden_size, self.vocab_size, self.dim = int(hidden_size), int(vocab_size), int(dim)
        self.table_width, self.offset = int(table_width), int(offset)
        self.table: Optional[torch.Tensor] = None
        self.gate: Optional[torch.Tensor] = None
        self.proj: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {"table": WeightSpec([(self.vocab_size, self.table_width)]),
                "gate": WeightSpec([(self.dim, self.hidden_size)]),
                "proj": WeightSpec([(self.hidden_size, self.dim)])}

    def activation_width(self) -> int:
        return 2 * self.dim + self.hidden_size

    def forward(self, ctx: StepContext, h: torch.Tensor) -> torch.Tensor:
        a = matmul_tn(h, self.gate)
        g = torch.empty((h.shape[0], self.dim), dtype=h.dtype, device=h.device)
        kernels.gelu_mul_gather(g, a, self.table, self.offset, ctx.token_ids, ctx.error_flag)
        return matmul_tn(g, self.proj)
