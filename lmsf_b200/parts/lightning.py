"""Linear attention with a decay per head ("lightning attention"): a recurrent mixer whose per-request state is one
[dk, dv] matrix per head, kept in float32 in a state slot.

  q, k = act(h Wq^T), act(h Wk^T)  [heads x dk];  v = act(h Wv^T)  [heads x dv]
  S_t = decay_h S_(t-1) + k_t v_t^T ;  o_t = S_t^T q_t           (no other scale)
  out = (norm(o over all heads) * w * sigmoid(h Wg^T)) Wo^T

q, k, v and the gate come from one merged product; the activation is applied by the scan kernel as it reads them
(float32, from the stored value); the state, the decays and o are float32; norm and gate are one kernel.
Prompt portions and single tokens run on the same kernel (csrc/lightning.cu), so the state after a prompt is the same
bits however the prompt was cut.
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import torch

from .. import kernels
from .base import LayerCache, Mixer, StateSpec, StepContext, WeightSpec, register_part
from .linear import matmul_tn


@register_part("mixer", "lightning_attention")
class LightningAttention(Mixer):
    graph_safe = True      # every index comes from device tensors; the launch depends on the batch's size only

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, value_dim: int, decay: Sequence[float],
                 eps: float, activation: Optional[str] = "silu"):
        if len(decay) != num_heads:
            raise ValueError(f"{len(decay)} decays for {num_heads} heads")
        if not (0 < head_dim <= kernels.LIGHTNING_MAX_DK):
            raise ValueError(f"head_dim {head_dim} is beyond the scan kernel (up to {kernels.LIGHTNING_MAX_DK})")
        if activation not in kernels.LIGHTNING_ACTS:
            raise ValueError(f"activation {activation!r} is not supported (known: silu, none)")
        self.hidden_size, self.num_heads, self.head_dim, self.value_dim = int(hidden_size), int(num_heads), int(head_dim), int(value_dim)
        self.decay_values = [float(d) for d in decay]
        self.eps, self.activation = float(eps), activation
        self.qk_size, self.v_size = self.num_heads * self.head_dim, self.num_heads * self.value_dim
        self.qkvg: Optional[torch.Tensor] = None
        self.o: Optional[torch.Tensor] = None
        self.norm: Optional[torch.Tensor] = None
        self._decay: Optional[torch.Tensor] = None
        self._norm32: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        D = self.hidden_size
        return {"qkvg": WeightSpec([(self.qk_size, D), (self.qk_size, D), (self.v_size, D), (self.v_size, D)]),
                "o": WeightSpec([(D, self.v_size)]),
                "norm": WeightSpec([(self.v_size,)], keep_fp32=True)}

    def state_spec(self) -> Optional[StateSpec]:
        return StateSpec((self.num_heads, self.head_dim, self.value_dim))

    def activation_width(self) -> int:
        return 2 * self.qk_size + 5 * self.v_size        # q, k, v, gate, o in float32 (two), the gated norm

    def prepare(self, dtype, device) -> None:
        self._decay = torch.tensor(self.decay_values, dtype=torch.float32, device=device)
        self._norm32 = self.norm.float().contiguous()

    def forward(self, ctx: StepContext, h: torch.Tensor, cache: LayerCache) -> torch.Tensor:
        p = matmul_tn(h, self.qkvg)
        a, b = self.qk_size, self.v_size
        q, k, v, g = p[:, :a], p[:, a:2 * a], p[:, 2 * a:2 * a + b], p[:, 2 * a + b:]
        o = torch.empty((ctx.n_tokens, b), dtype=torch.float32, device=p.device)
        kernels.lightning_scan(o, q, k, v, cache.state, self._decay, ctx.cu_q, ctx.state_slot, ctx.n_seqs, self.num_heads,
                               self.head_dim, self.value_dim, self.activation)
        y = torch.empty((ctx.n_tokens, b), dtype=p.dtype, device=p.device)
        kernels.gated_norm(y, o, g, self._norm32, self.eps)
        return matmul_tn(y, self.o)
