"""Linear attention with a decay per head ("lightning attention"): a recurrent mixer whose per-request state is one
[dk, dv] matrix per head, kept in float32 in a state slot.

  q, k = act(h Wq^T), act(h Wk^T)  [heads x dk];  v = act(h Wv^T)  [heads x dv]
  S_t = decay_h S_(t-1) + k_t v_t^T ;  o_t = S_t^T q_t           (no other scale)
  out = (norm(o over all heads) * w * sigmoid(h Wg^T)) Wo^T

q, k, v and the gate come from one merged product; the activation is applied by the scan kernel as it reads them
(float32, from the stored value); the state, the decays and o are float32; norm and gate are one kernel.
Prompt portions and single tokens run on the same kernel (csrc/lightning.cu); portions of LONG_PORTION tokens and more
are cut into chunks that run in parallel (two passes of that kernel around a prefix over the chunks' states).
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import torch

from .. import kernels
from .base import LayerCache, Mixer, StateSpec, StepContext, WeightSpec, register_part
from .linear import matmul_tn


LONG_PORTION = 256      # tokens from which a request's portion is cut into chunks that run in parallel
CHUNK_TOKENS = 64


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

    @staticmethod
    def _plan(ctx: StepContext):
        """None when no request brings a long portion.  Else (short, chunks, spans), made once a step from the host's copy
        of the portions' lengths and shared by all layers: `short` lists the requests that run whole (None if there are
        none), `chunks` cuts every long portion into pieces of CHUNK_TOKENS, `spans` names each long portion's pieces."""
        if not ctx.q_lens or max(ctx.q_lens) < LONG_PORTION:
            return None
        plan = ctx.extras.get("lightning_plan")
        if plan is None:
            short, chunks, spans, t0 = [], [], [], 0
            for s, n in enumerate(ctx.q_lens):
                if n >= LONG_PORTION:
                    first = len(chunks)
                    for c in range(t0, t0 + n, CHUNK_TOKENS):
                        chunks.append((s, c, min(c + CHUNK_TOKENS, t0 + n), len(chunks)))
                    spans.append((s, first, len(chunks), 0))
                else:
                    short.append((s, t0, t0 + n, 0))
                t0 += n
            flat = torch.tensor(short + chunks + spans, dtype=torch.int32).to(ctx.device, non_blocking=True)
            a, b = len(short), len(short) + len(chunks)
            plan = ctx.extras["lightning_plan"] = (flat[:a] if a else None, flat[a:b], flat[b:])
        return plan

    def forward(self, ctx: StepContext, h: torch.Tensor, cache: LayerCache) -> torch.Tensor:
        p = matmul_tn(h, self.qkvg)
        a, b = self.qk_size, self.v_size
        q, k, v, g = p[:, :a], p[:, a:2 * a], p[:, 2 * a:2 * a + b], p[:, 2 * a + b:]
        o = torch.empty((ctx.n_tokens, b), dtype=torch.float32, device=p.device)
        plan = self._plan(ctx)
        args = (o, q, k, v, cache.state, self._decay, ctx.cu_q, ctx.state_slot, ctx.n_seqs, self.num_heads, self.head_dim,
                self.value_dim, self.activation)
        if plan is None:                     # single tokens and short portions: one block row per request
            kernels.lightning_scan(*args)
        else:
            short, chunks, spans = plan
            if short is not None:
                kernels.lightning_scan(*args, items=short)
            scratch = torch.empty((chunks.shape[0], self.num_heads, self.head_dim, self.value_dim), dtype=torch.float32, device=p.device)
            kernels.lightning_scan(*args, items=chunks, scratch=scratch, mode=1)
            kernels.lightning_prefix(scratch, cache.state, self._decay, ctx.state_slot, chunks, spans)
            kernels.lightning_scan(*args, items=chunks, scratch=scratch, mode=2)
        y = torch.empty((ctx.n_tokens, b), dtype=p.dtype, device=p.device)
        kernels.gated_norm(y, o, g, self._norm32, self.eps)
        return matmul_tn(y, self.o)
