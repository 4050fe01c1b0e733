"""Recurrent mixers whose per-request state is one [dk, dv] matrix per head, kept in float32 in a state slot together
with the last inputs of a short causal convolution (csrc/recurrent.cu).

`selective_state_space` (a state-space layer with a scalar decay per head and token):
  [z | x | B | C | dt] = h Win^T;  (x, B, C) <- silu(conv(x, B, C) + b)
  dt = softplus(dt + dt_bias);  S_t = exp(-exp(A_log) dt) S_(t-1) + dt B_t x_t^T;  y_t = S_t^T C_t + D x_t
  out = (norm_g(y * silu(z)) * w) Wo^T                      (the gate before the norm; the norm over `norm_groups` parts)

`gated_delta_rule`:
  q, k, v = silu(conv(h Wq^T)), silu(conv(h Wk^T)), silu(conv(h Wv^T));  q, k made unit vectors, q times dk^(-1/2)
  a = exp(-exp(A_log) softplus(h Wa^T + dt_bias));  beta = sigmoid(h Wb^T)
  S <- a S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
  out = (norm_head(o) * w * silu(h Wg^T)) Wo^T               (the norm per head, its weight shared by the heads)

Both run prompt portions and single tokens on the same kernels; every index comes from device tensors, so decode steps can
be replayed from CUDA graphs.  Decays, step sizes, unit norms, the state and every sum of the recurrence are float32; the
projections, the convolution and their activation have the activation type.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels
from .base import LayerCache, Mixer, StateSpec, StepContext, WeightSpec, register_part
from .linear import matmul_tn


class _StateMatrixMixer(Mixer):
    graph_safe = True

    def _check_sizes(self, dk: int, taps: int) -> None:
        if not (0 < dk <= kernels.SCAN_MAX_DK):
            raise ValueError(f"a state of {dk} rows per head is beyond the scan kernel (up to {kernels.SCAN_MAX_DK})")
        if not (1 <= taps <= kernels.CONV_MAX_TAPS):
            raise ValueError(f"a convolution of {taps} taps is beyond the kernel (1 to {kernels.CONV_MAX_TAPS})")

    def _max_q(self, ctx: StepContext) -> int:
        return max(ctx.q_lens) if ctx.q_lens else 1


@register_part("mixer", "selective_state_space")
class SelectiveStateSpace(_StateMatrixMixer):
    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, state_size: int, groups: int, conv_taps: int,
                 norm_groups: int, eps: float):
        if num_heads % groups:
            raise ValueError(f"{num_heads} heads cannot share {groups} groups of B and C")
        self.hidden_size, self.num_heads, self.head_dim = int(hidden_size), int(num_heads), int(head_dim)
        self.state_size, self.groups, self.taps, self.norm_groups = int(state_size), int(groups), int(conv_taps), int(norm_groups)
        self.eps = float(eps)
        self.inner = self.num_heads * self.head_dim
        if self.inner % self.norm_groups:
            raise ValueError(f"{self.norm_groups} norm groups do not divide {self.inner} columns")
        self._check_sizes(self.state_size, self.taps)
        self.channels = self.inner + 2 * self.groups * self.state_size          # what passes the convolution
        self.in_size = 2 * self.inner + 2 * self.groups * self.state_size + self.num_heads
        self.matrix_floats = self.num_heads * self.head_dim * self.state_size
        self.in_proj = self.conv = self.conv_bias = self.dt_bias = self.a_log = self.skip = self.norm = self.o = None
        self._f32: Dict[str, torch.Tensor] = {}

    def weight_specs(self) -> Dict[str, WeightSpec]:
        H = self.num_heads
        return {"in_proj": WeightSpec([(self.in_size, self.hidden_size)]),
                "conv": WeightSpec([(self.channels, self.taps)], keep_fp32=True),
                "conv_bias": WeightSpec([(self.channels,)], keep_fp32=True),
                "dt_bias": WeightSpec([(H,)], keep_fp32=True), "a_log": WeightSpec([(H,)], keep_fp32=True),
                "skip": WeightSpec([(H,)], keep_fp32=True), "norm": WeightSpec([(self.inner,)], keep_fp32=True),
                "o": WeightSpec([(self.hidden_size, self.inner)])}

    def state_spec(self) -> Optional[StateSpec]:
        return StateSpec((self.matrix_floats + (self.taps - 1) * self.channels,))

    def activation_width(self) -> int:
        return self.in_size + self.channels + 3 * self.inner

    def prepare(self, dtype, device) -> None:
        self._f32 = {n: getattr(self, n).float().contiguous() for n in ("conv", "conv_bias", "dt_bias", "a_log", "skip", "norm")}

    def forward(self, ctx: StepContext, h: torch.Tensor, cache: LayerCache) -> torch.Tensor:
        n, I, GN, H = ctx.n_tokens, self.inner, self.groups * self.state_size, self.num_heads
        p = matmul_tn(h, self.in_proj)
        z, xbc, dt = p[:, :I], p[:, I:I + self.channels], p[:, I + self.channels:]
        c = torch.empty((n, self.channels), dtype=p.dtype, device=p.device)
        w = self._f32
        kernels.causal_conv(c, xbc, w["conv"], w["conv_bias"], cache.state, self.matrix_floats, ctx.cu_q, ctx.state_slot,
                            ctx.n_seqs, self._max_q(ctx), act="silu")
        y = torch.empty((n, I), dtype=torch.float32, device=p.device)
        kernels.gated_scan(y, c[:, I + GN:], c[:, I:I + GN], c[:, :I], dt, None, w["dt_bias"], w["a_log"], w["skip"],
                           cache.state, ctx.cu_q, ctx.state_slot, ctx.n_seqs, H, self.groups, self.state_size, self.head_dim,
                           delta=False, k_times_dt=True)
        g = torch.empty((n, I), dtype=p.dtype, device=p.device)
        kernels.grouped_gated_norm(g, y, z, w["norm"], I // self.norm_groups, self.eps, gate_act="silu", gate_first=True)
        return matmul_tn(g, self.o)


@register_part("mixer", "gated_delta_rule")
class GatedDeltaRule(_StateMatrixMixer):
    def __init__(self, hidden_size: int, num_heads: int, num_qk_heads: int, head_dim: int, value_dim: int, conv_taps: int,
                 eps: float, unit_eps: float = 1e-6):
        if num_heads % num_qk_heads:
            raise ValueError(f"{num_heads} heads cannot share {num_qk_heads} query/key heads")
        self.hidden_size, self.num_heads, self.num_qk_heads = int(hidden_size), int(num_heads), int(num_qk_heads)
        self.head_dim, self.value_dim, self.taps = int(head_dim), int(value_dim), int(conv_taps)
        self.eps, self.unit_eps = float(eps), float(unit_eps)
        self._check_sizes(self.head_dim, self.taps)
        self.qk_size, self.v_size = self.num_qk_heads * self.head_dim, self.num_heads * self.value_dim
        self.channels = 2 * self.qk_size + self.v_size
        self.matrix_floats = self.num_heads * self.value_dim * self.head_dim
        self.in_proj = self.conv = self.dt_bias = self.a_log = self.norm = self.o = None
        self._f32: Dict[str, torch.Tensor] = {}

    def weight_specs(self) -> Dict[str, WeightSpec]:
        D, H, QK, V = self.hidden_size, self.num_heads, self.qk_size, self.v_size
        # one merged product: q, k, v (which pass the convolution), the output gate, the write strength, the decay's input
        return {"in_proj": WeightSpec([(QK, D), (QK, D), (V, D), (V, D), (H, D), (H, D)]),
                "conv": WeightSpec([(QK, self.taps), (QK, self.taps), (V, self.taps)], keep_fp32=True),
                "dt_bias": WeightSpec([(H,)], keep_fp32=True), "a_log": WeightSpec([(H,)], keep_fp32=True),
                "norm": WeightSpec([(self.value_dim,)], keep_fp32=True),
                "o": WeightSpec([(D, V)])}

    def state_spec(self) -> Optional[StateSpec]:
        return StateSpec((self.matrix_floats + (self.taps - 1) * self.channels,))

    def activation_width(self) -> int:
        return 2 * self.channels + 4 * self.v_size

    def prepare(self, dtype, device) -> None:
        self._f32 = {n: getattr(self, n).float().contiguous() for n in ("conv", "dt_bias", "a_log", "norm")}

    def forward(self, ctx: StepContext, h: torch.Tensor, cache: LayerCache) -> torch.Tensor:
        n, QK, V, H = ctx.n_tokens, self.qk_size, self.v_size, self.num_heads
        p = matmul_tn(h, self.in_proj)
        C = self.channels
        gate, beta, dt = p[:, C:C + V], p[:, C + V:C + V + H], p[:, C + V + H:]
        c = torch.empty((n, C), dtype=p.dtype, device=p.device)
        w = self._f32
        kernels.causal_conv(c, p[:, :C], w["conv"], None, cache.state, self.matrix_floats, ctx.cu_q, ctx.state_slot,
                            ctx.n_seqs, self._max_q(ctx), act="silu")
        o = torch.empty((n, V), dtype=torch.float32, device=p.device)
        kernels.gated_scan(o, c[:, :QK], c[:, QK:2 * QK], c[:, 2 * QK:], dt, beta, w["dt_bias"], w["a_log"], None,
                           cache.state, ctx.cu_q, ctx.state_slot, ctx.n_seqs, H, self.num_qk_heads, self.head_dim,
                           self.value_dim, delta=True, unit_qk=True, unit_eps=self.unit_eps, q_scale=self.head_dim ** -0.5)
        g = torch.empty((n, V), dtype=p.dtype, device=p.device)
        kernels.grouped_gated_norm(g, o, gate, w["norm"], self.value_dim, self.eps, gate_act="silu", gate_first=False)
        return matmul_tn(g, self.o)
