"""Redarax: the description of the decoder as data, and its registry entry.

A plain embedding; layers that each hold one of three mixers (causal attention with biases, a norm of queries and keys
per head and a partial interleaved rotation; a selective state-space layer; the gated delta rule), a feed-forward (dense
or routed experts, both with clamped gate and up factors; or none) and a small branch gated by the stream that adds a
per-layer vector of the token; norms on the branches' outputs only, every branch scaled by one factor; a final norm and
a head whose logits are scaled and capped.  Tensor names: `embed`, `side.embed`, `final.norm`, `head`, and `l<i>.` +
`norm1`, `norm2`, `mix.*`, `mlp.*`, `side.*`.
"""
from __future__ import annotations

from ..config.redarax_config import RedaraxConfig
from ..config.registry import register_architecture
from ..parts.base import LayerCall, LayerSpec, ModelSpec, PartSpec


def redarax_spec(cfg: RedaraxConfig) -> ModelSpec:
    D = cfg.width
    norm = lambda name: PartSpec("rmsnorm", dict(hidden_size=D, eps=cfg.eps), {"weight": name})
    layers, ignored = [], []
    n_layers = len(cfg.layers)
    for i, L in enumerate(cfg.layers):
        p, m = f"l{i}.", L.mixer
        if m.type == "attention":
            rope = PartSpec("rotary", dict(rot_dim=m.rot_dims, theta=m.rot_base, is_neox=False)) if m.rot_dims else None
            mixer = PartSpec("paged_attention",
                             dict(hidden_size=D, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, value_dim=m.vdim,
                                  position_encoding=rope, scale=m.scale, bias=True, qk_norm=True, qk_norm_eps=cfg.eps),
                             {"qkv": [p + "mix.q", p + "mix.k", p + "mix.v"], "o": p + "mix.o",
                              "qkv_bias": [p + "mix.q.b", p + "mix.k.b", p + "mix.v.b"], "o_bias": p + "mix.o.b",
                              "q_norm": p + "mix.q.norm", "k_norm": p + "mix.k.norm"})
        elif m.type == "mamba2":
            mixer = PartSpec("selective_state_space",
                             dict(hidden_size=D, num_heads=m.heads, head_dim=m.vdim, state_size=m.state, groups=m.groups,
                                  conv_taps=m.conv, norm_groups=m.norm_groups, eps=cfg.eps),
                             {"in_proj": p + "mix.in", "conv": p + "mix.conv", "conv_bias": p + "mix.conv.b",
                              "dt_bias": p + "mix.dt_bias", "a_log": p + "mix.A_log", "skip": p + "mix.D",
                              "norm": p + "mix.norm", "o": p + "mix.o"})
        else:
            mixer = PartSpec("gated_delta_rule",
                             dict(hidden_size=D, num_heads=m.heads, num_qk_heads=m.kv_heads, head_dim=m.dim, value_dim=m.vdim,
                                  conv_taps=m.conv, eps=cfg.eps),
                             {"in_proj": [p + "mix.q", p + "mix.k", p + "mix.v", p + "mix.g", p + "mix.b", p + "mix.a"],
                              "conv": [p + "mix.q.conv", p + "mix.k.conv", p + "mix.v.conv"],
                              "dt_bias": p + "mix.dt_bias", "a_log": p + "mix.A_log", "norm": p + "mix.norm", "o": p + "mix.o"})
        parts = {"mixer": mixer, "mixer_post_norm": norm(p + "norm1")}
        f = L.mlp
        if f is None:
            ignored.append(rf"^l{i}\.norm2$")
        elif f.kind == "dense":
            parts.update(feed_forward=PartSpec("gated_mlp", dict(hidden_size=D, intermediate_size=f.ff, activation="clamped_swiglu",
                                                                 limit=f.limit),
                                               {"gate_up": [p + "mlp.gate", p + "mlp.up"], "down": p + "mlp.down"}),
                         ffn_post_norm=norm(p + "norm2"))
        else:
            up = [p + f"mlp.e{e}.{w}" for e in range(f.experts) for w in ("gate", "up")]
            parts.update(feed_forward=PartSpec("routed_experts",
                                               dict(hidden_size=D, num_experts=f.experts, top_k=f.top, expert_size=f.ff,
                                                    activation="clamped_swiglu", limit=f.limit, router_bias=True,
                                                    shared_gate=False, routing="sigmoid_groups", groups=f.groups,
                                                    group_keep=f.keep),
                                               {"up": up, "down": [p + f"mlp.e{e}.down" for e in range(f.experts)],
                                                "router": [p + "mlp.router"], "router_bias": p + "mlp.correction"}),
                         ffn_post_norm=norm(p + "norm2"))
        if cfg.side_dim:
            parts.update(side=PartSpec("token_gated_projection",
                                       dict(hidden_size=D, vocab_size=cfg.vocab, dim=cfg.side_dim,
                                            table_width=cfg.side_dim * n_layers, offset=i * cfg.side_dim),
                                       {"table": "side.embed", "gate": p + "side.gate", "proj": p + "side.proj"}),
                         side_post_norm=norm(p + "side.norm"))
        layers.append(LayerSpec("branch_norm", parts, dict(residual_mult=cfg.residual_mult)))
    return ModelSpec(
        hidden_size=D, vocab_size=cfg.vocab, max_model_len=cfg.max_model_len,
        embedding=PartSpec("token_embedding", dict(vocab_size=cfg.vocab, hidden_size=D), {"weight": "embed"}),
        layers=layers, order=[LayerCall(i) for i in range(n_layers)],
        final_norm=norm("final.norm"),
        lm_head=PartSpec("dense", dict(in_features=D, out_features=cfg.vocab, out_dtype="float32",
                                       out_scale=cfg.logit_scale, out_softcap=cfg.logit_softcap or None), {"weight": "head"}),
        eos_token_ids=list(cfg.eos_token_ids), ignored_weights=ignored,
    )


register_architecture("Redarax", RedaraxConfig.from_dict, redarax_spec, aliases=("redarax",))
