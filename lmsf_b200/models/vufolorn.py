"""Vufolorn: the description of the decoder as data, and its registry entry.

A normed embedding; layers that each hold one of two mixers (linear attention with a decay per head, or attention over a
cached low-rank vector inside a sliding window) and routed experts with a shared expert (or no feed-forward), with a
norm before and after every branch and a layer scale on the branch; a span of layers that runs several times with the
same weights (each run has a cache or state of its own; the embedding's output and a vector per pass are added at the
start of a pass); a final norm and the embedding table as the head.  Tensor names: `embed`, `embed.norm`, `final.norm`,
`loop.step`, and `l<i>.` + `norm1`, `norm1b`, `ls1`, `norm2`, `norm2b`, `ls2`, `mix.*`, `mlp.*`.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.vufolorn_config import VufolornConfig
from ..parts.base import LayerCall, LayerSpec, ModelSpec, PartSpec


def vufolorn_spec(cfg: VufolornConfig) -> ModelSpec:
    D = cfg.width
    norm = lambda name: PartSpec("rmsnorm", dict(hidden_size=D, eps=cfg.eps), {"weight": name})
    post = lambda name, ls: PartSpec("rmsnorm", dict(hidden_size=D, eps=cfg.eps, layer_scale=True), {"weight": name, "scale": ls})
    layers = []
    for i, L in enumerate(cfg.layers):
        p, m = f"l{i}.", L.mixer
        if m.type == "lightning":
            mixer = PartSpec("lightning_attention",
                             dict(hidden_size=D, num_heads=m.heads, head_dim=m.dim, value_dim=m.vdim, decay=list(m.decay),
                                  eps=cfg.eps, activation="silu"),
                             {"qkvg": [p + "mix.q", p + "mix.k", p + "mix.v", p + "mix.g"], "o": p + "mix.o", "norm": p + "mix.norm"})
        else:
            mixer = PartSpec("latent_attention",
                             dict(hidden_size=D, num_heads=m.heads, head_dim=m.dim, value_dim=m.vdim, kv_rank=m.kv_rank,
                                  eps=cfg.eps, scale=m.scale, window=m.window, gate=True),
                             {"qcg": [p + "mix.q", p + "mix.dkv", p + "mix.g"], "c_norm": p + "mix.dkv.norm",
                              "uk": p + "mix.uk", "uv": p + "mix.uv", "o": p + "mix.o"})
        parts = {"mixer_norm": norm(p + "norm1"), "mixer": mixer, "mixer_post_norm": post(p + "norm1b", p + "ls1")}
        if L.mlp is not None:
            f = L.mlp
            w = {"up": [p + f"mlp.e{e}.up" for e in range(f.experts)], "down": [p + f"mlp.e{e}.down" for e in range(f.experts)],
                 "router": [p + "mlp.router"] + ([p + "mlp.shared.sg"] if f.shared_ff else []), "router_bias": p + "mlp.router.b"}
            if f.shared_ff:
                w.update(shared_up=p + "mlp.shared.up", shared_down=p + "mlp.shared.down")
            parts.update(ffn_norm=norm(p + "norm2"),
                         feed_forward=PartSpec("routed_experts",
                                               dict(hidden_size=D, num_experts=f.experts, top_k=f.top, expert_size=f.expert_ff,
                                                    shared_size=f.shared_ff, activation="relu2", router_bias=True,
                                                    shared_gate=True), w),
                         ffn_post_norm=post(p + "norm2b", p + "ls2"))
        layers.append(LayerSpec("sandwich_norm", parts))
    order, entries = [], []
    if cfg.has_loop:
        entries.append(PartSpec("loop_entry", dict(hidden_size=D, times=cfg.loop_times, readd_first=True, step_vector=True),
                                {"step": "loop.step"}))
        order += [LayerCall(i) for i in range(cfg.loop_start)]
        for t in range(cfg.loop_times):
            for i in range(cfg.loop_start, cfg.loop_stop):
                order.append(LayerCall(i, entry=0, entry_pass=t) if i == cfg.loop_start else LayerCall(i))
        order += [LayerCall(i) for i in range(cfg.loop_stop, len(cfg.layers))]
    else:
        order = [LayerCall(i) for i in range(len(cfg.layers))]
    return ModelSpec(
        hidden_size=D, vocab_size=cfg.vocab, max_model_len=cfg.max_model_len,
        embedding=PartSpec("normed_token_embedding", dict(vocab_size=cfg.vocab, hidden_size=D, eps=cfg.eps),
                           {"weight": "embed", "norm": "embed.norm"}),
        layers=layers, order=order, entries=entries,
        final_norm=norm("final.norm"),
        lm_head=PartSpec("dense", dict(in_features=D, out_features=cfg.vocab, out_dtype="float32"), {"weight": "embed"}),
        eos_token_ids=list(cfg.eos_token_ids),
        ignored_weights=([] if cfg.has_loop else [r"^loop\.step$"]),
    )


register_architecture("Vufolorn", VufolornConfig.from_dict, vufolorn_spec, aliases=("vufolorn",))
