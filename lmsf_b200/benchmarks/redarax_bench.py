"""Prefill and decode throughput of the Redarax design at layer sizes that resemble a real model's, beside the Vufolorn
design (the engine's other model of recurrent and attention layers with routed experts) at equal width, layers and
experts, and the design's kernels alone beside the like kernel of that model.

    python bench.py --design redarax [--steps K] [--warmup W]

Random weights, seeded random token ids.  Timing as in bench.py: CUDA events on the launching stream after warm-up;
decode steps read weights and state far larger than L2; prefill and the kernels alone start from a flushed L2.
"""
from __future__ import annotations

import json

import torch

from . import design_bench
from .design_bench import CONTEXT, PREFILL_TOKENS, measure_model


def redarax_config(width, heads, kv_heads, dim, experts, top, ff, dense_ff, vocab, side=256):
    moe = {"kind": "moe", "expert": {"ff": ff, "limit": 7.0},
           "router": {"experts": experts, "top": top, "groups": {"count": 8, "keep": 4}}}
    att = {"type": "attention", "mlp": moe,
           "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "rot": {"dims": dim // 2, "base": 1.0e6}}}
    ssm = {"type": "mamba2", "mlp": moe,
           "mixer": {"heads": width // 64, "vdim": 64, "state": 128, "groups": 1, "norm_groups": 1, "conv": 4}}
    dlt = {"type": "delta", "mixer": {"heads": heads, "kv_heads": heads // 2, "dim": dim, "vdim": dim, "conv": 4}}
    return {"architecture": "Redarax", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "residual_mult": 0.7,
            "token_side": {"dim": side}, "logit_scale": 1.0, "logit_softcap": 30.0,
            "layers": [att, ssm, dict(dlt, mlp=moe), dict(dlt, mlp={"kind": "dense", "ff": dense_ff, "limit": 7.0})]}


SIZES = {
    "width2048": redarax_config(2048, 16, 4, 128, 32, 4, 1024, 4096, 32000),
    "width4096": redarax_config(4096, 32, 8, 128, 64, 6, 1408, 7552, 32000),
}


def kernels_alone(pk, width=4096, heads=32, dim=128, experts=64, top=6):
    """Each new kernel alone with the like kernel of the Vufolorn or Llama path beside it, and what each reaches of its
    roofline: the measured copy rate for kernels that stream, the device's nominal float32 FMA rate (148 SMs x 128 lanes
    x 2 x 1.9 GHz) for the float32 scans."""
    from lmsf_b200 import kernels
    from lmsf_b200.benchmarks.kernel_bench import Timer
    dev = torch.device("cuda:0")
    tm = Timer(dev)
    bf, f32, i32 = torch.bfloat16, torch.float32, torch.int32
    T = PREFILL_TOKENS
    hbm = pk["hbm_gbs"] * 1e9
    fp32_peak = 148 * 128 * 2 * 1.9e9
    rows = {}

    def rec(name, sec, bytes_=None, flops=None, like=None):
        r = {"us": round(sec * 1e6, 1)}
        if bytes_ is not None:
            r["frac_of_copy_rate"] = round(bytes_ / sec / hbm, 3)
        if flops is not None:
            r["frac_of_fp32_peak"] = round(flops / sec / fp32_peak, 3)
        if like:
            r["like"] = like
        rows[name] = r

    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *s, dtype=bf, scale=1.0: (torch.randn(*s, generator=g, device=dev, dtype=f32) * scale).to(dtype)
    ones = lambda n: torch.ones(n, device=dev)
    # ---- between two branches
    res, y, h = rnd(T, width, dtype=f32), rnd(T, width), torch.empty(T, width, dtype=bf, device=dev)
    w = ones(width)
    rec("stream_norm (branch norm, factor, add, stream handed on) 2048 x 4096",
        tm.run(lambda: kernels.stream_norm(res, y=y, w_post=w, eps_post=1e-5, h=h, branch_scale=0.7), 3, 10), bytes_=T * width * (4 + 4 + 2 + 2))
    rec("stream_norm (Vufolorn: post norm, layer scale, add, next norm) 2048 x 4096",
        tm.run(lambda: kernels.stream_norm(res, y=y, w_post=w, layer_scale=w, eps_post=1e-5, h=h, w_next=w, eps_next=1e-5), 3, 10),
        bytes_=T * width * (4 + 4 + 2 + 2))
    # ---- q/k norm + rotation + cache write against rotation + cache write
    H, G, bs = heads, heads // 4, 16
    qkv = rnd(T, (H + 2 * G) * dim)
    q, k, v = qkv[:, :H * dim], qkv[:, H * dim:(H + G) * dim], qkv[:, (H + G) * dim:]
    pages = T // bs
    cache = torch.zeros(pages + 1, 2, G, bs, dim, dtype=bf, device=dev)
    pos, seq = torch.arange(T, dtype=i32, device=dev), torch.zeros(T, dtype=i32, device=dev)
    table = torch.arange(pages, dtype=i32, device=dev).view(1, pages)
    inv = torch.tensor([1.0e6 ** (-2.0 * i / 64) for i in range(32)], dtype=f32, device=dev)
    moved = T * ((H + G) * dim * 2 * 2 + G * dim * 2 * 2)
    rec("qk_norm_rope_cache_write 2048 tokens, 32 + 8 heads of 128 (64 rotated, interleaved)",
        tm.run(lambda: kernels.qk_norm_rope_cache_write(q, k, v, pos, seq, table, bs, cache, inv, 64, False, H, G, dim, dim, ones(dim), ones(dim), 1e-5), 3, 10),
        bytes_=moved)
    inv_full = torch.tensor([1.0e6 ** (-2.0 * i / 128) for i in range(64)], dtype=f32, device=dev)
    rec("rope_cache_write (Llama: NeoX pairs, no norm) 2048 tokens, 32 + 8 heads of 128",
        tm.run(lambda: kernels.rope_cache_write(q, k, v, pos, seq, table, bs, cache, inv_full, 128, True, H, G, dim), 3, 10), bytes_=moved)
    # ---- convolution with carried inputs
    for name, C in (("delta rule: q, k, v", 2 * (H // 2) * dim + H * dim), ("state space: x, B, C", width + 2 * 128)):
        x, out = rnd(T, C), torch.empty(T, C, dtype=bf, device=dev)
        cw, cb = rnd(C, 4, dtype=f32), rnd(C, dtype=f32)
        st = torch.zeros(65, 3 * C, dtype=f32, device=dev)
        cu1, sl1 = torch.tensor([0, T], dtype=i32, device=dev), torch.zeros(1, dtype=i32, device=dev)
        rec(f"causal_conv + silu ({name}), one prompt of 2048 tokens x {C} channels, 4 taps",
            tm.run(lambda: kernels.causal_conv(out, x, cw, cb, st, 0, cu1, sl1, 1, T), 3, 10), bytes_=T * C * 4)
        cu64, sl64 = torch.arange(65, dtype=i32, device=dev), torch.arange(64, dtype=i32, device=dev)
        rec(f"causal_conv + silu ({name}), decode of 64 requests",
            tm.run(lambda: kernels.causal_conv(out[:64], x[:64], cw, cb, st, 0, cu64, sl64, 64, 1), 3, 10), bytes_=64 * C * (4 + 3 * 4 * 2))
    # ---- the scans
    cu1, sl1 = torch.tensor([0, T], dtype=i32, device=dev), torch.zeros(1, dtype=i32, device=dev)
    cu64, sl64 = torch.arange(65, dtype=i32, device=dev), torch.arange(64, dtype=i32, device=dev)
    for name, Hs, Gs, dk, dv, delta in (("gated_scan, delta rule, 32 heads 128 x 128 over 16 q/k heads", H, H // 2, dim, dim, True),
                                        ("gated_scan, state space, 64 heads 128 x 64 over one B/C group", width // 64, 1, 128, 64, False)):
        qs, ks, vs = rnd(T, Gs * dk), rnd(T, Gs * dk), rnd(T, Hs * dv)
        dt, beta = rnd(T, Hs), rnd(T, Hs)
        o = torch.empty(T, Hs * dv, dtype=f32, device=dev)
        state = torch.zeros(65, Hs * dk * dv, dtype=f32, device=dev)
        bias, alog, skip = rnd(Hs, dtype=f32), rnd(Hs, dtype=f32), (None if delta else ones(Hs))
        kw = dict(delta=delta, k_times_dt=not delta, unit_qk=delta, q_scale=dk ** -0.5 if delta else 1.0)
        per_token = (6.0 if delta else 4.0) * Hs * dk * dv
        rec(f"{name}: one prompt of 2048 tokens as one chain (prepare + scan)",
            tm.run(lambda: kernels.gated_scan(o, qs, ks, vs, dt, beta if delta else None, bias, alog, skip, state, cu1, sl1, 1, Hs, Gs, dk, dv, **kw), 1, 3),
            flops=per_token * T, like="lightning_scan as one chain below")
        rec(f"{name}: decode of 64 requests (reads and writes 64 x {Hs * dk * dv * 4 // 1024} KB of state; prepare + scan)",
            tm.run(lambda: kernels.gated_scan(o[:64], qs[:64], ks[:64], vs[:64], dt[:64], beta[:64] if delta else None, bias, alog, skip, state,
                                              cu64, sl64, 64, Hs, Gs, dk, dv, **kw), 3, 10),
            bytes_=64 * Hs * dk * dv * 4 * 2, like="lightning_scan decode below")
    ql, kl, vl = rnd(T, H * dim), rnd(T, H * dim), rnd(T, H * dim)
    ol = torch.empty(T, H * dim, dtype=f32, device=dev)
    lstate = torch.zeros(65, H, dim, dim, dtype=f32, device=dev)
    decay = torch.full((H,), 0.98, device=dev)
    rec("lightning_scan (Vufolorn), one prompt of 2048 tokens as one chain, 32 heads 128 x 128",
        tm.run(lambda: kernels.lightning_scan(ol, ql, kl, vl, lstate, decay, cu1, sl1, 1, H, dim, dim, "silu"), 1, 3), flops=4.0 * T * H * dim * dim)
    rec("lightning_scan (Vufolorn), decode of 64 requests",
        tm.run(lambda: kernels.lightning_scan(ol[:64], ql[:64], kl[:64], vl[:64], lstate, decay, cu64, sl64, 64, H, dim, dim, "silu"), 3, 10),
        bytes_=64 * H * dim * dim * 4 * 2)
    # ---- norm over groups with a gate
    xo, gate, yn = rnd(T, width, dtype=f32), rnd(T, width), torch.empty(T, width, dtype=bf, device=dev)
    rec("grouped_gated_norm, per head of 128, gate after (delta rule) 2048 x 4096",
        tm.run(lambda: kernels.grouped_gated_norm(yn, xo, gate, ones(dim), dim, 1e-5, gate_first=False), 3, 10), bytes_=T * width * (4 + 2 + 2))
    rec("grouped_gated_norm, whole row, gate first (state space) 2048 x 4096",
        tm.run(lambda: kernels.grouped_gated_norm(yn, xo, gate, ones(width), width, 1e-5, gate_first=True), 3, 10), bytes_=T * width * (4 + 2 + 2))
    rec("gated_norm (Vufolorn) 2048 x 4096", tm.run(lambda: kernels.gated_norm(yn, xo, gate, ones(width), 1e-5), 3, 10), bytes_=T * width * (4 + 2 + 2))
    # ---- routing and the experts' activation
    logits = rnd(T, experts, dtype=f32)
    ids, wts = torch.empty(T, top, dtype=i32, device=dev), torch.empty(T, top, dtype=f32, device=dev)
    corr = rnd(experts, dtype=f32, scale=0.1)
    rec("moe_topk_sigmoid, 2048 tokens, 6 of 64 in 4 of 8 groups", tm.run(lambda: kernels.moe_topk_sigmoid(ids, wts, logits, corr, experts, 8, 4), 3, 10))
    rec("moe_topk (Vufolorn), 2048 tokens, 6 of 64", tm.run(lambda: kernels.moe_topk(ids, wts, logits, None, experts), 3, 10))
    ff = 1408
    gu, act = rnd(T * top, 2 * ff), torch.empty(T * top, ff, dtype=bf, device=dev)
    rec("clamped_glu 12288 x 1408", tm.run(lambda: kernels.clamped_glu(act, gu, 7.0), 3, 10), bytes_=T * top * ff * 6)
    rec("gated_act (Llama, silu) 12288 x 1408", tm.run(lambda: kernels.gated_act(act, gu, "silu"), 3, 10), bytes_=T * top * ff * 6)
    return rows


def run(bench, steps, warmup, pk):
    sampler = bench.ClockSampler()
    sampler.start()
    sizes = {}
    for name, cfg in SIZES.items():
        sizes[name] = {"redarax": measure_model(cfg, [8, 64], steps, warmup, bench),
                       "vufolorn": measure_model(design_bench.SIZES[name][0], [8, 64], steps, warmup, bench)}
    alone = kernels_alone(pk)
    line = {"metric": "prefill and decode tokens/s of the Redarax design beside the Vufolorn design of equal width (4 layers each, random weights)",
            "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup, "dtype": "bf16", "data": "synthetic",
            "config": {"prefill_tokens": PREFILL_TOKENS, "context": CONTEXT, "block_size": design_bench.BLOCK_SIZE, "sizes": SIZES,
                       "vufolorn": {k: v[0] for k, v in design_bench.SIZES.items()}, "peaks": pk.get("source", "measured")},
            "sizes": sizes, "kernels_alone": alone, "clocks": sampler.stop(), "impl": "ours"}
    print(json.dumps(line))
    return 0
