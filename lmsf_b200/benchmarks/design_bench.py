"""Prefill and decode throughput of the Vufolorn design at layer sizes that resemble a real model's, beside the Llama
shape of equal width and equal parameters per token, and the design's kernels alone beside the like kernel of Llama.

    python bench.py --design vufolorn [--steps K] [--warmup W]

Random weights, seeded random token ids.  Timing as in bench.py: CUDA events on the launching stream after warm-up;
decode steps read weights and cache far larger than L2; prefill and the kernels alone start from a flushed L2.
"""
from __future__ import annotations

import json
import os
import tempfile

import torch

BLOCK_SIZE = 16
PREFILL_TOKENS = 2048
CONTEXT = 2048


def vufolorn_config(width, heads, dim, rank, window, experts, top, ff, shared, vocab, pairs=2):
    decay = [1.0 - 2.0 ** (-5.0 - 3.0 * h / max(1, heads - 1)) for h in range(heads)]
    mlp = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}, "shared": {"ff": shared}}
    lin = {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": dim, "decay": decay}, "mlp": mlp}
    lat = {"type": "latent_attention", "mlp": mlp,
           "mixer": {"heads": heads, "dim": dim, "vdim": dim, "kv_rank": rank, "scale": dim ** -0.5, "mask": {"size": window}}}
    return {"architecture": "Vufolorn", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "layers": [lin, lat] * pairs}


def llama_config(width, heads, kv_heads, dim, inter, vocab, layers):
    return dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_size=width, num_hidden_layers=layers,
                num_attention_heads=heads, num_key_value_heads=kv_heads, head_dim=dim, intermediate_size=inter, vocab_size=vocab,
                rope_theta=500000.0, rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=8192,
                hidden_act="silu", torch_dtype="bfloat16")


# name -> (Vufolorn, Llama of the same width, layers and matrix parameters that a token uses per layer)
SIZES = {
    "width2048": (vufolorn_config(2048, 16, 128, 128, 1024, 32, 4, 1024, 2048, 32000),
                  llama_config(2048, 16, 4, 128, 4096, 32000, 4)),
    "width4096": (vufolorn_config(4096, 32, 128, 128, 2048, 64, 6, 1408, 2816, 32000),
                  llama_config(4096, 32, 8, 128, 7552, 32000, 4)),
}


def measure_model(cfg, batches, steps, warmup, bench):
    """tokens/s of a prefill of PREFILL_TOKENS tokens and of decode steps at each batch size, through the engine's step
    function (`bench` is bench.py's module: its timing loops are used as they are)."""
    from lmsf_b200.engine.factory import build_model
    from lmsf_b200.engine.model_runner import ModelRunner
    folder = tempfile.mkdtemp(prefix="lmsf_design_")
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    dev = torch.device("cuda:0")
    model, _, dtype = build_model(folder, "bfloat16", dev, load_format="dummy")
    pages = (max(batches) * (CONTEXT + 64) + PREFILL_TOKENS) // BLOCK_SIZE + 64
    runner = ModelRunner(model, dtype, dev, BLOCK_SIZE, num_blocks=pages, max_num_seqs=max(batches) + 2, max_model_len=CONTEXT + 4096)
    for t in runner.storage.tensors:
        t.normal_(0.0, 1.0)
    mgr = runner.make_cache_manager()
    V = model.spec.vocab_size
    out = {}
    for b in batches:
        ids = bench.fill_requests(runner, mgr, b, CONTEXT, f"b{b}_")
        ms, launches = bench.time_decode(runner, mgr, ids, steps, warmup, V)
        for r in ids:
            mgr.free(r)
        out[f"decode_b{b}_tok_s"] = round(b / (ms * 1e-3), 1)
        out[f"decode_b{b}_ms"] = round(ms, 4)
        out[f"decode_b{b}_launches_per_step"] = launches // steps
    pf_ms = bench.time_prefill(runner, mgr, PREFILL_TOKENS, 3, 2, V)
    out["prefill_tok_s"] = round(PREFILL_TOKENS / (pf_ms * 1e-3), 1)
    out["prefill_ms"] = round(pf_ms, 3)
    params = sum(getattr(p, n).numel() for p, _ in model.parts_with_specs() for n in p.weight_specs() if getattr(p, n, None) is not None)
    out["weight_bytes"] = 2 * params
    del runner, mgr, model
    torch.cuda.empty_cache()
    return out


def kernels_alone(pk, width=4096, heads=32, dim=128, rank=128, window=2048, experts=64, top=6, ff=1408):
    """Each kernel of the design alone, with the like kernel of the Llama path beside it, and what each reaches of its
    roofline: the measured copy rate for kernels that stream, the measured bf16 product rate for tensor-core kernels,
    the device's nominal float32 FMA rate (148 SMs x 128 lanes x 2 x the clock seen) for the float32 scan."""
    from lmsf_b200 import kernels
    from lmsf_b200.benchmarks.kernel_bench import Timer
    dev = torch.device("cuda:0")
    tm = Timer(dev)
    bf, f32, i32 = torch.bfloat16, torch.float32, torch.int32
    T = PREFILL_TOKENS
    hbm, tflops = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    fp32_peak = 148 * 128 * 2 * 1.9e9
    rows = {}

    def rec(name, sec, bytes_=None, flops=None, peak=None, like=None):
        r = {"us": round(sec * 1e6, 1)}
        if bytes_ is not None:
            r["frac_of_copy_rate"] = round(bytes_ / sec / hbm, 3)
        if flops is not None:
            r["frac_of_peak"] = round(flops / sec / (peak or tflops), 3)
        if like:
            r["like"] = like
        rows[name] = r

    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *s, dtype=bf, scale=1.0: (torch.randn(*s, generator=g, device=dev, dtype=f32) * scale).to(dtype)
    # ---- norms between branches against add + norm
    res, y, h = rnd(T, width, dtype=f32), rnd(T, width), torch.empty(T, width, dtype=bf, device=dev)
    w = torch.ones(width, device=dev)
    rec("stream_norm (post norm, layer scale, add, next norm) 2048 x 4096",
        tm.run(lambda: kernels.stream_norm(res, y=y, w_post=w, layer_scale=w, eps_post=1e-5, h=h, w_next=w, eps_next=1e-5), 3, 10),
        bytes_=T * width * (4 + 4 + 2 + 2))
    wb = torch.ones(width, device=dev, dtype=bf)
    rec("add_rmsnorm (Llama) 2048 x 4096", tm.run(lambda: kernels.add_rmsnorm(h, y, res, wb, 1e-5, 2), 3, 10), bytes_=T * width * (4 + 4 + 2 + 2))
    # ---- the experts' products against the library's product of the same size
    E, P = experts, T * top
    x = rnd(T, width)
    up, down = rnd(E, ff, width, scale=0.02), rnd(E, width, ff, scale=0.02)
    logits = rnd(T, E, dtype=f32)
    ids, wts = torch.empty(T, top, dtype=i32, device=dev), torch.empty(T, top, dtype=f32, device=dev)
    kernels.moe_topk(ids, wts, logits, None, E)
    mt = kernels.moe_max_tiles(P, E, kernels.MOE_TC_TILE_ROWS)
    offsets, pair_row, row_token = (torch.empty(n, dtype=i32, device=dev) for n in (E + 1, P, P))
    tiles, meta = torch.empty(mt, 4, dtype=i32, device=dev), torch.empty(4, dtype=i32, device=dev)
    pr = pair_row.view(T, top)
    rec("moe_topk + moe_align, 2048 tokens, 6 of 64",
        tm.run(lambda: (kernels.moe_topk(ids, wts, logits, None, E), kernels.moe_align(ids, E, kernels.MOE_TC_TILE_ROWS, offsets, pr, row_token, tiles, meta)), 3, 10))
    yb, db = torch.empty(P, ff, dtype=bf, device=dev), torch.empty(P, width, dtype=f32, device=dev)
    rec("moe_grouped_tc up (+ relu^2), 12288 rows x 1408 x 4096, 64 experts",
        tm.run(lambda: kernels.moe_grouped_tc(yb, x, up, row_token, tiles, meta, act="relu2"), 3, 10), flops=2.0 * P * ff * width)
    rec("moe_grouped_tc down, 12288 rows x 4096 x 1408",
        tm.run(lambda: kernels.moe_grouped_tc(db, yb, down, None, tiles, meta), 3, 10), flops=2.0 * P * ff * width)
    xa, wa = rnd(P, width), rnd(ff, width, scale=0.02)
    rec("library product (Llama's gate/up kind) 12288 x 1408 x 4096", tm.run(lambda: torch.mm(xa, wa.t()), 3, 10), flops=2.0 * P * ff * width)
    # the same products in a decode step of 64 tokens: weight streaming
    n = 64
    xd = rnd(n, width)
    idd, wtd = torch.empty(n, top, dtype=i32, device=dev), torch.empty(n, top, dtype=f32, device=dev)
    kernels.moe_topk(idd, wtd, rnd(n, E, dtype=f32), None, E)
    Pd = n * top
    mtd = kernels.moe_max_tiles(Pd, E, kernels.MOE_TC_TILE_ROWS)
    od, prd, rtd = (torch.empty(k, dtype=i32, device=dev) for k in (E + 1, Pd, Pd))
    tld, med = torch.empty(mtd, 4, dtype=i32, device=dev), torch.empty(4, dtype=i32, device=dev)
    kernels.moe_align(idd, E, kernels.MOE_TC_TILE_ROWS, od, prd.view(n, top), rtd, tld, med)
    hit = int(torch.unique(idd).numel())
    ydd = torch.empty(Pd, ff, dtype=bf, device=dev)
    rec(f"moe_grouped_tc up, decode of 64 tokens ({hit} experts hit)",
        tm.run(lambda: kernels.moe_grouped_tc(ydd, xd, up, rtd, tld, med, act="relu2"), 3, 10), bytes_=hit * ff * width * 2)
    wg = rnd(hit * ff, width, scale=0.02)
    rec("library product of 64 rows against as many weights (Llama's decode at batch 64)", tm.run(lambda: torch.mm(xd, wg.t()), 3, 10),
        bytes_=hit * ff * width * 2)
    # ---- linear attention: a prompt, and a decode step of 64 requests
    H, dk = heads, dim
    q, k, v = rnd(T, H * dk), rnd(T, H * dk), rnd(T, H * dk)
    o = torch.empty(T, H * dk, dtype=f32, device=dev)
    state = torch.zeros(65, H, dk, dk, dtype=f32, device=dev)
    decay = torch.full((H,), 0.98, device=dev)
    cu1, sl1 = torch.tensor([0, T], dtype=i32, device=dev), torch.zeros(1, dtype=i32, device=dev)
    from lmsf_b200.parts.lightning import CHUNK_TOKENS
    chunks = torch.tensor([(0, c, min(c + CHUNK_TOKENS, T), i) for i, c in enumerate(range(0, T, CHUNK_TOKENS))], dtype=i32, device=dev)
    spans = torch.tensor([(0, 0, chunks.shape[0], 0)], dtype=i32, device=dev)
    scratch = torch.empty(chunks.shape[0], H, dk, dk, dtype=f32, device=dev)
    args = (o, q, k, v, state, decay, cu1, sl1, 1, H, dk, dk, "silu")

    def chunked():
        kernels.lightning_scan(*args, items=chunks, scratch=scratch, mode=1)
        kernels.lightning_prefix(scratch, state, decay, sl1, chunks, spans)
        kernels.lightning_scan(*args, items=chunks, scratch=scratch, mode=2)
    rec("lightning_scan, one prompt of 2048 tokens in parallel chunks, 32 heads 128 x 128 (float32 FMA, both passes)",
        tm.run(chunked, 2, 5), flops=2 * 4.0 * T * H * dk * dk, peak=fp32_peak, like="prefill attention of Llama below")
    rec("lightning_scan, the same prompt as one chain of tokens",
        tm.run(lambda: kernels.lightning_scan(*args), 1, 3), flops=4.0 * T * H * dk * dk, peak=fp32_peak)
    cu64, sl64 = torch.arange(65, dtype=i32, device=dev), torch.arange(64, dtype=i32, device=dev)
    rec("lightning_scan, decode of 64 requests (reads and writes 64 x 2 MB of state)",
        tm.run(lambda: kernels.lightning_scan(o[:64], q[:64], k[:64], v[:64], state, decay, cu64, sl64, 64, H, dk, dk, "silu"), 3, 10),
        bytes_=64 * H * dk * dk * 4 * 2, like="decode attention of Llama below")
    gate, yn = rnd(T, H * dk), torch.empty(T, H * dk, dtype=bf, device=dev)
    wn = torch.ones(H * dk, device=dev)
    rec("gated_norm 2048 x 4096", tm.run(lambda: kernels.gated_norm(yn, o, gate, wn, 1e-5), 3, 10), bytes_=T * H * dk * (4 + 2 + 2))
    return rows


def attention_alone(pk, heads=32, rank=128, window=2048):
    """The attention kernels on the one-plane cache (32 heads over one cached vector of 128 values, window 2,048) beside
    the same kernels on Llama's two planes (32 heads over 8 kv heads of 128): a prompt of 2,048 tokens and a decode step
    of 64 requests at 2,048-token contexts, through the parts' own dispatch."""
    from lmsf_b200.benchmarks.kernel_bench import Timer
    from lmsf_b200.parts.attention import paged_attend
    from lmsf_b200.parts.base import KVCacheSpec
    dev = torch.device("cuda:0")
    tm = Timer(dev)
    rows = {}
    for name, spec, kvh in (("one plane (latent, 32 heads x 1 vector of 128, window 2048)", KVCacheSpec(1, rank, window, planes=1), 1),
                            ("two planes (Llama, 32 heads over 8 kv heads of 128)", KVCacheSpec(8, 128, None), 8)):
        bs, pages = 16, 64 * (CONTEXT + 64) // 16 + 256
        cache = (torch.randn(pages + 1, spec.planes, spec.num_kv_heads, bs, spec.head_dim, device=dev) * 0.5).bfloat16()
        hd = spec.head_dim
        for what, seqs in (("prefill 2048", [(0, PREFILL_TOKENS)]), ("decode 64 x 2048", [(CONTEXT - 1, 1)] * 64)):
            ctx = _context(seqs, bs, pages, spec.window)
            q = (torch.randn(ctx.n_tokens, heads * hd, device=dev) * 0.5).bfloat16()
            out = torch.empty_like(q)
            fn = lambda: paged_attend(ctx, out, q, cache, ctx.groups[0], num_heads=heads, num_kv_heads=kvh, head_dim=hd,
                                      scale=hd ** -0.5, window=spec.window, kv_planes=spec.planes)
            sec = tm.run(fn, 3, 10)
            r = {"us": round(sec * 1e6, 1)}
            if what.startswith("decode"):
                seen = min(CONTEXT, spec.window or CONTEXT)
                r["frac_of_copy_rate"] = round(64 * seen * spec.planes * kvh * hd * 2 / sec / (pk["hbm_gbs"] * 1e9), 3)
            else:
                r["frac_of_peak"] = round(4.0 * heads * hd * PREFILL_TOKENS * PREFILL_TOKENS / 2 / sec / (pk["bf16_tflops"] * 1e12), 3)
            rows[f"attention, {what}, {name}"] = r
    return rows


def _context(seqs, block_size, n_pages, window):
    from lmsf_b200.parts.base import CacheGroupView, StepContext
    dev = torch.device("cuda:0")
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    pos, tseq, cu, ctx_lens, q_lens = [], [], [0], [], []
    max_blocks = max((s + n + block_size - 1) // block_size for s, n in seqs)
    table = torch.full((len(seqs), max_blocks), -1, dtype=torch.int32)
    nxt = 0
    for i, (start, n) in enumerate(seqs):
        pos += list(range(start, start + n))
        tseq += [i] * n
        cu.append(cu[-1] + n)
        ctx_lens.append(start + n)
        q_lens.append(n)
        nb = (start + n + block_size - 1) // block_size
        table[i, :nb] = torch.arange(nxt, nxt + nb, dtype=torch.int32)
        nxt += nb
    assert nxt <= n_pages
    dec = [i for i, (_, n) in enumerate(seqs) if n == 1]
    tiles = lambda size: [(i, q0) for i, (_, n) in enumerate(seqs) if n > 1 for q0 in range(0, n, size)][::-1]   # most keys first
    t64, t128 = tiles(64), tiles(128)
    return StepContext(n_tokens=len(pos), n_seqs=len(seqs), dtype=torch.bfloat16, device=dev, token_ids=i32([0] * len(pos)),
                       positions=i32(pos), token_seq=i32(tseq), cu_q=i32(cu), ctx_len=i32(ctx_lens), state_slot=i32([0] * len(seqs)),
                       groups=[CacheGroupView(table.to(dev), block_size)], q_lens=q_lens, ctx_lens=ctx_lens, state_slots=[0] * len(seqs),
                       error_flag=torch.zeros(1, dtype=torch.int32, device=dev), decode_seq_ids=i32(dec or [0]), n_decode_seqs=len(dec),
                       q_tile_seq=i32([t[0] for t in t64] or [0]), q_tile_q0=i32([t[1] for t in t64] or [0]), n_q_tiles=len(t64),
                       q_tile128_seq=i32([t[0] for t in t128] or [0]), q_tile128_q0=i32([t[1] for t in t128] or [0]), n_q_tiles128=len(t128))


def run(bench, steps, warmup, pk):
    sampler = bench.ClockSampler()
    sampler.start()
    sizes = {}
    for name, (vuf, llama) in SIZES.items():
        sizes[name] = {"vufolorn": measure_model(vuf, [8, 64], steps, warmup, bench), "llama": measure_model(llama, [8, 64], steps, warmup, bench)}
    alone = kernels_alone(pk)
    alone.update(attention_alone(pk))
    line = {"metric": "prefill and decode tokens/s of the Vufolorn design beside the Llama shape of equal width (4 layers each, random weights)",
            "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup, "dtype": "bf16", "data": "synthetic",
            "config": {"prefill_tokens": PREFILL_TOKENS, "context": CONTEXT, "block_size": BLOCK_SIZE, "sizes": {k: v[0] for k, v in SIZES.items()},
                       "llama": {k: v[1] for k, v in SIZES.items()}, "peaks": pk.get("source", "measured")},
            "sizes": sizes, "kernels_alone": alone, "clocks": sampler.stop(), "impl": "ours"}
    print(json.dumps(line))
    return 0
