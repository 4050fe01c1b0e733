"""The Vufolorn design in the engine against the plain implementation of tests/plain_vufolorn.py: every mechanism
alone, then whole models (tiny, random, sizes that share nothing with each other) through the step function, the
trace program and the generation entry point."""
import json
import math
import os
import random
import tempfile

import numpy as np
import pytest
import torch

import plain_vufolorn as P
import traces
import util

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TDT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dev(t, dtype=None):
    return t.to(DEV) if dtype is None else t.to(device=DEV, dtype=dtype)


# ----------------------------------------------------------------------------- tiny configurations

def lightning(heads, dim, vdim, decay):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}}


def latent(heads, dim, vdim, rank, window, scale):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m}


def moe(experts, top, ff, shared):
    f = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared:
        f["shared"] = {"ff": shared}
    return f


def with_mlp(layer, mlp):
    return dict(layer, mlp=mlp)


# X: a window that is no multiple of the page, a rank that needs padding, head sizes that are no power of two, a
# layer without feed-forward, one without a shared expert, a span of two layers that runs three times and does not
# start at layer 0, a decay of exactly 1
CFG_X = {"architecture": "Vufolorn", "vocab": 211, "width": 72, "norm": {"eps": 1e-5},
         "layers": [with_mlp(latent(3, 16, 24, 24, 9, 0.31), moe(5, 2, 40, 56)),
                    with_mlp(lightning(2, 24, 40, [0.7, 1.0]), moe(3, 3, 24, 0)),
                    with_mlp(latent(2, 8, 40, 16, 21, 0.5), None),
                    with_mlp(lightning(3, 20, 8, [0.35, 0.9, 0.99]), moe(6, 1, 32, 16))],
         "loop": {"start": 1, "stop": 3, "times": 3}}
# Y: no span, one head, one expert, attention without a window, another eps
CFG_Y = {"architecture": "Vufolorn", "vocab": 97, "width": 40, "norm": {"eps": 1e-3},
         "layers": [with_mlp(lightning(1, 12, 12, [0.8]), moe(1, 1, 16, 8)),
                    with_mlp(latent(1, 32, 16, 48, None, 0.2), moe(4, 2, 8, 0)),
                    with_mlp(latent(4, 16, 16, 32, 5, 0.25), moe(4, 4, 16, 24))]}
# Z: a span that is the whole model and runs twice; a window of one page and one of a single key
CFG_Z = {"architecture": "Vufolorn", "vocab": 130, "width": 64, "norm": {"eps": 1e-6},
         "layers": [with_mlp(latent(2, 16, 8, 32, 16, 0.4), moe(8, 3, 16, 32)),
                    with_mlp(lightning(4, 8, 16, [0.5, 0.6, 0.97, 0.999]), None),
                    with_mlp(latent(5, 8, 8, 8, 1, 0.3), moe(2, 1, 24, 0))],
         "loop": {"start": 0, "stop": 3, "times": 2}}
CONFIGS = {"X": CFG_X, "Y": CFG_Y, "Z": CFG_Z}
BLOCK = {"X": 8, "Y": 16, "Z": 16}
_folders, _oracles = {}, {}


def folder_of(name, gain=1.0):
    """(folder with config.json and model.safetensors in bfloat16, the weights as the plain implementation takes them)."""
    from lmsf_b200.weights.safetensors_io import write_safetensors
    key = (name, gain)
    if key not in _folders:
        cfg = CONFIGS[name]
        w = P.random_weights(cfg, seed=sum(map(ord, name)), dtype=torch.bfloat16, gain=gain)
        d = tempfile.mkdtemp(prefix=f"lmsf_vuf_{name}_")
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(cfg, f)
        write_safetensors(os.path.join(d, "model.safetensors"), [(n, t.dtype, tuple(t.shape)) for n, t in w.items()], lambda n: w[n])
        _folders[key] = (d, w)
    return _folders[key]


def oracle(name, reqs, gain=1.0):
    _, w = folder_of(name, gain)
    out = {}
    for rid, toks in reqs.items():
        key = (name, gain, tuple(toks))
        if key not in _oracles:
            _oracles[key] = P.forward(CONFIGS[name], w, toks, dtype=torch.float64).float().numpy()
        out[rid] = _oracles[key]
    return out


def requests_for(name, lengths, seed=0):
    return {f"q{i}": util.random_ids(n, CONFIGS[name]["vocab"], seed + 11 * i) for i, n in enumerate(lengths)}


def worst_rel(rows, ref):
    scale = max(float(np.abs(r).max()) for r in ref.values())
    return max(float(np.abs(row - ref[rid][pos]).max()) for (rid, pos), row in rows.items()) / scale


TOL = {"float32": 2e-5, "bfloat16": 4e-2}


def position_errors(rows, ref):
    """Per position: root mean square of the difference of the logits (mean taken off) over that of the logits, sorted."""
    errs = []
    for (rid, pos), row in rows.items():
        d = row - ref[rid][pos]
        d = d - d.mean()
        errs.append(float(np.sqrt((d ** 2).mean()) / np.sqrt((ref[rid][pos] ** 2).mean())))
    return np.sort(np.asarray(errs))


def assert_close(rows, ref, dtype, what):
    """float32: every logit within 2e-5 of the largest.  bfloat16: these tiny random models route by close calls, and a
    token whose rounded router logits choose another expert moves far (seen: a few positions in a hundred by 0.1 to 0.9 of
    the logits' size, the same in every way of cutting), so the bound is on the bulk: half the positions within 1.2 %,
    nine in ten within 4 %.  What bfloat16 could hide beyond that (a window's edge, a far key) is tested on the kernels
    alone with inputs made to show it."""
    if dtype == "float32":
        assert worst_rel(rows, ref) <= TOL[dtype], (what, worst_rel(rows, ref))
    else:
        e = position_errors(rows, ref)
        assert e[len(e) // 2] <= 1.2e-2 and e[int(0.9 * len(e))] <= 4e-2, (what, e[len(e) // 2], e[int(0.9 * len(e))])


# ----------------------------------------------------------------------------- mechanisms alone

def test_stream_norm_does_what_lies_between_two_branches():
    from lmsf_b200 import kernels
    g = torch.Generator().manual_seed(1)
    for hidden in (40, 257, 1100):
        n = 5
        res = torch.randn(n, hidden, generator=g)
        y = torch.randn(n, hidden, generator=g) * 3
        first = torch.randn(n, hidden, generator=g)
        wp, ls, wn, vec = (1 + 0.3 * torch.randn(hidden, generator=g) for _ in range(4))
        for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2e-2)):
            yd = y.to(dtype)
            want_res = res.double() + P.rms_norm(yd.double(), wp.double(), 1e-5) * ls.double() + first.double() + vec.double()
            want_h = P.rms_norm(want_res, wn.double(), 1e-4)
            r, h = dev(res.clone()), torch.empty(n, hidden, dtype=dtype, device=DEV)
            kernels.stream_norm(r, y=dev(yd), w_post=dev(wp), layer_scale=dev(ls), eps_post=1e-5, first=dev(first), vec=dev(vec),
                                h=h, w_next=dev(wn), eps_next=1e-4)
            assert torch.allclose(r.cpu().double(), want_res, rtol=1e-5, atol=1e-5)          # the stream itself is float32
            assert torch.allclose(h.cpu().double(), want_h, rtol=tol, atol=tol)
            # nothing to add: the stream stays as it is, bit for bit
            r2 = dev(res.clone())
            kernels.stream_norm(r2, h=h, w_next=dev(wn), eps_next=1e-4)
            assert torch.equal(r2.cpu(), res)
            assert torch.allclose(h.cpu().double(), P.rms_norm(res.double(), wn.double(), 1e-4), rtol=tol, atol=tol)


def test_normed_embedding_leaves_a_float32_stream_and_a_copy():
    from lmsf_b200 import kernels
    g = torch.Generator().manual_seed(2)
    table = torch.randn(50, 72, generator=g).bfloat16()
    w = 1 + 0.3 * torch.randn(72, generator=g)
    ids = torch.tensor([3, 49, 0, 3], dtype=torch.int32)
    res, keep = torch.empty(4, 72, device=DEV), torch.empty(4, 72, device=DEV)
    kernels.embed_norm(res, keep, dev(table), dev(ids), dev(w), 1e-5)
    want = P.rms_norm(table.double()[ids.long()], w.double(), 1e-5)
    assert torch.allclose(res.cpu().double(), want, rtol=1e-5, atol=1e-6) and torch.equal(res, keep)


def plain_scan(q, k, v, decay, S):
    """The recurrence, token by token (float64).  q, k: [T, H, dk]; v: [T, H, dv]; S: [H, dk, dv], changed in place."""
    out = torch.zeros(q.shape[0], q.shape[1], v.shape[2], dtype=torch.float64)
    for t in range(q.shape[0]):
        for h in range(q.shape[1]):
            S[h] = decay[h] * S[h] + torch.outer(k[t, h], v[t, h])
            out[t, h] = S[h].T @ q[t, h]
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,dk,dv", [(3, 24, 40), (1, 7, 5), (2, 130, 33), (4, 64, 32)])
def test_lightning_scan_in_portions_and_token_by_token(dtype, heads, dk, dv):
    """Requests of unequal length in one launch, each with a state slot of its own; then the same tokens cut into
    portions (down to one token): the outputs and the final states must agree with the plain recurrence."""
    from lmsf_b200 import kernels
    g = torch.Generator().manual_seed(heads * 100 + dk)
    tdt = TDT[dtype]
    lens = [37, 1, 18]
    n = sum(lens)
    q, k, v = (torch.randn(n, heads * d, generator=g).to(tdt) for d in (dk, dk, dv))
    decay = torch.tensor([0.3, 1.0, 0.97, 0.999][:heads], dtype=torch.float32)
    silu = lambda z: P.silu(z.double())
    want, states, off = [], [], 0
    for L in lens:
        S = torch.zeros(heads, dk, dv, dtype=torch.float64)
        want.append(plain_scan(silu(q[off:off + L]).view(L, heads, dk), silu(k[off:off + L]).view(L, heads, dk),
                               silu(v[off:off + L]).view(L, heads, dv), decay.double(), S).reshape(L, heads * dv))
        states.append(S)
        off += L
    want = torch.cat(want)
    slots = [4, 0, 2]
    tol = 1e-5 if dtype == "float32" else 1e-4       # inputs are the same rounded values; the scan itself is float32

    def run(cuts):
        state = torch.full((6, heads, dk, dv), 7.0, device=DEV)            # slots hold rubbish until they are zeroed
        for s in slots:
            state[s].zero_()
        out = torch.empty(n, heads * dv, device=DEV)
        done = [0] * len(lens)
        starts = [0, lens[0], lens[0] + lens[1]]
        while any(d < L for d, L in zip(done, lens)):
            rows, cu, sl = [], [0], []
            for i, L in enumerate(lens):
                c = min(cuts[(done[i] + i) % len(cuts)], L - done[i])
                if c > 0:
                    rows += list(range(starts[i] + done[i], starts[i] + done[i] + c))
                    cu.append(cu[-1] + c)
                    sl.append(slots[i])
                    done[i] += c
            idx = torch.tensor(rows)
            o = torch.empty(len(rows), heads * dv, device=DEV)
            kernels.lightning_scan(o, dev(q[idx]), dev(k[idx]), dev(v[idx]), state, dev(decay), dev(torch.tensor(cu, dtype=torch.int32)),
                                   dev(torch.tensor(sl, dtype=torch.int32)), len(sl), heads, dk, dv, "silu")
            out[idx.to(DEV)] = o
        return out.cpu(), state.cpu()

    whole, st = run([1000])
    scale = float(want.abs().max())
    assert float((whole.double() - want).abs().max()) <= tol * scale
    for i, s in enumerate(slots):
        assert float((st[s].double() - states[i]).abs().max()) <= tol * max(1.0, float(states[i].abs().max()))
    assert torch.all(st[1] == 7.0)                                        # a slot nobody holds is not touched
    for cuts in ([1], [2, 5, 1, 16, 17], [16], [3]):
        part, st2 = run(cuts)
        assert torch.equal(part, whole) and torch.equal(st2, st), cuts      # the same operations in the same order


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_lightning_scan_of_a_long_portion_in_parallel_chunks(dtype):
    """A long portion that starts from a state that is not zero, cut into chunks of unequal size that run in parallel (from
    a zero state, then a prefix over the chunks' states, then again from the true state), beside a short request that runs
    whole: outputs and final states agree with the plain recurrence."""
    from lmsf_b200 import kernels
    g = torch.Generator().manual_seed(17)
    tdt = TDT[dtype]
    heads, dk, dv = 3, 40, 48
    lens = [5, 333]
    n = sum(lens)
    q, k, v = (torch.randn(n, heads * d, generator=g).to(tdt) for d in (dk, dk, dv))
    decay = torch.tensor([0.5, 0.97, 1.0], dtype=torch.float32)
    S0 = torch.randn(2, heads, dk, dv, generator=g)
    silu = lambda z: P.silu(z.double())
    want, states, off = [], [], 0
    for i, L in enumerate(lens):
        S = S0[i].double().clone()
        want.append(plain_scan(silu(q[off:off + L]).view(L, heads, dk), silu(k[off:off + L]).view(L, heads, dk),
                               silu(v[off:off + L]).view(L, heads, dv), decay.double(), S).reshape(L, heads * dv))
        states.append(S)
        off += L
    want = torch.cat(want)
    state = torch.zeros(4, heads, dk, dv, device=DEV)
    state[3], state[1] = dev(S0[0]), dev(S0[1])
    slots = dev(torch.tensor([3, 1], dtype=torch.int32))
    cu = dev(torch.tensor([0, 5, n], dtype=torch.int32))
    cuts = [5, 69, 70, 134, 198, 262, 326, n]                    # the long portion's chunks: 64 tokens, one of 1, a last one of 12
    chunks = dev(torch.tensor([(1, a, b, i) for i, (a, b) in enumerate(zip(cuts[:-1], cuts[1:]))], dtype=torch.int32))
    spans = dev(torch.tensor([(1, 0, len(cuts) - 1, 0)], dtype=torch.int32))
    short = dev(torch.tensor([(0, 0, 5, 0)], dtype=torch.int32))
    out = torch.zeros(n, heads * dv, device=DEV)
    scratch = torch.full((len(cuts) - 1, heads, dk, dv), 3.0, device=DEV)
    args = (out, dev(q), dev(k), dev(v), state, dev(decay), cu, slots, 2, heads, dk, dv, "silu")
    kernels.lightning_scan(*args, items=short)
    kernels.lightning_scan(*args, items=chunks, scratch=scratch, mode=1)
    kernels.lightning_prefix(scratch, state, dev(decay), slots, chunks, spans)
    kernels.lightning_scan(*args, items=chunks, scratch=scratch, mode=2)
    tol = 2e-5 if dtype == "float32" else 1e-4
    assert float((out.cpu().double() - want).abs().max()) <= tol * float(want.abs().max())
    for i, s in enumerate([3, 1]):
        assert float((state[s].cpu().double() - states[i]).abs().max()) <= tol * float(states[i].abs().max())
    assert torch.all(state[0] == 0) and torch.all(state[2] == 0)


def test_gated_norm_norms_all_heads_of_a_token_together():
    from lmsf_b200 import kernels
    g = torch.Generator().manual_seed(3)
    x, gate, w = torch.randn(6, 88, generator=g) * 4, torch.randn(6, 200, generator=g), 1 + 0.2 * torch.randn(88, generator=g)
    for dtype, tol in ((torch.float32, 1e-5), (torch.bfloat16, 1e-2)):
        gd = gate.to(dtype)[:, 100:188]                                 # a view into a wider row, as the merged product leaves it
        out = torch.empty(6, 88, dtype=dtype, device=DEV)
        kernels.gated_norm(out, dev(x), dev(gate.to(dtype))[:, 100:188], dev(w), 1e-5)
        want = P.rms_norm(x.double(), w.double(), 1e-5) * P.sigmoid(gd.double())
        assert torch.allclose(out.cpu().double(), want, rtol=tol, atol=tol)


def _paged_latents(c, block_size, n_pages, padded, dtype, rng):
    """Writes the rows of c ([T, padded]) into randomly chosen pages; returns (cache, block table row)."""
    T = c.shape[0]
    n_blocks = (T + block_size - 1) // block_size
    pages = rng.sample(range(n_pages), n_blocks)
    cache = torch.randn(n_pages + 1, 1, 1, block_size, padded).to(dtype) * 50           # rubbish wherever nothing is written
    for t in range(T):
        cache[pages[t // block_size], 0, 0, t % block_size] = c[t]
    return cache, pages


@pytest.mark.parametrize("R", [32, 272])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_over_one_cached_vector_sees_exactly_its_window(dtype, R):
    """One key is made to stand out (a large c aligned with the query); the output must be that key's c when it is the
    oldest key inside the window, and must not contain it when it is one further back; the same at a page border, for a
    key far back without a window, and for the first tokens of a sequence."""
    from lmsf_b200 import kernels
    tdt = TDT[dtype]
    rng = random.Random(5)
    g = torch.Generator().manual_seed(5)
    heads, bs = 3, 8
    T = 300
    for window, qpos, hot in [(9, 100, 92), (9, 100, 91), (16, 47, 32), (16, 47, 31), (8, 15, 8), (8, 15, 7),
                              (0, 299, 3), (0, 299, 0), (5, 2, 0), (1, 40, 40), (1, 40, 39), (72, 271, 200), (72, 271, 199)]:
        c = torch.randn(T, R, generator=g) * 0.1
        direction = torch.randn(R, generator=g)
        direction /= direction.norm()
        c[hot] = 6.0 * direction
        q = (torch.randn(heads, R, generator=g) * 0.1 + 8.0 * direction).to(tdt)
        c = c.to(tdt)
        cache, pages = _paged_latents(c, bs, 60, R, tdt, rng)
        table = torch.full((1, 64), -1, dtype=torch.int32)
        table[0, :len(pages)] = torch.tensor(pages, dtype=torch.int32)
        gate = torch.randn(1, heads, generator=g).to(tdt)
        out = torch.empty(1, heads * R, dtype=tdt, device=DEV)
        kernels.attention_shared_kv(out, dev(q.reshape(1, heads * R)), dev(cache), dev(table), bs, dev(torch.zeros(1, dtype=torch.int32)),
                                    dev(torch.tensor([qpos], dtype=torch.int32)), 0.7, window, heads, R, gate=dev(gate))
        lo = max(0, qpos - window + 1) if window else 0
        keys = c[lo:qpos + 1].double()
        p = torch.softmax((q.double() @ keys.T) * 0.7, dim=-1)
        want = (p @ keys) * P.sigmoid(gate.double()).T
        got = out.cpu().double().view(heads, R)
        tol = 1e-5 if dtype == "float32" else 2e-2
        assert torch.allclose(got, want, rtol=tol, atol=tol), (window, qpos, hot)
        seen = lo <= hot <= qpos
        share = float((got / P.sigmoid(gate.double()).T @ direction.double()).min()) / 6.0
        assert (share > 0.9) == seen, (window, qpos, hot, share)


def test_latent_norm_is_written_to_the_page_of_its_position():
    from lmsf_b200 import kernels
    g = torch.Generator().manual_seed(6)
    R, padded, bs = 24, 32, 8
    x = torch.randn(5, 100, generator=g)
    w = 1 + 0.3 * torch.randn(R, generator=g)
    cache = torch.full((7, 1, 1, bs, padded), 9.0, device=DEV)
    table = torch.tensor([[4, -1, 2], [6, 1, -1]], dtype=torch.int32)
    pos = torch.tensor([7, 16, 23, 0, 9], dtype=torch.int32)
    seq = torch.tensor([0, 0, 0, 1, 1], dtype=torch.int32)
    kernels.latent_norm_cache_write(dev(x)[:, 30:30 + R], dev(w), 1e-5, cache, dev(pos), dev(seq), dev(table), bs, R)
    want = P.rms_norm(x[:, 30:30 + R].double(), w.double(), 1e-5)
    for t, (page, slot) in enumerate([(4, 7), (2, 0), (2, 7), (6, 0), (1, 1)]):
        row = cache[page, 0, 0, slot].cpu().double()
        assert torch.allclose(row[:R], want[t], rtol=1e-5, atol=1e-6) and torch.all(row[R:] == 0)
    assert int((cache == 9.0).sum()) == cache.numel() - 5 * padded


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n,E,top,ff,shared", [(70, 5, 2, 40, 56), (3, 1, 1, 16, 0), (150, 8, 8, 24, 8), (9, 12, 3, 72, 0)])
def test_routed_experts_part(dtype, n, E, top, ff, shared):
    from lmsf_b200.parts.moe import RoutedExperts
    g = torch.Generator().manual_seed(n + E)
    D = 48
    tdt = TDT[dtype]
    f = {"router": {"experts": E, "top": top}, "expert": {"ff": ff}, "shared": {"ff": shared} if shared else None}
    W = {"router": torch.randn(E, D, generator=g) * 0.5, "router.b": torch.randn(E, generator=g)}
    for e in range(E):
        W[f"e{e}.up"], W[f"e{e}.down"] = torch.randn(ff, D, generator=g) / 7, torch.randn(D, ff, generator=g) / 6
    if shared:
        W["shared.up"], W["shared.down"], W["shared.sg"] = torch.randn(shared, D, generator=g) / 7, torch.randn(D, shared, generator=g) / 6, torch.randn(1, D, generator=g)
    W = {k: v.to(tdt) for k, v in W.items()}
    h = torch.randn(n, D, generator=g).to(tdt)
    part = RoutedExperts(hidden_size=D, num_experts=E, top_k=top, expert_size=ff, shared_size=shared)
    weights = {"up": torch.cat([W[f"e{e}.up"] for e in range(E)]), "down": torch.cat([W[f"e{e}.down"] for e in range(E)]),
               "router": torch.cat([W["router"]] + ([W["shared.sg"]] if shared else [])), "router_bias": W["router.b"]}
    if shared:
        weights.update(shared_up=W["shared.up"], shared_down=W["shared.down"])
    part.set_weights({k: dev(v) for k, v in weights.items()})
    part.prepare(tdt, torch.device(DEV))
    got = part.forward(None, dev(h)).cpu().double()
    want = P.moe_feed_forward(h.double(), {k: v.double() for k, v in W.items()}, f)
    tol = 1e-5 if dtype == "float32" else 3e-2
    assert float((got - want).abs().max()) <= tol * float(want.abs().max())


def test_router_picks_the_largest_logits_and_weighs_only_those():
    from lmsf_b200 import kernels
    g = torch.Generator().manual_seed(8)
    for E, top in ((8, 3), (33, 5), (2, 2), (70, 1)):
        z = torch.randn(40, E + 1, generator=g) * 2                       # one more column than experts: not a logit
        b = torch.randn(E, generator=g)
        ids = torch.empty(40, top, dtype=torch.int32, device=DEV)
        wts = torch.empty(40, top, device=DEV)
        kernels.moe_topk(ids, wts, dev(z), dev(b), E)
        val, idx = torch.topk(z[:, :E] + b, top, dim=-1)
        assert torch.equal(ids.cpu().long(), idx)
        assert torch.allclose(wts.cpu(), torch.softmax(val, dim=-1), rtol=1e-5, atol=1e-6)


# ----------------------------------------------------------------------------- whole models through the step function

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["X", "Y", "Z"])
def test_every_way_of_cutting_agrees_with_the_plain_implementation(name, dtype):
    """Whole prompts, prefill then token by token, portions of several sizes down to two tokens, and batches of unequal
    requests with few pages and three state slots (pages and slots are used again)."""
    folder, _ = folder_of(name)
    reqs = requests_for(name, [61, 5, 1, 130, 33, 18, 300 if name == "X" else 77])     # 300: a portion long enough for parallel chunks
    ref = oracle(name, reqs)
    bs = BLOCK[name]
    modes = {"whole": traces.whole(reqs), "decode": traces.whole(reqs, tail=30), "portions": traces.portions(reqs, [2, 7, 3, 16, 2, 29]),
             "pairs": traces.portions(reqs, [2]), "mixed": traces.mixed(reqs, seed=4, max_live=3, tail=10)}
    got = {}
    for mode, steps in modes.items():
        out = traces.run_inprocess(folder, dtype, steps, bs, traces.max_live_tokens(steps, 64), max_live=3)
        got[mode] = traces.collect(steps, out)
        assert len(got[mode]) == sum(len(t) for t in reqs.values())
        assert_close(got[mode], ref, dtype, mode)
    if dtype == "float32":                            # a position's logits do not depend on the cut beyond rounding
        for mode in modes:
            for key, row in got[mode].items():
                assert np.abs(row - got["whole"][key]).max() <= 2e-5 * np.abs(got["whole"][key]).max(), (mode, key)


def test_long_decoding_passes_windows_and_pages_and_replays_graphs():
    """A short prompt, then 150 single tokens: the windows, several pages and the state pass over decoded tokens; the
    decode steps are replayed from a CUDA graph, and must equal the eager steps."""
    from lmsf_b200.engine.factory import build_model
    from lmsf_b200.engine.model_runner import ModelRunner, StepEntry
    folder, _ = folder_of("X")
    reqs = requests_for("X", [160, 158], seed=3)
    ref = oracle("X", reqs)
    model, _, tdt = build_model(folder, "float32", DEV)
    assert all(getattr(p, "graph_safe", False) for p, _ in model.parts_with_specs())
    rows = {}
    for eager in (False, True):
        runner = ModelRunner(model, tdt, torch.device(DEV), 8, num_blocks=16, max_num_seqs=3, enforce_eager=eager)
        mgr = runner.make_cache_manager()
        for rid in reqs:
            mgr.add(rid)
        runner.step([StepEntry(rid, reqs[rid][:8], []) for rid in reqs], mgr)
        got = {rid: [] for rid in reqs}
        for t in range(8, 158):
            lg = runner.step([StepEntry(rid, [reqs[rid][t]], [0]) for rid in reqs], mgr)
            for j, rid in enumerate(reqs):
                got[rid].append(lg[j].cpu().numpy())
        assert (len(runner._graphs) > 0) == (not eager)
        rows[eager] = got
        for rid in reqs:
            mgr.free(rid)
    for rid in reqs:
        scale = float(np.abs(ref[rid]).max())
        for i, (a, b) in enumerate(zip(rows[False][rid], rows[True][rid])):
            assert np.abs(a - ref[rid][8 + i]).max() <= 2e-5 * scale, (rid, i)
            assert np.abs(a - b).max() <= 1e-5 * scale


def test_a_freed_state_slot_starts_from_zero():
    """One state slot: a second request gets the slot of the first, whose state must not leak into it."""
    folder, _ = folder_of("Y")
    reqs = requests_for("Y", [40, 40], seed=9)
    ref = oracle("Y", reqs)
    steps = traces.portions(reqs, [13, 2])
    out = traces.run_inprocess(folder, "float32", steps, 16, 64, max_live=1)
    assert worst_rel(traces.collect(steps, out), ref) <= TOL["float32"]


def test_larger_weights_keep_the_comparison_sharp():
    """With three times the weights the attention and the router are far from uniform; float32 still agrees."""
    folder, _ = folder_of("Z", gain=3.0)
    reqs = requests_for("Z", [90, 17], seed=5)
    ref = oracle("Z", reqs, gain=3.0)
    steps = traces.mixed(reqs, seed=1, max_live=2, tail=6)
    out = traces.run_inprocess(folder, "float32", steps, 16, traces.max_live_tokens(steps, 64), max_live=2)
    assert worst_rel(traces.collect(steps, out), ref) <= 5e-5


def test_the_trace_program_runs_the_design():
    folder, _ = folder_of("Y")
    reqs = requests_for("Y", [30, 9], seed=2)
    ref = oracle("Y", reqs)
    steps = traces.mixed(reqs, seed=3, max_live=2, tail=4)
    out = traces.run_program(folder, "float32", steps, traces.max_live_tokens(steps, 64))
    assert worst_rel(traces.collect(steps, out), ref) <= TOL["float32"]


def test_greedy_generation_through_the_engine():
    """The generation entry point with its scheduler, continuous batching and sampler: greedy tokens in float32 equal
    those of the plain implementation fed its own tokens back."""
    from lmsf_b200 import LLM, SamplingParams
    folder, w = folder_of("X")
    cfg = CONFIGS["X"]
    prompts = [util.random_ids(n, cfg["vocab"], 50 + i) for i, n in enumerate([23, 4, 41])]
    llm = LLM(folder, dtype="float32", block_size=8, num_gpu_blocks=48, max_num_batched_tokens=24, max_num_seqs=3)
    outs = llm.generate(prompt_token_ids=prompts, sampling_params=SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
    for p, o in zip(prompts, outs):
        toks = list(p)
        for _ in range(12):
            lg = P.forward(cfg, w, toks, dtype=torch.float64)[-1]
            top2 = torch.topk(lg, 2).values
            nxt = int(lg.argmax())
            got = o.outputs[0].token_ids[len(toks) - len(p)]
            if got != nxt:                             # only a near tie may be decided otherwise
                assert float(top2[0] - lg[got]) <= 1e-4 * float(lg.abs().max())
            toks.append(got)


# ----------------------------------------------------------------------------- the tensor-core attention kernels on a cache of one plane

def _hand_made_context(seqs, block_size, n_pages, rng, window):
    """A StepContext for requests [(cached tokens, new tokens)] with randomly chosen pages; pages that the window has
    passed before the step are given back (-1), as the cache manager does."""
    from lmsf_b200.parts.base import CacheGroupView, StepContext
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    pos, tseq, cu, ctx_lens, q_lens = [], [], [0], [], []
    max_blocks = max((s + n + block_size - 1) // block_size for s, n in seqs)
    table = torch.full((len(seqs), max_blocks), -1, dtype=torch.int32)
    free = list(range(n_pages))
    rng.shuffle(free)
    for i, (start, n) in enumerate(seqs):
        pos += list(range(start, start + n))
        tseq += [i] * n
        cu.append(cu[-1] + n)
        ctx_lens.append(start + n)
        q_lens.append(n)
        first_seen = max(0, start - window + 1) if window else 0
        for b in range((start + n + block_size - 1) // block_size):
            if (b + 1) * block_size > first_seen:
                table[i, b] = free.pop()
    dec = [i for i, (_, n) in enumerate(seqs) if n == 1]
    tiles = lambda size: [(i, q0) for i, (_, n) in enumerate(seqs) if n > 1 for q0 in range(0, n, size)]
    t64, t128 = tiles(64), tiles(128)
    return StepContext(n_tokens=len(pos), n_seqs=len(seqs), dtype=torch.bfloat16, device=torch.device(DEV), token_ids=i32([0] * len(pos)),
                       positions=i32(pos), token_seq=i32(tseq), cu_q=i32(cu), ctx_len=i32(ctx_lens), state_slot=i32([0] * len(seqs)),
                       groups=[CacheGroupView(table.to(DEV), block_size)], q_lens=q_lens, ctx_lens=ctx_lens, state_slots=[0] * len(seqs),
                       error_flag=torch.zeros(1, dtype=torch.int32, device=DEV), decode_seq_ids=i32(dec or [0]), n_decode_seqs=len(dec),
                       q_tile_seq=i32([t[0] for t in t64] or [0]), q_tile_q0=i32([t[1] for t in t64] or [0]), n_q_tiles=len(t64),
                       q_tile128_seq=i32([t[0] for t in t128] or [0]), q_tile128_q0=i32([t[1] for t in t128] or [0]), n_q_tiles128=len(t128))


@pytest.mark.parametrize("rank,heads,window,block_size", [(64, 4, 72, 16), (24, 3, 9, 8), (128, 5, 40, 16), (48, 2, None, 16), (64, 17, 130, 32)])
def test_tensor_core_attention_on_one_cached_vector_agrees_with_the_plain_kernel(rank, heads, window, block_size):
    """Prompt portions (from the start, from the middle of a window, across several query tiles) and single tokens (just
    past a window, at a page's first and last slot, at position 0) in one batch: the split-key decode kernel and the tiled
    prefill kernels read the cache's one plane as key and as value; the plain kernel is their twin."""
    from lmsf_b200 import kernels
    from lmsf_b200.parts.latent_attention import LatentAttention
    rng = random.Random(rank + heads)
    g = torch.Generator().manual_seed(rank * 7 + heads)
    part = LatentAttention(hidden_size=32, num_heads=heads, head_dim=16, value_dim=16, kv_rank=rank, eps=1e-5, scale=0.3, window=window)
    Rp = part.padded_rank
    w = window or 0
    seqs = [(0, 150), (37, 90), (w + 3, 1), (2 * block_size - 1, 1), (2 * block_size, 1), (0, 1), (200, 2), (max(w - 1, 1), 1), (500, 1)]
    for batch in (seqs, [s for s in seqs if s[1] == 1], [s for s in seqs if s[1] > 1]):
        ctx = _hand_made_context(batch, block_size, 200, rng, window)
        cache = (torch.randn(201, 1, 1, block_size, Rp, generator=g) * 0.7).bfloat16().to(DEV)
        cache[..., rank:] = 0
        q = torch.randn(ctx.n_tokens, heads * Rp, generator=g).bfloat16().to(DEV)
        gate = torch.randn(ctx.n_tokens, heads, generator=g).bfloat16().to(DEV)
        fast, plain = torch.zeros_like(q), torch.zeros_like(q)
        part.attend(ctx, fast, q, cache, ctx.groups[0], gate)
        kernels.attention_shared_kv(plain, q, cache, ctx.groups[0].block_table, block_size, ctx.token_seq, ctx.positions, 0.3, w, heads, Rp, gate=gate)
        assert int(ctx.error_flag.item()) == 0
        diff = (fast.float() - plain.float()).abs().max(dim=1).values.cpu()
        assert float(diff.max()) <= 2e-2 * float(plain.float().abs().max()), (len(batch), int(diff.argmax()), float(diff.max()))


# ----------------------------------------------------------------------------- random configurations

def random_config(seed):
    """Sizes that are no multiples of anything in particular: widths that 8 does not divide, odd head counts, ranks and
    windows around page borders, every optional piece present or absent by chance."""
    rng = random.Random(seed)
    width = rng.choice([36, 50, 72, 100, 136])
    layers = []
    for _ in range(rng.randint(2, 4)):
        heads = rng.randint(1, 5)
        mlp = None
        if rng.random() < 0.8:
            experts = rng.randint(1, 9)
            mlp = moe(experts, rng.randint(1, experts), rng.choice([8, 12, 20, 40]), rng.choice([0, 0, 10, 24]))
        if rng.random() < 0.5:
            layer = lightning(heads, rng.choice([4, 10, 16, 36]), rng.choice([6, 16, 33, 70]),
                              [rng.choice([0.3, 0.8, 0.95, 0.999, 1.0]) for _ in range(heads)])
        else:
            layer = latent(heads, rng.choice([4, 12, 16, 40]), rng.choice([6, 16, 24]), rng.choice([8, 20, 32, 48, 130]),
                           rng.choice([None, 1, 3, 8, 17, 33]), rng.choice([0.1, 0.3, 0.6]))
        layers.append(with_mlp(layer, mlp))
    cfg = {"architecture": "Vufolorn", "vocab": rng.choice([61, 128, 257]), "width": width,
           "norm": {"eps": rng.choice([1e-6, 1e-5, 1e-3])}, "layers": layers}
    if rng.random() < 0.7:
        start = rng.randint(0, len(layers) - 1)
        cfg["loop"] = {"start": start, "stop": rng.randint(start + 1, len(layers)), "times": rng.randint(1, 3)}
    return cfg


@pytest.mark.parametrize("seed", range(8))
def test_random_configurations(seed):
    name = f"R{seed}"
    CONFIGS[name] = random_config(seed)
    folder, _ = folder_of(name)
    rng = random.Random(seed)
    reqs = requests_for(name, [rng.randint(1, 70) for _ in range(4)], seed=seed)
    ref = oracle(name, reqs)
    bs = rng.choice([8, 16, 32])
    for dtype in ("float32", "bfloat16"):
        for steps in (traces.whole(reqs, tail=5), traces.mixed(reqs, seed=seed, max_live=2, tail=4)):
            out = traces.run_inprocess(folder, dtype, steps, bs, traces.max_live_tokens(steps, 64), max_live=2)
            rows = traces.collect(steps, out)
            if dtype == "float32":
                assert worst_rel(rows, ref) <= 5e-5, (CONFIGS[name], worst_rel(rows, ref))
            else:
                e = position_errors(rows, ref)
                assert e[len(e) // 2] <= 2e-2, (CONFIGS[name], e[len(e) // 2])
