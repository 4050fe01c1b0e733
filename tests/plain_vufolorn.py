"""A plain, slow implementation of the Vufolorn design on whole sequences: one function per mechanism, float64 or
float32 on the CPU, no cache, no batching, nothing shared with the package.  The tests compare the engine with it.

A model is (config dict, {tensor name: tensor}).  Notation: T tokens, D width, x the residual stream [T, D].
"""
import math

import torch


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last dimension."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def silu(z):
    return z / (1 + torch.exp(-z))


def sigmoid(z):
    return 1 / (1 + torch.exp(-z))


def relu_squared(z):
    return torch.clamp(z, min=0) ** 2


def lightning_mixer(h, W, m, eps):
    """Linear attention with a decay per head.  S_t = a S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, token by token."""
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ W["q"].T).reshape(T, H, dk)
    k = silu(h @ W["k"].T).reshape(T, H, dk)
    v = silu(h @ W["v"].T).reshape(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hd in range(H):
        a = float(m["decay"][hd])
        S = torch.zeros(dk, dv, dtype=h.dtype)
        for t in range(T):
            S = a * S + torch.outer(k[t, hd], v[t, hd])
            out[t, hd] = S.T @ q[t, hd]
    o = rms_norm(out.reshape(T, H * dv), W["norm"], eps)
    o = o * sigmoid(h @ W["g"].T)
    return o @ W["o"].T


def latent_attention_mixer(h, W, m, eps):
    """Attention whose keys and values are expanded from one low-rank vector per token; a sliding window of
    m['mask']['size'] keys (the query's own among them); a sigmoid gate per head; no positions."""
    T = h.shape[0]
    H, dk, dv, r = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
    q = (h @ W["q"].T).reshape(T, H, dk)
    c = rms_norm(h @ W["dkv"].T, W["dkv.norm"], eps)
    k = (c @ W["uk"].T).reshape(T, H, dk)
    v = (c @ W["uv"].T).reshape(T, H, dv)
    window = (m.get("mask") or {}).get("size")
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = j <= i
    if window:
        seen = seen & (i - j < window)
    gate = sigmoid(h @ W["g"].T)                       # [T, H]
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hd in range(H):
        s = (q[:, hd] @ k[:, hd].T) * m["scale"]
        s = s.masked_fill(~seen, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, hd] = (p @ v[:, hd]) * gate[:, hd:hd + 1]
    return out.reshape(T, H * dv) @ W["o"].T


def expert(h, up, down):
    return relu_squared(h @ up.T) @ down.T


def moe_feed_forward(h, W, f):
    """Routed experts (softmax over the chosen logits only) plus a shared expert behind a sigmoid gate per token."""
    E, top = f["router"]["experts"], f["router"]["top"]
    z = h @ W["router"].T + W["router.b"]
    val, idx = torch.topk(z, top, dim=-1)
    wgt = torch.softmax(val, dim=-1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            out[t] += wgt[t, j] * expert(h[t:t + 1], W[f"e{e}.up"], W[f"e{e}.down"])[0]
    if f.get("shared"):
        out = out + expert(h, W["shared.up"], W["shared.down"]) * sigmoid(h @ W["shared.sg"].T)
    return out


def sub(weights, prefix):
    n = len(prefix)
    return {k[n:]: v for k, v in weights.items() if k.startswith(prefix)}


def layer(x, cfg, weights, i):
    L, eps = cfg["layers"][i], cfg["norm"]["eps"]
    W = sub(weights, f"l{i}.")
    h = rms_norm(x, W["norm1"], eps)
    mix = {"lightning": lightning_mixer, "latent_attention": latent_attention_mixer}[L["type"]]
    a = mix(h, sub(W, "mix."), L["mixer"], eps)
    x = x + rms_norm(a, W["norm1b"], eps) * W["ls1"]
    if L.get("mlp"):
        h = rms_norm(x, W["norm2"], eps)
        f = moe_feed_forward(h, sub(W, "mlp."), L["mlp"])
        x = x + rms_norm(f, W["norm2b"], eps) * W["ls2"]
    return x


def run_order(cfg):
    """[(layer, pass number or None, whether a pass starts here)]: the layers in the order they run; the span that
    runs several times is repeated."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop or loop["times"] < 1 or loop["stop"] <= loop["start"]:
        return [(i, None, False) for i in range(n)]
    order = [(i, None, False) for i in range(loop["start"])]
    for t in range(loop["times"]):
        order += [(i, t, i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    order += [(i, None, False) for i in range(loop["stop"], n)]
    return order


def forward(cfg, weights, tokens, dtype=torch.float64, streams=None):
    """Logits [T, vocab] of one whole sequence.  `streams`, a list, receives the residual stream after every layer run."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x = rms_norm(W["embed"][torch.tensor(tokens)], W["embed.norm"], eps)
    x0 = x
    for i, t, first in run_order(cfg):
        if first:
            if t > 0:
                x = x + x0
            x = x + W["loop.step"][t]
        x = layer(x, cfg, W, i)
        if streams is not None:
            streams.append(x)
    return rms_norm(x, W["final.norm"], eps) @ W["embed"].T


# ----------------------------------------------------------------------------- random models of this design

def tensor_shapes(cfg):
    D, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, D), "embed.norm": (D,), "final.norm": (D,)}
    if cfg.get("loop"):
        out["loop.step"] = (cfg["loop"]["times"], D)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        for n in ("norm1", "norm1b", "ls1"):
            out[p + n] = (D,)
        H, dk, dv = m["heads"], m["dim"], m["vdim"]
        if L["type"] == "lightning":
            out.update({p + "mix.q": (H * dk, D), p + "mix.k": (H * dk, D), p + "mix.v": (H * dv, D),
                        p + "mix.g": (H * dv, D), p + "mix.o": (D, H * dv), p + "mix.norm": (H * dv,)})
        else:
            r = m["kv_rank"]
            out.update({p + "mix.q": (H * dk, D), p + "mix.dkv": (r, D), p + "mix.dkv.norm": (r,),
                        p + "mix.uk": (H * dk, r), p + "mix.uv": (H * dv, r), p + "mix.g": (H, D), p + "mix.o": (D, H * dv)})
        f = L.get("mlp")
        if f:
            for n in ("norm2", "norm2b", "ls2"):
                out[p + n] = (D,)
            for e in range(f["router"]["experts"]):
                out[p + f"mlp.e{e}.up"] = (f["expert"]["ff"], D)
                out[p + f"mlp.e{e}.down"] = (D, f["expert"]["ff"])
            out[p + "mlp.router"] = (f["router"]["experts"], D)
            out[p + "mlp.router.b"] = (f["router"]["experts"],)
            if f.get("shared"):
                out[p + "mlp.shared.up"] = (f["shared"]["ff"], D)
                out[p + "mlp.shared.down"] = (D, f["shared"]["ff"])
                out[p + "mlp.shared.sg"] = (1, D)
    return out


def random_weights(cfg, seed, dtype=torch.bfloat16, gain=1.0):
    """Matrices N(0, gain^2 / fan_in); norm weights and layer scales near 1; router biases and loop vectors small."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.rsplit(".", 1)[-1]
        if len(shape) == 1 and (last.startswith("norm") or last in ("ls1", "ls2")):
            t = 1 + 0.2 * torch.randn(shape, generator=g)
        elif name.endswith("router.b"):
            t = 0.3 * torch.randn(shape, generator=g)
        elif name in ("embed", "loop.step"):
            t = torch.randn(shape, generator=g) * (1.0 if name == "embed" else 0.3)
        else:
            t = torch.randn(shape, generator=g) * gain / math.sqrt(shape[-1])
        out[name] = t.to(dtype)
    return out
