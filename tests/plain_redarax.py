"""A plain, slow implementation of the Redarax design on whole sequences: one function per mechanism, float64 or
float32 on the CPU, no cache, no batching, nothing shared with the package.  The tests compare the engine with it.

A model is (config dict, {tensor name: tensor}).  Notation: T tokens, D width, x the residual stream [T, D].
"""
import math

import torch


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last dimension (w may be None)."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def silu(z):
    return z / (1 + torch.exp(-z))


def sigmoid(z):
    return 1 / (1 + torch.exp(-z))


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate_interleaved(x, positions, dims, base):
    """x [T, heads, dim]: the first `dims` values of every head are rotated in pairs (2i, 2i + 1) by the angle
    position * base^(-2i / dims); the rest pass."""
    out = x.clone()
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=x.dtype)
    a = positions.to(x.dtype)[:, None] * f[None, :]                      # [T, half]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def causal_conv(x, w, b=None):
    """x [T, C], w [C, taps]: y_t = sum_j w[:, j] * x_(t - (taps - 1) + j), zeros before the start."""
    T, C = x.shape
    taps = w.shape[1]
    xp = torch.cat([torch.zeros(taps - 1, C, dtype=x.dtype), x], 0)
    y = torch.zeros(T, C, dtype=x.dtype)
    for j in range(taps):
        y = y + xp[j:j + T] * w[:, j]
    return y if b is None else y + b


def attention_mixer(h, W, m, eps, positions=None):
    """Causal softmax attention with grouped key/value heads, biases, a norm of q and k per head and a partial rotation."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    positions = torch.arange(T) if positions is None else positions
    q = (h @ W["q"].T + W["q.b"]).reshape(T, H, dk)
    k = (h @ W["k"].T + W["k.b"]).reshape(T, G, dk)
    v = (h @ W["v"].T + W["v.b"]).reshape(T, G, dv)
    q = rms_norm(q, W["q.norm"], eps)
    k = rms_norm(k, W["k.norm"], eps)
    rot = m.get("rot")
    if rot:
        q = rotate_interleaved(q, positions, rot["dims"], rot["base"])
        k = rotate_interleaved(k, positions, rot["dims"], rot["base"])
    seen = torch.arange(T)[None, :] <= torch.arange(T)[:, None]
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * m["scale"]
        s = s.masked_fill(~seen, float("-inf"))
        p = torch.softmax(s, -1)
        out[:, hd] = p @ v[:, g]
    return out.reshape(T, H * dv) @ W["o"].T + W["o.b"]


def mamba2_mixer(h, W, m, eps):
    """A selective state-space layer with one scalar decay per head and token."""
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    p = h @ W["in"].T
    z, xbc, dt = p[:, :inner], p[:, inner:2 * inner + 2 * G * N], p[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, W["conv"], W["conv.b"]))
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + W["dt_bias"])                                     # [T, H]
    A = torch.exp(W["A_log"])
    y = torch.zeros(T, H, P, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        S = torch.zeros(N, P, dtype=h.dtype)
        for t in range(T):
            S = torch.exp(-A[hd] * dt[t, hd]) * S + dt[t, hd] * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = S.T @ C[t, g] + W["D"][hd] * x[t, hd]
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = rms_norm(y.reshape(T, parts, inner // parts), None, eps).reshape(T, inner) * W["norm"]
    return y @ W["o"].T


def delta_mixer(h, W, m, eps):
    """The gated delta rule: the state forgets by a factor, then is corrected towards v along k, then is read."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ W["q"].T, W["q.conv"])).reshape(T, G, dk)
    k = silu(causal_conv(h @ W["k"].T, W["k.conv"])).reshape(T, G, dk)
    v = silu(causal_conv(h @ W["v"].T, W["v.conv"])).reshape(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = sigmoid(h @ W["b"].T)                                         # [T, H]
    decay = torch.exp(-torch.exp(W["A_log"]) * softplus(h @ W["a"].T + W["dt_bias"]))
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        S = torch.zeros(dk, dv, dtype=h.dtype)
        for t in range(T):
            S = decay[t, hd] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            o[t, hd] = S.T @ q[t, g]
    o = rms_norm(o, W["norm"], eps).reshape(T, H * dv)
    o = o * silu(h @ W["g"].T)
    return o @ W["o"].T


def clamped_glu(h, gate, up, down, limit):
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, min=-limit, max=limit)
    return (g * sigmoid(1.702 * g) * (u + 1)) @ down.T


def route(h, W, r):
    """(chosen experts [T, top], their weights [T, top]).  Choice by sigmoid score + correction inside the kept
    groups of neighbouring experts; a group's score is the sum of its two largest choice scores; the weights are the
    sigmoid scores themselves."""
    T = h.shape[0]
    E, top = r["experts"], r["top"]
    s = sigmoid(h @ W["router"].T)
    c = s + W["correction"]
    groups = r.get("groups")
    if groups and groups["count"] > 1:
        n, keep = groups["count"], groups["keep"]
        cg = c.reshape(T, n, E // n)
        gs = cg.topk(min(2, E // n), -1).values.sum(-1)                  # [T, n]
        best = gs.topk(keep, -1).indices
        allowed = torch.zeros(T, n, dtype=torch.bool)
        allowed.scatter_(1, best, True)
        c = torch.where(allowed[:, :, None].expand(T, n, E // n).reshape(T, E), c, torch.full_like(c, float("-inf")))
    ids = c.topk(top, -1).indices
    return ids, s.gather(1, ids)


def moe(h, W, f):
    r = f["router"]
    ids, wts = route(h, W, r)
    out = torch.zeros(h.shape[0], W["e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for e, w in zip(ids[t].tolist(), wts[t]):
            out[t] += w * clamped_glu(h[t:t + 1], W[f"e{e}.gate"], W[f"e{e}.up"], W[f"e{e}.down"], f["expert"]["limit"])[0]
    return out


def feed_forward(h, W, f):
    if f["kind"] == "dense":
        return clamped_glu(h, W["gate"], W["up"], W["down"], f["limit"])
    return moe(h, W, f)


def sub(weights, prefix):
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(config, weights, tokens, dtype=torch.float64, layers_out=None):
    """Logits [T, vocab] of one sequence.  layers_out: a list that receives the stream after every layer."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps, m = config["norm"]["eps"], config["residual_mult"]
    tok = torch.as_tensor(tokens, dtype=torch.long)
    x = W["embed"][tok]
    side = config.get("token_side")
    for i, L in enumerate(config["layers"]):
        p = f"l{i}."
        mix = {"attention": attention_mixer, "mamba2": mamba2_mixer, "delta": delta_mixer}[L["type"]]
        x = x + m * rms_norm(mix(x, sub(W, p + "mix."), L["mixer"], eps), W[p + "norm1"], eps)
        if L.get("mlp"):
            x = x + m * rms_norm(feed_forward(x, sub(W, p + "mlp."), L["mlp"]), W[p + "norm2"], eps)
        if side:
            d = side["dim"]
            e = W["side.embed"][tok][:, i * d:(i + 1) * d]
            y = (gelu_tanh(x @ W[p + "side.gate"].T) * e) @ W[p + "side.proj"].T
            x = x + m * rms_norm(y, W[p + "side.norm"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    h = rms_norm(x, W["final.norm"], eps)
    logits = (h @ W["head"].T) * config.get("logit_scale", 1.0)
    cap = config.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits


def tensor_shapes(config):
    """{name: shape} of every tensor a model of this configuration stores."""
    D, V = config["width"], config["vocab"]
    out = {"embed": (V, D), "final.norm": (D,), "head": (V, D)}
    side = config.get("token_side")
    if side:
        out["side.embed"] = (V, side["dim"] * len(config["layers"]))
    for i, L in enumerate(config["layers"]):
        p, m = f"l{i}.", L["mixer"]
        out[p + "norm1"] = (D,)
        if L["type"] == "attention":
            H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out.update({p + "mix.q": (H * dk, D), p + "mix.q.b": (H * dk,), p + "mix.k": (G * dk, D), p + "mix.k.b": (G * dk,),
                        p + "mix.v": (G * dv, D), p + "mix.v.b": (G * dv,), p + "mix.q.norm": (dk,), p + "mix.k.norm": (dk,),
                        p + "mix.o": (D, H * dv), p + "mix.o.b": (D,)})
        elif L["type"] == "mamba2":
            H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
            ch = H * P + 2 * G * N
            out.update({p + "mix.in": (2 * H * P + 2 * G * N + H, D), p + "mix.conv": (ch, m["conv"]), p + "mix.conv.b": (ch,),
                        p + "mix.dt_bias": (H,), p + "mix.A_log": (H,), p + "mix.D": (H,), p + "mix.norm": (H * P,),
                        p + "mix.o": (D, H * P)})
        else:
            H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out.update({p + "mix.q": (G * dk, D), p + "mix.q.conv": (G * dk, m["conv"]), p + "mix.k": (G * dk, D),
                        p + "mix.k.conv": (G * dk, m["conv"]), p + "mix.v": (H * dv, D), p + "mix.v.conv": (H * dv, m["conv"]),
                        p + "mix.b": (H, D), p + "mix.a": (H, D), p + "mix.A_log": (H,), p + "mix.dt_bias": (H,),
                        p + "mix.norm": (dv,), p + "mix.g": (H * dv, D), p + "mix.o": (D, H * dv)})
        f = L.get("mlp")
        if f:
            out[p + "norm2"] = (D,)
            if f["kind"] == "dense":
                out.update({p + "mlp.gate": (f["ff"], D), p + "mlp.up": (f["ff"], D), p + "mlp.down": (D, f["ff"])})
            else:
                E, F = f["router"]["experts"], f["expert"]["ff"]
                for e in range(E):
                    out.update({p + f"mlp.e{e}.gate": (F, D), p + f"mlp.e{e}.up": (F, D), p + f"mlp.e{e}.down": (D, F)})
                out.update({p + "mlp.router": (E, D), p + "mlp.correction": (E,)})
        if side:
            out.update({p + "side.gate": (side["dim"], D), p + "side.proj": (D, side["dim"]), p + "side.norm": (D,)})
    return out


def random_weights(config, seed=0, dtype=torch.bfloat16, gain=1.0):
    """Random weights of a size that keeps every branch alive: matrices N(0, gain^2 / fan-in), norm weights near 1, decays
    and step sizes spread over their useful range, corrections and biases small but not zero."""
    g = torch.Generator().manual_seed(seed)
    rnd = lambda *s: torch.randn(*s, generator=g)
    uni = lambda n, lo, hi: lo + (hi - lo) * torch.rand(n, generator=g)
    out = {}
    for name, shape in tensor_shapes(config).items():
        leaf = name.split(".", 1)[1] if name.startswith("l") and name[1].isdigit() else name
        if leaf in ("norm1", "norm2", "final.norm", "side.norm", "mix.norm", "mix.q.norm", "mix.k.norm"):
            t = 1.0 + 0.2 * rnd(*shape)
        elif leaf == "mix.A_log":
            t = torch.log(uni(shape[0], 0.3, 4.0))
        elif leaf == "mix.dt_bias":
            t = uni(shape[0], -3.0, 0.5)
        elif leaf == "mix.D":
            t = 1.0 + 0.3 * rnd(*shape)
        elif leaf == "mlp.correction":
            t = 0.2 * rnd(*shape)
        elif leaf.endswith(".b") and len(shape) == 1:
            t = 0.2 * rnd(*shape)
        elif leaf.endswith("conv"):
            t = 0.6 * rnd(*shape)
        elif leaf in ("embed", "side.embed"):
            t = rnd(*shape)
        else:
            t = rnd(*shape) * gain / math.sqrt(shape[-1])
        out[name] = t.to(dtype)
    return out
