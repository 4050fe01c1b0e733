"""Tiny Redarax configurations for the tests: sizes that share nothing with each other, every branch of the design."""


def attention(heads, kv_heads, dim, vdim, scale, rot_dims=None, base=10000.0):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot_dims:
        m["rot"] = {"dims": rot_dims, "base": base}
    return {"type": "attention", "mixer": m}


def mamba2(heads, vdim, state, groups, norm_groups, conv):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups,
                                        "norm_groups": norm_groups, "conv": conv}}


def delta(heads, kv_heads, dim, vdim, conv):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts, top, ff, limit, count=None, keep=None):
    r = {"experts": experts, "top": top}
    if count:
        r["groups"] = {"count": count, "keep": keep}
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": r}


def layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


# X: key and value sizes that differ and are no multiple of 16, a partial rotation, several groups of B and C, a norm in
# three parts, query/key heads shared by several heads of the delta rule, a layer without feed-forward, groups of experts
# of which two are kept, taps from 2 to 4
CFG_X = {"architecture": "Redarax", "vocab": 211, "width": 72, "norm": {"eps": 1e-5}, "residual_mult": 0.6,
         "token_side": {"dim": 6}, "logit_scale": 1.7, "logit_softcap": 9.0,
         "layers": [layer(delta(4, 2, 12, 20, 2), moe(6, 2, 24, 1.2, 3, 2)),
                    layer(attention(6, 2, 24, 8, 0.21, 10, 7000.0), dense(56, 2.0)),
                    layer(mamba2(6, 12, 10, 2, 3, 4), None),
                    layer(attention(3, 3, 16, 40, 0.3, 16, 300.0), moe(8, 3, 16, 0.8, 4, 2)),
                    layer(delta(3, 3, 20, 8, 3), dense(40, 0.7))]}
# Y: no side branch, no cap and no scale on the logits, a factor of 1, one head, one expert, one group, a convolution of one
# tap, attention without rotation, another eps
CFG_Y = {"architecture": "Redarax", "vocab": 97, "width": 40, "norm": {"eps": 1e-3}, "residual_mult": 1.0,
         "layers": [layer(mamba2(1, 24, 7, 1, 1, 1), moe(1, 1, 16, 3.0)),
                    layer(attention(1, 1, 32, 32, 0.18), moe(4, 4, 8, 1.0, 2, 2)),
                    layer(delta(1, 1, 9, 5, 4), dense(24, 1.5)),
                    layer(attention(4, 2, 8, 8, 0.5, 2, 50.0), None)]}
# Z: heads as wide as the tensor-core attention kernels take them whole, states of more than 64 rows, groups of one expert
CFG_Z = {"architecture": "Redarax", "vocab": 130, "width": 64, "norm": {"eps": 1e-6}, "residual_mult": 0.35,
         "token_side": {"dim": 16}, "logit_scale": 0.8, "logit_softcap": 30.0,
         "layers": [layer(attention(4, 2, 64, 64, 0.125, 32, 1.0e6), moe(5, 2, 16, 1.5, 5, 3)),
                    layer(mamba2(4, 16, 72, 2, 1, 3), dense(48, 1.0)),
                    layer(delta(2, 1, 80, 48, 4), moe(4, 1, 24, 2.5, 2, 1)),
                    layer(mamba2(2, 40, 16, 1, 2, 2), moe(6, 2, 8, 1.0))]}
CONFIGS = {"X": CFG_X, "Y": CFG_Y, "Z": CFG_Z}
BLOCK = {"X": 8, "Y": 16, "Z": 16}
