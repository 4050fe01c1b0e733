"""The typed configuration of the Redarax design, read from config.json.

config.json of this design is nested: `layers` lists every layer with its `type` (which of three mixers: `attention`,
`mamba2`, `delta`), the mixer's sizes (`mixer`) and its feed-forward (`mlp`: `kind` dense or moe, or null for none);
`norm.eps`, `residual_mult`, `token_side.dim`, `logit_scale`, `logit_softcap`, `vocab` and `width` are global.  Every
size and every constant that may differ between models of the design is read from there; nothing is assumed equal
between layers.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .model_config import ConfigError
from .vufolorn_config import _need, _pos_int

MIXER_TYPES = ("attention", "mamba2", "delta")


def _number(v, what: str, positive: bool = True) -> float:
    if isinstance(v, bool) or not isinstance(v, (int, float)) or (positive and not v > 0):
        raise ConfigError(f"config.json: {what} must be a {'positive ' if positive else ''}number, got {v!r}")
    return float(v)


@dataclass
class RedaraxMixer:
    type: str
    heads: int
    vdim: int
    dim: int = 0                      # attention, delta: size of a query/key head
    kv_heads: int = 0                 # attention: key/value heads; delta: query/key heads
    scale: float = 0.0                # attention
    rot_dims: int = 0                 # attention: 0 = no rotation
    rot_base: float = 10000.0
    conv: int = 0                     # mamba2, delta: taps of the short convolution
    state: int = 0                    # mamba2
    groups: int = 1                   # mamba2: groups of B and C
    norm_groups: int = 1              # mamba2


@dataclass
class RedaraxFeedForward:
    kind: str                         # "dense" or "moe"
    ff: int
    limit: float
    experts: int = 0
    top: int = 0
    groups: int = 1
    keep: int = 1


@dataclass
class RedaraxLayer:
    mixer: RedaraxMixer
    mlp: Optional[RedaraxFeedForward]


@dataclass
class RedaraxConfig:
    vocab: int
    width: int
    eps: float
    residual_mult: float
    layers: List[RedaraxLayer]
    side_dim: int = 0                 # 0: no side branch
    logit_scale: float = 1.0
    logit_softcap: float = 0.0        # 0: no cap
    max_model_len: int = 1 << 20      # angles are computed from the position: bounded by the cache alone
    torch_dtype: str = "bfloat16"
    eos_token_ids: List[int] = field(default_factory=list)
    raw: Dict[str, Any] = field(default_factory=dict)

    @staticmethod
    def from_dict(d: Dict[str, Any]) -> "RedaraxConfig":
        vocab = _pos_int(_need(d, "vocab", "the model"), "vocab")
        width = _pos_int(_need(d, "width", "the model"), "width")
        eps = _number(_need(_need(d, "norm", "the model"), "eps", "norm"), "norm.eps")
        mult = _number(d.get("residual_mult", 1.0), "residual_mult", positive=False)
        raw_layers = _need(d, "layers", "the model")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, L in enumerate(raw_layers):
            where = f"layers[{i}]"
            kind = _need(L, "type", where)
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of this design ({', '.join(MIXER_TYPES)})")
            m, wm = _need(L, "mixer", where), where + ".mixer"
            mixer = RedaraxMixer(kind, _pos_int(_need(m, "heads", wm), "heads"), _pos_int(_need(m, "vdim", wm), "vdim"))
            if kind in ("attention", "delta"):
                mixer.dim = _pos_int(_need(m, "dim", wm), "dim")
                mixer.kv_heads = _pos_int(_need(m, "kv_heads", wm), "kv_heads")
                if mixer.heads % mixer.kv_heads:
                    raise ConfigError(f"config.json: {wm}: {mixer.heads} heads cannot be grouped over {mixer.kv_heads} kv_heads")
            if kind == "attention":
                mixer.scale = _number(_need(m, "scale", wm), "scale")
                rot = m.get("rot")
                if rot:
                    mixer.rot_dims = _pos_int(_need(rot, "dims", wm + ".rot"), "rot.dims")
                    mixer.rot_base = _number(_need(rot, "base", wm + ".rot"), "rot.base")
                    if mixer.rot_dims % 2 or mixer.rot_dims > mixer.dim:
                        raise ConfigError(f"config.json: {wm}.rot.dims {mixer.rot_dims} must be even and at most dim {mixer.dim}")
            else:
                mixer.conv = _pos_int(_need(m, "conv", wm), "conv")
            if kind == "mamba2":
                mixer.state = _pos_int(_need(m, "state", wm), "state")
                mixer.groups = _pos_int(m.get("groups", 1), "groups")
                mixer.norm_groups = _pos_int(m.get("norm_groups", 1), "norm_groups")
                if mixer.heads % mixer.groups or (mixer.heads * mixer.vdim) % mixer.norm_groups:
                    raise ConfigError(f"config.json: {wm}: groups {mixer.groups} / norm_groups {mixer.norm_groups} do not divide "
                                      f"{mixer.heads} heads of {mixer.vdim}")
            f = L.get("mlp")
            mlp = None
            if f:
                wf = where + ".mlp"
                kind_f = _need(f, "kind", wf)
                if kind_f == "dense":
                    mlp = RedaraxFeedForward("dense", _pos_int(_need(f, "ff", wf), "ff"), _number(_need(f, "limit", wf), "limit"))
                elif kind_f == "moe":
                    ex, r = _need(f, "expert", wf), _need(f, "router", wf)
                    mlp = RedaraxFeedForward("moe", _pos_int(_need(ex, "ff", wf + ".expert"), "ff"),
                                             _number(_need(ex, "limit", wf + ".expert"), "limit"),
                                             _pos_int(_need(r, "experts", wf + ".router"), "experts"),
                                             _pos_int(_need(r, "top", wf + ".router"), "top"))
                    g = r.get("groups")
                    if g:
                        mlp.groups = _pos_int(_need(g, "count", wf + ".router.groups"), "groups.count")
                        mlp.keep = _pos_int(_need(g, "keep", wf + ".router.groups"), "groups.keep")
                    if mlp.experts % mlp.groups or mlp.keep > mlp.groups or mlp.top > mlp.keep * (mlp.experts // mlp.groups):
                        raise ConfigError(f"config.json: {wf}.router: {mlp.experts} experts in {mlp.groups} groups of which "
                                          f"{mlp.keep} are kept cannot give {mlp.top} choices")
                else:
                    raise ConfigError(f"config.json: {wf}.kind {kind_f!r} is not a feed-forward of this design (dense, moe)")
            layers.append(RedaraxLayer(mixer, mlp))
        cfg = RedaraxConfig(vocab, width, eps, mult, layers, raw=dict(d))
        side = d.get("token_side")
        if side:
            cfg.side_dim = _pos_int(_need(side, "dim", "token_side"), "token_side.dim")
        if d.get("logit_scale") is not None:
            cfg.logit_scale = _number(d["logit_scale"], "logit_scale")
        if d.get("logit_softcap"):
            cfg.logit_softcap = _number(d["logit_softcap"], "logit_softcap")
        if d.get("max_len"):
            cfg.max_model_len = _pos_int(d["max_len"], "max_len")
        dt = d.get("torch_dtype", d.get("dtype"))
        if dt is not None:
            cfg.torch_dtype = str(dt).replace("torch.", "")
        eos = d.get("eos_token_id")
        if eos is not None:
            cfg.eos_token_ids = [int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos])]
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        return dict(self.raw)
