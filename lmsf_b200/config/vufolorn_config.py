"""The typed configuration of the Vufolorn design, read from config.json.

config.json of this design is nested: `layers` lists every layer with its `type` (which mixer), the mixer's sizes
(`mixer`) and its feed-forward (`mlp`, or null for none); `loop` names a span of layers that runs several times;
`norm.eps`, `vocab` and `width` are global.  Every size and every constant that may differ between models of the design
is read from there; nothing is assumed equal between layers.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .model_config import ConfigError

MIXER_TYPES = ("lightning", "latent_attention")


def _need(d: Dict[str, Any], key: str, where: str):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: {where} lacks {key!r}")
    return d[key]


def _pos_int(v, what: str) -> int:
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {what} must be a positive integer, got {v!r}")
    return v


@dataclass
class VufolornMixer:
    type: str
    heads: int
    dim: int
    vdim: int
    decay: List[float] = field(default_factory=list)     # lightning: one per head
    kv_rank: int = 0                                     # latent attention
    scale: Optional[float] = None
    window: Optional[int] = None                         # mask.size; None: every earlier token is seen


@dataclass
class VufolornFeedForward:
    experts: int
    top: int
    expert_ff: int
    shared_ff: int = 0                                   # 0: no shared expert


@dataclass
class VufolornLayer:
    mixer: VufolornMixer
    mlp: Optional[VufolornFeedForward]


@dataclass
class VufolornConfig:
    vocab: int
    width: int
    eps: float
    layers: List[VufolornLayer]
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1                                  # a span [start, stop) that runs `times` times; no span: stop == start
    has_loop: bool = False
    max_model_len: int = 1 << 20                         # no position encoding: bounded by the cache alone
    torch_dtype: str = "bfloat16"
    eos_token_ids: List[int] = field(default_factory=list)
    raw: Dict[str, Any] = field(default_factory=dict)

    @staticmethod
    def from_dict(d: Dict[str, Any]) -> "VufolornConfig":
        vocab = _pos_int(_need(d, "vocab", "the model"), "vocab")
        width = _pos_int(_need(d, "width", "the model"), "width")
        eps = float(_need(_need(d, "norm", "the model"), "eps", "norm"))
        if not (eps > 0):
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps!r}")
        raw_layers = _need(d, "layers", "the model")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, L in enumerate(raw_layers):
            where = f"layers[{i}]"
            kind = _need(L, "type", where)
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of this design ({', '.join(MIXER_TYPES)})")
            m = _need(L, "mixer", where)
            mixer = VufolornMixer(kind, _pos_int(_need(m, "heads", where + ".mixer"), "heads"),
                                  _pos_int(_need(m, "dim", where + ".mixer"), "dim"),
                                  _pos_int(_need(m, "vdim", where + ".mixer"), "vdim"))
            if kind == "lightning":
                decay = _need(m, "decay", where + ".mixer")
                if not isinstance(decay, list) or len(decay) != mixer.heads:
                    raise ConfigError(f"config.json: {where}.mixer.decay must list one decay per head ({mixer.heads})")
                mixer.decay = [float(a) for a in decay]
            else:
                mixer.kv_rank = _pos_int(_need(m, "kv_rank", where + ".mixer"), "kv_rank")
                mixer.scale = float(m["scale"]) if m.get("scale") is not None else None     # None: dim ** -0.5
                mask = m.get("mask")
                if mask and mask.get("size") is not None:
                    mixer.window = _pos_int(mask["size"], "mask.size")
            f = L.get("mlp")
            mlp = None
            if f:
                kind_f = f.get("kind", "moe")
                if kind_f != "moe":
                    raise ConfigError(f"config.json: {where}.mlp.kind {kind_f!r} is not a feed-forward of this design (moe)")
                r = _need(f, "router", where + ".mlp")
                shared = f.get("shared")
                mlp = VufolornFeedForward(_pos_int(_need(r, "experts", where + ".mlp.router"), "experts"),
                                          _pos_int(_need(r, "top", where + ".mlp.router"), "top"),
                                          _pos_int(_need(_need(f, "expert", where + ".mlp"), "ff", where + ".mlp.expert"), "ff"),
                                          _pos_int(_need(shared, "ff", where + ".mlp.shared"), "ff") if shared else 0)
                if mlp.top > mlp.experts:
                    raise ConfigError(f"config.json: {where}.mlp.router: top {mlp.top} of {mlp.experts} experts")
            layers.append(VufolornLayer(mixer, mlp))
        cfg = VufolornConfig(vocab, width, eps, layers, raw=dict(d))
        loop = d.get("loop")
        if loop:
            start, stop, times = int(_need(loop, "start", "loop")), int(_need(loop, "stop", "loop")), int(_need(loop, "times", "loop"))
            if not (0 <= start <= stop <= len(layers)) or times < 1:
                raise ConfigError(f"config.json: loop {loop!r} does not fit {len(layers)} layers")
            if stop > start:
                cfg.loop_start, cfg.loop_stop, cfg.loop_times, cfg.has_loop = start, stop, times, True
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
