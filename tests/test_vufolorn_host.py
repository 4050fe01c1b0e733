"""Host side of the Vufolorn design: its configuration, its description as data, its tensor names, and two identities
that the engine's kernels rest on, checked on the plain implementation alone."""
import copy
import json

import pytest
import torch

import plain_vufolorn as P

CFG = {"architecture": "Vufolorn", "vocab": 50, "width": 32, "norm": {"eps": 1e-5},
       "layers": [{"type": "lightning", "mixer": {"heads": 2, "dim": 8, "vdim": 12, "decay": [0.5, 0.9]},
                   "mlp": {"kind": "moe", "router": {"experts": 3, "top": 2}, "expert": {"ff": 16}, "shared": {"ff": 8}}},
                  {"type": "latent_attention", "mixer": {"heads": 3, "dim": 8, "vdim": 4, "kv_rank": 20, "scale": 0.3, "mask": {"size": 6}},
                   "mlp": None},
                  {"type": "latent_attention", "mixer": {"heads": 1, "dim": 16, "vdim": 16, "kv_rank": 16, "scale": 0.25},
                   "mlp": {"kind": "moe", "router": {"experts": 2, "top": 1}, "expert": {"ff": 8}}}],
       "loop": {"start": 1, "stop": 3, "times": 2}}


def build(cfg):
    from lmsf_b200.config.registry import resolve_architecture
    from lmsf_b200.parts.decoder import DecoderModel
    arch = resolve_architecture(cfg)
    typed = arch.parse_config(cfg)
    return typed, DecoderModel(arch.build_spec(typed))


def test_the_design_is_found_by_its_name_and_described_as_data():
    from lmsf_b200.cache.storage import plan_groups
    typed, model = build(CFG)
    assert typed.has_loop and (typed.loop_start, typed.loop_stop, typed.loop_times) == (1, 3, 2)
    assert [(c.layer, c.entry, c.entry_pass) for c in model.calls] == [(0, None, 0), (1, 0, 0), (2, None, 0), (1, 0, 1), (2, None, 0)]
    groups, where = plan_groups(model)
    # one vector per token is cached (one plane), padded to what the attention kernels take; every run of a layer owns a cache
    assert [(g.spec.head_dim, g.spec.window, g.spec.planes, g.calls) for g in groups] == [(32, 6, 1, [1, 3]), (16, None, 1, [2, 4])]
    assert model.call_state_spec(0).shape == (2, 8, 12) and model.call_state_spec(1) is None
    assert model.blocks[1].feed_forward is None and model.blocks[2].feed_forward.shared_size == 0


def test_tensor_names_and_shapes_are_those_of_the_design():
    from lmsf_b200.weights.loader import collect_requirements
    _, model = build(CFG)
    asked = {}
    for _, _, wspec, names in collect_requirements(model):
        asked.update(dict(zip(names, [tuple(s) for s in wspec.shapes])))
    assert asked == {k: tuple(v) for k, v in P.tensor_shapes(CFG).items()}


def test_without_a_span_nothing_is_added_and_no_vector_is_asked_for():
    cfg = copy.deepcopy(CFG)
    del cfg["loop"]
    typed, model = build(cfg)
    assert not typed.has_loop and model.entries == [] and [c.layer for c in model.calls] == [0, 1, 2]


@pytest.mark.parametrize("change,needle", [
    (lambda c: c["layers"][0].update(type="convolution"), "type"),
    (lambda c: c["layers"][0]["mixer"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=4), "top"),
    (lambda c: c.update(loop={"start": 2, "stop": 5, "times": 2}), "loop"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["norm"].update(eps=0), "eps"),
])
def test_a_configuration_that_does_not_fit_is_refused_with_its_key(change, needle):
    from lmsf_b200.config import ConfigError
    cfg = copy.deepcopy(CFG)
    change(cfg)
    with pytest.raises(ConfigError) as e:
        build(cfg)
    assert needle in str(e.value)


def test_missing_and_misshapen_tensors_are_reported_together(tmp_path):
    from lmsf_b200.weights.loader import WeightError, check_tensors
    from lmsf_b200.weights.safetensors_io import open_model_tensors, write_safetensors
    _, model = build(CFG)
    w = P.random_weights(CFG, 0)
    del w["l1.mix.dkv.norm"]
    w["l0.ls1"] = torch.ones(31, dtype=torch.bfloat16)
    w["l9.extra"] = torch.ones(2, dtype=torch.bfloat16)
    (tmp_path / "config.json").write_text(json.dumps(CFG))
    write_safetensors(str(tmp_path / "model.safetensors"), [(n, t.dtype, tuple(t.shape)) for n, t in w.items()], lambda n: w[n])
    with pytest.raises(WeightError) as e:
        check_tensors(model, open_model_tensors(str(tmp_path)), str(tmp_path))
    assert e.value.missing == ["l1.mix.dkv.norm"] and e.value.unexpected == ["l9.extra"] and e.value.wrong_shape[0][0] == "l0.ls1"


def test_attention_on_the_cached_vector_equals_attention_on_expanded_keys_and_values():
    """q . (Wuk c) = (Wuk^T q) . c and sum p (Wuv c) = Wuv (sum p c): the identity behind caching c alone."""
    g = torch.Generator().manual_seed(0)
    m = CFG["layers"][1]["mixer"]
    H, dk, dv, r, D, T = m["heads"], m["dim"], m["vdim"], m["kv_rank"], 32, 15
    W = {"q": torch.randn(H * dk, D, generator=g), "dkv": torch.randn(r, D, generator=g), "dkv.norm": torch.rand(r, generator=g) + 0.5,
         "uk": torch.randn(H * dk, r, generator=g), "uv": torch.randn(H * dv, r, generator=g), "g": torch.randn(H, D, generator=g),
         "o": torch.randn(D, H * dv, generator=g)}
    W = {k: v.double() for k, v in W.items()}
    h = torch.randn(T, D, generator=g).double()
    want = P.latent_attention_mixer(h, W, m, 1e-5)
    c = P.rms_norm(h @ W["dkv"].T, W["dkv.norm"], 1e-5)
    q = (h @ W["q"].T).view(T, H, dk)
    out = torch.zeros(T, H, dv, dtype=torch.float64)
    for i in range(T):
        lo = max(0, i - m["mask"]["size"] + 1)
        for hd in range(H):
            qa = W["uk"][hd * dk:(hd + 1) * dk].T @ q[i, hd]
            p = torch.softmax((c[lo:i + 1] @ qa) * m["scale"], dim=0)
            out[i, hd] = W["uv"][hd * dv:(hd + 1) * dv] @ (p @ c[lo:i + 1]) * P.sigmoid(h[i] @ W["g"][hd])
    assert torch.allclose(out.view(T, H * dv) @ W["o"].T, want, rtol=1e-9, atol=1e-9)


def test_the_plain_model_runs_its_span_with_one_state_per_pass():
    """Shuffling the tokens after position t must not change the logits up to t (causality through every mechanism),
    and a span that runs once more changes them."""
    w = P.random_weights(CFG, 1, dtype=torch.float32)
    toks = [3, 9, 1, 44, 20, 7, 7, 30, 12, 5]
    a = P.forward(CFG, w, toks)
    b = P.forward(CFG, w, toks[:6] + [1, 2, 3, 4])
    assert torch.allclose(a[:6], b[:6], rtol=1e-9, atol=1e-9) and not torch.allclose(a[6:], b[6:], atol=1e-3)
    more = copy.deepcopy(CFG)
    more["loop"]["times"] = 3
    w3 = dict(w, **{"loop.step": torch.cat([w["loop.step"], w["loop.step"][:1]])})
    assert not torch.allclose(P.forward(more, w3, toks), a, atol=1e-3)
