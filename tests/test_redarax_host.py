"""The Redarax design without a GPU: its configuration and the errors it raises, its description as data against the
plain implementation's list of tensors, the registry, and properties of the plain implementation itself."""
import copy

import pytest
import torch

import plain_redarax as P
from redarax_configs import CONFIGS

from lmsf_b200.config import ConfigError
from lmsf_b200.config.registry import resolve_architecture
from lmsf_b200.parts.decoder import DecoderModel
from lmsf_b200.weights.random_init import tensor_list


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_description_names_exactly_the_tensors_of_the_design(name):
    cfg = CONFIGS[name]
    arch = resolve_architecture(cfg)
    assert arch.name == "Redarax"
    model = DecoderModel(arch.build_spec(arch.parse_config(cfg)))
    got = {n: tuple(s) for n, s, _ in tensor_list(model)}
    assert got == {n: tuple(s) for n, s in P.tensor_shapes(cfg).items()}
    assert [c.layer for c in model.calls] == list(range(len(cfg["layers"])))


def test_every_size_and_constant_is_read_per_layer():
    typed = resolve_architecture(CONFIGS["X"]).parse_config(CONFIGS["X"])
    assert [L.mixer.type for L in typed.layers] == ["delta", "attention", "mamba2", "attention", "delta"]
    assert (typed.layers[1].mixer.rot_dims, typed.layers[1].mixer.rot_base, typed.layers[1].mixer.scale) == (10, 7000.0, 0.21)
    assert (typed.layers[3].mixer.dim, typed.layers[3].mixer.vdim) == (16, 40)
    assert typed.layers[2].mlp is None and typed.layers[0].mlp.groups == 3 and typed.layers[0].mlp.keep == 2
    assert (typed.residual_mult, typed.side_dim, typed.logit_scale, typed.logit_softcap) == (0.6, 6, 1.7, 9.0)
    y = resolve_architecture(CONFIGS["Y"]).parse_config(CONFIGS["Y"])
    assert (y.side_dim, y.logit_scale, y.logit_softcap, y.layers[1].mixer.rot_dims) == (0, 1.0, 0.0, 0)


def test_caches_and_states_follow_the_mixers():
    cfg = CONFIGS["X"]
    arch = resolve_architecture(cfg)
    model = DecoderModel(arch.build_spec(arch.parse_config(cfg)))
    specs = [(model.call_cache_spec(j), model.call_state_spec(j)) for j in range(len(model.calls))]
    assert specs[0][0] is None and specs[0][1].shape == (4 * 12 * 20 + (2 - 1) * (2 * 2 * 12 + 4 * 20),)
    assert specs[1][1] is None and (specs[1][0].num_kv_heads, specs[1][0].head_dim) == (2, 32)    # 24 and 8 share a width of 32
    assert specs[2][1].shape == (6 * 12 * 10 + (4 - 1) * (6 * 12 + 2 * 2 * 10),)
    assert specs[3][0].head_dim == 48


@pytest.mark.parametrize("path,value", [(("layers", 0, "type"), "lstm"), (("layers", 1, "mixer", "kv_heads"), 4),
                                         (("layers", 1, "mixer", "rot", "dims"), 26), (("layers", 2, "mixer", "norm_groups"), 5),
                                         (("layers", 0, "mlp", "router", "top"), 5), (("layers", 1, "mlp", "kind"), "glu"),
                                         (("norm", "eps"), 0.0), (("width",), -3)])
def test_a_configuration_that_cannot_be_a_model_is_refused(path, value):
    cfg = copy.deepcopy(CONFIGS["X"])
    d = cfg
    for k in path[:-1]:
        d = d[k]
    d[path[-1]] = value
    with pytest.raises(ConfigError):
        resolve_architecture(cfg).parse_config(cfg)


def test_a_missing_key_is_named():
    cfg = copy.deepcopy(CONFIGS["X"])
    del cfg["layers"][2]["mixer"]["state"]
    with pytest.raises(ConfigError, match="state"):
        resolve_architecture(cfg).parse_config(cfg)


# ----------------------------------------------------------------------------- the plain implementation itself

def test_the_plain_implementation_is_causal_and_every_branch_matters():
    cfg = CONFIGS["X"]
    w = P.random_weights(cfg, seed=3, dtype=torch.float64)
    a = list(range(5, 45))
    b = a[:30] + [7] * 10
    la, lb = P.forward(cfg, w, a), P.forward(cfg, w, b)
    assert torch.equal(la[:30], lb[:30]) and not torch.allclose(la[30:], lb[30:])
    for name in ("l0.mix.a", "l2.mix.D", "l1.mix.k.norm", "l3.mlp.correction", "l4.side.gate", "side.embed", "l1.mix.o.b"):
        w2 = dict(w)
        w2[name] = w[name] + torch.linspace(-1, 1, w[name].numel(), dtype=torch.float64).reshape(w[name].shape)
        assert not torch.allclose(P.forward(cfg, w2, a), la), name


def test_convolution_against_its_definition():
    x, w, b = torch.randn(9, 3, dtype=torch.float64), torch.randn(3, 4, dtype=torch.float64), torch.randn(3, dtype=torch.float64)
    y = P.causal_conv(x, w, b)
    for t in range(9):
        for c in range(3):
            want = b[c] + sum(w[c, j] * x[t - 3 + j, c] for j in range(4) if t - 3 + j >= 0)
            assert abs(float(y[t, c] - want)) < 1e-12


def test_routing_keeps_to_the_best_groups_even_with_negative_scores():
    h = torch.eye(4, dtype=torch.float64)
    W = {"router": torch.tensor([[9., 0, 0, 0], [-9, 0, 0, 0], [2, 0, 0, 0], [1.5, 0, 0, 0], [3, 0, 0, 0], [-9, 0, 0, 0]], dtype=torch.float64),
         "correction": torch.tensor([0., 0, 0, 0, 0, -5], dtype=torch.float64)}
    r = {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 1}}
    ids, wts = P.route(h[:1], W, r)
    # group scores: {0,1}: ~1 + ~0, {2,3}: 0.88 + 0.82, {4,5}: 0.95 + (0 - 5): the middle group wins although expert 0 is the best
    assert sorted(ids[0].tolist()) == [2, 3]
    assert torch.allclose(wts[0], torch.sigmoid(torch.tensor([2.0, 1.5], dtype=torch.float64)))
    r["groups"] = {"count": 3, "keep": 2}
    ids, _ = P.route(h[:1], W, r)
    assert sorted(ids[0].tolist()) == [0, 2]             # the kept groups: {2,3} and {0,1}; the largest two of their four
    W["correction"] = torch.full((6,), -3.0, dtype=torch.float64)      # every choice score negative: still two of the kept
    r["groups"] = {"count": 3, "keep": 1}
    ids, wts = P.route(h[:1], W, r)
    assert sorted(ids[0].tolist()) == [2, 3] and float(wts.min()) > 0.8


def test_delta_rule_with_full_strength_stores_and_recalls():
    """beta -> 1, no decay, orthogonal keys: reading with k_i returns v_i exactly."""
    dk, dv = 4, 3
    S = torch.zeros(dk, dv, dtype=torch.float64)
    keys, vals = torch.eye(dk, dtype=torch.float64), torch.randn(dk, dv, dtype=torch.float64)
    for i in range(dk):
        u = 1.0 * (vals[i] - S.T @ keys[i])
        S = S + torch.outer(keys[i], u)
    for i in range(dk):
        assert torch.allclose(S.T @ keys[i], vals[i])
