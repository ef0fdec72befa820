"""Vazepel without a GPU: config to parts, tensor names and shapes, the cache plan, config errors, and the plain statement's own
pieces against hand-made numbers."""

import copy
import math

import pytest
import torch

import vazepel_util as VU
from plain import vazepel_plain as VP


def _model(cfg):
    from oxr_inference_b200.weights.random_init import shape_only_model

    return shape_only_model(cfg)


def test_architecture_is_found_by_its_single_name():
    from oxr_inference_b200.config.registry import resolve_architecture

    assert resolve_architecture(VU.MODEL_R).name == "Vazepel"


def test_tensor_names_and_shapes():
    m = _model(VU.MODEL_P)
    named = {k: tuple(v[2].shape) for k, v in m.named_parameters().items()}
    assert named["embed"] == (131, 48) and named["head"] == (131, 48) and named["final.norm"] == (48,) and named["final.norm.b"] == (48,)
    assert named["l0.norm1"] == (48,) and named["l0.norm1.b"] == (48,) and "l0.norm2" not in named
    assert named["l0.mix.q"] == (64, 48) and named["l0.mix.k"] == (32, 48) and named["l0.mix.v"] == (48, 48) and named["l0.mix.g"] == (96, 48)
    assert named["l0.mix.o"] == (48, 96) and named["l0.mix.o.b"] == (48,) and named["l0.mix.q.b"] == (64,) and named["l0.mix.talk"] == (4, 4)
    assert named["l2.mix.talk"] == (6, 6) and named["l2.mix.g"] == (96, 48) and named["l3.mix.v"] == (32, 48)
    assert named["l0.rg1"] == (48, 48) and named["l0.rg2.b"] == (48,) and named["l2.rg1.b"] == (48,)
    assert "l2.rg2" not in named and not any(k.startswith("l2.mlp") for k in named)         # a layer without a feed-forward
    assert [named[f"l{i}.dwa"] for i in range(4)] == [(2,), (3,), (4,), (5,)]
    assert named["l1.mlp.up"] == (56, 48) and named["l1.mlp.down"] == (48, 56)
    assert named["l0.mlp.router"] == (6, 48) and named["l0.mlp.e5.gate"] == (24, 48) and named["l0.mlp.e5.down"] == (48, 24)
    assert named["l0.mlp.shared.up"] == (40, 48) and "l3.mlp.shared.up" not in named and named["l3.mlp.e7.up"] == (16, 48)


def test_cache_plan_has_pools_of_separate_key_and_value_size():
    from oxr_inference_b200.parts.base import PagedKVNeed

    m = _model(VU.MODEL_P)
    plan = m.cache_plan
    needs = [plan.groups[e.group].need for e in plan.entries]
    assert needs[0] == PagedKVNeed(2, 16, 0, value_dim=24) and needs[1] == PagedKVNeed(2, 8, 0, value_dim=8)
    assert needs[2] == PagedKVNeed(2, 32, 0, value_dim=16) and needs[3] == PagedKVNeed(1, 16, 0, value_dim=32)
    assert all(e.state is None for e in plan.entries)


def test_the_gate_of_an_absent_feed_forward_may_be_stored():
    import re

    allowed = [re.compile(p + "$") for p in _model(VU.MODEL_P).spec.ignored_tensors]
    assert any(r.match("l2.rg2") for r in allowed) and any(r.match("l11.rg2.b") for r in allowed)
    assert not any(r.match(name) for r in allowed for name in ("l2.rg1", "l2.rg22", "xl2.rg2", "l2.mlp.up", "head"))


@pytest.mark.parametrize("change,words", [
    (lambda c: c["layers"][0].update(type="retention"), "is not one of"),
    (lambda c: c["layers"][0]["mlp"].update(kind="glu"), "is not one of"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "lacks 'scale'"),
    (lambda c: c["layers"][0]["mixer"].pop("softcap"), "lacks 'softcap'"),
    (lambda c: c["layers"][0]["mixer"].update(heads=5), "not a multiple"),
    (lambda c: c["layers"][0]["mixer"].update(softcap=0.0), "softcap"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "do not fit"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4), "do not fit"),
    (lambda c: c["layers"][0]["mlp"]["expert"].update(limit=-1.0), "limit"),
    (lambda c: c["layers"][1]["mlp"].pop("ff"), "lacks 'ff'"),
    (lambda c: c.pop("norm"), "lacks 'norm'"),
    (lambda c: c.update(layers=[]), "non-empty"),
])
def test_config_errors(change, words):
    from oxr_inference_b200.config.model_config import ConfigError
    from oxr_inference_b200.config.registry import resolve_architecture

    cfg = copy.deepcopy(VU.MODEL_P)
    change(cfg)
    with pytest.raises(ConfigError, match=words):
        resolve_architecture(cfg).config_from_dict(cfg, None)


# ------------------------------------------------------------------------------------------------ the plain statement's pieces
def test_plain_layer_norm_and_gelu():
    x = torch.tensor([[1.0, 2.0, 3.0, 6.0]], dtype=torch.float64)
    w, b = torch.tensor([1.0, 2.0, 1.0, 0.5], dtype=torch.float64), torch.tensor([0.0, 1.0, 0.0, -1.0], dtype=torch.float64)
    y = VP.layer_norm(x, w, b, 0.0)
    sd = math.sqrt((4 + 1 + 0 + 9) / 4)
    assert torch.allclose(y, torch.tensor([[-2 / sd, -2 / sd + 1, 0.0, 1.5 / sd - 1]], dtype=torch.float64))
    z = torch.tensor([-3.0, 0.0, 0.5, 4.0], dtype=torch.float64)
    assert torch.allclose(VP.gelu_tanh(z), torch.nn.functional.gelu(z, approximate="tanh"))


def test_plain_rotation_turns_pairs_of_neighbours_and_leaves_the_rest():
    x = torch.zeros(3, 1, 6, dtype=torch.float64)
    x[:, 0, 0], x[:, 0, 3], x[:, 0, 4] = 1.0, 2.0, 7.0
    y = VP.rotate_pairs(x, 4, 100.0)
    for p in range(3):
        a0, a1 = p * 1.0, p * 100.0 ** (-0.5)
        assert torch.allclose(y[p, 0], torch.tensor([math.cos(a0), math.sin(a0), -2 * math.sin(a1), 2 * math.cos(a1), 7.0, 0.0], dtype=torch.float64))


def test_plain_router_takes_softmax_scores_of_the_kept_groups_as_they_are():
    z = torch.tensor([[2.0, 0.1, 0.0, 3.0, -1.0, -1.0, 1.9, 1.8]], dtype=torch.float64)
    s = torch.softmax(z, -1)
    # groups of two, best score each: (2.0), (3.0), (-1), (1.9): with two kept only experts 0..3 can be chosen, so 6 and 7 lose to 1
    ids, wts, margin = VP.choose_experts(z, 3, 4, 2)
    assert ids[0].tolist() == [3, 0, 1] and torch.allclose(wts[0], s[0, [3, 0, 1]]) and wts.sum() < 1.0
    assert abs(margin.item() - min(s[0, 0] - s[0, 6], s[0, 1] - s[0, 2]).item()) < 1e-12
    ids, _, _ = VP.choose_experts(z, 3, 1, 1)
    assert ids[0].tolist() == [3, 0, 6]


def test_plain_expert_clamps_gate_from_above_and_up_on_both_sides():
    w = {"e.gate": torch.tensor([[1.0]], dtype=torch.float64), "e.up": torch.tensor([[2.0]], dtype=torch.float64), "e.down": torch.tensor([[1.0]], dtype=torch.float64)}
    h = torch.tensor([[-3.0], [0.2], [5.0]], dtype=torch.float64)
    y = VP.clamped_unit(h, w, "e.", 1.5)

    def unit(g, u):
        return g / (1 + math.exp(-1.702 * g)) * (u + 1)

    assert torch.allclose(y[:, 0], torch.tensor([unit(-3.0, -1.5), unit(0.2, 0.4), unit(1.5, 1.5)], dtype=torch.float64))


def test_plain_attention_sink_and_head_mixing():
    """One key, two heads, mixing matrix [[1, 1], [0, -1]]: with scores a and b the weights are e^(a+b) / (1 + e^(a+b)) and
    e^(-b) / (1 + e^(-b)); the cap bends a large score to nearly its limit."""
    m = {"heads": 2, "kv_heads": 1, "dim": 2, "vdim": 1, "scale": 1.0, "softcap": 3.0}
    eye2 = torch.eye(2, dtype=torch.float64)
    w = {"q": torch.cat([eye2, 10 * eye2]), "k": eye2, "v": torch.tensor([[1.0, 0.0]], dtype=torch.float64), "g": torch.zeros(2, 2, dtype=torch.float64),
         "o": eye2, "talk": torch.tensor([[1.0, 1.0], [0.0, -1.0]], dtype=torch.float64)}
    w = {"p." + k: v for k, v in w.items()}
    for name, n in (("q.b", 4), ("k.b", 2), ("v.b", 1), ("o.b", 2)):
        w["p." + name] = torch.zeros(n, dtype=torch.float64)
    h = torch.tensor([[1.0, 0.5]], dtype=torch.float64)
    y = VP.mixed_head_attention(h, w, "p.", m)
    a, b = 3.0 * math.tanh(1.25 / 3.0), 3.0 * math.tanh(12.5 / 3.0)
    want = [0.5 * math.exp(a + b) / (1 + math.exp(a + b)), 0.5 * math.exp(-b) / (1 + math.exp(-b))]   # the output gate is sigmoid(0)
    assert torch.allclose(y[0], torch.tensor(want, dtype=torch.float64))


def test_plain_forward_looks_at_nothing_ahead():
    cfg = VU.MODEL_R
    torch.manual_seed(0)
    w = {name: torch.randn(info.shape, dtype=torch.float64) * 0.3 for name, (_, _, info) in _model(cfg).named_parameters().items()}
    ids = VU.tokens(cfg, 12, seed=1)
    whole = VP.forward(cfg, w, ids)
    for n in (1, 5, 12):
        assert torch.allclose(VP.forward(cfg, w, ids[:n])[-1], whole[n - 1], atol=1e-10)
