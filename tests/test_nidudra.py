"""Nidudra without a GPU: config to parts, tensor names and shapes, the cache plan (a borrowed cache, first keys kept behind a window, a pair
of mixers that shares one state row), config errors, the pages of kept first keys in the cache manager, the rotation's frequency
rescalings, and the plain statement's own pieces against hand-made numbers."""

import copy
import math

import pytest
import torch

import nidudra_util as NU
from plain import nidudra_plain as NP


def _model(cfg):
    from oxr_inference_b200.weights.random_init import shape_only_model

    return shape_only_model(cfg)


def test_architecture_is_found_by_its_single_name():
    from oxr_inference_b200.config.registry import resolve_architecture

    assert resolve_architecture(NU.MODEL_B).name == "Nidudra"


def test_tensor_names_and_shapes():
    m = _model(NU.MODEL_A)
    named = {k: tuple(v[2].shape) for k, v in m.named_parameters().items()}
    assert named["embed"] == (131, 48) and named["head"] == (131, 48) and named["final.norm"] == (48,)
    assert named["l0.norm1"] == (48,) and named["l0.norm2"] == (48,) and "l4.norm2" not in named      # the last layer has no feed-forward
    assert named["l0.mix.q"] == (64, 48) and named["l0.mix.k"] == (32, 48) and named["l0.mix.v"] == (48, 48) and named["l0.mix.g"] == (96, 48)
    assert named["l0.mix.o"] == (48, 96) and named["l0.mix.q.norm"] == (16,) and named["l0.mix.k.norm"] == (16,)
    assert named["l0.mlp.gate"] == (56, 48) and named["l0.mlp.down"] == (48, 56)
    assert named["l1.mix.sink"] == (4,) and named["l1.mix.g"] == (4, 48) and "l1.mix.q.norm" not in named
    assert named["l1.mlp.router"] == (6, 48) and named["l1.mlp.e5.gate"] == (24, 48) and named["l1.mlp.e0.down"] == (48, 24)
    assert named["l1.mlp.shared.up"] == (40, 48) and named["l1.mlp.shared.sg"] == (1, 48)
    assert named["l2.mix.left.q"] == (64, 48) and named["l2.mix.left.k"] == (32, 48) and "l2.mix.left.v" not in named
    assert named["l2.mix.left.q.b"] == (64,) and named["l2.mix.left.k.conv"] == (32, 3) and named["l2.mix.left.k.norm"] == (16,)
    assert named["l2.mix.right.q"] == (36, 48) and named["l2.mix.right.v"] == (60, 48) and named["l2.mix.right.g"] == (60, 48)
    assert named["l2.mix.right.a1"] == (5, 48) and named["l2.mix.right.a2"] == (36, 5) and named["l2.mix.right.a2.b"] == (36,)
    assert named["l2.mix.right.norm"] == (20,) and named["l2.mix.left.out"] == (48,) and named["l2.mix.right.out"] == (48,)
    # a layer that reads another's keys and values has queries, norm, gate and output of its own and nothing else
    assert sorted(k for k in named if k.startswith("l3.mix.")) == ["l3.mix.g", "l3.mix.o", "l3.mix.q", "l3.mix.q.norm"]
    assert "l3.mlp.shared.up" in named and named["l3.mlp.e4.up"] == (16, 48)


def test_the_decay_rank_comes_from_the_checkpoint_shapes():
    from oxr_inference_b200.config.registry import resolve_architecture

    arch = resolve_architecture(NU.MODEL_A)
    cfg = copy.deepcopy(NU.MODEL_A)
    del cfg["layers"][2]["mixer"]["right"]["rank"]
    config = arch.config_from_dict(cfg, None)
    spec = arch.spec_for(config, {"l2.mix.right.a1": (11, 48)})
    assert spec.layers[2].mixer.params["right"]["params"]["decay_rank"] == 11
    assert arch.spec_for(config, None).layers[2].mixer.params["right"]["params"]["decay_rank"] == 16


def test_cache_plan_borrowed_cache_kept_first_keys_and_a_shared_state_row():
    from oxr_inference_b200.parts.base import PagedKVNeed, StateNeed

    plan = _model(NU.MODEL_B).cache_plan
    e = plan.entries
    # layer 2 reads layer 1's cache: the group keeps what either mask needs (windows of 20 and 7, first keys 0 and 10)
    assert e[2].group == e[1].group and e[2].layer_in_group == e[1].layer_in_group and not e[2].store and e[1].store
    assert plan.groups[e[1].group].need == PagedKVNeed(3, 32, 20, keep_first=10)
    # the pair: pages of the left side and one state row for both (the filter's tails, then the recurrence's matrices)
    assert plan.groups[e[0].group].need == PagedKVNeed(1, 32, 0) and plan.states[e[0].state] == StateNeed(((64 + 32) * 1 + 1 * 40 * 8,))
    assert plan.states[e[4].state] == StateNeed(((144 + 144) * 3 + 4 * 70 * 33,))
    assert plan.groups[e[3].group].need == PagedKVNeed(1, 32, 0, value_dim=16)
    a = _model(NU.MODEL_A).cache_plan
    assert a.groups[a.entries[0].group].need == PagedKVNeed(2, 16, 9, value_dim=24, keep_first=3) and a.entries[3].group == a.entries[0].group


@pytest.mark.parametrize("change,words", [
    (lambda c: c["layers"][0].update(type="retention"), "is not one of"),
    (lambda c: c["layers"][0]["mlp"].update(kind="glu"), "is not one of"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "lacks 'scale'"),
    (lambda c: c["layers"][0]["mixer"].pop("mask"), "lacks 'mask'"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), "mask.size"),
    (lambda c: c["layers"][0]["mixer"].update(heads=5), "not a multiple"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=18), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"]["rot"]["scaling"].pop("high"), "lacks 'high'"),
    (lambda c: c["layers"][2]["mixer"]["left"].update(vdim=24), "vdim must equal dim"),
    (lambda c: c["layers"][2]["mixer"]["right"].update(tau=0.0), "tau"),
    (lambda c: c["layers"][2]["mixer"].pop("right"), "lacks 'right'"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "earlier layer"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=1), "no keys and values of this kind"),
    (lambda c: c["layers"][3]["mixer"].update(dim=32), "differs from layer 0"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=7), "cannot be chosen"),
    (lambda c: c["layers"][0]["mlp"].pop("ff"), "lacks 'ff'"),
    (lambda c: c.pop("norm"), "lacks 'norm'"),
    (lambda c: c.update(layers=[]), "non-empty"),
])
def test_config_errors(change, words):
    from oxr_inference_b200.config.model_config import ConfigError
    from oxr_inference_b200.config.registry import resolve_architecture

    cfg = copy.deepcopy(NU.MODEL_A)
    change(cfg)
    with pytest.raises(ConfigError, match=words):
        resolve_architecture(cfg).config_from_dict(cfg, None)


# ------------------------------------------------------------------------------------------------ the cache manager
def test_pages_of_kept_first_keys_stay_while_the_window_moves_on_and_come_back_at_the_end():
    from oxr_inference_b200.cache import RELEASED, CacheManager, make_cache_plan
    from oxr_inference_b200.parts.base import PagedKVNeed

    plan = make_cache_plan([PagedKVNeed(2, 16, 10, keep_first=9), PagedKVNeed(2, 16, 0)], [None, None])
    m = CacheManager(plan, page_size=4, num_pages=20, max_requests=2)
    assert m.kept_pages == [3, 0]
    a = m.open("a")
    assert m.reserve(a, 11)
    m.advance(a, 11)
    assert RELEASED not in a.tables[0], "nothing but kept pages lies behind the window yet"
    assert m.reserve(a, 40)
    m.advance(a, 40)       # the next query sits at 40 and sees keys 31..: pages 0-2 are kept, 3-6 are given back, 7 holds key 31
    assert [p == RELEASED for p in a.tables[0]] == [False] * 3 + [True] * 4 + [False] * 3 and RELEASED not in a.tables[1]
    m.check()
    free = m.pools[0].free
    b = m.open("b")
    assert m.reserve(b, 16), "the pages the window passed are handed out again"
    assert set(b.tables[0]) & set(p for p in a.tables[0] if p != RELEASED) == set()
    m.advance(b, 16)
    m.check()
    m.close(a)
    m.close(b)
    m.check()
    assert m.pools[0].free == free + 6 and m.pools[1].free == 19
    # a window that still reaches into the kept keys releases nothing
    c = m.open("c")
    assert m.reserve(c, 14)
    m.advance(c, 14)
    assert RELEASED not in c.tables[0]
    m.check()


# ------------------------------------------------------------------------------------------------ frequencies
def test_banded_frequencies_by_hand():
    from oxr_inference_b200.parts.rope import banded_frequencies

    # wavelengths 2 pi / f against original / high = 16 and original / low = 64
    f = [1.0, 2 * math.pi / 32.0, 2 * math.pi / 64.5, 0.01]
    got = banded_frequencies(f, factor=6.0, low=1.0, high=4.0, original=64)
    s = (64 / 32.0 - 1.0) / 3.0
    assert got[0] == 1.0 and got[3] == 0.01 / 6.0 and got[2] == f[2] / 6.0
    assert abs(got[1] - ((1 - s) * f[1] / 6.0 + s * f[1])) < 1e-15


def test_ramped_frequencies_by_hand():
    from oxr_inference_b200.parts.rope import banded_frequencies, ramped_frequencies

    dims, base = 16, 100.0
    f = [base ** (-2.0 * i / dims) for i in range(8)]
    got, mag = ramped_frequencies(f, dims=dims, base=base, factor=5.0, original=40, fast=4.0, slow=0.5)
    index = lambda t: dims * math.log(40 / (2 * math.pi * t)) / (2 * math.log(base))
    lo, hi = max(math.floor(index(4.0)), 0), min(math.ceil(index(0.5)), dims - 1)
    assert (lo, hi) == (0, 5)
    for i in range(8):
        r = min(max((i - lo) / (hi - lo), 0.0), 1.0)
        assert abs(got[i] - (f[i] / 5.0 * r + f[i] * (1 - r))) < 1e-15
    assert got[0] == f[0] and got[5] == f[5] / 5.0 and got[7] == f[7] / 5.0 and abs(mag - (0.1 * math.log(5.0) + 1.0)) < 1e-15
    # the plain statement, written apart, says the same
    want, want_mag = NP.ramp_frequencies(dims, base, {"factor": 5.0, "original": 40, "fast": 4.0, "slow": 0.5})
    assert got == pytest.approx(want, rel=1e-14) and mag == pytest.approx(want_mag)
    assert NP.banded_frequencies(dims, base, NU.bands()) == pytest.approx(banded_frequencies(f, **NU.bands()), rel=1e-14)


# ------------------------------------------------------------------------------------------------ the plain statement's pieces
def test_plain_mask_keeps_the_first_keys_behind_the_window():
    seen = NP.visible(7, window=3, keep_first=2)
    assert seen[6].tolist() == [True, True, False, False, True, True, True]
    assert seen[3].tolist() == [True, True, True, True, False, False, False]
    assert seen[2].tolist() == [True, True, True, False, False, False, False]
    assert NP.visible(4).tolist() == torch.tril(torch.ones(4, 4, dtype=torch.bool)).tolist()


def test_plain_rotation_pairs_entry_i_with_entry_i_plus_half_and_leaves_the_rest():
    x = torch.zeros(3, 1, 6, dtype=torch.float64)
    x[:, 0, 0], x[:, 0, 3], x[:, 0, 5] = 1.0, 2.0, 7.0
    y = NP.rotate_halves(x, [1.0, 0.1], magnitude=1.5)
    for p in range(3):
        a0, a1 = p * 1.0, p * 0.1
        want = [1.5 * math.cos(a0), -3.0 * math.sin(a1), 1.5 * math.sin(a0), 3.0 * math.cos(a1), 0.0, 7.0]
        assert torch.allclose(y[p, 0], torch.tensor(want, dtype=torch.float64))


def test_plain_filter_puts_the_last_tap_on_the_current_token():
    u = torch.tensor([[1.0], [10.0], [100.0], [1000.0]], dtype=torch.float64)
    y = NP.causal_filter(u, torch.tensor([[3.0, 2.0, 1.0]], dtype=torch.float64))
    assert y[:, 0].tolist() == [1.0, 12.0, 123.0, 1230.0]


def test_plain_sink_joins_the_denominator_only():
    q = torch.tensor([[[2.0]]], dtype=torch.float64)
    k = torch.tensor([[[1.5]]], dtype=torch.float64)
    v = torch.tensor([[[4.0]]], dtype=torch.float64)
    o = NP.softmax_attention(q, k, v, 0.5, NP.visible(1), sink=torch.tensor([0.7], dtype=torch.float64))
    assert abs(o.item() - 4.0 * math.exp(1.5) / (math.exp(1.5) + math.exp(0.7))) < 1e-12


def test_plain_decay_acts_on_key_channels():
    """One head, two key channels, one value: with alpha = (a, b) the state after two tokens is (a k0 v0 + k0' v1, b k1 v0 + k1' v1)."""
    eye = torch.eye(2, dtype=torch.float64)
    w = {"p.q": eye * math.sqrt(2.0), "p.k": eye, "p.v": torch.tensor([[1.0, 1.0]], dtype=torch.float64), "p.g": torch.tensor([[50.0, 0.0]], dtype=torch.float64),
         "p.o": torch.ones(1, 1, dtype=torch.float64), "p.a1": eye, "p.a2": torch.zeros(2, 2, dtype=torch.float64),
         "p.a2.b": torch.tensor([0.0, 2.0], dtype=torch.float64), "p.norm": torch.ones(1, dtype=torch.float64)}
    m = {"heads": 1, "dim": 2, "vdim": 1, "tau": 2.0}
    h = torch.tensor([[1.0, 2.0], [3.0, 1.0]], dtype=torch.float64)
    a, b = 0.5 ** 0.5, (1 / (1 + math.exp(-2.0))) ** 0.5
    o1 = (a * 1.0 * 3.0 + 3.0 * 4.0) * 3.0 + (b * 2.0 * 3.0 + 1.0 * 4.0) * 1.0          # S_1^T q_1 with q = h (sqrt(2) / sqrt(dim))
    y = NP.decayed_linear_attention(h, w, "p.", m, 0.0)
    # the head norm over one entry leaves the sign; the gate silu(50 h_0) is h_0 * 50 to many digits
    assert abs(y[1, 0].item() - math.copysign(1.0, o1) * 150.0) < 1e-9 and abs(y[0, 0].item() - 50.0) < 1e-9


def test_plain_experts_scale_their_input_by_the_score():
    w = {"p.router": torch.tensor([[1.0], [-1.0], [3.0]], dtype=torch.float64)}
    for e in range(3):
        w[f"p.e{e}.gate"] = torch.tensor([[1.0 + e]], dtype=torch.float64)
        w[f"p.e{e}.up"] = torch.tensor([[2.0]], dtype=torch.float64)
        w[f"p.e{e}.down"] = torch.tensor([[1.0]], dtype=torch.float64)
    h = torch.tensor([[0.5]], dtype=torch.float64)
    y = NP.routed_experts(h, w, "p.", {"router": {"experts": 3, "top": 2}})
    s = lambda z: 1 / (1 + math.exp(-z))
    unit = lambda x, g: (g * x) * s(g * x) * (2.0 * x)
    assert abs(y.item() - (unit(s(1.5) * 0.5, 3.0) + unit(s(0.5) * 0.5, 1.0))) < 1e-12
    assert NP.choice_margin(NP.router_scores(h, w, "p."), 2).item() == pytest.approx(s(0.5) - s(-0.5))


def test_plain_forward_looks_at_nothing_ahead():
    cfg = NU.MODEL_A
    torch.manual_seed(0)
    w = {name: torch.randn(info.shape, dtype=torch.float64) * 0.3 for name, (_, _, info) in _model(cfg).named_parameters().items()}
    ids = NU.tokens(cfg, 14, seed=1)
    whole = NP.forward(cfg, w, ids)
    for n in (1, 5, 14):
        assert torch.allclose(NP.forward(cfg, w, ids[:n])[-1], whole[n - 1], atol=1e-9)
