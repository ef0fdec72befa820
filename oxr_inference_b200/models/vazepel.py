"""Vazepel: a decoder of parallel blocks whose config.json lists its layers one by one, from typed config to a description made of
registered parts.

Every layer reads ONE layer norm (weight and bias), ``h = norm1(x)``, with both sublayers: ``X = x + (rg1(h) * mixer(h) + rg2(h) * ff(h))``
where ``rg(h) = sigmoid(W h + b)`` gates each sublayer's result entry by entry. What the next layer (and the output) sees is not X but a
learned weighted sum of the embedding's output and the results X of all layers so far (``dwa``, one weight more per layer). The mixer is
grouped-query attention with biased projections, entry pairs of q and k rotated by position, scores capped by a tanh and mixed between the
heads by a learned matrix, one added to the softmax denominator, and a sigmoid gate on the concatenated heads. The feed-forward is null, a
two-matrix layer with the tanh form of GELU (``dense``), or clamped gated experts chosen by softmax scores among the best groups, their
scores as weights, plus a shared expert (``moe``). The model ends in a layer norm and an untied head.

Tensor names: ``embed``, ``head``, ``final.norm`` (+ ``.b``), and per layer ``l<i>.norm1`` (+ ``.b``), ``l<i>.rg1`` / ``l<i>.rg2`` (+ ``.b``),
``l<i>.dwa``, ``l<i>.mix.{q,k,v,o}`` (+ ``.b``), ``l<i>.mix.{g,talk}`` and ``l<i>.mlp.{up,down}`` or
``l<i>.mlp.{router, e<j>.{gate,up,down}, shared.{gate,up,down}}``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from oxr_inference_b200.config.model_config import ConfigError
from oxr_inference_b200.config.registry import Architecture, register_architecture
from oxr_inference_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

MAX_POSITIONS = 1 << 20
"""The design has no table over positions and config.json gives no limit; this bounds a request's length for the scheduler."""
GATE_ALPHA = 1.702
"""The experts' gate is ``g sigmoid(1.702 g)``; the design fixes the factor."""
HISTORY_KEY = "vazepel_layer_results"


def _need(d: Mapping[str, Any], key: str, where: str) -> Any:
    if not isinstance(d, Mapping) or key not in d:
        raise ConfigError(f"config.json: {where} lacks {key!r}")
    return d[key]


def _pos_int(d: Mapping[str, Any], key: str, where: str) -> int:
    v = _need(d, key, where)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {where}.{key} must be a positive integer, got {v!r}")
    return v


@dataclass(frozen=True)
class VazepelLayer:
    type: str
    mixer: Mapping[str, Any]
    mlp: Mapping[str, Any] | None


@dataclass(frozen=True)
class VazepelConfig:
    width: int
    vocab: int
    eps: float
    layers: tuple[VazepelLayer, ...]
    eos_token_ids: tuple[int, ...] = ()
    architecture: str = "Vazepel"

    @staticmethod
    def from_dict(raw: Mapping[str, Any], generation: Mapping[str, Any] | None = None) -> "VazepelConfig":
        layers = []
        listed = _need(raw, "layers", "the top level")
        if not isinstance(listed, list) or not listed:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        for i, entry in enumerate(listed):
            where = f"layers[{i}]"
            kind = _need(entry, "type", where)
            if kind not in _MIXERS:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not one of {sorted(_MIXERS)}")
            mlp = entry.get("mlp")
            if mlp is not None and _need(mlp, "kind", where + ".mlp") not in _FEED_FORWARDS:
                raise ConfigError(f"config.json: {where}.mlp.kind {mlp['kind']!r} is not one of {sorted(_FEED_FORWARDS)}")
            layers.append(VazepelLayer(kind, dict(_need(entry, "mixer", where)), dict(mlp) if mlp is not None else None))
        eos = raw.get("eos_token_id", [])
        if generation is not None and generation.get("eos_token_id") is not None:
            eos = generation["eos_token_id"]
        eos = [] if eos is None else (list(eos) if isinstance(eos, list) else [eos])
        config = VazepelConfig(
            width=_pos_int(raw, "width", "the top level"), vocab=_pos_int(raw, "vocab", "the top level"),
            eps=float(_need(_need(raw, "norm", "the top level"), "eps", "norm")),
            layers=tuple(layers), eos_token_ids=tuple(int(t) for t in eos), architecture=str(raw.get("architecture", "Vazepel")))
        vazepel_model_spec(config)   # sizes that do not fit each other are config errors, found here
        return config


# ---- one function per mixer kind: config.json's mixer entry -> (mixer part, position part or None)
def _attention(c: VazepelConfig, m: Mapping[str, Any], prefix: str):
    where = prefix + "mixer"
    params = {"hidden_size": c.width, "num_heads": _pos_int(m, "heads", where), "num_kv_heads": _pos_int(m, "kv_heads", where),
              "key_dim": _pos_int(m, "dim", where), "value_dim": _pos_int(m, "vdim", where), "scale": float(_need(m, "scale", where)),
              "biases": True, "softcap": float(_need(m, "softcap", where)), "head_mix": True, "unit_sink": True, "output_gate": True}
    if params["num_heads"] % params["num_kv_heads"]:
        raise ConfigError(f"config.json: {where}: {params['num_heads']} heads are not a multiple of {params['num_kv_heads']} kv_heads")
    if not params["softcap"] > 0:
        raise ConfigError(f"config.json: {where}.softcap must be positive")
    position = None
    rot = m.get("rot")
    if rot:
        position = PartSpec("rope_pairs", {"dims": _pos_int(rot, "dims", where + ".rot"), "base": float(_need(rot, "base", where + ".rot"))})
        if position.params["dims"] % 2 or position.params["dims"] > params["key_dim"]:
            raise ConfigError(f"config.json: {where}.rot.dims must be even and at most the heads' size {params['key_dim']}")
    return PartSpec("mixed_head_attention", params, prefix=prefix + "mix."), position


_MIXERS = {"attention": _attention}


# ---- one function per feed-forward kind
def _dense(c: VazepelConfig, mlp: Mapping[str, Any], prefix: str) -> PartSpec:
    return PartSpec("gelu_mlp", {"hidden_size": c.width, "intermediate_size": _pos_int(mlp, "ff", prefix + "mlp")}, prefix=prefix + "mlp.")


def _gated_unit(c: VazepelConfig, sizes: Mapping[str, Any], where: str) -> dict[str, Any]:
    limit = float(_need(sizes, "limit", where))
    if not limit > 0:
        raise ConfigError(f"config.json: {where}.limit must be positive")
    return {"hidden_size": c.width, "intermediate_size": _pos_int(sizes, "ff", where), "limit": limit, "alpha": GATE_ALPHA}


def _experts(c: VazepelConfig, mlp: Mapping[str, Any], prefix: str) -> PartSpec:
    where = prefix + "mlp"
    router = _need(mlp, "router", where)
    groups = router.get("groups") or {}
    params = {**_gated_unit(c, _need(mlp, "expert", where), where + ".expert"),
              "experts": _pos_int(router, "experts", where + ".router"), "top": _pos_int(router, "top", where + ".router"),
              "groups": _pos_int(groups, "count", where + ".router.groups") if groups else 1,
              "keep": _pos_int(groups, "keep", where + ".router.groups") if groups else 1,
              "activation": "clamped_glu", "score": "softmax", "group_score": "max", "renormalize": False}
    E, G, K, top = params["experts"], params["groups"], params["keep"], params["top"]
    if E % G or K > G or top > K * (E // G):
        raise ConfigError(f"config.json: {where}.router: {top} of {E} experts in {K} of {G} groups do not fit each other")
    if mlp.get("shared"):
        params["shared"] = {"kind": "clamped_glu", "params": _gated_unit(c, mlp["shared"], where + ".shared")}
    return PartSpec("routed_experts", params, prefix=prefix + "mlp.")


_FEED_FORWARDS = {"dense": _dense, "moe": _experts}


def vazepel_model_spec(c: VazepelConfig) -> ModelSpec:
    def norm(name: str) -> PartSpec:
        return PartSpec("layer_norm", {"size": c.width, "eps": c.eps, "bias": True}, prefix=name, names={"weight": "", "bias": ".b"})

    layers = []
    n = len(c.layers)
    for i, layer in enumerate(c.layers):
        p = f"l{i}."
        mixer, position = _MIXERS[layer.type](c, layer.mixer, p)
        ff = _FEED_FORWARDS[layer.mlp["kind"]](c, layer.mlp, p) if layer.mlp is not None else None
        # layer i hands on a weighted sum of the embedding's output and the i + 1 layer results so far
        block = PartSpec("parallel", {"hidden_size": c.width, "gated": True, "depth_states": i + 2, "history_slots": n + 1,
                                      "history_key": HISTORY_KEY}, prefix=p)
        layers.append(LayerSpec(mixer=mixer, mixer_norm=norm(p + "norm1"), feed_forward=ff, feed_forward_norm=None, arrangement="parallel",
                                position=position, block=block))
    return ModelSpec(
        architecture=c.architecture, hidden_size=c.width, vocab_size=c.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": c.vocab, "hidden_size": c.width, "scale": 1.0, "whole_stream": True},
                           prefix="embed", names={"weight": ""}),
        layers=tuple(layers), schedule=tuple(ScheduleEntry(i) for i in range(n)),
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"vocab_size": c.vocab, "hidden_size": c.width, "tied": False}, prefix="head", names={"weight": ""}),
        max_positions=MAX_POSITIONS, eos_token_ids=c.eos_token_ids,
        # a layer without a feed-forward may still carry the gate of one
        ignored_tensors=(r"l\d+\.rg2(\.b)?",))


VAZEPEL = register_architecture(Architecture("Vazepel", VazepelConfig.from_dict, vazepel_model_spec))
