"""Nidudra: a decoder whose config.json lists its layers one by one, from typed config to a description made of registered parts.

Every layer is ``x += norm1(mixer(x))`` and, unless its ``mlp`` is null, ``x += norm2(ff(x))``: the sublayers read the stream itself and the
only norms (RMS, with a weight) stand on their outputs. Three mixers. ``attention``: grouped-query attention without rotation, q and k
RMS-normed per head with a weight, a window beside which a sequence's first tokens stay visible, a sigmoid gate per channel on the
concatenated heads; with ``kv_from: j`` it has no key and value tensors and attends to what layer j cached. ``attention_2``: causal attention
whose first ``rot.dims`` entries per head turn in the half-split layout with frequencies rescaled in three bands, q and k divided by their
root mean square after the rotation, a learned sink per head in the softmax denominator, one sigmoid gate per head. ``parallel``: two mixers
side by side, causal attention with biased q and k behind a short causal filter (the values are the filtered keys; weighted q/k norm, then a
rotation with ramp-rescaled frequencies) and gated linear attention with a low-rank decay per key channel; the two results are RMS-normed
over the width and averaged. Feed-forwards: a SiLU-gated layer (``dense``) or routed SiLU-gated experts chosen by sigmoid scores, which scale
the expert's INPUT, beside a shared expert behind a per-token sigmoid gate (``moe``). The model ends in an RMS norm, an untied head and a
tanh cap on the logits.

Tensor names: ``embed``, ``head``, ``final.norm``, and per layer ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*`` and ``l<i>.mlp.*``:
``mix.{q,k,v,g,o}``, ``mix.{q,k}.norm``, ``mix.sink``; ``mix.left.{q,k,o}``, ``mix.left.{q,k}.{b,conv,norm}``, ``mix.right.{q,k,v,g,o,a1,a2,a2.b,norm}``,
``mix.{left,right}.out``; ``mlp.{gate,up,down}`` or ``mlp.{router, e<j>.{gate,up,down}, shared.{gate,up,down,sg}}``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from oxr_inference_b200.config.model_config import ConfigError
from oxr_inference_b200.config.registry import Architecture, register_architecture
from oxr_inference_b200.parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

DECAY_RANK = 16
"""Width of the decay's low-rank map where nothing says it: config.json does not give it, a checkpoint's ``mix.right.a1`` does by its shape
(random-weights mode may name it as ``rank`` in the mixer's ``right`` entry)."""
MAX_POSITIONS = 1 << 20
"""The design has no table over positions and config.json gives no limit; this bounds a request's length for the scheduler."""

_SWIGLU_NAMES = {"gate_proj.weight": "gate", "up_proj.weight": "up", "down_proj.weight": "down"}


def _need(d: Mapping[str, Any], key: str, where: str) -> Any:
    if not isinstance(d, Mapping) or key not in d:
        raise ConfigError(f"config.json: {where} lacks {key!r}")
    return d[key]


def _pos_int(d: Mapping[str, Any], key: str, where: str) -> int:
    v = _need(d, key, where)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {where}.{key} must be a positive integer, got {v!r}")
    return v


def _int(d: Mapping[str, Any], key: str, where: str) -> int:
    v = _need(d, key, where)
    if isinstance(v, bool) or not isinstance(v, int) or v < 0:
        raise ConfigError(f"config.json: {where}.{key} must be an integer >= 0, got {v!r}")
    return v


@dataclass(frozen=True)
class NidudraLayer:
    type: str
    mixer: Mapping[str, Any]
    mlp: Mapping[str, Any] | None


@dataclass(frozen=True)
class NidudraConfig:
    width: int
    vocab: int
    eps: float
    logit_softcap: float
    layers: tuple[NidudraLayer, ...]
    eos_token_ids: tuple[int, ...] = ()
    architecture: str = "Nidudra"

    @staticmethod
    def from_dict(raw: Mapping[str, Any], generation: Mapping[str, Any] | None = None) -> "NidudraConfig":
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
            layers.append(NidudraLayer(kind, dict(_need(entry, "mixer", where)), dict(mlp) if mlp is not None else None))
        eos = raw.get("eos_token_id", [])
        if generation is not None and generation.get("eos_token_id") is not None:
            eos = generation["eos_token_id"]
        eos = [] if eos is None else (list(eos) if isinstance(eos, list) else [eos])
        cap = raw.get("logit_softcap") or 0.0
        if not float(cap) >= 0:
            raise ConfigError("config.json: logit_softcap must not be negative")
        config = NidudraConfig(
            width=_pos_int(raw, "width", "the top level"), vocab=_pos_int(raw, "vocab", "the top level"),
            eps=float(_need(_need(raw, "norm", "the top level"), "eps", "norm")), logit_softcap=float(cap),
            layers=tuple(layers), eos_token_ids=tuple(int(t) for t in eos), architecture=str(raw.get("architecture", "Nidudra")))
        nidudra_model_spec(config)   # sizes that do not fit each other are config errors, found here
        return config


# ---- the pieces of a mixer entry
def _head_sizes(c: NidudraConfig, m: Mapping[str, Any], where: str) -> dict[str, Any]:
    out = {"hidden_size": c.width, "num_heads": _pos_int(m, "heads", where), "num_kv_heads": _pos_int(m, "kv_heads", where),
           "key_dim": _pos_int(m, "dim", where), "value_dim": _pos_int(m, "vdim", where), "scale": float(_need(m, "scale", where)), "eps": c.eps}
    if out["num_heads"] % out["num_kv_heads"]:
        raise ConfigError(f"config.json: {where}: {out['num_heads']} heads are not a multiple of {out['num_kv_heads']} kv_heads")
    return out


def _rotation(m: Mapping[str, Any], where: str, key_dim: int, scaling_kind: str, scaling_keys: tuple[str, ...]) -> dict[str, Any] | None:
    """The ``rot`` entry of a mixer as the parameters of the half-split rotation, None without one."""
    rot = m.get("rot")
    if not rot:
        return None
    params: dict[str, Any] = {"dims": _pos_int(rot, "dims", where + ".rot"), "base": float(_need(rot, "base", where + ".rot"))}
    if params["dims"] % 2 or params["dims"] > key_dim:
        raise ConfigError(f"config.json: {where}.rot.dims must be even and at most the heads' size {key_dim}")
    if not params["base"] > 1:
        raise ConfigError(f"config.json: {where}.rot.base must be above 1")
    scaling = rot.get("scaling")
    if scaling:
        params["scaling"] = {"kind": scaling_kind, **{k: float(_need(scaling, k, where + ".rot.scaling")) for k in scaling_keys}}
        if not params["scaling"]["factor"] > 0:
            raise ConfigError(f"config.json: {where}.rot.scaling.factor must be positive")
    return params


def _mask(m: Mapping[str, Any], where: str) -> tuple[int, int]:
    mask = _need(m, "mask", where)
    return _pos_int(mask, "size", where + ".mask"), _int(mask, "keep_first", where + ".mask") if "keep_first" in mask else 0


# ---- one function per mixer kind: (config, layer index, checkpoint shapes or None) -> (mixer part, position part, schedule entry's cache_of)
def _windowed_attention(c: NidudraConfig, i: int, shapes=None):
    m, where, prefix = c.layers[i].mixer, f"layers[{i}].mixer", f"l{i}.mix."
    params = _head_sizes(c, m, where)
    window, keep = _mask(m, where)
    params.update(qk_norm="weighted", window=window, keep_first=keep, output_gate="channel")
    source = m.get("kv_from")
    owner = i if source is None else source
    readers = [j for j, other in enumerate(c.layers) if other.type == "attention" and other.mixer.get("kv_from") == owner and j != owner]
    if source is not None:
        if isinstance(source, bool) or not isinstance(source, int) or not 0 <= source < i:
            raise ConfigError(f"config.json: {where}.kv_from must name an earlier layer, got {source!r}")
        theirs = c.layers[source]
        if theirs.type != "attention" or theirs.mixer.get("kv_from") is not None:
            raise ConfigError(f"config.json: {where}.kv_from names layer {source}, which has no keys and values of this kind of its own")
        for key in ("kv_heads", "dim", "vdim"):
            if theirs.mixer.get(key) != m.get(key):
                raise ConfigError(f"config.json: {where}.{key} differs from layer {source}'s, whose keys and values it reads")
        params["borrows_kv"] = True
    # what the shared cache keeps: enough for the owner's mask and every reader's
    masks = [_mask(c.layers[j].mixer, f"layers[{j}].mixer") for j in [owner, *readers]]
    params["cache_window"] = max(w for w, _ in masks)
    params["cache_keep_first"] = max(k for _, k in masks)
    return PartSpec("gated_attention", params, prefix=prefix), None, source


def _sink_attention(c: NidudraConfig, i: int, shapes=None):
    m, where, prefix = c.layers[i].mixer, f"layers[{i}].mixer", f"l{i}.mix."
    params = _head_sizes(c, m, where)
    params.update(qk_norm="unit", norm_after_rotation=True, sink=True, output_gate="head")
    rot = _rotation(m, where, params["key_dim"], "bands", ("factor", "low", "high", "original"))
    return PartSpec("gated_attention", params, prefix=prefix), PartSpec("rope_halves", rot) if rot else None, None


def _side_by_side(c: NidudraConfig, i: int, shapes=None):
    m, where, prefix = c.layers[i].mixer, f"layers[{i}].mixer", f"l{i}.mix."
    left, right = _need(m, "left", where), _need(m, "right", where)
    lp = _head_sizes(c, left, where + ".left")
    if lp["value_dim"] != lp["key_dim"]:
        raise ConfigError(f"config.json: {where}.left: the values are the keys, so vdim must equal dim")
    lp.update(qk_norm="weighted", qk_biases=True, conv_taps=_int(left, "conv", where + ".left") if left.get("conv") else 0, values_are_keys=True)
    rot = _rotation(left, where + ".left", lp["key_dim"], "ramp", ("factor", "original", "fast", "slow"))
    rp = {"hidden_size": c.width, "num_heads": _pos_int(right, "heads", where + ".right"), "key_dim": _pos_int(right, "dim", where + ".right"),
          "value_dim": _pos_int(right, "vdim", where + ".right"), "tau": float(_need(right, "tau", where + ".right")), "eps": c.eps}
    stored = (shapes or {}).get(prefix + "right.a1")
    rp["decay_rank"] = int(stored[0]) if stored else (_pos_int(right, "rank", where + ".right") if "rank" in right else DECAY_RANK)
    if not rp["tau"] > 0:
        raise ConfigError(f"config.json: {where}.right.tau must be positive")
    return PartSpec("mixer_pair", {
        "hidden_size": c.width, "eps": c.eps,
        "left": {"kind": "gated_attention", "params": lp, "position": {"kind": "rope_halves", "params": rot} if rot else None},
        "right": {"kind": "gated_linear_attention", "params": rp}}, prefix=prefix), None, None


_MIXERS = {"attention": _windowed_attention, "attention_2": _sink_attention, "parallel": _side_by_side}


# ---- one function per feed-forward kind
def _dense(c: NidudraConfig, mlp: Mapping[str, Any], prefix: str) -> PartSpec:
    return PartSpec("swiglu", {"hidden_size": c.width, "intermediate_size": _pos_int(mlp, "ff", prefix + "mlp")}, prefix=prefix + "mlp.",
                    names=_SWIGLU_NAMES)


def _experts(c: NidudraConfig, mlp: Mapping[str, Any], prefix: str) -> PartSpec:
    where = prefix + "mlp"
    router = _need(mlp, "router", where)
    params = {"hidden_size": c.width, "intermediate_size": _pos_int(_need(mlp, "expert", where), "ff", where + ".expert"),
              "experts": _pos_int(router, "experts", where + ".router"), "top": _pos_int(router, "top", where + ".router"),
              "activation": "silu_glu", "score": "sigmoid", "renormalize": False, "weight_on": "input"}
    if params["top"] > params["experts"]:
        raise ConfigError(f"config.json: {where}.router: {params['top']} of {params['experts']} experts cannot be chosen")
    names = {}
    if mlp.get("shared"):
        params["shared"] = {"kind": "swiglu", "params": {"hidden_size": c.width, "intermediate_size": _pos_int(mlp["shared"], "ff", where + ".shared")}}
        params["shared_gate"] = True
        names = {"shared." + local: "shared." + stored for local, stored in _SWIGLU_NAMES.items()}
    return PartSpec("routed_experts", params, prefix=prefix + "mlp.", names=names)


_FEED_FORWARDS = {"dense": _dense, "moe": _experts}


def nidudra_model_spec(c: NidudraConfig, shapes: Mapping[str, tuple[int, ...]] | None = None) -> ModelSpec:
    """``shapes``: the checkpoint's tensor shapes (None without a checkpoint); they give the one size config.json leaves out."""
    def norm(name: str) -> PartSpec:
        return PartSpec("rms_norm", {"size": c.width, "eps": c.eps}, prefix=name, names={"weight": ""})

    layers, schedule = [], []
    for i, layer in enumerate(c.layers):
        p = f"l{i}."
        mixer, position, cache_of = _MIXERS[layer.type](c, i, shapes)
        ff = _FEED_FORWARDS[layer.mlp["kind"]](c, layer.mlp, p) if layer.mlp is not None else None
        layers.append(LayerSpec(mixer=mixer, mixer_norm=norm(p + "norm1"), feed_forward=ff, feed_forward_norm=norm(p + "norm2") if ff else None,
                                arrangement="output_norm", position=position))
        schedule.append(ScheduleEntry(i, cache_of=cache_of))
    return ModelSpec(
        architecture=c.architecture, hidden_size=c.width, vocab_size=c.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": c.vocab, "hidden_size": c.width, "scale": 1.0, "whole_stream": True},
                           prefix="embed", names={"weight": ""}),
        layers=tuple(layers), schedule=tuple(schedule),
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"vocab_size": c.vocab, "hidden_size": c.width, "tied": False, "softcap": c.logit_softcap}, prefix="head",
                      names={"weight": ""}),
        max_positions=MAX_POSITIONS, eos_token_ids=c.eos_token_ids,
        # a layer without a feed-forward may still carry the norm of one
        ignored_tensors=(r"l\d+\.norm2",))


NIDUDRA = register_architecture(Architecture("Nidudra", NidudraConfig.from_dict, nidudra_model_spec, shapes_matter=True))
