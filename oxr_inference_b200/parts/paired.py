"""Two mixers side by side that read the same input; what comes out is the mean of their normed results."""

from __future__ import annotations

from typing import Any, Mapping

import torch

from oxr_inference_b200 import ops
from oxr_inference_b200.parts.base import MIXERS, POSITION_ENCODINGS, LayerCache, Mixer, ParamInfo, PositionEncoding, Runtime, StateNeed, StepContext


@MIXERS.register("mixer_pair")
class MixerPair(Mixer):
    """``0.5 * (rmsnorm(left(h)) * left.out + rmsnorm(right(h)) * right.out)``: two registered mixers (``left`` and ``right``: ``{"kind": ...,
    "params": {...}, "position": {"kind": ..., "params": {...}} or None}``, tensors under ``left.`` / ``right.``), each result RMS-normed over the
    model width with a weight of its own before the two are averaged.

    What the two keep between steps is kept side by side: at most one of them may keep pages of keys and values (it gets the layer's page
    group); their fixed-size states share one fp32 row per request, the left one's first."""

    def __init__(self, runtime: Runtime, position: PositionEncoding | None, *, hidden_size: int, eps: float, left: Mapping[str, Any],
                 right: Mapping[str, Any]):
        if position is not None:
            raise ValueError("mixer_pair takes no position encoding of its own: each side names its own")
        self.runtime, self.hidden, self.eps = runtime, int(hidden_size), float(eps)
        self.sides: dict[str, Mixer] = {}
        for name, spec in (("left", left), ("right", right)):
            pos = spec.get("position")
            pos_part = POSITION_ENCODINGS.build(pos["kind"], runtime, **pos.get("params", {})) if pos else None
            self.sides[name] = MIXERS.build(spec["kind"], runtime, pos_part, **spec.get("params", {}))
        from oxr_inference_b200.cache.plan import split_need   # here: the cache package imports the parts' interfaces

        self.weights: dict[str, torch.Tensor] = {}
        needs = {name: split_need(m.cache_need(), f"{name} side: ") for name, m in self.sides.items()}
        if needs["left"][0] is not None and needs["right"][0] is not None:
            raise ValueError("only one side of a mixer pair may keep pages of keys and values")
        self.paged = needs["left"][0] or needs["right"][0]
        self.paged_side = "left" if needs["left"][0] is not None else ("right" if needs["right"][0] is not None else None)
        self.state_cols: dict[str, tuple[int, int]] = {}
        at = 0
        for name, (_, state) in needs.items():
            if state is not None:
                if state.dtype != torch.float32 or len(state.shape) != 1:
                    raise ValueError("the sides' states must be fp32 rows to share one")
                self.state_cols[name] = (at, at + state.shape[0])
                at += state.shape[0]
        self.state_size = at

    def parameters(self) -> dict[str, ParamInfo]:
        out = {f"{name}.out": ParamInfo((self.hidden,), init="around_one", role="vector") for name in self.sides}
        for name, m in self.sides.items():
            out.update({f"{name}.{local}": info for local, info in m.parameters().items()})
        return out

    def assign(self, name: str, tensor: torch.Tensor) -> None:
        side, _, local = name.partition(".")
        if side not in self.sides or not local:
            raise KeyError(name)
        if local == "out":
            self.weights[side] = tensor.to(device=self.runtime.device, dtype=torch.float32).contiguous()
        else:
            self.sides[side].assign(local, tensor)

    def finish_loading(self) -> None:
        for m in self.sides.values():
            m.finish_loading()

    def cache_need(self):
        state = StateNeed((self.state_size,), torch.float32) if self.state_size else None
        if self.paged is not None and state is not None:
            return self.paged, state
        return self.paged if self.paged is not None else state

    def tile_specs(self) -> list[tuple[int, int, int]]:
        return [spec for m in self.sides.values() for spec in m.tile_specs()]

    def kernel_head_dims(self) -> tuple[int, ...]:
        return tuple(d for m in self.sides.values() for d in m.kernel_head_dims())

    def _side_cache(self, name: str, cache: LayerCache) -> LayerCache:
        state = None
        if name in self.state_cols:
            lo, hi = self.state_cols[name]
            state = cache.state[:, lo:hi]        # a view: the kernels take the row stride
        return LayerCache(group=cache.group if name == self.paged_side else None, layer_in_group=cache.layer_in_group, store=cache.store, state=state)

    def forward(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        a = self.sides["left"].forward(h, ctx, self._side_cache("left", cache))
        b = self.sides["right"].forward(h, ctx, self._side_cache("right", cache))
        if b.dtype != a.dtype:
            b = ops.cast(b, a.dtype)
        return ops.pair_norm_mean(a, b, self.weights["left"], self.weights["right"], self.eps)
