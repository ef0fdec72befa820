"""Rotary position encodings: the half-split (GPT-NeoX) table, and per-step angles for the interleaved-pairs form."""

from __future__ import annotations

import math

import torch

from oxr_inference_b200 import ops
from oxr_inference_b200.parts.base import POSITION_ENCODINGS, PositionEncoding, Runtime, StepContext


@POSITION_ENCODINGS.register("rope_neox")
class RotaryTable(PositionEncoding):
    """fp32 ``cos`` and ``sin`` of ``position * theta^(-2i/dim)`` for i < dim/2, one row per position.

    Built exactly as the reference builds it: fp32 ``inv_freq``, fp32 outer product, then cos/sin
    (oxr_runtime/language.py:160-165). The reference then rounds the table to the model dtype
    (language.py:167-170); here the angles stay fp32 whatever the activation dtype. The table is computed on the
    host so that it does not depend on the device's math library, then copied once.
    """

    def __init__(self, runtime: Runtime, *, dim: int, theta: float):
        if dim % 2:
            raise ValueError(f"rotary dimension {dim} is odd")
        self.dim, self.theta = int(dim), float(theta)
        inv_freq = 1.0 / (self.theta ** (torch.arange(0, self.dim, 2, dtype=torch.float) / self.dim))
        freqs = torch.outer(torch.arange(runtime.max_positions, dtype=torch.float), inv_freq)
        self.cos = freqs.cos().to(runtime.device).contiguous()
        self.sin = freqs.sin().to(runtime.device).contiguous()

    def tables(self) -> tuple[torch.Tensor, torch.Tensor]:
        return self.cos, self.sin


@POSITION_ENCODINGS.register("rope_pairs")
class RotaryPairs(PositionEncoding):
    """Rotary encoding of entry pairs (2i, 2i+1) of the first ``dims`` entries of a vector: the pair (u, v) at position p becomes
    ``(u cos a - v sin a, v cos a + u sin a)`` with ``a = p * base^(-2i/dims)``. There is no table over all positions: each step
    computes cos and sin for its own tokens, once, shared by every layer with the same ``dims`` and ``base`` (the frequencies, the
    product with the position and the functions in fp64, rounded once to fp32), so no position limit comes from here."""

    def __init__(self, runtime: Runtime, *, dims: int, base: float):
        if dims % 2 or dims <= 0:
            raise ValueError(f"rotary dimension {dims} must be even and positive")
        self.dims, self.base = int(dims), float(base)
        freq = torch.tensor([self.base ** (-2.0 * i / self.dims) for i in range(self.dims // 2)], dtype=torch.float64)
        self.freq = freq.to(runtime.device)

    def tables(self):
        raise NotImplementedError("rope_pairs has per-step angles (step_angles), not a table over all positions")

    def step_angles(self, ctx: StepContext) -> tuple[torch.Tensor, torch.Tensor]:
        key = ("rope_pairs", self.dims, self.base)
        if key not in ctx.shared:
            ctx.shared[key] = ops.rotary_angles(ctx.positions, self.freq)
        return ctx.shared[key]


def banded_frequencies(freq: list[float], *, factor: float, low: float, high: float, original: float) -> list[float]:
    """Frequencies rescaled in three bands by wavelength ``l = 2 pi / f``: kept where ``l < original / high``, divided by ``factor`` where
    ``l > original / low``, and between the two blended linearly in ``s = (original / l - low) / (high - low)`` as
    ``(1 - s) f / factor + s f``."""
    out = []
    for f in freq:
        wave = 2.0 * math.pi / f
        if wave < original / high:
            out.append(f)
        elif wave > original / low:
            out.append(f / factor)
        else:
            s = (original / wave - low) / (high - low)
            out.append((1.0 - s) * f / factor + s * f)
    return out


def ramped_frequencies(freq: list[float], *, dims: int, base: float, factor: float, original: float, fast: float, slow: float) -> tuple[list[float], float]:
    """Frequencies rescaled by a ramp over the pair index: with ``index(t) = dims ln(original / (2 pi t)) / (2 ln base)``, the ramp rises from
    0 at ``max(floor(index(fast)), 0)`` to 1 at ``min(ceil(index(slow)), dims - 1)``, and pair i turns at ``f_i / factor * ramp_i + f_i (1 -
    ramp_i)``. Also returns the factor ``0.1 ln(factor) + 1`` that both cos and sin are multiplied by."""
    def index(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index(fast)), 0)
    hi = min(math.ceil(index(slow)), dims - 1)
    out = []
    for i, f in enumerate(freq):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


@POSITION_ENCODINGS.register("rope_halves")
class RotaryHalves(PositionEncoding):
    """Rotary encoding of the first ``dims`` entries of a vector in the half-split layout: entry i is paired with entry ``i + dims / 2`` and the
    pair (u, v) at position p becomes ``(u cos a - v sin a, v cos a + u sin a)`` with ``a = p * f_i``, ``f_i = base^(-2i/dims)``. ``scaling``
    rescales the frequencies: ``{"kind": "bands", factor, low, high, original}`` (:func:`banded_frequencies`) or ``{"kind": "ramp", factor,
    original, fast, slow}`` (:func:`ramped_frequencies`, which also multiplies cos and sin by a constant). Like ``rope_pairs`` it has no
    table over positions: each step computes cos and sin ``[tokens, dims / 2]`` for its own tokens once (frequencies, product and functions in
    fp64, rounded once to fp32) and layers with equal parameters share them."""

    def __init__(self, runtime: Runtime, *, dims: int, base: float, scaling: dict | None = None):
        if dims % 2 or dims <= 0:
            raise ValueError(f"rotary dimension {dims} must be even and positive")
        self.dims, self.base, self.scaling = int(dims), float(base), dict(scaling) if scaling else None
        freq = [self.base ** (-2.0 * i / self.dims) for i in range(self.dims // 2)]
        self.magnitude = 1.0
        if self.scaling:
            kind = self.scaling.get("kind")
            rest = {k: float(v) for k, v in self.scaling.items() if k != "kind"}
            if kind == "bands":
                freq = banded_frequencies(freq, **rest)
            elif kind == "ramp":
                freq, self.magnitude = ramped_frequencies(freq, dims=self.dims, base=self.base, **rest)
            else:
                raise ValueError(f"rotary scaling {kind!r} is not one of 'bands', 'ramp'")
        self.freq = torch.tensor(freq, dtype=torch.float64).to(runtime.device)

    def tables(self):
        raise NotImplementedError("rope_halves has per-step angles (step_angles), not a table over all positions")

    def step_angles(self, ctx: StepContext) -> tuple[torch.Tensor, torch.Tensor]:
        key = ("rope_halves", self.dims, self.base, tuple(sorted(self.scaling.items())) if self.scaling else None)
        if key not in ctx.shared:
            cos, sin = ops.rotary_angles(ctx.positions, self.freq)
            if self.magnitude != 1.0:
                ops.scale_(cos, self.magnitude)
                ops.scale_(sin, self.magnitude)
            ctx.shared[key] = (cos, sin)
        return ctx.shared[key]
