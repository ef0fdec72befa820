"""Dense feed-forwards: SiLU-gated, clamped gated, and a plain two-matrix layer with the tanh form of GELU."""

from __future__ import annotations

import torch

from oxr_inference_b200 import ops
from oxr_inference_b200.parts.base import FEED_FORWARDS, DeferredLinear, FeedForward, ParamInfo, Runtime
from oxr_inference_b200.parts.linear import StackedLinear


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    """``down( silu(h W_gate^T) * (h W_up^T) )`` with gate and up as one product (oxr_runtime/language.py:266-269,
    102-104). No biases (language.py:229-231)."""

    def __init__(self, runtime: Runtime, *, hidden_size: int, intermediate_size: int):
        self.hidden, self.inter = int(hidden_size), int(intermediate_size)
        # gate and up rows alternate in groups of 8 where the size allows: the decode kernel then holds a gate and its
        # up in one block and applies SiLU in its epilogue
        self.gate_up = StackedLinear(runtime, self.hidden, {"gate_proj.weight": self.inter, "up_proj.weight": self.inter},
                                     interleave=ops.GATE_UP_INTERLEAVE)
        self.down = StackedLinear(runtime, self.inter, {"down_proj.weight": self.hidden})

    def parameters(self) -> dict[str, ParamInfo]:
        return {**self.gate_up.parameters(), **self.down.parameters()}

    def assign(self, name: str, tensor: torch.Tensor) -> None:
        if name in self.gate_up.outs:
            self.gate_up.assign(name, tensor)
        elif name in self.down.outs:
            self.down.assign(name, tensor)
        else:
            raise KeyError(name)

    accepts_lazy_input = True   # h goes into the gate|up projection and nowhere else

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        return self.down(self._gated(h))

    def forward_deferred(self, h: torch.Tensor) -> DeferredLinear:
        return DeferredLinear(self._gated(h), self.down)

    def _gated(self, h: torch.Tensor) -> torch.Tensor:
        return ops.gated_silu_linear(h, self.gate_up.weight, self.gate_up.interleave)


@FEED_FORWARDS.register("clamped_glu")
class ClampedGLU(FeedForward):
    """``down( g sigmoid(alpha g) (u + 1) )`` with ``g = min(h W_gate^T, limit)`` and ``u = clamp(h W_up^T, -limit, limit)``: a gated unit
    whose gate is a sigmoid-approximated GELU (``alpha`` = 1.702), whose linear branch is shifted by one and whose two branches are
    clamped. Gate and up are one product whose epilogue applies the activation (bfloat16, sizes that allow it)."""

    def __init__(self, runtime: Runtime, *, hidden_size: int, intermediate_size: int, limit: float, alpha: float = 1.702):
        self.hidden, self.inter, self.limit, self.alpha = int(hidden_size), int(intermediate_size), float(limit), float(alpha)
        # rows alternate in groups of 8 where the size allows, as in SwiGLU: the products' epilogues then apply the gate form
        self.gate_up = StackedLinear(runtime, self.hidden, {"gate": self.inter, "up": self.inter}, interleave=ops.GATE_UP_INTERLEAVE)
        self.down = StackedLinear(runtime, self.inter, {"down": self.hidden})

    def parameters(self) -> dict[str, ParamInfo]:
        return {**self.gate_up.parameters(), **self.down.parameters()}

    def assign(self, name: str, tensor: torch.Tensor) -> None:
        if name in self.gate_up.outs:
            self.gate_up.assign(name, tensor)
        elif name in self.down.outs:
            self.down.assign(name, tensor)
        else:
            raise KeyError(name)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        return self.down(ops.gated_linear(h, self.gate_up.weight, self.gate_up.interleave, kind="clamped", alpha=self.alpha, limit=self.limit))


@FEED_FORWARDS.register("gelu_mlp")
class GeluMLP(FeedForward):
    """``down( gelu_tanh(h W_up^T) )`` with ``gelu_tanh(z) = 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))``: two matrices, no gate, no
    biases. The activation is evaluated in fp32 on the product's rounded output."""

    def __init__(self, runtime: Runtime, *, hidden_size: int, intermediate_size: int):
        self.hidden, self.inter = int(hidden_size), int(intermediate_size)
        self.up = StackedLinear(runtime, self.hidden, {"up": self.inter})
        self.down = StackedLinear(runtime, self.inter, {"down": self.hidden})

    def parameters(self) -> dict[str, ParamInfo]:
        return {**self.up.parameters(), **self.down.parameters()}

    def assign(self, name: str, tensor: torch.Tensor) -> None:
        if name in self.up.outs:
            self.up.assign(name, tensor)
        elif name in self.down.outs:
            self.down.assign(name, tensor)
        else:
            raise KeyError(name)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        return self.down(ops.gelu_tanh_(self.up(h)))
