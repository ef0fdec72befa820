"""Gated linear attention: a recurrence with a decay per key channel and a fixed-size per-request state instead of a cache that grows."""

from __future__ import annotations

import torch

from oxr_inference_b200 import ops
from oxr_inference_b200.parts.base import MIXERS, LayerCache, Mixer, ParamInfo, PositionEncoding, Runtime, StateNeed, StepContext
from oxr_inference_b200.parts.linear import StackedLinear


@MIXERS.register("gated_linear_attention")
class GatedLinearAttention(Mixer):
    """``q = W_q h / sqrt(key_dim)``, ``k = W_k h`` (``heads x key_dim``), ``v = W_v h`` (``heads x value_dim``); a decay per key channel
    ``alpha = sigmoid(z)^(1 / tau)`` with ``z = W_a2 (W_a1 h) + a2.b`` (a low-rank map, ``heads x key_dim`` wide). Per head, with S zero at a
    sequence's start:

        S_t = diag(alpha_t) S_(t-1) + k_t v_t^T        o_t = S_t^T q_t

    then each head's o is RMS-normed over ``value_dim`` times ``norm [value_dim]`` (shared by the heads), the heads side by side are multiplied
    by ``silu(W_g h)``, then ``W_o``. q, k, v, the gate and the first decay map are one product; the second decay map's result stays in fp32,
    as does everything that enters the recurrence behind the projections. Per request the mixer keeps one fp32 state row: S ``[heads,
    key_dim, value_dim]``; zero for a new request, carried from step to step whatever the cut."""

    def __init__(self, runtime: Runtime, position: PositionEncoding | None, *, hidden_size: int, num_heads: int, key_dim: int, value_dim: int,
                 decay_rank: int, tau: float, eps: float):
        if position is not None:
            raise ValueError("gated_linear_attention takes no position encoding")
        if not tau > 0:
            raise ValueError(f"the decay's temperature must be positive, got {tau}")
        if key_dim > 256:
            raise ValueError(f"the recurrence kernel keeps keys of up to 256 entries per head, got {key_dim}")
        self.runtime = runtime
        self.hidden, self.H, self.DK, self.DV, self.rank = int(hidden_size), int(num_heads), int(key_dim), int(value_dim), int(decay_rank)
        self.tau, self.eps = float(tau), float(eps)
        self.inner, self.keys = self.H * self.DV, self.H * self.DK
        self.in_proj = StackedLinear(runtime, self.hidden, {"q": self.keys, "k": self.keys, "v": self.inner, "g": self.inner, "a1": self.rank})
        self.decay = StackedLinear(runtime, self.rank, {"a2": self.keys})
        self.out = StackedLinear(runtime, self.inner, {"o": self.hidden})
        self.vectors: dict[str, torch.Tensor] = {}
        self.head_norm: torch.Tensor | None = None

    def parameters(self) -> dict[str, ParamInfo]:
        return {**self.in_proj.parameters(), **self.decay.parameters(), **self.out.parameters(),
                "a2.b": ParamInfo((self.keys,), role="vector"), "norm": ParamInfo((self.DV,), init="around_one", role="vector")}

    def assign(self, name: str, tensor: torch.Tensor) -> None:
        for stack in (self.in_proj, self.decay, self.out):
            if name in stack.outs:
                stack.assign(name, tensor)
                return
        if name not in ("a2.b", "norm"):
            raise KeyError(name)
        self.vectors[name] = tensor.to(device=self.runtime.device, dtype=torch.float32).contiguous()

    def finish_loading(self) -> None:
        self.head_norm = self.vectors["norm"].repeat(self.H).contiguous()     # the norm kernel takes one weight per (head, entry)

    def cache_need(self) -> StateNeed:
        return StateNeed((self.H * self.DK * self.DV,), torch.float32)

    def forward(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        proj = self.in_proj(h)                                          # [tokens, q | k | v | g | a1]
        a1_col0 = 2 * self.keys + 2 * self.inner
        z = self.decay(proj[:, a1_col0:].contiguous(), torch.float32)   # [tokens, heads * key_dim], kept in fp32
        o = ops.gla_scan(proj, 0, self.keys, 2 * self.keys, z, self.vectors["a2.b"], heads=self.H, key_dim=self.DK, value_dim=self.DV, tau=self.tau,
                         q_scale=self.DK ** -0.5, state=cache.state, cu_q=ctx.cu_q, state_slots=ctx.state_slots, n_requests=ctx.n_requests)
        return self.out(ops.head_norm_gate(o, proj, 2 * self.keys + self.inner, self.head_norm, self.H, self.eps, silu=True))
