"""A feed-forward of routed experts: each token runs a few of many small feed-forward layers, chosen by a router."""

from __future__ import annotations

from typing import Any, Mapping

import torch

from oxr_inference_b200 import ops
from oxr_inference_b200.parts.base import FEED_FORWARDS, FeedForward, ParamInfo, Runtime


@FEED_FORWARDS.register("routed_experts")
class RoutedExperts(FeedForward):
    """``experts`` feed-forward layers ``e<i>``, no biases, of which each token runs ``top``. An expert is ``down_i( relu(up_i h)^2 )``
    (``activation="relu2"``) or the clamped gated unit ``down_i( g sigmoid(alpha g) (u + 1) )`` with ``g = min(gate_i h, limit)`` and
    ``u = clamp(up_i h, -limit, limit)`` (``"clamped_glu"``) or the SiLU-gated unit ``down_i( silu(gate_i h) * (up_i h) )`` (``"silu_glu"``). The router's logits ``z = W_router h`` are computed in fp32; scores
    ``s = sigmoid(z)`` or the softmax of z over all experts (``score``). The experts form ``groups`` equal groups of neighbours; a group's
    score is the sum of its two largest scores or its largest one (``group_score``), and only experts of the ``keep`` best groups can be
    chosen. Each token runs the ``top`` allowed experts with the largest scores; their outputs are added with weights
    ``s / (sum of the chosen s + 1e-20) * scale`` or, with ``renormalize=False``, ``s * scale``. With ``weight_on="input"`` the weight multiplies
    what the expert READS instead of what it returns: the layer's output is the sum of ``expert_i(w_i h)``. ``shared``: a feed-forward
    (``{"kind": ..., "params": {...}}``, tensors under ``shared.``) that every token runs and whose output is added; with ``shared_gate`` it is
    first multiplied by ``sigmoid(W_sg h)``, one number per token (tensor ``shared.sg [1, hidden]``, the logit in fp32).

    Two forms. Few tokens (decode steps, short portions; also whatever is captured in a CUDA graph): all experts' up-projections are
    stacked into one matrix ``[experts * ff, hidden]`` and their down-projections side by side into ``[hidden, experts * ff]``, so the layer
    is two products whatever the choices: the activation kernel multiplies each expert's stretch of columns by the token's weight for that
    expert (zero when it was not chosen), and the sum over experts happens inside the second product's reduction. With a handful of tokens
    nearly every expert is chosen by someone, and the products are bound by reading the weights, which this form reads exactly once.
    From ``grouped_min_rows`` tokens on the work of the experts nobody chose would dominate, so the (token, choice) pairs are ordered by
    expert on the device and every expert multiplies just its own rows: in bfloat16 as one grouped product per projection (each expert's
    rows padded to whole tiles, each tile with its own expert's matrix; no size comes back to the host), in 32-bit expert by expert after
    the host has read the counts; a last kernel adds each token's ``top`` results with their weights in the order of the choices. Either way a token's result does
    not depend on what else is in the batch beyond rounding."""

    GROUPED_MIN_ROWS = 256

    def __init__(self, runtime: Runtime, *, hidden_size: int, intermediate_size: int, experts: int, top: int, groups: int = 1, keep: int = 1,
                 scale: float = 1.0, grouped_min_rows: int | None = None, activation: str = "relu2", limit: float = 0.0, alpha: float = 1.702,
                 score: str = "sigmoid", group_score: str = "top2_sum", renormalize: bool = True, shared: Mapping[str, Any] | None = None,
                 weight_on: str = "output", shared_gate: bool = False):
        self.runtime = runtime
        if activation not in ("relu2", "clamped_glu", "silu_glu"):
            raise ValueError(f"expert activation {activation!r} is not one of 'relu2', 'clamped_glu', 'silu_glu'")
        if weight_on not in ("output", "input"):
            raise ValueError(f"weight_on {weight_on!r} is not one of 'output', 'input'")
        if weight_on == "input" and activation != "silu_glu":
            raise ValueError("weights on the experts' input are built for the SiLU-gated unit")
        if shared_gate and not shared:
            raise ValueError("a gate on the shared expert needs a shared expert")
        self.activation, self.on_input, self.shared_gate = activation, weight_on == "input", bool(shared_gate)
        self.shared_gate_weight: torch.Tensor | None = None
        if score not in ops.ROUTE_SCORES or group_score not in ops.ROUTE_GROUP_SCORES:
            raise ValueError(f"router score {score!r} / group score {group_score!r}: known are {sorted(ops.ROUTE_SCORES)} / {sorted(ops.ROUTE_GROUP_SCORES)}")
        self.gated = activation in ("clamped_glu", "silu_glu")
        self.limit, self.alpha = float(limit), float(alpha)
        self.score, self.group_score, self.renormalize = score, group_score, bool(renormalize)
        self.shared = FEED_FORWARDS.build(shared["kind"], runtime, **shared.get("params", {})) if shared else None
        self.hidden, self.ff, self.E, self.top = int(hidden_size), int(intermediate_size), int(experts), int(top)
        self.groups, self.keep, self.scale = int(groups), int(keep), float(scale)
        if self.groups < 1 or self.E % self.groups:
            raise ValueError(f"{self.E} experts do not form {self.groups} equal groups")
        if not 1 <= self.keep <= self.groups:
            raise ValueError(f"{self.keep} of {self.groups} groups cannot be kept")
        if not 1 <= self.top <= self.keep * (self.E // self.groups):
            raise ValueError(f"{self.top} experts cannot be chosen from {self.keep} groups of {self.E // self.groups}")
        self.grouped_min_rows = self.GROUPED_MIN_ROWS if grouped_min_rows is None else int(grouped_min_rows)
        self.up_rows = (2 if self.gated else 1) * self.ff     # rows of one expert in the stack: [gate | up] for a gated unit
        self.up: torch.Tensor | None = None       # [E * up_rows, hidden]
        self.down: torch.Tensor | None = None     # [hidden, E * ff]
        self.down_by_expert: torch.Tensor | None = None   # [E, hidden, ff]: made at the first grouped step
        self.router: torch.Tensor | None = None   # [E, hidden]

    def parameters(self) -> dict[str, ParamInfo]:
        out = {"router": ParamInfo((self.E, self.hidden))}
        for e in range(self.E):
            if self.gated:
                out[f"e{e}.gate"] = ParamInfo((self.ff, self.hidden))
            out[f"e{e}.up"] = ParamInfo((self.ff, self.hidden))
            out[f"e{e}.down"] = ParamInfo((self.hidden, self.ff))
        if self.shared is not None:
            out.update({"shared." + name: info for name, info in self.shared.parameters().items()})
        if self.shared_gate:
            out["shared.sg"] = ParamInfo((1, self.hidden))
        return out

    def _stack(self, have: torch.Tensor | None, shape: tuple[int, int], dtype: torch.dtype) -> torch.Tensor:
        if have is None:
            return torch.empty(shape, dtype=dtype, device=self.runtime.device)
        # one expert stored in 32-bit: the whole stack is then kept and multiplied in 32-bit
        return have.float() if dtype == torch.float32 and have.dtype != torch.float32 else have

    def assign(self, name: str, tensor: torch.Tensor) -> None:
        infos = self.parameters()
        if name not in infos:
            raise KeyError(name)
        dtype = self.runtime.store_dtype(infos[name], tensor.dtype)
        if name == "shared.sg" and self.shared_gate:
            self.shared_gate_weight = tensor.to(device=self.runtime.device, dtype=dtype).contiguous()
            return
        if name.startswith("shared."):
            self.shared.assign(name[len("shared."):], tensor)
            return
        if name == "router":
            self.router = tensor.to(device=self.runtime.device, dtype=dtype).contiguous()
            return
        expert, which = name.split(".")
        e = int(expert[1:])
        if which in ("up", "gate"):
            self.up = self._stack(self.up, (self.E * self.up_rows, self.hidden), dtype)
            lo = e * self.up_rows + (self.ff if self.gated and which == "up" else 0)
            self.up[lo:lo + self.ff].copy_(tensor)
        else:
            self.down = self._stack(self.down, (self.hidden, self.E * self.ff), dtype)
            self.down[:, e * self.ff:(e + 1) * self.ff].copy_(tensor)

    def finish_loading(self) -> None:
        if self.shared is not None:
            self.shared.finish_loading()

    def _act(self, u: torch.Tensor, gate: torch.Tensor | None) -> torch.Tensor:
        """The experts' activation over stacked columns, each expert's stretch times the token's weight for it (``gate`` None: one expert)."""
        if self.activation == "silu_glu":
            return ops.expert_silu_glu(u, gate, self.ff, on_input=self.on_input)
        if self.gated:
            return ops.expert_clamped_glu(u, gate, self.ff, alpha=self.alpha, limit=self.limit)
        return ops.gated_relu2(u, gate, self.ff, out=u if gate is None else None)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        z = ops.linear(h, self.router, torch.float32)
        gate, ids, weights = ops.route(z, top=self.top, groups=self.groups, keep=self.keep, scale=self.scale, score=self.score,
                                       group_score=self.group_score, renormalize=self.renormalize)
        if self.top < self.E and h.shape[0] >= self.grouped_min_rows > 0 and not torch.cuda.is_current_stream_capturing():
            y = self._grouped(h, ids, weights)
        else:
            y = ops.linear(self._act(ops.linear(h, self.up), gate), self.down)
        if self.shared is None:
            return y
        if self.shared_gate:
            return ops.add_row_gated_(y, self.shared.forward(h), ops.linear(h, self.shared_gate_weight, torch.float32))
        return ops.add_(y, self.shared.forward(h))

    def _grouped(self, h: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
        """Every expert over the rows that chose it."""
        if self.down_by_expert is None:
            # a second copy of the down-projections, expert by expert (the stacked one is laid out for the single product)
            self.down_by_expert = self.down.view(self.hidden, self.E, self.ff).permute(1, 0, 2).contiguous()
        if ops.grouped_linear_takes(h.dtype, self.up, self.hidden) and ops.grouped_linear_takes(h.dtype, self.down_by_expert, self.ff):
            # bfloat16: each expert's rows padded to whole tiles, then ONE product for all up-projections and one for all
            # down-projections, each tile of rows with its own expert's matrix; nothing comes back to the host
            _, order, place, tile_group = ops.expert_sort(ids, self.E, pad=ops.GROUP_TILE_ROWS)
            x = ops.gather_rows(h, order, self.top)
            if self.on_input:
                ops.scale_placed_rows_(x, place, weights)
                weights = torch.ones_like(weights)
            if self.activation == "silu_glu":
                a = ops.silu_mul(ops.grouped_linear(x, self.up, tile_group, self.up_rows))
            elif self.gated:
                a = ops.clamped_glu(ops.grouped_linear(x, self.up, tile_group, self.up_rows), alpha=self.alpha, limit=self.limit)
            else:
                a = ops.grouped_linear(x, self.up, tile_group, self.ff, relu2=True)     # the activation in the product's epilogue
            y = ops.grouped_linear(a, self.down_by_expert.view(self.E * self.hidden, self.ff), tile_group, self.hidden)
            return ops.combine_rows(y, place, weights)
        counts, order, place, _ = ops.expert_sort(ids, self.E)
        x = ops.gather_rows(h, order, self.top)                  # [tokens * top, hidden], ordered by expert
        if self.on_input:
            ops.scale_placed_rows_(x, place, weights)
            weights = torch.ones_like(weights)
        y = torch.empty((x.shape[0], self.hidden), dtype=x.dtype, device=x.device)
        at = 0
        for e, c in enumerate(counts.tolist()):                  # 32-bit and odd sizes: the host reads the counts (one synchronisation)
            if c:
                u = ops.linear(x[at:at + c], self.up[e * self.up_rows:(e + 1) * self.up_rows])
                ops.linear(self._act(u, None), self.down_by_expert[e], out=y[at:at + c])
                at += c
        return ops.combine_rows(y, place, weights)
