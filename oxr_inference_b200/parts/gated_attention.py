"""Grouped-query softmax attention whose heads pass optional steps between projection and cache, whose mask may keep a sequence's first
keys in sight behind a window, whose softmax may have a sink, and whose output may pass a sigmoid gate."""

from __future__ import annotations

import torch

from oxr_inference_b200 import ops
from oxr_inference_b200.parts.base import MIXERS, LayerCache, Mixer, PagedKVNeed, ParamInfo, PositionEncoding, Runtime, StateNeed, StepContext
from oxr_inference_b200.parts.linear import StackedLinear


@MIXERS.register("gated_attention")
class GatedAttention(Mixer):
    """``q, k, v = h W^T`` -> steps on the q and k heads -> K and V into the paged cache -> softmax attention of each new token over the keys
    it sees -> gate -> ``W_o``. Query head h reads key/value head ``h // (heads / kv_heads)``; keys have ``key_dim`` entries, values
    ``value_dim``. Every option stands alone:

    * ``qk_biases``: tensors ``q.b`` and ``k.b`` are added to the projections.
    * ``conv_taps`` > 0: every channel of q and k passes a causal filter over time (``q.conv``, ``k.conv`` ``[channels, taps]``, the last tap on
      the current token, zeros before a sequence's start); the last ``taps - 1`` projected values of each request live in a state slot.
    * ``values_are_keys``: there is no value projection; the values are the keys as they leave the filter (before norm and rotation).
    * ``qk_norm``: ``"weighted"`` = per-head RMS norm times ``q.norm`` / ``k.norm [key_dim]`` (shared by the heads), ``"unit"`` = without a weight;
      ``norm_after_rotation`` puts it behind the rotation instead of before it.
    * a position encoding with per-step angles (``step_angles``) turns the pairs ``(i, i + half)`` of each q and k head.
    * mask: causal; ``window`` > 0: position i sees j only if ``i - j < window`` or ``j < keep_first``.
    * ``sink``: a learned number per head (tensor ``sink``) whose exponential joins the softmax denominator; no key, no value, not scaled.
    * ``output_gate``: ``"channel"`` multiplies the concatenated heads by ``sigmoid(h W_g^T)`` entry by entry (``g [heads * value_dim, hidden]``),
      ``"head"`` multiplies head h by one number ``sigmoid(h W_g^T)_h`` (``g [heads, hidden]``).
    * ``borrows_kv``: the mixer has no key and value tensors at all; its queries attend to the cache that another layer run fills (the
      schedule entry's ``cache_of``). ``cache_window`` / ``cache_keep_first`` say what the shared cache keeps when that differs from this
      mixer's own mask (the owner and every borrower name the same).

    All projections that read h are one product. What stands between it and attention (bias, filter, norm, rotation, cache write) is one
    kernel in fp32 arithmetic."""

    def __init__(self, runtime: Runtime, position: PositionEncoding | None, *, hidden_size: int, num_heads: int, num_kv_heads: int, key_dim: int,
                 value_dim: int, scale: float, eps: float = 0.0, qk_norm: str | None = None, norm_after_rotation: bool = False, qk_biases: bool = False,
                 conv_taps: int = 0, values_are_keys: bool = False, window: int = 0, keep_first: int = 0, sink: bool = False,
                 output_gate: str | None = None, borrows_kv: bool = False, cache_window: int | None = None, cache_keep_first: int | None = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads are not a multiple of {num_kv_heads} KV heads")
        if qk_norm not in ops.HEAD_NORMS:
            raise ValueError(f"qk_norm {qk_norm!r} is not one of {list(ops.HEAD_NORMS)}")
        if output_gate not in (None, "channel", "head"):
            raise ValueError(f"output_gate {output_gate!r} is not one of None, 'channel', 'head'")
        if position is not None and not hasattr(position, "step_angles"):
            raise ValueError("gated_attention rotates by per-step angles (a position encoding with step_angles)")
        if position is not None and position.dims > key_dim:
            raise ValueError(f"{position.dims} rotated entries do not fit heads of {key_dim}")
        if values_are_keys and value_dim != key_dim:
            raise ValueError("values that are the keys have the keys' size")
        if borrows_kv and (values_are_keys or conv_taps > 1):
            raise ValueError("a mixer that borrows keys and values has no key steps of its own")
        if keep_first and not window:
            raise ValueError("first keys are kept in sight behind a window only")
        self.runtime, self.position = runtime, position
        self.hidden, self.H, self.KV, self.DK, self.DV = int(hidden_size), int(num_heads), int(num_kv_heads), int(key_dim), int(value_dim)
        self.scale, self.eps, self.qk_norm, self.norm_after = float(scale), float(eps), qk_norm, bool(norm_after_rotation)
        self.qk_biases, self.taps, self.values_are_keys = bool(qk_biases), int(conv_taps), bool(values_are_keys)
        self.window, self.keep_first, self.has_sink, self.output_gate = int(window), int(keep_first), bool(sink), output_gate
        self.borrows = bool(borrows_kv)
        self.cache_window = self.window if cache_window is None else int(cache_window)
        self.cache_keep_first = self.keep_first if cache_keep_first is None else int(cache_keep_first)
        self.cq, self.ck = self.H * self.DK, 0 if self.borrows else self.KV * self.DK
        self.cv = 0 if (self.borrows or self.values_are_keys) else self.KV * self.DV
        outs = {"q": self.cq}
        if self.ck:
            outs["k"] = self.ck
        if self.cv:
            outs["v"] = self.cv
        if output_gate == "channel":
            outs["g"] = self.H * self.DV
        elif output_gate == "head":
            outs["g"] = self.H
        self.proj = StackedLinear(runtime, self.hidden, outs)
        self.out = StackedLinear(runtime, self.H * self.DV, {"o": self.hidden})
        self.vectors: dict[str, torch.Tensor] = {}
        self.bias: torch.Tensor | None = None
        self.conv: torch.Tensor | None = None
        self.conv_t: torch.Tensor | None = None

    def _vector_shapes(self) -> dict[str, tuple[int, ...]]:
        out: dict[str, tuple[int, ...]] = {}
        sides = {"q": self.cq, **({"k": self.ck} if self.ck else {})}
        if self.qk_biases:
            out.update({f"{n}.b": (c,) for n, c in sides.items()})
        if self.taps > 0:
            out.update({f"{n}.conv": (c, self.taps) for n, c in sides.items()})
        if self.qk_norm == "weighted":
            out.update({f"{n}.norm": (self.DK,) for n in sides})
        if self.has_sink:
            out["sink"] = (self.H,)
        return out

    def parameters(self) -> dict[str, ParamInfo]:
        out = {**self.proj.parameters(), **self.out.parameters()}
        out.update({name: ParamInfo(shape, init="around_one" if name.endswith(".norm") else "normal", role="vector")
                    for name, shape in self._vector_shapes().items()})
        return out

    def assign(self, name: str, tensor: torch.Tensor) -> None:
        if name in self.proj.outs:
            self.proj.assign(name, tensor)
        elif name in self.out.outs:
            self.out.assign(name, tensor)
        elif name in self._vector_shapes():
            self.vectors[name] = tensor.to(device=self.runtime.device, dtype=torch.float32).contiguous()
        else:
            raise KeyError(name)

    def finish_loading(self) -> None:
        v = self.vectors
        sides = ["q"] + (["k"] if self.ck else [])
        if self.qk_biases:
            self.bias = torch.cat([v[f"{n}.b"] for n in sides]).contiguous()
        if self.taps > 0:
            self.conv = torch.cat([v[f"{n}.conv"] for n in sides]).contiguous()
            self.conv_t = self.conv.t().contiguous()      # [taps, channels]: what the 16-byte kernel reads

    # ---- what the mixer keeps
    def cache_need(self):
        paged = PagedKVNeed(self.KV, self.DK, self.cache_window, value_dim=None if self.DV == self.DK else self.DV,
                            keep_first=self.cache_keep_first if self.cache_window > 0 else 0)
        if self.taps > 1:
            return paged, StateNeed(((self.cq + self.ck) * (self.taps - 1),), torch.float32)
        return paged

    @property
    def tiled(self) -> bool:
        """Keys and values of one size that the tensor-core attention kernels take (bfloat16)."""
        return self.DK == self.DV and ops.tiled_attention_takes(self.DK, self.DV, self.runtime.dtype)

    @property
    def plain(self) -> bool:
        """Causal or windowed softmax without a sink or kept first keys: what the TMA / tcgen05 attention kernels take."""
        return not self.has_sink and not (self.window > 0 and self.keep_first > 0)

    def kernel_head_dims(self) -> tuple[int, ...]:
        return (self.DK,) if self.tiled else ()

    def tile_specs(self) -> list[tuple[int, int, int]]:
        if not self.tiled:
            return []
        return ops.attention_tile_specs(self.H, self.KV, self.DK, self.runtime.dtype, self.runtime.page_size if self.plain else None)

    # ---- the step
    def forward(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        group = cache.group
        k_pool, v_pool = group.k_pool[cache.layer_in_group], group.v_pool[cache.layer_in_group]
        n = ctx.n_tokens
        proj = self.proj(h)
        if proj.dtype != k_pool.dtype:
            proj = ops.cast(proj, k_pool.dtype)
        cos = sin = None
        if self.position is not None:
            cos, sin = self.position.step_angles(ctx)
        v = self.vectors
        q = ops.head_prep(proj, q_col0=0, k_col0=self.cq if self.ck else None, v_col0=self.cq + self.ck if self.cv else None,
                          values_are_keys=self.values_are_keys, num_heads=self.H, num_kv_heads=self.KV, key_dim=self.DK, value_dim=self.DV,
                          bias=self.bias, taps=self.conv, taps_t=self.conv_t, tails=cache.state, norm=self.qk_norm, norm_after_rotation=self.norm_after,
                          q_weight=v.get("q.norm"), k_weight=v.get("k.norm"), eps=self.eps, cos=cos, sin=sin, k_pool=k_pool, v_pool=v_pool,
                          slots=group.slots if cache.store else ctx.no_store_slots, req_of_token=ctx.req_of_token, cu_q=ctx.cu_q,
                          state_slots=ctx.state_slots, n_requests=ctx.n_requests, status=ctx.status)
        sink = v.get("sink")
        if self.tiled and q.dtype == torch.bfloat16:
            q3 = q.view(n, self.H, self.DK)
            if self.plain:
                o = ops.paged_attention(q3, k_pool, v_pool, tiles=ctx.tiles, cu_q=ctx.cu_q, ctx_lens=ctx.ctx_lens, block_table=group.block_table,
                                        page_size=group.page_size, scale=self.scale, window=self.window, kv_len_bound=ctx.kv_len_bound,
                                        status=ctx.status, kv_maps=group.kv_maps, layer_in_pool=cache.layer_in_group, uneven=ctx.uneven)
            else:
                o = ops.paged_attention(q3, k_pool, v_pool, tiles=ctx.tiles, cu_q=ctx.cu_q, ctx_lens=ctx.ctx_lens, block_table=group.block_table,
                                        page_size=group.page_size, scale=self.scale, window=self.window, keep_first=self.keep_first,
                                        kv_len_bound=ctx.kv_len_bound, status=ctx.status, sink=sink)
            o = o.view(n, self.H * self.DV)
        else:
            o = ops.attention_rows(q, self.H, k_pool, v_pool, value_dim=self.DV, positions=ctx.positions, req_of_token=ctx.req_of_token,
                                   block_table=group.block_table, scale=self.scale, window=self.window, keep_first=self.keep_first, sink=sink,
                                   status=ctx.status)
        if self.output_gate is not None:
            ops.sigmoid_gate_(o, proj, self.cq + self.ck + self.cv, self.DV, per_head=self.output_gate == "head")
        return self.out(o)
