"""Attention mixers whose mask, sizes and extras are arguments: grouped-query attention within chunks with a bias by distance,
latent attention (one compressed row per token that serves as key and value of every head) with a softmax sink, and attention
whose heads' scores are capped and mixed with each other before the softmax."""

from __future__ import annotations

import math

import torch

from oxr_inference_b200 import ops
from oxr_inference_b200.parts.base import MIXERS, LayerCache, Mixer, PagedKVNeed, ParamInfo, PositionEncoding, Runtime, StateNeed, StepContext
from oxr_inference_b200.parts.linear import StackedLinear


def distance_bucket(n: int, rows: int, far: float) -> int:
    """Row of a ``rows``-row bias table for a key ``n`` positions back: one row per distance below ``rows // 2``, then rows spaced
    evenly in the logarithm of the distance up to ``far``; everything at or beyond ``far`` shares the last row."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def bias_by_distance(table: torch.Tensor, far: float) -> torch.Tensor:
    """Expand a bucketed bias table ``[rows, heads]`` into one row per distance ``0 .. ceil(far)``; the last row stands for every
    larger distance (all of them fall into the last bucket). The buckets are worked out on the host in double precision, once."""
    rows = table.shape[0]
    half = rows // 2
    if rows < 2 or far <= half:
        raise ValueError(f"a distance-bias table of {rows} rows needs its far distance ({far}) beyond {half}")
    last = max(half, int(math.ceil(far)))
    index = [distance_bucket(n, rows, far) for n in range(last + 1)]
    if index[-1] != rows - 1:
        raise ValueError("the far distance does not reach the table's last row")
    return table[torch.tensor(index, device=table.device)].contiguous()


@MIXERS.register("masked_attention")
class MaskedAttention(Mixer):
    """``q, k, v = h W^T`` (no rotation) -> K and V into the paged cache -> softmax attention of each new token over the keys it
    sees -> ``W_o``. Query head h reads key/value head ``h // (heads / kv_heads)``; keys have ``key_dim`` entries, values
    ``value_dim``. ``chunk`` > 0: position i sees j <= i only inside its own chunk of that many positions, counted from 0 (not from
    where a prompt was cut). ``window`` > 0: only the last ``window`` keys. ``bias_rows`` > 0: a learned table ``rel [bias_rows, heads]``
    is added to the scaled score by bucketed distance (:func:`distance_bucket`, ``bias_far``).

    Optional, between the projection and the cache: ``biases`` (tensors ``q.b``, ``k.b``, ``v.b`` added to the projections and ``o.b`` to
    the output); ``conv_taps`` > 0: every channel of q, k and v passes a causal filter over time (``q.conv`` ... ``[channels, taps]``, the
    last tap on the current token, zeros before a sequence's start; the last ``taps - 1`` projected values of each request are kept in a
    state slot); ``temp_every`` > 0: the query at position p is multiplied by ``1 + temp_coef ln(floor((p + 1) / temp_every) + 1)``;
    ``value_mix``: ``"keep"`` leaves this layer's values in the step's shared dictionary under ``value_mix_key``, ``"blend"`` replaces its own
    by ``(1 - vmix) v + vmix kept`` (a learned number ``vmix``; the blended values are what the cache holds). Both kinds own a ``vmix``
    tensor; the keeping layer does not use its one."""

    def __init__(self, runtime: Runtime, position: PositionEncoding | None, *, hidden_size: int, num_heads: int, num_kv_heads: int, key_dim: int,
                 value_dim: int, scale: float, chunk: int = 0, window: int = 0, bias_rows: int = 0, bias_far: float = 0.0, biases: bool = False,
                 conv_taps: int = 0, temp_coef: float = 0.0, temp_every: int = 0, value_mix: str | None = None,
                 value_mix_key: str = "kept_values"):
        if position is not None:
            raise ValueError("masked_attention takes no position encoding: positions enter through its mask and bias")
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads are not a multiple of {num_kv_heads} KV heads")
        if value_mix not in (None, "keep", "blend"):
            raise ValueError(f"value_mix {value_mix!r} is not one of None, 'keep', 'blend'")
        self.runtime = runtime
        self.hidden, self.H, self.KV, self.DK, self.DV = int(hidden_size), int(num_heads), int(num_kv_heads), int(key_dim), int(value_dim)
        self.scale, self.chunk, self.window = float(scale), int(chunk), int(window)
        self.bias_rows, self.bias_far = int(bias_rows), float(bias_far)
        self.biases, self.taps = bool(biases), int(conv_taps)
        self.temp_coef, self.temp_every = float(temp_coef), int(temp_every)
        self.value_mix, self.value_mix_key = value_mix, str(value_mix_key)
        self.cq, self.ck, self.cv = self.H * self.DK, self.KV * self.DK, self.KV * self.DV
        self.qkv = StackedLinear(runtime, self.hidden, {"q": self.cq, "k": self.ck, "v": self.cv})
        self.out = StackedLinear(runtime, self.H * self.DV, {"o": self.hidden})
        self.rel: torch.Tensor | None = None
        self.dist_bias: torch.Tensor | None = None
        self.vectors: dict[str, torch.Tensor] = {}
        self.qkv_bias: torch.Tensor | None = None
        self.qkv_conv: torch.Tensor | None = None
        self.qkv_conv_t: torch.Tensor | None = None

    @property
    def between(self) -> bool:
        """Whether anything happens between the projection and the cache (then one kernel does all of it and the cache write)."""
        return self.biases or self.taps > 0 or self.temp_every > 0 or self.value_mix is not None

    @property
    def padded(self) -> int:
        """The one size that keys and values are padded to in the cache (0: no padding). Where keys and values differ in size, the
        tiled tensor-core kernels would not take them; a bfloat16 mixer that writes its cache through ``conv_qkv_store`` and has a plain
        mask therefore keeps both at the larger size (the padding stays zero: it adds nothing to a score and its share of the output
        is dropped), which costs cache space and buys the TMA / tcgen05 kernels instead of the CUDA-core one."""
        size = max(self.DK, self.DV)
        if (self.DK != self.DV and self.between and self.chunk == 0 and self.bias_rows == 0 and self.DK % 8 == 0 and self.DV % 8 == 0
                and ops.tiled_attention_takes(size, size, self.runtime.dtype)):
            return size
        return 0

    @property
    def plain(self) -> bool:
        """Causal or windowed softmax over keys and values of one size: what the TMA / tcgen05 attention kernels take."""
        return self.chunk == 0 and self.bias_rows == 0 and (self.DK == self.DV or self.padded > 0)

    def _vector_shapes(self) -> dict[str, tuple[int, ...]]:
        out: dict[str, tuple[int, ...]] = {}
        sizes = {"q": self.cq, "k": self.ck, "v": self.cv}
        if self.biases:
            out.update({f"{n}.b": (c,) for n, c in sizes.items()})
            out["o.b"] = (self.hidden,)
        if self.taps > 0:
            out.update({f"{n}.conv": (c, self.taps) for n, c in sizes.items()})
        if self.value_mix is not None:
            out["vmix"] = ()
        return out

    def parameters(self) -> dict[str, ParamInfo]:
        out = {**self.qkv.parameters(), **self.out.parameters()}
        if self.bias_rows:
            out["rel"] = ParamInfo((self.bias_rows, self.H), role="vector")
        out.update({name: ParamInfo(shape, role="vector") for name, shape in self._vector_shapes().items()})
        return out

    def assign(self, name: str, tensor: torch.Tensor) -> None:
        if name in self.qkv.outs:
            self.qkv.assign(name, tensor)
        elif name in self.out.outs:
            self.out.assign(name, tensor)
        elif name == "rel" and self.bias_rows:
            self.rel = tensor.to(device=self.runtime.device, dtype=torch.float32).contiguous()
        elif name in self._vector_shapes():
            self.vectors[name] = tensor.to(device=self.runtime.device, dtype=torch.float32).contiguous()
        else:
            raise KeyError(name)

    def finish_loading(self) -> None:
        if self.rel is not None:
            self.dist_bias = bias_by_distance(self.rel, self.bias_far)
        v = self.vectors
        if self.biases:
            self.qkv_bias = torch.cat([v["q.b"], v["k.b"], v["v.b"]]).contiguous()
        if self.taps > 0:
            self.qkv_conv = torch.cat([v["q.conv"], v["k.conv"], v["v.conv"]]).contiguous()
            self.qkv_conv_t = self.qkv_conv.t().contiguous()      # [taps, channels]: what the 16-byte kernel reads
        if self.value_mix is not None:
            v["vmix"] = v["vmix"].reshape(1)

    def cache_need(self):
        # keys and values of one size under a causal or windowed mask: the need of plain grouped-query attention, whose pools get TMA maps
        paged = (PagedKVNeed(self.KV, self.padded or self.DK, self.window) if self.plain else
                 PagedKVNeed(self.KV, self.DK, self.window, value_dim=self.DV, chunk=self.chunk))
        if self.taps > 1:
            return paged, StateNeed(((self.cq + self.ck + self.cv) * (self.taps - 1),), torch.float32)
        return paged

    @property
    def tiled(self) -> bool:
        return self.padded > 0 or ops.tiled_attention_takes(self.DK, self.DV, self.runtime.dtype)

    def kernel_head_dims(self) -> tuple[int, ...]:
        return (self.padded or self.DK,) if self.tiled else ()

    def tile_specs(self) -> list[tuple[int, int, int]]:
        if not self.tiled:
            return []
        return ops.attention_tile_specs(self.H, self.KV, self.padded or self.DK, self.runtime.dtype, self.runtime.page_size if self.plain else None)

    def forward(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        y = self.out(self._attend(h, ctx, cache))
        if self.biases:
            ops.add_bias_(y, self.vectors["o.b"])
        return y

    def _attend(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        group = cache.group
        k_pool, v_pool = group.k_pool[cache.layer_in_group], group.v_pool[cache.layer_in_group]
        qkv = self.qkv(h)
        if qkv.dtype != k_pool.dtype:
            qkv = ops.cast(qkv, k_pool.dtype)
        if self.between:
            blend = first = None
            if self.value_mix == "blend":
                if self.value_mix_key not in ctx.shared:
                    raise ValueError(f"no layer before this one kept its values under {self.value_mix_key!r}")
                blend, first = self.vectors["vmix"], ctx.shared[self.value_mix_key]
            q, kept = ops.conv_qkv_store(
                qkv, self.cq, self.ck, self.cv, conv=self.qkv_conv, conv_t=self.qkv_conv_t, bias=self.qkv_bias, tails=cache.state, k_pool=k_pool, v_pool=v_pool,
                slots=group.slots if cache.store else ctx.no_store_slots, req_of_token=ctx.req_of_token, cu_q=ctx.cu_q,
                state_slots=ctx.state_slots, positions=ctx.positions, n_requests=ctx.n_requests, status=ctx.status, temp_coef=self.temp_coef,
                temp_every=self.temp_every, blend=blend, first=first, keep_values=self.value_mix == "keep", single_tokens=ctx.single_tokens,
                q_head_width=self.padded or None)
            if self.value_mix == "keep":
                ctx.shared[self.value_mix_key] = kept
            q_width = q.shape[1]
        else:
            if cache.store:
                ops.scatter_rows(k_pool, qkv, self.cq, group.slots, ctx.status, pool2=v_pool)   # the k columns, then the v columns
            q, q_width = qkv, qkv.shape[1]
        if self.tiled and q.dtype == torch.bfloat16:
            # keys and values of one size the tiled kernels are built for: tensor cores, split-KV for single tokens
            if self.padded:
                o = ops.paged_attention(q.view(ctx.n_tokens, self.H, self.padded), k_pool, v_pool, tiles=ctx.tiles, cu_q=ctx.cu_q, ctx_lens=ctx.ctx_lens,
                                        block_table=group.block_table, page_size=group.page_size, scale=self.scale, window=self.window,
                                        kv_len_bound=ctx.kv_len_bound, status=ctx.status, kv_maps=group.kv_maps, layer_in_pool=cache.layer_in_group,
                                        uneven=ctx.uneven)
                return o[:, :, :self.DV].contiguous().view(ctx.n_tokens, self.H * self.DV)   # the padding's share of the output is dropped
            q = (q if q_width == self.cq else q[:, :self.cq].contiguous()).view(ctx.n_tokens, self.H, self.DK)
            if self.plain:
                o = ops.paged_attention(q, k_pool, v_pool, tiles=ctx.tiles, cu_q=ctx.cu_q, ctx_lens=ctx.ctx_lens, block_table=group.block_table,
                                        page_size=group.page_size, scale=self.scale, window=self.window, kv_len_bound=ctx.kv_len_bound,
                                        status=ctx.status, kv_maps=group.kv_maps, layer_in_pool=cache.layer_in_group, uneven=ctx.uneven)
            else:
                o = ops.paged_attention(q, k_pool, v_pool, tiles=ctx.tiles, cu_q=ctx.cu_q, ctx_lens=ctx.ctx_lens, block_table=group.block_table,
                                        page_size=group.page_size, scale=self.scale, window=self.window, kv_len_bound=ctx.kv_len_bound,
                                        status=ctx.status, chunk=self.chunk, dist_bias=self.dist_bias)
            return o.view(ctx.n_tokens, self.H * self.DV)
        return ops.attention_rows(q, self.H, k_pool, v_pool, value_dim=self.DV, positions=ctx.positions, req_of_token=ctx.req_of_token,
                                  block_table=group.block_table, scale=self.scale, chunk=self.chunk, window=self.window,
                                  dist_bias=self.dist_bias, status=ctx.status)


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    """Attention over a compressed cache. Per token ``W_dkv h`` gives ``rank`` entries that are RMS-normed (weight ``dkv.norm``) into
    the latent ``c`` and ``rot_dim`` more that are rotated into a key part shared by all heads; only ``[c | rotated part]`` is
    cached. Per head the unrotated key is ``W_uk c`` and the value ``W_uv c``; the query ``W_q h`` is laid out head by head as
    ``[key_dim unrotated | rot_dim rotated]``; the score is ``(q_u . k_u + q_r . k_r) * scale``; causal; optional ``sink``: a learned
    number per head whose exponential joins the softmax denominator (it has no key, no value and is not scaled).

    Computed in the absorbed form, which never builds per-head keys or values: ``q_u . (W_uk c) = (W_uk^T q_u) . c``, so every head
    attends with the query ``[W_uk^T q_u | q_r]`` over the one cached row per token (whose first ``rank`` entries are the value as
    well), and ``W_uv`` is applied to the attention's output."""

    def __init__(self, runtime: Runtime, position: PositionEncoding | None, *, hidden_size: int, num_heads: int, key_dim: int, rot_dim: int,
                 value_dim: int, rank: int, scale: float, eps: float, sink: bool = True):
        if rot_dim and position is None:
            raise ValueError("latent_attention with a rotated part needs a position encoding")
        self.runtime, self.position = runtime, position
        self.hidden, self.H, self.D, self.R, self.DV, self.L = int(hidden_size), int(num_heads), int(key_dim), int(rot_dim), int(value_dim), int(rank)
        self.scale, self.eps, self.has_sink = float(scale), float(eps), bool(sink)
        self.q_dkv = StackedLinear(runtime, self.hidden, {"q": self.H * (self.D + self.R), "dkv": self.L + self.R})
        self.out = StackedLinear(runtime, self.H * self.DV, {"o": self.hidden})
        self.c_norm: torch.Tensor | None = None
        self.sink: torch.Tensor | None = None
        self.uk: torch.Tensor | None = None   # [H, D, L]: W_uk head by head, input-major for q_u -> latent space
        self.uv: torch.Tensor | None = None   # [H, L, DV]: W_uv^T head by head

    def parameters(self) -> dict[str, ParamInfo]:
        out = {**self.q_dkv.parameters(), **self.out.parameters(),
               "dkv.norm": ParamInfo((self.L,), init="around_one", role="vector"),
               "uk": ParamInfo((self.H * self.D, self.L)), "uv": ParamInfo((self.H * self.DV, self.L))}
        if self.has_sink:
            out["sink"] = ParamInfo((self.H,), role="vector")
        return out

    def assign(self, name: str, tensor: torch.Tensor) -> None:
        rt = self.runtime
        if name in self.q_dkv.outs:
            self.q_dkv.assign(name, tensor)
        elif name in self.out.outs:
            self.out.assign(name, tensor)
        elif name == "dkv.norm":
            self.c_norm = tensor.to(device=rt.device, dtype=torch.float32).contiguous()
        elif name == "sink" and self.has_sink:
            self.sink = tensor.to(device=rt.device, dtype=torch.float32).contiguous()
        elif name == "uk":
            self.uk = tensor.to(device=rt.device, dtype=rt.dtype).view(self.H, self.D, self.L).contiguous()
        elif name == "uv":
            self.uv = tensor.to(device=rt.device, dtype=rt.dtype).view(self.H, self.DV, self.L).transpose(1, 2).contiguous()
        else:
            raise KeyError(name)

    def cache_need(self) -> PagedKVNeed:
        return PagedKVNeed(1, self.L + self.R, 0, value_dim=0)

    @property
    def tiled(self) -> bool:
        """The tiled kernels take the cached row as key and as value (both ``rank + rot_dim`` wide; the output's last ``rot_dim`` entries
        are dropped), when that width is one of theirs."""
        return ops.tiled_attention_takes(self.L + self.R, self.L + self.R, self.runtime.dtype)

    def kernel_head_dims(self) -> tuple[int, ...]:
        return (self.L + self.R,) if self.tiled else ()

    def tile_specs(self) -> list[tuple[int, int, int]]:
        return ops.attention_tile_specs(self.H, 1, self.L + self.R, self.runtime.dtype) if self.tiled else []

    def forward(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        group = cache.group
        pool = group.k_pool[cache.layer_in_group]
        n, H, D, R, L = ctx.n_tokens, self.H, self.D, self.R, self.L
        both = self.q_dkv(h)
        if both.dtype != pool.dtype:
            both = ops.cast(both, pool.dtype)
        q_cols = H * (D + R)
        q = both[:, :q_cols].contiguous().view(n, H, D + R)
        down = both[:, q_cols:].contiguous()
        if self.position is not None:
            cos, sin = self.position.step_angles(ctx)
        else:   # no rotated part at all
            cos = sin = torch.empty((n, 0), dtype=torch.float32, device=pool.device)
        q_abs = torch.empty((n, H, L + R), dtype=pool.dtype, device=pool.device)
        ops.latent_prep(pool, down, L, R, self.c_norm, self.eps, q, H, D + R, D, q_abs, L + R, L, cos, sin,
                        group.slots if cache.store else ctx.no_store_slots, ctx.status)
        ops.head_linear(q_abs, 0, q, 0, self.uk)
        if self.tiled and pool.dtype == torch.bfloat16:
            o_lat = ops.paged_attention(q_abs, pool, pool, tiles=ctx.tiles, cu_q=ctx.cu_q, ctx_lens=ctx.ctx_lens, block_table=group.block_table,
                                        page_size=group.page_size, scale=self.scale, window=0, kv_len_bound=ctx.kv_len_bound, status=ctx.status,
                                        sink=self.sink)                       # [n, H, L + R]: the first L entries are the latent output
        else:
            o_lat = ops.attention_rows(q_abs.view(n, H * (L + R)), H, pool, None, value_dim=L, positions=ctx.positions,
                                       req_of_token=ctx.req_of_token, block_table=group.block_table, scale=self.scale, sink=self.sink,
                                       status=ctx.status).view(n, H, L)
        o = torch.empty((n, H, self.DV), dtype=pool.dtype, device=pool.device)
        ops.head_linear(o, 0, o_lat, 0, self.uv)
        return self.out(o.view(n, H * self.DV))


@MIXERS.register("mixed_head_attention")
class MixedHeadAttention(Mixer):
    """Grouped-query attention in which the heads see each other's scores. ``q, k, v = h W^T`` (+ ``q.b``, ``k.b``, ``v.b`` with ``biases``);
    with a position encoding of rotated entry pairs, the first ``dims`` entries of every q and k head turn by the position's angles; the
    scaled score ``s_g = (q_g . k) * scale`` is capped as ``softcap * tanh(s_g / softcap)`` (``softcap`` 0: not capped); with ``head_mix`` a
    learned matrix ``talk [heads, heads]`` makes head h's score ``sum_g talk[h, g] s_g``; causal (``window`` > 0: the last ``window`` keys
    only); ``unit_sink`` adds one to the softmax denominator (a place with score 0 that holds no value); with ``output_gate`` the
    concatenated heads are multiplied by ``sigmoid(h W_g^T)`` (tensor ``g``) before ``W_o`` (+ ``o.b``). Every option stands alone.

    q, k, v and the gate are one product. ``forward_parts`` returns the output projection's result and its bias apart, so that an
    arrangement whose add takes a bias saves the pass over the rows."""

    def __init__(self, runtime: Runtime, position: PositionEncoding | None, *, hidden_size: int, num_heads: int, num_kv_heads: int, key_dim: int,
                 value_dim: int, scale: float, biases: bool = False, softcap: float = 0.0, head_mix: bool = False, unit_sink: bool = False,
                 output_gate: bool = False, window: int = 0):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads are not a multiple of {num_kv_heads} KV heads")
        if position is not None and not hasattr(position, "step_angles"):
            raise ValueError("mixed_head_attention rotates entry pairs by per-step angles (a position encoding with step_angles)")
        if position is not None and position.dims > key_dim:
            raise ValueError(f"{position.dims} rotated entries do not fit heads of {key_dim}")
        if softcap < 0:
            raise ValueError("softcap must not be negative (0 turns it off)")
        self.runtime, self.position = runtime, position
        self.hidden, self.H, self.KV, self.DK, self.DV = int(hidden_size), int(num_heads), int(num_kv_heads), int(key_dim), int(value_dim)
        self.scale, self.softcap, self.window = float(scale), float(softcap), int(window)
        self.biases, self.head_mix, self.unit_sink, self.output_gate = bool(biases), bool(head_mix), bool(unit_sink), bool(output_gate)
        self.cq, self.ck, self.cv = self.H * self.DK, self.KV * self.DK, self.KV * self.DV
        outs = {"q": self.cq, "k": self.ck, "v": self.cv}
        if self.output_gate:
            outs["g"] = self.H * self.DV
        self.qkvg = StackedLinear(runtime, self.hidden, outs)
        self.out = StackedLinear(runtime, self.H * self.DV, {"o": self.hidden})
        self.talk: torch.Tensor | None = None
        self.vectors: dict[str, torch.Tensor] = {}
        self.qkv_bias: torch.Tensor | None = None

    def _vector_shapes(self) -> dict[str, tuple[int, ...]]:
        if not self.biases:
            return {}
        return {"q.b": (self.cq,), "k.b": (self.ck,), "v.b": (self.cv,), "o.b": (self.hidden,)}

    def parameters(self) -> dict[str, ParamInfo]:
        out = {**self.qkvg.parameters(), **self.out.parameters()}
        if self.head_mix:
            out["talk"] = ParamInfo((self.H, self.H), role="vector")
        out.update({name: ParamInfo(shape, role="vector") for name, shape in self._vector_shapes().items()})
        return out

    def assign(self, name: str, tensor: torch.Tensor) -> None:
        if name in self.qkvg.outs:
            self.qkvg.assign(name, tensor)
        elif name in self.out.outs:
            self.out.assign(name, tensor)
        elif name == "talk" and self.head_mix:
            self.talk = tensor.to(device=self.runtime.device, dtype=torch.float32).contiguous()
        elif name in self._vector_shapes():
            self.vectors[name] = tensor.to(device=self.runtime.device, dtype=torch.float32).contiguous()
        else:
            raise KeyError(name)

    def finish_loading(self) -> None:
        if self.biases:
            v = self.vectors
            self.qkv_bias = torch.cat([v["q.b"], v["k.b"], v["v.b"]]).contiguous()

    def cache_need(self) -> PagedKVNeed:
        return PagedKVNeed(self.KV, self.DK, self.window, value_dim=self.DV)

    @property
    def tile(self) -> tuple[int, int] | None:
        """(tokens per tile, query parts per block) of the tensor-core kernel, None where the sizes or the dtype leave the rows kernel."""
        if not hasattr(self, "_tile"):
            self._tile = ops.attention_mix_tile(self.H, self.KV, self.DK, self.DV, self.runtime.dtype)
        return self._tile

    def tile_specs(self) -> list[tuple[int, int, int]]:
        return [(self.tile[0], 1, 1 << 30)] if self.tile is not None else []

    def forward(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        y, bias = self.forward_parts(h, ctx, cache)
        return y if bias is None else ops.add_bias_(y, bias)

    def forward_parts(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> tuple[torch.Tensor, torch.Tensor | None]:
        """``(W_o o, o.b or None)``: the output without its bias, and the bias (fp32) for whoever adds next."""
        group = cache.group
        k_pool, v_pool = group.k_pool[cache.layer_in_group], group.v_pool[cache.layer_in_group]
        proj = self.qkvg(h)
        if proj.dtype != k_pool.dtype:
            proj = ops.cast(proj, k_pool.dtype)
        cos = sin = None
        if self.position is not None:
            cos, sin = self.position.step_angles(ctx)
        ops.bias_rope_store(proj, self.cq, self.ck, self.cv, self.DK, bias=self.qkv_bias, cos=cos, sin=sin, k_pool=k_pool, v_pool=v_pool,
                            slots=group.slots if cache.store else ctx.no_store_slots, status=ctx.status)
        gate = proj[:, self.cq + self.ck + self.cv:] if self.output_gate else None
        if self.tile is not None and proj.dtype == torch.bfloat16:
            o = ops.attention_mix_tiled(proj, self.H, k_pool, v_pool, tile=self.tile, tiles=ctx.tiles[self.tile_specs()[0]], cu_q=ctx.cu_q,
                                        positions=ctx.positions, block_table=group.block_table, kv_len_bound=ctx.kv_len_bound, scale=self.scale,
                                        softcap=self.softcap, head_mix=self.talk, unit_sink=self.unit_sink, window=self.window, gate=gate,
                                        status=ctx.status, single_tokens=ctx.single_tokens)
            return self.out(o), (self.vectors["o.b"] if self.biases else None)
        o = ops.attention_mix_rows(proj, self.H, k_pool, v_pool, positions=ctx.positions, req_of_token=ctx.req_of_token,
                                   block_table=group.block_table, scale=self.scale, softcap=self.softcap, head_mix=self.talk,
                                   unit_sink=self.unit_sink, window=self.window, gate=gate, status=ctx.status)
        return self.out(o), (self.vectors["o.b"] if self.biases else None)
