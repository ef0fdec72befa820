"""How a mixer and a feed-forward are arranged into one block."""

from __future__ import annotations

import torch

from oxr_inference_b200 import ops
from oxr_inference_b200.parts.base import ARRANGEMENTS, DeferredLinear, FeedForward, LayerCache, Mixer, Norm, ParamInfo, Part, Runtime, StepContext
from oxr_inference_b200.parts.linear import StackedLinear


@ARRANGEMENTS.register("pre_norm")
class PreNormBlock:
    """``x += mixer(norm1(x)); x += feed_forward(norm2(x))`` (the second sublayer only when the block has a feed-forward), carried as
    (last output not yet added, residual):
    each norm first adds the pending output into the fp32 residual stream (oxr_runtime/language.py:184-187,
    253-257,266-269). Returns the feed-forward's output and the residual; whoever comes next adds them.

    Two optional hand-overs take the norm kernels out of a decode step; each happens only when both sides say that they can.
    A norm that ``accepts_deferred`` gets the part before it with its last projection still to do (:class:`DeferredLinear`;
    with ``defer_output`` the block's own output is left like that for the next block's norm, which the decoder asks for only
    when the next block ``accepts_deferred_input``), so that the product can add itself into the residual stream. And when
    the part behind such a norm ``accepts_lazy_input``, the norm may hand it a not yet normalised ``h`` that its first
    projection normalises itself."""

    supports_deferred = True

    def __init__(self, mixer: Mixer, mixer_norm: Norm, feed_forward: FeedForward | None, feed_forward_norm: Norm | None):
        if (feed_forward is None) != (feed_forward_norm is None):
            raise ValueError("a feed-forward comes with its norm or not at all")
        self.mixer, self.mixer_norm = mixer, mixer_norm
        self.feed_forward, self.feed_forward_norm = feed_forward, feed_forward_norm

    def parts(self) -> dict[str, object]:
        out = {"mixer": self.mixer, "mixer_norm": self.mixer_norm}
        if self.feed_forward is not None:
            out.update(feed_forward=self.feed_forward, feed_forward_norm=self.feed_forward_norm)
        return out

    @property
    def accepts_deferred_input(self) -> bool:
        return bool(self.mixer_norm.accepts_deferred)

    @staticmethod
    def _norm(norm: Norm, x, residual, behind) -> tuple:
        if norm.accepts_deferred:
            return norm.forward(x, residual, lazy=bool(getattr(behind, "accepts_lazy_input", False)))
        if isinstance(x, DeferredLinear):
            x = x.materialize()
        return norm.forward(x, residual)

    def forward(self, x, residual: torch.Tensor | None, ctx: StepContext, cache: LayerCache, defer_output: bool = False):
        if residual is None and torch.is_tensor(x) and x.dtype == torch.float32 and getattr(self.mixer_norm, "runtime", None) is not None \
                and self.mixer_norm.runtime.dtype != torch.float32 and hasattr(self.mixer_norm, "stream_norm"):
            # the embedding handed over the fp32 stream itself (not 16-bit activations): it is the residual, nothing is pending
            h, residual = self.mixer_norm.stream_norm(x), x
        elif x is None:
            # the block before kept the stream whole
            h = self.mixer_norm.stream_norm(residual)
        else:
            h, residual = self._norm(self.mixer_norm, x, residual, self.mixer)
        if self.feed_forward is None:   # the mixer's sublayer only: its output stays pending for whoever comes next
            return self.mixer.forward(h, ctx, cache), residual
        if self.feed_forward_norm.accepts_deferred:
            a = self.mixer.forward_deferred(h, ctx, cache)
        else:
            a = self.mixer.forward(h, ctx, cache)
        h, residual = self._norm(self.feed_forward_norm, a, residual, self.feed_forward)
        return (self.feed_forward.forward_deferred(h) if defer_output else self.feed_forward.forward(h)), residual


@ARRANGEMENTS.register("sandwich_norm")
class SandwichNormBlock:
    """``x += post_norm(mixer(pre_norm(x)))`` and, when the block has a feed-forward, ``x += post_norm(ff(pre_norm(x)))``: a norm on
    both sides of each sublayer. Nothing can stay pending between sublayers (the output is normalised before it is added), so the
    fp32 stream is kept whole: ``forward`` takes it in ``residual`` (or, for the first block, in ``x``), updates it in place and
    returns ``(None, stream)``. The post-norm, the add and the pre-norm that follows inside the block are one kernel."""

    supports_deferred = False
    accepts_deferred_input = False

    def __init__(self, mixer: Mixer, mixer_norm: Norm, feed_forward: FeedForward | None, feed_forward_norm: Norm | None, *,
                 mixer_post_norm: Norm, feed_forward_post_norm: Norm | None = None):
        if (feed_forward is None) != (feed_forward_norm is None) or (feed_forward is None) != (feed_forward_post_norm is None):
            raise ValueError("a feed-forward comes with both of its norms or not at all")
        self.mixer, self.mixer_norm, self.mixer_post_norm = mixer, mixer_norm, mixer_post_norm
        self.feed_forward, self.feed_forward_norm, self.feed_forward_post_norm = feed_forward, feed_forward_norm, feed_forward_post_norm

    def parts(self) -> dict[str, object]:
        out = {"mixer": self.mixer, "mixer_norm": self.mixer_norm, "mixer_post_norm": self.mixer_post_norm}
        if self.feed_forward is not None:
            out.update(feed_forward=self.feed_forward, feed_forward_norm=self.feed_forward_norm, feed_forward_post_norm=self.feed_forward_post_norm)
        return out

    def forward(self, x, residual: torch.Tensor | None, ctx: StepContext, cache: LayerCache, defer_output: bool = False):
        if residual is None:
            if isinstance(x, DeferredLinear):
                x = x.materialize()
            if x.dtype != torch.float32:
                raise ValueError("this arrangement keeps the stream in fp32: the embedding must hand it over whole")
            stream = x
        elif x is not None:
            raise ValueError("this arrangement takes the stream whole; the block before it left an output that is not yet added")
        else:
            stream = residual
        a = self.mixer.forward(self.mixer_norm.stream_norm(stream), ctx, cache)
        if self.feed_forward is None:
            self.mixer_post_norm.add_normed(stream, a)
            return None, stream
        h = self.mixer_post_norm.add_normed(stream, a, then=self.feed_forward_norm)
        self.feed_forward_post_norm.add_normed(stream, self.feed_forward.forward(h))
        return None, stream


@ARRANGEMENTS.register("output_norm")
class OutputNormBlock:
    """``x += norm1(mixer(x))`` and, when the block has a feed-forward, ``x += norm2(ff(x))``: the sublayers read the stream itself and the only
    norms stand on their OUTPUTS. The fp32 stream is kept whole, as in ``sandwich_norm``: ``forward`` takes it in ``residual`` (the first block:
    in ``x``), updates it in place and returns ``(None, stream)``. What a sublayer reads is the stream rounded to the activation dtype (in a
    32-bit engine the stream itself); the norm of a sublayer's output, the add and that rounding for the next sublayer are one kernel. The
    rounded stream a block ends with travels to the next block of this arrangement in the step's shared dictionary."""

    supports_deferred = False
    accepts_deferred_input = False
    _KEY = "output_norm_rounded_stream"

    def __init__(self, mixer: Mixer, mixer_norm: Norm, feed_forward: FeedForward | None, feed_forward_norm: Norm | None):
        if (feed_forward is None) != (feed_forward_norm is None):
            raise ValueError("a feed-forward comes with its norm or not at all")
        if not hasattr(mixer_norm, "add_normed"):
            raise ValueError("the output_norm arrangement keeps the stream whole: its norms must offer add_normed")
        self.mixer, self.mixer_norm, self.feed_forward, self.feed_forward_norm = mixer, mixer_norm, feed_forward, feed_forward_norm

    def parts(self) -> dict[str, object]:
        out = {"mixer": self.mixer, "mixer_norm": self.mixer_norm}
        if self.feed_forward is not None:
            out.update(feed_forward=self.feed_forward, feed_forward_norm=self.feed_forward_norm)
        return out

    def forward(self, x, residual: torch.Tensor | None, ctx: StepContext, cache: LayerCache, defer_output: bool = False):
        if residual is None:
            if isinstance(x, DeferredLinear):
                x = x.materialize()
            if x.dtype != torch.float32:
                raise ValueError("this arrangement keeps the stream in fp32: the embedding must hand it over whole")
            stream = x
        elif x is not None:
            raise ValueError("this arrangement takes the stream whole; the block before it left an output that is not yet added")
        else:
            stream = residual
        dtype = self.mixer_norm.runtime.dtype
        whole = dtype == torch.float32           # a 32-bit engine's sublayers read the stream itself
        kept = ctx.shared.pop(self._KEY, None)
        h = stream if whole else (kept[1] if kept is not None and kept[0] is stream else ops.cast(stream, dtype))
        a = self.mixer.forward(h, ctx, cache)
        h = self.mixer_norm.add_normed(stream, a, rounded=not whole)
        if self.feed_forward is not None:
            h = self.feed_forward_norm.add_normed(stream, self.feed_forward.forward(stream if whole else h), rounded=not whole)
        if not whole:
            ctx.shared[self._KEY] = (stream, h)
        return None, stream


@ARRANGEMENTS.register("parallel")
class ParallelBlock(Part):
    """``x <- x + (mixer(h) + feed_forward(h))`` with ONE norm, ``h = norm(x)``, that both sublayers read (the feed-forward may be absent).
    Two options, each with tensors of the block's own:

    * ``gated``: each sublayer's result is multiplied element by element by ``sigmoid(W h + b)`` before it is added: ``rg1`` / ``rg1.b`` for
      the mixer, ``rg2`` / ``rg2.b`` for the feed-forward (both maps are one product);
    * ``depth_states`` = d > 0: the block keeps its result X as state d - 1 of the step's history (state 0 is the embedding's output, put
      there by the first such block; ``history_slots`` says how many states the model has) and hands on ``sum_{j < d} dwa[j] X_j``
      instead of X. The history lives in the step's shared dictionary under ``history_key``.

    The stream is kept whole in fp32, as in ``sandwich_norm``: ``forward`` takes it in ``residual`` (the first block: in ``x``), updates it
    in place and returns ``(None, stream)``. Gates, both adds, the history entry and the weighted sum are one kernel. When the next block
    is of this arrangement too (``keeps_add_for``), the block hands its sublayers' results on unadded (a :class:`PendingParallelAdd`) and that
    kernel also runs the next block's norm, whose input it has at hand."""

    supports_deferred = False
    accepts_deferred_input = False

    def keeps_add_for(self, after) -> bool:
        """Whether ``after`` (the block that runs next, or None) takes this block's add into its norm."""
        return isinstance(after, ParallelBlock) and hasattr(after.mixer_norm, "after_gated_residual")

    def __init__(self, mixer: Mixer, mixer_norm: Norm, feed_forward: FeedForward | None, feed_forward_norm: Norm | None, *, runtime: Runtime,
                 hidden_size: int, gated: bool = False, depth_states: int = 0, history_slots: int = 0, history_key: str = "depth_history"):
        if feed_forward_norm is not None:
            raise ValueError("the parallel arrangement has one norm: its feed-forward reads the mixer's")
        if depth_states and not 2 <= depth_states <= history_slots:
            raise ValueError(f"a block that averages {depth_states} states needs at least 2 and a history of at least as many slots ({history_slots})")
        if not hasattr(mixer_norm, "stream_norm"):
            raise ValueError("the parallel arrangement keeps the stream whole: its norm must offer stream_norm")
        self.runtime, self.hidden = runtime, int(hidden_size)
        self.mixer, self.mixer_norm, self.feed_forward = mixer, mixer_norm, feed_forward
        self.gated, self.depth_states, self.history_slots, self.history_key = bool(gated), int(depth_states), int(history_slots), str(history_key)
        outs = {"rg1": self.hidden, **({"rg2": self.hidden} if feed_forward is not None else {})}
        self.gates = StackedLinear(runtime, self.hidden, outs) if self.gated else None
        self.vectors: dict[str, torch.Tensor] = {}
        self.gate_bias: torch.Tensor | None = None

    def parts(self) -> dict[str, object]:
        out = {"mixer": self.mixer, "mixer_norm": self.mixer_norm}
        if self.feed_forward is not None:
            out["feed_forward"] = self.feed_forward
        return out

    def _vector_shapes(self) -> dict[str, tuple[int, ...]]:
        out: dict[str, tuple[int, ...]] = {}
        if self.gated:
            out.update({name + ".b": (self.hidden,) for name in self.gates.outs})
        if self.depth_states:
            out["dwa"] = (self.depth_states,)
        return out

    def parameters(self) -> dict[str, ParamInfo]:
        out = dict(self.gates.parameters()) if self.gated else {}
        out.update({name: ParamInfo(shape, role="vector") for name, shape in self._vector_shapes().items()})
        return out

    def assign(self, name: str, tensor: torch.Tensor) -> None:
        if self.gated and name in self.gates.outs:
            self.gates.assign(name, tensor)
        elif name in self._vector_shapes():
            self.vectors[name] = tensor.to(device=self.runtime.device, dtype=torch.float32).contiguous()
        else:
            raise KeyError(name)

    def finish_loading(self) -> None:
        if self.gated:
            self.gate_bias = torch.cat([self.vectors[name + ".b"] for name in self.gates.outs]).contiguous()

    def forward(self, x, residual: torch.Tensor | None, ctx: StepContext, cache: LayerCache, defer_output: bool = False):
        h = None
        if isinstance(x, PendingParallelAdd):
            # the block before left its add to this block's norm: one kernel for both
            stream = residual
            h = x.apply(stream, then=self.mixer_norm)
        elif residual is None:
            if isinstance(x, DeferredLinear):
                x = x.materialize()
            if x.dtype != torch.float32:
                raise ValueError("this arrangement keeps the stream in fp32: the embedding must hand it over whole")
            stream = x
        elif x is not None:
            raise ValueError("this arrangement takes the stream whole; the block before it left an output that is not yet added")
        else:
            stream = residual
        history = None
        if self.depth_states:
            history = ctx.shared.get(self.history_key)
            if history is None:
                # the first averaging block of the step: state 0 is the stream as it came from the embedding
                history = torch.empty((self.history_slots, *stream.shape), dtype=torch.float32, device=stream.device)
                history[0].copy_(stream)
                ctx.shared[self.history_key] = history
        if h is None:
            h = self.mixer_norm.stream_norm(stream)
        a_bias = None
        if hasattr(self.mixer, "forward_parts"):
            a, a_bias = self.mixer.forward_parts(h, ctx, cache)
        else:
            a = self.mixer.forward(h, ctx, cache)
        f = self.feed_forward.forward(h) if self.feed_forward is not None else None
        if f is not None and f.dtype != a.dtype:
            f = ops.cast(f, a.dtype)
        gates = self.gates(h) if self.gated else None
        if gates is not None and gates.dtype != a.dtype:
            gates = ops.cast(gates, a.dtype)
        pending = PendingParallelAdd(a, f, gates, self.gate_bias, a_bias, history, self.depth_states - 1, self.vectors.get("dwa"))
        if defer_output:
            return pending, stream
        pending.apply(stream)
        return None, stream


class PendingParallelAdd:
    """A parallel block's sublayer results, gates and history entry, not yet added to the stream."""

    def __init__(self, a, f, gates, gate_bias, a_bias, history, index, weights):
        self.args = (a, f)
        self.kwargs = dict(gates=gates, gate_bias=gate_bias, a_bias=a_bias, history=history, index=index, weights=weights)

    def apply(self, stream: torch.Tensor, then=None):
        """Add to the stream in place; with ``then`` (a norm that offers ``after_gated_residual``) return that norm's output of the new stream."""
        a, f = self.args
        if then is None:
            ops.gated_residual(stream, a, f, **self.kwargs)
            return None
        return then.after_gated_residual(stream, a, f, **self.kwargs)
