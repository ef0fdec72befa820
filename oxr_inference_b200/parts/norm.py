"""RMSNorm with the residual add fused in; layer norm (mean and variance, weight and bias) of a stream kept whole."""

from __future__ import annotations

import torch

from oxr_inference_b200 import ops
from oxr_inference_b200.parts.base import NORMS, DeferredLinear, Norm, ParamInfo, Runtime


@NORMS.register("rms_norm")
class RMSNorm(Norm):
    """``out = (x + residual) * rsqrt(mean((x + residual)^2) + eps) * weight`` with the sum kept as the new fp32
    residual (oxr_runtime/language.py:69-72,94-99; layer 0 has no residual yet, language.py:253-257)."""

    def __init__(self, runtime: Runtime, *, size: int, eps: float):
        self.runtime, self.size, self.eps = runtime, int(size), float(eps)
        self.weight: torch.Tensor | None = None

    def parameters(self) -> dict[str, ParamInfo]:
        return {"weight": ParamInfo((self.size,), init="around_one", role="vector")}

    def assign(self, name: str, tensor: torch.Tensor) -> None:
        if name != "weight":
            raise KeyError(name)
        self.weight = tensor.to(device=self.runtime.device, dtype=torch.float32).contiguous()

    accepts_deferred = True

    def forward(self, x, residual, lazy: bool = False):
        """``x``: a tensor, or the part before with its last projection still to do. ``lazy``: whoever takes the result
        passes it to a product and nowhere else, so the row's scale may be left to that product."""
        if isinstance(x, DeferredLinear):
            weight = getattr(x.linear, "weight", None)
            if lazy and weight is not None:
                # a decode step: the product adds itself into the residual stream and leaves the rows' sums of squares;
                # the next part's first projection scales its sums (no norm kernel at all)
                fused = ops.linear_add(x.x, weight, residual, self.weight, self.eps)
                if fused is not None:
                    return fused
            x = x.materialize()
        return ops.add_rms_norm(x, residual, self.weight, self.eps)

    def forward_rows(self, x, residual, rows):
        if isinstance(x, DeferredLinear):
            x = x.materialize()
        return ops.add_rms_norm(x, residual, self.weight, self.eps, rows=rows)[0]

    # ---- for blocks that keep the residual stream whole in fp32 (nothing pending between sublayers)
    def stream_norm(self, stream: torch.Tensor) -> torch.Tensor:
        """``rmsnorm(stream) * weight`` in the activation dtype."""
        return ops.stream_rms_norm(stream, self.weight, self.eps, self.runtime.dtype)

    def stream_rows(self, stream: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
        return ops.stream_rms_norm(stream, self.weight, self.eps, self.runtime.dtype, rows=rows)

    def add_normed(self, stream: torch.Tensor, y: torch.Tensor, then: "RMSNorm | None" = None, rounded: bool = False) -> torch.Tensor | None:
        """``stream += rmsnorm(y) * weight`` in place; with ``then`` (the next sublayer's pre-norm) also returns its output, from the
        same pass over the row; with ``rounded`` (and no ``then``) the new stream rounded to ``y``'s dtype."""
        if then is None:
            return ops.norm_add_norm(stream, y, self.weight, self.eps, rounded=rounded)
        return ops.norm_add_norm(stream, y, self.weight, self.eps, then.weight, then.eps)


@NORMS.register("layer_norm")
class LayerNorm(Norm):
    """``(x - mean(x)) / sqrt(var(x) + eps) * weight + bias`` with the variance as the mean of the squared deviations, computed in fp32 on
    the fp32 stream. It serves arrangements that keep the stream whole (``stream_norm`` / ``stream_rows``); ``bias=False`` leaves the bias
    tensor out."""

    def __init__(self, runtime: Runtime, *, size: int, eps: float, bias: bool = True):
        self.runtime, self.size, self.eps, self.has_bias = runtime, int(size), float(eps), bool(bias)
        self.weight: torch.Tensor | None = None
        self.bias: torch.Tensor | None = None

    def parameters(self) -> dict[str, ParamInfo]:
        out = {"weight": ParamInfo((self.size,), init="around_one", role="vector")}
        if self.has_bias:
            out["bias"] = ParamInfo((self.size,), role="vector")
        return out

    def assign(self, name: str, tensor: torch.Tensor) -> None:
        if name not in self.parameters():
            raise KeyError(name)
        setattr(self, name, tensor.to(device=self.runtime.device, dtype=torch.float32).contiguous())

    def forward(self, x, residual):
        raise ValueError("layer_norm normalises a stream that is kept whole in fp32 (stream_norm); it takes no pending block output")

    def forward_rows(self, x, residual, rows):
        raise ValueError("layer_norm normalises a stream that is kept whole in fp32 (stream_rows); it takes no pending block output")

    def stream_norm(self, stream: torch.Tensor) -> torch.Tensor:
        return ops.stream_layer_norm(stream, self.weight, self.bias, self.eps, self.runtime.dtype)

    def stream_rows(self, stream: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
        return ops.stream_layer_norm(stream, self.weight, self.bias, self.eps, self.runtime.dtype, rows=rows)

    def after_gated_residual(self, stream: torch.Tensor, a: torch.Tensor, f: torch.Tensor | None, **gated) -> torch.Tensor:
        """The gated add of a block's sublayers into the stream (``ops.gated_residual``) and this norm of the result: one kernel with a block
        per row for up to ``FUSED_ROWS`` rows (decode steps and short portions, where a launch and a second pass over the row count), the
        element-wise kernel and then the norm beyond (a prompt's 2,048 rows of 4,096: 95 + 24 us against 267 us in one kernel)."""
        if stream.shape[0] > self.FUSED_ROWS:
            ops.gated_residual(stream, a, f, **gated)
            return self.stream_norm(stream)
        return ops.gated_residual(stream, a, f, norm=(self.weight, self.bias, self.eps), out_dtype=a.dtype, **gated)

    FUSED_ROWS = 256
