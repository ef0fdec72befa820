"""Python entry points of the hand-written sm_100a kernels (``csrc/``), one function per kernel.

Every function launches on torch's current CUDA stream, takes and returns torch tensors (used as storage
only) and raises :class:`KernelError` when a launcher refuses its arguments. There is no CPU path and no
fallback: tensors that are not on a CUDA device are an error, and a missing compiler or failed build raises
``BuildError`` at the first call.

Matrix products (the reference's go to cuBLAS through ``nn.Linear``, oxr_runtime/language.py:223-244): the 32-bit
path, the decode-sized bf16 products (at most ``SKINNY_MAX_ROWS`` rows) and the larger bf16 products all run on
this package's own kernels; ``torch.mm`` is kept only for bf16 matrices whose rows TMA cannot fetch.
"""

from __future__ import annotations

import ctypes
import functools
import os
from ctypes import c_float, c_int, c_longlong, c_size_t, c_void_p

import torch

from oxr_inference_b200.ops import build
from oxr_inference_b200.ops.build import BuildError  # noqa: F401

SKINNY_MAX_ROWS = 16
STREAM_MAX_ROWS = 16
STREAM_GEMM = os.environ.get("OXR_B200_STREAM", "1") != "0"
"""Whether bf16 products of at most ``STREAM_MAX_ROWS`` rows (decode steps) run the weight-streaming kernel (a persistent
block per SM whose producer warp fills a shared-memory ring with cp.async.bulk, also while the kernel before it still
runs) instead of the register-fed skinny kernel. ``OXR_B200_STREAM=0`` switches back, for comparisons."""
STATUS_NAMES = {
    1: "token id outside the vocabulary", 2: "cache slot outside the pool", 3: "position outside the rotary table",
    4: "block table names a page outside the pool", 5: "a bounded wait inside a kernel ran out",
}
_DT = {torch.float32: 0, torch.bfloat16: 1}

CHAIN_KERNELS = os.environ.get("OXR_B200_CHAIN", "1") != "0"
"""Whether RMSNorm, q/k norm + RoPE, split-KV attention and the tcgen05 GEMMs are launched programmatically
dependent on the kernel before them: each is scheduled while its predecessor finishes, fetches what no kernel of the step
writes (weights, old keys) and waits with ``griddepcontrol.wait`` before it touches activations. ``OXR_B200_CHAIN=0``
turns it off."""

launch_count = 0
"""Kernels of this package launched so far in this process (cuBLAS calls are not counted)."""


class KernelError(RuntimeError):
    pass


def _dtype_code(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"dtype {t.dtype} is not supported; kernels take float32 and bfloat16") from None


def _need(t: torch.Tensor, name: str, dtype: torch.dtype | None = None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} is on {t.device}; the kernels run on a CUDA device only (there is no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None) or torch.cuda.current_device


def _stream() -> int:
    """Handle of the current CUDA stream. The raw getter costs a fraction of a microsecond; `torch.cuda.current_stream()`
    builds a Stream object per call (several microseconds, per kernel launch of an eager step)."""
    if _raw_stream is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _done(code: int, what: str) -> None:
    global launch_count
    if code != 0:
        if code >= 1000:
            raise KernelError(f"{what}: CUDA error {code - 1000} at launch")
        raise KernelError(f"{what}: launcher refused its arguments (code {code})")
    launch_count += 1


_core = None


def _lib():
    global _core
    if _core is None:
        lib = build.core_library()
        p, i, f = c_void_p, c_int, c_float
        lib.oxr_embedding.argtypes = [p, p, p, i, i, i, i, i, f, p, p]
        lib.oxr_add_rms_norm.argtypes = [p, p, p, p, p, p, i, i, f, i, p]
        lib.oxr_silu_mul.argtypes = [p, p, i, i, i, i, p]
        lib.oxr_cast.argtypes = [p, p, c_size_t, i, i, p]
        lib.oxr_qk_norm_rope_store.argtypes = [p, p, p, p, p, p, p, p, p, p, i, i, i, i, f, i, c_longlong, i, i, i, i, p, p]
        lib.oxr_gemm_f32_nt.argtypes = [p, p, p, i, i, i, p]
        lib.oxr_gemm_skinny_bf16.argtypes = [p, p, p, i, i, i, i, p]
        lib.oxr_gemm_skinny_gated_bf16.argtypes = [p, p, p, i, i, i, p]
        lib.oxr_gemm_stream_bf16.argtypes = [p, p, p, i, i, i, i, p, p]
        lib.oxr_gemm_stream_gated_bf16.argtypes = [p, p, p, i, i, i, p, p]
        lib.oxr_gemm_stream_add_bf16.argtypes = [p, p, p, p, p, p, p, i, i, i, p, p]
        lib.oxr_gemm_stream_add_bf16.restype = c_int
        lib.oxr_gemm_stream_scaled_bf16.argtypes = [p, p, p, i, f, p, i, i, i, i, p, p]
        lib.oxr_gemm_stream_scaled_bf16.restype = c_int
        lib.oxr_gemm_stream_blocks.argtypes = [i]
        lib.oxr_gemm_stream_blocks.restype = c_int
        lib.oxr_gemm_tcgen05_bf16.argtypes = [p, p, p, i, i, i, i, i, i, p, p, p, p]
        lib.oxr_gemm_tcgen05_pair_bf16.argtypes = [p, p, p, i, i, i, i, i, p, p]
        lib.oxr_gemm_tcgen05_gated_bf16.argtypes = [p, p, p, i, i, i, i, p, p]
        lib.oxr_gemm_few_rows_cluster_bf16.argtypes = [p, p, p, i, i, i, i, i, p, p]
        lib.oxr_gemm_few_rows_max_clusters.argtypes = [i]
        lib.oxr_gemm_tcgen05_pair_gated_bf16.argtypes = [p, p, p, i, i, i, i, p, p]
        lib.oxr_sample.argtypes = [p, p, i, i, p, p, p, p, p, p]
        lib.oxr_sample_chunks.argtypes = [i]
        lib.oxr_sample_chunks.restype = c_int
        lib.oxr_repetition_penalty.argtypes = [p, p, p, p, i, i, p]
        lib.oxr_mark_seen.argtypes = [p, p, p, i, i, p]
        ll = c_longlong
        lib.oxr_stream_rms_norm.argtypes = [p, p, p, p, i, i, f, i, p]
        lib.oxr_norm_add_norm.argtypes = [p, p, p, p, p, i, i, f, f, i, p]
        lib.oxr_concat2_cast.argtypes = [p, p, p, i, i, i, p]
        lib.oxr_add_row_f32.argtypes = [p, p, i, i, p]
        lib.oxr_clamped_glu.argtypes = [p, p, i, i, i, f, f, i, p]
        lib.oxr_rotary_angles.argtypes = [p, p, p, p, i, i, p]
        lib.oxr_mamba_conv.argtypes = [p, p, i, i, i, i, i, i, p, p, p, ll, p, p, p, i, p]
        lib.oxr_mamba_scan.argtypes = [p, p, p, i, i, i, i, i, i, i, p, p, p, p, ll, p, p, i, p]
        lib.oxr_gated_group_norm.argtypes = [p, p, p, i, i, i, p, i, i, f, i, p]
        lib.oxr_attention_rows.argtypes = [p, p, i, p, ll, i, p, ll, i, i, i, i, i, i, p, p, p, i, i, i, f, i, i, i, p, i, p, i, p, p]
        lib.oxr_scatter_rows.argtypes = [p, ll, ll, p, i, i, i, p, i, i, p, p, ll, i, p]
        lib.oxr_latent_prep.argtypes = [p, ll, ll, p, i, i, p, f, p, i, i, i, p, i, i, p, p, i, p, i, i, p, p]
        lib.oxr_head_linear.argtypes = [p, i, i, p, i, i, p, i, i, i, i, i, p]
        lib.oxr_conv_qkv_store.argtypes = [p, p, p, i, i, i, i, i, i, i, p, p, p, p, ll, p, p, p, p, f, i, p, p, p, p, p, ll, i, i, i, i, i, i, i, p, p]
        lib.oxr_add_bias.argtypes = [p, p, i, i, i, p]
        lib.oxr_scale_f32.argtypes = [p, f, ll, p]
        lib.oxr_mlstm_scan.argtypes = [p, p, p, i, i, i, i, i, p, p, i, i, i, f, f, p, ll, p, p, i, p]
        lib.oxr_head_norm_gate.argtypes = [p, p, p, i, i, i, p, i, i, f, i, i, p]
        lib.oxr_route.argtypes = [p, p, p, p, i, i, i, i, i, f, i, i, i, p]
        lib.oxr_gated_relu2.argtypes = [p, p, p, i, i, i, i, p]
        lib.oxr_expert_sort.argtypes = [p, p, p, p, p, i, i, i, i, p]
        lib.oxr_gemm_tcgen05_grouped_bf16.argtypes = [p, p, p, i, i, i, i, p, i, i, i, p, p]
        lib.oxr_gather_rows.argtypes = [p, p, p, i, i, i, i, p]
        lib.oxr_combine_rows.argtypes = [p, p, p, p, i, i, i, i, p]
        lib.oxr_stream_layer_norm.argtypes = [p, p, p, p, p, i, i, f, i, p]
        lib.oxr_gated_residual.argtypes = [p, p, p, p, p, p, i, p, p, i, p, i, i, i, p]
        lib.oxr_gated_residual_norm.argtypes = [p, p, p, p, p, p, p, i, p, p, i, p, i, i, p, p, f, i, p]
        lib.oxr_gelu_tanh.argtypes = [p, p, ll, i, p]
        lib.oxr_add_inplace.argtypes = [p, p, ll, i, p]
        lib.oxr_add_inplace.restype = c_int
        lib.oxr_attention_mix_rows.argtypes = [p, p, i, p, ll, i, p, ll, i, i, i, i, i, i, p, p, p, i, i, i, f, f, p, i, i, p, i, i, p, p]
        lib.oxr_bias_rope_store.argtypes = [p, i, i, i, i, i, p, p, p, i, p, p, ll, p, i, i, p, p]
        lib.oxr_attention_mix_mma.argtypes = [p, p, i, p, p, i, i, i, i, i, i, p, p, i, p, p, i, p, i, i, i, f, f, p, i, i, p, i, i, p, p, p, p]
        lib.oxr_attention_mix_mma.restype = c_int
        lib.oxr_attention_mix_mma_smem.argtypes = [i, i, i, i, i, i]
        lib.oxr_attention_mix_mma_smem.restype = c_longlong
        lib.oxr_expert_clamped_glu.argtypes = [p, p, p, i, i, i, f, f, i, p]
        lib.oxr_head_prep.argtypes = [p, p, p, p, i, i, i, i, i, i, i, i, i, i, i, i, p, p, p, i, p, ll, i, i, p, p, f, p, p, i, p, ll, p, p, p, i, p, p]
        lib.oxr_sigmoid_gate.argtypes = [p, p, i, i, i, i, i, i, i, p]
        lib.oxr_gla_scan.argtypes = [p, p, i, i, i, i, i, p, p, f, i, i, i, f, p, ll, p, p, i, i, p]
        lib.oxr_pair_norm_mean.argtypes = [p, p, p, p, p, i, i, f, i, p]
        lib.oxr_tanh_cap.argtypes = [p, f, ll, p]
        lib.oxr_expert_silu_glu.argtypes = [p, p, p, i, i, i, i, i, p]
        lib.oxr_scale_placed_rows.argtypes = [p, p, p, i, i, i, p]
        lib.oxr_add_row_gated.argtypes = [p, p, p, i, i, i, p]
        for name in ("oxr_head_prep", "oxr_sigmoid_gate", "oxr_gla_scan", "oxr_pair_norm_mean", "oxr_tanh_cap", "oxr_expert_silu_glu",
                     "oxr_scale_placed_rows", "oxr_add_row_gated"):
            getattr(lib, name).restype = c_int
        for name in ("oxr_stream_layer_norm", "oxr_gated_residual", "oxr_gelu_tanh", "oxr_attention_mix_rows", "oxr_bias_rope_store", "oxr_gated_residual_norm",
                     "oxr_expert_clamped_glu"):
            getattr(lib, name).restype = c_int
        for name in ("oxr_stream_rms_norm", "oxr_norm_add_norm", "oxr_concat2_cast", "oxr_add_row_f32", "oxr_clamped_glu", "oxr_rotary_angles",
                     "oxr_mamba_conv", "oxr_mamba_scan", "oxr_gated_group_norm", "oxr_attention_rows", "oxr_scatter_rows", "oxr_latent_prep",
                     "oxr_head_linear", "oxr_conv_qkv_store", "oxr_add_bias", "oxr_scale_f32", "oxr_mlstm_scan", "oxr_head_norm_gate", "oxr_route",
                     "oxr_gated_relu2", "oxr_expert_sort", "oxr_gather_rows", "oxr_combine_rows", "oxr_gemm_tcgen05_grouped_bf16"):
            getattr(lib, name).restype = c_int
        for name in ("oxr_embedding", "oxr_add_rms_norm", "oxr_silu_mul", "oxr_cast", "oxr_qk_norm_rope_store",
                     "oxr_gemm_f32_nt", "oxr_gemm_skinny_bf16", "oxr_gemm_skinny_gated_bf16", "oxr_gemm_stream_bf16", "oxr_gemm_stream_gated_bf16", "oxr_gemm_tcgen05_bf16", "oxr_gemm_tcgen05_pair_bf16", "oxr_gemm_tcgen05_gated_bf16", "oxr_gemm_few_rows_cluster_bf16", "oxr_gemm_few_rows_max_clusters",
                     "oxr_gemm_tcgen05_pair_gated_bf16", "oxr_sample", "oxr_repetition_penalty", "oxr_mark_seen"):
            getattr(lib, name).restype = c_int
        lib.oxr_set_chain.argtypes = [c_int]
        lib.oxr_set_chain.restype = None
        lib.oxr_set_chain(int(CHAIN_KERNELS))
        lib.oxr_set_gate_form.argtypes = [c_int, c_float, c_float]
        lib.oxr_set_gate_form.restype = None
        _core = lib
    return _core


_attn: dict[int, ctypes.CDLL] = {}


def _attn_lib(head_dim: int):
    lib = _attn.get(head_dim)
    if lib is None:
        lib = build.attention_library(head_dim)
        p, i, f = c_void_p, c_int, c_float
        lib.oxr_paged_attention.argtypes = [p, p, p, p, p, p, i, p, p, p, i, i, i, i, i, f, i, i, p, p]
        lib.oxr_paged_attention.restype = c_int
        lib.oxr_paged_attention_bf16.argtypes = [p, p, p, p, p, p, i, p, p, i, p, p, p, i, i, i, i, i, f, i, i, p, p, p, p, i, i, i, i, p, p]
        lib.oxr_paged_attention_masked_bf16.argtypes = [p, p, p, p, p, p, i, p, p, i, p, p, p, i, i, i, i, i, f, i, i, i, p, i, p, i, p, p, p, p, p]
        lib.oxr_paged_attention_masked_bf16.restype = c_int
        lib.oxr_attn_make_kv_maps.argtypes = [p, p, p, ctypes.c_ulonglong, i, i]
        lib.oxr_attn_make_kv_maps.restype = c_int
        lib.oxr_paged_attention_fused_decode_bf16.argtypes = [p, p, p, p, p, p, i, p, p, p, i, i, i, i, i, f, i, i, p, p, p, p, i, i, p, p, p, p, f, i, i,
                                                              p, p]
        lib.oxr_paged_attention_fused_decode_bf16.restype = c_int
        lib.oxr_attn_one_round_of_pieces.argtypes = []
        lib.oxr_attn_one_round_of_pieces.restype = c_int
        lib.oxr_attn_even_cut_slots.argtypes = [i]
        lib.oxr_attn_even_cut_slots.restype = c_int
        lib.oxr_paged_attention_bf16.restype = c_int
        lib.oxr_attn_tile_rows.argtypes = [i]
        lib.oxr_attn_tile_rows.restype = c_int
        lib.oxr_attn_head_dim.restype = c_int
        lib.oxr_attn_last_short_kernel.restype = c_int
        if lib.oxr_attn_head_dim() != head_dim:
            raise BuildError(f"attention library for head size {head_dim} reports {lib.oxr_attn_head_dim()}")
        rows = tuple(lib.oxr_attn_tile_rows(kind) for kind in range(4))
        if rows != (GENERIC_ROWS, DECODE_ROWS, PREFILL_ROWS, PREFILL_ROWS_TMA):
            raise BuildError(f"attention library tiles have {rows} rows; the host builds its tile lists for "
                             f"{(GENERIC_ROWS, DECODE_ROWS, PREFILL_ROWS, PREFILL_ROWS_TMA)}")
        lib.oxr_set_chain.argtypes = [c_int]
        lib.oxr_set_chain.restype = None
        lib.oxr_set_chain(int(CHAIN_KERNELS))
        _attn[head_dim] = lib
    return lib


SHORT_KERNELS = {0: None, 1: "attn_mma_decode_kernel", 2: "attn_tma_decode_kernel", 3: "attn_tma_decode_walk_kernel",
                 4: "attn_tma_decode_walk_kernel (one round)"}


def last_short_attention_kernel(head_dim: int) -> str | None:
    """Name of the split-KV kernel that the last ``paged_attention`` call with short tiles launched for this head size."""
    return SHORT_KERNELS[_attn_lib(head_dim).oxr_attn_last_short_kernel()]


def warm_up(head_dims: tuple[int, ...] = ()) -> None:
    """Build and load what a model needs, before the first step."""
    _lib()
    for d in head_dims:
        _attn_lib(d)


_status: dict[torch.device, torch.Tensor] = {}


def new_status(device: torch.device | str = "cuda") -> torch.Tensor:
    """The device's status word: [code, detail, 0, 0]; kernels write the first error they meet. One per device, shared
    by everything that runs there."""
    device = torch.device(device)
    if device.type == "cuda" and device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    if device not in _status:
        _status[device] = torch.zeros(4, dtype=torch.int32, device=device)
    return _status[device]


def check_status(status: torch.Tensor) -> None:
    """Read the status word (synchronises) and raise if a kernel reported an error; clears it."""
    code, detail = status[:2].tolist()
    if code != 0:
        status.zero_()
        raise KernelError(f"a kernel reported: {STATUS_NAMES.get(code, code)} (at index {detail})")


# --------------------------------------------------------------------------------------------------- ops
def embedding(ids: torch.Tensor, table: torch.Tensor, out_dtype: torch.dtype, status: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """``out[t] = table[ids[t]] * scale`` (oxr_runtime/decode_graph.py:75 has no scale); an id outside the table sets the status word."""
    _need(ids, "ids", torch.int32)
    _need(table, "table")
    n, (vocab, hidden) = ids.numel(), table.shape
    out = torch.empty((n, hidden), dtype=out_dtype, device=table.device)
    code = _lib().oxr_embedding(out.data_ptr(), table.data_ptr(), ids.data_ptr(), n, hidden, vocab, _dtype_code(table),
                                _DT[out_dtype], float(scale), status.data_ptr(), _stream())
    _done(code, "embedding")
    return out


def add_rms_norm(x: torch.Tensor, residual: torch.Tensor | None, weight: torch.Tensor, eps: float, *,
                 rows: torch.Tensor | None = None, keep_residual: bool = True):
    """RMSNorm with the residual add fused in (oxr_runtime/language.py:69-72,94-99).

    ``sum = x + residual`` (fp32; just ``x`` when ``residual`` is None), ``out = sum * rsqrt(mean(sum^2) + eps) *
    weight`` rounded to ``x.dtype``. The fp32 residual stream is updated in place (created when None) and returned
    unless ``keep_residual`` is False. With ``rows`` (int32 indices) only those rows are normalised, output row i
    coming from input row ``rows[i]``; the residual is then left untouched.
    """
    _need(x, "x")
    _need(weight, "weight", torch.float32)
    n, hidden = x.shape
    if weight.numel() != hidden:
        raise KernelError(f"norm weight has {weight.numel()} entries for rows of {hidden}")
    if residual is not None:
        _need(residual, "residual", torch.float32)
        if residual.shape != x.shape:
            raise KernelError(f"residual {tuple(residual.shape)} does not match x {tuple(x.shape)}")
    if rows is not None:
        _need(rows, "rows", torch.int32)
        n_out, res_out = rows.numel(), None
    else:
        n_out = n
        res_out = None if not keep_residual else (residual if residual is not None else
                                                  torch.empty((n, hidden), dtype=torch.float32, device=x.device))
    out = torch.empty((n_out, hidden), dtype=x.dtype, device=x.device)
    code = _lib().oxr_add_rms_norm(out.data_ptr(), _ptr(res_out), x.data_ptr(), _ptr(residual), weight.data_ptr(),
                                   _ptr(rows), n_out, hidden, float(eps), _dtype_code(x), _stream())
    _done(code, "add_rms_norm")
    return out, res_out


def silu_mul(gate_up: torch.Tensor, interleave: int = 0) -> torch.Tensor:
    """``silu(gate) * up`` (oxr_runtime/language.py:102-104) for ``gate_up = [gate | up]`` along the last axis, or,
    with ``interleave`` 8, for gate and up alternating in groups of 8 columns (what ``GATE_UP_INTERLEAVE`` rows of a
    stacked weight produce)."""
    _need(gate_up, "gate_up")
    n, two_i = gate_up.shape
    if two_i % 2:
        raise KernelError("gate_up must have an even number of columns")
    if interleave not in (0, GATE_UP_INTERLEAVE) or (interleave and two_i % (2 * interleave)):
        raise KernelError(f"silu_mul: interleave {interleave} with {two_i} columns")
    out = torch.empty((n, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    code = _lib().oxr_silu_mul(out.data_ptr(), gate_up.data_ptr(), n, two_i // 2, interleave, _dtype_code(gate_up), _stream())
    _done(code, "silu_mul")
    return out


GATE_UP_INTERLEAVE = 8
"""Rows per group when a weight stacks a gate and an up projection alternately: what one block of the skinny GEMM sees
as its rows g and g + 8."""


def gated_silu_linear(x: torch.Tensor, weight: torch.Tensor, interleave: int = 0) -> torch.Tensor:
    """``silu(x Wg^T) * (x Wu^T)``: :func:`gated_linear` with the SiLU form."""
    return gated_linear(x, weight, interleave)


GATE_KINDS = {"silu": 0, "clamped": 1}


def gated_linear(x: torch.Tensor, weight: torch.Tensor, interleave: int = 0, *, kind: str = "silu", alpha: float = 1.0,
                 limit: float = 0.0) -> torch.Tensor:
    """``gate_form(x Wg^T, x Wu^T)`` for a weight that stacks Wg and Wu: side by side (``interleave`` 0: one product,
    then the activation kernel) or alternating in groups of 8 rows. ``kind`` "silu": ``silu(g) * u``; "clamped": with ``g' = min(g, limit)``
    and ``u' = clamp(u, -limit, limit)``, ``g' * sigmoid(alpha g') * (u' + 1)``. With alternating rows a bf16 product runs the kernel
    ``linear`` would pick for its size (skinny, one-SM or two-SM tcgen05) with an epilogue that applies the form to the fp32
    sums and writes the gated product alone; 32-bit runs the product and then the activation kernel on interleaved columns.
    ``x`` may be a :class:`NormedLazily`."""
    _lib().oxr_set_gate_form(GATE_KINDS[kind], float(alpha), float(limit))   # read by the gated launchers below, handed to their kernels by value
    if isinstance(x, NormedLazily):
        out = _scaled_linear(x, weight, gated=True) if interleave == GATE_UP_INTERLEAVE else None
        if out is not None:
            return out
        x = x.materialize()
    _need(x, "x")
    _need(weight, "weight")
    m, k = x.shape
    n = weight.shape[0]
    fused = (interleave == GATE_UP_INTERLEAVE and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and n % 16 == 0
             and k % 8 == 0 and weight.shape[1] == k and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0)
    if fused:
        lib = _lib()
        out = torch.empty((m, n // 2), dtype=torch.bfloat16, device=x.device)
        if STREAM_GEMM and m <= STREAM_MAX_ROWS:
            _done(lib.oxr_gemm_stream_gated_bf16(out.data_ptr(), x.data_ptr(), weight.data_ptr(), m, n, k,
                                                 new_status(x.device).data_ptr(), _stream()), "gemm_stream_gated")
        elif m <= SKINNY_MAX_ROWS:
            _done(lib.oxr_gemm_skinny_gated_bf16(out.data_ptr(), x.data_ptr(), weight.data_ptr(), m, n, k, _stream()), "gemm_skinny_gated")
        elif _gemm_pair_plan(m, n, k):
            _done(lib.oxr_gemm_tcgen05_pair_gated_bf16(out.data_ptr(), x.data_ptr(), weight.data_ptr(), m, n, k, _gemm_pair_plan(m, n, k),
                                                       new_status(x.device).data_ptr(), _stream()), "gemm_tcgen05_pair_gated")
        else:
            tile_n, _ = _gemm_plan(m, n, k, False)   # the gated epilogue has no shares of k
            _done(lib.oxr_gemm_tcgen05_gated_bf16(out.data_ptr(), x.data_ptr(), weight.data_ptr(), m, n, k, tile_n,
                                                  new_status(x.device).data_ptr(), _stream()), "gemm_tcgen05_gated")
        return out
    if kind == "silu":
        return silu_mul(linear(x, weight), interleave)
    return clamped_glu(linear(x, weight), alpha=alpha, limit=limit, interleave=interleave)


def cast(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    if x.dtype == dtype:
        return x
    _need(x, "x")
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    code = _lib().oxr_cast(out.data_ptr(), x.data_ptr(), x.numel(), _dtype_code(x), _DT[dtype], _stream())
    _done(code, "cast")
    return out


def qk_norm_rope_store(qkv: torch.Tensor, q_weight: torch.Tensor | None, k_weight: torch.Tensor | None,
                       cos: torch.Tensor | None, sin: torch.Tensor | None, positions: torch.Tensor,
                       slots: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, num_heads: int,
                       num_kv_heads: int, head_dim: int, eps: float, status: torch.Tensor) -> torch.Tensor:
    """Per-head RMSNorm of q and k, rotary encoding of both, K and V stored at ``slots`` of one layer's pool;
    returns q ``[n, H, D]`` (oxr_runtime/kernels.py:66-99). A None weight skips that norm, None tables skip the
    rotation, a negative slot skips that token's store."""
    _need(qkv, "qkv")
    _need(positions, "positions", torch.int32)
    _need(slots, "slots", torch.int32)
    _need(k_cache, "k_cache", qkv.dtype)
    _need(v_cache, "v_cache", qkv.dtype)
    n = qkv.shape[0]
    width = (num_heads + 2 * num_kv_heads) * head_dim
    if qkv.shape[1] != width:
        raise KernelError(f"qkv has {qkv.shape[1]} columns, expected (H + 2 KV) * D = {width}")
    for w, nm in ((q_weight, "q_weight"), (k_weight, "k_weight")):
        if w is not None:
            _need(w, nm, torch.float32)
            if w.numel() != head_dim:
                raise KernelError(f"{nm} has {w.numel()} entries for head size {head_dim}")
    rotate = cos is not None
    max_positions = 0
    if rotate:
        _need(cos, "cos", torch.float32)
        _need(sin, "sin", torch.float32)
        if cos.shape[1] != head_dim // 2 or sin.shape != cos.shape:
            raise KernelError("rotary tables must be [max_positions, head_dim / 2]")
        max_positions = cos.shape[0]
    num_slots = k_cache.numel() // (num_kv_heads * head_dim)
    q = torch.empty((n, num_heads, head_dim), dtype=qkv.dtype, device=qkv.device)
    code = _lib().oxr_qk_norm_rope_store(
        q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), qkv.data_ptr(), _ptr(q_weight), _ptr(k_weight), _ptr(cos),
        _ptr(sin), positions.data_ptr(), slots.data_ptr(), n, num_heads, num_kv_heads, head_dim, float(eps),
        max_positions, num_slots, int(q_weight is not None), int(k_weight is not None), int(rotate), _dtype_code(qkv),
        status.data_ptr(), _stream())
    _done(code, "qk_norm_rope_store")
    return q


GENERIC_ROWS, DECODE_ROWS, PREFILL_ROWS, PREFILL_ROWS_TMA = 16, 16, 64, 256
SHORT_MAX_TOKENS = 8
"""Requests that bring at most this many tokens go to the split-KV kernel, longer portions to the prefill kernel."""
MAX_SPLITS = 32


@functools.lru_cache(maxsize=None)
def num_sms() -> int:
    """Multiprocessors of the current device (the launchers ask the device as well); where no device is present, as
    when plans are inspected on a machine without a GPU, a B200's 148."""
    if torch.cuda.is_available():
        return int(torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count)
    return 148


def _tokens_per_tile(num_heads: int, num_kv_heads: int, rows: int) -> int:
    return rows // min(num_heads // num_kv_heads, rows)


def tma_gathers_possible(head_dim: int, page_size: int, dtype: torch.dtype) -> bool:
    """Whether K and V of such a cache can be fetched by TMA: bf16, head size a multiple of 64, pages of 8 * 2^k tokens."""
    return dtype == torch.bfloat16 and head_dim % 64 == 0 and page_size >= 8 and page_size & (page_size - 1) == 0


def _long_rows(head_dim: int, tma: bool) -> int:
    return PREFILL_ROWS_TMA if tma and head_dim <= 128 else PREFILL_ROWS


def attention_tile_specs(num_heads: int, num_kv_heads: int, head_dim: int, dtype: torch.dtype,
                         page_size: int | None = None) -> list[tuple[int, int, int]]:
    """The tile lists the attention kernels of this dtype read: (tokens per tile, fewest, most new tokens of the
    requests the list covers). The host cuts each request's new tokens into such tiles. With a ``page_size`` that
    allows TMA gathers the long tiles are 256 rows (the tcgen05 prefill kernel), else 64."""
    build.check_head_dim(head_dim)
    big = 1 << 30
    if dtype == torch.bfloat16:
        tma = page_size is not None and tma_gathers_possible(head_dim, page_size, dtype)
        return [(_tokens_per_tile(num_heads, num_kv_heads, DECODE_ROWS), 1, SHORT_MAX_TOKENS),
                (_tokens_per_tile(num_heads, num_kv_heads, _long_rows(head_dim, tma)), SHORT_MAX_TOKENS + 1, big)]
    return [(_tokens_per_tile(num_heads, num_kv_heads, GENERIC_ROWS), 1, big)]


DECODE_BLOCKS_PER_SM = 2
"""Blocks of the split-KV kernel that fit on one SM (its shared memory is the limit)."""


DECODE_CUT = os.environ.get("OXR_B200_DECODE_CUT", "auto")
"""How the split-KV kernel with TMA gathers cuts a step's keys: ``equal``: every request
into the same number of pieces; ``even``: ALL key blocks of the step dealt out evenly to one round of blocks, so that
requests of very different lengths still give every block the same share (a block's run may end one request and begin the
next); ``auto`` (default): the even cut for the steps whose caller says that the lengths differ much (``uneven``), equal
pieces otherwise (with lengths alike the even cut only costs: 3 us per layer at batch 8), and equal pieces also for more than
``EVEN_CUT_MAX_TILES`` requests: the engine runs a decode step's requests longest first, so that hundreds of them dealt out
piece by piece come out even by themselves (decode steps of Qwen3-4B sizes, contexts drawn up to 2,048 to 8,192 keys, eight
layers: 8 requests 0.98 against 1.05 ms, 64: 1.83 against 2.10, 128: 1.97 against 2.30, 256: 3.34 against 3.24)."""
EVEN_CUT_MAX_TILES = 192


def attention_splits(n_short_tiles: int, num_heads: int, num_kv_heads: int, kv_len_bound: int) -> int:
    """Into how many pieces the split-KV kernel cuts each request's keys. Blocks run in waves of
    ``num_sms() * DECODE_BLOCKS_PER_SM``; a block walks its piece's 64-key blocks one after the other and spends about
    as long as 4.5 of them before its first keys arrive and after its last (measured on a B200: 7 us against 1.6 us per
    block). The number of pieces with the least waves x (4.5 + blocks per piece) wins, the smaller among equals; no
    piece is shorter than 128 keys. Depends only on sizes the host knows before the step (fixed inside a CUDA
    graph)."""
    group = num_heads // num_kv_heads
    blocks = max(1, n_short_tiles * num_kv_heads * -(-group // min(group, DECODE_ROWS)))
    slots = num_sms() * DECODE_BLOCKS_PER_SM
    key_blocks = max(1, -(-kv_len_bound // 64))
    best, best_cost = 1, None
    for splits in range(1, max(1, min(MAX_SPLITS, kv_len_bound // 128)) + 1):
        cost = -(-blocks * splits // slots) * (4.5 + -(-key_blocks // splits))
        if best_cost is None or cost < best_cost:
            best, best_cost = splits, cost
    return best


class KVMaps:
    """The two TMA tensor maps (K, V) of one cache group's pool, in 64-byte aligned host memory."""

    def __init__(self, raw: ctypes.Array, address: int, pool_ptrs: tuple[int, int], rows_per_layer: int):
        self.raw, self.address, self.pool_ptrs, self.rows_per_layer = raw, address, pool_ptrs, rows_per_layer


def make_kv_maps(k_pool: torch.Tensor, v_pool: torch.Tensor, page_size: int) -> KVMaps | None:
    """Tensor maps over a group's whole pool ``[layers, pages, page_size, KV, D]`` so that the split-KV kernel can
    fetch K and V by TMA; None when the sizes do not allow it (the kernel then gathers with cp.async)."""
    if k_pool.dtype != torch.bfloat16 or not k_pool.is_cuda:
        return None
    layers, pages, page, kv, d = k_pool.shape
    if d % 64 != 0 or page_size < 8 or page_size & (page_size - 1):
        return None
    raw = ctypes.create_string_buffer(2 * 128 + 64)
    address = (ctypes.addressof(raw) + 63) & ~63
    code = _attn_lib(d).oxr_attn_make_kv_maps(address, k_pool.data_ptr(), v_pool.data_ptr(), layers * pages * page, kv * d, page_size)
    if code != 0:
        return None
    return KVMaps(raw, address, (k_pool.data_ptr(), v_pool.data_ptr()), pages * page)


def tiled_attention_takes(head_dim: int, value_dim: int, dtype: torch.dtype) -> bool:
    """Whether the tiled tensor-core attention (``paged_attention``; one library per head size) serves these sizes: bfloat16, keys and
    values of one size that is a multiple of 16 up to 256. Other sizes, and float32, go to ``attention_rows``."""
    return dtype == torch.bfloat16 and head_dim == value_dim and head_dim % 16 == 0 and 16 <= head_dim <= 256


def paged_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, *, tiles: dict, cu_q: torch.Tensor,
                    ctx_lens: torch.Tensor, block_table: torch.Tensor, page_size: int, scale: float, window: int,
                    kv_len_bound: int, status: torch.Tensor, generic: bool = False, kv_maps: KVMaps | None = None,
                    layer_in_pool: int = 0, uneven: bool = False, chunk: int = 0, dist_bias: torch.Tensor | None = None,
                    sink: torch.Tensor | None = None, keep_first: int = 0) -> torch.Tensor:
    """Causal grouped-query attention of the step's new tokens over the paged cache
    (oxr_runtime/attention.py:47-109). ``q`` is ``[tokens, H, D]``; ``k_cache`` / ``v_cache`` are one layer's pool
    ``[pages, page_size, KV, D]``; ``window`` > 0 limits a query to its last ``window`` keys; ``tiles`` maps each
    spec of :func:`attention_tile_specs` to ``(tile_req, tile_tok0, count)``; ``kv_len_bound`` is an upper bound of
    the context lengths. float32 runs the fp32 CUDA-core kernel, bfloat16 the tensor-core kernels (``generic``
    forces the CUDA-core kernel, which then needs the float32 tile spec). With ``kv_maps`` (of the pool that
    ``k_cache`` / ``v_cache`` are layer ``layer_in_pool`` of) the split-KV kernel fetches K and V by TMA. ``uneven``: the
    caller knows that the requests' lengths differ much (see ``DECODE_CUT``).

    bfloat16 only, on the cp.async tensor-core kernels (no ``kv_maps``): ``chunk`` > 0 lets position p see only keys j with
    ``j // chunk == p // chunk``; ``dist_bias [rows, H]`` (fp32) is added to the scaled score by distance p - j (the last row for all
    larger ones); ``sink [H]`` (fp32) adds ``exp(sink)`` to the softmax denominator; with a window, ``keep_first`` > 0 keeps the request's
    first ``keep_first`` keys visible to every later query. ``v_cache`` may be ``k_cache`` itself (a latent
    cache whose rows are key and value at once)."""
    _need(q, "q")
    _need(k_cache, "k_cache", q.dtype)
    _need(v_cache, "v_cache", q.dtype)
    keep_first = int(keep_first) if window > 0 else 0
    masked = chunk > 0 or dist_bias is not None or sink is not None or keep_first > 0
    if masked and (q.dtype != torch.bfloat16 or generic or kv_maps is not None):
        raise KernelError("paged_attention: chunk, dist_bias and sink run on the bfloat16 cp.async kernels only (no kv_maps)")
    for t, nm in ((cu_q, "cu_q"), (ctx_lens, "ctx_lens"), (block_table, "block_table")):
        _need(t, nm, torch.int32)
    _, num_heads, head_dim = q.shape
    num_pages, page, num_kv_heads, d2 = k_cache.shape
    if page != page_size or d2 != head_dim or v_cache.shape != k_cache.shape:
        raise KernelError(f"cache pool {tuple(k_cache.shape)} does not fit page size {page_size} / head size {head_dim}")
    lib = _attn_lib(head_dim)
    out = torch.empty_like(q)
    common = (cu_q.data_ptr(), ctx_lens.data_ptr(), block_table.data_ptr(), block_table.shape[-1], page_size, num_pages,
              num_heads, num_kv_heads, float(scale), int(window))
    if q.dtype == torch.float32 or generic:
        (spec,) = attention_tile_specs(num_heads, num_kv_heads, head_dim, torch.float32)
        tile_req, tile_tok0, n = tiles[spec]
        code = lib.oxr_paged_attention(out.data_ptr(), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), tile_req.data_ptr(),
                                       tile_tok0.data_ptr(), n, *common, _dtype_code(q), status.data_ptr(), _stream())
        _done(code, "paged_attention")
        return out
    long_rows = _long_rows(head_dim, kv_maps is not None)
    short, long_ = attention_tile_specs(num_heads, num_kv_heads, head_dim, torch.bfloat16, page_size if kv_maps is not None else None)
    if long_ not in tiles:
        raise KernelError(f"no tile list for long tiles of {long_rows} rows: the batch was cut for {sorted(tiles)}")
    s_req, s_tok, n_short = tiles[short]
    l_req, l_tok, n_long = tiles[long_]
    splits, cut, part_o, part_ml, counters = _split_kv_plan(lib, n_short, num_heads, num_kv_heads, head_dim, kv_len_bound, kv_maps is not None,
                                                            uneven, q.device)
    if masked:
        for t, nm in ((dist_bias, "dist_bias"), (sink, "sink")):
            if t is not None:
                _need(t, nm, torch.float32)
        if dist_bias is not None and (dist_bias.dim() != 2 or dist_bias.shape[1] != num_heads):
            raise KernelError("paged_attention: the distance bias must be [rows, heads]")
        if sink is not None and sink.numel() != num_heads:
            raise KernelError("paged_attention: one sink per head")
        code = lib.oxr_paged_attention_masked_bf16(out.data_ptr(), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), s_req.data_ptr(),
                                                   s_tok.data_ptr(), n_short, l_req.data_ptr(), l_tok.data_ptr(), n_long, *common, int(chunk), keep_first,
                                                   _ptr(dist_bias), dist_bias.shape[0] if dist_bias is not None else 0, _ptr(sink), splits,
                                                   _ptr(part_o), _ptr(part_ml), _ptr(counters), status.data_ptr(), _stream())
        global launch_count
        _done(code, "paged_attention_masked_bf16")
        launch_count += 1 if n_long and n_short else 0
        return out
    code = lib.oxr_paged_attention_bf16(out.data_ptr(), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), s_req.data_ptr(),
                                        s_tok.data_ptr(), n_short, l_req.data_ptr(), l_tok.data_ptr(), n_long, *common, splits,
                                        _ptr(part_o), _ptr(part_ml), _ptr(counters),
                                        kv_maps.address if kv_maps is not None else None,
                                        layer_in_pool * kv_maps.rows_per_layer if kv_maps is not None else 0, long_rows, q.shape[0], cut,
                                        status.data_ptr(), _stream())
    _done(code, "paged_attention_bf16")
    launch_count += 1 if n_long and n_short else 0
    return out


def _wants_even_cut(n_short: int, tma: bool, uneven: bool) -> bool:
    return bool(n_short) and tma and (DECODE_CUT == "even" or (DECODE_CUT == "auto" and uneven and n_short <= EVEN_CUT_MAX_TILES))


def _split_kv_plan(lib, n_short: int, num_heads: int, num_kv_heads: int, head_dim: int, kv_len_bound: int, tma: bool, uneven: bool,
                   device: torch.device):
    """Pieces per request, the cut (0 equal pieces, 1 the even cut) and the scratch of the split-KV kernel for ``n_short`` tiles."""
    splits = attention_splits(n_short, num_heads, num_kv_heads, kv_len_bound) if n_short else 1
    part_o = part_ml = counters = None
    cut = 0
    group = num_heads // num_kv_heads
    units = n_short * num_kv_heads * -(-group // min(group, DECODE_ROWS))
    slots = units * splits if splits > 1 else 0
    if _wants_even_cut(n_short, tma, uneven):
        # all key blocks of the step dealt out evenly to one round of blocks (requests of any mix of lengths): the library
        # says how many partial results that can make, or 0 if it cannot do it for so many units
        even = lib.oxr_attn_even_cut_slots(units)
        if even > 0:
            cut, slots = 1, max(slots, even)
    if slots:
        part_o = torch.empty(slots * DECODE_ROWS * head_dim, dtype=torch.float32, device=device)
        part_ml = torch.empty(slots * DECODE_ROWS * 2, dtype=torch.float32, device=device)
        counters = _ticket_counters(device, units)
    return splits, cut, part_o, part_ml, counters


FUSE_QKV = os.environ.get("OXR_B200_FUSE_QKV", "1") != "0"
"""Whether a decode step's attention takes the raw q|k|v projections itself (``decode_attention_from_projections``) where it can."""


def attention_takes_projections(head_dim: int, dtype: torch.dtype, page_size: int, kv_maps: KVMaps | None, *, requests: int = 0,
                                num_heads: int = 0, num_kv_heads: int = 0, kv_len_bound: int = 0, uneven: bool = False) -> bool:
    """Whether ``decode_attention_from_projections`` can run: bfloat16, the cache group's tensor maps, a head size that is a
    multiple of 64 and pages of 8 * 2^k tokens (what the split-KV kernel with TMA gathers needs); and, when ``requests`` says
    how many single-token requests the step has, that their pieces get a block each (no more than one round of blocks, not
    the even cut): only that form of the kernel takes the projections. (A block that walks over many pieces would prepare q
    for each of them; at 64 requests of 2,048 keys that cost more than the kernel it saves.)"""
    if not (FUSE_QKV and dtype == torch.bfloat16 and kv_maps is not None and head_dim % 64 == 0 and page_size >= 8
            and page_size & (page_size - 1) == 0):
        return False
    if requests:
        if _wants_even_cut(requests, True, uneven):
            return False
        group = num_heads // num_kv_heads
        units = requests * num_kv_heads * -(-group // min(group, DECODE_ROWS))
        if units * attention_splits(requests, num_heads, num_kv_heads, kv_len_bound) > _attn_lib(head_dim).oxr_attn_one_round_of_pieces():
            return False
    return True


def decode_attention_from_projections(qkv: torch.Tensor, q_weight: torch.Tensor | None, k_weight: torch.Tensor | None,
                                      cos: torch.Tensor | None, sin: torch.Tensor | None, k_cache: torch.Tensor, v_cache: torch.Tensor, *,
                                      store: bool, num_heads: int, num_kv_heads: int, head_dim: int, eps: float, tiles: dict,
                                      cu_q: torch.Tensor, ctx_lens: torch.Tensor, block_table: torch.Tensor, page_size: int, scale: float,
                                      window: int, kv_len_bound: int, status: torch.Tensor, kv_maps: KVMaps, layer_in_pool: int = 0,
                                      uneven: bool = False) -> torch.Tensor:
    """``qk_norm_rope_store`` and ``paged_attention`` of a step in which EVERY request brings one token, as one kernel: row r of
    ``qkv`` ``[n, (H + 2 KV) * D]`` is request r's token, its position is ``ctx_lens[r] - 1``, its cache row the one the block
    table names for that position. ``store=False`` writes nothing and attends to what the cache holds. Returns ``[n, H, D]``.
    Call it only where ``attention_takes_projections`` (asked with the step's requests) says yes. Measured on a B200, Qwen3-8B
    sizes, 8 requests of 2,048 keys: the decode step 3.32 against 3.42 ms."""
    _need(qkv, "qkv", torch.bfloat16)
    _need(k_cache, "k_cache", qkv.dtype)
    _need(v_cache, "v_cache", qkv.dtype)
    for t, nm in ((cu_q, "cu_q"), (ctx_lens, "ctx_lens"), (block_table, "block_table")):
        _need(t, nm, torch.int32)
    n = qkv.shape[0]
    if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim:
        raise KernelError(f"qkv has {qkv.shape[1]} columns, expected (H + 2 KV) * D = {(num_heads + 2 * num_kv_heads) * head_dim}")
    num_pages, page, kvh, d2 = k_cache.shape
    if page != page_size or d2 != head_dim or kvh != num_kv_heads or v_cache.shape != k_cache.shape:
        raise KernelError(f"cache pool {tuple(k_cache.shape)} does not fit page size {page_size} / {num_kv_heads} heads of {head_dim}")
    if not attention_takes_projections(head_dim, qkv.dtype, page_size, kv_maps, requests=n, num_heads=num_heads, num_kv_heads=num_kv_heads,
                                       kv_len_bound=kv_len_bound, uneven=uneven):
        raise KernelError(f"attention cannot take the projections itself for {n} requests at head size {head_dim}, page size {page_size}")
    for w, nm in ((q_weight, "q_weight"), (k_weight, "k_weight")):
        if w is not None:
            _need(w, nm, torch.float32)
            if w.numel() != head_dim:
                raise KernelError(f"{nm} has {w.numel()} entries for head size {head_dim}")
    max_positions = 0
    if cos is not None:
        _need(cos, "cos", torch.float32)
        _need(sin, "sin", torch.float32)
        if cos.shape[1] != head_dim // 2 or sin.shape != cos.shape:
            raise KernelError("rotary tables must be [max_positions, head_dim / 2]")
        max_positions = cos.shape[0]
    lib = _attn_lib(head_dim)
    short, _ = attention_tile_specs(num_heads, num_kv_heads, head_dim, torch.bfloat16, page_size)
    s_req, s_tok, n_short = tiles[short]
    if n_short != n or cu_q.numel() < n + 1:
        raise KernelError(f"{n} rows of projections but {n_short} single-token tiles: not a step of one token per request")
    splits, cut, part_o, part_ml, counters = _split_kv_plan(lib, n_short, num_heads, num_kv_heads, head_dim, kv_len_bound, True, uneven,
                                                            qkv.device)
    out = torch.empty((n, num_heads, head_dim), dtype=qkv.dtype, device=qkv.device)
    code = lib.oxr_paged_attention_fused_decode_bf16(
        out.data_ptr(), qkv.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), s_req.data_ptr(), s_tok.data_ptr(), n_short,
        cu_q.data_ptr(), ctx_lens.data_ptr(), block_table.data_ptr(), block_table.shape[-1], page_size, num_pages, num_heads, num_kv_heads,
        float(scale), int(window), splits, _ptr(part_o), _ptr(part_ml), _ptr(counters), kv_maps.address,
        layer_in_pool * kv_maps.rows_per_layer, cut, _ptr(q_weight), _ptr(k_weight), _ptr(cos), _ptr(sin), float(eps), max_positions,
        int(store), status.data_ptr(), _stream())
    _done(code, "paged_attention_fused_decode_bf16")
    return out


_counters: dict[torch.device, torch.Tensor] = {}
_outgrown: list[torch.Tensor] = []


def _ticket_counters(device: torch.device, units: int) -> torch.Tensor:
    """Zeroed ticket counters of the split-KV kernel, one per (tile, KV head group). The kernel leaves them zero, so
    one array serves every launch on a stream. An array that is outgrown is kept, not freed: a captured CUDA graph
    may hold its address."""
    t = _counters.get(device)
    if t is None or t.numel() < units:
        if t is not None:
            _outgrown.append(t)
        t = torch.zeros(max(units, 1 << 16), dtype=torch.int32, device=device)
        _counters[device] = t
    return t


GEMM_SPLITS = (1, 2, 3, 4, 6, 8)
GEMM_WORKSPACE_BYTES = 64 << 20
_GEMM_RING_BYTES = 227 * 1024 - 1024 - 256    # shared memory the kernel's stage ring may fill
_split_buffers: dict = {}


def _gemm_cost(m: int, n: int, k: int, tile_n: int, splits: int) -> float:
    """Microseconds the tcgen05 product is expected to take with tiles of 128 x ``tile_n`` and ``splits`` shares per
    tile. The constants are fitted to this kernel on a B200 (Qwen3-8B's four products at 17 to 8192 rows):

    * a 64-wide k step of one block takes 0.085 + 0.00144 * tile_n microseconds (shared-memory fill from L2), and no
      less than 0.24 (the round trip of a stage through TMA and the tensor core, divided by the stages in flight);
    * a wave of blocks takes at least the time HBM needs for the parts of W it streams (5.9 TB/s), and the two
      limits overlap all but about 15 %;
    * a split unit writes its partial tile and the last unit of a tile adds them up: 6.4 microseconds plus 0.065 per
      row and 128 columns, which later waves hide only by half;
    * 2.2 microseconds before the first block computes.
    """
    rows = -(-m // 128)
    tiles, steps = rows * -(-n // tile_n), -(-k // 64)
    per = -(-steps // splits)
    step_us = max(0.24, 0.085 + 0.00144 * tile_n)
    units = tiles * splits
    w_bytes = tile_n * 128 * per / rows        # blocks of the same wave share the W tiles of their column
    t = 2.2
    full, rest = divmod(units, num_sms())
    for active, count in ((num_sms(), full), (rest, 1 if rest else 0)):
        fill, stream = per * step_us, active * w_bytes / 5.9e6
        t += count * (max(fill, stream) + 0.15 * min(fill, stream))
    if splits > 1:
        waves = -(-units // num_sms())
        t += (1 + 0.5 * (waves - 1)) * (6.4 + 0.065 * min(m, 128) * tile_n / 128)
    return t


@functools.lru_cache(maxsize=None)
def _gemm_plan(m: int, n: int, k: int, may_split: bool = True) -> tuple[int, int]:
    """(tile width, shares of k per tile) of the tcgen05 product: the cheapest by ``_gemm_cost`` among widths of 32 to
    256 columns in steps of 16 and 1 to 8 shares whose partial tiles fit the workspace; the first found among equals."""
    best, best_cost = (128, 1), None
    steps = -(-k // 64)
    for tile_n in range(256, 16, -16):
        tiles = -(-m // 128) * -(-n // tile_n)
        for splits in (GEMM_SPLITS if may_split else (1,)):
            if splits > steps or (splits > 1 and splits * tiles * 128 * tile_n * 4 > GEMM_WORKSPACE_BYTES):
                continue
            cost = _gemm_cost(m, n, k, tile_n, splits)
            if best_cost is None or cost < best_cost - 1e-9:
                best, best_cost = (tile_n, splits), cost
    return best


GEMM_FEW_ROWS = 256          # the widest tile of a tcgen05 product
GEMM_FEW_ROWS_ANY_SHARES = 192


@functools.lru_cache(maxsize=None)
def _few_rows_clusters(shares: int) -> int:
    """Clusters of ``shares`` blocks of the few-rows kernel that the GPU holds at a time."""
    return int(_lib().oxr_gemm_few_rows_max_clusters(shares))


def _gemm_few_rows_plan(m: int, n: int, k: int) -> int:
    """Shares of k for the few-rows kernel (W on the 128-row side of the tiles, the rows of x as the tile's width, the
    shares of a tile the blocks of one cluster), or 0 where the ordinary kernel is to run. It stages no padding rows
    and adds the shares' partial tiles through distributed shared memory, which pays when W is narrow: N / 128 tiles
    are then far fewer than SMs and k is dealt out so that about one block per SM results. The plan is the most shares
    with which the clusters of all tiles run at once, at least two and at most four (clusters of five and more were
    level or up to 1.5 us slower, except with many rows and a long k: from 193 rows and 128 k steps on at most 8, a
    portable cluster). Measured on
    a B200 with Qwen3-8B's and 32B's products: level with cuBLAS or ahead of it from 17 to 128 rows (down projection at
    64 rows: 20.0 us, cuBLAS 22.1, the ordinary kernel with shares through a workspace 23.1); from 193 rows on only
    three shares or more still beat the ordinary kernel (each block fetches all rows of x for its k steps)."""
    if m > GEMM_FEW_ROWS:
        return 0
    tiles, steps = -(-n // 128), -(-k // 64)
    most = 8 if (m > GEMM_FEW_ROWS_ANY_SHARES and steps >= 128) else 4
    for shares in range(min(most, num_sms() // tiles, steps), 1, -1):
        if tiles <= _few_rows_clusters(shares):
            return shares if (m <= GEMM_FEW_ROWS_ANY_SHARES or shares >= 3) else 0
    return 0


GEMM_PAIR_MIN_ROWS = 512
STEP_TILE_ROWS = 256
"""Rows of the widest GEMM tile (the two-SM kernel's): a step of a few tokens more than a multiple of it pays for a whole
tile row. Whoever plans steps may ask for it."""


@functools.lru_cache(maxsize=None)
def _gemm_pair_plan(m: int, n: int, k: int) -> int:
    """Tile width for the two-SM product kernel (256 x width tiles, a pair of blocks each), or 0 where the one-SM
    kernel is to run. In isolated short runs the two kernels are level below about 3,000 rows; in long runs, where
    the power cap sets the clock, the pair kernel (a third less shared-memory traffic per flop) is 5 to 8 % faster
    from 512 rows on (sum of Qwen3-8B's four products, 150 calls each: 173 against 190 us at 512 rows, 604 against
    649 us at 2,048), and a 2,048-token prefill step takes 28.1 instead of 30.5 ms. The width is the one with the
    least waves of pairs times the time of a k step at that width (0.094 + 0.00128 width microseconds)."""
    if m < GEMM_PAIR_MIN_ROWS:
        return 0
    pairs = num_sms() // 2
    best, best_cost = 0, None
    for tile_n in (256, 224, 192, 160, 128, 96, 64):
        tiles = -(-m // 256) * -(-n // tile_n)
        cost = -(-tiles // pairs) * (0.094 + 0.00128 * tile_n)
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = tile_n, cost
    return best


GEMM_MAX_SPLIT_TILES = GEMM_WORKSPACE_BYTES // (2 * 128 * 16 * 4)   # the most tiles a split product can have


def _gemm_split_buffers(device: torch.device) -> tuple[torch.Tensor, torch.Tensor]:
    """Workspace of the split product (one fp32 partial tile per unit) and its zeroed tickets (one per tile), made once
    per device at their full size and never replaced: a captured CUDA graph keeps their addresses. Products on one
    stream follow one another, and the kernel leaves the tickets zeroed."""
    got = _split_buffers.get(device)
    if got is None:
        got = (torch.empty(GEMM_WORKSPACE_BYTES // 4, dtype=torch.float32, device=device),
               torch.zeros(GEMM_MAX_SPLIT_TILES, dtype=torch.int32, device=device))
        _split_buffers[device] = got
    return got


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """``x @ weight.T`` for ``weight [out, in]``, no bias (oxr_runtime/language.py:223-231), fp32 accumulation.

    float32 x float32 runs the fp32 CUDA-core kernel (no TF32). bfloat16 x bfloat16 runs the skinny kernel up to
    ``SKINNY_MAX_ROWS`` rows and the TMA + tcgen05 kernel beyond (cuBLAS only when a row is not a whole number of
    16-byte words). A weight kept in float32 under bfloat16 activations is multiplied in fp32 and the result
    rounded once. ``out`` (contiguous ``[rows, out]`` of the output dtype) receives the product instead of a new tensor.
    """
    if isinstance(x, NormedLazily):
        out = _scaled_linear(x, weight, gated=False) if out_dtype in (None, torch.bfloat16) else None
        if out is not None:
            return out
        x = x.materialize()
    _need(x, "x")
    _need(weight, "weight")
    m, k = x.shape
    n, k2 = weight.shape
    if k != k2:
        raise KernelError(f"linear: x has {k} columns, weight has {k2}")
    out_dtype = out_dtype or x.dtype
    if out is not None:
        _need(out, "out", out_dtype)
        if out.shape != (m, n):
            raise KernelError(f"linear: out is {tuple(out.shape)} for a product of {(m, n)}")
    given = out
    lib = _lib()
    if weight.dtype == torch.float32:
        x32 = cast(x, torch.float32)
        out = given if given is not None and out_dtype == torch.float32 else torch.empty((m, n), dtype=torch.float32, device=x.device)
        _done(lib.oxr_gemm_f32_nt(out.data_ptr(), x32.data_ptr(), weight.data_ptr(), m, n, k, _stream()), "gemm_f32")
        if given is not None and out_dtype != torch.float32:
            given.copy_(out)
            return given
        return cast(out, out_dtype)
    if x.dtype != torch.bfloat16:
        raise KernelError(f"linear: activations {x.dtype} with weight {weight.dtype} is not a supported pair")
    if STREAM_GEMM and m <= STREAM_MAX_ROWS and k % 8 == 0 and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0:
        out = given if given is not None else torch.empty((m, n), dtype=out_dtype, device=x.device)
        _done(lib.oxr_gemm_stream_bf16(out.data_ptr(), x.data_ptr(), weight.data_ptr(), m, n, k, _DT[out_dtype],
                                       new_status(x.device).data_ptr(), _stream()), "gemm_stream")
        return out
    if m <= SKINNY_MAX_ROWS and k % 8 == 0 and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0:
        out = given if given is not None else torch.empty((m, n), dtype=out_dtype, device=x.device)
        _done(lib.oxr_gemm_skinny_bf16(out.data_ptr(), x.data_ptr(), weight.data_ptr(), m, n, k, _DT[out_dtype], _stream()),
              "gemm_skinny")
        return out
    if k % 8 == 0 and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0:
        out = given if given is not None else torch.empty((m, n), dtype=out_dtype, device=x.device)
        few = _gemm_few_rows_plan(m, n, k)
        if few:
            _done(lib.oxr_gemm_few_rows_cluster_bf16(out.data_ptr(), x.data_ptr(), weight.data_ptr(), m, n, k, _DT[out_dtype], few,
                                                     new_status(x.device).data_ptr(), _stream()), "gemm_few_rows_cluster")
            return out
        pair_tile = _gemm_pair_plan(m, n, k)
        if pair_tile:
            _done(lib.oxr_gemm_tcgen05_pair_bf16(out.data_ptr(), x.data_ptr(), weight.data_ptr(), m, n, k, _DT[out_dtype], pair_tile,
                                                 new_status(x.device).data_ptr(), _stream()), "gemm_tcgen05_pair")
            return out
        tile_n, splits = _gemm_plan(m, n, k)
        partial = tickets = None
        if splits > 1:
            if splits * -(-m // 128) * -(-n // tile_n) * 128 * tile_n * 4 > GEMM_WORKSPACE_BYTES:
                raise KernelError(f"linear: {splits} shares of {m} x {n} in tiles of {tile_n} columns outgrow the workspace")
            partial, tickets = _gemm_split_buffers(x.device)
        code = lib.oxr_gemm_tcgen05_bf16(out.data_ptr(), x.data_ptr(), weight.data_ptr(), m, n, k, _DT[out_dtype], tile_n, splits,
                                         _ptr(partial), _ptr(tickets), new_status(x.device).data_ptr(), _stream())
        _done(code, "gemm_tcgen05")
        return out
    # rows that are not whole 16-byte words cannot be fetched by TMA: the library product takes them
    got = torch.mm(x, weight.t(), out_dtype=torch.float32) if out_dtype == torch.float32 else torch.mm(x, weight.t())
    if given is not None:
        given.copy_(got)
        return given
    return got


FUSE_MAX_ROWS = min(16, int(os.environ.get("OXR_B200_FUSE_ROWS", "16")))
"""Decode steps of up to this many rows fold their norms into the products around them (0: never)."""
"""Most rows for which a decode step's RMSNorms are folded into the products around them."""


class NormedLazily:
    """``RMSNorm(residual) * weight`` with the row's scale still to be applied: ``y = bf16(residual * weight)`` and, per block
    of the product that wrote it, the sums of squares of the block's columns of the residual (``ops.linear_add``).
    ``ops.linear`` and ``ops.gated_silu_linear`` take it in place of x and scale their sums by rsqrt(mean + eps) row by row;
    ``materialize()`` runs the norm kernel on the residual for anyone else."""

    def __init__(self, y: torch.Tensor, residual: torch.Tensor, sums: torch.Tensor, blocks: int, weight: torch.Tensor, eps: float):
        self.y, self.residual, self.sums, self.blocks, self.weight, self.eps = y, residual, sums, blocks, weight, float(eps)

    @property
    def shape(self) -> torch.Size:
        return self.y.shape

    def materialize(self) -> torch.Tensor:
        return add_rms_norm(torch.zeros_like(self.y), self.residual, self.weight, self.eps, keep_residual=False)[0]


def linear_add(x: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor | None, norm_weight: torch.Tensor, eps: float
               ) -> tuple[NormedLazily, torch.Tensor] | None:
    """``add_rms_norm(linear(x, weight), residual, norm_weight, eps)`` for a decode step without the norm kernel: ONE kernel
    multiplies, rounds the product to bf16 as ``linear`` would, adds it into the fp32 residual stream (in place when one is
    given), and leaves the new residual times the norm's weight in bf16 and the rows' sums of squares, block by block; the
    row's scale rsqrt(mean + eps) is applied by the product that takes the result (:class:`NormedLazily`) to its fp32 sums.
    None when the sizes do not allow it (more than ``FUSE_MAX_ROWS`` rows, not bf16, ...): the caller then runs the two
    kernels."""
    m, k = x.shape
    n = weight.shape[0]
    if not (STREAM_GEMM and 0 < m <= FUSE_MAX_ROWS and x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
            and k % 8 == 0 and n % 8 == 0 and weight.shape[1] == k and x.is_contiguous() and x.data_ptr() % 16 == 0
            and weight.data_ptr() % 16 == 0 and norm_weight.numel() == n and norm_weight.dtype == torch.float32):
        return None
    if residual is not None:
        _need(residual, "residual", torch.float32)
        if residual.shape != (m, n):
            raise KernelError(f"residual {tuple(residual.shape)} does not match the product's {(m, n)}")
    lib = _lib()
    blocks = lib.oxr_gemm_stream_blocks(n)
    res_out = residual if residual is not None else torch.empty((m, n), dtype=torch.float32, device=x.device)
    y = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
    sums = torch.empty((blocks, 16), dtype=torch.float32, device=x.device)
    code = lib.oxr_gemm_stream_add_bf16(res_out.data_ptr(), _ptr(residual), y.data_ptr(), sums.data_ptr(), norm_weight.data_ptr(),
                                        x.data_ptr(), weight.data_ptr(), m, n, k, new_status(x.device).data_ptr(), _stream())
    _done(code, "gemm_stream_add")
    return NormedLazily(y, res_out, sums, blocks, norm_weight, eps), res_out


def _scaled_linear(x: NormedLazily, weight: torch.Tensor, gated: bool) -> torch.Tensor | None:
    """``linear`` (or, ``gated``, silu(gate) * up on a weight with alternating rows) of a lazily normalised x in ONE kernel
    that scales its sums row by row; None when the sizes do not allow it."""
    m, k = x.y.shape
    n = weight.shape[0]
    if not (STREAM_GEMM and m <= STREAM_MAX_ROWS and weight.dtype == torch.bfloat16 and weight.shape[1] == k and k % 8 == 0
            and weight.data_ptr() % 16 == 0 and x.blocks <= num_sms() and (not gated or n % 16 == 0)):
        return None
    out = torch.empty((m, n // 2 if gated else n), dtype=torch.bfloat16, device=weight.device)
    code = _lib().oxr_gemm_stream_scaled_bf16(out.data_ptr(), x.y.data_ptr(), x.sums.data_ptr(), x.blocks, x.eps, weight.data_ptr(), m, n, k,
                                              int(gated), new_status(weight.device).data_ptr(), _stream())
    _done(code, "gemm_stream_scaled")
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor | None = None, seed_lo: torch.Tensor | None = None,
           seed_hi: torch.Tensor | None = None, counter: torch.Tensor | None = None) -> torch.Tensor:
    """One token per row of fp32 ``logits``: the first maximum where ``temperature`` <= 0 (or None), else a draw
    from softmax(logits / temperature) decided by (seed, counter) alone."""
    _need(logits, "logits", torch.float32)
    rows, vocab = logits.shape
    if temperature is not None:
        _need(temperature, "temperature", torch.float32)
        for t, nm in ((seed_lo, "seed_lo"), (seed_hi, "seed_hi"), (counter, "counter")):
            if t is None:
                raise KernelError(f"sample: {nm} is required with a temperature")
            _need(t, nm, torch.int32)
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    lib = _lib()
    # per row and vocabulary chunk: maximum, its index, sum of exponentials
    scratch = torch.empty(3 * rows * lib.oxr_sample_chunks(vocab), dtype=torch.int32, device=logits.device)
    code = lib.oxr_sample(out.data_ptr(), logits.data_ptr(), rows, vocab, _ptr(temperature), _ptr(seed_lo),
                          _ptr(seed_hi), _ptr(counter), scratch.data_ptr(), _stream())
    _done(code, "sample")
    global launch_count
    launch_count += 1  # two kernels
    return out


def repetition_penalty(logits: torch.Tensor, seen: torch.Tensor, row_slot: torch.Tensor, penalty: torch.Tensor) -> None:
    """In place: for tokens marked in ``seen[row_slot[r]]`` a positive logit is divided by ``penalty[r]``, any other
    multiplied (oxr_runtime/engine.py:632-639)."""
    _need(logits, "logits", torch.float32)
    _need(seen, "seen", torch.uint8)
    _need(row_slot, "row_slot", torch.int32)
    _need(penalty, "penalty", torch.float32)
    rows, vocab = logits.shape
    code = _lib().oxr_repetition_penalty(logits.data_ptr(), seen.data_ptr(), row_slot.data_ptr(), penalty.data_ptr(), rows,
                                         vocab, _stream())
    _done(code, "repetition_penalty")


def mark_seen(seen: torch.Tensor, slots: torch.Tensor, tokens: torch.Tensor) -> None:
    """``seen[slots[i], tokens[i]] = 1``."""
    _need(seen, "seen", torch.uint8)
    _need(slots, "slots", torch.int32)
    _need(tokens, "tokens", torch.int32)
    code = _lib().oxr_mark_seen(seen.data_ptr(), slots.data_ptr(), tokens.data_ptr(), tokens.numel(), seen.shape[1], _stream())
    _done(code, "mark_seen")


# --------------------------------------------------------------------------------------------------- a whole fp32 stream
def stream_rms_norm(stream: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype, rows: torch.Tensor | None = None) -> torch.Tensor:
    """``stream * rsqrt(mean(stream^2) + eps) * weight`` of an fp32 stream ``[tokens, hidden]``, rounded to ``out_dtype``; with
    ``rows`` (int32) only those rows, output row i from stream row ``rows[i]``."""
    _need(stream, "stream", torch.float32)
    _need(weight, "weight", torch.float32)
    n, hidden = stream.shape
    if rows is not None:
        _need(rows, "rows", torch.int32)
        n = rows.numel()
    out = torch.empty((n, hidden), dtype=out_dtype, device=stream.device)
    _done(_lib().oxr_stream_rms_norm(out.data_ptr(), stream.data_ptr(), weight.data_ptr(), _ptr(rows), n, hidden, float(eps), _DT[out_dtype], _stream()),
          "stream_rms_norm")
    return out


def norm_add_norm(stream: torch.Tensor, y: torch.Tensor, post_weight: torch.Tensor, post_eps: float, next_weight: torch.Tensor | None = None,
                  next_eps: float = 0.0, rounded: bool = False) -> torch.Tensor | None:
    """In place ``stream += rmsnorm(y) * post_weight`` (fp32); with ``next_weight`` also returns ``rmsnorm(stream) * next_weight`` in
    ``y.dtype``: a sublayer's post-norm, the residual add and the next sublayer's pre-norm in one pass over the row. ``rounded`` (without a
    next weight): also returns the new stream rounded to ``y.dtype``, for a sublayer that reads the stream itself."""
    _need(stream, "stream", torch.float32)
    _need(y, "y")
    _need(post_weight, "post_weight", torch.float32)
    if y.shape != stream.shape:
        raise KernelError(f"norm_add_norm: y {tuple(y.shape)} does not match the stream {tuple(stream.shape)}")
    n, hidden = stream.shape
    out = None
    if next_weight is not None:
        _need(next_weight, "next_weight", torch.float32)
    if next_weight is not None or rounded:
        out = torch.empty((n, hidden), dtype=y.dtype, device=y.device)
    _done(_lib().oxr_norm_add_norm(stream.data_ptr(), y.data_ptr(), post_weight.data_ptr(), _ptr(out), _ptr(next_weight), n, hidden, float(post_eps),
                                   float(next_eps), _dtype_code(y), _stream()), "norm_add_norm")
    return out


def concat2_cast(a: torch.Tensor, b: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """``[a | b]`` along the last axis for two fp32 ``[tokens, hidden]`` tensors, rounded to ``out_dtype``."""
    _need(a, "a", torch.float32)
    _need(b, "b", torch.float32)
    if a.shape != b.shape:
        raise KernelError("concat2_cast: shapes differ")
    n, hidden = a.shape
    out = torch.empty((n, 2 * hidden), dtype=out_dtype, device=a.device)
    _done(_lib().oxr_concat2_cast(out.data_ptr(), a.data_ptr(), b.data_ptr(), n, hidden, _DT[out_dtype], _stream()), "concat2_cast")
    return out


def add_row_(x: torch.Tensor, row: torch.Tensor) -> torch.Tensor:
    """In place ``x[t] += row`` for fp32 ``x [tokens, hidden]``."""
    _need(x, "x", torch.float32)
    _need(row, "row", torch.float32)
    if row.numel() != x.shape[1]:
        raise KernelError("add_row_: the row does not fit")
    _done(_lib().oxr_add_row_f32(x.data_ptr(), row.data_ptr(), x.shape[0], x.shape[1], _stream()), "add_row")
    return x


def clamped_glu(gate_up: torch.Tensor, *, alpha: float, limit: float, interleave: int = 0) -> torch.Tensor:
    """``g * sigmoid(alpha g) * (u + 1)`` with ``g = min(gate, limit)``, ``u = clamp(up, -limit, limit)`` for ``gate_up = [gate | up]``
    along the last axis (or alternating in groups of ``interleave`` columns)."""
    _need(gate_up, "gate_up")
    n, two_i = gate_up.shape
    if two_i % 2:
        raise KernelError("gate_up must have an even number of columns")
    out = torch.empty((n, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    _done(_lib().oxr_clamped_glu(out.data_ptr(), gate_up.data_ptr(), n, two_i // 2, int(interleave), float(alpha), float(limit), _dtype_code(gate_up),
                                 _stream()), "clamped_glu")
    return out


def rotary_angles(positions: torch.Tensor, freq: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """fp32 ``cos`` and ``sin`` ``[tokens, len(freq)]`` of ``position * freq[i]`` for this step's tokens; the product and the functions are
    evaluated in fp64 (``freq`` is a float64 device tensor) and rounded once, so the table is exact to fp32 at any position."""
    _need(positions, "positions", torch.int32)
    _need(freq, "freq", torch.float64)
    n, half = positions.numel(), freq.numel()
    cos = torch.empty((n, half), dtype=torch.float32, device=positions.device)
    sin = torch.empty_like(cos)
    _done(_lib().oxr_rotary_angles(cos.data_ptr(), sin.data_ptr(), positions.data_ptr(), freq.data_ptr(), n, half, _stream()), "rotary_angles")
    return cos, sin


def stream_layer_norm(stream: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, eps: float, out_dtype: torch.dtype,
                      rows: torch.Tensor | None = None) -> torch.Tensor:
    """``(x - mean) / sqrt(mean((x - mean)^2) + eps) * weight + bias`` of an fp32 stream ``[tokens, hidden]``, rounded to ``out_dtype``; with
    ``rows`` (int32) only those rows."""
    _need(stream, "stream", torch.float32)
    _need(weight, "weight", torch.float32)
    if bias is not None:
        _need(bias, "bias", torch.float32)
    n, hidden = stream.shape
    if rows is not None:
        _need(rows, "rows", torch.int32)
        n = rows.numel()
    out = torch.empty((n, hidden), dtype=out_dtype, device=stream.device)
    _done(_lib().oxr_stream_layer_norm(out.data_ptr(), stream.data_ptr(), weight.data_ptr(), _ptr(bias), _ptr(rows), n, hidden, float(eps),
                                       _DT[out_dtype], _stream()), "stream_layer_norm")
    return out


def gated_residual(stream: torch.Tensor, a: torch.Tensor, f: torch.Tensor | None = None, *, gates: torch.Tensor | None = None,
                   gate_bias: torch.Tensor | None = None, a_bias: torch.Tensor | None = None, f_bias: torch.Tensor | None = None,
                   history: torch.Tensor | None = None, index: int = 0, weights: torch.Tensor | None = None,
                   norm: tuple[torch.Tensor, torch.Tensor | None, float] | None = None, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """In place on the fp32 stream: ``X = stream + (a' + f')`` where ``a' = (a + a_bias) * sigmoid(gates[:, :hidden] + gate_bias[:hidden])`` and
    ``f'`` likewise with the second half of ``gates`` (no gates: the sublayers' outputs as they are; ``f`` None: one sublayer). With a
    ``history [slots, tokens, hidden]`` (fp32) X is kept as ``history[index]`` and the stream becomes ``sum_{j <= index} weights[j] history[j]``. With ``norm = (weight, bias or None, eps)`` the same
    kernel goes on to the layer norm that reads the new stream next and returns its output in ``out_dtype``; else returns the stream."""
    _need(stream, "stream", torch.float32)
    _need(a, "a")
    n, hidden = stream.shape
    if a.shape != stream.shape or (f is not None and (f.shape != stream.shape or f.dtype != a.dtype)):
        raise KernelError("gated_residual: the sublayers' outputs do not match the stream")
    stride = 0
    if gates is not None:
        _need(gates, "gates", a.dtype)
        stride = gates.shape[1]
        if gates.shape[0] != n or stride < (2 if f is not None else 1) * hidden:
            raise KernelError("gated_residual: the gates do not fit")
    for t, name in ((gate_bias, "gate_bias"), (a_bias, "a_bias"), (f_bias, "f_bias")):
        if t is not None:
            _need(t, name, torch.float32)
    if history is not None:
        _need(history, "history", torch.float32)
        _need(weights, "weights", torch.float32)
        if history.shape[1:] != stream.shape or not 0 <= index < history.shape[0] or weights.numel() <= index:
            raise KernelError("gated_residual: the history does not fit")
    if norm is not None:
        weight, bias, eps = norm
        _need(weight, "norm weight", torch.float32)
        if bias is not None:
            _need(bias, "norm bias", torch.float32)
        if out_dtype != a.dtype:
            raise KernelError("gated_residual: the norm's output has the sublayers' dtype")
        out = torch.empty((n, hidden), dtype=out_dtype, device=stream.device)
        _done(_lib().oxr_gated_residual_norm(out.data_ptr(), stream.data_ptr(), a.data_ptr(), _ptr(a_bias), _ptr(f), _ptr(f_bias), _ptr(gates), stride,
                                             _ptr(gate_bias), _ptr(history), int(index), _ptr(weights), n, hidden, weight.data_ptr(), _ptr(bias),
                                             float(eps), _dtype_code(a), _stream()), "gated_residual_norm")
        return out
    _done(_lib().oxr_gated_residual(stream.data_ptr(), a.data_ptr(), _ptr(a_bias), _ptr(f), _ptr(f_bias), _ptr(gates), stride, _ptr(gate_bias),
                                    _ptr(history), int(index), _ptr(weights), n, hidden, _dtype_code(a), _stream()), "gated_residual")
    return stream


def gelu_tanh_(x: torch.Tensor) -> torch.Tensor:
    """In place ``0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3)))``, fp32 arithmetic."""
    _need(x, "x")
    _done(_lib().oxr_gelu_tanh(x.data_ptr(), x.data_ptr(), x.numel(), _dtype_code(x), _stream()), "gelu_tanh")
    return x


def add_(y: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """In place ``y += x`` (tensors of one shape and type; the sum in fp32, rounded once)."""
    _need(y, "y")
    _need(x, "x", y.dtype)
    if x.shape != y.shape:
        raise KernelError("add_: shapes differ")
    _done(_lib().oxr_add_inplace(y.data_ptr(), x.data_ptr(), y.numel(), _dtype_code(y), _stream()), "add_")
    return y


def bias_rope_store(proj: torch.Tensor, cq: int, ck: int, cv: int, key_dim: int, *, bias: torch.Tensor | None, cos: torch.Tensor | None,
                    sin: torch.Tensor | None, k_pool: torch.Tensor, v_pool: torch.Tensor, slots: torch.Tensor, status: torch.Tensor) -> None:
    """Between a stacked ``[q | k | v | ...]`` product and attention: every entry of q, k and v gets its ``bias`` (fp32 ``[cq + ck + cv]``), entry
    pairs (2i, 2i+1) of the first ``2 * cos.shape[1]`` entries of every q and k head turn by the token's angles (``cos`` / ``sin``
    ``[tokens, pairs]``), q goes back in place, k and v go to their pools at ``slots`` (slot -1: not stored)."""
    _need(proj, "proj")
    _need(k_pool, "k_pool", proj.dtype)
    _need(v_pool, "v_pool", proj.dtype)
    n = proj.shape[0]
    half = 0
    if cos is not None:
        _need(cos, "cos", torch.float32)
        _need(sin, "sin", torch.float32)
        half = cos.shape[1]
    if bias is not None:
        _need(bias, "bias", torch.float32)
        if bias.numel() != cq + ck + cv:
            raise KernelError("bias_rope_store: the bias does not fit")
    if k_pool[0, 0].numel() != ck or v_pool[0, 0].numel() != cv or k_pool.shape[:2] != v_pool.shape[:2]:
        raise KernelError("bias_rope_store: the pools do not fit the projections")
    _done(_lib().oxr_bias_rope_store(proj.data_ptr(), proj.shape[1], int(cq), int(ck), int(cv), int(key_dim), _ptr(bias), _ptr(cos), _ptr(sin), half,
                                     k_pool.data_ptr(), v_pool.data_ptr(), k_pool.shape[0] * k_pool.shape[1], slots.data_ptr(), n, _dtype_code(proj),
                                     status.data_ptr(), _stream()), "bias_rope_store")


def attention_mix_rows(q: torch.Tensor, num_heads: int, k_pool: torch.Tensor, v_pool: torch.Tensor, *, positions: torch.Tensor,
                       req_of_token: torch.Tensor, block_table: torch.Tensor, scale: float, softcap: float = 0.0,
                       head_mix: torch.Tensor | None = None, unit_sink: bool = False, window: int = 0, gate: torch.Tensor | None = None,
                       status: torch.Tensor) -> torch.Tensor:
    """Attention of the step's tokens over the paged cache in which the heads' scores are mixed before the softmax, in fp32 arithmetic.

    ``q [tokens, >= H * DK]`` (the queries are the first columns, so a stacked product can be handed over); ``k_pool [pages, page_size, KV, DK]``,
    ``v_pool [pages, page_size, KV, DV]``. Token t at position p sees keys j <= p (the last ``window`` only, when given). The scaled score is
    capped as ``softcap * tanh(s / softcap)`` (0: no cap), then ``head_mix [H, H]`` (fp32) makes head h's score ``sum_g head_mix[h, g] s_g``;
    ``unit_sink`` adds one to the softmax denominator; ``gate`` (a view ``[tokens, H * DV]`` whose rows may be strided) multiplies the output by
    its sigmoid. Returns ``[tokens, H * DV]``."""
    _need(q, "q")
    _need(k_pool, "k_pool", q.dtype)
    _need(v_pool, "v_pool", q.dtype)
    n, H = q.shape[0], int(num_heads)
    pages, page_size, KV, DK = k_pool.shape
    DV = v_pool.shape[3]
    if q.dim() != 2 or q.shape[1] < H * DK or v_pool.shape[:3] != k_pool.shape[:3]:
        raise KernelError("attention_mix_rows: sizes do not fit")
    if head_mix is not None:
        _need(head_mix, "head_mix", torch.float32)
        if head_mix.shape != (H, H):
            raise KernelError("attention_mix_rows: the mixing matrix must be [heads, heads]")
    gate_stride = 0
    if gate is not None:
        if gate.dtype != q.dtype or gate.shape != (n, H * DV) or gate.stride(1) != 1 or not gate.is_cuda:
            raise KernelError("attention_mix_rows: the gate does not fit")
        gate_stride = gate.stride(0)
    out = torch.empty((n, H * DV), dtype=q.dtype, device=q.device)
    _done(_lib().oxr_attention_mix_rows(out.data_ptr(), q.data_ptr(), q.shape[1], k_pool.data_ptr(), KV * DK, DK, v_pool.data_ptr(), KV * DV, DV, DK, DV, H,
                                        KV, n, positions.data_ptr(), req_of_token.data_ptr(), block_table.data_ptr(), block_table.shape[1], page_size,
                                        pages, float(scale), float(softcap), _ptr(head_mix), int(bool(unit_sink)), int(window),
                                        gate.data_ptr() if gate is not None else None, gate_stride, _dtype_code(q), status.data_ptr(), _stream()),
          "attention_mix_rows")
    return out


MIX_TILE_SMEM_LIMIT = 227 * 1024
MIX_TILE_KEYS = 16
"""Keys per block of the tiled head-mixing kernel."""


def attention_mix_tile(num_heads: int, num_kv_heads: int, key_dim: int, value_dim: int, dtype: torch.dtype) -> tuple[int, int] | None:
    """``(query tokens per tile, query parts per block)`` with which the tensor-core kernel of head-mixing attention takes these sizes, or None
    when it does not (then ``attention_mix_rows`` is the kernel): bfloat16, keys and values of 64 or 128, 1, 2, 4, 8 or 16 query heads per
    key/value head (a 16-row MMA tile then holds 16 / that many queries of one key/value head), at most 16 key/value heads (one warp each per
    query part). The block takes as many query parts as 16 warps and its shared memory allow."""
    H, KV, DK, DV = int(num_heads), int(num_kv_heads), int(key_dim), int(value_dim)
    if dtype != torch.bfloat16 or KV <= 0 or H % KV or DK not in (64, 128) or DV not in (64, 128) or KV > 16:
        return None
    per = H // KV
    if per > 16 or 16 % per:
        return None
    rows_per_part, padded_heads = 16 // per, (H + 3) & ~3
    for parts in range(16 // KV, 0, -1):
        # queries, one K and one V block of all key/value heads (rows padded by 8), the heads' scores, the mixing matrix, two slot lists
        need = (KV * parts * 16 * (DK + 8) * 2 + KV * MIX_TILE_KEYS * (DK + 8 + DV + 8) * 2 + padded_heads * parts * rows_per_part * MIX_TILE_KEYS * 4
                + H * padded_heads * 4 + 2 * MIX_TILE_KEYS * 8)
        if need <= MIX_TILE_SMEM_LIMIT:
            return parts * rows_per_part, parts
    return None


def attention_mix_splits(n_tiles: int, kv_len_bound: int, blocks_per_sm: int = 1) -> int:
    """Pieces into which the tiled head-mixing kernel cuts every tile's keys: enough blocks for all SMs, at least four key blocks each."""
    if n_tiles <= 0:
        return 1
    most = max(1, -(-int(kv_len_bound) // MIX_TILE_KEYS) // 4)
    return max(1, min(most, blocks_per_sm * num_sms() // n_tiles, 64))


def attention_mix_tiled(q: torch.Tensor, num_heads: int, k_pool: torch.Tensor, v_pool: torch.Tensor, *, tile: tuple[int, int],
                        tiles: tuple[torch.Tensor, torch.Tensor, int], cu_q: torch.Tensor, positions: torch.Tensor, block_table: torch.Tensor,
                        kv_len_bound: int, scale: float, softcap: float = 0.0, head_mix: torch.Tensor | None = None, unit_sink: bool = False,
                        window: int = 0, gate: torch.Tensor | None = None, status: torch.Tensor, splits: int | None = None,
                        single_tokens: bool = False) -> torch.Tensor:
    """The function of :func:`attention_mix_rows` in bfloat16 on the tensor cores. ``tile`` is what :func:`attention_mix_tile` gave for
    the sizes; ``tiles = (tile_req, tile_tok0, count)`` cuts every request's new tokens into runs of ``tile[0]`` tokens (the batch builder's
    list for the spec ``(tile[0], 1, any)``); ``kv_len_bound`` bounds every request's context and, with the number of tiles, decides into
    how many pieces the keys are cut (``splits`` overrides it). ``single_tokens``: every request brings one token (a decode step); the blocks are
    then half as large and two share an SM. Scores, the mixing, the softmax weights and all sums are fp32; the weights
    are rounded to bfloat16 for the product with the values."""
    global launch_count
    _need(q, "q", torch.bfloat16)
    _need(k_pool, "k_pool", torch.bfloat16)
    _need(v_pool, "v_pool", torch.bfloat16)
    n, H = q.shape[0], int(num_heads)
    pages, page_size, KV, DK = k_pool.shape
    DV = v_pool.shape[3]
    if q.dim() != 2 or q.shape[1] < H * DK or v_pool.shape[:3] != k_pool.shape[:3] or q.shape[1] % 8 or q.data_ptr() % 16:
        raise KernelError("attention_mix_tiled: sizes do not fit")
    if head_mix is not None:
        _need(head_mix, "head_mix", torch.float32)
        if head_mix.shape != (H, H):
            raise KernelError("attention_mix_tiled: the mixing matrix must be [heads, heads]")
    gate_stride = 0
    if gate is not None:
        if gate.dtype != q.dtype or gate.shape != (n, H * DV) or gate.stride(1) != 1 or not gate.is_cuda or gate.data_ptr() % 4:
            raise KernelError("attention_mix_tiled: the gate does not fit")
        gate_stride = gate.stride(0)
    tile_req, tile_tok0, n_tiles = tiles
    if single_tokens and n != n_tiles:
        raise KernelError("attention_mix_tiled: single tokens mean one tile per token")
    if splits is None:
        splits = attention_mix_splits(n_tiles, kv_len_bound, 2 if single_tokens else 1)
    out = torch.empty((n, H * DV), dtype=q.dtype, device=q.device)
    part_o = part_ml = None
    if splits > 1:
        part_o = torch.empty((n, splits, H * DV), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n, splits, H, 2), dtype=torch.float32, device=q.device)
    _done(_lib().oxr_attention_mix_mma(out.data_ptr(), q.data_ptr(), q.shape[1], k_pool.data_ptr(), v_pool.data_ptr(), DK, DV, H, KV,
                                       1 if single_tokens else int(tile[1]), int(bool(single_tokens)),
                                       tile_req.data_ptr(), tile_tok0.data_ptr(), int(n_tiles), cu_q.data_ptr(), positions.data_ptr(), n,
                                       block_table.data_ptr(), block_table.shape[1], page_size, pages, float(scale), float(softcap), _ptr(head_mix),
                                       int(bool(unit_sink)), int(window), gate.data_ptr() if gate is not None else None, gate_stride, int(splits),
                                       _ptr(part_o), _ptr(part_ml), status.data_ptr(), _stream()), "attention_mix_tiled")
    launch_count += 1 if splits > 1 else 0   # the pieces' combine
    return out


# --------------------------------------------------------------------------------------------------- Mamba-2
def mamba_conv(proj: torch.Tensor, col0: int, channels: int, weight: torch.Tensor, bias: torch.Tensor, tail: torch.Tensor, *, req_of_token: torch.Tensor,
               cu_q: torch.Tensor, state_slots: torch.Tensor, n_requests: int) -> torch.Tensor:
    """Causal per-channel convolution with SiLU over columns ``[col0, col0 + channels)`` of ``proj`` for a packed step; ``tail``
    ``[slots, ...]`` (fp32, a view whose first axis is the slot) holds each request's last ``taps - 1`` inputs and is rolled forward."""
    _need(proj, "proj")
    _need(weight, "conv weight", torch.float32)
    _need(bias, "conv bias", torch.float32)
    if tail.dtype != torch.float32 or tail.stride(-1) != 1:
        raise KernelError("mamba_conv: the tail must be fp32 with a dense last axis")
    n = proj.shape[0]
    taps = weight.shape[1]
    out = torch.empty((n, channels), dtype=proj.dtype, device=proj.device)
    _done(_lib().oxr_mamba_conv(out.data_ptr(), proj.data_ptr(), n, n_requests, proj.shape[1], col0, channels, taps, weight.data_ptr(), bias.data_ptr(),
                                tail.data_ptr(), tail.stride(0), req_of_token.data_ptr(), cu_q.data_ptr(), state_slots.data_ptr(), _dtype_code(proj),
                                _stream()), "mamba_conv")
    return out


def mamba_scan(xbc: torch.Tensor, proj: torch.Tensor, dt_col0: int, *, heads: int, vdim: int, state: int, groups: int, dt_bias: torch.Tensor,
               a_log: torch.Tensor, d_skip: torch.Tensor, ssm: torch.Tensor, cu_q: torch.Tensor, state_slots: torch.Tensor, n_requests: int) -> torch.Tensor:
    """The selective-state recurrence over a packed step: fp32 ``y [tokens, heads * vdim]``; ``ssm`` (fp32 view, first axis the slot, each
    slot ``[heads, state, vdim]``) is read and left at the state after each request's last token."""
    _need(xbc, "xbc")
    _need(proj, "proj")
    if ssm.dtype != torch.float32 or ssm.stride(-1) != 1:
        raise KernelError("mamba_scan: the state must be fp32 with a dense last axis")
    n = xbc.shape[0]
    y = torch.empty((n, heads * vdim), dtype=torch.float32, device=xbc.device)
    _done(_lib().oxr_mamba_scan(y.data_ptr(), xbc.data_ptr(), proj.data_ptr(), n_requests, proj.shape[1], dt_col0, heads, vdim, state, groups,
                                dt_bias.data_ptr(), a_log.data_ptr(), d_skip.data_ptr(), ssm.data_ptr(), ssm.stride(0), cu_q.data_ptr(),
                                state_slots.data_ptr(), _dtype_code(xbc), _stream()), "mamba_scan")
    return y


def gated_group_norm(y: torch.Tensor, proj: torch.Tensor, z_col0: int, weight: torch.Tensor, parts: int, eps: float) -> torch.Tensor:
    """``v = y * silu(z)`` with z the columns ``[z_col0, z_col0 + inner)`` of ``proj``; each of ``parts`` equal stretches of ``v`` is divided by
    its own root mean square, times ``weight``; rounded to ``proj.dtype``."""
    _need(y, "y", torch.float32)
    _need(proj, "proj")
    _need(weight, "weight", torch.float32)
    n, inner = y.shape
    out = torch.empty((n, inner), dtype=proj.dtype, device=y.device)
    _done(_lib().oxr_gated_group_norm(out.data_ptr(), y.data_ptr(), proj.data_ptr(), n, proj.shape[1], z_col0, weight.data_ptr(), inner, parts,
                                      float(eps), _dtype_code(proj), _stream()), "gated_group_norm")
    return out


# --------------------------------------------------------------------------------------------------- attention with mask and sizes as arguments
def scatter_rows(pool: torch.Tensor, src: torch.Tensor, col0: int, slots: torch.Tensor, status: torch.Tensor, pool2: torch.Tensor | None = None) -> None:
    """``pool[slots[t]] = src[t, col0 : col0 + width]`` for a pool ``[pages, page_size, ...]`` whose slot rows hold ``width`` values; slot -1
    skips. With ``pool2`` (the values beside the keys) the columns that follow go to its slot rows in the same launch."""
    _need(pool, "pool")
    _need(src, "src", pool.dtype)
    n_slots = pool.shape[0] * pool.shape[1]
    row = pool[0, 0].numel()
    row2 = 0
    if pool2 is not None:
        _need(pool2, "pool2", pool.dtype)
        if pool2.shape[:2] != pool.shape[:2]:
            raise KernelError("scatter_rows: the two pools differ in pages or page size")
        row2 = pool2[0, 0].numel()
    if col0 + row + row2 > src.shape[1]:
        raise KernelError(f"scatter_rows: columns {col0}..{col0 + row + row2} are beyond the source's {src.shape[1]}")
    _done(_lib().oxr_scatter_rows(pool.data_ptr(), row, n_slots, src.data_ptr(), src.shape[1], col0, row, slots.data_ptr(), src.shape[0],
                                  _dtype_code(src), status.data_ptr(), _ptr(pool2), row2, row2, _stream()), "scatter_rows")


def latent_prep(pool: torch.Tensor, down: torch.Tensor, rank: int, rot: int, weight: torch.Tensor, eps: float, q: torch.Tensor, heads: int,
                q_head_dim: int, q_rot0: int, q_out: torch.Tensor, qo_head_dim: int, qo_rot0: int, cos: torch.Tensor, sin: torch.Tensor,
                slots: torch.Tensor, status: torch.Tensor) -> None:
    """Per token: the latent cache row ``[rmsnorm(down[:rank]) * weight | rotate(down[rank:])]`` goes to ``pool[slot]`` (slot -1: not stored), and
    every head's rotated query part ``rotate(q[h, q_rot0 : q_rot0 + rot])`` to ``q_out[h, qo_rot0 : ...]``. ``rotate`` turns entry pairs (2i, 2i+1)
    by the token's angle i (``cos``/``sin`` ``[tokens, half]``); entries past ``2 * half`` pass unchanged."""
    _need(pool, "pool")
    _need(down, "down", pool.dtype)
    _need(q, "q", pool.dtype)
    _need(q_out, "q_out", pool.dtype)
    _need(cos, "cos", torch.float32)
    n = down.shape[0]
    if down.shape[1] != rank + rot or pool[0, 0].numel() != rank + rot:
        raise KernelError("latent_prep: sizes of the down projection and the pool do not fit")
    _done(_lib().oxr_latent_prep(pool.data_ptr(), rank + rot, pool.shape[0] * pool.shape[1], down.data_ptr(), rank, rot, weight.data_ptr(), float(eps),
                                 q.data_ptr(), heads, q_head_dim, q_rot0, q_out.data_ptr(), qo_head_dim, qo_rot0, cos.data_ptr(), sin.data_ptr(),
                                 cos.shape[1], slots.data_ptr(), n, _dtype_code(down), status.data_ptr(), _stream()), "latent_prep")


def head_linear(out: torch.Tensor, out0: int, x: torch.Tensor, x0: int, weight: torch.Tensor) -> torch.Tensor:
    """``out[t, h, out0 : out0 + n_out] = x[t, h, x0 : x0 + n_in] @ weight[h]`` for ``weight [heads, n_in, n_out]``; ``x`` and ``out`` are
    ``[tokens, heads, *]``; fp32 sums."""
    _need(out, "out")
    _need(x, "x", out.dtype)
    _need(weight, "weight", out.dtype)
    heads, n_in, n_out = weight.shape
    n = x.shape[0]
    if x.shape[1] != heads or out.shape[1] != heads or x0 + n_in > x.shape[2] or out0 + n_out > out.shape[2]:
        raise KernelError("head_linear: sizes do not fit")
    _done(_lib().oxr_head_linear(out.data_ptr(), out.shape[2], out0, x.data_ptr(), x.shape[2], x0, weight.data_ptr(), n_in, n_out, heads, n,
                                 _dtype_code(x), _stream()), "head_linear")
    return out


def attention_rows(q: torch.Tensor, num_heads: int, k_pool: torch.Tensor, v_pool: torch.Tensor | None, *, value_dim: int, positions: torch.Tensor,
                   req_of_token: torch.Tensor, block_table: torch.Tensor, scale: float, chunk: int = 0, window: int = 0, keep_first: int = 0,
                   dist_bias: torch.Tensor | None = None, sink: torch.Tensor | None = None, status: torch.Tensor) -> torch.Tensor:
    """Attention of the step's tokens over the paged cache with the mask and every size as an argument, in fp32 arithmetic.

    ``q [tokens, >= H * DK]``: the queries are the first ``H * DK`` columns (so a stacked q|k|v product can be handed over as it is);
    ``k_pool [pages, page_size, KV, DK]``; ``v_pool [pages, page_size, KV, DV]`` or None, when the values are the first ``value_dim`` entries
    of the key rows (a latent cache). Token t at position p of its request sees keys j <= p, within its chunk of ``chunk`` positions
    (counted from 0) and within its last ``window`` keys when those are given; with a window the request's first ``keep_first`` keys stay
    visible too. ``dist_bias [rows, H]`` (fp32) is added to the scaled score by
    distance p - j (the last row for all larger ones); ``sink [H]`` adds ``exp(sink)`` to the softmax denominator.
    Returns ``[tokens, H * value_dim]``."""
    _need(q, "q")
    _need(k_pool, "k_pool", q.dtype)
    n, H = q.shape[0], int(num_heads)
    pages, page_size, KV, DK = k_pool.shape
    if q.dim() != 2 or q.shape[1] < H * DK:
        raise KernelError(f"attention_rows: {H} heads of {DK} do not fit rows of {tuple(q.shape)}")
    if v_pool is None:
        v, v_slot, v_head = k_pool, KV * DK, DK
        if value_dim > DK:
            raise KernelError("attention_rows: values read from key rows cannot be wider than the keys")
    else:
        _need(v_pool, "v_pool", q.dtype)
        if v_pool.shape[:3] != k_pool.shape[:3] or v_pool.shape[3] != value_dim:
            raise KernelError("attention_rows: the value pool does not fit the key pool")
        v, v_slot, v_head = v_pool, KV * value_dim, value_dim
    bias_rows = 0
    if dist_bias is not None:
        _need(dist_bias, "dist_bias", torch.float32)
        if dist_bias.dim() != 2 or dist_bias.shape[1] != H:
            raise KernelError("attention_rows: the distance bias must be [rows, heads]")
        bias_rows = dist_bias.shape[0]
    if sink is not None:
        _need(sink, "sink", torch.float32)
    out = torch.empty((n, H * value_dim), dtype=q.dtype, device=q.device)
    _done(_lib().oxr_attention_rows(out.data_ptr(), q.data_ptr(), q.shape[1], k_pool.data_ptr(), KV * DK, DK, v.data_ptr(), v_slot, v_head, DK, value_dim, H,
                                    KV, n, positions.data_ptr(), req_of_token.data_ptr(), block_table.data_ptr(), block_table.shape[1], page_size, pages,
                                    float(scale), int(chunk), int(window), int(keep_first) if window > 0 else 0, _ptr(dist_bias), bias_rows, _ptr(sink), _dtype_code(q), status.data_ptr(),
                                    _stream()), "attention_rows")
    return out


# --------------------------------------------------------------------------------------------------- convolved q|k|v, biases
def conv_qkv_store(proj: torch.Tensor, cq: int, ck: int, cv: int, *, conv: torch.Tensor | None, bias: torch.Tensor | None, tails: torch.Tensor | None,
                   k_pool: torch.Tensor, v_pool: torch.Tensor, slots: torch.Tensor, req_of_token: torch.Tensor, cu_q: torch.Tensor,
                   state_slots: torch.Tensor, positions: torch.Tensor, n_requests: int, status: torch.Tensor, temp_coef: float = 0.0,
                   temp_every: int = 0, blend: torch.Tensor | None = None, first: torch.Tensor | None = None, keep_values: bool = False,
                   single_tokens: bool = False, conv_t: torch.Tensor | None = None, q_head_width: int | None = None
                   ) -> tuple[torch.Tensor, torch.Tensor | None]:
    """From a packed step's stacked projection ``proj [tokens, >= cq + ck + cv]`` to queries and cache rows in one launch (and one more that
    rolls the tails): add ``bias [cq + ck + cv]``, filter every channel causally with ``conv [channels, taps]`` (the last tap meets the current
    token; what stands before a step's first token comes from the request's ``tails`` row ``[channels, taps - 1]``, zero for a new request,
    which is rolled forward), multiply the queries by ``1 + temp_coef ln(floor((p + 1) / temp_every) + 1)`` (``temp_every`` 0: not), blend the
    values as ``(1 - blend) v + blend first`` (``blend``: one fp32 number on the device; ``first [tokens, cv]``), and write keys and values to
    ``k_pool`` / ``v_pool`` (one layer's ``[pages, page_size, KV, D]``) at ``slots`` (-1 skips). ``conv`` None: no filter. ``conv_t``: the same filter
    transposed, ``[taps, channels]``, which the 16-byte bfloat16 kernel reads (without it the scalar kernel runs). ``single_tokens``: the
    caller knows that every request brings exactly one token (token r is request r's); the bfloat16 kernel then rolls the tails itself.
    The pools' last axis may be wider than a key or value head (a cache that pads both to one size): only the first entries of each head are
    written. ``q_head_width``: the width a query head takes in the result (zeros behind its entries; default: its own size).
    Returns the queries ``[tokens, heads * q_head_width]`` and, with ``keep_values``, the values ``[tokens, cv]`` as they were cached."""
    _need(proj, "proj")
    _need(k_pool, "k_pool", proj.dtype)
    _need(v_pool, "v_pool", proj.dtype)
    n, channels = proj.shape[0], cq + ck + cv
    taps = 0
    if conv is not None:
        _need(conv, "conv", torch.float32)
        if conv.shape[0] != channels:
            raise KernelError(f"conv_qkv_store: the filter has {conv.shape[0]} channels for {channels}")
        taps = conv.shape[1]
        if conv_t is not None:
            _need(conv_t, "conv_t", torch.float32)
            if conv_t.shape != (taps, channels):
                raise KernelError("conv_qkv_store: the transposed filter must be [taps, channels]")
    if bias is not None:
        _need(bias, "bias", torch.float32)
        if bias.numel() != channels:
            raise KernelError("conv_qkv_store: one bias per channel")
    if taps > 1:
        if tails is None or tails.dtype != torch.float32 or tails.stride(-1) != 1 or tails[0].numel() < channels * (taps - 1):
            raise KernelError("conv_qkv_store: the tails must be fp32 rows of channels x (taps - 1) with a dense last axis")
    kv_heads, kw, vw = k_pool.shape[2], k_pool.shape[3], v_pool.shape[3]
    if ck % kv_heads or cv % kv_heads or k_pool.shape[:3] != v_pool.shape[:3]:
        raise KernelError("conv_qkv_store: the pools do not fit the key and value columns")
    dk, dv = ck // kv_heads, cv // kv_heads
    qw = dk if q_head_width is None else int(q_head_width)
    if kw < dk or vw < dv or qw < dk or cq % dk:
        raise KernelError("conv_qkv_store: a head of the pools or of the result is narrower than the projection's")
    if blend is not None:
        _need(blend, "blend", torch.float32)
        _need(first, "first", proj.dtype)
        if first.shape != (n, cv):
            raise KernelError("conv_qkv_store: the values to blend with must be [tokens, cv]")
    q = (torch.empty if qw == dk else torch.zeros)((n, cq // dk * qw), dtype=proj.dtype, device=proj.device)
    v = torch.empty((n, cv), dtype=proj.dtype, device=proj.device) if keep_values else None
    _done(_lib().oxr_conv_qkv_store(q.data_ptr(), _ptr(v), proj.data_ptr(), n, n_requests, proj.shape[1], cq, ck, cv, taps, _ptr(conv), _ptr(conv_t) if conv is not None else None, _ptr(bias),
                                    _ptr(tails), tails.stride(0) if tails is not None else 0, req_of_token.data_ptr(), cu_q.data_ptr(),
                                    state_slots.data_ptr(), positions.data_ptr(), float(temp_coef), int(temp_every), _ptr(blend), _ptr(first),
                                    k_pool.data_ptr(), v_pool.data_ptr(), slots.data_ptr(), k_pool.shape[0] * k_pool.shape[1], _dtype_code(proj),
                                    int(bool(single_tokens) and n == n_requests), dk, dv, qw, kw, vw, status.data_ptr(), _stream()), "conv_qkv_store")
    global launch_count
    launch_count += 1 if taps > 1 and not (single_tokens and n == n_requests and proj.dtype == torch.bfloat16 and conv_t is not None) else 0
    return q, v


def add_bias_(x: torch.Tensor, row: torch.Tensor) -> torch.Tensor:
    """``x[t] += row`` in place (the sum in fp32)."""
    _need(x, "x")
    _need(row, "row", torch.float32)
    if x.dim() != 2 or row.numel() != x.shape[1]:
        raise KernelError("add_bias_: one entry per column")
    _done(_lib().oxr_add_bias(x.data_ptr(), row.data_ptr(), x.shape[0], x.shape[1], _dtype_code(x), _stream()), "add_bias")
    return x


def scale_(x: torch.Tensor, scale: float) -> torch.Tensor:
    """``x *= scale`` in place for an fp32 tensor."""
    _need(x, "x", torch.float32)
    _done(_lib().oxr_scale_f32(x.data_ptr(), float(scale), x.numel(), _stream()), "scale")
    return x


# --------------------------------------------------------------------------------------------------- matrix memory (mLSTM)
def mlstm_scan(proj: torch.Tensor, q_col0: int, k_col0: int, v_col0: int, gates: torch.Tensor, gate_bias: torch.Tensor, *, heads: int, key_dim: int,
               value_dim: int, cap: float, q_scale: float, state: torch.Tensor, cu_q: torch.Tensor, state_slots: torch.Tensor, n_requests: int
               ) -> torch.Tensor:
    """The matrix-memory recurrence over a packed step: fp32 ``o [tokens, heads * value_dim]`` (before the per-head norm). ``proj`` holds q, k and
    v head by head from the given columns; ``gates [tokens, 2 * heads]`` (fp32) the input- and forget-gate projections, ``gate_bias [2 * heads]``
    their biases; ``state`` (fp32, first axis the slot: S ``[heads, key_dim, value_dim]``, n ``[heads, key_dim]``, m ``[heads]``) is read and left at
    the state after each request's last token."""
    _need(proj, "proj")
    _need(gates, "gates", torch.float32)
    _need(gate_bias, "gate_bias", torch.float32)
    if state.dtype != torch.float32 or state.stride(-1) != 1 or state[0].numel() < heads * key_dim * (value_dim + 1) + heads:
        raise KernelError("mlstm_scan: the state must be fp32 rows of heads x (key_dim x value_dim + key_dim + 1)")
    n = proj.shape[0]
    if gates.shape != (n, 2 * heads) or gate_bias.numel() != 2 * heads:
        raise KernelError("mlstm_scan: gates must be [tokens, 2 * heads] with one bias each")
    y = torch.empty((n, heads * value_dim), dtype=torch.float32, device=proj.device)
    coef = torch.empty((n, heads, 3), dtype=torch.float32, device=proj.device)   # per token and head: what the gate kernel hands the recurrence
    global launch_count
    launch_count += 1
    _done(_lib().oxr_mlstm_scan(y.data_ptr(), coef.data_ptr(), proj.data_ptr(), n_requests, proj.shape[1], q_col0, k_col0, v_col0, gates.data_ptr(), gate_bias.data_ptr(),
                                heads, key_dim, value_dim, float(cap), float(q_scale), state.data_ptr(), state.stride(0), cu_q.data_ptr(),
                                state_slots.data_ptr(), _dtype_code(proj), _stream()), "mlstm_scan")
    return y


def head_norm_gate(y: torch.Tensor, proj: torch.Tensor, gate_col0: int, weight: torch.Tensor, heads: int, eps: float, silu: bool = False) -> torch.Tensor:
    """``y [tokens, heads * d]`` (fp32): every head's stretch divided by its own root mean square, times ``weight``, times the sigmoid (``silu``:
    the SiLU) of the columns ``[gate_col0, gate_col0 + heads * d)`` of ``proj``; rounded to ``proj.dtype``."""
    _need(y, "y", torch.float32)
    _need(proj, "proj")
    _need(weight, "weight", torch.float32)
    n, inner = y.shape
    if inner % heads or weight.numel() != inner or gate_col0 + inner > proj.shape[1]:
        raise KernelError("head_norm_gate: sizes do not fit")
    out = torch.empty((n, inner), dtype=proj.dtype, device=y.device)
    _done(_lib().oxr_head_norm_gate(out.data_ptr(), y.data_ptr(), proj.data_ptr(), n, proj.shape[1], gate_col0, weight.data_ptr(), heads, inner // heads,
                                    float(eps), int(bool(silu)), _dtype_code(proj), _stream()), "head_norm_gate")
    return out


# --------------------------------------------------------------------------------------------------- routed experts
ROUTE_SCORES = {"sigmoid": 0, "softmax": 1}
ROUTE_GROUP_SCORES = {"top2_sum": 0, "max": 1}


def route(z: torch.Tensor, *, top: int, groups: int, keep: int, scale: float, score: str = "sigmoid", group_score: str = "top2_sum",
          renormalize: bool = True) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Router logits ``z [tokens, E]`` (fp32) to the choice of ``top`` experts per token. Scores are ``sigmoid(z)`` or, with ``score="softmax"``,
    the softmax of z over all experts; of ``groups`` equal groups of neighbouring experts only the ``keep`` best may be chosen from, a group's
    score being the sum of its two best scores (``"top2_sum"``) or its best score (``"max"``); the weights are the chosen scores over their sum
    (``renormalize``) or as they are, times ``scale``. Returns ``gate [tokens, E]`` (fp32: a chosen expert's weight, else 0), ``ids [tokens, top]``
    (int32) and ``weights [tokens, top]`` (fp32)."""
    _need(z, "z", torch.float32)
    n, E = z.shape
    gate = torch.empty((n, E), dtype=torch.float32, device=z.device)
    ids = torch.empty((n, top), dtype=torch.int32, device=z.device)
    wts = torch.empty((n, top), dtype=torch.float32, device=z.device)
    _done(_lib().oxr_route(gate.data_ptr(), ids.data_ptr(), wts.data_ptr(), z.data_ptr(), n, E, int(top), int(groups), int(keep), float(scale),
                           ROUTE_SCORES[score], ROUTE_GROUP_SCORES[group_score], int(bool(renormalize)), _stream()), "route")
    return gate, ids, wts


def expert_clamped_glu(gu: torch.Tensor, gate: torch.Tensor | None, ff: int, *, alpha: float, limit: float) -> torch.Tensor:
    """The clamped gated unit over the stacked gate and up projections of all experts: ``gu [tokens, E * 2 ff]`` holds, expert by expert,
    ``[gate (ff) | up (ff)]``; ``a[t, e ff + c] = gate[t, e] * g sigmoid(alpha g) (u + 1)`` with ``g = min(gate_c, limit)`` and
    ``u = clamp(up_c, -limit, limit)``; ``gate`` None: no weight (one expert's rows)."""
    _need(gu, "gu")
    n, cols2 = gu.shape
    E = cols2 // (2 * ff)
    if cols2 != E * 2 * ff or E < 1:
        raise KernelError("expert_clamped_glu: sizes do not fit")
    if gate is not None:
        _need(gate, "gate", torch.float32)
        if gate.shape != (n, E):
            raise KernelError("expert_clamped_glu: sizes do not fit")
    a = torch.empty((n, E * ff), dtype=gu.dtype, device=gu.device)
    _done(_lib().oxr_expert_clamped_glu(a.data_ptr(), gu.data_ptr(), _ptr(gate), n, E, int(ff), float(alpha), float(limit), _dtype_code(gu), _stream()),
          "expert_clamped_glu")
    return a


def gated_relu2(u: torch.Tensor, gate: torch.Tensor | None, ff: int, out: torch.Tensor | None = None) -> torch.Tensor:
    """``a[t, c] = gate[t, c // ff] * relu(u[t, c])^2`` for the stacked up-projections ``u [tokens, E * ff]`` of all experts; ``gate`` None: plain
    ``relu(u)^2``. ``out`` may be ``u`` itself."""
    _need(u, "u")
    n, cols = u.shape
    E = cols // ff
    if gate is not None:
        _need(gate, "gate", torch.float32)
        if gate.shape != (n, E):
            raise KernelError("gated_relu2: sizes do not fit")
    if cols != E * ff:
        raise KernelError("gated_relu2: sizes do not fit")
    a = torch.empty_like(u) if out is None else out
    _done(_lib().oxr_gated_relu2(a.data_ptr(), u.data_ptr(), _ptr(gate), n, E, int(ff), _dtype_code(u), _stream()), "gated_relu2")
    return a


GROUP_TILE_ROWS = 128
"""Rows per tile of the grouped product: every group's rows are padded to a multiple of it."""


def expert_sort(ids: torch.Tensor, experts: int, pad: int = 1) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor | None]:
    """The (token, choice) pairs of ``ids [tokens, top]`` ordered by expert: ``counts [experts]`` (int32), ``order`` (the flat pair index at each
    place of the ordered list, -1 at padding places) and ``place [tokens * top]`` (where each pair stands in the list). Pairs of one expert stand
    in no particular order. ``pad`` > 1: every expert's stretch starts at a multiple of ``pad``; the list then has room for the worst case
    (``tokens * top + experts * (pad - 1)``, rounded up), and the fourth result says which expert each tile of ``pad`` places belongs to."""
    _need(ids, "ids", torch.int32)
    total = ids.numel()
    capacity = total if pad <= 1 else -(-(total + experts * (pad - 1)) // pad) * pad
    counts = torch.empty(experts, dtype=torch.int32, device=ids.device)
    order = torch.empty(capacity, dtype=torch.int32, device=ids.device)
    place = torch.empty(total, dtype=torch.int32, device=ids.device)
    tile_group = torch.empty(capacity // pad, dtype=torch.int32, device=ids.device) if pad > 1 else None
    _done(_lib().oxr_expert_sort(counts.data_ptr(), order.data_ptr(), place.data_ptr(), _ptr(tile_group), ids.data_ptr(), total, int(experts), int(pad),
                                 capacity, _stream()), "expert_sort")
    return counts, order, place, tile_group


def grouped_linear_takes(x_dtype: torch.dtype, weight: torch.Tensor, k: int) -> bool:
    """Whether :func:`grouped_linear` serves these operands: bfloat16 with rows of whole 16-byte words."""
    return x_dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and k % 8 == 0 and weight.data_ptr() % 16 == 0


def grouped_linear(x: torch.Tensor, weight: torch.Tensor, tile_group: torch.Tensor, n: int, out_dtype: torch.dtype | None = None,
                   relu2: bool = False) -> torch.Tensor:
    """``out[r] = x[r] @ weight[g n : (g + 1) n].T`` with ``g = tile_group[r // GROUP_TILE_ROWS]``: rows ordered by the matrix they multiply (each
    group padded to whole tiles of rows), ``weight [groups * n, k]`` the matrices stacked. One launch of the TMA + tcgen05 kernel, whatever
    the groups' sizes, which stay on the device. A tile whose group is -1 is not computed (its rows of ``out`` are left unwritten: nobody
    may read them). ``relu2``: the epilogue writes ``relu(out)^2`` of the fp32 sums."""
    _need(x, "x", torch.bfloat16)
    _need(weight, "weight", torch.bfloat16)
    _need(tile_group, "tile_group", torch.int32)
    m, k = x.shape
    if weight.shape[1] != k or weight.shape[0] % n or m % GROUP_TILE_ROWS or tile_group.numel() != m // GROUP_TILE_ROWS or k % 8:
        raise KernelError("grouped_linear: sizes do not fit")
    out_dtype = out_dtype or x.dtype
    out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    tile_n, _ = _gemm_plan(m, n, k, False)
    _done(_lib().oxr_gemm_tcgen05_grouped_bf16(out.data_ptr(), x.data_ptr(), weight.data_ptr(), m, n, k, weight.shape[0] // n, tile_group.data_ptr(),
                                               _DT[out_dtype], tile_n, int(relu2), new_status(x.device).data_ptr(), _stream()), "gemm_tcgen05_grouped")
    return out


def gather_rows(x: torch.Tensor, order: torch.Tensor, per_row: int) -> torch.Tensor:
    """``out[i] = x[order[i] // per_row]``: the rows of ``x`` repeated and put in the order of a sorted list of (row, choice) pairs."""
    _need(x, "x")
    _need(order, "order", torch.int32)
    out = torch.empty((order.numel(), x.shape[1]), dtype=x.dtype, device=x.device)
    _done(_lib().oxr_gather_rows(out.data_ptr(), x.data_ptr(), order.data_ptr(), order.numel(), x.shape[1], int(per_row), _dtype_code(x), _stream()),
          "gather_rows")
    return out


def combine_rows(y: torch.Tensor, place: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
    """``out[t] = sum_j weights[t, j] * y[place[t * top + j]]`` with the sum in fp32 in the order of j; ``y [>= tokens * top, width]``."""
    _need(y, "y")
    _need(place, "place", torch.int32)
    _need(weights, "weights", torch.float32)
    n, top = weights.shape
    if place.numel() != n * top or y.shape[0] < n * top:
        raise KernelError("combine_rows: sizes do not fit")
    out = torch.empty((n, y.shape[1]), dtype=y.dtype, device=y.device)
    _done(_lib().oxr_combine_rows(out.data_ptr(), y.data_ptr(), place.data_ptr(), weights.data_ptr(), n, top, y.shape[1], _dtype_code(y), _stream()),
          "combine_rows")
    return out


# --------------------------------------------------------------------------------------------------- heads between projection and attention
HEAD_NORMS = {None: 0, "weighted": 1, "unit": 2}


def head_prep(proj: torch.Tensor, *, q_col0: int, k_col0: int | None, v_col0: int | None, values_are_keys: bool = False, num_heads: int,
              num_kv_heads: int, key_dim: int, value_dim: int, bias: torch.Tensor | None = None, taps: torch.Tensor | None = None,
              taps_t: torch.Tensor | None = None, tails: torch.Tensor | None = None, norm: str | None = None, norm_after_rotation: bool = False, q_weight: torch.Tensor | None = None,
              k_weight: torch.Tensor | None = None, eps: float = 0.0, cos: torch.Tensor | None = None, sin: torch.Tensor | None = None,
              k_pool: torch.Tensor | None = None, v_pool: torch.Tensor | None = None, slots: torch.Tensor, req_of_token: torch.Tensor,
              cu_q: torch.Tensor, state_slots: torch.Tensor, n_requests: int, status: torch.Tensor) -> torch.Tensor:
    """Query and key heads on their way from the projections ``proj [tokens, *]`` to attention, and the cache write. In this order, each step
    optional: ``bias [H DK + KV DK]`` (fp32, q then k) is added; every channel passes a causal filter ``taps [channels, n]`` (the last tap on
    the current token; ``taps_t``, the same transposed, lets the 16-byte bfloat16 kernel run; earlier tokens come from the step's rows or from
    the request's row of ``tails``, fp32 ``[slots, (n - 1) * channels]``, the oldest value of all channels first, which is moved on afterwards); with ``values_are_keys`` the filtered keys are stored as the values; every head is RMS-normed
    (``norm="weighted"``: times ``q_weight`` / ``k_weight [DK]``; ``"unit"``: no weight) before or after the rotation; the pairs
    ``(i, i + half)`` of each head's first ``2 half`` entries turn by the token's angles (``cos``, ``sin`` fp32 ``[tokens, half]``). Keys and
    values go to ``k_pool`` / ``v_pool [pages, page_size, KV, D]`` at ``slots`` (-1: not stored); ``k_col0`` None: queries only. Returns
    ``q [tokens, H * DK]``. All arithmetic fp32, one rounding."""
    _need(proj, "proj")
    n = proj.shape[0]
    H, KV, DK, DV = int(num_heads), int(num_kv_heads), int(key_dim), int(value_dim)
    has_k = k_col0 is not None
    v_mode = 0 if not has_k else (2 if values_are_keys else (1 if v_col0 is not None else 0))
    pool_slots = 0
    if has_k:
        _need(k_pool, "k_pool", proj.dtype)
        _need(v_pool, "v_pool", proj.dtype)
        if tuple(k_pool.shape[2:]) != (KV, DK) or tuple(v_pool.shape[2:]) != (KV, DV) or v_pool.shape[:2] != k_pool.shape[:2]:
            raise KernelError("head_prep: the pools do not fit the heads")
        pool_slots = k_pool.shape[0] * k_pool.shape[1]
    channels = H * DK + (KV * DK if has_k else 0)
    n_taps = 0
    tail_stride = 0
    if bias is not None:
        _need(bias, "bias", torch.float32)
        if bias.numel() != channels:
            raise KernelError("head_prep: one bias per query and key channel")
    if taps is not None:
        _need(taps, "taps", torch.float32)
        n_taps = taps.shape[1]
        if taps.shape[0] != channels:
            raise KernelError("head_prep: one filter per query and key channel")
        if taps_t is not None:
            _need(taps_t, "taps_t", torch.float32)
            if taps_t.shape != (n_taps, channels):
                raise KernelError("head_prep: taps_t must be taps transposed")
        if n_taps > 1:
            if tails is None or tails.dtype != torch.float32 or tails.stride(-1) != 1 or tails.shape[1] < channels * (n_taps - 1):
                raise KernelError("head_prep: the filter needs fp32 tails of channels * (taps - 1) per slot")
            tail_stride = tails.stride(0)
    half = 0
    if cos is not None:
        _need(cos, "cos", torch.float32)
        _need(sin, "sin", torch.float32)
        half = cos.shape[1]
        if cos.shape != (n, half) or sin.shape != (n, half):
            raise KernelError("head_prep: angles must be [tokens, half]")
    for w in (q_weight, k_weight):
        if w is not None:
            _need(w, "norm weight", torch.float32)
    q = torch.empty((n, H * DK), dtype=proj.dtype, device=proj.device)
    _done(_lib().oxr_head_prep(q.data_ptr(), _ptr(k_pool) if has_k else None, _ptr(v_pool) if has_k else None, proj.data_ptr(), n, int(n_requests),
                               proj.shape[1], int(q_col0), int(k_col0 or 0), int(v_col0 or 0), H, KV, DK, DV, int(has_k), v_mode, _ptr(bias), _ptr(taps),
                               _ptr(taps_t) if taps is not None else None, n_taps, _ptr(tails) if n_taps > 1 else None, tail_stride, HEAD_NORMS[norm], int(bool(norm_after_rotation)), _ptr(q_weight),
                               _ptr(k_weight), float(eps), _ptr(cos), _ptr(sin), half, slots.data_ptr(), pool_slots, req_of_token.data_ptr(),
                               cu_q.data_ptr(), state_slots.data_ptr(), _dtype_code(proj), status.data_ptr(), _stream()), "head_prep")
    global launch_count
    launch_count += 1 if n_taps > 1 else 0      # the kernel that moves the tails on
    return q


def sigmoid_gate_(o: torch.Tensor, proj: torch.Tensor, gate_col0: int, value_dim: int, per_head: bool) -> torch.Tensor:
    """In place ``o[t, h * d + j] *= sigmoid(proj[t, gate_col0 + c])`` with ``c = h`` (``per_head``: one gate per head) or ``c = h * d + j`` (one per
    channel); the sigmoid in fp32."""
    _need(o, "o")
    _need(proj, "proj", o.dtype)
    n, inner = o.shape
    cols = inner // value_dim if per_head else inner
    if inner % value_dim or gate_col0 + cols > proj.shape[1]:
        raise KernelError("sigmoid_gate: sizes do not fit")
    _done(_lib().oxr_sigmoid_gate(o.data_ptr(), proj.data_ptr(), n, proj.shape[1], int(gate_col0), inner, int(value_dim), int(bool(per_head)),
                                  _dtype_code(o), _stream()), "sigmoid_gate")
    return o


def gla_scan(proj: torch.Tensor, q_col0: int, k_col0: int, v_col0: int, z: torch.Tensor, z_bias: torch.Tensor, *, heads: int, key_dim: int,
             value_dim: int, tau: float, q_scale: float, state: torch.Tensor, cu_q: torch.Tensor, state_slots: torch.Tensor, n_requests: int,
             key_entries_per_thread: int = 0) -> torch.Tensor:
    """Gated linear attention over a packed step: per head ``S_t = diag(alpha_t) S_(t-1) + k_t v_t^T``, ``o_t = S_t^T (q_t * q_scale)`` with the decay
    ``alpha_t = sigmoid(z_t + z_bias)^(1 / tau)`` per key channel. ``proj`` holds q, k and v head by head from the given columns; ``z [tokens, heads *
    key_dim]`` is fp32; ``state`` (fp32, first axis the slot: S ``[heads, key_dim, value_dim]``) is read and left at the state after each request's
    last token. Returns fp32 ``o [tokens, heads * value_dim]``. ``key_entries_per_thread`` (16 or 32) forces the kernel's split of a head's
    key channels over threads; 0 chooses by the step's shape."""
    _need(proj, "proj")
    _need(z, "z", torch.float32)
    _need(z_bias, "z_bias", torch.float32)
    if state.dtype != torch.float32 or state.stride(-1) != 1 or state.shape[1] < heads * key_dim * value_dim:
        raise KernelError("gla_scan: the state must be fp32 rows of heads x key_dim x value_dim")
    n = proj.shape[0]
    if z.shape != (n, heads * key_dim) or z_bias.numel() != heads * key_dim:
        raise KernelError("gla_scan: the decay logits must be [tokens, heads * key_dim] with one bias each")
    y = torch.empty((n, heads * value_dim), dtype=torch.float32, device=proj.device)
    if not key_entries_per_thread:
        # portions of prompts: twice the warps per head hide the loop's latencies (1,069 -> 770 us for 2,048 tokens of 16 heads of 128 x 256);
        # single tokens: the state's trip through the registers is all there is, and fewer partial sums are cheaper (20.5 against 24.6 us)
        key_entries_per_thread = 16 if n > 2 * n_requests else 32
    _done(_lib().oxr_gla_scan(y.data_ptr(), proj.data_ptr(), int(n_requests), proj.shape[1], int(q_col0), int(k_col0), int(v_col0), z.data_ptr(),
                              z_bias.data_ptr(), float(tau), int(heads), int(key_dim), int(value_dim), float(q_scale), state.data_ptr(), state.stride(0),
                              cu_q.data_ptr(), state_slots.data_ptr(), _dtype_code(proj), int(key_entries_per_thread), _stream()), "gla_scan")
    return y


def pair_norm_mean(a: torch.Tensor, b: torch.Tensor, wa: torch.Tensor, wb: torch.Tensor, eps: float) -> torch.Tensor:
    """``0.5 * (rmsnorm(a) * wa + rmsnorm(b) * wb)`` row by row (fp32 arithmetic, rounded once to ``a.dtype``)."""
    _need(a, "a")
    _need(b, "b", a.dtype)
    _need(wa, "wa", torch.float32)
    _need(wb, "wb", torch.float32)
    if a.shape != b.shape or wa.numel() != a.shape[1] or wb.numel() != a.shape[1]:
        raise KernelError("pair_norm_mean: sizes do not fit")
    out = torch.empty_like(a)
    _done(_lib().oxr_pair_norm_mean(out.data_ptr(), a.data_ptr(), b.data_ptr(), wa.data_ptr(), wb.data_ptr(), a.shape[0], a.shape[1], float(eps),
                                    _dtype_code(a), _stream()), "pair_norm_mean")
    return out


def tanh_cap_(x: torch.Tensor, cap: float) -> torch.Tensor:
    """In place ``x <- cap * tanh(x / cap)`` (fp32)."""
    _need(x, "x", torch.float32)
    _done(_lib().oxr_tanh_cap(x.data_ptr(), float(cap), x.numel(), _stream()), "tanh_cap")
    return x


def expert_silu_glu(gu: torch.Tensor, gate: torch.Tensor | None, ff: int, *, on_input: bool) -> torch.Tensor:
    """The SiLU-gated unit over the stacked gate and up projections of all experts: ``gu [tokens, E * 2 ff]`` holds, expert by expert,
    ``[gate (ff) | up (ff)]``. With the token's weight ``w = gate[t, e]`` (0: not chosen, the columns become 0; ``gate`` None: 1):
    ``on_input``: ``silu(w g) * (w u)``, the weight on what the expert reads; else ``w * silu(g) * u``."""
    _need(gu, "gu")
    n, cols2 = gu.shape
    E = cols2 // (2 * ff)
    if cols2 != E * 2 * ff or E < 1:
        raise KernelError("expert_silu_glu: sizes do not fit")
    if gate is not None:
        _need(gate, "gate", torch.float32)
        if gate.shape != (n, E):
            raise KernelError("expert_silu_glu: sizes do not fit")
    a = torch.empty((n, E * ff), dtype=gu.dtype, device=gu.device)
    _done(_lib().oxr_expert_silu_glu(a.data_ptr(), gu.data_ptr(), _ptr(gate), n, E, int(ff), int(bool(on_input)), _dtype_code(gu), _stream()),
          "expert_silu_glu")
    return a


def scale_placed_rows_(x: torch.Tensor, place: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
    """In place ``x[place[p]] *= weights[p]`` for every (token, choice) pair p (``place`` as ``expert_sort`` returns it)."""
    _need(x, "x")
    _need(place, "place", torch.int32)
    _need(weights, "weights", torch.float32)
    if place.numel() != weights.numel():
        raise KernelError("scale_placed_rows: one weight per pair")
    _done(_lib().oxr_scale_placed_rows(x.data_ptr(), place.data_ptr(), weights.data_ptr(), place.numel(), x.shape[1], _dtype_code(x), _stream()),
          "scale_placed_rows")
    return x


def add_row_gated_(y: torch.Tensor, s: torch.Tensor, z: torch.Tensor) -> torch.Tensor:
    """In place ``y[t] += sigmoid(z[t]) * s[t]`` with one fp32 logit ``z[t]`` per row."""
    _need(y, "y")
    _need(s, "s", y.dtype)
    _need(z, "z", torch.float32)
    if s.shape != y.shape or z.numel() != y.shape[0]:
        raise KernelError("add_row_gated: sizes do not fit")
    _done(_lib().oxr_add_row_gated(y.data_ptr(), s.data_ptr(), z.data_ptr(), y.shape[0], y.shape[1], _dtype_code(y), _stream()), "add_row_gated")
    return y
