"""Drop-in ``rmsnorm_fp4quant`` / ``add_rmsnorm_fp4quant``.

Same call signatures as the flashinfer CuTe-DSL operators the reference loads
and runs (call sites tests/python/test_flashinfer_norm_verbatim.py:134 and
:155-164; tools/perf/bench_flashinfer_norm.py:53-60).  The work is one CUDA
kernel launch on the current stream through ``b200fp4_rmsnorm_fp4quant`` /
``b200fp4_add_rmsnorm_fp4quant``; nothing is computed in Python and there is
no CPU path.

``global_scale`` MULTIPLIES before quantisation (sf = amax * gs / 6), the
convention of the reference's golden (same file, lines 58-68).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib
from .layout import ceil_div, swizzled_sf_numel, swizzled_sf_shape

_DTYPES = {torch.float16: 0, torch.bfloat16: 1}
_ONES = {}


def _unit_scale(device) -> torch.Tensor:
    key = (device.type, device.index)
    if key not in _ONES:
        _ONES[key] = torch.ones(1, dtype=torch.float32, device=device)
    return _ONES[key]


def _check_common(input, weight, block_size, scale_format):
    if not input.is_cuda:
        raise ValueError("input must be a CUDA tensor (there is no CPU implementation)")
    if input.dtype not in _DTYPES:
        raise ValueError(f"input dtype {input.dtype} is not float16/bfloat16")
    if weight.dtype != input.dtype or weight.device != input.device:
        raise ValueError("weight must have the dtype and device of input")
    if block_size != 16:
        raise NotImplementedError("only NVFP4 (block_size=16, e4m3 scale factors) is implemented")
    if scale_format not in (None, "e4m3"):
        raise NotImplementedError(f"scale_format={scale_format!r}: only e4m3 is implemented")
    if input.dim() not in (2, 3):
        raise ValueError("input must be [B, H] or [B, S, H]")
    hidden = input.shape[-1]
    if weight.dim() != 1 or weight.shape[0] != hidden:
        raise ValueError("weight must be [H]")
    if hidden % 16 != 0 or hidden < 64:
        raise ValueError("hidden size must be a multiple of 16 and at least 64")
    if input.stride(-1) != 1:
        raise ValueError("the last dimension of input must be contiguous")


def _rows_view(t: torch.Tensor) -> torch.Tensor:
    """[B,S,H] -> [B*S,H] without copying when possible; [B,H] is returned as is."""
    return t if t.dim() == 2 else t.reshape(-1, t.shape[-1])


def _prep_outputs(rows, hidden, lead_shape, device, y_fp4, block_scale, swizzled):
    kb = hidden // 16
    if y_fp4 is None:
        y_fp4 = torch.empty(*lead_shape, hidden // 2, dtype=torch.uint8, device=device)
    else:
        if y_fp4.numel() * y_fp4.element_size() != rows * hidden // 2 or not y_fp4.is_contiguous():
            raise ValueError("y_fp4 must be contiguous with hidden/2 bytes per row")
    if block_scale is None:
        if swizzled:
            block_scale = torch.empty(swizzled_sf_shape(rows, kb), dtype=torch.uint8, device=device)
        else:
            block_scale = torch.empty(*lead_shape, kb, dtype=torch.uint8, device=device)
    else:
        need = swizzled_sf_numel(rows, kb) if swizzled else rows * kb
        if block_scale.element_size() != 1 or block_scale.numel() < need or not block_scale.is_contiguous():
            raise ValueError(f"block_scale must be a contiguous 1-byte tensor with at least {need} elements")
    return y_fp4, block_scale


def rmsnorm_fp4quant(
    input: torch.Tensor,
    weight: torch.Tensor,
    y_fp4: Optional[torch.Tensor] = None,
    block_scale: Optional[torch.Tensor] = None,
    global_scale: Optional[torch.Tensor] = None,
    eps: float = 1e-6,
    block_size: int = 16,
    scale_format: Optional[str] = None,
    is_sf_swizzled_layout: bool = False,
    enable_pdl: Optional[bool] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """y = RMSNorm(input) * weight, quantised to NVFP4.

    Returns ``(y_fp4, block_scale)``: packed e2m1 codes ``[..., H/2]`` (uint8,
    even element in the low nibble) and e4m3 scale factors, row-major
    ``[..., H/16]`` or, with ``is_sf_swizzled_layout``, in 128x4 tiles.
    ``enable_pdl`` is accepted for signature compatibility and ignored.
    """
    _check_common(input, weight, block_size, scale_format)
    x2 = _rows_view(input)
    rows, hidden = x2.shape
    y_fp4, block_scale = _prep_outputs(rows, hidden, input.shape[:-1], input.device, y_fp4, block_scale,
                                       is_sf_swizzled_layout)
    gs = _unit_scale(input.device) if global_scale is None else global_scale
    if gs.dtype != torch.float32 or gs.device != input.device:
        raise ValueError("global_scale must be a float32 tensor on the input's device")
    if rows == 0:
        return y_fp4, block_scale
    with _lib.on_device(input.device):
        _lib.check(_lib.lib.b200fp4_rmsnorm_fp4quant(
            x2.data_ptr(), weight.contiguous().data_ptr(), y_fp4.data_ptr(), block_scale.data_ptr(), None,
            gs.data_ptr(), float(eps), rows, hidden, x2.stride(0) if rows > 1 else hidden, _DTYPES[input.dtype],
            1 if is_sf_swizzled_layout else 0, _lib.current_stream_ptr(input.device)))
    return y_fp4, block_scale


def add_rmsnorm_fp4quant(
    input: torch.Tensor,
    residual: torch.Tensor,
    weight: torch.Tensor,
    y_fp4: Optional[torch.Tensor] = None,
    block_scale: Optional[torch.Tensor] = None,
    global_scale: Optional[torch.Tensor] = None,
    eps: float = 1e-6,
    block_size: int = 16,
    scale_format: Optional[str] = None,
    is_sf_swizzled_layout: bool = False,
    output_both_sf_layouts: bool = False,
    block_scale_unswizzled: Optional[torch.Tensor] = None,
    enable_pdl: Optional[bool] = None,
):
    """residual <- input + residual (in place); y = RMSNorm(residual) * weight -> NVFP4.

    Returns ``(y_fp4, block_scale)`` or, with ``output_both_sf_layouts``,
    ``(y_fp4, block_scale, block_scale_unswizzled)`` where ``block_scale`` is
    tiled and the third tensor row-major.
    """
    _check_common(input, weight, block_size, scale_format)
    if residual.shape != input.shape or residual.dtype != input.dtype or residual.device != input.device:
        raise ValueError("residual must match input in shape, dtype and device")
    if residual.stride(-1) != 1:
        raise ValueError("the last dimension of residual must be contiguous")
    x2, r2 = _rows_view(input), _rows_view(residual)
    if r2.data_ptr() != residual.data_ptr() or (residual.dim() == 3 and not residual.is_contiguous()):
        raise ValueError("a 3-D residual must be contiguous: it is updated in place")
    rows, hidden = x2.shape
    swizzled = is_sf_swizzled_layout or output_both_sf_layouts
    y_fp4, block_scale = _prep_outputs(rows, hidden, input.shape[:-1], input.device, y_fp4, block_scale, swizzled)
    layout = 2 if output_both_sf_layouts else (1 if swizzled else 0)
    if output_both_sf_layouts:
        if block_scale_unswizzled is None:
            block_scale_unswizzled = torch.empty(*input.shape[:-1], hidden // 16, dtype=torch.uint8,
                                                 device=input.device)
        elif block_scale_unswizzled.numel() < rows * hidden // 16 or block_scale_unswizzled.element_size() != 1:
            raise ValueError("block_scale_unswizzled is too small")
    gs = _unit_scale(input.device) if global_scale is None else global_scale
    if gs.dtype != torch.float32 or gs.device != input.device:
        raise ValueError("global_scale must be a float32 tensor on the input's device")
    if rows == 0:
        return (y_fp4, block_scale, block_scale_unswizzled) if output_both_sf_layouts else (y_fp4, block_scale)
    with _lib.on_device(input.device):
        _lib.check(_lib.lib.b200fp4_add_rmsnorm_fp4quant(
            x2.data_ptr(), r2.data_ptr(), weight.contiguous().data_ptr(), y_fp4.data_ptr(), block_scale.data_ptr(),
            _lib.ptr(block_scale_unswizzled), gs.data_ptr(), float(eps), rows, hidden,
            x2.stride(0) if rows > 1 else hidden, r2.stride(0) if rows > 1 else hidden, _DTYPES[input.dtype], layout,
            _lib.current_stream_ptr(input.device)))
    if output_both_sf_layouts:
        return y_fp4, block_scale, block_scale_unswizzled
    return y_fp4, block_scale


__all__ = ["rmsnorm_fp4quant", "add_rmsnorm_fp4quant", "ceil_div"]
