"""Host-side helpers for NVFP4 storage: packed e2m1 codes and the 128x4 tiled
scale-factor layout (python/cutlass_compat/cutlass/utils/blockscaled_layout.py:17-42,
tests/python/test_flashinfer_b12x_verbatim.py:68-89 in the reference).  These
only move bytes around with torch indexing; no arithmetic happens here."""
from __future__ import annotations

import torch

SF_VEC = 16


def ceil_div(a: int, b: int) -> int:
    return -(-a // b)


def swizzled_sf_numel(rows: int, k_blocks: int) -> int:
    return ceil_div(rows, 128) * ceil_div(k_blocks, 4) * 512


def swizzled_sf_shape(rows: int, k_blocks: int):
    """2-D shape conventionally used for a tiled scale tensor: rows padded to
    128, K-blocks padded to 4 (the bytes are NOT row-major inside)."""
    return (ceil_div(rows, 128) * 128, ceil_div(k_blocks, 4) * 4)


def _offsets(rows: int, k_blocks: int, device) -> torch.Tensor:
    rk = ceil_div(k_blocks, 4)
    m = torch.arange(rows, device=device, dtype=torch.int64)[:, None]
    kb = torch.arange(k_blocks, device=device, dtype=torch.int64)[None, :]
    return (m % 32) * 16 + ((m // 32) % 4) * 4 + kb % 4 + (kb // 4) * 512 + (m // 128) * rk * 512


def swizzle_sf(sf: torch.Tensor) -> torch.Tensor:
    """[..., rows, k_blocks] (uint8 or float8_e4m3fn) -> [..., tiles*512] uint8,
    padding written as zero."""
    s = sf.contiguous().view(torch.uint8)
    rows, kb = s.shape[-2:]
    lead = s.shape[:-2]
    out = torch.zeros(*lead, swizzled_sf_numel(rows, kb), dtype=torch.uint8, device=s.device)
    out[..., _offsets(rows, kb, s.device).reshape(-1)] = s.reshape(*lead, rows * kb)
    return out


def unswizzle_sf(swz: torch.Tensor, rows: int, k_blocks: int) -> torch.Tensor:
    """[..., tiles*512] tiled bytes -> [..., rows, k_blocks] uint8."""
    s = swz.contiguous().view(torch.uint8)
    n = swizzled_sf_numel(rows, k_blocks)
    if s.shape[-1] != n:
        s = s.reshape(-1) if s.numel() == n else s.reshape(*s.shape[:-2], n)
    return s[..., _offsets(rows, k_blocks, s.device).reshape(-1)].reshape(*s.shape[:-1], rows, k_blocks)


def six_mode_to_storage(sf6: torch.Tensor) -> torch.Tensor:
    """The MoE weight scale factors arrive as the six-mode view
    (32, 4, m_tiles, 4, k_tiles, E) of storage [E, m_tiles, k_tiles, 32, 4, 4]
    (tests/python/test_flashinfer_b12x_verbatim.py:68-89).  Return that storage
    as a contiguous uint8 tensor [E, m_tiles*k_tiles*512] without copying when
    the view already sits on it."""
    if sf6.dim() != 6 or sf6.shape[0] != 32 or sf6.shape[1] != 4 or sf6.shape[3] != 4:
        raise ValueError(f"expected a (32,4,m_tiles,4,k_tiles,E) scale tensor, got {tuple(sf6.shape)}")
    st = sf6.permute(5, 2, 4, 0, 1, 3)
    if not st.is_contiguous():
        st = st.contiguous()
    return st.view(torch.uint8).reshape(st.shape[0], -1)


def pack_e2m1(codes: torch.Tensor) -> torch.Tensor:
    """[..., K] 4-bit codes (uint8) -> [..., K/2] bytes, even index in the low nibble."""
    return (codes[..., 0::2] | (codes[..., 1::2] << 4)).contiguous()


def unpack_e2m1(packed: torch.Tensor) -> torch.Tensor:
    p = packed.view(torch.uint8)
    return torch.stack([p & 0xF, p >> 4], dim=-1).reshape(*p.shape[:-1], p.shape[-1] * 2)
