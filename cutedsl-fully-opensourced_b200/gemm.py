"""NVFP4 block-scaled dense GEMM behind the interface of the CUTLASS demo the
reference runs verbatim (third_party/cutlass/examples/python/CuTeDSL/cute/
blackwell_geforce/kernel/blockscaled_gemm/dense_blockscaled_gemm_persistent_cooperative.py):

* ``Sm120BlockScaledGemmKernel(acc_dtype, sf_vec_size, tile_shape_mnk, epi_tile)``
  with ``__call__(a, b, sfa, sfb, c, max_active_clusters, stream)``  (:149-439);
  the class keeps its name so call sites need no edit, ``Sm100BlockScaledGemmKernel``
  is an alias.
* ``compile(gemm, a, b, sfa, sfb, c, max_active_clusters, stream)`` returning a
  callable ``(a, b, sfa, sfb, c, stream)``  (calling convention of :1773-1787).
* ``run(...)`` / ``run_bs(...)``: the demo's entry points with the same
  arguments (:1529-1903): build integer-valued operands, run, check against an
  f32 product of the de-quantised operands, time, return microseconds.
* ``nvfp4_gemm`` is the plain functional form.

Operands are torch CUDA tensors: A ``[M, K/2]`` and B ``[N, K/2]`` uint8 (two
e2m1 codes per byte, lower K index in the low nibble; an optional leading or
trailing batch mode is accepted), scale factors as bytes in the 128x4 tiled
layout, C ``[M, N]`` fp16 / bf16 / f32.  The kernel is ``b200fp4_nvfp4_gemm``.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib
from .layout import ceil_div, pack_e2m1, swizzle_sf, swizzled_sf_numel


# ---- dtype tokens with the names the demo uses -------------------------------------------
class _DType:
    def __init__(self, name: str, width: int, torch_dtype=None):
        self.name, self.width, self.torch_dtype = name, width, torch_dtype

    def __repr__(self):
        return self.name


Float4E2M1FN = _DType("Float4E2M1FN", 4)
Float8E4M3FN = _DType("Float8E4M3FN", 8, torch.float8_e4m3fn)
Float8E5M2 = _DType("Float8E5M2", 8, torch.float8_e5m2)
Float8E8M0FNU = _DType("Float8E8M0FNU", 8)
Float16 = _DType("Float16", 16, torch.float16)
BFloat16 = _DType("BFloat16", 16, torch.bfloat16)
Float32 = _DType("Float32", 32, torch.float32)
_BY_NAME = {d.name: d for d in (Float4E2M1FN, Float8E4M3FN, Float8E5M2, Float8E8M0FNU, Float16, BFloat16, Float32)}
_C_CODES = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}


def _dtype_token(d) -> _DType:
    if isinstance(d, _DType):
        return d
    name = d if isinstance(d, str) else getattr(d, "name", getattr(d, "__name__", str(d)))
    if name not in _BY_NAME:
        raise ValueError(f"unknown dtype {d!r}")
    return _BY_NAME[name]


def _as_lmk(t: torch.Tensor, what: str) -> torch.Tensor:
    """Accept [R, C], [L, R, C] or the demo's (R, C, L) view with L slowest in memory;
    return a contiguous-in-memory [L, R, C] view without copying."""
    if t.dim() == 2:
        t = t.unsqueeze(0)
    elif t.dim() == 3 and not t.is_contiguous() and t.permute(2, 0, 1).is_contiguous():
        t = t.permute(2, 0, 1)
    if t.dim() != 3 or not t.is_contiguous():
        raise ValueError(f"{what} must be contiguous [rows, cols], [L, rows, cols] or an (rows, cols, L) view of it")
    return t


def gemm_workspace_bytes(m: int, n: int, k: int) -> int:
    """Bytes of f32 scratch with which an [m, k] x [n, k] problem runs split-K (0: it does not split)."""
    return int(_lib.lib.b200fp4_nvfp4_gemm_workspace_bytes(m, n, k))


def nvfp4_gemm(a: torch.Tensor, b: torch.Tensor, sfa: torch.Tensor, sfb: torch.Tensor,
               alpha: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
               out_dtype: torch.dtype = torch.bfloat16, tile_n: int = 0,
               workspace: Optional[torch.Tensor] = None, sf_vec_size: int = 16) -> torch.Tensor:
    """C = alpha * (A*SFA) @ (B*SFB)^T with f32 accumulation on the tensor cores.

    ``sf_vec_size`` 16: NVFP4 (one e4m3 scale byte per 16 K-elements); 32: MXFP4 (one ue8m0 scale byte per 32
    K-elements, same 128x4 tiles; single-CTA tile variants only).

    ``workspace=`` (uint8, ``gemm_workspace_bytes(m, n, k)`` bytes) opts a problem with few output tiles and a long
    reduction into split-K.  It is off by default: at M = 128, N = K = 8192 the split kernel takes the same 15 us as
    the unsplit 64-wide tiles and the reduction adds 4."""
    if not (a.is_cuda and b.is_cuda and sfa.is_cuda and sfb.is_cuda):
        raise ValueError("operands must be CUDA tensors (there is no CPU implementation)")
    a3, b3 = _as_lmk(a.view(torch.uint8), "a"), _as_lmk(b.view(torch.uint8), "b")
    l, m, kh = a3.shape
    lb, n, khb = b3.shape
    if lb != l or khb != kh:
        raise ValueError(f"a {tuple(a3.shape)} and b {tuple(b3.shape)} disagree on batch or K")
    k = kh * 2
    if k % 32 != 0 or n % 8 != 0:
        raise ValueError("Invalid tensor alignment")
    if sf_vec_size not in (16, 32):
        raise NotImplementedError("sf_vec_size must be 16 (NVFP4) or 32 (MXFP4)")
    need_a = l * swizzled_sf_numel(m, ceil_div(k, sf_vec_size))
    need_b = l * swizzled_sf_numel(n, ceil_div(k, sf_vec_size))
    if sfa.element_size() != 1 or sfb.element_size() != 1 or sfa.numel() < need_a or sfb.numel() < need_b:
        raise ValueError(f"scale factors must be 1-byte tensors in the 128x4 tiled layout "
                         f"({need_a} and {need_b} bytes)")
    if out is None:
        shape = (m, n) if a.dim() == 2 else (l, m, n)
        out = torch.empty(shape, dtype=out_dtype, device=a.device)
    out3 = _as_lmk(out, "c")
    if tuple(out3.shape) != (l, m, n) or out.dtype not in _C_CODES:
        raise ValueError(f"c must be [{m}, {n}] (x{l}) in float16, bfloat16 or float32")
    if alpha is not None and (alpha.dtype != torch.float32 or not alpha.is_cuda):
        raise ValueError("alpha must be a float32 CUDA tensor")
    if sf_vec_size == 32:
        with _lib.on_device(a.device):
            _lib.check(_lib.lib.b200fp4_mxfp4_gemm(
                a3.data_ptr(), b3.data_ptr(), sfa.data_ptr(), sfb.data_ptr(), out3.data_ptr(), _lib.ptr(alpha),
                m, n, k, l, _C_CODES[out.dtype], tile_n, _lib.current_stream_ptr(a.device)))
        return out
    ws_ptr, ws_bytes = None, 0
    if workspace is not None and tile_n == 0:
        ws_bytes = gemm_workspace_bytes(m, n, k)
        if ws_bytes:
            if not workspace.is_cuda or workspace.device != a.device or workspace.numel() * workspace.element_size() < ws_bytes:
                raise ValueError(f"workspace must be a CUDA tensor on {a.device} of at least {ws_bytes} bytes")
            ws_ptr = workspace.data_ptr()
    with _lib.on_device(a.device):
        _lib.check(_lib.lib.b200fp4_nvfp4_gemm_ws(
            a3.data_ptr(), b3.data_ptr(), sfa.data_ptr(), sfb.data_ptr(), out3.data_ptr(), _lib.ptr(alpha),
            m, n, k, l, _C_CODES[out.dtype], tile_n, ws_ptr, ws_bytes, _lib.current_stream_ptr(a.device)))
    return out


def mxfp8_gemm(a: torch.Tensor, b: torch.Tensor, sfa: torch.Tensor, sfb: torch.Tensor,
               alpha: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
               out_dtype: torch.dtype = torch.bfloat16, tile_n: int = 0) -> torch.Tensor:
    """MXFP8 flavour: A ``[M, K]`` and B ``[N, K]`` are ``torch.float8_e4m3fn`` or ``torch.float8_e5m2`` (each
    operand its own format), scale factors ue8m0 bytes, one per 32 K-elements, in the 128x4 tiled layout
    (``swizzled_sf_numel(rows, ceil(K / 32))`` bytes).  Same kernel family as ``nvfp4_gemm``; single-CTA tiles."""
    fmts = {torch.float8_e4m3fn: 0, torch.float8_e5m2: 1}
    if a.dtype not in fmts or b.dtype not in fmts:
        raise ValueError("a and b must be float8_e4m3fn or float8_e5m2 tensors")
    if not (a.is_cuda and b.is_cuda and sfa.is_cuda and sfb.is_cuda):
        raise ValueError("operands must be CUDA tensors (there is no CPU implementation)")
    a3, b3 = _as_lmk(a.view(torch.uint8), "a"), _as_lmk(b.view(torch.uint8), "b")
    l, m, k = a3.shape
    lb, n, kb_ = b3.shape
    if lb != l or kb_ != k:
        raise ValueError(f"a {tuple(a3.shape)} and b {tuple(b3.shape)} disagree on batch or K")
    if k % 16 != 0 or n % 8 != 0:
        raise ValueError("Invalid tensor alignment")
    need_a = l * swizzled_sf_numel(m, ceil_div(k, 32))
    need_b = l * swizzled_sf_numel(n, ceil_div(k, 32))
    if sfa.element_size() != 1 or sfb.element_size() != 1 or sfa.numel() < need_a or sfb.numel() < need_b:
        raise ValueError(f"scale factors must be 1-byte tensors in the 128x4 tiled layout ({need_a} and {need_b} bytes)")
    if out is None:
        out = torch.empty((m, n) if a.dim() == 2 else (l, m, n), dtype=out_dtype, device=a.device)
    out3 = _as_lmk(out, "c")
    if tuple(out3.shape) != (l, m, n) or out.dtype not in _C_CODES:
        raise ValueError(f"c must be [{m}, {n}] (x{l}) in float16, bfloat16 or float32")
    if alpha is not None and (alpha.dtype != torch.float32 or not alpha.is_cuda):
        raise ValueError("alpha must be a float32 CUDA tensor")
    with _lib.on_device(a.device):
        _lib.check(_lib.lib.b200fp4_mxfp8_gemm(
            a3.data_ptr(), b3.data_ptr(), sfa.data_ptr(), sfb.data_ptr(), out3.data_ptr(), _lib.ptr(alpha),
            m, n, k, l, _C_CODES[out.dtype], tile_n, fmts[a.dtype], fmts[b.dtype], _lib.current_stream_ptr(a.device)))
    return out


class Sm120BlockScaledGemmKernel:
    """Same constructor and call signature as the demo's kernel class.  Implemented: f32 accumulate, e2m1 operands
    with sf_vec_size 16 and e4m3 scale factors (NVFP4, the configuration the reference exercises) or sf_vec_size 32
    and ue8m0 scale factors (MXFP4), float8 operands with sf_vec_size 32 and ue8m0 scale factors (MXFP8; the operand
    flavour is taken from the tensors' dtype), K-major A and B, N-major C."""

    def __init__(self, acc_dtype, sf_vec_size: int, tile_shape_mnk: Tuple[int, int, int], epi_tile: Tuple[int, int]):
        if _dtype_token(acc_dtype) is not Float32:
            raise TypeError("Only Float32 accumulation is supported in FP4 mma")
        if sf_vec_size not in (16, 32):
            raise NotImplementedError("sf_vec_size must be 16 (NVFP4, e4m3 scales) or 32 (MXFP4, ue8m0 scales)")
        tm, tn, tk = tile_shape_mnk
        if tm % 128 or tn % 128 or tk % 64:
            raise ValueError("tile_shape_mnk must be multiples of (128, 128, 64)")
        self.acc_dtype, self.sf_vec_size = Float32, sf_vec_size
        self.tile_shape_mnk, self.epi_tile = tuple(tile_shape_mnk), tuple(epi_tile)
        # the hardware tile is 128 x {128,256} x 256; the requested N picks between the two
        self._tile_n = 256 if tn >= 256 else 0

    @staticmethod
    def is_valid_tensor_alignment(m, n, k, l, ab_dtype, c_dtype, a_major, b_major, c_major) -> bool:
        def ok(dtype, mode0_major, shape):
            return shape[0 if mode0_major else 1] % (16 * 8 // _dtype_token(dtype).width) == 0
        return (ok(ab_dtype, a_major == "m", (m, k, l)) and ok(ab_dtype, b_major == "n", (n, k, l))
                and ok(c_dtype, c_major == "m", (m, n, l)))

    def __call__(self, a, b, sfa, sfb, c, max_active_clusters=None, stream=None):
        if stream is not None and not isinstance(stream, torch.cuda.Stream):
            stream = torch.cuda.ExternalStream(int(stream))
        ctx = torch.cuda.stream(stream) if stream is not None else torch.cuda.stream(torch.cuda.current_stream())
        with ctx:
            if a.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):        # MXFP8: 8-bit operands
                if self.sf_vec_size != 32:
                    raise NotImplementedError("8-bit operands take ue8m0 scale factors per 32 elements")
                mxfp8_gemm(a, b, sfa, sfb, out=c, tile_n=self._tile_n)
            else:
                nvfp4_gemm(a, b, sfa, sfb, out=c, tile_n=self._tile_n, sf_vec_size=self.sf_vec_size)
        return c


Sm100BlockScaledGemmKernel = Sm120BlockScaledGemmKernel


def compile(gemm, a, b, sfa, sfb, c, max_active_clusters=None, stream=None):  # noqa: A001
    """Ahead-of-time kernels need no compilation; returns the callable of the demo's
    convention, ``compiled(a, b, sfa, sfb, c, stream)``."""
    def compiled(a, b, sfa, sfb, c, stream=None):
        return gemm(a, b, sfa, sfb, c, max_active_clusters, stream)
    return compiled


# ---- operand construction for run() ------------------------------------------------------
_E2M1_OF_INT = {-2: 0xC, -1: 0xA, 0: 0x0, 1: 0x2}      # value -> e2m1 code


def _integer_operand(rows: int, k: int, l: int, device, dtype: Optional[_DType] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Values in {-2,-1,0,1} (the demo's integer RANDOM init): returns ([L,rows,K/2] packed e2m1 or [L,rows,K]
    float8, [L,rows,K] f32)."""
    vals = torch.randint(-2, 2, (l, rows, k), device=device, dtype=torch.int32)
    if dtype is not None and dtype.width == 8:
        return vals.float().to(dtype.torch_dtype), vals.float()
    lut = torch.tensor([0xC, 0xA, 0x0, 0x2], dtype=torch.uint8, device=device)
    codes = lut[(vals + 2).long()]
    return pack_e2m1(codes), vals.float()


def _integer_scales(rows: int, k: int, l: int, device, sf_vec: int = 16) -> Tuple[torch.Tensor, torch.Tensor]:
    """Scale factors in {1, 2}: returns (tiled bytes [L, tiles*512], f32 per element [L, rows, K]).
    sf_vec 16: e4m3 bytes; 32: ue8m0 bytes (127 = 1, 128 = 2)."""
    blocks = ceil_div(k, sf_vec)
    sf = torch.randint(1, 3, (l, rows, blocks), device=device, dtype=torch.int32)
    if sf_vec == 16:
        bits = sf.float().to(torch.float8_e4m3fn).view(torch.uint8)
    else:
        bits = (sf + 126).to(torch.uint8)
    return swizzle_sf(bits), sf.float().repeat_interleave(sf_vec, dim=-1)[..., :k]


def run_bs(mnkl, a_dtype, b_dtype, sf_dtype, sf_vec_size, c_dtype, acc_dtype, a_major, b_major, c_major,
           tile_shape_mnk, epi_tile, tolerance, warmup_iterations, iterations, skip_ref_check,
           use_cold_l2=False, **kwargs) -> float:
    m, n, k, l = mnkl
    a_dtype, b_dtype, sf_dtype, c_dtype = (_dtype_token(d) for d in (a_dtype, b_dtype, sf_dtype, c_dtype))
    fp8 = (Float8E4M3FN, Float8E5M2)
    if not ((a_dtype, b_dtype, sf_dtype, sf_vec_size) in ((Float4E2M1FN, Float4E2M1FN, Float8E4M3FN, 16),
                                                          (Float4E2M1FN, Float4E2M1FN, Float8E8M0FNU, 32))
            or (a_dtype in fp8 and b_dtype in fp8 and (sf_dtype, sf_vec_size) == (Float8E8M0FNU, 32))):
        raise NotImplementedError("implemented: Float4E2M1FN x Float4E2M1FN with Float8E4M3FN scales per 16 (NVFP4) or "
                                  "Float8E8M0FNU scales per 32 (MXFP4), and Float8E4M3FN / Float8E5M2 operands with "
                                  "Float8E8M0FNU scales per 32 (MXFP8); mixed 4-bit x 8-bit operands are not")
    if (a_major, b_major, c_major) != ("k", "k", "n"):
        raise NotImplementedError("A and B must be K-major and C N-major")
    if c_dtype.torch_dtype not in _C_CODES:
        raise NotImplementedError(f"C dtype {c_dtype} is not implemented")
    if not Sm120BlockScaledGemmKernel.is_valid_tensor_alignment(m, n, k, l, a_dtype, c_dtype, a_major, b_major, c_major):
        raise ValueError("Invalid tensor alignment")
    if not torch.cuda.is_available():
        raise RuntimeError("GPU is required to run this example!")
    dev = torch.device("cuda")
    gemm = Sm120BlockScaledGemmKernel(acc_dtype, sf_vec_size, tile_shape_mnk, epi_tile)
    sets = max(1, min(10, iterations)) if use_cold_l2 else 1

    def make():
        a, a_ref = _integer_operand(m, k, l, dev, a_dtype)
        b, b_ref = _integer_operand(n, k, l, dev, b_dtype)
        sfa, sfa_ref = _integer_scales(m, k, l, dev, sf_vec_size)
        sfb, sfb_ref = _integer_scales(n, k, l, dev, sf_vec_size)
        c = torch.zeros(l, m, n, dtype=c_dtype.torch_dtype, device=dev)
        return (a, b, sfa, sfb, c), (a_ref, b_ref, sfa_ref, sfb_ref)

    work, refs = make()
    compiled = compile(gemm, *work, None, None)
    if not skip_ref_check:
        compiled(*work)
        torch.cuda.synchronize()
        _lib.raise_on_device_status()
        a_ref, b_ref, sfa_ref, sfb_ref = refs
        ref = torch.einsum("lmk,lnk->lmn", a_ref * sfa_ref, b_ref * sfb_ref)
        torch.testing.assert_close(work[4].float(), ref, atol=tolerance, rtol=1e-2)
    worksets = [work] + [make()[0] for _ in range(sets - 1)]
    for i in range(warmup_iterations):
        compiled(*worksets[i % sets])
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for i in range(iterations):
        compiled(*worksets[i % sets])
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) * 1e3 / max(1, iterations)


def run(mnkl, a_dtype, b_dtype, sf_dtype, sf_vec_size, c_dtype, a_major="k", b_major="k", c_major="n",
        tile_shape_mnk=(128, 128, 128), epi_tile=(128, 128), tolerance=1e-01, warmup_iterations=0, iterations=1,
        skip_ref_check=False, use_cold_l2=False, **kwargs) -> float:
    return run_bs(mnkl, a_dtype, b_dtype, sf_dtype, sf_vec_size, c_dtype, Float32, a_major, b_major, c_major,
                  tile_shape_mnk, epi_tile, tolerance, warmup_iterations, iterations, skip_ref_check, use_cold_l2)


_E2M1_MIDPOINTS = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)


def _quantize_rows(xf: torch.Tensor, gs: float):
    """[rows, K] f32 -> (codes uint8 [rows, K], scale bytes uint8 [rows, K/16]) with global scale gs."""
    rows, k = xf.shape
    blocks = xf.reshape(rows, k // 16, 16)
    sf = (blocks.abs().amax(-1) * gs / 6.0).clamp(max=448.0).to(torch.float8_e4m3fn)
    sfq = sf.float()
    scaled = torch.where(sfq[..., None] > 0, blocks * gs / sfq[..., None], torch.zeros_like(blocks))
    mids = torch.tensor(_E2M1_MIDPOINTS, device=xf.device)
    idx = torch.bucketize(scaled.abs(), mids).to(torch.uint8)          # number of midpoints strictly below |v|
    codes = (idx | (((scaled < 0) & (idx > 0)).to(torch.uint8) << 3)).reshape(rows, k)
    return codes, sf.view(torch.uint8)


def quantize_operand(x: torch.Tensor, global_scale: Optional[float] = None):
    """Host-side convenience used by examples and benchmarks: quantise an f32 [rows, K] matrix to
    NVFP4 with torch ops (amax-based e4m3 scale per 16 elements, nearest e2m1 code, ties to the smaller
    magnitude: the recipe of tests/python/test_flashinfer_norm_verbatim.py:58-68).  Returns
    (packed uint8 [rows, K/2], tiled scale bytes, global_scale).  Not on the hot path."""
    xf = x.float()
    gs = float(448.0 * 6.0 / xf.abs().max()) if global_scale is None else float(global_scale)
    codes, sf_bits = _quantize_rows(xf, gs)
    return pack_e2m1(codes), swizzle_sf(sf_bits), gs


def quantize_operand_batched(w: torch.Tensor):
    """[E, rows, K] -> (codes uint8 [E, rows, K], scale bytes uint8 [E, rows, K/16], global scales f32 [E]),
    every expert with its own global scale 448 * 6 / amax.  One expert at a time to bound the temporaries."""
    e, rows, k = w.shape
    codes = torch.empty(e, rows, k, dtype=torch.uint8, device=w.device)
    sf = torch.empty(e, rows, k // 16, dtype=torch.uint8, device=w.device)
    gs = torch.empty(e, dtype=torch.float32, device=w.device)
    for i in range(e):
        wf = w[i].float()
        g = float(448.0 * 6.0 / wf.abs().max().clamp_min(1e-30))
        codes[i], sf[i] = _quantize_rows(wf, g)
        gs[i] = g
    return codes, sf, gs


def mm_fp4(a: torch.Tensor, b: torch.Tensor, a_descale: torch.Tensor, b_descale: torch.Tensor,
           alpha: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16,
           out: Optional[torch.Tensor] = None, block_size: int = 16, use_8x4_sf_layout: bool = False,
           backend: str = "b200fp4") -> torch.Tensor:
    """flashinfer-style front door of the same kernel: ``out = alpha * (a * a_descale) @ (b * b_descale)``.

    ``a`` [m, k/2] packed e2m1 with its 128x4-tiled e4m3 block scales ``a_descale`` is exactly what
    ``rmsnorm_fp4quant`` / ``add_rmsnorm_fp4quant(..., is_sf_swizzled_layout=True)`` produce
    (tests/python/test_flashinfer_norm_verbatim.py:155-164), so the norm output feeds the GEMM
    (.../dense_blockscaled_gemm_persistent_cooperative.py:281-439) without a layout step.  ``b`` is the weight,
    either [n, k/2] row-major or, as flashinfer passes it, the [k/2, n] transposed view of that storage;
    ``b_descale`` likewise (tiled over [n, k/16]).  ``alpha`` = 1 / (global_scale_a * global_scale_b)."""
    if block_size != 16 or use_8x4_sf_layout:
        raise NotImplementedError("only NVFP4 (block_size=16) with the 128x4 scale layout is implemented")
    if out_dtype not in (torch.bfloat16, torch.float16, torch.float32):
        raise NotImplementedError(f"out_dtype {out_dtype}")
    bu = b.view(torch.uint8)
    if bu.dim() == 2 and not bu.is_contiguous() and bu.t().is_contiguous():
        bu = bu.t()
    sfb = b_descale
    if sfb.dim() == 2 and not sfb.is_contiguous() and sfb.t().is_contiguous():
        sfb = sfb.t()
    return nvfp4_gemm(a.view(torch.uint8), bu, a_descale.contiguous().view(torch.uint8), sfb.contiguous().view(torch.uint8),
                      alpha=alpha, out=out, out_dtype=out_dtype)
