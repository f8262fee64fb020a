"""B200 (sm_100a) implementation of the NVFP4 quantized-inference hot path:
fused RMSNorm / add-RMSNorm + NVFP4 quantisation, the NVFP4 block-scaled GEMM
and the fused NVFP4 MoE, behind the Python call signatures of the operators
the reference runs.  All compute is in ``lib/libb200fp4.so`` (hand-written
CUDA, built by ``build.py``); importing this package loads that library and
fails if it is absent.
"""
from . import _lib, layout  # noqa: F401
from . import gemm  # noqa: F401
from .gemm import (Sm100BlockScaledGemmKernel, Sm120BlockScaledGemmKernel, mm_fp4, mxfp8_gemm, nvfp4_gemm)  # noqa: F401
from . import moe, parallel  # noqa: F401
from .moe import B12xMoEWrapper, b12x_fused_moe, pack_moe_weights, topk_route  # noqa: F401
from .norm import add_rmsnorm_fp4quant, rmsnorm_fp4quant  # noqa: F401
from . import compat_shim  # noqa: F401
from ._lib import B200Fp4Error, synchronize  # noqa: F401

__all__ = ["rmsnorm_fp4quant", "add_rmsnorm_fp4quant", "nvfp4_gemm", "mxfp8_gemm", "mm_fp4", "b12x_fused_moe", "B12xMoEWrapper",
           "pack_moe_weights", "topk_route", "moe", "Sm120BlockScaledGemmKernel", "Sm100BlockScaledGemmKernel", "gemm",
           "layout", "parallel", "compat_shim", "synchronize", "B200Fp4Error"]
