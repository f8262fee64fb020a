"""ctypes binding of libb200fp4.so, the C-ABI in ``include/b200fp4.h``.

There is deliberately no fallback: if the library has not been built the import
fails, and every failing C call is turned into a Python exception carrying the
library's own message.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "lib", "libb200fp4.so")

OK, INVALID_ARGUMENT, UNSUPPORTED, CUDA_ERROR, DEVICE_TIMEOUT, NOT_INITIALISED = range(6)

_vp, _i32, _i64, _f32, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t

# name -> (restype, argtypes); kept in the order of include/b200fp4.h
SIGNATURES = {
    "b200fp4_last_error": (C.c_char_p, []),
    "b200fp4_version": (_i32, []),
    "b200fp4_rmsnorm_fp4quant": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _f32, _i64, _i32, _i64, _i32, _i32, _vp]),
    "b200fp4_add_rmsnorm_fp4quant": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _f32, _i64, _i32, _i64, _i64,
                                            _i32, _i32, _vp]),
    "b200fp4_nvfp4_gemm": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp]),
    "b200fp4_topk_route": (_i32, [_vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp]),
    "b200fp4_moe_workspace_bytes": (_sz, [_i64, _i32, _i32, _i32, _i32]),
    "b200fp4_moe_fused": (_i32, [_vp] * 11 + [_i64, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _sz, _vp]),
    "b200fp4_moe_fused_noalloc": (_i32, [_vp] * 11 + [_i64, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _vp]),
    "b200fp4_moe_ep_buffer_bytes": (_sz, [_i64, _i32, _i32, _i32, _i32, _i32]),
    "b200fp4_moe_ep_stage": (_i32, [_vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _i32, _vp]),
    "b200fp4_moe_ep_compute": (_i32, [_vp, _i32, _i32] + [_vp] * 7 + [_i64, _i32, _i32, _i32, _i32, _vp]),
    "b200fp4_moe_ep_combine": (_i32, [_vp, _i32, _i32, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _vp]),
    "b200fp4_device_status": (_i32, [_vp, C.POINTER(C.c_int), _i32]),
}


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python {os.path.join(_PKG, 'build.py')}` "
            "(needs nvcc; there is no CPU or JIT fallback)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError here = header and library out of sync
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


class B200Fp4Error(RuntimeError):
    pass


def check(rc: int) -> None:
    """Raise the Python exception that matches a non-zero status code."""
    if rc == OK:
        return
    msg = (lib.b200fp4_last_error() or b"").decode("utf-8", "replace")
    if rc == INVALID_ARGUMENT:
        raise ValueError(msg)
    if rc == UNSUPPORTED:
        raise NotImplementedError(msg)
    raise B200Fp4Error(f"libb200fp4 status {rc}: {msg}")


def device_status(clear: bool = True, device=None) -> int:
    """Synchronise the current stream and return the device status word (0 = healthy)."""
    out = C.c_int(0)
    check(lib.b200fp4_device_status(current_stream_ptr(device), C.byref(out), 1 if clear else 0))
    return out.value


def raise_on_device_status(device=None) -> None:
    st = device_status(True, device)
    if st:
        what = []
        if st & 7:
            what.append("a device-side wait expired")
        if st & 8:
            what.append("a fused-MoE call with at most 32 tokens named one expert more than 32 times")
        raise B200Fp4Error(f"{'; '.join(what) or 'device error'} (status bits {st:#x}); results are invalid")


def ptr(t) -> int:
    """Device pointer of a torch tensor (or of anything with data_ptr()); None -> NULL."""
    return None if t is None else t.data_ptr()


def current_stream_ptr(device=None) -> int:
    import torch

    return torch.cuda.current_stream(device).cuda_stream
