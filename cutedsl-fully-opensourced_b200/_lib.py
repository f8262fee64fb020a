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

_vp, _i32, _i64, _f32, _f64, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_double, C.c_size_t

# name -> (restype, argtypes); kept in the order of include/b200fp4.h
SIGNATURES = {
    "b200fp4_last_error": (C.c_char_p, []),
    "b200fp4_version": (_i32, []),
    "b200fp4_rmsnorm_fp4quant": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _f32, _i64, _i32, _i64, _i32, _i32, _vp]),
    "b200fp4_add_rmsnorm_fp4quant": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _f32, _i64, _i32, _i64, _i64,
                                            _i32, _i32, _vp]),
    "b200fp4_nvfp4_gemm": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp]),
    "b200fp4_nvfp4_gemm_workspace_bytes": (_sz, [_i32, _i32, _i32]),
    "b200fp4_nvfp4_gemm_ws": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _sz, _vp]),
    "b200fp4_mxfp4_gemm": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp]),
    "b200fp4_mxfp8_gemm": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _vp]),
    "b200fp4_topk_route": (_i32, [_vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp]),
    "b200fp4_moe_workspace_bytes": (_sz, [_i64, _i32, _i32, _i32, _i32]),
    "b200fp4_moe_fused": (_i32, [_vp] * 11 + [_i64, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _sz, _vp]),
    "b200fp4_moe_fused_routed": (_i32, [_vp, _vp, _i32, _i32] + [_vp] * 10 + [_i64, _i32, _i32, _i32, _i32, _i32, _i32, _i32,
                                               _vp, _sz, _vp]),
    "b200fp4_moe_fused_noalloc": (_i32, [_vp] * 11 + [_i64, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _vp]),
    "b200fp4_moe_ep_buffer_bytes": (_sz, [_i64, _i32, _i32, _i32, _i32, _i32]),
    "b200fp4_moe_ep_reset": (_i32, [_vp, _i64, _i32, _i32, _i32, _i32, _i32, _vp]),
    "b200fp4_moe_ep_dispatch": (_i32, [_vp, _vp, _vp, _vp, _i32, _vp, _i32, _i32, _i64, _i32, _i32, _i32, _i32, _i32, _f64, _vp]),
    "b200fp4_moe_ep_dispatch_count": (_i32, [_vp, _vp, _vp, _vp, _i32, _vp, _i32, _i32, _i64, _i32, _i32, _i32, _i32, _i32, _f64, _vp]),
    "b200fp4_moe_ep_dispatch_place": (_i32, [_vp, _vp, _vp, _vp, _i32, _vp, _i32, _i32, _i64, _i32, _i32, _i32, _i32, _i32, _f64, _vp]),
    "b200fp4_moe_ep_compute": (_i32, [_vp, _i32, _i32] + [_vp] * 7 + [_i64, _i32, _i32, _i32, _i32, _i32, _f64, _vp]),
    "b200fp4_moe_ep_combine": (_i32, [_vp, _i32, _i32, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _i32, _f64, _vp]),
    "b200fp4_moe_ep_routing": (_i32, [_vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _i32, _vp]),
    "b200fp4_selftest_peer_wait": (_i32, [_vp, _i32, _f64, _i64, _i32, _i32, _i32, _i32, _vp]),
    "b200fp4_selftest_bounded_wait": (_i32, [C.c_longlong, _vp, _vp]),
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


STATUS_GEMM_WAIT = 7          # bits 1 | 2 | 4: producer / MMA / epilogue wait of a GEMM kernel expired
STATUS_ROWS_EXCEED_TILE = 8
STATUS_PEER_WAIT = 16         # a wait for another rank of an expert-parallel group expired


def describe_status(st: int) -> str:
    what = []
    if st & STATUS_GEMM_WAIT:
        what.append("a wait inside a GEMM kernel expired")
    if st & STATUS_ROWS_EXCEED_TILE:
        what.append("a few-row GEMM launch met a row block with more rows than it loads")
    if st & STATUS_PEER_WAIT:
        what.append("a wait for another rank of the expert-parallel group expired (a peer is late or gone)")
    return "; ".join(what) or "unknown device error"


def raise_on_device_status(device=None) -> None:
    """The sync point of the error contract: synchronise the current stream, read and clear the device status
    word, and raise if a kernel reported trouble since the last check (kernels never trap; they record and
    return)."""
    st = device_status(True, device)
    if st:
        raise B200Fp4Error(f"{describe_status(st)} (status bits {st:#x}); results since the last check are invalid")


def synchronize(device=None) -> None:
    """``torch.cuda.synchronize`` for users of this package: waits for the current stream and raises
    ``B200Fp4Error`` if any kernel of the library reported an expired wait."""
    raise_on_device_status(device)


class _NoGuard:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NO_GUARD = _NoGuard()


def on_device(device):
    """Context that makes ``device`` current for the C call inside it; free when it already is (switching devices
    through torch costs several microseconds, more than the launch of a small kernel)."""
    import torch

    if device.index is None or torch.cuda.current_device() == device.index:
        return _NO_GUARD
    return torch.cuda.device(device)


def ptr(t) -> int:
    """Device pointer of a torch tensor (or of anything with data_ptr()); None -> NULL."""
    return None if t is None else t.data_ptr()


def current_stream_ptr(device=None) -> int:
    import torch

    return torch.cuda.current_stream(device).cuda_stream
