"""Module-name shim: makes this package answer to the import names under which the reference finds its operators.

The reference never imports its hot-path operators from a package of its own: its tests and benches resolve them
by MODULE PATH through a loader (tests/python/support/flashinfer_verbatim.py:49-108 ``ensure_loaded`` /
``load_operator``, :111-162 ``load_b12x_operator``) and import the GEMM demo by its file name
(tests/python/test_blockscaled_verbatim.py:23,35).  ``install()`` registers the same names in ``sys.modules``,
pointing at this package's functions:

    flashinfer.cute_dsl.rmsnorm_fp4quant          .rmsnorm_fp4quant
    flashinfer.cute_dsl.add_rmsnorm_fp4quant      .add_rmsnorm_fp4quant
    flashinfer.fused_moe.cute_dsl.b12x_moe        .b12x_fused_moe, .B12xMoEWrapper
    dense_blockscaled_gemm_persistent_cooperative .run, .run_bs, .Sm120BlockScaledGemmKernel, ...

so ``ops = load_operator("rmsnorm_fp4quant"); ops.rmsnorm_fp4quant(...)`` and
``import dense_blockscaled_gemm_persistent_cooperative as bs; bs.run(...)`` run the B200 kernels with the call
sites unchanged.  Nothing is registered at import time: an installed ``flashinfer`` is only shadowed after an
explicit ``install()``, and ``uninstall()`` puts back whatever was there before.
"""
from __future__ import annotations

import sys
import types
from typing import Dict, Optional

from . import gemm as _gemm
from . import moe as _moe
from . import norm as _norm

GEMM_DEMO_MODULE = "dense_blockscaled_gemm_persistent_cooperative"
_OPERATOR_MODULES = {
    "flashinfer.cute_dsl.rmsnorm_fp4quant": {"rmsnorm_fp4quant": _norm.rmsnorm_fp4quant},
    "flashinfer.cute_dsl.add_rmsnorm_fp4quant": {"add_rmsnorm_fp4quant": _norm.add_rmsnorm_fp4quant},
    "flashinfer.fused_moe.cute_dsl.b12x_moe": {"b12x_fused_moe": _moe.b12x_fused_moe,
                                              "B12xMoEWrapper": _moe.B12xMoEWrapper},
}
_PACKAGES = ("flashinfer", "flashinfer.cute_dsl", "flashinfer.fused_moe", "flashinfer.fused_moe.cute_dsl")

_MISSING = object()
_saved: Optional[Dict[str, object]] = None        # what sys.modules held under our names before install()
_saved_attrs = []                                 # (parent module, attribute, previous value) set on foreign parents


def _is_ours(mod) -> bool:
    return getattr(mod, "__b200fp4_shim__", False)


def _new_module(name: str, package: bool) -> types.ModuleType:
    mod = types.ModuleType(name)
    mod.__b200fp4_shim__ = True
    mod.__doc__ = f"b200fp4 stand-in for {name} (see cutedsl_fully_opensourced_b200.compat_shim)"
    if package:
        mod.__path__ = []                          # a namespace with no files behind it
    return mod


def installed() -> bool:
    return _saved is not None


def install() -> None:
    """Register the operator module names (idempotent).  Parent packages that already exist (an imported real
    flashinfer) are kept and only get the operator sub-modules attached; missing ones are created as empty
    packages."""
    global _saved
    if _saved is not None:
        return
    _saved = {}
    for name in _PACKAGES:
        if name not in sys.modules:
            _saved[name] = _MISSING
            sys.modules[name] = _new_module(name, package=True)
    for name in _PACKAGES[1:]:
        parent, _, leaf = name.rpartition(".")
        _set_attr(sys.modules[parent], leaf, sys.modules[name])
    for name, members in _OPERATOR_MODULES.items():
        _saved[name] = sys.modules.get(name, _MISSING)
        mod = _new_module(name, package=False)
        for attr, value in members.items():
            setattr(mod, attr, value)
        sys.modules[name] = mod
        parent, _, leaf = name.rpartition(".")
        _set_attr(sys.modules[parent], leaf, mod)
    _saved[GEMM_DEMO_MODULE] = sys.modules.get(GEMM_DEMO_MODULE, _MISSING)
    sys.modules[GEMM_DEMO_MODULE] = _gemm


def _set_attr(parent, leaf, value) -> None:
    _saved_attrs.append((parent, leaf, getattr(parent, leaf, _MISSING)))
    setattr(parent, leaf, value)


def uninstall() -> None:
    """Undo ``install()``: every name goes back to what ``sys.modules`` held before."""
    global _saved
    if _saved is None:
        return
    for parent, leaf, old in reversed(_saved_attrs):
        if old is _MISSING:
            if hasattr(parent, leaf):
                delattr(parent, leaf)
        else:
            setattr(parent, leaf, old)
    _saved_attrs.clear()
    for name, old in _saved.items():
        if old is _MISSING:
            sys.modules.pop(name, None)
        else:
            sys.modules[name] = old
    _saved = None


# ---- the loader API of tests/python/support/flashinfer_verbatim.py, same names and return values -----------------
def ensure_loaded() -> types.ModuleType:
    """Returns the ``flashinfer.cute_dsl`` package (flashinfer_verbatim.py:49-98)."""
    install()
    return sys.modules["flashinfer.cute_dsl"]


def load_operator(module_name: str) -> types.ModuleType:
    """``load_operator("rmsnorm_fp4quant").rmsnorm_fp4quant(...)`` (flashinfer_verbatim.py:101-108)."""
    install()
    full = f"flashinfer.cute_dsl.{module_name}"
    if full not in sys.modules or not _is_ours(sys.modules[full]):
        raise ImportError(f"{full} is not provided by this package (operators: rmsnorm_fp4quant, add_rmsnorm_fp4quant)")
    return sys.modules[full]


def load_b12x_operator() -> types.ModuleType:
    """Returns the ``flashinfer.fused_moe.cute_dsl.b12x_moe`` module (flashinfer_verbatim.py:111-162)."""
    install()
    return sys.modules["flashinfer.fused_moe.cute_dsl.b12x_moe"]
