"""The C-ABI library loads without a GPU and exports every function that
include/b200fp4.h declares (no compute is launched here)."""
import ctypes
import os
import re

from conftest import ROOT


def _declared():
    text = open(os.path.join(ROOT, "include", "b200fp4.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200fp4_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(lib_built):
    names = _declared()
    assert "b200fp4_rmsnorm_fp4quant" in names and "b200fp4_add_rmsnorm_fp4quant" in names
    lib = ctypes.CDLL(lib_built)
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/b200fp4.h but not exported"


def test_python_binding_covers_header(b200):
    assert sorted(b200._lib.SIGNATURES) == _declared()


def test_version_and_error_string(b200):
    assert b200._lib.lib.b200fp4_version() >= 1
    assert isinstance(b200._lib.lib.b200fp4_last_error(), bytes)


def test_argument_errors_surface_before_any_launch(b200):
    # null pointers are rejected by the library itself, no device needed
    rc = b200._lib.lib.b200fp4_rmsnorm_fp4quant(None, None, None, None, None, None, 1e-6, 4, 128, 128, 1, 0, None)
    assert rc == b200._lib.INVALID_ARGUMENT
    assert b"null" in b200._lib.lib.b200fp4_last_error()
    import pytest
    with pytest.raises(ValueError):
        b200._lib.check(rc)


def test_cpu_tensors_are_refused(b200):
    import pytest
    import torch
    x = torch.randn(4, 128, dtype=torch.bfloat16)
    w = torch.ones(128, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        b200.rmsnorm_fp4quant(x, w)
    with pytest.raises(ValueError):
        b200.add_rmsnorm_fp4quant(x, x.clone(), w)
