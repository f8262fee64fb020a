"""Host-side logic that needs no GPU: the module-name shim, argument / device checks that must raise before any
kernel is launched, and the checkpoint-side weight packer (checked against the oracle's quantiser and layout)."""
import importlib
import sys

import numpy as np
import pytest
import torch

from oracle import nvfp4_oracle as O


def test_shim_registers_and_removes_the_reference_module_names(b200):
    shim = b200.compat_shim
    names = ["flashinfer.cute_dsl.rmsnorm_fp4quant", "flashinfer.cute_dsl.add_rmsnorm_fp4quant",
             "flashinfer.fused_moe.cute_dsl.b12x_moe", "dense_blockscaled_gemm_persistent_cooperative"]
    before = {n: sys.modules.get(n) for n in names + ["flashinfer"]}
    assert not shim.installed()                       # nothing is shadowed without an explicit install()
    shim.install()
    try:
        assert shim.installed()
        # the reference's loader calls (tests/python/support/flashinfer_verbatim.py:101-108,111-162)
        assert shim.load_operator("rmsnorm_fp4quant").rmsnorm_fp4quant is b200.rmsnorm_fp4quant
        assert shim.load_operator("add_rmsnorm_fp4quant").add_rmsnorm_fp4quant is b200.add_rmsnorm_fp4quant
        assert shim.load_b12x_operator().b12x_fused_moe is b200.b12x_fused_moe
        assert shim.ensure_loaded() is sys.modules["flashinfer.cute_dsl"]
        # plain imports by module path resolve too
        m = importlib.import_module("flashinfer.cute_dsl.rmsnorm_fp4quant")
        assert m.rmsnorm_fp4quant is b200.rmsnorm_fp4quant
        from flashinfer.fused_moe.cute_dsl.b12x_moe import B12xMoEWrapper, b12x_fused_moe
        assert b12x_fused_moe is b200.b12x_fused_moe and B12xMoEWrapper is b200.B12xMoEWrapper
        bs = importlib.import_module("dense_blockscaled_gemm_persistent_cooperative")
        assert bs.run is b200.gemm.run and bs.Sm120BlockScaledGemmKernel is b200.Sm120BlockScaledGemmKernel
        with pytest.raises(ImportError):
            shim.load_operator("layernorm")
        shim.install()                                # idempotent
    finally:
        shim.uninstall()
    assert not shim.installed()
    for n, old in before.items():
        assert sys.modules.get(n) is old


def _cpu_moe_args(experts=2, hidden=256, inter=128, tokens=4, top_k=1):
    w1 = torch.zeros(experts, 2 * inter, hidden // 2, dtype=torch.uint8)
    w2 = torch.zeros(experts, hidden, inter // 2, dtype=torch.uint8)
    s1 = torch.zeros(experts, (2 * inter // 128) * (hidden // 64) * 512, dtype=torch.uint8)
    s2 = torch.zeros(experts, (hidden // 128) * (inter // 64) * 512, dtype=torch.uint8)
    x = torch.zeros(tokens, hidden, dtype=torch.bfloat16)
    ids = torch.zeros(tokens, top_k, dtype=torch.int32)
    w = torch.ones(tokens, top_k)
    return x, w1, s1, w2, s2, ids, w


def test_operators_refuse_cpu_tensors_before_any_launch(b200):
    """No CPU fallback and no pointer of a CPU tensor ever reaches a kernel."""
    x, w1, s1, w2, s2, ids, w = _cpu_moe_args()
    with pytest.raises(ValueError):
        b200.b12x_fused_moe(x, w1, s1, w2, s2, ids, w, 2, 1)
    with pytest.raises(ValueError):
        b200.rmsnorm_fp4quant(torch.zeros(4, 128, dtype=torch.bfloat16), torch.ones(128, dtype=torch.bfloat16))
    with pytest.raises(ValueError):
        b200.nvfp4_gemm(torch.zeros(128, 64, dtype=torch.uint8), torch.zeros(128, 64, dtype=torch.uint8),
                        torch.zeros(512, dtype=torch.uint8), torch.zeros(512, dtype=torch.uint8))
    with pytest.raises(ValueError):
        b200.topk_route(torch.zeros(4, 8), 2)


def test_moe_device_check_names_the_offending_argument(b200):
    from cutedsl_fully_opensourced_b200.moe import _on_device
    dev = torch.device("cuda", 0)
    with pytest.raises(ValueError, match="token_selected_experts"):
        _on_device(dev, token_selected_experts=torch.zeros(2, 2, dtype=torch.int32))
    with pytest.raises(ValueError, match="w1_alpha"):
        _on_device(dev, x=None, w1_alpha=torch.ones(2))
    _on_device(dev, fc2_input_scale=None)            # optional tensors may be absent


def test_pack_moe_weights_matches_the_oracle_quantiser_and_layout(b200):
    torch.manual_seed(0)
    e, inter, hidden = 3, 128, 256
    w1 = 0.02 * torch.randn(e, 2 * inter, hidden)
    w2 = 0.02 * torch.randn(e, hidden, inter)
    packed = b200.pack_moe_weights(w1, w2, fc2_input_scale=2.0)
    for name, w, extra in (("w1", w1, 1.0), ("w2", w2, 2.0)):
        for i in range(e):
            gs = float(448.0 * 6.0 / w[i].abs().max())
            codes, sf = O.quantize_nvfp4(w[i].numpy(), gs)
            assert np.array_equal(packed[f"{name}_weight"][i].numpy(), O.pack_e2m1(codes))
            storage = b200.layout.six_mode_to_storage(packed[f"{name}_weight_sf"])[i].numpy()
            assert np.array_equal(storage, O.swizzle_sf(sf))
            assert abs(float(packed[f"{name}_alpha"][i]) * gs * extra - 1.0) < 1e-6
    assert tuple(packed["w1_weight_sf"].shape) == (32, 4, 2, 4, 4, e)
    with pytest.raises(ValueError):
        b200.pack_moe_weights(w1, w2[:2])


def test_mm_fp4_refuses_other_block_formats(b200):
    z = torch.zeros(1, dtype=torch.uint8)
    with pytest.raises(NotImplementedError):
        b200.mm_fp4(z, z, z, z, block_size=32)
    with pytest.raises(NotImplementedError):
        b200.mm_fp4(z, z, z, z, use_8x4_sf_layout=True)
