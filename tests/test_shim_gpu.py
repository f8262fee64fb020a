"""The reference's own acceptance logic, run through the names that its loader resolves: the operators are
looked up with compat_shim's ``load_operator`` / ``load_b12x_operator`` / ``import
dense_blockscaled_gemm_persistent_cooperative`` exactly as tests/python/test_flashinfer_norm_verbatim.py:120-173,
tests/python/test_flashinfer_b12x_verbatim.py:99-165 and tests/python/test_blockscaled_verbatim.py:23-42 do, and
checked against the oracle (codes and scale bytes exact, residual exact, MoE bit-exact)."""
import importlib

import numpy as np
import pytest
import torch

from oracle import nvfp4_oracle as O
from conftest import golden

pytestmark = pytest.mark.gpu


@pytest.fixture()
def shim(b200):
    b200.compat_shim.install()
    yield b200.compat_shim
    b200.compat_shim.uninstall()


@pytest.mark.parametrize("B,H", [(1, 128), (4, 128), (7, 256), (3, 512)])
def test_norm_cases_of_the_reference_through_the_loader(shim, B, H):
    torch.manual_seed(42)
    x = torch.randn(B, H, device="cuda", dtype=torch.float16)
    residual = torch.randn(B, H, device="cuda", dtype=torch.float16)
    w = torch.randn(H, device="cuda", dtype=torch.float16)
    gs = (448 * 448 * 6.0) ** 0.5 / 448.0
    gs_t = torch.tensor([gs], device="cuda", dtype=torch.float32)
    y = torch.empty(B, H // 2, device="cuda", dtype=torch.uint8)
    s = torch.empty(B, H // 16, device="cuda", dtype=torch.uint8)
    ops = shim.load_operator("rmsnorm_fp4quant")
    ops.rmsnorm_fp4quant(x, w, y, s, global_scale=gs_t, eps=1e-6, block_size=16)
    torch.cuda.synchronize()
    codes, sf = O.rmsnorm_fp4quant_ref(x.cpu(), w.cpu(), 1e-6, float(np.float32(gs)))
    assert np.array_equal(y.cpu().numpy(), O.pack_e2m1(codes)) and np.array_equal(s.cpu().numpy(), sf)
    ops = shim.load_operator("add_rmsnorm_fp4quant")
    res = residual.clone()
    ops.add_rmsnorm_fp4quant(x, res, w, y, s, global_scale=gs_t, eps=1e-6, block_size=16)
    torch.cuda.synchronize()
    res_ref, codes, sf = O.add_rmsnorm_fp4quant_ref(x.cpu(), residual.cpu(), w.cpu(), 1e-6, float(np.float32(gs)))
    assert torch.equal(res.cpu(), res_ref)
    assert np.array_equal(y.cpu().numpy(), O.pack_e2m1(codes)) and np.array_equal(s.cpu().numpy(), sf)


@pytest.mark.parametrize("tokens", [8, 641])
def test_moe_uniform_routing_of_the_reference_through_the_loader(shim, tokens):
    from test_moe_gpu import six_mode
    b12x_ops = shim.load_b12x_operator()
    expected = torch.from_numpy(golden("moe.npz")["uniform_expected"].copy()).view(torch.bfloat16)
    experts, hidden, inter = 2, 256, 128
    x = torch.full((tokens, hidden), 0.1, dtype=torch.bfloat16, device="cuda")
    w1 = torch.from_numpy(O.pack_e2m1(np.broadcast_to(np.array([1, 2], np.uint8)[:, None, None],
                                                       (experts, 2 * inter, hidden)).copy())).cuda()
    w2 = torch.from_numpy(O.pack_e2m1(np.broadcast_to(np.array([1, 2], np.uint8)[:, None, None],
                                                       (experts, hidden, inter)).copy())).cuda()
    sfb = O.e4m3_encode(np.float32(0.015625))
    s1 = six_mode(np.full((experts, 2 * inter, hidden // 16), sfb, np.uint8))
    s2 = six_mode(np.full((experts, hidden, inter // 16), sfb, np.uint8))
    ids = (torch.arange(tokens, dtype=torch.int32, device="cuda") % experts)[:, None].contiguous()
    routes = torch.ones(tokens, 1, device="cuda")
    alpha = torch.ones(experts, device="cuda")
    out = b12x_ops.b12x_fused_moe(x, w1, s1, w2, s2, ids, routes, experts, 1, w1_alpha=alpha, w2_alpha=alpha,
                                  fc2_input_scale=torch.ones(1, device="cuda"), quant_mode="nvfp4")
    torch.cuda.synchronize()
    assert torch.equal(out.cpu(), expected[ids[:, 0].cpu().long(), None].expand(tokens, hidden))


def test_gemm_demo_by_its_module_name(shim):
    bs = importlib.import_module("dense_blockscaled_gemm_persistent_cooperative")
    torch.manual_seed(0)
    us = bs.run((1024, 1024, 1024, 1), "Float4E2M1FN", "Float4E2M1FN", "Float8E4M3FN", 16, "Float16", a_major="k",
                b_major="k", c_major="n", tile_shape_mnk=(128, 128, 128), epi_tile=(128, 128), tolerance=0.1,
                warmup_iterations=0, iterations=1, skip_ref_check=False)
    assert us > 0
