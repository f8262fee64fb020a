"""The CPU oracle replayed against the frozen outputs of the reference's own
torch goldens (fixtures written by tests/golden/make_golden.py)."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import nvfp4_oracle as O
from conftest import GOLDEN, golden


def _t16(bits, dtype_code):
    dt = torch.float16 if int(dtype_code) == 0 else torch.bfloat16
    return torch.from_numpy(bits.copy()).view(dt)


NORM_FILES = sorted(os.path.basename(p) for p in glob.glob(os.path.join(GOLDEN, "norm_*.npz")))


def test_fixture_inventory():
    assert len(NORM_FILES) >= 8
    for name in ("quantiser.npz", "sf_layout.npz", "moe.npz", "gemm.npz"):
        assert os.path.exists(os.path.join(GOLDEN, name))


@pytest.mark.parametrize("fname", NORM_FILES)
def test_rmsnorm_oracle_matches_reference_golden(fname):
    g = golden(fname)
    x, w = _t16(g["x"], g["dtype"]), _t16(g["w"], g["dtype"])
    codes, sf = O.rmsnorm_fp4quant_ref(x, w, float(g["eps"]), float(g["gs_rms"]))
    assert np.array_equal(O.pack_e2m1(codes), g["rms_packed"])
    assert np.array_equal(sf, g["rms_sf"])


@pytest.mark.parametrize("fname", NORM_FILES)
def test_add_rmsnorm_oracle_matches_reference_golden(fname):
    g = golden(fname)
    x, r, w = (_t16(g[k], g["dtype"]) for k in ("x", "r", "w"))
    res, codes, sf = O.add_rmsnorm_fp4quant_ref(x, r, w, float(g["eps"]), float(g["gs_add"]))
    assert np.array_equal(res.view(torch.int16).numpy(), g["add_res"])
    assert np.array_equal(O.pack_e2m1(codes), g["add_packed"])
    assert np.array_equal(sf, g["add_sf"])


@pytest.mark.parametrize("tag", ["gs1", "gs2p449", "gs600"])
def test_quantiser_matches_reference_golden(tag):
    g = golden("quantiser.npz")
    c, s = O.quantize_nvfp4(g["values"], float(g[f"{tag}_gs"]))
    assert np.array_equal(O.pack_e2m1(c), g[f"{tag}_packed"])
    assert np.array_equal(s, g[f"{tag}_sf"])
    cf, sf = O.quantize_nvfp4(g["values"], float(g[f"{tag}_gs"]), implicit_one_packing=True)
    assert np.array_equal(O.pack_e2m1(cf), g[f"{tag}_fast_packed"])
    assert np.array_equal(sf, g[f"{tag}_fast_sf"])


def test_midpoints_take_the_smaller_magnitude_and_zero_is_positive():
    mids = O.E2M1_MIDPOINTS
    assert np.array_equal(O.e2m1_nearest_codes(mids), np.arange(7, dtype=np.uint8))
    assert np.array_equal(O.e2m1_nearest_codes(-mids), np.array([0, 9, 10, 11, 12, 13, 14], np.uint8))
    up = np.nextafter(mids, np.float32(10))
    assert np.array_equal(O.e2m1_nearest_codes(up), np.arange(1, 8, dtype=np.uint8))
    assert O.e2m1_nearest_codes(np.float32(-0.1)) == 0
    assert O.e2m1_nearest_codes(np.float32(7.5)) == 7 and O.e2m1_nearest_codes(np.float32(-1e9)) == 15


def test_e4m3_roundtrip_all_codes_and_torch_cast():
    codes = np.arange(0, 0x7F, dtype=np.uint8)          # 0 .. 448
    assert np.array_equal(O.e4m3_encode(O.e4m3_decode(codes)), codes)
    sweep = torch.cat([torch.linspace(0, 448, 50001), torch.logspace(-12, 2.6, 20001)]).clamp(max=448.0)
    assert np.array_equal(O.e4m3_encode(sweep.numpy()), sweep.to(torch.float8_e4m3fn).view(torch.uint8).numpy())
    assert O.e4m3_decode(np.uint8(1)) == np.float32(2.0 ** -9)
    assert O.e4m3_decode_implicit_one(np.uint8(1)) == np.float32(2.0 ** -7 * 1.125)


def test_sf_layout_matches_reference_storage():
    g = golden("sf_layout.npz")
    keys = [k[:-8] for k in g.files if k.endswith("_logical")]
    assert keys
    for k in keys:
        logical, swz = g[k + "_logical"], g[k + "_swizzled"]
        assert np.array_equal(O.swizzle_sf(logical), swz)
        assert np.array_equal(O.unswizzle_sf(swz, *logical.shape[-2:]), logical)
    # layout facts pinned by the reference's host-only tests:
    # tile_atom_to_shape_SF((128,128,1),16) has strides (16,4,1024,1,512,1024)
    off = O.sf_swizzled_offsets(128, 8)
    for m in range(128):
        for kg in range(8):
            assert off[m, kg] == (m % 32) * 16 + (m // 32) * 4 + (kg % 4) + (kg // 4) * 512


def test_torch_side_layout_helpers_agree_with_oracle():
    from cutedsl_fully_opensourced_b200 import layout

    rng = np.random.default_rng(0)
    logical = rng.integers(0, 255, size=(3, 200, 20), dtype=np.uint8)
    swz = layout.swizzle_sf(torch.from_numpy(logical)).numpy()
    assert np.array_equal(swz, O.swizzle_sf(logical))
    assert np.array_equal(layout.unswizzle_sf(torch.from_numpy(swz), 200, 20).numpy(), logical)
    six = torch.from_numpy(swz).view(3, 2, 5, 32, 4, 4).permute(3, 4, 1, 5, 2, 0)
    assert np.array_equal(layout.six_mode_to_storage(six).numpy(), swz)
    codes = rng.integers(0, 16, size=(4, 64), dtype=np.uint8)
    assert np.array_equal(layout.pack_e2m1(torch.from_numpy(codes)).numpy(), O.pack_e2m1(codes))
    assert np.array_equal(layout.unpack_e2m1(torch.from_numpy(O.pack_e2m1(codes))).numpy(), codes)


def test_gemm_oracle_exact_on_integer_data():
    g = golden("gemm.npz")
    for m, n, k in [(128, 128, 128), (128, 128, 256), (256, 384, 512)]:
        ac, sfa, bc, sfb = O.integer_gemm_operands(m, n, k, seed=m + n + k)
        assert np.array_equal(O.gemm_nvfp4_ref(ac, sfa, bc, sfb).numpy(), g[f"int_{m}x{n}x{k}_c"])


def test_moe_oracle_matches_reference_cases():
    g = golden("moe.npz")
    x = torch.from_numpy(g["rand_x"].copy()).view(torch.bfloat16)
    got = O.moe_ref(x, O.unpack_e2m1(g["rand_w1"]), g["rand_w1_sf"], O.unpack_e2m1(g["rand_w2"]),
                    g["rand_w2_sf"], torch.from_numpy(g["rand_ids"]), torch.from_numpy(g["rand_routes"]))
    assert np.array_equal(got.view(torch.int16).numpy(), g["rand_oracle"])
    # the reference's acceptance statistics, against its own per-token loop output
    ref = torch.from_numpy(g["rand_ref_f32"])
    diff = (got.float() - ref).abs()
    assert diff.mean() <= 0.02
    assert torch.linalg.vector_norm(diff) / torch.linalg.vector_norm(ref) <= 0.10
    # uniform routing: bit-exact expected values per expert
    exp = torch.from_numpy(g["uniform_expected"].copy()).view(torch.bfloat16)
    tokens, hidden, inter = 9, 256, 128
    sfb = O.e4m3_encode(np.float32(0.015625))
    w1c = np.broadcast_to(np.array([1, 2], np.uint8)[:, None, None], (2, 2 * inter, hidden)).copy()
    w2c = np.broadcast_to(np.array([1, 2], np.uint8)[:, None, None], (2, hidden, inter)).copy()
    ids = (torch.arange(tokens, dtype=torch.int32) % 2)[:, None]
    out = O.moe_ref(torch.full((tokens, hidden), 0.1, dtype=torch.bfloat16), w1c,
                    np.full((2, 2 * inter, hidden // 16), sfb, np.uint8), w2c,
                    np.full((2, hidden, inter // 16), sfb, np.uint8), ids, torch.ones(tokens, 1))
    assert torch.equal(out, exp[ids[:, 0].long(), None].expand_as(out))


def test_route_topk_properties():
    torch.manual_seed(0)
    logits = torch.randn(37, 128)
    ids, w = O.route_topk_ref(logits, 8)
    assert ids.shape == (37, 8) and w.shape == (37, 8)
    assert torch.allclose(w.sum(-1), torch.ones(37), atol=1e-6)
    assert bool((w[:, :-1] >= w[:, 1:]).all())
    top = torch.topk(logits, 8, dim=-1).indices
    assert torch.equal(ids.long().sort(-1).values, top.sort(-1).values)
