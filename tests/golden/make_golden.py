#!/usr/bin/env python3
"""Pin the CPU oracle against the reference's own torch goldens and freeze fixtures.

Run in a container that has the reference tree mounted:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's acceptance-test modules by file path, feeds seeded
inputs to BOTH the reference's golden functions and ``oracle/nvfp4_oracle.py``,
asserts bit-equality, and writes the inputs + expected outputs to
``tests/golden/*.npz``.  The fixtures are what the CPU test-suite and the GPU
parity tests replay; the reference tree is not needed to run those.
"""
from __future__ import annotations

import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle import nvfp4_oracle as O  # noqa: E402


def _load(name, path):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _bits16(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().copy()


def _codes_of_values(vals: torch.Tensor) -> np.ndarray:
    """Reference goldens return grid VALUES; map them back to 4-bit codes with
    sign of zero dropped (the reference compares decoded values)."""
    v = vals.numpy()
    idx = np.searchsorted(O.E2M1_GRID, np.abs(v)).astype(np.uint8)
    assert np.array_equal(O.E2M1_GRID[idx], np.abs(v))
    return idx | (((v < 0) & (idx > 0)).astype(np.uint8) << 3)


def _sf_bits_of_values(sf: torch.Tensor) -> np.ndarray:
    return sf.to(torch.float8_e4m3fn).view(torch.uint8).numpy().copy()


def norm_cases(N):
    out = {}
    gs_fixed = (448 * 448 * 6.0) ** 0.5 / 448.0
    cases = []
    # the reference's own acceptance shapes: fp16, seed 42, fixed global scale
    for b, h in [(1, 128), (4, 128), (7, 256), (3, 512)]:
        cases.append((f"fp16_{b}x{h}", b, h, torch.float16, 42, gs_fixed, "randn"))
    # bf16 with weight = 1 + 0.1 N(0,1) and gs = 448*6/amax (benchmark configs)
    cases.append(("bf16_128x4096", 128, 4096, torch.bfloat16, 0, None, "ones"))
    cases.append(("bf16_8x7168", 8, 7168, torch.bfloat16, 0, None, "ones"))
    cases.append(("bf16_5x64", 5, 64, torch.bfloat16, 1, None, "ones"))
    cases.append(("fp16_33x2048", 33, 2048, torch.float16, 2, gs_fixed, "randn"))
    for name, b, h, dt, seed, gs, wkind in cases:
        torch.manual_seed(seed)
        x = torch.randn(b, h).to(dt)
        r = torch.randn(b, h).to(dt)
        w = torch.randn(h).to(dt) if wkind == "randn" else (1 + 0.1 * torch.randn(h)).to(dt)
        gs_r = gs if gs is not None else O.nvfp4_global_scale(O.rmsnorm_true(x, w, 1e-6))
        gs_a = gs if gs is not None else O.nvfp4_global_scale(
            O.rmsnorm_true((x.float() + r.float()).to(dt), w, 1e-6))
        # ---- reference goldens
        _, yq, sfq = N.ref_rmsnorm_fp4(x, w, 1e-6, gs_r)
        res_ref, _, yq_a, sfq_a = N.ref_add_rmsnorm_fp4(x, r, w, 1e-6, gs_a)
        # ---- oracle
        c, s = O.rmsnorm_fp4quant_ref(x, w, 1e-6, gs_r)
        res, ca, sa = O.add_rmsnorm_fp4quant_ref(x, r, w, 1e-6, gs_a)
        assert np.array_equal(c, _codes_of_values(yq)), name
        assert np.array_equal(s, _sf_bits_of_values(sfq)), name
        assert torch.equal(res, res_ref), name
        assert np.array_equal(ca, _codes_of_values(yq_a)), name
        assert np.array_equal(sa, _sf_bits_of_values(sfq_a)), name
        # decoders agree with the reference's decoders too
        assert np.array_equal(O.e2m1_decode(O.unpack_e2m1(O.pack_e2m1(c))),
                              N._fp4_dequant(torch.from_numpy(O.pack_e2m1(c))).numpy())
        assert np.array_equal(O.e4m3_decode(s), N._e4m3_bits_to_float(torch.from_numpy(s)).numpy())
        out[name] = dict(
            dtype=np.array(0 if dt == torch.float16 else 1), x=_bits16(x), r=_bits16(r), w=_bits16(w),
            gs_rms=np.float32(gs_r), gs_add=np.float32(gs_a), eps=np.float32(1e-6),
            rms_packed=O.pack_e2m1(c), rms_sf=s,
            add_res=_bits16(res), add_packed=O.pack_e2m1(ca), add_sf=sa)
        print("norm", name, "ok")
    return out


def quantiser_cases(N, M):
    torch.manual_seed(7)
    rows = []
    rows.append(torch.randn(8, 256) * 3)
    # exact midpoints and their float neighbours, both signs, with sf_q == 1 (amax 6, gs 1)
    mids = torch.tensor(O.E2M1_MIDPOINTS)
    near = torch.cat([mids, torch.nextafter(mids, torch.tensor(10.0)), torch.nextafter(mids, torch.tensor(-10.0))])
    blockvals = torch.cat([near, -near, torch.tensor([6.0, -6.0, 0.0, -0.0, 1e-30, -1e-30])])
    blocks = blockvals.reshape(-1, 1).repeat(1, 16)
    blocks[:, 0] = 6.0
    rows.append(blocks.reshape(-1, 256)[:3])
    rows.append(torch.randn(4, 256) * 1e-3)        # subnormal / zero scale factors
    rows.append(torch.randn(4, 256) * 1e4)         # clamped scale factors (saturating codes)
    rows.append(torch.zeros(2, 256))
    vals = torch.cat(rows).contiguous()
    res = {}
    for tag, gs in [("gs1", 1.0), ("gs2p449", (448 * 448 * 6.0) ** 0.5 / 448.0), ("gs600", 600.625)]:
        yq, sfq = N._quantize_nvfp4_reference(vals, gs)
        c, s = O.quantize_nvfp4(vals.numpy(), gs)
        assert np.array_equal(c, _codes_of_values(yq)), tag
        assert np.array_equal(s, _sf_bits_of_values(sfq)), tag
        packed_f, sf_f, deq_f = M._quantize_nvfp4_fast(vals, gs)
        cf, sfb = O.quantize_nvfp4(vals.numpy(), gs, implicit_one_packing=True)
        assert np.array_equal(O.pack_e2m1(cf), packed_f.numpy()), tag     # argmin codes: -0 never produced
        assert np.array_equal(sfb, sf_f.numpy()), tag
        assert np.array_equal(O.dequantize_nvfp4(cf, sfb, gs), deq_f.numpy()), tag
        res[f"{tag}_packed"] = O.pack_e2m1(c)
        res[f"{tag}_sf"] = s
        res[f"{tag}_fast_packed"] = O.pack_e2m1(cf)
        res[f"{tag}_fast_sf"] = sfb
        res[f"{tag}_gs"] = np.float32(gs)
        print("quantiser", tag, "ok")
    res["values"] = vals.numpy()
    # all 256 scale bytes through both decoders
    allb = np.arange(256, dtype=np.uint8)
    ok = (allb & 0x7F) != 0x7F
    assert np.array_equal(O.e4m3_decode(allb)[ok], N._e4m3_bits_to_float(torch.from_numpy(allb)).numpy()[ok])
    assert np.array_equal(O.e4m3_decode_implicit_one(allb & 0x7F),
                          M._fast_scale_decode(torch.from_numpy(allb & 0x7F)).numpy())
    # encoder against torch's cast on a dense sweep of [0, 448]
    sweep = torch.cat([torch.linspace(0, 448, 200001), torch.logspace(-12, 2.6, 50001)]).clamp(max=448.0)
    assert np.array_equal(O.e4m3_encode(sweep.numpy()), sweep.to(torch.float8_e4m3fn).view(torch.uint8).numpy())
    print("e4m3 encode/decode ok")
    return res


def layout_cases(M, ref_root):
    sys.path.insert(0, os.path.join(ref_root, "python"))
    sys.path.insert(0, os.path.join(ref_root, "python/cutlass_compat"))
    from cutlass.utils import blockscaled_layout
    from self_cutedsl.frontend.cute_objects import _flatten
    res = {}
    for rows, k in [(128, 128), (256, 256), (200, 320), (1536, 2048)]:
        kb = k // 16
        rng = np.random.default_rng(rows + k)
        logical = rng.integers(0, 127, size=(2, rows, kb), dtype=np.uint8)
        six = M._mma_scale_layout(torch.from_numpy(logical), rows, k, 2)
        # six-mode view (32,4,m_tiles,4,k_tiles,E) back to its storage order [E,m_tiles,k_tiles,32,4,4]
        storage = six.permute(5, 2, 4, 0, 1, 3).contiguous().view(torch.uint8).numpy().reshape(2, -1)
        assert np.array_equal(O.swizzle_sf(logical), storage), (rows, k)
        assert np.array_equal(O.unswizzle_sf(storage, rows, kb), logical)
        lay = blockscaled_layout.tile_atom_to_shape_SF((rows, k, 1), 16)
        shp, strd = tuple(_flatten(lay.shape)), tuple(_flatten(lay.stride))
        # (32,4,rm,4,rk,l) with the strides of the closed-form offset
        off = O.sf_swizzled_offsets(rows, kb)
        for m in (0, 1, 31, 32, 97, rows - 1):
            for b in (0, 1, 3, kb - 1):
                co = (m % 32, (m // 32) % 4, m // 128, b % 4, b // 4, 0)
                assert off[m, b] == sum(c * s for c, s in zip(co, strd)), (rows, k, m, b)
        if rows * k <= 256 * 320:       # the large case is checked here but not stored
            res[f"sf_{rows}x{k}_logical"] = logical
            res[f"sf_{rows}x{k}_swizzled"] = storage
        print("layout", rows, k, shp, strd, "ok")
    return res


def moe_cases(M):
    res = {}
    # --- random-weight case of the reference (its loop, run on the CPU)
    torch.manual_seed(123)
    tokens, experts, hidden, inter = 64, 2, 256, 128
    x = (torch.randn(tokens, hidden) * 0.2).to(torch.bfloat16)
    w1s = (torch.randn(experts, 2 * inter, hidden) * 0.15).to(torch.bfloat16)
    w2s = (torch.randn(experts, hidden, inter) * 0.15).to(torch.bfloat16)
    w1p, w1sc, w1dq = M._quantize_nvfp4_fast(w1s)
    w2p, w2sc, w2dq = M._quantize_nvfp4_fast(w2s)
    ids = (torch.arange(tokens, dtype=torch.int32) % experts)[:, None]
    routes = torch.ones(tokens, 1)
    _, _, xdq = M._quantize_nvfp4_fast(x)
    ref = torch.empty(tokens, hidden)
    for t in range(tokens):
        e = int(ids[t, 0])
        fc1 = xdq[t] @ w1dq[e].T
        up, gate = fc1[:inter], fc1[inter:]
        act = (torch.nn.functional.silu(gate) * up).to(torch.bfloat16).float()
        _, _, adq = M._quantize_nvfp4_fast(act[None, :])
        ref[t] = adq[0] @ w2dq[e].T
    got = O.moe_ref(x, O.unpack_e2m1(w1p.numpy()), w1sc.numpy(), O.unpack_e2m1(w2p.numpy()), w2sc.numpy(),
                    ids, routes)
    # same math, but batched matmuls may sum in another order: compare after the bf16 rounding
    diff = (got.float() - ref.to(torch.bfloat16).float()).abs()
    ulp_ok = diff <= ref.abs() * 2.0 ** -7 + 1e-6
    print("moe random: max diff", diff.max().item(), "mismatching", int((diff > 0).sum()))
    assert bool(ulp_ok.all()) and float((diff > 0).float().mean()) < 0.02
    res.update(rand_x=_bits16(x), rand_w1=w1p.numpy(), rand_w1_sf=w1sc.numpy(), rand_w2=w2p.numpy(),
               rand_w2_sf=w2sc.numpy(), rand_ids=ids.numpy(), rand_routes=routes.numpy(),
               rand_ref_f32=ref.numpy(), rand_oracle=_bits16(got))
    # --- exact uniform-routing construction of the reference
    lut = torch.tensor(M._E2M1_VALUES)
    hidden, inter, experts = 256, 128, 2
    codes = torch.tensor([0x11, 0x22], dtype=torch.uint8)
    scale = torch.full((experts,), 0.015625)
    x1 = torch.full((1, hidden), 0.1, dtype=torch.bfloat16)
    _, _, xdq = M._quantize_nvfp4_fast(x1)
    expected = []
    for e in range(experts):
        wv = lut[(codes[e] & 0xF).long()] * scale[e]
        fc1 = (xdq[0] * wv).sum()
        act = (torch.nn.functional.silu(fc1) * fc1).to(torch.bfloat16).float()
        _, _, adq = M._quantize_nvfp4_fast(act.expand(1, inter))
        expected.append((adq[0] * wv).sum().to(torch.bfloat16))
    expected = torch.stack(expected)
    for tokens in (8, 64, 256, 641):
        xt = torch.full((tokens, hidden), 0.1, dtype=torch.bfloat16)
        idt = (torch.arange(tokens, dtype=torch.int32) % experts)[:, None]
        w1c = np.broadcast_to(np.array([1, 2], np.uint8)[:, None, None], (experts, 2 * inter, hidden)).copy()
        w2c = np.broadcast_to(np.array([1, 2], np.uint8)[:, None, None], (experts, hidden, inter)).copy()
        sfb = O.e4m3_encode(np.float32(0.015625))
        got = O.moe_ref(xt, w1c, np.full((experts, 2 * inter, hidden // 16), sfb, np.uint8),
                        w2c, np.full((experts, hidden, inter // 16), sfb, np.uint8), idt, torch.ones(tokens, 1))
        assert torch.equal(got, expected[idt[:, 0].long(), None].expand_as(got)), tokens
    assert not torch.equal(expected[0], expected[1])
    res["uniform_expected"] = _bits16(expected)
    print("moe uniform exact ok", expected.tolist())
    return res


def gemm_cases():
    """The demo's check (COOP:1791-1793): scale each operand element-wise, then a
    f32 einsum.  Integer-valued data make it exact, so equality is required."""
    res = {}
    for m, n, k in [(128, 128, 128), (128, 128, 256), (256, 384, 512)]:
        ac, sfa, bc, sfb = O.integer_gemm_operands(m, n, k, seed=m + n + k)
        a_ref = torch.from_numpy(O.e2m1_decode(ac))
        b_ref = torch.from_numpy(O.e2m1_decode(bc))
        sfa_ref = torch.from_numpy(np.repeat(O.e4m3_decode(sfa), 16, axis=-1))
        sfb_ref = torch.from_numpy(np.repeat(O.e4m3_decode(sfb), 16, axis=-1))
        ref = torch.einsum("mk,nk->mn", torch.einsum("mk,mk->mk", a_ref, sfa_ref),
                           torch.einsum("nk,nk->nk", b_ref, sfb_ref))
        got = O.gemm_nvfp4_ref(ac, sfa, bc, sfb)
        assert torch.equal(ref, got)
        res[f"int_{m}x{n}x{k}_c"] = got.numpy()
        print("gemm", m, n, k, "ok")
    return res


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <path to a checkout of the reference repository>")
    ref_root = sys.argv[1]
    N = _load("ref_normtest", os.path.join(ref_root, "tests/python/test_flashinfer_norm_verbatim.py"))
    M = _load("ref_moetest", os.path.join(ref_root, "tests/python/test_flashinfer_b12x_verbatim.py"))
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    for name, case in norm_cases(N).items():
        np.savez_compressed(os.path.join(HERE, f"norm_{name}.npz"), **case)
    np.savez_compressed(os.path.join(HERE, "quantiser.npz"), **quantiser_cases(N, M))
    np.savez_compressed(os.path.join(HERE, "sf_layout.npz"), **layout_cases(M, ref_root))
    np.savez_compressed(os.path.join(HERE, "moe.npz"), **moe_cases(M))
    np.savez_compressed(os.path.join(HERE, "gemm.npz"), **gemm_cases())
    print("all fixtures written to", HERE)


if __name__ == "__main__":
    main()
