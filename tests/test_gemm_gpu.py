"""GPU parity of the NVFP4 block-scaled GEMM (through the C-ABI).

* integer-valued operands (values in {-2..1}, scale factors in {1,2}, the
  reference demo's own test data): every partial sum is exact in f32, so the
  result must EQUAL the f32 product of the de-quantised operands after the
  rounding to the output type;
* arbitrary codes and scale factors: f32 accumulation order differs from the
  CPU's, tolerance rel-L2 <= 1e-5 (the stated bar for N(0,1) operands against
  the de-quantised f32 reference is rel-L2 <= 1e-2).
"""
import numpy as np
import pytest
import torch

from oracle import nvfp4_oracle as O

pytestmark = pytest.mark.gpu


def _dev_operands(ac, sfa, bc, sfb):
    a = torch.from_numpy(O.pack_e2m1(ac)).cuda()
    b = torch.from_numpy(O.pack_e2m1(bc)).cuda()
    sa = torch.from_numpy(O.swizzle_sf(sfa)).cuda()
    sb = torch.from_numpy(O.swizzle_sf(sfb)).cuda()
    return a, b, sa, sb


def _check_status(b200):
    assert b200._lib.device_status() == 0, "a device-side wait expired"


@pytest.mark.parametrize("m,n,k,tile_n", [
    (128, 128, 128, 128), (128, 128, 256, 128), (128, 256, 256, 256), (256, 384, 512, 128),
    (256, 512, 1024, 256), (1024, 1024, 1024, 0), (256, 256, 64, 512), (512, 768, 1024, 512), (128, 128, 128, 512), (128, 192, 512, 64), (256, 64, 128, 64),
])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_integer_operands_exact(b200, m, n, k, tile_n, out_dtype):
    ac, sfa, bc, sfb = O.integer_gemm_operands(m, n, k, seed=m + n + k)
    ref = O.gemm_nvfp4_ref(ac, sfa, bc, sfb)
    a, b, sa, sb = _dev_operands(ac, sfa, bc, sfb)
    c = b200.nvfp4_gemm(a, b, sa, sb, out_dtype=out_dtype, tile_n=tile_n)
    torch.cuda.synchronize()
    _check_status(b200)
    assert torch.equal(c.cpu().float(), ref.to(out_dtype).float())


@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (200, 264, 96), (130, 8, 32), (1, 136, 416), (333, 520, 1280)])
@pytest.mark.parametrize("tile_n", [64, 128, 256, 512])
def test_ragged_shapes_random_codes(b200, m, n, k, tile_n):
    rng = np.random.default_rng(m * 7 + n * 3 + k)
    ac = rng.integers(0, 16, size=(m, k), dtype=np.uint8)
    bc = rng.integers(0, 16, size=(n, k), dtype=np.uint8)
    sfa = rng.integers(0x20, 0x48, size=(m, k // 16), dtype=np.uint8)      # e4m3 2^-3 .. 4
    sfb = rng.integers(0x20, 0x48, size=(n, k // 16), dtype=np.uint8)
    ref = O.gemm_nvfp4_ref(ac, sfa, bc, sfb, alpha=0.375)
    a, b, sa, sb = _dev_operands(ac, sfa, bc, sfb)
    alpha = torch.tensor([0.375], device="cuda")
    c = b200.nvfp4_gemm(a, b, sa, sb, alpha=alpha, out_dtype=torch.float32, tile_n=tile_n)
    torch.cuda.synchronize()
    _check_status(b200)
    err = torch.linalg.vector_norm(c.cpu() - ref) / torch.linalg.vector_norm(ref)
    assert err <= 1e-5, float(err)


def test_quantised_normal_operands_against_f32_reference(b200):
    """A, B ~ N(0,1) quantised with the golden quantiser; rel-L2 of the GEMM against the f32
    product of the de-quantised operands must be <= 1e-2 (it is ~1e-6: same numbers, other order)."""
    torch.manual_seed(0)
    m, n, k = 256, 384, 2048
    A, B = torch.randn(m, k), torch.randn(n, k)
    gsa, gsb = O.nvfp4_global_scale(A), O.nvfp4_global_scale(B)
    ac, sfa = O.quantize_nvfp4(A.numpy(), gsa)
    bc, sfb = O.quantize_nvfp4(B.numpy(), gsb)
    alpha = 1.0 / (gsa * gsb)
    ref = O.gemm_nvfp4_ref(ac, sfa, bc, sfb, alpha=alpha)
    a, b, sa, sb = _dev_operands(ac, sfa, bc, sfb)
    c = b200.nvfp4_gemm(a, b, sa, sb, alpha=torch.tensor([alpha], device="cuda"), out_dtype=torch.bfloat16)
    torch.cuda.synchronize()
    _check_status(b200)
    err = torch.linalg.vector_norm(c.cpu().float() - ref) / torch.linalg.vector_norm(ref)
    assert err <= 1e-2, float(err)
    assert err <= 4e-3      # bf16 output rounding alone is ~2e-3
    # and it is a faithful quantised product of the true matrices
    true = A @ B.t()
    assert torch.linalg.vector_norm(c.cpu().float() - true) / torch.linalg.vector_norm(true) < 0.2


def test_batched_and_demo_views(b200):
    ac, sfa, bc, sfb = O.integer_gemm_operands(256, 128, 256, seed=5)
    ac2, sfa2, bc2, sfb2 = O.integer_gemm_operands(256, 128, 256, seed=6)
    a = torch.from_numpy(np.stack([O.pack_e2m1(ac), O.pack_e2m1(ac2)])).cuda()
    b = torch.from_numpy(np.stack([O.pack_e2m1(bc), O.pack_e2m1(bc2)])).cuda()
    sa = torch.from_numpy(np.stack([O.swizzle_sf(sfa), O.swizzle_sf(sfa2)])).cuda()
    sb = torch.from_numpy(np.stack([O.swizzle_sf(sfb), O.swizzle_sf(sfb2)])).cuda()
    c = torch.zeros(2, 256, 128, dtype=torch.float32, device="cuda")
    # the demo hands over (m, k, l) views with l slowest in memory
    kern = b200.Sm120BlockScaledGemmKernel(b200.gemm.Float32, 16, (128, 128, 128), (128, 128))
    compiled = b200.gemm.compile(kern, a.permute(1, 2, 0), b.permute(1, 2, 0), sa, sb, c.permute(1, 2, 0), 148, None)
    compiled(a.permute(1, 2, 0), b.permute(1, 2, 0), sa, sb, c.permute(1, 2, 0), None)
    torch.cuda.synchronize()
    _check_status(b200)
    assert torch.equal(c[0].cpu(), O.gemm_nvfp4_ref(ac, sfa, bc, sfb))
    assert torch.equal(c[1].cpu(), O.gemm_nvfp4_ref(ac2, sfa2, bc2, sfb2))


@pytest.mark.parametrize("mnkl", [(128, 128, 128, 1), (1024, 1024, 1024, 1), (128, 128, 256, 1)])
def test_demo_run_entry_point(b200, mnkl):
    """The reference's acceptance test calls run(...) with these arguments
    (tests/python/test_blockscaled_verbatim.py:32-42); it checks itself and returns microseconds."""
    torch.manual_seed(0)
    g = b200.gemm
    us = g.run(mnkl, g.Float4E2M1FN, g.Float4E2M1FN, g.Float8E4M3FN, 16, g.Float16, a_major="k", b_major="k",
               c_major="n", tile_shape_mnk=(128, 128, 128), epi_tile=(128, 128), tolerance=0.1,
               warmup_iterations=0, iterations=1, skip_ref_check=False)
    assert us > 0


def test_alignment_and_argument_errors(b200):
    g = b200.gemm
    with pytest.raises(ValueError, match="Invalid tensor alignment"):
        g.run((128, 128, 48, 1), g.Float4E2M1FN, g.Float4E2M1FN, g.Float8E4M3FN, 16, g.Float16)
    with pytest.raises(ValueError, match="Invalid tensor alignment"):
        g.run((128, 100, 128, 1), g.Float4E2M1FN, g.Float4E2M1FN, g.Float8E4M3FN, 16, g.Float16)
    with pytest.raises(NotImplementedError):
        g.run((128, 128, 128, 1), g.Float4E2M1FN, g.Float8E4M3FN, g.Float8E8M0FNU, 32, g.Float16)      # mixed 4 x 8 bit
    with pytest.raises(NotImplementedError):
        g.run((128, 128, 128, 1), g.Float8E4M3FN, g.Float8E4M3FN, g.Float8E4M3FN, 16, g.Float16)
    a = torch.zeros(128, 64, dtype=torch.uint8, device="cuda")
    sf = torch.zeros(512, dtype=torch.uint8, device="cuda")
    with pytest.raises(ValueError):
        b200.nvfp4_gemm(a, a, sf[:100], sf)


def test_large_square_integer_exact(b200):
    """4096^3 and the benchmark's 8192^3 with integer data: compared on the GPU against torch's f32
    matmul of the de-quantised operands (exact for these values), bf16 output."""
    from cutedsl_fully_opensourced_b200.layout import unpack_e2m1, unswizzle_sf
    for size, tile_n in [(4096, 0), (8192, 256), (8192, 128), (8192, 512)]:
        torch.manual_seed(size)
        a, a_ref = b200.gemm._integer_operand(size, size, 1, "cuda")
        b, b_ref = b200.gemm._integer_operand(size, size, 1, "cuda")
        sa, sa_ref = b200.gemm._integer_scales(size, size, 1, "cuda")
        sb, sb_ref = b200.gemm._integer_scales(size, size, 1, "cuda")
        c = b200.nvfp4_gemm(a[0], b[0], sa[0], sb[0], out_dtype=torch.bfloat16, tile_n=tile_n)
        torch.cuda.synchronize()
        _check_status(b200)
        torch.backends.cuda.matmul.allow_tf32 = False
        ref = ((a_ref[0] * sa_ref[0]) @ (b_ref[0] * sb_ref[0]).t()).to(torch.bfloat16)
        assert torch.equal(c, ref), f"{size}: {(c != ref).float().mean().item():.3e} of outputs differ"
        del a, b, sa, sb, a_ref, b_ref, sa_ref, sb_ref, c, ref


def test_benchmark_config_data_small_m_sweep(b200):
    """The benchmark's GEMM configuration with its stated data at the small ends of the M sweep: A, B ~ N(0,1)
    quantised by the golden quantiser with per-tensor global scales, alpha = 1 / (gs_A * gs_B), bf16 output,
    N = K = 8192, M in {1024, 128}, through every tile variant that the automatic choice can take there.
    Golden: dequantise-then-f32-product (.../dense_blockscaled_gemm_persistent_cooperative.py:1791-1806)."""
    torch.manual_seed(0)
    n = k = 8192
    A, B = torch.randn(1024, k), torch.randn(n, k)
    gsa, gsb = O.nvfp4_global_scale(A), O.nvfp4_global_scale(B)
    ac, sfa = O.quantize_nvfp4(A.numpy(), gsa)
    bc, sfb = O.quantize_nvfp4(B.numpy(), gsb)
    alpha = 1.0 / (gsa * gsb)
    ref = O.gemm_nvfp4_ref(ac, sfa, bc, sfb, alpha=alpha)
    alpha_d = torch.tensor([alpha], device="cuda")
    for m, tiles in ((1024, (0, 512, 256, 128)), (128, (0, 64, 128, 256))):
        a, b, sa, sb = _dev_operands(ac[:m], sfa[:m], bc, sfb)
        for tile_n in tiles:
            c = b200.nvfp4_gemm(a, b, sa, sb, alpha=alpha_d, out_dtype=torch.bfloat16, tile_n=tile_n)
            torch.cuda.synchronize()
            _check_status(b200)
            err = torch.linalg.vector_norm(c.cpu().float() - ref[:m]) / torch.linalg.vector_norm(ref[:m])
            assert err <= 1e-2 and err <= 4e-3, (m, tile_n, float(err))


def test_norm_quant_output_feeds_the_gemm(b200):
    """add_rmsnorm_fp4quant(..., is_sf_swizzled_layout=True) -> its y_fp4 / block_scale are the GEMM's A / SFA
    with no layout step in between (K = 7168, ragged row count), through nvfp4_gemm and the mm_fp4 front door;
    compared with the same chain on the CPU oracle (tests/python/test_flashinfer_norm_verbatim.py:155-164 feeding
    .../dense_blockscaled_gemm_persistent_cooperative.py:281-439)."""
    torch.manual_seed(1)
    rows, hidden, n = 200, 7168, 384
    x = torch.randn(rows, hidden).to(torch.bfloat16)
    r = torch.randn(rows, hidden).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(hidden)).to(torch.bfloat16)
    W = 0.05 * torch.randn(n, hidden)
    gs_x = O.nvfp4_global_scale(O.rmsnorm_true((x.float() + r.float()).to(torch.bfloat16), w, 1e-6))
    gs_w = O.nvfp4_global_scale(W)
    _, ac, sfa = O.add_rmsnorm_fp4quant_ref(x, r, w, 1e-6, gs_x)
    bc, sfb = O.quantize_nvfp4(W.numpy(), gs_w)
    alpha = 1.0 / (gs_x * gs_w)
    ref = O.gemm_nvfp4_ref(ac, sfa, bc, sfb, alpha=alpha)
    y, sf = b200.add_rmsnorm_fp4quant(x.cuda(), r.cuda(), w.cuda(), global_scale=torch.tensor([gs_x], device="cuda"),
                                      eps=1e-6, is_sf_swizzled_layout=True)
    b = torch.from_numpy(O.pack_e2m1(bc)).cuda()
    sb = torch.from_numpy(O.swizzle_sf(sfb)).cuda()
    alpha_d = torch.tensor([alpha], device="cuda")
    c = b200.nvfp4_gemm(y, b, sf, sb, alpha=alpha_d, out_dtype=torch.bfloat16)
    # flashinfer's calling convention: the weight and its scales as transposed views
    c2 = b200.mm_fp4(y, b.t(), sf, sb.view(torch.float8_e4m3fn), alpha_d, torch.bfloat16)
    torch.cuda.synchronize()
    _check_status(b200)
    assert torch.equal(c, c2)
    err = torch.linalg.vector_norm(c.cpu().float() - ref) / torch.linalg.vector_norm(ref)
    assert err <= 1e-2, float(err)
    # the plain variant's tiled scale output is an operand of the same kind
    y3, sf3 = b200.rmsnorm_fp4quant(x.cuda(), w.cuda(), global_scale=torch.tensor([gs_x], device="cuda"),
                                    is_sf_swizzled_layout=True)
    c3 = b200.mm_fp4(y3, b.t(), sf3, sb, alpha_d, torch.float32)
    ac3, sfa3 = O.rmsnorm_fp4quant_ref(x, w, 1e-6, gs_x)
    ref3 = O.gemm_nvfp4_ref(ac3, sfa3, bc, sfb, alpha=alpha)
    torch.cuda.synchronize()
    assert torch.linalg.vector_norm(c3.cpu() - ref3) / torch.linalg.vector_norm(ref3) <= 1e-2


def test_bounded_wait_gives_up_and_the_next_launch_is_healthy(b200):
    """The GEMM kernels' bounded wait, exercised on an mbarrier on which nothing ever arrives, with a limit of
    about a millisecond: the kernel returns, the status bit is set, and the next GEMM runs normally."""
    lib, check = b200._lib.lib, b200._lib.check
    b200._lib.device_status()
    gave_up = torch.zeros(1, dtype=torch.int32, device="cuda")
    check(lib.b200fp4_selftest_bounded_wait(1_000_000, gave_up.data_ptr(), torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert int(gave_up.item()) == 1
    with pytest.raises(b200.B200Fp4Error, match="wait inside a GEMM kernel expired"):
        b200.synchronize()
    ac, sfa, bc, sfb = O.integer_gemm_operands(256, 256, 512, seed=1)
    a, b, sa, sb = _dev_operands(ac, sfa, bc, sfb)
    c = b200.nvfp4_gemm(a, b, sa, sb, out_dtype=torch.float32)
    b200.synchronize()
    assert torch.equal(c.cpu(), O.gemm_nvfp4_ref(ac, sfa, bc, sfb))


def test_two_devices_in_one_process(b200):
    """Launch configuration (shared-memory opt-in, SM count) is kept per device."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ac, sfa, bc, sfb = O.integer_gemm_operands(256, 512, 1024, seed=2)
    ref = O.gemm_nvfp4_ref(ac, sfa, bc, sfb)
    for dev in ("cuda:0", "cuda:1"):
        ops = [torch.from_numpy(t).to(dev) for t in (O.pack_e2m1(ac), O.pack_e2m1(bc), O.swizzle_sf(sfa), O.swizzle_sf(sfb))]
        for tile_n in (128, 256, 512):
            c = b200.nvfp4_gemm(*ops, out_dtype=torch.float32, tile_n=tile_n)
            torch.cuda.synchronize(dev)
            assert torch.equal(c.cpu(), ref)


@pytest.mark.parametrize("m,n,k", [(128, 1024, 4096), (200, 520, 2304), (64, 256, 8192)])
def test_split_k_integer_exact(b200, m, n, k):
    """Few output tiles and a long reduction: with a workspace the K tiles of every output tile are dealt to several
    CTAs (split-K, f32 partial matrices in the workspace, summed in slice order).  Integer-valued operands must still
    give the exact product, equal to the unsplit kernels'."""
    assert b200.gemm.gemm_workspace_bytes(m, n, k) > 0, "this shape is expected to split"
    ac, sfa, bc, sfb = O.integer_gemm_operands(m, n, k, seed=m + n + k)
    ref = O.gemm_nvfp4_ref(ac, sfa, bc, sfb, alpha=0.5)
    a, b, sa, sb = _dev_operands(ac, sfa, bc, sfb)
    alpha = torch.tensor([0.5], device="cuda")
    for out_dtype in (torch.float32, torch.bfloat16):
        ws = torch.empty(b200.gemm.gemm_workspace_bytes(m, n, k), dtype=torch.uint8, device="cuda")
        c = b200.nvfp4_gemm(a, b, sa, sb, alpha=alpha, out_dtype=out_dtype, workspace=ws)
        c2 = b200.nvfp4_gemm(a, b, sa, sb, alpha=alpha, out_dtype=out_dtype)            # unsplit default
        unsplit = b200.nvfp4_gemm(a, b, sa, sb, alpha=alpha, out_dtype=out_dtype, tile_n=256)
        torch.cuda.synchronize()
        _check_status(b200)
        assert torch.equal(c.cpu().float(), ref.to(out_dtype).float())
        assert torch.equal(c, c2) and torch.equal(c, unsplit)
    with pytest.raises(ValueError):
        b200.nvfp4_gemm(a, b, sa, sb, workspace=torch.empty(16, dtype=torch.uint8, device="cuda"))


@pytest.mark.parametrize("m,n,k,tile_n", [(128, 128, 128, 128), (256, 384, 512, 0), (200, 264, 1184, 256), (128, 192, 4096, 64),
                                          (1024, 1024, 1024, 0)])
def test_mxfp4_block32_ue8m0(b200, m, n, k, tile_n):
    """The MXFP4 flavour of the demo (sf_vec_size 32, ue8m0 scales; blockscaled_gemm_dispatch.py:34-43): random e2m1
    codes with random power-of-two scales per 32 elements.  Every product and every scale is a power of two times a
    small integer, so f32 sums differ from the oracle's only by summation order: rel-L2 <= 1e-5; integer-valued data
    through run() must be exact."""
    rng = np.random.default_rng(m + n + k)
    ac = rng.integers(0, 16, size=(m, k), dtype=np.uint8)
    bc = rng.integers(0, 16, size=(n, k), dtype=np.uint8)
    kb = -(-k // 32)
    sfa = rng.integers(122, 131, size=(m, kb), dtype=np.uint8)        # 2^-5 .. 2^3
    sfb = rng.integers(122, 131, size=(n, kb), dtype=np.uint8)
    ref = O.gemm_nvfp4_ref(ac, sfa, bc, sfb, alpha=0.25, sf_vec=32)
    a, b, sa, sb = _dev_operands(ac, sfa, bc, sfb)
    c = b200.nvfp4_gemm(a, b, sa, sb, alpha=torch.tensor([0.25], device="cuda"), out_dtype=torch.float32, tile_n=tile_n,
                        sf_vec_size=32)
    torch.cuda.synchronize()
    _check_status(b200)
    err = torch.linalg.vector_norm(c.cpu() - ref) / torch.linalg.vector_norm(ref)
    assert err <= 1e-5, float(err)


def test_mxfp4_through_the_demo_entry(b200):
    torch.manual_seed(0)
    g = b200.gemm
    us = g.run((256, 256, 512, 1), g.Float4E2M1FN, g.Float4E2M1FN, g.Float8E8M0FNU, 32, g.Float16, a_major="k",
               b_major="k", c_major="n", tile_shape_mnk=(128, 128, 128), epi_tile=(128, 128), tolerance=0.1,
               warmup_iterations=0, iterations=1, skip_ref_check=False)
    assert us > 0


@pytest.mark.parametrize("m,n,k,tile_n", [(128, 128, 128, 128), (256, 384, 512, 0), (200, 264, 1168, 256), (128, 192, 2048, 64)])
@pytest.mark.parametrize("a_e5m2,b_e5m2", [(False, False), (True, False), (True, True)])
def test_mxfp8_block32_ue8m0(b200, m, n, k, tile_n, a_e5m2, b_e5m2):
    """The MXFP8 flavours of the demo (8-bit operands, ue8m0 scale per 32 elements; blockscaled_gemm_dispatch.py:34-43):
    random finite e4m3 / e5m2 bytes of moderate magnitude with random power-of-two scales; rel-L2 <= 1e-5 against the
    de-quantised f32 product (summation order is the only difference)."""
    rng = np.random.default_rng(m + n + k + a_e5m2 + 2 * b_e5m2)

    def operand(rows, e5m2):
        # exponent fields in the middle of the range (no inf / nan, no overflow of the f32 sums), random sign / mantissa
        if e5m2:
            exp = rng.integers(10, 18, size=(rows, k), dtype=np.uint8)
            return (rng.integers(0, 2, size=(rows, k), dtype=np.uint8) << 7) | (exp << 2) | rng.integers(0, 4, size=(rows, k), dtype=np.uint8)
        exp = rng.integers(3, 10, size=(rows, k), dtype=np.uint8)
        return (rng.integers(0, 2, size=(rows, k), dtype=np.uint8) << 7) | (exp << 3) | rng.integers(0, 8, size=(rows, k), dtype=np.uint8)

    ab, bb = operand(m, a_e5m2).astype(np.uint8), operand(n, b_e5m2).astype(np.uint8)
    kb = -(-k // 32)
    sfa = rng.integers(122, 131, size=(m, kb), dtype=np.uint8)
    sfb = rng.integers(122, 131, size=(n, kb), dtype=np.uint8)
    ref = O.gemm_mxfp8_ref(ab, sfa, bb, sfb, alpha=0.25, a_e5m2=a_e5m2, b_e5m2=b_e5m2)
    a = torch.from_numpy(ab).cuda().view(torch.float8_e5m2 if a_e5m2 else torch.float8_e4m3fn)
    b = torch.from_numpy(bb).cuda().view(torch.float8_e5m2 if b_e5m2 else torch.float8_e4m3fn)
    sa = torch.from_numpy(O.swizzle_sf(sfa)).cuda()
    sb = torch.from_numpy(O.swizzle_sf(sfb)).cuda()
    c = b200.mxfp8_gemm(a, b, sa, sb, alpha=torch.tensor([0.25], device="cuda"), out_dtype=torch.float32, tile_n=tile_n)
    torch.cuda.synchronize()
    _check_status(b200)
    err = torch.linalg.vector_norm(c.cpu() - ref) / torch.linalg.vector_norm(ref)
    assert err <= 1e-5, float(err)


def test_mxfp8_through_the_demo_entry(b200):
    torch.manual_seed(0)
    g = b200.gemm
    for a_dt, b_dt in ((g.Float8E4M3FN, g.Float8E4M3FN), (g.Float8E5M2, g.Float8E4M3FN)):
        us = g.run((256, 256, 512, 1), a_dt, b_dt, g.Float8E8M0FNU, 32, g.BFloat16, a_major="k", b_major="k",
                   c_major="n", tile_shape_mnk=(128, 128, 128), epi_tile=(128, 128), tolerance=0.1,
                   warmup_iterations=0, iterations=1, skip_ref_check=False)
        assert us > 0
