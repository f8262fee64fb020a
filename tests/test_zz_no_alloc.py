"""b200fp4_moe_fused_noalloc, the MoE entry point for callers that must not allocate.

Inference engines that reserve all device memory up front (and forbid cudaMalloc afterwards), plugins that
are only handed raw pointers, and latency-critical loops cannot supply the scratch buffer that
b200fp4_moe_fused asks for.  The no-alloc entry point keeps its scratch in a fixed 32 MiB array inside the
library instead.  This test drives it straight through the C-ABI (ctypes), twice in a row because all calls
share that one array and it keeps the previous call's contents, and requires the same bits as the regular
entry point produces with a caller-provided workspace.  It also checks that a problem too large for the
built-in scratch is refused with a clear message rather than run.

This file sorts last on purpose: with `pytest -x` every other test has already run if this one fails.
"""
import ctypes

import numpy as np
import pytest
import torch

from oracle import nvfp4_oracle as O

pytestmark = pytest.mark.gpu


def _six_mode_storage(sf_logical):
    return torch.from_numpy(O.swizzle_sf(sf_logical)).cuda()       # [E, tiles*512] tiled bytes


def _problem(tokens, experts, hidden, inter, top_k, seed):
    rng = np.random.default_rng(seed)
    torch.manual_seed(seed)
    w1c = rng.integers(0, 16, size=(experts, 2 * inter, hidden), dtype=np.uint8)
    w2c = rng.integers(0, 16, size=(experts, hidden, inter), dtype=np.uint8)
    w1s = rng.integers(0x18, 0x30, size=(experts, 2 * inter, hidden // 16), dtype=np.uint8)
    w2s = rng.integers(0x18, 0x30, size=(experts, hidden, inter // 16), dtype=np.uint8)
    x = torch.randn(tokens, hidden).to(torch.bfloat16)
    ids, wts = O.route_topk_ref(torch.randn(tokens, experts), top_k)
    dev = dict(
        x=x.cuda(), w1=torch.from_numpy(O.pack_e2m1(w1c)).cuda(), s1=_six_mode_storage(w1s),
        w2=torch.from_numpy(O.pack_e2m1(w2c)).cuda(), s2=_six_mode_storage(w2s), ids=ids.cuda(),
        wts=wts.contiguous().cuda(), a1=torch.full((experts,), 0.02, device="cuda"))
    host = (x, w1c, w1s, w2c, w2s, ids, wts)
    return dev, host


def _call_regular(lib, d, out, tokens, hidden, inter, experts, top_k, stream):
    need = lib.b200fp4_moe_workspace_bytes(tokens, hidden, inter, experts, top_k)
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    return lib.b200fp4_moe_fused(
        d["x"].data_ptr(), d["w1"].data_ptr(), d["s1"].data_ptr(), d["w2"].data_ptr(), d["s2"].data_ptr(),
        d["ids"].data_ptr(), d["wts"].data_ptr(), d["a1"].data_ptr(), None, None, out.data_ptr(), tokens, hidden,
        inter, experts, top_k, 0, 0, 1, ws.data_ptr(), need, stream), ws


def _call_noalloc(lib, d, out, status, tokens, hidden, inter, experts, top_k, stream):
    return lib.b200fp4_moe_fused_noalloc(
        d["x"].data_ptr(), d["w1"].data_ptr(), d["s1"].data_ptr(), d["w2"].data_ptr(), d["s2"].data_ptr(),
        d["ids"].data_ptr(), d["wts"].data_ptr(), d["a1"].data_ptr(), None, None, out.data_ptr(), tokens, hidden,
        inter, experts, top_k, 0, 0, status.data_ptr(), stream)


def test_noalloc_entry_matches_regular_entry_on_two_calls_in_a_row(b200):
    lib = b200._lib.lib
    stream = torch.cuda.current_stream().cuda_stream
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    # two different problems back to back, so the second call meets the first call's leftovers in the array
    for (tokens, experts, hidden, inter, top_k, seed) in [(3, 8, 512, 256, 4, 1), (2, 16, 1024, 384, 8, 2)]:
        d, host = _problem(tokens, experts, hidden, inter, top_k, seed)
        ref_out = torch.zeros(tokens, hidden, dtype=torch.bfloat16, device="cuda")
        rc, ws = _call_regular(lib, d, ref_out, tokens, hidden, inter, experts, top_k, stream)
        assert rc == 0, lib.b200fp4_last_error()
        outs = [torch.full((tokens, hidden), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(2)]
        free_before = None
        for out in outs:
            rc = _call_noalloc(lib, d, out, status, tokens, hidden, inter, experts, top_k, stream)
            assert rc == 0, lib.b200fp4_last_error()
            torch.cuda.synchronize()
            # the entry point allocates nothing: once its first call on this GPU has been made, the device's free
            # memory does not move across further calls (outputs were allocated beforehand)
            free_now = torch.cuda.mem_get_info()[0]
            assert free_before is None or free_now == free_before, "the no-alloc entry point changed free memory"
            free_before = free_now
            assert int(status.item()) == 0, "a device-side wait expired"
            assert torch.equal(out, ref_out), "no-alloc entry point disagrees with b200fp4_moe_fused"
        # and both agree with the CPU oracle within the MoE tolerance of the other tests
        x, w1c, w1s, w2c, w2s, ids, wts = host
        ref = O.moe_ref(x, w1c, w1s, w2c, w2s, ids, wts, np.full(experts, 0.02, np.float32))
        err = torch.linalg.vector_norm(ref_out.cpu().float() - ref.float()) / torch.linalg.vector_norm(ref.float())
        assert err <= 1e-2
    assert b200._lib.device_status() == 0


def test_noalloc_entry_refuses_problems_beyond_its_scratch(b200):
    lib = b200._lib.lib
    tokens, experts, hidden, inter, top_k = 64, 128, 2048, 768, 8
    assert lib.b200fp4_moe_workspace_bytes(tokens, hidden, inter, experts, top_k) > (32 << 20)
    one = torch.zeros(16, dtype=torch.uint8, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    p = one.data_ptr()
    rc = lib.b200fp4_moe_fused_noalloc(p, p, p, p, p, p, p, None, None, None, p, tokens, hidden, inter, experts,
                                       top_k, 0, 0, status.data_ptr(), None)
    assert rc == b200._lib.UNSUPPORTED
    msg = lib.b200fp4_last_error().decode()
    assert "built-in scratch" in msg and "b200fp4_moe_fused" in msg
    rc = lib.b200fp4_moe_fused_noalloc(p, p, p, p, p, p, p, None, None, None, p, 2, 512, 256, 8, 2, 0, 0, None, None)
    assert rc == b200._lib.INVALID_ARGUMENT
