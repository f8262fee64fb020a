"""The expert-parallel MoE kernels (dispatch / compute / combine over "peer" buffers) on ONE GPU.

The ranks of a group are emulated as separate buffers of the same device and their kernels are issued on one
stream in an order in which every cross-rank wait is already satisfied when its kernel starts: all ranks' count
kernels, then all place kernels, all computes, all combines.  No kernel ever waits for a later launch, so nothing
spins; the waits are given a short bound anyway.  The bar is bit-equality with the single-GPU operator on the
same tokens (same bf16 per-slot rows, same slot order, one rounding) and rel-L2 <= 1e-2 against the CPU oracle.
"""
import ctypes

import numpy as np
import pytest
import torch

from oracle import nvfp4_oracle as O

pytestmark = pytest.mark.gpu

WAIT_MS = 200.0


def _problem(tokens, experts, hidden, inter, top_k, seed, hot=False):
    rng = np.random.default_rng(seed)
    torch.manual_seed(seed)
    w1c = rng.integers(0, 16, size=(experts, 2 * inter, hidden), dtype=np.uint8)
    w2c = rng.integers(0, 16, size=(experts, hidden, inter), dtype=np.uint8)
    w1s = rng.integers(0x18, 0x30, size=(experts, 2 * inter, hidden // 16), dtype=np.uint8)
    w2s = rng.integers(0x18, 0x30, size=(experts, hidden, inter // 16), dtype=np.uint8)
    x = torch.randn(tokens, hidden).to(torch.bfloat16)
    logits = torch.randn(tokens, experts)
    if hot:
        logits[: max(1, tokens // 4), 1] += 1e4          # a hot expert: one rank receives far more rows
    ids, wts = O.route_topk_ref(logits, top_k)
    return (w1c, w1s, w2c, w2s), x, logits, ids, wts.contiguous()


def _dev_weights(w, sl):
    w1c, w1s, w2c, w2s = w
    return dict(w1=torch.from_numpy(O.pack_e2m1(w1c[sl])).cuda(), s1=torch.from_numpy(O.swizzle_sf(w1s[sl])).cuda(),
                w2=torch.from_numpy(O.pack_e2m1(w2c[sl])).cuda(), s2=torch.from_numpy(O.swizzle_sf(w2s[sl])).cuda(),
                a1=torch.full((sl.stop - sl.start,), 0.02, device="cuda"))


class EmulatedGroup:
    def __init__(self, lib, check, world, tokens_local, hidden, inter, experts, top_k, mode=0):
        self.lib, self.check, self.world, self.mode = lib, check, world, mode
        self.shape = (tokens_local, hidden, inter, experts // world, top_k)
        nbytes = lib.b200fp4_moe_ep_buffer_bytes(*self.shape, world)
        assert nbytes > 0
        self.bufs = [torch.empty(nbytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
        self.peers = (ctypes.c_void_p * world)(*[b.data_ptr() for b in self.bufs])
        self.stream = torch.cuda.current_stream().cuda_stream
        for b in self.bufs:
            check(lib.b200fp4_moe_ep_reset(b.data_ptr(), *self.shape, world, self.stream))

    def step(self, xs, ids, wts, weights, logits=None):
        lib, check, w = self.lib, self.check, self.world
        t, h = xs[0].shape
        outs = [torch.full((t, h), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(w)]
        routed = logits is not None
        for fn in (lib.b200fp4_moe_ep_dispatch_count, lib.b200fp4_moe_ep_dispatch_place):
            for r in range(w):
                check(fn(xs[r].data_ptr(), None if routed else ids[r].data_ptr(),
                         None if routed else wts[r].data_ptr(), logits[r].data_ptr() if routed else None, 1,
                         self.peers, r, w, *self.shape, self.mode, WAIT_MS, self.stream))
        for r in range(w):
            d = weights[r]
            check(lib.b200fp4_moe_ep_compute(self.peers, r, w, d["w1"].data_ptr(), d["s1"].data_ptr(),
                                             d["w2"].data_ptr(), d["s2"].data_ptr(), d["a1"].data_ptr(), None, None,
                                             *self.shape, self.mode, WAIT_MS, self.stream))
        for r in range(w):
            check(lib.b200fp4_moe_ep_combine(self.peers, r, w, None if routed else ids[r].data_ptr(),
                                             None if routed else wts[r].data_ptr(), outs[r].data_ptr(), *self.shape,
                                             self.mode, WAIT_MS, self.stream))
        return outs


@pytest.mark.parametrize("world,tokens,experts,hidden,inter,top_k,hot", [
    (1, 40, 8, 512, 256, 4, False),
    (2, 96, 8, 512, 256, 4, False),
    (4, 512, 16, 1024, 384, 8, True),        # several 128-row blocks per expert, skewed towards one rank
    (8, 64, 32, 2304, 1280, 8, True),        # decode-like: few tokens per rank, long reductions (256-wide FC2 tiles)
    (2, 24, 4, 2304, 1280, 2, False),        # at most 32 tokens in total: the few-row tiles
])
@pytest.mark.parametrize("mode", [0, 1], ids=["per_slot", "per_rank"])
def test_emulated_ranks_match_single_gpu(b200, world, tokens, experts, hidden, inter, top_k, hot, mode):
    """Per-slot return: bit for bit the single-GPU operator.  Per-rank return: the same sum grouped by serving
    rank with one bf16 rounding per partial sum (bound on the difference: a few bf16 ulps, rel-L2 4e-3)."""
    lib, check = b200._lib.lib, b200._lib.check
    w, x, logits, ids, wts = _problem(tokens, experts, hidden, inter, top_k, seed=world * 7 + tokens, hot=hot)
    ids = ids.clone()
    ids[0, top_k - 1] = -1                   # a masked slot: never computed, must not be summed
    if tokens > 3:
        ids[3, 0] = experts + 5              # an id outside the group's experts
    t = tokens // world
    el = experts // world
    g = EmulatedGroup(lib, check, world, t, hidden, inter, experts, top_k, mode)
    xs = [x[r * t:(r + 1) * t].contiguous().cuda() for r in range(world)]
    idr = [ids[r * t:(r + 1) * t].contiguous().cuda() for r in range(world)]
    wtr = [wts[r * t:(r + 1) * t].contiguous().cuda() for r in range(world)]
    weights = [_dev_weights(w, slice(r * el, (r + 1) * el)) for r in range(world)]
    full = _dev_weights(w, slice(0, experts))
    single = b200.b12x_fused_moe(x.cuda(), full["w1"], full["s1"], full["w2"], full["s2"], ids.cuda(), wts.cuda(),
                                 experts, top_k, w1_alpha=full["a1"])
    for step in range(3):                    # several steps: signals and buffers are reused
        outs = g.step(xs, idr, wtr, weights)
        torch.cuda.synchronize()
        assert b200._lib.device_status() == 0, "a wait expired"
        got = torch.cat(outs)
        if mode == 0:
            assert torch.equal(got, single), f"step {step}: expert-parallel result differs from the single-GPU operator"
        else:
            assert bool(torch.isfinite(got.float()).all())
            diff = torch.linalg.vector_norm(got.float() - single.float()) / torch.linalg.vector_norm(single.float())
            assert diff <= 4e-3, f"step {step}: rel-L2 {float(diff)} against the single-GPU operator"
            if step == 0:
                first = got.clone()
            assert torch.equal(got, first), "the per-rank sums are taken in a fixed order: same bits every step"
    valid = (ids >= 0) & (ids < experts)
    ref = O.moe_ref(x, *w, torch.where(valid, ids, torch.zeros_like(ids)), torch.where(valid, wts, torch.zeros_like(wts)),
                    np.full(experts, 0.02, np.float32))
    err = torch.linalg.vector_norm(got.cpu().float() - ref.float()) / torch.linalg.vector_norm(ref.float())
    assert err <= 1e-2


@pytest.mark.parametrize("mode", [0, 1], ids=["per_slot", "per_rank"])
def test_emulated_ranks_route_from_logits_inside_the_dispatch(b200, mode):
    lib, check = b200._lib.lib, b200._lib.check
    world, tokens, experts, hidden, inter, top_k = 4, 128, 16, 512, 256, 4
    w, x, logits, ids, wts = _problem(tokens, experts, hidden, inter, top_k, seed=99)
    t, el = tokens // world, experts // world
    g = EmulatedGroup(lib, check, world, t, hidden, inter, experts, top_k, mode)
    xs = [x[r * t:(r + 1) * t].contiguous().cuda() for r in range(world)]
    lg = [logits[r * t:(r + 1) * t].contiguous().cuda() for r in range(world)]
    weights = [_dev_weights(w, slice(r * el, (r + 1) * el)) for r in range(world)]
    outs = g.step(xs, None, None, weights, logits=lg)
    # the routing computed on the GPU equals the oracle's
    for r in range(world):
        ids_r = torch.empty(t, top_k, dtype=torch.int32, device="cuda")
        w_r = torch.empty(t, top_k, dtype=torch.float32, device="cuda")
        check(lib.b200fp4_moe_ep_routing(g.bufs[r].data_ptr(), ids_r.data_ptr(), w_r.data_ptr(), *g.shape, world,
                                         g.stream))
        torch.cuda.synchronize()
        assert torch.equal(ids_r.cpu(), ids[r * t:(r + 1) * t])
        assert torch.allclose(w_r.cpu(), wts[r * t:(r + 1) * t], rtol=1e-5, atol=1e-7)
    assert b200._lib.device_status() == 0
    full = _dev_weights(w, slice(0, experts))
    ids_d, w_d = b200.topk_route(logits.cuda(), top_k)
    single = b200.b12x_fused_moe(x.cuda(), full["w1"], full["s1"], full["w2"], full["s2"], ids_d, w_d, experts, top_k,
                                 w1_alpha=full["a1"])
    torch.cuda.synchronize()
    if mode == 0:
        assert torch.equal(torch.cat(outs), single)
    else:
        got = torch.cat(outs).float()
        assert float(torch.linalg.vector_norm(got - single.float()) / torch.linalg.vector_norm(single.float())) <= 4e-3


@pytest.mark.parametrize("mode", [0, 1], ids=["per_slot", "per_rank"])
def test_wait_for_a_rank_that_never_signals_gives_up_and_reports(b200, mode):
    """A group of two whose second rank never runs: rank 0's place kernel waits for counts that nobody publishes.
    The wait gives up after its bound, the kernels that follow touch nothing, the status word carries bit 16 and
    the host raises; after a reset the same buffers work again."""
    lib, check = b200._lib.lib, b200._lib.check
    world, tokens, experts, hidden, inter, top_k = 2, 32, 4, 512, 256, 2
    w, x, logits, ids, wts = _problem(tokens, experts, hidden, inter, top_k, seed=5)
    t, el = tokens // world, experts // world
    g = EmulatedGroup(lib, check, world, t, hidden, inter, experts, top_k, mode)
    xs = [x[r * t:(r + 1) * t].contiguous().cuda() for r in range(world)]
    idr = [ids[r * t:(r + 1) * t].contiguous().cuda() for r in range(world)]
    wtr = [wts[r * t:(r + 1) * t].contiguous().cuda() for r in range(world)]
    weights = [_dev_weights(w, slice(r * el, (r + 1) * el)) for r in range(world)]
    b200._lib.device_status()                                        # clear
    out = torch.zeros(t, hidden, dtype=torch.bfloat16, device="cuda")
    d = weights[0]
    short = 2.0                                                      # milliseconds
    check(lib.b200fp4_moe_ep_dispatch(xs[0].data_ptr(), idr[0].data_ptr(), wtr[0].data_ptr(), None, 1, g.peers, 0,
                                      world, *g.shape, mode, short, g.stream))
    check(lib.b200fp4_moe_ep_compute(g.peers, 0, world, d["w1"].data_ptr(), d["s1"].data_ptr(), d["w2"].data_ptr(),
                                     d["s2"].data_ptr(), d["a1"].data_ptr(), None, None, *g.shape, mode, short,
                                     g.stream))
    check(lib.b200fp4_moe_ep_combine(g.peers, 0, world, idr[0].data_ptr(), wtr[0].data_ptr(), out.data_ptr(),
                                     *g.shape, mode, short, g.stream))
    with pytest.raises(b200.B200Fp4Error, match="another rank"):
        b200.synchronize()
    assert b200._lib.device_status() == 0                            # reading cleared it
    # recovery: reset both buffers, run a healthy step
    for b in g.bufs:
        check(lib.b200fp4_moe_ep_reset(b.data_ptr(), *g.shape, world, g.stream))
    outs = g.step(xs, idr, wtr, weights)
    b200.synchronize()
    full = _dev_weights(w, slice(0, experts))
    single = b200.b12x_fused_moe(x.cuda(), full["w1"], full["s1"], full["w2"], full["s2"], ids.cuda(), wts.cuda(),
                                 experts, top_k, w1_alpha=full["a1"])
    torch.cuda.synchronize()
    if mode == 0:
        assert torch.equal(torch.cat(outs), single)
    else:
        got = torch.cat(outs).float()
        assert float(torch.linalg.vector_norm(got - single.float()) / torch.linalg.vector_norm(single.float())) <= 4e-3


def test_peer_wait_selftest_sets_the_status_bit(b200):
    lib, check = b200._lib.lib, b200._lib.check
    shape = (8, 256, 128, 2, 2)
    nbytes = lib.b200fp4_moe_ep_buffer_bytes(*shape, 2)
    buf = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    b200._lib.device_status()
    check(lib.b200fp4_selftest_peer_wait(buf.data_ptr(), 2, 1.0, *shape, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert b200._lib.device_status() == b200._lib.STATUS_PEER_WAIT
    assert b200._lib.device_status() == 0
