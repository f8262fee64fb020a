"""Expert-parallel MoE on two GPUs (one process per GPU, NCCL + symmetric memory) against the single-GPU operator:
the peer-memory path (bit-equal, with ids and with the router inside the dispatch, a masked slot included) and the
all-to-all-v fallback.  Needs two devices; on a one-GPU box it reports a skip with that reason (the same kernels
are covered there by tests/test_moe_ep_emulated_gpu.py, which emulates the ranks on one GPU)."""
import os

import numpy as np
import pytest
import torch

from oracle import nvfp4_oracle as O

pytestmark = pytest.mark.gpu


def _problem():
    rng = np.random.default_rng(11)
    torch.manual_seed(11)
    experts, hidden, inter, top_k, tokens = 8, 512, 256, 4, 96
    w1c = rng.integers(0, 16, size=(experts, 2 * inter, hidden), dtype=np.uint8)
    w2c = rng.integers(0, 16, size=(experts, hidden, inter), dtype=np.uint8)
    w1s = rng.integers(0x18, 0x30, size=(experts, 2 * inter, hidden // 16), dtype=np.uint8)
    w2s = rng.integers(0x18, 0x30, size=(experts, hidden, inter // 16), dtype=np.uint8)
    x = torch.randn(tokens, hidden).to(torch.bfloat16)
    ids, wts = O.route_topk_ref(_logits(), top_k)
    ids = ids.clone()
    ids[5, 1] = -1                      # a masked slot: contributes nothing on either path
    return (w1c, w1s, w2c, w2s), x, ids, wts.contiguous(), experts, top_k


def _logits():
    return torch.randn(96, 8, generator=torch.Generator().manual_seed(12))


def _dev_weights(w1c, w1s, w2c, w2s, sl, dev):
    return {"w1": torch.from_numpy(O.pack_e2m1(w1c[sl])).to(dev), "w1_sf": torch.from_numpy(O.swizzle_sf(w1s[sl])).to(dev),
            "w2": torch.from_numpy(O.pack_e2m1(w2c[sl])).to(dev), "w2_sf": torch.from_numpy(O.swizzle_sf(w2s[sl])).to(dev),
            "w1_alpha": torch.full((sl.stop - sl.start,), 0.02, device=dev)}


def _worker(rank, world, port, result_dir):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import cutedsl_fully_opensourced_b200 as b200
        (w1c, w1s, w2c, w2s), x, ids, wts, experts, top_k = _problem()
        dev = torch.device("cuda", rank)
        t = x.shape[0] // world
        mine = slice(rank * t, (rank + 1) * t)
        for kind in ("collective", "peer", "peer_rank"):
            if kind == "collective":
                ep = b200.parallel.ExpertParallelMoE(experts, top_k)
            else:
                ep = b200.parallel.PeerExpertParallelMoE(experts, top_k, t, x.shape[1], w2c.shape[2],
                                                         return_rows="per_slot" if kind == "peer" else "per_rank")
            sl = slice(ep.expert_lo, ep.expert_lo + ep.local_experts)
            w = _dev_weights(w1c, w1s, w2c, w2s, sl, dev)
            for _ in range(3):          # several steps: buffers are reused
                out = ep.forward(x[mine].to(dev), ids[mine].to(dev), wts[mine].to(dev), w)
            b200.synchronize()          # raises if a wait expired
            torch.save(out.cpu(), os.path.join(result_dir, f"out_{kind}{rank}.pt"))
            if kind == "peer":
                logits = _logits()[mine].to(dev)
                out = ep.forward(x[mine].to(dev), None, None, w, router_logits=logits, check=True)
                ids_r, w_r = ep.last_routing()
                torch.save((out.cpu(), ids_r.cpu(), w_r.cpu()), os.path.join(result_dir, f"routed{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_expert_parallel_two_gpus_matches_single_gpu(b200, tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world, port = 2, 29600 + os.getpid() % 2000
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    (w1c, w1s, w2c, w2s), x, ids, wts, experts, top_k = _problem()
    w = _dev_weights(w1c, w1s, w2c, w2s, slice(0, experts), "cuda")
    single = b200.b12x_fused_moe(x.cuda(), w["w1"], w["w1_sf"], w["w2"], w["w2_sf"], ids.cuda(), wts.cuda(), experts,
                                 top_k, w1_alpha=w["w1_alpha"]).cpu()
    valid = ids >= 0
    ref = O.moe_ref(x, w1c, w1s, w2c, w2s, torch.where(valid, ids, torch.zeros_like(ids)),
                    torch.where(valid, wts, torch.zeros_like(wts)), np.full(experts, 0.02, np.float32))
    # routed inside the dispatch: same bits as routing with topk_route and the single-GPU operator
    ids_g, w_g = b200.topk_route(_logits().cuda(), top_k)
    single_routed = b200.b12x_fused_moe(x.cuda(), w["w1"], w["w1_sf"], w["w2"], w["w2_sf"], ids_g, w_g, experts, top_k,
                                        w1_alpha=w["w1_alpha"]).cpu()
    parts = [torch.load(os.path.join(tmp_path, f"routed{r}.pt")) for r in range(world)]
    assert torch.equal(torch.cat([p[1] for p in parts]), ids_g.cpu())
    assert torch.equal(torch.cat([p[0] for p in parts]), single_routed)
    for kind in ("collective", "peer", "peer_rank"):
        got = torch.cat([torch.load(os.path.join(tmp_path, f"out_{kind}{r}.pt")) for r in range(world)])
        if kind == "peer":
            # same bf16 per-slot rows, same slot order, same single rounding as on one GPU
            assert torch.equal(got, single), "peer-memory expert parallelism differs from the single-GPU result"
        else:
            # collective: bf16 rows both ways, f32 weighted sum by torch: only the summation order may differ.
            # peer_rank: the sum is grouped by serving rank, one bf16 rounding per partial sum.
            base = single.float()
            err = torch.linalg.vector_norm(got.float() - base) / torch.linalg.vector_norm(base)
            assert err <= (4e-3 if kind == "peer_rank" else 2e-3), float(err)
        assert torch.linalg.vector_norm(got.float() - ref.float()) / torch.linalg.vector_norm(ref.float()) <= 1e-2
