"""Host-side partitioning logic and the expert-parallel gather / reduce-scatter bookkeeping, run as two CPU
ranks over the gloo backend (the local expert compute is the CPU oracle, injected in place of the CUDA op)."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import nvfp4_oracle as O


def test_shard_rows_covers_everything_in_128_row_blocks(b200):
    from cutedsl_fully_opensourced_b200.parallel import shard_rows
    for rows in (0, 1, 127, 128, 129, 1000, 8192, 8192 * 3 + 5):
        for world in (1, 2, 3, 4, 8):
            spans = [shard_rows(rows, world, r) for r in range(world)]
            assert spans[0][0] == 0
            for (s0, c0), (s1, _) in zip(spans, spans[1:]):
                assert s0 + c0 == s1
            assert spans[-1][0] + spans[-1][1] == rows
            for s, c in spans[:-1]:
                assert c == 0 or (s % 128 == 0 and (c % 128 == 0 or s + c == rows))
    assert shard_rows(8192, 8, 3) == (3072, 1024)
    with pytest.raises(ValueError):
        shard_rows(10, 2, 2)


def test_shard_experts(b200):
    from cutedsl_fully_opensourced_b200.parallel import shard_experts
    assert [shard_experts(128, 8, r) for r in range(8)] == [(16 * r, 16) for r in range(8)]
    assert shard_experts(256, 1, 0) == (0, 256)
    with pytest.raises(ValueError):
        shard_experts(10, 4, 0)


def _problem():
    rng = np.random.default_rng(3)
    torch.manual_seed(3)
    experts, hidden, inter, top_k, tokens = 4, 128, 128, 2, 12
    w1c = rng.integers(0, 16, size=(experts, 2 * inter, hidden), dtype=np.uint8)
    w2c = rng.integers(0, 16, size=(experts, hidden, inter), dtype=np.uint8)
    w1s = rng.integers(0x18, 0x30, size=(experts, 2 * inter, hidden // 16), dtype=np.uint8)
    w2s = rng.integers(0x18, 0x30, size=(experts, hidden, inter // 16), dtype=np.uint8)
    x = torch.randn(tokens, hidden).to(torch.bfloat16)
    ids, wts = O.route_topk_ref(torch.randn(tokens, experts), top_k)
    return (w1c, w1s, w2c, w2s), x, ids, wts.contiguous(), experts, top_k


def _local_oracle(weights):
    w1c, w1s, w2c, w2s = weights

    def fn(x_all, ids_all, w_all, lo, n):
        # slots of foreign experts contribute nothing: give them weight 0 and a valid local id
        local = (ids_all >= lo) & (ids_all < lo + n)
        ids_l = torch.where(local, ids_all - lo, torch.zeros_like(ids_all))
        w_l = torch.where(local, w_all, torch.zeros_like(w_all))
        sl = slice(lo, lo + n)
        out = torch.zeros(x_all.shape, dtype=torch.float32)
        for slot in range(ids_all.shape[1]):
            part = O.moe_ref(x_all, w1c[sl], w1s[sl], w2c[sl], w2s[sl], ids_l[:, slot:slot + 1],
                             torch.ones(x_all.shape[0], 1), np.full(n, 0.02, np.float32))
            out += w_l[:, slot:slot + 1] * part.float()
        return out
    return fn


def _worker(rank, world, port, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import cutedsl_fully_opensourced_b200  # noqa: F401  (loads the library; no GPU needed for that)
        from cutedsl_fully_opensourced_b200.parallel import ExpertParallelMoE
        weights, x, ids, wts, experts, top_k = _problem()
        ep = ExpertParallelMoE(experts, top_k, local_moe=_local_oracle(weights))
        assert (ep.expert_lo, ep.local_experts) == (rank * 2, 2)
        t = x.shape[0] // world
        sl = slice(rank * t, (rank + 1) * t)
        out = ep.forward(x[sl], ids[sl], wts[sl])
        torch.save(out, os.path.join(result_dir, f"out{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_expert_parallel_bookkeeping_two_gloo_ranks(tmp_path, lib_built):
    world = 2
    port = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    weights, x, ids, wts, experts, top_k = _problem()
    single = _local_oracle(weights)(x, ids, wts, 0, experts).to(torch.bfloat16)
    got = torch.cat([torch.load(os.path.join(tmp_path, f"out{r}.pt")) for r in range(world)])
    assert got.shape == single.shape
    err = torch.linalg.vector_norm(got.float() - single.float()) / torch.linalg.vector_norm(single.float())
    assert err <= 1e-2
