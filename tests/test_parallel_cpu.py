"""Host-side partitioning logic, the all-to-all-v dispatch / combine bookkeeping and the peer health check, run as
two CPU ranks over the gloo backend (the local expert compute is the CPU oracle, injected in place of the CUDA op)."""
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
    """One expert per row, as the all-to-all-v path asks for: rows [n, H], local expert ids [n] -> rows [n, H]."""
    w1c, w1s, w2c, w2s = weights

    def fn(rows, ids_local, lo, n):
        sl = slice(lo, lo + n)
        return O.moe_ref(rows, w1c[sl], w1s[sl], w2c[sl], w2s[sl], ids_local.reshape(-1, 1).to(torch.int32),
                         torch.ones(rows.shape[0], 1), np.full(n, 0.02, np.float32))
    return fn


def _worker(rank, world, port, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import cutedsl_fully_opensourced_b200  # noqa: F401  (loads the library; no GPU needed for that)
        from cutedsl_fully_opensourced_b200.parallel import ExpertParallelMoE
        weights, x, ids, wts, experts, top_k = _problem()
        ids = ids.clone()
        ids[1, 0] = -1                       # a masked slot contributes nothing
        ep = ExpertParallelMoE(experts, top_k, local_moe=_local_oracle(weights))
        assert (ep.expert_lo, ep.local_experts) == (rank * 2, 2)
        t = x.shape[0] // world
        sl = slice(rank * t, (rank + 1) * t)
        out = ep.forward(x[sl], ids[sl], wts[sl])
        torch.save(out, os.path.join(result_dir, f"out{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_expert_parallel_all_to_all_two_gloo_ranks(tmp_path, lib_built):
    world = 2
    port = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    weights, x, ids, wts, experts, top_k = _problem()
    wts = wts.clone()
    wts[1, 0] = 0.0                          # the reference result of the masked slot
    single = O.moe_ref(x, *[weights[i] for i in (0, 1, 2, 3)], ids, wts, np.full(experts, 0.02, np.float32))
    got = torch.cat([torch.load(os.path.join(tmp_path, f"out{r}.pt")) for r in range(world)])
    assert got.shape == single.shape
    err = torch.linalg.vector_norm(got.float() - single.float()) / torch.linalg.vector_norm(single.float())
    assert err <= 1e-2


def _leaver(rank, world, port, result_dir):
    """Two ranks run a healthy step; then rank 1 leaves (between steps, nothing in flight) and rank 0's health
    check before its next step must raise instead of hanging."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import cutedsl_fully_opensourced_b200  # noqa: F401
    from cutedsl_fully_opensourced_b200.parallel import PeerHealth
    health = PeerHealth(timeout_s=3.0)
    health.check()                           # step 1: both ranks are there
    if rank == 1:
        os._exit(0)                          # leaves without a word
    try:
        health.check()                       # step 2
        outcome = "no error"
    except RuntimeError as e:
        outcome = f"raised: {e}"
    with open(os.path.join(result_dir, "outcome.txt"), "w") as f:
        f.write(outcome)
    os._exit(0)                              # the group cannot be torn down cleanly any more


def test_survivor_raises_when_a_rank_leaves_between_steps(tmp_path, lib_built):
    world = 2
    port = 31500 + os.getpid() % 2000
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_leaver, args=(r, world, port, str(tmp_path))) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
        assert not p.is_alive(), "a rank hung"
    outcome = open(os.path.join(tmp_path, "outcome.txt")).read()
    assert outcome.startswith("raised: expert-parallel group is incomplete"), outcome
