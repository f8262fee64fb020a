"""One process per GPU over ``torch.distributed``: how the hot path is partitioned.

* RMSNorm-quant and the GEMM shard by rows (``shard_rows``): rows are independent, every rank calls the
  single-GPU operator on its block and nothing is communicated.  Blocks are multiples of 128 rows so that a rank
  owns whole 128x4 scale-factor tiles.
* The MoE shards by expert (``shard_experts``, weights never move) and by token (each rank owns a slice of the
  batch).  Two implementations of the dispatch / combine exchange:

  ``PeerExpertParallelMoE`` (the product path): the exchange lives inside the kernels.  Each rank quantises its
  tokens once and stores every (token, slot) row straight into the FC1 operand of the rank that owns the slot's
  expert (NVLink peer stores over torch symmetric memory); FC2's epilogue stores every output row straight into
  the buffer of the rank that owns the token.  The ranks synchronise through three bounded signals per step that
  the kernels themselves raise and wait for; there is no host-side or library barrier in a step.

  ``ExpertParallelMoE`` (portable fallback): a classic all-to-all-v dispatch / combine over
  ``torch.distributed`` (NCCL on GPUs, gloo in the CPU tests): rows are sorted by destination rank on the host
  side with torch ops, exchanged with ``all_to_all_single``, computed by the single-GPU operator as top-1 rows,
  sent back and summed with the routing weights.  It synchronises the host once per step (the split sizes) and
  moves bf16 rows both ways, so it is slower than the peer-memory path; it exists for fabrics without peer
  access and as the cross-check of the peer-memory path.

The reference itself is single-GPU (it has no collective anywhere); this layer is new.
"""
from __future__ import annotations

import datetime
from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist

from ._shard import shard_experts, shard_rows  # noqa: F401  (re-exported)


class PeerHealth:
    """Host-side liveness check of the ranks of a group, for callers of ``PeerExpertParallelMoE``.

    The kernels of the peer-memory path wait for their peers with a time bound and report an expired wait
    through the device status word; that is discovered only after the fact.  ``check()`` finds a missing rank
    BEFORE the next launch: it is a ``monitored_barrier`` with a timeout on a gloo group (CPU side, so it works
    whatever state the GPUs are in) and raises ``RuntimeError`` naming the ranks that did not arrive.
    It costs a host round trip, so call it every N steps or after an error, not in every step."""

    def __init__(self, group: Optional[dist.ProcessGroup] = None, timeout_s: float = 10.0):
        self.timeout = datetime.timedelta(seconds=timeout_s)
        base = group if group is not None else dist.group.WORLD
        if dist.get_backend(base) == "gloo":
            self.group = base
        else:
            self.group = dist.new_group(ranks=dist.get_process_group_ranks(base), backend="gloo",
                                        timeout=self.timeout)

    def check(self) -> None:
        try:
            dist.monitored_barrier(self.group, timeout=self.timeout, wait_all_ranks=True)
        except RuntimeError as e:           # gloo reports which ranks failed to join
            raise RuntimeError(f"expert-parallel group is incomplete: {e}") from e


class ExpertParallelMoE:
    """Expert-parallel fused MoE as an all-to-all-v dispatch / combine over a process group (NCCL or gloo).

    ``local_moe(x_rows, local_ids, expert_lo, local_experts) -> rows`` computes, for every received row, the
    output row of ONE expert (float32 or bfloat16 ``[rows, hidden]``); by default it is the CUDA operator of this
    package called with top-1 routing.  Tests on CPU ranks inject a stand-in to exercise the exchange
    bookkeeping with the gloo backend.
    """

    def __init__(self, num_experts: int, top_k: int, group: Optional[dist.ProcessGroup] = None,
                 local_moe: Optional[Callable] = None):
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.num_experts, self.top_k = num_experts, top_k
        self.expert_lo, self.local_experts = shard_experts(num_experts, self.world, self.rank)
        self._local_moe = local_moe

    def _run_local(self, rows, ids_local, weights):
        if self._local_moe is not None:
            return self._local_moe(rows, ids_local, self.expert_lo, self.local_experts)
        from .moe import b12x_fused_moe
        n = rows.shape[0]
        ones = torch.ones(n, 1, dtype=torch.float32, device=rows.device)
        return b12x_fused_moe(rows, weights["w1"], weights["w1_sf"], weights["w2"], weights["w2_sf"],
                              ids_local.reshape(n, 1).to(torch.int32).contiguous(), ones, self.local_experts, 1,
                              w1_alpha=weights.get("w1_alpha"), w2_alpha=weights.get("w2_alpha"),
                              fc2_input_scale=weights.get("fc2_input_scale"))

    def forward(self, x: torch.Tensor, ids: torch.Tensor, scales: torch.Tensor, weights: Optional[dict] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x bf16 [t, H], ids int32 [t, k] (global expert ids; ids outside the group's experts contribute
        nothing), scales f32 [t, k] of THIS rank's tokens; ``weights`` holds this rank's experts.
        Returns bf16 [t, H]."""
        t, h = x.shape
        k, w = self.top_k, self.world
        flat = ids.reshape(-1).to(torch.int64)
        valid = (flat >= 0) & (flat < self.num_experts)
        dest = torch.where(valid, flat // self.local_experts, torch.full_like(flat, w))     # w = dropped
        order = torch.argsort(dest, stable=True)
        send_counts = torch.bincount(dest, minlength=w + 1)[:w]
        n_send = int(send_counts.sum())
        order = order[:n_send]
        send_rows = x[order // k].contiguous()
        send_ids = (flat[order] % self.local_experts).to(torch.int32).contiguous()
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        send_split = send_counts.tolist()                      # the one host synchronisation of the step
        recv_split = recv_counts.tolist()
        n_recv = sum(recv_split)
        recv_rows = torch.empty(n_recv, h, dtype=x.dtype, device=x.device)
        recv_ids = torch.empty(n_recv, dtype=torch.int32, device=x.device)
        dist.all_to_all_single(recv_rows, send_rows, recv_split, send_split, group=self.group)
        dist.all_to_all_single(recv_ids, send_ids, recv_split, send_split, group=self.group)
        if n_recv:
            done = self._run_local(recv_rows, recv_ids, weights).to(torch.bfloat16).contiguous()
        else:
            done = torch.empty(0, h, dtype=torch.bfloat16, device=x.device)
        back = torch.empty(n_send, h, dtype=torch.bfloat16, device=x.device)
        dist.all_to_all_single(back, done, send_split, recv_split, group=self.group)
        # weighted sum in f32 in slot order: rows return in `order`; put them back at (token, slot)
        slot_rows = torch.zeros(t * k, h, dtype=torch.float32, device=x.device)
        slot_rows[order] = back.float()
        res = (slot_rows.view(t, k, h) * scales.reshape(t, k, 1).float()).sum(1)
        if out is None:
            out = torch.empty(t, h, dtype=torch.bfloat16, device=x.device)
        out.copy_(res)
        return out


class PeerExpertParallelMoE:
    """Expert-parallel fused MoE whose dispatch and combine are peer-memory stores inside the kernels.

    Per step and rank, all on the current stream and without any host synchronisation:
    ``b200fp4_moe_ep_dispatch`` ((route +) count, publish counts, wait, quantise own tokens, place the rows at the
    expert owners), ``b200fp4_moe_ep_compute`` (wait, FC1, FC2 whose epilogue sends every output row home),
    ``b200fp4_moe_ep_combine`` (wait, weighted sum).  The exchange buffer comes from
    ``torch.distributed._symmetric_memory``.  Shapes are fixed at construction: every rank passes
    ``tokens_local`` tokens per call.

    ``return_rows``: how FC2's output travels back to the rank that owns the token.  ``"per_slot"``: FC2's
    epilogue stores every (token, slot) row into the owner's buffer and the owner sums a token's k rows -- the
    arithmetic of the single-GPU operator, bit for bit.  ``"per_rank"``: FC2 keeps its rows, a second
    kernel on the expert's GPU sums the rows of each (source rank, token) with their routing weights (f32, slot
    order, one bf16 rounding) and sends ONE row per (token, serving rank); the owner adds those in rank order.
    A token's k experts sit on at most ``world`` ranks, so 75 / 55 / 34 % fewer bytes cross NVLink at 2 / 4 / 8
    ranks (top-8), at the price of bf16 roundings of the per-rank partial sums.  ``"auto"`` (default) takes
    ``"per_rank"`` when the group routes at least 4096 (token, slot) rows per step and ``"per_slot"`` below that
    (decode steps are latency-bound: the extra kernel costs more than the bytes save; measured on 2 GPUs: prefill
    205 -> 182 us, 64-token decode 503 -> 532 us).

    Every cross-rank wait inside the kernels gives up after ``wait_timeout_ms`` and records bit 16 in the device
    status word; ``forward(..., check=True)`` (or ``raise_if_failed()`` at a sync point of the caller)
    synchronises and raises.  After such a failure the group must call ``reset()`` together.
    """

    def __init__(self, num_experts: int, top_k: int, tokens_local: int, hidden: int, intermediate: int,
                 group: Optional[dist.ProcessGroup] = None, device: Optional[torch.device] = None,
                 wait_timeout_ms: float = 2000.0, return_rows: str = "auto"):
        import ctypes

        import torch.distributed._symmetric_memory as symm_mem

        from . import _lib
        self._lib = _lib
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.num_experts, self.top_k = num_experts, top_k
        self.tokens_local, self.hidden, self.inter = tokens_local, hidden, intermediate
        self.expert_lo, self.local_experts = shard_experts(num_experts, self.world, self.rank)
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.wait_timeout_ms = float(wait_timeout_ms)
        if return_rows not in ("auto", "per_rank", "per_slot"):
            raise ValueError("return_rows must be 'auto', 'per_rank' or 'per_slot'")
        if return_rows == "auto":
            return_rows = "per_rank" if tokens_local * self.world * top_k >= 4096 and top_k <= 32 else "per_slot"
        self.return_rows = return_rows
        self._mode = 1 if return_rows == "per_rank" else 0
        self._shape = (tokens_local, hidden, intermediate, self.local_experts, top_k)
        nbytes = int(_lib.lib.b200fp4_moe_ep_buffer_bytes(*self._shape, self.world))
        if nbytes == 0:
            raise ValueError("bad expert-parallel MoE shape")
        self.buffer = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
        self.handle = symm_mem.rendezvous(self.buffer, self.group)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self._peer_array = (ctypes.c_void_p * self.world)(*ptrs)
        self._own_ptr = ptrs[self.rank]
        self.reset()

    def reset(self) -> None:
        """Clear signals, counters and the abort mark (collective: every rank of the group calls it)."""
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)
        with self._lib.on_device(self.device):
            self._lib.check(self._lib.lib.b200fp4_moe_ep_reset(self._own_ptr, *self._shape, self.world,
                                                               self._lib.current_stream_ptr(self.device)))
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)

    def raise_if_failed(self) -> None:
        """Synchronise the current stream and raise if a kernel recorded an expired wait."""
        self._lib.raise_on_device_status(self.device)

    def forward(self, x: torch.Tensor, ids: Optional[torch.Tensor], scales: Optional[torch.Tensor], weights: dict,
                out: Optional[torch.Tensor] = None, router_logits: Optional[torch.Tensor] = None,
                renormalize: bool = True, check: bool = False) -> torch.Tensor:
        """x bf16 [tokens_local, H] and either (ids int32, scales f32) [tokens_local, k] with global expert ids, or
        ``router_logits`` f32 [tokens_local, num_experts] to route inside the dispatch kernel."""
        from .moe import _on_device, _sf_storage
        lib, chk = self._lib.lib, self._lib.check
        t, h = x.shape
        if (t, h) != (self.tokens_local, self.hidden) or x.dtype != torch.bfloat16 or not x.is_contiguous():
            raise ValueError(f"x must be contiguous bfloat16 [{self.tokens_local}, {self.hidden}]")
        _on_device(self.device, x=x, ids=ids, scales=scales, out=out, router_logits=router_logits,
                   **{f"weights[{k!r}]": v for k, v in weights.items()})
        if router_logits is None:
            if ids is None or scales is None:
                raise ValueError("ids and scales are required without router_logits")
            if ids.dtype != torch.int32 or tuple(ids.shape) != (t, self.top_k) or not ids.is_contiguous():
                raise ValueError("ids must be contiguous int32 [tokens, top_k]")
            if scales.dtype != torch.float32 or tuple(scales.shape) != (t, self.top_k) or not scales.is_contiguous():
                raise ValueError("scales must be contiguous float32 [tokens, top_k]")
        elif (router_logits.dtype != torch.float32 or tuple(router_logits.shape) != (t, self.num_experts)
              or not router_logits.is_contiguous()):
            raise ValueError(f"router_logits must be contiguous float32 [{t}, {self.num_experts}]")
        w1 = weights["w1"].view(torch.uint8)
        w2 = weights["w2"].view(torch.uint8)
        if tuple(w1.shape) != (self.local_experts, 2 * self.inter, h // 2) or not w1.is_contiguous():
            raise ValueError(f"weights['w1'] must be contiguous [{self.local_experts}, {2 * self.inter}, {h // 2}]")
        if tuple(w2.shape) != (self.local_experts, h, self.inter // 2) or not w2.is_contiguous():
            raise ValueError(f"weights['w2'] must be contiguous [{self.local_experts}, {h}, {self.inter // 2}]")
        s1 = _sf_storage(weights["w1_sf"], self.local_experts, 2 * self.inter, h, "w1_sf")
        s2 = _sf_storage(weights["w2_sf"], self.local_experts, h, self.inter, "w2_sf")
        if out is None:
            out = torch.empty(t, h, dtype=torch.bfloat16, device=x.device)
        elif tuple(out.shape) != (t, h) or out.dtype != torch.bfloat16 or not out.is_contiguous():
            raise ValueError("out must be contiguous bfloat16 [tokens, hidden]")
        stream = self._lib.current_stream_ptr(x.device)
        ms = self.wait_timeout_ms
        routed = router_logits is not None
        with self._lib.on_device(x.device):
            chk(lib.b200fp4_moe_ep_dispatch(
                x.data_ptr(), None if routed else ids.data_ptr(), None if routed else scales.data_ptr(),
                self._lib.ptr(router_logits), 1 if renormalize else 0, self._peer_array, self.rank, self.world,
                *self._shape, self._mode, ms, stream))
            chk(lib.b200fp4_moe_ep_compute(
                self._peer_array, self.rank, self.world, w1.data_ptr(), s1.data_ptr(), w2.data_ptr(), s2.data_ptr(),
                self._lib.ptr(weights.get("w1_alpha")), self._lib.ptr(weights.get("w2_alpha")),
                self._lib.ptr(weights.get("fc2_input_scale")), *self._shape, self._mode, ms, stream))
            chk(lib.b200fp4_moe_ep_combine(
                self._peer_array, self.rank, self.world, None if routed else ids.data_ptr(),
                None if routed else scales.data_ptr(), out.data_ptr(), *self._shape, self._mode, ms, stream))
        if check:
            self.raise_if_failed()
        return out

    def last_routing(self) -> Tuple[torch.Tensor, torch.Tensor]:
        """(ids, scales) that the last ``forward(..., router_logits=...)`` computed on the GPU."""
        ids = torch.empty(self.tokens_local, self.top_k, dtype=torch.int32, device=self.device)
        w = torch.empty(self.tokens_local, self.top_k, dtype=torch.float32, device=self.device)
        with self._lib.on_device(self.device):
            self._lib.check(self._lib.lib.b200fp4_moe_ep_routing(
                self._own_ptr, ids.data_ptr(), w.data_ptr(), *self._shape, self.world,
                self._lib.current_stream_ptr(self.device)))
        return ids, w
