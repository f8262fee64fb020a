"""One process per GPU over ``torch.distributed``: how the hot path is partitioned.

* RMSNorm-quant and the GEMM shard by rows (``shard_rows``): rows are independent, every rank calls the
  single-GPU operator on its block and nothing is communicated.  Blocks are multiples of 128 rows so that a rank
  owns whole 128x4 scale-factor tiles.
* The MoE shards by expert (``shard_experts``, weights never move) and by token (each rank owns a slice of the
  batch).  ``ExpertParallelMoE`` gathers the tokens and their routing over NCCL, runs the local experts of every
  token with ``b12x_fused_moe(num_local_experts=, local_expert_offset=, output_dtype=float32)`` and
  reduce-scatters the f32 partial outputs, so each rank ends with the finished rows of its own tokens.  With
  top_k >= world size nearly every token visits every rank, so this moves the same bytes as a dispatch /
  combine all-to-all while letting NVSwitch do the reduction.

  ``PeerExpertParallelMoE`` is the same partition with the exchange inside the kernels: every rank publishes its
  quantised tokens in a buffer that the others address directly (NVLink peer loads over torch symmetric memory),
  expert owners pull the rows they need, and the combine kernel reads the output rows from wherever they were
  computed.  Two stream-ordered cross-rank barriers per step replace the collectives.

The reference itself is single-GPU (it has no collective anywhere); this layer is new.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist


def shard_rows(rows: int, world: int, rank: int, multiple: int = 128) -> Tuple[int, int]:
    """Contiguous row block of ``rank``: (start, count).  Blocks are multiples of ``multiple`` except that the
    last ranks may get fewer (or zero) rows when ``rows`` runs out."""
    if world < 1 or not 0 <= rank < world or rows < 0:
        raise ValueError("bad rows / world / rank")
    units = -(-rows // multiple)
    per, extra = divmod(units, world)
    start_u = rank * per + min(rank, extra)
    count_u = per + (1 if rank < extra else 0)
    start = min(rows, start_u * multiple)
    end = min(rows, (start_u + count_u) * multiple)
    return start, end - start


def shard_experts(num_experts: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous expert range of ``rank``: (first expert, number of local experts)."""
    if num_experts % world != 0:
        raise ValueError(f"{num_experts} experts do not divide over {world} ranks")
    per = num_experts // world
    return rank * per, per


class ExpertParallelMoE:
    """Expert-parallel fused MoE over a process group.

    ``local_moe`` computes ``f32 [tokens, hidden]`` partial outputs of this rank's experts for ANY token set; by
    default it is the CUDA operator of this package.  (Tests on CPU ranks inject a stand-in here to exercise the
    gather / reduce-scatter bookkeeping with the gloo backend.)
    """

    def __init__(self, num_experts: int, top_k: int, group: Optional[dist.ProcessGroup] = None,
                 local_moe: Optional[Callable] = None):
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.num_experts, self.top_k = num_experts, top_k
        self.expert_lo, self.local_experts = shard_experts(num_experts, self.world, self.rank)
        self._local_moe = local_moe
        self._buffers = {}

    def _buf(self, name, shape, dtype, device):
        key = (name, tuple(shape), dtype)
        t = self._buffers.get(key)
        if t is None:
            t = torch.empty(shape, dtype=dtype, device=device)
            self._buffers[key] = t
        return t

    def _run_local(self, x_all, ids_all, w_all, weights, partial):
        if self._local_moe is not None:
            partial.copy_(self._local_moe(x_all, ids_all, w_all, self.expert_lo, self.local_experts))
            return
        from .moe import b12x_fused_moe
        b12x_fused_moe(x_all, weights["w1"], weights["w1_sf"], weights["w2"], weights["w2_sf"], ids_all, w_all,
                       self.num_experts, self.top_k, w1_alpha=weights.get("w1_alpha"),
                       w2_alpha=weights.get("w2_alpha"), fc2_input_scale=weights.get("fc2_input_scale"),
                       num_local_experts=self.local_experts, local_expert_offset=self.expert_lo,
                       output=partial, output_dtype=torch.float32)

    def forward(self, x: torch.Tensor, ids: torch.Tensor, scales: torch.Tensor, weights: Optional[dict] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x bf16 [t, H], ids int32 [t, k], scales f32 [t, k] of THIS rank's tokens (same t on every rank);
        ``weights`` holds this rank's experts.  Returns bf16 [t, H]."""
        t, h = x.shape
        w = self.world
        if w == 1:
            partial = self._buf("partial", (t, h), torch.float32, x.device)
            self._run_local(x, ids, scales, weights, partial)
            res = partial
        else:
            x_all = self._buf("x_all", (w * t, h), x.dtype, x.device)
            ids_all = self._buf("ids_all", (w * t, self.top_k), ids.dtype, x.device)
            w_all = self._buf("w_all", (w * t, self.top_k), scales.dtype, x.device)
            dist.all_gather_into_tensor(x_all, x.contiguous(), group=self.group)
            dist.all_gather_into_tensor(ids_all, ids.contiguous(), group=self.group)
            dist.all_gather_into_tensor(w_all, scales.contiguous(), group=self.group)
            partial = self._buf("partial", (w * t, h), torch.float32, x.device)
            self._run_local(x_all, ids_all, w_all, weights, partial)
            res = self._buf("mine", (t, h), torch.float32, x.device)
            dist.reduce_scatter_tensor(res, partial, op=dist.ReduceOp.SUM, group=self.group)
        if out is None:
            out = torch.empty(t, h, dtype=torch.bfloat16, device=x.device)
        out.copy_(res)
        return out


class PeerExpertParallelMoE:
    """Expert-parallel fused MoE whose dispatch and combine are peer-memory loads inside the kernels.

    Per step and rank: ``b200fp4_moe_ep_stage`` (quantise own tokens, publish), barrier,
    ``b200fp4_moe_ep_compute`` (gather rows of local experts from all ranks, FC1, FC2), barrier,
    ``b200fp4_moe_ep_combine`` (weighted sum of rows read from their owners).  The exchange buffer comes from
    ``torch.distributed._symmetric_memory``; the barriers are its signal-pad barrier on the current stream.
    Shapes are fixed at construction: every rank passes ``tokens_local`` tokens per call.
    """

    def __init__(self, num_experts: int, top_k: int, tokens_local: int, hidden: int, intermediate: int,
                 group: Optional[dist.ProcessGroup] = None, device: Optional[torch.device] = None):
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
        nbytes = int(_lib.lib.b200fp4_moe_ep_buffer_bytes(tokens_local, hidden, intermediate, self.local_experts, top_k,
                                                          self.world))
        if nbytes == 0:
            raise ValueError("bad expert-parallel MoE shape")
        self.buffer = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
        self.handle = symm_mem.rendezvous(self.buffer, self.group)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self._peer_array = (ctypes.c_void_p * self.world)(*ptrs)
        self._own_ptr = ptrs[self.rank]
        self.handle.barrier()

    def forward(self, x: torch.Tensor, ids: torch.Tensor, scales: torch.Tensor, weights: dict,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
        lib, chk = self._lib.lib, self._lib.check
        t, h = x.shape
        if (t, h) != (self.tokens_local, self.hidden) or x.dtype != torch.bfloat16 or not x.is_contiguous():
            raise ValueError(f"x must be contiguous bfloat16 [{self.tokens_local}, {self.hidden}]")
        if ids.dtype != torch.int32 or tuple(ids.shape) != (t, self.top_k) or not ids.is_contiguous():
            raise ValueError("ids must be contiguous int32 [tokens, top_k]")
        if scales.dtype != torch.float32 or tuple(scales.shape) != (t, self.top_k) or not scales.is_contiguous():
            raise ValueError("scales must be contiguous float32 [tokens, top_k]")
        from .moe import _sf_storage
        w1 = weights["w1"].view(torch.uint8)
        w2 = weights["w2"].view(torch.uint8)
        s1 = _sf_storage(weights["w1_sf"], self.local_experts, 2 * self.inter, h, "w1_sf")
        s2 = _sf_storage(weights["w2_sf"], self.local_experts, h, self.inter, "w2_sf")
        if out is None:
            out = torch.empty(t, h, dtype=torch.bfloat16, device=x.device)
        stream = self._lib.current_stream_ptr(x.device)
        args = (t, h, self.inter, self.local_experts, self.top_k)
        with torch.cuda.device(x.device):
            chk(lib.b200fp4_moe_ep_stage(x.data_ptr(), ids.data_ptr(), self._own_ptr, *args, self.world, stream))
            self.handle.barrier()
            chk(lib.b200fp4_moe_ep_compute(
                self._peer_array, self.rank, self.world, w1.data_ptr(), s1.data_ptr(), w2.data_ptr(), s2.data_ptr(),
                self._lib.ptr(weights.get("w1_alpha")), self._lib.ptr(weights.get("w2_alpha")),
                self._lib.ptr(weights.get("fc2_input_scale")), *args, stream))
            self.handle.barrier()
            chk(lib.b200fp4_moe_ep_combine(self._peer_array, self.rank, self.world, ids.data_ptr(), scales.data_ptr(),
                                           out.data_ptr(), *args, stream))
        return out
