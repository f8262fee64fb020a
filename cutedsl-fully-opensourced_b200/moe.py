"""Drop-in ``b12x_fused_moe`` (NVFP4 weights, bf16 tokens), the router, the wrapper object and the weight packer.

Call signature of flashinfer's ``fused_moe.cute_dsl.b12x_moe.b12x_fused_moe`` as
the reference calls it (tests/python/test_flashinfer_b12x_verbatim.py:99-116,
tools/perf/bench_flashinfer_b12x.py:77-81).  One call = a fixed sequence of CUDA
kernels on the current stream inside ``b200fp4_moe_fused``: (route +) count,
quantise + place, grouped FC1 with SwiGLU and re-quantisation, grouped FC2,
weighted combine.  Scratch memory comes from ``workspace=`` or from a
``B12xMoEWrapper`` (allocated once); without either, a per-device buffer that
only grows is used.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib
from .layout import pack_e2m1, six_mode_to_storage, swizzle_sf

_WORKSPACES = {}


def moe_workspace_bytes(tokens: int, hidden: int, intermediate: int, local_experts: int, top_k: int) -> int:
    return int(_lib.lib.b200fp4_moe_workspace_bytes(tokens, hidden, intermediate, local_experts, top_k))


def _workspace(device, nbytes: int) -> torch.Tensor:
    key = (device.type, device.index)
    ws = _WORKSPACES.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _WORKSPACES[key] = ws
    return ws


def _on_device(device, **tensors) -> None:
    """Every tensor argument must live on the GPU that runs the kernels: a CPU tensor or one on another GPU would
    hand the kernels an address they cannot read."""
    for name, t in tensors.items():
        if t is None:
            continue
        if not isinstance(t, torch.Tensor) or not t.is_cuda or t.device != device:
            where = getattr(t, "device", type(t).__name__)
            raise ValueError(f"{name} must be a CUDA tensor on {device} (got {where})")


def _sf_storage(sf: torch.Tensor, experts: int, rows: int, k: int, name: str) -> torch.Tensor:
    """Accept the six-mode view (32,4,m_tiles,4,k_tiles,E) or already-flat tiled bytes [E, tiles*512]."""
    need = -(-rows // 128) * -(-(k // 16) // 4) * 512
    if sf.dim() == 6:
        st = six_mode_to_storage(sf)
    else:
        st = sf.contiguous().view(torch.uint8).reshape(experts, -1)
    if st.shape[0] != experts or st.shape[1] != need:
        raise ValueError(f"{name}: expected {experts} x {need} scale bytes in 128x4 tiles, got {tuple(st.shape)}")
    return st


def topk_route(router_logits: torch.Tensor, top_k: int, renormalize: bool = True):
    """softmax -> top-k -> (renormalised) weights on the GPU; returns (ids int32, weights float32)."""
    if not router_logits.is_cuda or router_logits.dtype != torch.float32 or router_logits.dim() != 2:
        raise ValueError("router_logits must be a float32 CUDA tensor [tokens, experts]")
    logits = router_logits.contiguous()
    t, e = logits.shape
    ids = torch.empty(t, top_k, dtype=torch.int32, device=logits.device)
    w = torch.empty(t, top_k, dtype=torch.float32, device=logits.device)
    with _lib.on_device(logits.device):
        _lib.check(_lib.lib.b200fp4_topk_route(logits.data_ptr(), ids.data_ptr(), w.data_ptr(), t, e, top_k,
                                               1 if renormalize else 0, _lib.current_stream_ptr(logits.device)))
    return ids, w


def b12x_fused_moe(
    x: torch.Tensor,
    w1_weight: torch.Tensor,
    w1_weight_sf: torch.Tensor,
    w2_weight: torch.Tensor,
    w2_weight_sf: torch.Tensor,
    token_selected_experts: Optional[torch.Tensor],
    token_final_scales: Optional[torch.Tensor],
    num_experts: int,
    top_k: int,
    *,
    w1_alpha: Optional[torch.Tensor] = None,
    w2_alpha: Optional[torch.Tensor] = None,
    fc2_input_scale: Optional[torch.Tensor] = None,
    quant_mode: str = "nvfp4",
    num_local_experts: Optional[int] = None,
    local_expert_offset: int = 0,
    output: Optional[torch.Tensor] = None,
    output_dtype: torch.dtype = torch.bfloat16,
    activation: str = "silu",
    activation_precision: Optional[str] = None,
    accumulate: bool = False,
    workspace: Optional[torch.Tensor] = None,
    slot_rows_dtype: Optional[torch.dtype] = None,
    router_logits: Optional[torch.Tensor] = None,
    renormalize: bool = True,
) -> torch.Tensor:
    """out[t] = sum_j scale[t,j] * FC2_e(quant(silu(gate) * up)),  [up|gate] = FC1_e(quant(x[t])), e = expert[t,j].

    ``w1_weight`` [E_local, 2I, H/2] uint8 holds the up rows first, then the gate rows; scale tensors are the
    six-mode e4m3 views the reference builds.  With ``num_local_experts`` / ``local_expert_offset`` only the experts
    of this rank are computed and other slots contribute zero.

    ``router_logits`` (float32 [tokens, num_experts]): route on the GPU inside the operator's first kernel instead
    of taking ids and scales.  ``token_selected_experts`` / ``token_final_scales`` may then be ``None`` or
    pre-allocated tensors that receive the routing.

    ``slot_rows_dtype``: storage of the k per-expert output rows of a token between FC2 and the weighted sum.
    The sum itself always runs in float32 in slot order and is rounded once.  ``torch.bfloat16`` (default for a
    bfloat16 output) rounds every expert's row to the activation dtype first -- still finer than the reference
    kernel, which scatter-adds into the bfloat16 output -- and nearly halves the time of FC2 and of the sum;
    ``torch.float32`` (always used for a float32 output) keeps the rows exact."""
    if quant_mode != "nvfp4" or activation_precision not in (None, "fp4", "nvfp4"):
        raise NotImplementedError("only NVFP4 weights with NVFP4 activations are implemented")
    if activation not in ("silu", "swiglu"):
        raise NotImplementedError(f"activation {activation!r}: only silu (SwiGLU) is implemented")
    if output_dtype not in (torch.bfloat16, torch.float32) or x.dtype != torch.bfloat16:
        raise NotImplementedError("tokens must be bfloat16 and the output bfloat16 (or float32 partial sums)")
    if not x.is_cuda:
        raise ValueError("x must be a CUDA tensor (there is no CPU implementation)")
    if x.dim() != 2 or not x.is_contiguous():
        raise ValueError("x must be contiguous [tokens, hidden]")
    tokens, hidden = x.shape
    dev = x.device
    local = num_experts if num_local_experts is None else num_local_experts
    ids, scales = token_selected_experts, token_final_scales
    _on_device(dev, w1_weight=w1_weight, w1_weight_sf=w1_weight_sf, w2_weight=w2_weight, w2_weight_sf=w2_weight_sf,
               token_selected_experts=ids, token_final_scales=scales, w1_alpha=w1_alpha, w2_alpha=w2_alpha,
               fc2_input_scale=fc2_input_scale, output=output, workspace=workspace, router_logits=router_logits)
    w1 = w1_weight.view(torch.uint8)
    w2 = w2_weight.view(torch.uint8)
    if w1.dim() != 3 or w1.shape[0] != local or w1.shape[2] * 2 != hidden or not w1.is_contiguous():
        raise ValueError(f"w1_weight must be contiguous [{local}, 2*I, {hidden // 2}]")
    inter = w1.shape[1] // 2
    if tuple(w2.shape) != (local, hidden, inter // 2) or not w2.is_contiguous():
        raise ValueError(f"w2_weight must be contiguous [{local}, {hidden}, {inter // 2}]")
    if router_logits is not None:
        if (router_logits.dtype != torch.float32 or tuple(router_logits.shape) != (tokens, num_experts)
                or not router_logits.is_contiguous()):
            raise ValueError(f"router_logits must be contiguous float32 [{tokens}, {num_experts}]")
        if ids is None:
            ids = torch.empty(tokens, top_k, dtype=torch.int32, device=dev)
        if scales is None:
            scales = torch.empty(tokens, top_k, dtype=torch.float32, device=dev)
    elif ids is None or scales is None:
        raise ValueError("token_selected_experts and token_final_scales are required without router_logits")
    if ids.dtype != torch.int32 or tuple(ids.shape) != (tokens, top_k) or not ids.is_contiguous():
        raise ValueError("token_selected_experts must be contiguous int32 [tokens, top_k]")
    if scales.dtype != torch.float32 or tuple(scales.shape) != (tokens, top_k) or not scales.is_contiguous():
        raise ValueError("token_final_scales must be contiguous float32 [tokens, top_k]")
    s1 = _sf_storage(w1_weight_sf, local, 2 * inter, hidden, "w1_weight_sf")
    s2 = _sf_storage(w2_weight_sf, local, hidden, inter, "w2_weight_sf")
    for name, a in (("w1_alpha", w1_alpha), ("w2_alpha", w2_alpha)):
        if a is not None and (a.dtype != torch.float32 or a.numel() != local or not a.is_contiguous()):
            raise ValueError(f"{name} must be float32 [{local}]")
    if fc2_input_scale is not None and (fc2_input_scale.dtype != torch.float32 or fc2_input_scale.numel() != 1):
        raise ValueError("fc2_input_scale must be one float32")
    if output is None:
        output = torch.empty(tokens, hidden, dtype=output_dtype, device=dev)
        if accumulate:
            output.zero_()
    elif (tuple(output.shape) != (tokens, hidden) or output.dtype not in (torch.bfloat16, torch.float32)
          or not output.is_contiguous()):
        raise ValueError("output must be contiguous bfloat16 or float32 [tokens, hidden]")
    if slot_rows_dtype is None:
        slot_rows_dtype = torch.float32 if output.dtype == torch.float32 else torch.bfloat16
    if slot_rows_dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("slot_rows_dtype must be torch.bfloat16 or torch.float32")
    if output.dtype == torch.float32 and slot_rows_dtype != torch.float32:
        raise NotImplementedError("a float32 output keeps float32 per-slot rows")
    if tokens == 0:
        return output
    need = moe_workspace_bytes(tokens, hidden, inter, local, top_k)
    ws = _workspace(dev, need) if workspace is None else workspace
    if ws.numel() * ws.element_size() < need:
        raise ValueError(f"workspace too small: {need} bytes needed")
    out_code = 2 if output.dtype == torch.float32 else (3 if slot_rows_dtype == torch.bfloat16 else 1)
    tail = (_lib.ptr(w1_alpha), _lib.ptr(w2_alpha), _lib.ptr(fc2_input_scale), output.data_ptr(), tokens, hidden,
            inter, local, top_k, int(local_expert_offset), 1 if accumulate else 0, out_code, ws.data_ptr(),
            ws.numel() * ws.element_size(), _lib.current_stream_ptr(dev))
    with _lib.on_device(dev):
        if router_logits is None:
            _lib.check(_lib.lib.b200fp4_moe_fused(x.data_ptr(), w1.data_ptr(), s1.data_ptr(), w2.data_ptr(),
                                                  s2.data_ptr(), ids.data_ptr(), scales.data_ptr(), *tail))
        else:
            _lib.check(_lib.lib.b200fp4_moe_fused_routed(
                x.data_ptr(), router_logits.data_ptr(), num_experts, 1 if renormalize else 0, w1.data_ptr(),
                s1.data_ptr(), w2.data_ptr(), s2.data_ptr(), ids.data_ptr(), scales.data_ptr(), *tail))
    return output


class B12xMoEWrapper:
    """The wrapper object upstream callers build once and call every step (flashinfer's ``B12xMoEWrapper``; the
    reference's bench calls the functional form, tools/perf/bench_flashinfer_b12x.py:70-81).

    Construction fixes the problem shape and allocates the workspace and the routing buffers for ``max_num_tokens``
    once, so ``run`` allocates nothing (and can be captured in a CUDA graph by the caller).  ``run`` accepts either
    the routing (ids + scales) or ``router_logits``.
    """

    def __init__(self, num_experts: int, top_k: int, hidden_size: int, intermediate_size: int, *,
                 max_num_tokens: int, num_local_experts: Optional[int] = None, local_expert_offset: int = 0,
                 output_dtype: torch.dtype = torch.bfloat16, slot_rows_dtype: Optional[torch.dtype] = None,
                 device: Optional[torch.device] = None, quant_mode: str = "nvfp4", activation: str = "silu"):
        if quant_mode != "nvfp4" or activation not in ("silu", "swiglu"):
            raise NotImplementedError("only NVFP4 with SwiGLU is implemented")
        self.num_experts, self.top_k = num_experts, top_k
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.num_local_experts = num_experts if num_local_experts is None else num_local_experts
        self.local_expert_offset = local_expert_offset
        self.max_num_tokens = max_num_tokens
        self.output_dtype, self.slot_rows_dtype = output_dtype, slot_rows_dtype
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        need = max(moe_workspace_bytes(t, hidden_size, intermediate_size, self.num_local_experts, top_k)
                   for t in {1, min(32, max_num_tokens), min(33, max_num_tokens), max_num_tokens})
        if need == 0:
            raise ValueError("bad MoE shape")
        self.workspace = torch.empty(need, dtype=torch.uint8, device=self.device)
        self._ids = torch.empty(max_num_tokens, top_k, dtype=torch.int32, device=self.device)
        self._scales = torch.empty(max_num_tokens, top_k, dtype=torch.float32, device=self.device)

    def run(self, x, w1_weight, w1_weight_sf, w2_weight, w2_weight_sf, token_selected_experts=None,
            token_final_scales=None, *, router_logits=None, w1_alpha=None, w2_alpha=None, fc2_input_scale=None,
            output=None, renormalize: bool = True):
        tokens = x.shape[0]
        if tokens > self.max_num_tokens:
            raise ValueError(f"{tokens} tokens exceed max_num_tokens={self.max_num_tokens}")
        if router_logits is not None and token_selected_experts is None:
            token_selected_experts, token_final_scales = self._ids[:tokens], self._scales[:tokens]
        if output is None:
            output = torch.empty(tokens, self.hidden_size, dtype=self.output_dtype, device=x.device)
        return b12x_fused_moe(
            x, w1_weight, w1_weight_sf, w2_weight, w2_weight_sf, token_selected_experts, token_final_scales,
            self.num_experts, self.top_k, w1_alpha=w1_alpha, w2_alpha=w2_alpha, fc2_input_scale=fc2_input_scale,
            num_local_experts=self.num_local_experts, local_expert_offset=self.local_expert_offset, output=output,
            output_dtype=self.output_dtype, workspace=self.workspace, slot_rows_dtype=self.slot_rows_dtype,
            router_logits=router_logits, renormalize=renormalize)

    def last_routing(self, tokens: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """(ids, scales) written by the last ``run(..., router_logits=...)`` that did not pass its own buffers."""
        return self._ids[:tokens], self._scales[:tokens]


def pack_moe_weights(w1: torch.Tensor, w2: torch.Tensor, *, fc2_input_scale: float = 1.0) -> dict:
    """Checkpoint-side packer: bf16 / f32 expert weights -> what ``b12x_fused_moe`` consumes.

    ``w1`` [E, 2I, H] (up rows, then gate rows) and ``w2`` [E, H, I] are quantised per expert to NVFP4 with a
    per-expert global scale ``gs_e = 448 * 6 / amax(|W_e|)`` (the recipe of
    tests/python/test_flashinfer_norm_verbatim.py:58-68 applied per expert), packed two codes per byte (lower K
    index in the low nibble), and their e4m3 block scales are laid out in the six-mode MMA view
    ``(32, 4, m_tiles, 4, k_tiles, E)`` (tests/python/test_flashinfer_b12x_verbatim.py:68-89).  The reciprocal
    global scales are returned as ``w1_alpha`` / ``w2_alpha`` (``w2_alpha`` also carries 1 / fc2_input_scale, the
    operator's convention for undoing the activation quantiser's global scale).  Runs on whatever device the
    weights are on; not a hot path."""
    from .gemm import quantize_operand_batched
    if w1.dim() != 3 or w2.dim() != 3 or w1.shape[0] != w2.shape[0]:
        raise ValueError("w1 must be [E, 2I, H] and w2 [E, H, I]")
    e, two_i, h = w1.shape
    if tuple(w2.shape) != (e, h, two_i // 2) or two_i % 256 or h % 64:
        raise ValueError("shapes must be w1 [E, 2I, H], w2 [E, H, I] with I a multiple of 128 and H of 64")
    out = {}
    for name, w, extra in (("w1", w1, 1.0), ("w2", w2, float(fc2_input_scale))):
        codes, sf_bits, gs = quantize_operand_batched(w)
        rows, k = w.shape[1], w.shape[2]
        storage = swizzle_sf(sf_bits).view(e, -(-rows // 128), -(-(k // 16) // 4), 32, 4, 4)
        out[f"{name}_weight"] = pack_e2m1(codes)
        out[f"{name}_weight_sf"] = storage.view(torch.float8_e4m3fn).permute(3, 4, 1, 5, 2, 0)
        out[f"{name}_alpha"] = (1.0 / (gs * extra)).to(torch.float32).contiguous()
    out["fc2_input_scale"] = torch.tensor([float(fc2_input_scale)], dtype=torch.float32, device=w1.device)
    return out
