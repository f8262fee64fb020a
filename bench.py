#!/usr/bin/env python3
"""Benchmark of the NVFP4 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--parts a,b,...]

One invocation times every part of the metric "NVFP4 GEMM TFLOP/s; norm-quant HBM GB/s; MoE tokens/s" on
seeded synthetic inputs that are already resident in HBM, and prints ONE JSON line:

* headline (``metric`` / ``value``): fused NVFP4 MoE, prefill configuration (4096 tokens in total, hidden 2048,
  128 experts, top-8, intermediate 768), tokens/s.  With N > 1 (one process per GPU under torch.distributed.run)
  the same 4096 tokens and 128 experts are split over the ranks (``"scaling": "strong"``) and dispatch / combine
  cross NVLink inside the kernels.
* ``parts``: ``norm_quant`` (add_rmsnorm_fp4quant bf16 [8192, 7168]; rows split over the ranks), ``gemm_8192``
  (M = N = K = 8192; rows of A / C split), ``gemm_m1024`` / ``gemm_m128`` (the M sweep, one GPU), ``moe_decode_t64`` /
  ``_t8`` / ``_t1`` (hidden 7168, 256 experts, top-8, intermediate 2048, 1 % of rows forced onto one hot expert;
  expert-parallel with N > 1 where the batch divides).  Each part carries its own value, roofline, end-to-end
  number, step statistics and (N = 1) CPU baseline.

A "step" is one pass of a part over its batch.  Steps are timed one by one with CUDA events on the launching
stream (median / p10 / p90 / min are reported; the value uses the mean), after >= 3 warm-up steps, as the
maximum over ranks.  ``e2e`` is the same step through the public Python API with host buffers: the host->device
copy of the inputs and the device->host copy of the result are inside the timed region (two buffer sets, so that
the copies of neighbouring steps overlap the kernels of the current one, as in a serving loop).  ``roofline`` compares
algorithmic bytes (or flops) per step with the measured peaks of MEASURED_PEAKS.json.  ``cpu_baseline`` is the
oracle port of the reference's CPU golden path timed on the host cores over a bounded sample.
``--impl reference`` prints that CPU arm alone, for the same parts.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HBM_FALLBACK_GBS = 6650.0      # earlier measurement on this pool, used only without MEASURED_PEAKS.json
FP4_NOMINAL_TFLOPS = 9000.0    # dense FP4 peak of a B200 (nominal; MEASURED_PEAKS.json has no FP4 figure)
L2_BYTES = 126 << 20


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d.get("bf16_tflops", 0.0)),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", 0.0)), "source": "measured"}
    except Exception:
        return {"hbm_gbs": HBM_FALLBACK_GBS, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
                "source": "fallback"}


def host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def pct(xs, q):
    s = sorted(xs)
    if not s:
        return float("nan")
    i = min(len(s) - 1, max(0, int(round(q * (len(s) - 1)))))
    return s[i]


def stats_us(ms):
    return {"median": round(1e3 * statistics.median(ms), 2), "p10": round(1e3 * pct(ms, 0.1), 2),
            "p90": round(1e3 * pct(ms, 0.9), 2), "min": round(1e3 * min(ms), 2), "mean": round(1e3 * statistics.mean(ms), 2)}


# ---------------------------------------------------------------------------
# clocks during the timed region
# ---------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        threading.Thread(target=self._pump, daemon=True).start()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def window(self, t0: float, t1: float):
        """Summary of the samples taken between two wall-clock times (the sampler keeps running).  A sample reports
        the clocks of the moment it was taken, and a short timed region falls between two samples, so the window
        is widened by one sampling period on either side."""
        time.sleep(0.06)                     # let the samples of the region's end arrive
        sm, mx, reasons, power = [], [], set(), []
        for ts, line in list(self.lines):
            if ts < t0 - 0.03 or ts > t1 + 0.05:
                continue
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
                power.append(float(parts[3]))
            except ValueError:
                continue
            for name, val in zip(self.NAMES, parts[4:8]):
                if val.lower() == "active":
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "reasons": sorted(reasons), "samples": len(sm)}

    def stop(self):
        if self.proc is None:
            return
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()


# ---------------------------------------------------------------------------
# parts
# ---------------------------------------------------------------------------
class Part:
    """One workload of the metric.  `units_per_step` is what ALL ranks together process in a step (bytes, flops or
    tokens); `alg_bytes` / `alg_flops` are the algorithmic traffic / work of THIS rank's launch."""
    name = ""
    metric = ""
    unit = ""
    dtype = ""
    bound = "hbm"
    kernel = ""
    scaling = "strong"
    use_graph = False
    launches_per_step = 1
    flush = None

    def supported(self, world):
        return True

    def restore(self):
        if self.flush is not None:
            self.flush.zero_()

    def checks(self, pkg, world, rank):
        return None

    def free(self):
        for k in list(self.__dict__):
            if k not in ("rank", "world"):
                self.__dict__[k] = None


def _flush_buffer():
    import torch
    return torch.empty(256 << 20, dtype=torch.uint8, device="cuda")


class NormPart(Part):
    """add_rmsnorm_fp4quant, bf16 [8192, 7168] in total, weight 1 + 0.1 N(0,1), eps 1e-6, per-tensor global scale
    448*6/amax, scale factors in the 128x4 tiled layout.  Rows are split over the ranks (128-row multiples)."""
    name = "add_rmsnorm_fp4quant_bf16_8192x7168"
    metric = "norm-quant HBM GB/s"
    unit = "GB/s"
    dtype = "bf16"
    kernel = "norm_quant_kernel<bf16, add>"
    total_rows, hidden = 8192, 7168
    bytes_per_element = 2 + 2 + 2 + 0.5 + 0.0625      # x in, residual in+out, codes, scale bytes
    # DRAM bytes inside the kernel window per element, from an ncu capture of a 4096-row launch (reads equal the
    # algorithmic reads; most of the writes are still dirty in L2 when the kernel ends and drain later)
    traffic_per_element = (117496064 + 26109440) / (4096 * 7168)

    def __init__(self, rank, world):
        from cutedsl_fully_opensourced_b200_shard import shard_rows
        self.rank, self.world = rank, world
        self.row0, self.rows = shard_rows(self.total_rows, world, rank)
        self.alg_bytes = int(self.rows * self.hidden * self.bytes_per_element)
        self.units_per_step = float(self.total_rows * self.hidden * self.bytes_per_element)
        per_set = max(1, self.alg_bytes)
        self.sets = max(4, math.ceil(3 * L2_BYTES / per_set) + 1)
        # a rank's share of the rows takes less device time than an eager launch through Python costs on the host
        # once the rows are split over several GPUs: those launches are replayed from CUDA graphs (one per set)
        self.use_graph = self.rows <= 4096
        self.graph_variants = self.sets

    def config(self, world):
        return {"workload": self.name, "rows": self.total_rows, "rows_per_gpu": self.total_rows // world,
                "hidden": self.hidden, "sf_layout": "swizzled_128x4", "parallelism": f"rows split x{world}, no collective",
                "l2": "rotating sets of inputs and outputs whose bytes between two uses of a set exceed the 126 MB L2"}

    def setup(self, pkg):
        import torch
        from cutedsl_fully_opensourced_b200.layout import swizzled_sf_numel
        self.pkg = pkg
        g = torch.Generator(device="cuda").manual_seed(1000 + self.rank)
        self.w = (1 + 0.1 * torch.randn(self.hidden, device="cuda")).to(torch.bfloat16)
        self.xs, self.rs, self.ys, self.sfs = [], [], [], []
        for _ in range(self.sets):
            self.xs.append(torch.randn(self.rows, self.hidden, generator=g, device="cuda").to(torch.bfloat16))
            self.rs.append(torch.randn(self.rows, self.hidden, generator=g, device="cuda").to(torch.bfloat16))
            self.ys.append(torch.empty(self.rows, self.hidden // 2, dtype=torch.uint8, device="cuda"))
            self.sfs.append(torch.empty(swizzled_sf_numel(self.rows, self.hidden // 16), dtype=torch.uint8,
                                        device="cuda"))
        self.r0 = self.rs[0].clone()
        h = self.xs[0].float() + self.rs[0].float()
        normed = h.to(torch.bfloat16).float() * torch.rsqrt(h.square().mean(-1, keepdim=True) + 1e-6) * self.w.float()
        # RMSNorm output is scale-free, so this global scale stays valid while the residual streams keep
        # absorbing x over the steps
        self.gs = (448.0 * 6.0 / normed.abs().max()).reshape(1).float()
        del h, normed
        self.i = 0

    def step(self):
        j = self.i % self.sets
        self.i += 1
        self.pkg.add_rmsnorm_fp4quant(self.xs[j], self.rs[j], self.w, self.ys[j], self.sfs[j], global_scale=self.gs,
                                      eps=1e-6, block_size=16, is_sf_swizzled_layout=True)

    def setup_e2e(self):
        import torch
        self.hx = self.xs[0].cpu().pin_memory()
        self.hr = self.r0.cpu().pin_memory()
        self.hy = [torch.empty(self.ys[0].shape, dtype=torch.uint8).pin_memory() for _ in range(2)]
        self.hsf = [torch.empty(self.sfs[0].shape, dtype=torch.uint8).pin_memory() for _ in range(2)]
        self.hres = [torch.empty(self.rs[0].shape, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
        self.h2d = self.hx.numel() * 2 + self.hr.numel() * 2
        self.d2h = self.hy[0].numel() + self.hsf[0].numel() + self.hres[0].numel() * 2

    def e2e_h2d(self, b):
        self.xs[b].copy_(self.hx, non_blocking=True)
        self.rs[b].copy_(self.hr, non_blocking=True)

    def e2e_compute(self, b):
        self.pkg.add_rmsnorm_fp4quant(self.xs[b], self.rs[b], self.w, self.ys[b], self.sfs[b], global_scale=self.gs,
                                      eps=1e-6, block_size=16, is_sf_swizzled_layout=True)

    def e2e_d2h(self, b):
        self.hy[b].copy_(self.ys[b], non_blocking=True)
        self.hsf[b].copy_(self.sfs[b], non_blocking=True)
        self.hres[b].copy_(self.rs[b], non_blocking=True)

    def roofline_extra(self):
        return {"traffic": int(self.traffic_per_element * self.rows * self.hidden)}

    # CPU arm: the oracle port on all 8192 rows (a step costs ~0.1-0.2 s on 16 cores)
    def cpu_setup(self):
        import torch
        g = torch.Generator().manual_seed(1000)
        self.cx = torch.randn(self.total_rows, self.hidden, generator=g).to(torch.bfloat16)
        self.cr = torch.randn(self.total_rows, self.hidden, generator=g).to(torch.bfloat16)
        self.cw = (1 + 0.1 * torch.randn(self.hidden, generator=torch.Generator().manual_seed(7))).to(torch.bfloat16)

    def cpu_run(self, threads: int):
        import torch
        from concurrent.futures import ThreadPoolExecutor
        from oracle import nvfp4_oracle as O
        rows = self.total_rows
        chunk = max(16, rows // max(1, threads * 2))
        spans = [(i, min(rows, i + chunk)) for i in range(0, rows, chunk)]
        torch.set_num_threads(1)
        t0 = time.perf_counter()
        with ThreadPoolExecutor(max_workers=threads) as pool:
            list(pool.map(lambda s: O.add_rmsnorm_fp4quant_ref(self.cx[s[0]:s[1]], self.cr[s[0]:s[1]], self.cw, 1e-6,
                                                               500.0), spans))
        dt = time.perf_counter() - t0
        return rows * self.hidden * self.bytes_per_element / dt / 1e9, dt, \
            f"all {rows} rows x {self.hidden} (global scale fixed at 500), oracle port (numpy+torch), {threads} threads"


class GemmPart(Part):
    """NVFP4 block-scaled GEMM, N = K = 8192: A, B ~ N(0,1) quantised to e2m1 with e4m3 scale factors per
    16 K-elements and a per-tensor global scale, f32 accumulate, bf16 output, alpha = 1/(gs_A*gs_B)."""
    metric = "NVFP4 GEMM TFLOP/s"
    unit = "TFLOP/s"
    dtype = "nvfp4 (e2m1 x e2m1, ue4m3 scales, f32 accumulate)"
    tile_n = 0

    def __init__(self, rank, world, m=8192, n=8192, k=8192):
        from cutedsl_fully_opensourced_b200_shard import shard_rows
        self.rank, self.world = rank, world
        self.m_total, self.n, self.k = m, n, k
        _, self.m = shard_rows(m, world, rank)
        self.name = f"nvfp4_gemm_{m}x{n}x{k}_bf16out"
        self.units_per_step = 2.0 * m * n * k
        self.alg_flops = 2.0 * self.m * n * k
        self.alg_bytes = self.m * k // 2 + n * k // 2 + (self.m + n) * k // 16 + 2 * self.m * n
        # M = 128 streams the weights once: HBM-bound; the larger problems are bound by the tensor pipe
        self.bound = "hbm" if m <= 256 else "tensor"
        self.kernel = ("nvfp4_gemm_pair_kernel (256x256 tiles on CTA pairs) for a full wave of such tiles, else "
                       "nvfp4_gemm_kernel<256|128|64>")
        self.sets = max(3, math.ceil(2 * L2_BYTES / max(1, self.alg_bytes)) + 1)
        # the small problems take less device time than an eager launch through Python costs on the host: they
        # are replayed from CUDA graphs (one per operand set); the large ones are launched eagerly
        self.use_graph = m <= 2048
        self.graph_variants = self.sets

    def supported(self, world):
        return self.m_total % (128 * world) == 0

    def config(self, world):
        return {"workload": self.name, "m": self.m_total, "m_per_gpu": self.m_total // world, "n": self.n, "k": self.k,
                "parallelism": f"rows of A / C split x{world}, B replicated, no collective",
                "l2": "rotating operand sets whose bytes between two uses of a set exceed the 126 MB L2"}

    def setup(self, pkg):
        import torch
        self.pkg = pkg
        self.ops = []
        gb = torch.Generator(device="cuda").manual_seed(77)
        for i in range(self.sets):
            g = torch.Generator(device="cuda").manual_seed(100 * self.rank + i)
            a = torch.randn(self.m, self.k, generator=g, device="cuda")
            aq, sfa, gsa = pkg.gemm.quantize_operand(a)
            del a
            b = torch.randn(self.n, self.k, generator=gb, device="cuda")
            bq, sfb, gsb = pkg.gemm.quantize_operand(b)
            del b
            alpha = torch.tensor([1.0 / (gsa * gsb)], device="cuda")
            c = torch.empty(self.m, self.n, dtype=torch.bfloat16, device="cuda")
            self.ops.append((aq, bq, sfa, sfb, alpha, c))
        self.i = 0

    def step(self):
        aq, bq, sfa, sfb, alpha, c = self.ops[self.i % self.sets]
        self.i += 1
        self.pkg.nvfp4_gemm(aq, bq, sfa, sfb, alpha=alpha, out=c, tile_n=self.tile_n)

    def setup_e2e(self):
        import torch
        aq, bq, sfa, sfb, alpha, c = self.ops[0]
        self.h = [t.cpu().pin_memory() for t in (aq, bq, sfa, sfb)]
        self.hc = [torch.empty(c.shape, dtype=c.dtype).pin_memory() for _ in range(2)]
        self.h2d = sum(t.numel() * t.element_size() for t in self.h)
        self.d2h = self.hc[0].numel() * 2

    def e2e_h2d(self, b):
        for d, h in zip(self.ops[b][:4], self.h):
            d.copy_(h, non_blocking=True)

    def e2e_compute(self, b):
        aq, bq, sfa, sfb, alpha, c = self.ops[b]
        self.pkg.nvfp4_gemm(aq, bq, sfa, sfb, alpha=alpha, out=c, tile_n=self.tile_n)

    def e2e_d2h(self, b):
        self.hc[b].copy_(self.ops[b][5], non_blocking=True)

    def roofline_extra(self):
        return {"traffic": None}

    def cpu_setup(self):
        import torch
        from oracle import nvfp4_oracle as O
        m, n, k = min(self.m_total, 512), min(self.n, 1024), self.k
        g = torch.Generator().manual_seed(0)
        self.c_ac, self.c_sfa = O.quantize_nvfp4(torch.randn(m, k, generator=g).numpy(), 500.0)
        self.c_bc, self.c_sfb = O.quantize_nvfp4(torch.randn(n, k, generator=g).numpy(), 500.0)
        self.c_mnk = (m, n, k)

    def cpu_run(self, threads: int):
        import torch
        from oracle import nvfp4_oracle as O
        torch.set_num_threads(threads)
        m, n, k = self.c_mnk
        t0 = time.perf_counter()
        O.gemm_nvfp4_ref(self.c_ac, self.c_sfa, self.c_bc, self.c_sfb, alpha=1.0 / 250000.0)
        dt = time.perf_counter() - t0
        return 2.0 * m * n * k / dt / 1e12, dt, \
            (f"{m}x{n}x{k} block of the {self.m_total}x{self.n}x{self.k} problem: de-quantise + f32 matmul "
             f"(the demo's golden), {threads} threads")


class MoePart(Part):
    """Fused NVFP4 MoE.  prefill: 4096 tokens, hidden 2048, 128 experts, top-8, intermediate 768.
    decode: T tokens, hidden 7168, 256 experts, top-8, intermediate 2048, max(1, ceil(1 % of T)) rows forced onto
    expert 0.  Tokens bf16 ~ N(0,1); expert weights N(0, 0.02) quantised to NVFP4 per expert (global scale
    448*6/amax folded into w1_alpha / w2_alpha); router logits ~ N(0,1), softmax top-k renormalised.
    A step = router + fused MoE (the router runs inside the operator's first kernel)."""
    metric = "MoE tokens/s"
    unit = "tokens/s"
    dtype = "nvfp4 weights and activations, bf16 tokens, f32 accumulate"
    kernel = "whole step: count(+route), quantise+place, grouped FC1 (SwiGLU, re-quantise), grouped FC2, weighted sum"
    use_graph = True

    def __init__(self, rank, world, kind="prefill", tokens=None):
        self.rank, self.world, self.kind = rank, world, kind
        if kind == "prefill":
            self.tokens, self.hidden, self.experts, self.top_k, self.inter = tokens or 4096, 2048, 128, 8, 768
        else:
            self.tokens, self.hidden, self.experts, self.top_k, self.inter = tokens or 64, 7168, 256, 8, 2048
        self.name = f"moe_{kind}_T{self.tokens}_H{self.hidden}_E{self.experts}_k{self.top_k}_I{self.inter}"
        self.local_tokens = self.tokens // max(1, world)
        self.local_experts = self.experts // max(1, world)
        self.expert_lo = rank * self.local_experts
        self.units_per_step = float(self.tokens)
        self.expert_bytes = 3 * self.hidden * self.inter // 2 + 3 * self.hidden * self.inter // 16
        # kernels of this library per step: count(+route), place, FC1, FC2, sum; few slots: prepare(+route), quantise,
        # FC1, FC2, sum; expert-parallel: the same five, plus the pre-sum kernel with the per-rank return (set in setup)
        self.launches_per_step = 5

    def supported(self, world):
        return self.tokens % world == 0 and self.experts % world == 0 and self.tokens >= world

    def config(self, world):
        return {"workload": self.name, "tokens": self.tokens, "tokens_per_gpu": self.tokens // world,
                "hidden": self.hidden, "experts": self.experts, "experts_per_gpu": self.experts // world,
                "top_k": self.top_k, "intermediate": self.inter, "slot_rows": "bf16",
                "return_rows": ("n/a" if world == 1 else getattr(getattr(self, "ep", None), "return_rows",
                                                                  os.environ.get("B200FP4_EP_RETURN", "auto"))),
                "parallelism": ("single GPU" if world == 1 else
                                f"experts x{world}, tokens x{world}; dispatch / combine as NVLink peer stores inside "
                                "the kernels, three bounded in-kernel signals per step (no NCCL call in a step)"),
                "l2": "a 256 MB buffer is rewritten (untimed) between steps to flush the 126 MB L2"}

    def _expert_weights(self, pkg, lo, n):
        """NVFP4 weights of experts [lo, lo+n): every expert is generated from its own seed, so any rank can
        rebuild any expert."""
        import torch
        from cutedsl_fully_opensourced_b200.layout import swizzled_sf_numel
        h, i = self.hidden, self.inter
        out = {}
        for name, rows, k, seed in (("w1", 2 * i, h, 11), ("w2", h, i, 12)):
            codes = torch.empty(n, rows, k // 2, dtype=torch.uint8, device="cuda")
            sf = torch.empty(n, swizzled_sf_numel(rows, k // 16), dtype=torch.uint8, device="cuda")
            inv_gs = torch.empty(n, dtype=torch.float32, device="cuda")
            for j in range(n):
                g = torch.Generator(device="cuda").manual_seed(seed * 100003 + lo + j)
                w = 0.02 * torch.randn(rows, k, generator=g, device="cuda")
                c, s, gs = pkg.gemm.quantize_operand(w)
                codes[j], sf[j], inv_gs[j] = c, s, 1.0 / gs
            out[name], out[name + "_sf"], out[name + "_alpha"] = codes, sf, inv_gs
        out["fc2_input_scale"] = torch.ones(1, device="cuda")
        return out

    def _inputs(self, rank):
        """Tokens and router logits of one rank's slice (seeded per rank: any rank can rebuild any slice)."""
        import torch
        t = self.local_tokens
        g = torch.Generator(device="cuda").manual_seed(1000 + rank)
        x = torch.randn(t, self.hidden, generator=g, device="cuda").to(torch.bfloat16)
        logits = torch.randn(t, self.experts, generator=g, device="cuda")
        if self.kind == "decode" and rank == 0:
            n_hot = max(1, -(-self.tokens // 100))
            logits[:n_hot, 0] += 1e4
        return x, logits

    def setup(self, pkg):
        import torch
        self.pkg = pkg
        t, h, e, k, i = self.local_tokens, self.hidden, self.experts, self.top_k, self.inter
        self.weights = self._expert_weights(pkg, self.expert_lo, self.local_experts)
        self.x, self.logits = self._inputs(self.rank)
        self.out = torch.empty(t, h, dtype=torch.bfloat16, device="cuda")
        ids, _ = pkg.topk_route(self.logits, k)
        local = (ids >= self.expert_lo) & (ids < self.expert_lo + self.local_experts)
        # experts of this rank that the WHOLE batch touches are not known to one rank; the roofline uses the
        # rank's own view at N = 1 and the expectation over uniform routing otherwise
        if self.world == 1:
            active = int(torch.unique(ids[local]).numel())
        else:
            p_idle = (1.0 - 1.0 / e) ** (self.tokens * k)
            active = round(self.local_experts * (1.0 - p_idle))
        self.active_experts = active
        self.alg_bytes = active * self.expert_bytes + 2 * t * h * 2
        self.ep = None
        if self.world > 1:
            self.ep = pkg.parallel.PeerExpertParallelMoE(
                e, k, t, h, i, return_rows=os.environ.get("B200FP4_EP_RETURN", "auto"))
            self.launches_per_step = 6 if self.ep.return_rows == "per_rank" else 5
            self.ep_weights = {"w1": self.weights["w1"], "w1_sf": self.weights["w1_sf"], "w2": self.weights["w2"],
                               "w2_sf": self.weights["w2_sf"], "w1_alpha": self.weights["w1_alpha"],
                               "w2_alpha": self.weights["w2_alpha"], "fc2_input_scale": self.weights["fc2_input_scale"]}
        else:
            self.wrapper = pkg.B12xMoEWrapper(e, k, h, i, max_num_tokens=t)
        self.flush = _flush_buffer()

    def step(self, x=None, logits=None, out=None):
        w = self.weights
        x = self.x if x is None else x
        logits = self.logits if logits is None else logits
        out = self.out if out is None else out
        if self.ep is not None:
            self.ep.forward(x, None, None, self.ep_weights, out=out, router_logits=logits)
            return
        self.wrapper.run(x, w["w1"], w["w1_sf"], w["w2"], w["w2_sf"], router_logits=logits,
                         w1_alpha=w["w1_alpha"], w2_alpha=w["w2_alpha"], fc2_input_scale=w["fc2_input_scale"],
                         output=out)

    def setup_e2e(self):
        import torch
        self.hx = self.x.cpu().pin_memory()
        self.hl = self.logits.cpu().pin_memory()
        self.ho = [torch.empty(self.out.shape, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
        self.ex = [self.x, torch.empty_like(self.x)]
        self.el = [self.logits, torch.empty_like(self.logits)]
        self.eo = [self.out, torch.empty_like(self.out)]
        self.h2d = self.hx.numel() * 2 + self.hl.numel() * 4
        self.d2h = self.ho[0].numel() * 2

    def e2e_h2d(self, b):
        self.ex[b].copy_(self.hx, non_blocking=True)
        self.el[b].copy_(self.hl, non_blocking=True)

    def e2e_compute(self, b):
        self.step(self.ex[b], self.el[b], self.eo[b])

    def e2e_d2h(self, b):
        self.ho[b].copy_(self.eo[b], non_blocking=True)

    def roofline_extra(self):
        return {"traffic": None, "active_experts": self.active_experts,
                "flops_per_step": 6.0 * self.local_tokens * self.top_k * self.hidden * self.inter}

    # ---- parity of what is being timed
    def checks(self, pkg, world, rank):
        """One untimed step; the ranks' outputs are gathered on rank 0 and compared with the single-GPU operator
        on the same tokens (must be EQUAL) and with the CPU oracle on a sample of tokens (rel-L2 <= 1e-2)."""
        import numpy as np
        import torch
        import torch.distributed as dist
        from cutedsl_fully_opensourced_b200.layout import unpack_e2m1, unswizzle_sf
        from oracle import nvfp4_oracle as O
        self.step()
        torch.cuda.synchronize()
        status = pkg._lib.device_status()
        mine = self.out.clone()
        if world > 1:
            gathered = [torch.empty_like(mine) for _ in range(world)] if rank == 0 else None
            dist.gather(mine, gathered, dst=0)
            st = torch.tensor([status], device="cuda")
            dist.all_reduce(st, op=dist.ReduceOp.MAX)
            status = int(st.item())
        else:
            gathered = [mine]
        result = None
        if rank == 0:
            got = torch.cat(gathered)
            result = {"device_status": status}
            xs, ls = zip(*[self._inputs(r) for r in range(world)])
            x_all, logits_all = torch.cat(xs), torch.cat(ls)
            ids_all, w_all = pkg.topk_route(logits_all, self.top_k)
            if world > 1:
                full = self._expert_weights(pkg, 0, self.experts)
                single = pkg.b12x_fused_moe(x_all, full["w1"], full["w1_sf"], full["w2"], full["w2_sf"], ids_all, w_all,
                                            self.experts, self.top_k, w1_alpha=full["w1_alpha"],
                                            w2_alpha=full["w2_alpha"], fc2_input_scale=full["fc2_input_scale"])
                torch.cuda.synchronize()
                if self.ep is not None and self.ep.return_rows == "per_slot":
                    result["equals_single_gpu_operator"] = bool(torch.equal(got, single))
                else:
                    # per-rank return: the same sum grouped by serving rank, one bf16 rounding per partial sum
                    diff = float(torch.linalg.vector_norm(got.float() - single.float()) /
                                 torch.linalg.vector_norm(single.float()))
                    result["rel_l2_vs_single_gpu_operator"] = round(diff, 6)
            else:
                full = self.weights
            # oracle on a sample of tokens (only their experts are de-quantised on the host)
            n_s = 4 if self.kind == "prefill" else 2
            sample = torch.linspace(0, self.tokens - 1, n_s).long().unique()
            ids_s, w_s = ids_all[sample].cpu(), w_all[sample].cpu()
            used = sorted(set(ids_s.reshape(-1).tolist()))
            remap = {e: j for j, e in enumerate(used)}
            idx = torch.tensor(used, device="cuda")
            h, i = self.hidden, self.inter
            w1c = unpack_e2m1(full["w1"][idx]).cpu().numpy()
            w2c = unpack_e2m1(full["w2"][idx]).cpu().numpy()
            w1s = unswizzle_sf(full["w1_sf"][idx], 2 * i, h // 16).cpu().numpy()
            w2s = unswizzle_sf(full["w2_sf"][idx], h, i // 16).cpu().numpy()
            ids_m = torch.tensor([[remap[int(e)] for e in row] for row in ids_s.tolist()], dtype=torch.int32)
            ref = O.moe_ref(x_all[sample].cpu(), w1c, w1s, w2c, w2s, ids_m, w_s,
                            full["w1_alpha"][idx].cpu().numpy(), full["w2_alpha"][idx].cpu().numpy(), 1.0)
            err = float(torch.linalg.vector_norm(got[sample].cpu().float() - ref.float()) /
                        torch.linalg.vector_norm(ref.float()))
            result["oracle_rel_l2_on_sampled_tokens"] = round(err, 6)
            result["oracle_tokens"] = int(sample.numel())
            result["ok"] = (status == 0 and err <= 1e-2 and result.get("equals_single_gpu_operator", True)
                            and result.get("rel_l2_vs_single_gpu_operator", 0.0) <= 4e-3)
            del full
        return result

    # ---- CPU arm: a bounded sample of the same shape
    def cpu_setup(self):
        import numpy as np
        import torch
        from oracle import nvfp4_oracle as O
        # prefill: 64 tokens over 8 experts, top-8; decode (experts of 44 M weights each): up to 8 tokens over 2
        # experts, top-2, so that a step stays near a second
        t, e = (min(self.tokens, 64), 8) if self.kind == "prefill" else (min(self.tokens, 8), 2)
        rng = np.random.default_rng(0)
        self.c_w = (rng.integers(0, 16, size=(e, 2 * self.inter, self.hidden), dtype=np.uint8),
                    rng.integers(0x18, 0x30, size=(e, 2 * self.inter, self.hidden // 16), dtype=np.uint8),
                    rng.integers(0, 16, size=(e, self.hidden, self.inter), dtype=np.uint8),
                    rng.integers(0x18, 0x30, size=(e, self.hidden, self.inter // 16), dtype=np.uint8))
        self.c_x = torch.randn(t, self.hidden).to(torch.bfloat16)
        self.c_ids, self.c_wts = O.route_topk_ref(torch.randn(t, e), min(self.top_k, e))
        self.c_t, self.c_e = t, e

    def cpu_run(self, threads: int):
        import torch
        from oracle import nvfp4_oracle as O
        torch.set_num_threads(threads)
        t0 = time.perf_counter()
        O.moe_ref(self.c_x, *self.c_w, self.c_ids, self.c_wts, weight_key=lambda ex: ex)
        dt = time.perf_counter() - t0
        return self.c_t / dt, dt, (f"{self.c_t} tokens over {self.c_e} experts of this shape, top-{min(self.top_k, self.c_e)}: "
                                   f"oracle port (numpy+torch), {threads} threads")


def make_parts(rank, world, wanted, nk=8192):
    table = [
        ("moe_prefill", lambda: MoePart(rank, world, "prefill")),
        ("norm_quant", lambda: NormPart(rank, world)),
        ("gemm_8192", lambda: GemmPart(rank, world, nk, nk, nk)),
        ("gemm_m1024", lambda: GemmPart(rank, 1, 1024, nk, nk)),
        ("gemm_m128", lambda: GemmPart(rank, 1, 128, nk, nk)),
        ("moe_decode_t64", lambda: MoePart(rank, world, "decode", 64)),
        ("moe_decode_t8", lambda: MoePart(rank, world, "decode", 8)),
        ("moe_decode_t1", lambda: MoePart(rank, world, "decode", 1)),
    ]
    parts = []
    for key, make in table:
        if wanted and key not in wanted:
            continue
        if world > 1 and key in ("gemm_m1024", "gemm_m128"):
            continue                                 # the M sweep is a one-GPU measurement
        part = make()
        if part.supported(world):
            parts.append((key, part))
    return parts


# ---------------------------------------------------------------------------
# CPU arm
# ---------------------------------------------------------------------------
def cpu_part(part, steps, warmup, budget_s):
    """Time the oracle port: `steps` steps when a step is cheap, otherwise as many as fit the budget (>= 1)."""
    threads = host_threads()
    part.cpu_setup()
    for _ in range(min(warmup, 1)):
        part.cpu_run(threads)
    vals, times, spent, sample = [], [], 0.0, ""
    while len(vals) < steps and (not vals or spent + times[-1] <= budget_s):
        v, dt, sample = part.cpu_run(threads)
        vals.append(v)
        times.append(dt)
        spent += dt
    value = statistics.median(vals)
    return {"value": round(value, 4), "unit": part.unit, "cores": threads, "kind": "port",
            "sample": f"{sample}; median of {len(vals)} steps", "steps": len(vals), "seconds": round(spent, 2),
            "ms_per_step": round(1e3 * spent / len(vals), 3)}


def run_reference_arm(args, world):
    """The reference's CPU golden path (restated in oracle/) for every part, timed on the host cores."""
    parts = make_parts(0, world, args.parts, args.nk)
    out, head = {}, None
    for key, part in parts:
        budget = 20.0 if key == "moe_prefill" else 6.0
        res = cpu_part(part, args.steps, args.warmup, budget)
        res["metric"] = part.metric
        res["config"] = part.config(world)
        if head is None:
            head = (key, part, res)
        else:
            out[key] = res
    key, part, res = head
    line = {
        "impl": "reference", "metric": part.metric, "value": res["value"], "unit": part.unit, "n_gpus": args.gpus,
        "steps": res["steps"], "warmup": min(args.warmup, 1), "ms_per_step": res["ms_per_step"],
        "higher_is_better": True, "scaling": part.scaling, "vs_baseline": None, "dtype": part.dtype,
        "data": "synthetic", "config": part.config(world),
        "cpu_baseline": {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": res["value"], "unit": part.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "parts": out,
        "note": "CPU arm: the oracle port of the reference's torch golden path on the host cores; a step is the bounded "
                "sample named in cpu_baseline.sample (the full configurations take minutes per step on a CPU)",
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------
class E2EPipeline:
    """The end-to-end leg as a serving loop would run it: every step copies its inputs from pinned host memory,
    computes through the public API and copies its result back, all inside the timed region; two buffer sets let
    the copies of neighbouring steps (separate copy streams, both DMA directions) overlap the kernels of the
    current one.  A step's kernels start only when its own inputs have landed, and a buffer set is reused only
    when the step that used it two steps earlier has delivered its result."""

    def __init__(self, part):
        import torch
        self.torch, self.part, self.i = torch, part, 0
        self.s_in, self.s_out = torch.cuda.Stream(), torch.cuda.Stream()
        self.ev_in = [torch.cuda.Event() for _ in range(2)]
        self.ev_cmp = [torch.cuda.Event() for _ in range(2)]
        self.ev_out = [torch.cuda.Event() for _ in range(2)]

    def step(self):
        torch, part, b = self.torch, self.part, self.i % 2
        cur = torch.cuda.current_stream()
        if self.i < 2:
            self.s_in.wait_stream(cur)
        with torch.cuda.stream(self.s_in):
            if self.i >= 2:
                self.s_in.wait_event(self.ev_cmp[b])      # the kernels that read this input set have finished
            part.e2e_h2d(b)
            self.ev_in[b].record(self.s_in)
        cur.wait_event(self.ev_in[b])
        if self.i >= 2:
            cur.wait_event(self.ev_out[b])                # this set's previous result has left the device
        part.e2e_compute(b)
        self.ev_cmp[b].record(cur)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(self.ev_cmp[b])
            part.e2e_d2h(b)
            self.ev_out[b].record(self.s_out)
        self.i += 1

    def drain(self):
        cur = self.torch.cuda.current_stream()
        for ev in self.ev_out[:min(2, self.i)]:
            cur.wait_event(ev)


def run_part(key, part, pkg, args, rank, world, barrier, sampler, peaks, all_reduce_max):
    import torch
    steps, warmup = max(1, args.steps), max(3, args.warmup)
    part.setup(pkg)
    check = part.checks(pkg, world, rank) if not args.no_checks else None
    # the ranks meet before they step together: rank 0 spent seconds on the check, and the kernels of an
    # expert-parallel step wait for their peers with a time bound
    barrier()
    for _ in range(warmup):
        part.restore()
        part.step()
    pkg.synchronize()
    step_fn, launch = part.step, "eager"
    graphs = []
    if part.use_graph and not args.no_graph:
        # one graph per rotating operand set (a graph pins its pointers); the MoE parts have one set
        torch.cuda.synchronize()
        part.i = 0
        for _ in range(getattr(part, "graph_variants", 1)):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                part.step()
            graphs.append(g)
        turn = [0]

        def replay_next():
            graphs[turn[0] % len(graphs)].replay()
            turn[0] += 1
        step_fn, launch = replay_next, "cuda graph replay"
    barrier()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    # untimed pre-roll right behind the barrier: the timed steps do not start on a GPU that idled while ranks met
    for _ in range(3):
        part.restore()
        step_fn()
    t0 = time.time()
    for a, b in ev:
        part.restore()
        a.record()
        step_fn()
        b.record()
    barrier()
    t1 = time.time()
    step_ms = [a.elapsed_time(b) for a, b in ev]
    status = pkg._lib.device_status()
    clocks = sampler.window(t0, t1) if sampler is not None else None

    e2e_steps, e2e_ms = min(steps, 10), float("nan")
    if not args.no_e2e:
        part.setup_e2e()
        pipe = E2EPipeline(part)
        for _ in range(2):
            pipe.step()
        pipe.drain()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(e2e_steps):
            pipe.step()
        pipe.drain()
        e1.record()
        barrier()
        e2e_ms = e0.elapsed_time(e1)
    # per-step maximum over ranks (a step is finished when its slowest rank is)
    red = all_reduce_max(step_ms + [e2e_ms, float(status)])
    step_ms_max, e2e_ms, status = red[:steps], red[steps], int(red[steps + 1])
    total_ms = sum(step_ms_max)
    res = None
    if rank == 0:
        ms_per_step = total_ms / steps
        scale = {"GB/s": 1e9, "TFLOP/s": 1e12}.get(part.unit, 1.0)
        value = part.units_per_step / (ms_per_step * 1e-3) / scale
        k_ms = statistics.mean(step_ms)           # rank 0's own launches
        if part.bound == "hbm":
            achieved, peak, roof_unit = part.alg_bytes / (k_ms * 1e-3) / 1e9, peaks["hbm_gbs"], "GB/s"
            peak_src = f"{peaks['source']} copy bandwidth"
        else:
            achieved, peak, roof_unit = part.alg_flops / (k_ms * 1e-3) / 1e12, FP4_NOMINAL_TFLOPS, "TFLOP/s"
            peak_src = ("nominal dense FP4 (no measured FP4 peak; 4x measured bf16 burst = %.0f TFLOP/s, "
                        "frac_of_that = %.3f)" % (4 * peaks["bf16_tflops"], achieved / max(1e-9, 4 * peaks["bf16_tflops"])))
        roof = {"bound": part.bound, "kernel": part.kernel, "achieved": round(achieved, 1), "peak": peak,
                "peak_source": peak_src, "unit": roof_unit, "frac": round(achieved / peak, 4),
                "algorithmic_bytes_per_launch": int(part.alg_bytes), "kernel_us": round(k_ms * 1e3, 2),
                "kernel_us_min": round(min(step_ms) * 1e3, 2)}
        roof.update(part.roofline_extra())
        res = {"metric": part.metric, "value": round(value, 2), "unit": part.unit, "ms_per_step": round(ms_per_step, 5),
               "steps": steps, "step_us": stats_us(step_ms_max), "scaling": part.scaling if world > 1 else "n/a (one GPU)",
               "config": part.config(world), "launch": launch, "roofline": roof, "clocks": clocks,
               "gpu_launches": part.launches_per_step * steps * world, "device_status": status, "dtype": part.dtype}
        if not args.no_e2e:
            res["e2e"] = {"value": round(part.units_per_step / (e2e_ms / e2e_steps * 1e-3) / scale, 3), "unit": part.unit,
                          "h2d_bytes_per_step": part.h2d * world, "d2h_bytes_per_step": part.d2h * world,
                          "steps": e2e_steps}
        if check is not None:
            res["checks"] = check
        if not args.no_cpu_baseline and world == 1:
            res["cpu_baseline"] = cpu_part(part, 50, 0, 3.0 if key != "moe_prefill" else 6.0)
    del graphs
    part.free()
    import gc
    gc.collect()
    torch.cuda.empty_cache()
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--parts", default="", help="comma-separated subset of: moe_prefill, norm_quant, gemm_8192, "
                    "gemm_m1024, gemm_m128, moe_decode_t64, moe_decode_t8, moe_decode_t1 (default: all)")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU arm inside the GPU run")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--no-checks", action="store_true", help="skip the parity check of the MoE parts")
    ap.add_argument("--no-graph", action="store_true", help="launch the MoE steps eagerly instead of replaying a CUDA graph")
    ap.add_argument("--tile-n", type=int, default=0, help="gemm parts: force a tile variant (64/128/256/512)")
    ap.add_argument("--nk", type=int, default=8192, help="gemm parts: N = K (and M of gemm_8192); smaller values are "
                    "for profiler captures of a small case")
    args = ap.parse_args()
    args.parts = [p for p in args.parts.split(",") if p]

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    # shard_rows without importing the CUDA package (the CPU arm must not need the library)
    import importlib.util
    spec = importlib.util.spec_from_file_location(
        "cutedsl_fully_opensourced_b200_shard", os.path.join(ROOT, "cutedsl-fully-opensourced_b200", "_shard.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules["cutedsl_fully_opensourced_b200_shard"] = mod

    if args.impl == "reference":
        if rank == 0:
            run_reference_arm(args, world)
        return 0

    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    if args.gpus != world and rank == 0:
        print(f"note: --gpus {args.gpus} but WORLD_SIZE={world}; using {world}", file=sys.stderr)

    import cutedsl_fully_opensourced_b200 as pkg
    peaks = load_peaks()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def all_reduce_max(values):
        t = torch.tensor(values, dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(v) for v in t.cpu()]

    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler is not None:
        sampler.start()
        time.sleep(0.2)
    results = {}
    failed = False
    for key, part in make_parts(rank, world, args.parts, args.nk):
        part.tile_n = args.tile_n
        res = run_part(key, part, pkg, args, rank, world, barrier, sampler, peaks, all_reduce_max)
        if rank == 0:
            results[key] = res
            if res.get("device_status") or (res.get("checks") or {}).get("ok") is False:
                failed = True
    if sampler is not None:
        sampler.stop()
    if rank == 0:
        keys = list(results)
        head_key = keys[0]
        head = results.pop(head_key)
        line = {
            "metric": head["metric"], "value": head["value"], "unit": head["unit"], "n_gpus": world,
            "steps": head["steps"], "warmup": max(3, args.warmup), "ms_per_step": head["ms_per_step"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": head["dtype"],
            "data": "synthetic", "config": head["config"], "launch": head["launch"], "step_us": head["step_us"],
            "e2e": head.get("e2e"), "gpu_launches": head["gpu_launches"], "roofline": head["roofline"],
            "clocks": head["clocks"], "device_status": head["device_status"],
        }
        for opt in ("checks", "cpu_baseline"):
            if opt in head:
                line[opt] = head[opt]
        line["parts"] = results
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())
