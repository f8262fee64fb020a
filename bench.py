#!/usr/bin/env python3
"""Benchmark of the NVFP4 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One "step" is one pass of the selected workload over one batch of seeded
synthetic input that is already resident in HBM.  The default workload is the
configuration the headline metric is quoted on: add_rmsnorm_fp4quant over bf16
[8192, 7168] (385 MB of algorithmic traffic per step, larger than L2).  With
N > 1 (launched by torch.distributed.run, one process per GPU) every rank owns
its own row block of the same size -- rows are independent, so there is no
data-path collective -- and the value is the aggregate over ranks divided by
the slowest rank's device time.

The JSON line printed by rank 0 carries the device-timed throughput
(``value``), the same metric through the public Python API with host buffers
(``e2e``), the roofline of the dominant kernel and a CPU baseline (the oracle
port timed on the host cores over a bounded sample).  ``--impl reference``
prints only that CPU arm.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HBM_FALLBACK_GBS = 6650.0      # earlier measurement on this pool, used only without MEASURED_PEAKS.json


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
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0: float, t1: float):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        for ts, line in self.lines:
            if ts < t0 - 0.05 or ts > t1 + 0.15:
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


# ---------------------------------------------------------------------------
# workloads
# ---------------------------------------------------------------------------
class AddRmsNormWorkload:
    """add_rmsnorm_fp4quant, bf16 [8192, 7168], weight 1 + 0.1 N(0,1), eps 1e-6,
    per-tensor global scale 448*6/amax, scale factors in the 128x4 tiled layout."""
    name = "add_rmsnorm_fp4quant_bf16_8192x7168"
    metric = "norm-quant HBM GB/s"
    unit = "GB/s"
    dtype = "bf16"
    rows, hidden = 8192, 7168
    bytes_per_element = 2 + 2 + 2 + 0.5 + 0.0625      # x in, residual in+out, codes, scale bytes
    kernel = "norm_quant_kernel<bf16, add>"
    bound = "hbm"
    # DRAM bytes inside the kernel window per element, from the ncu capture summarised in
    # profiles/norm_quant_add_bf16.md (reads equal the algorithmic reads; most writes drain from L2 later)
    traffic_per_element = (117496064 + 26109440) / (4096 * 7168)

    def __init__(self, rank: int):
        self.rank = rank
        self.alg_bytes = int(self.rows * self.hidden * self.bytes_per_element)

    @property
    def work(self):                 # units of the metric per step: bytes
        return float(self.alg_bytes)

    def config(self, world):
        return {"workload": self.name, "rows_per_gpu": self.rows, "hidden": self.hidden,
                "sf_layout": "swizzled_128x4", "parallelism": f"rows x{world}",
                "l2": f"{self.sets} rotating sets of inputs and outputs (385 MB of traffic each, 126 MB L2): a "
                      "step never finds its inputs in L2; the residual streams are updated in place and keep "
                      "absorbing x from step to step"}

    def host_inputs(self, rows=None):
        import torch
        rows = rows or self.rows
        g = torch.Generator().manual_seed(1000 + self.rank)
        x = torch.randn(rows, self.hidden, generator=g).to(torch.bfloat16)
        r = torch.randn(rows, self.hidden, generator=g).to(torch.bfloat16)
        w = (1 + 0.1 * torch.randn(self.hidden, generator=torch.Generator().manual_seed(7))).to(torch.bfloat16)
        return x, r, w

    sets = 4      # rotating (x, residual, outputs) sets: a step never finds its inputs in L2

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
        self.x, self.r, self.y, self.sf = self.xs[0], self.rs[0], self.ys[0], self.sfs[0]
        self.r0 = self.r.clone()
        h = self.x.float() + self.r.float()
        normed = h.to(torch.bfloat16).float() * torch.rsqrt(h.square().mean(-1, keepdim=True) + 1e-6) * self.w.float()
        # RMSNorm output is scale-free, so this global scale stays valid while the residual streams
        # keep absorbing x over the steps
        self.gs = (448.0 * 6.0 / normed.abs().max()).reshape(1).float()
        del h, normed
        self.i = 0

    def restore(self):
        pass

    def step(self):
        j = self.i % self.sets
        self.i += 1
        self.pkg.add_rmsnorm_fp4quant(self.xs[j], self.rs[j], self.w, self.ys[j], self.sfs[j], global_scale=self.gs,
                                      eps=1e-6, block_size=16, is_sf_swizzled_layout=True)

    launches_per_step = 1

    # ---- end to end through the public API with host buffers
    def setup_e2e(self):
        import torch
        self.hx = self.x.cpu().pin_memory()
        self.hr = self.r0.cpu().pin_memory()
        self.hy = torch.empty(self.y.shape, dtype=torch.uint8).pin_memory()
        self.hsf = torch.empty(self.sf.shape, dtype=torch.uint8).pin_memory()
        self.hres = torch.empty(self.r.shape, dtype=torch.bfloat16).pin_memory()
        self.h2d = self.hx.numel() * 2 + self.hr.numel() * 2
        self.d2h = self.hy.numel() + self.hsf.numel() + self.hres.numel() * 2

    def step_e2e(self):
        self.x.copy_(self.hx, non_blocking=True)
        self.r.copy_(self.hr, non_blocking=True)
        self.pkg.add_rmsnorm_fp4quant(self.x, self.r, self.w, self.y, self.sf, global_scale=self.gs, eps=1e-6,
                                      block_size=16, is_sf_swizzled_layout=True)
        self.hy.copy_(self.y, non_blocking=True)
        self.hsf.copy_(self.sf, non_blocking=True)
        self.hres.copy_(self.r, non_blocking=True)

    # ---- CPU arm: the oracle port on a bounded sample of the same workload
    cpu_sample_rows = 8192

    def cpu_run(self, threads: int):
        import torch
        from concurrent.futures import ThreadPoolExecutor
        from oracle import nvfp4_oracle as O
        rows = self.cpu_sample_rows
        x, r, w = self.host_inputs(rows)
        gs = 500.0
        chunk = max(16, rows // max(1, threads * 2))
        spans = [(i, min(rows, i + chunk)) for i in range(0, rows, chunk)]
        torch.set_num_threads(1)
        t0 = time.perf_counter()
        with ThreadPoolExecutor(max_workers=threads) as pool:
            list(pool.map(lambda s: O.add_rmsnorm_fp4quant_ref(x[s[0]:s[1]], r[s[0]:s[1]], w, 1e-6, gs), spans))
        dt = time.perf_counter() - t0
        return rows * self.hidden * self.bytes_per_element / dt / 1e9, dt, \
            f"{rows} of {self.rows} rows x {self.hidden}, oracle port (numpy+torch), {threads} threads"


class GemmWorkload:
    """NVFP4 block-scaled GEMM M=N=K=8192: A, B ~ N(0,1) quantised to e2m1 with e4m3 scale factors per
    16 K-elements and a per-tensor global scale, f32 accumulate, bf16 output, alpha = 1/(gs_A*gs_B)."""
    metric = "NVFP4 GEMM TFLOP/s"
    unit = "TFLOP/s"
    dtype = "nvfp4 (e2m1 x e2m1, ue4m3 scales, f32 accumulate)"
    kernel = "nvfp4_gemm_kernel<256>"
    bound = "tensor"
    launches_per_step = 1
    sets = 3                      # rotating operand sets so no step finds its operands in L2
    FP4_NOMINAL_TFLOPS = 9000.0   # dense FP4 peak of a B200 (nominal; no measured FP4 peak exists)

    def __init__(self, rank: int, m: int = 8192, n: int = 8192, k: int = 8192):
        self.rank, self.m, self.n, self.k = rank, m, n, k
        self.rows, self.hidden = m, k
        self.name = f"nvfp4_gemm_{m}x{n}x{k}_bf16out"
        self.work = 2.0 * m * n * k
        self.alg_bytes = m * k // 2 + n * k // 2 + (m + n) * k // 16 + 2 * m * n

    def setup(self, pkg):
        import torch
        self.pkg = pkg
        self.ops = []
        for i in range(self.sets):
            g = torch.Generator(device="cuda").manual_seed(100 * self.rank + i)
            a = torch.randn(self.m, self.k, generator=g, device="cuda")
            b = torch.randn(self.n, self.k, generator=g, device="cuda")
            aq, sfa, gsa = pkg.gemm.quantize_operand(a)
            del a
            bq, sfb, gsb = pkg.gemm.quantize_operand(b)
            del b
            alpha = torch.tensor([1.0 / (gsa * gsb)], device="cuda")
            c = torch.empty(self.m, self.n, dtype=torch.bfloat16, device="cuda")
            self.ops.append((aq, bq, sfa, sfb, alpha, c))
        self.i = 0

    def restore(self):
        pass

    def step(self):
        aq, bq, sfa, sfb, alpha, c = self.ops[self.i % self.sets]
        self.i += 1
        self.pkg.nvfp4_gemm(aq, bq, sfa, sfb, alpha=alpha, out=c, tile_n=self.tile_n)

    tile_n = 0

    def config(self, world):
        return {"workload": self.name, "m_per_gpu": self.m, "n": self.n, "k": self.k,
                "parallelism": f"rows of A/C x{world}, B replicated",
                "l2": f"{self.sets} rotating operand sets of 72 MB + 134 MB output each, so a step never "
                      "finds its operands in the 126 MB L2"}

    def setup_e2e(self):
        import torch
        aq, bq, sfa, sfb, alpha, c = self.ops[0]
        self.h = [t.cpu().pin_memory() for t in (aq, bq, sfa, sfb)]
        self.hc = torch.empty(c.shape, dtype=c.dtype).pin_memory()
        self.h2d = sum(t.numel() * t.element_size() for t in self.h)
        self.d2h = self.hc.numel() * 2

    def step_e2e(self):
        aq, bq, sfa, sfb, alpha, c = self.ops[0]
        for d, h in zip((aq, bq, sfa, sfb), self.h):
            d.copy_(h, non_blocking=True)
        self.pkg.nvfp4_gemm(aq, bq, sfa, sfb, alpha=alpha, out=c, tile_n=self.tile_n)
        self.hc.copy_(c, non_blocking=True)

    def cpu_run(self, threads: int):
        import numpy as np
        import torch
        from oracle import nvfp4_oracle as O
        m, n, k = min(self.m, 1024), min(self.n, 1024), self.k
        torch.set_num_threads(threads)
        g = torch.Generator().manual_seed(0)
        ac, sfa = O.quantize_nvfp4(torch.randn(m, k, generator=g).numpy(), 500.0)
        bc, sfb = O.quantize_nvfp4(torch.randn(n, k, generator=g).numpy(), 500.0)
        t0 = time.perf_counter()
        O.gemm_nvfp4_ref(ac, sfa, bc, sfb, alpha=1.0 / 250000.0)
        dt = time.perf_counter() - t0
        return 2.0 * m * n * k / dt / 1e12, dt, \
            f"{m}x{n}x{k} block of the {self.m}x{self.n}x{self.k} problem: de-quantise + f32 matmul, {threads} threads"


class MoeWorkload:
    """Fused NVFP4 MoE.  prefill: 4096 tokens, hidden 2048, 128 experts, top-8, intermediate 768.
    decode: T tokens, hidden 7168, 256 experts, top-8, intermediate 2048, 1% of rows forced onto expert 0.
    Tokens bf16 ~ N(0,1); expert weights N(0, 0.02) quantised to NVFP4 per expert (global scale
    448*6/amax folded into w1_alpha / w2_alpha); router logits ~ N(0,1), softmax top-k renormalised.
    A step = router kernel + the fused MoE call."""
    metric = "MoE tokens/s"
    unit = "tokens/s"
    dtype = "nvfp4 weights and activations, bf16 tokens, f32 accumulate"
    kernel = "nvfp4_gemm_kernel<swiglu> + nvfp4_gemm_kernel (grouped FC1 / FC2)"
    bound = "hbm"
    launches_per_step = 8      # route, count, scan, scatter-quant, FC1, FC2, combine (+ 2 memsets not counted) 

    scaling = "strong"         # the token batch is fixed; more GPUs split it (and the experts)

    def __init__(self, rank, kind="prefill", tokens=None, world=1):
        self.rank, self.kind, self.world = rank, kind, world
        if kind == "prefill":
            self.tokens, self.hidden, self.experts, self.top_k, self.inter = tokens or 4096, 2048, 128, 8, 768
        else:
            self.tokens, self.hidden, self.experts, self.top_k, self.inter = tokens or 64, 7168, 256, 8, 2048
        self.rows = self.tokens
        self.name = f"moe_{kind}_T{self.tokens}_H{self.hidden}_E{self.experts}_k{self.top_k}_I{self.inter}"
        if self.tokens % world or self.experts % world:
            raise SystemExit(f"{self.tokens} tokens / {self.experts} experts do not divide over {world} ranks")
        self.local_tokens = self.tokens // world
        self.local_experts = self.experts // world
        self.expert_lo = rank * self.local_experts
        self.work = float(self.local_tokens)      # per rank; the bench multiplies by the world size
        self.expert_bytes = 3 * self.hidden * self.inter // 2 + 3 * self.hidden * self.inter // 16

    def _quant_experts(self, pkg, rows, k, seed):
        import torch
        from cutedsl_fully_opensourced_b200.layout import swizzled_sf_numel
        e = self.local_experts                   # this rank's experts only; they never move
        codes = torch.empty(e, rows, k // 2, dtype=torch.uint8, device="cuda")
        sf = torch.empty(e, swizzled_sf_numel(rows, k // 16), dtype=torch.uint8, device="cuda")
        inv_gs = torch.empty(e, dtype=torch.float32, device="cuda")
        for i in range(e):
            g = torch.Generator(device="cuda").manual_seed(seed * 100003 + self.expert_lo + i)
            w = 0.02 * torch.randn(rows, k, generator=g, device="cuda")
            c, s, gs = pkg.gemm.quantize_operand(w)
            codes[i], sf[i], inv_gs[i] = c, s, 1.0 / gs
        return codes, sf, inv_gs

    def setup(self, pkg):
        import torch
        self.pkg = pkg
        t, h, e, k, i = self.local_tokens, self.hidden, self.experts, self.top_k, self.inter
        self.w1, self.w1_sf, self.a1 = self._quant_experts(pkg, 2 * i, h, 11)
        self.w2, self.w2_sf, self.a2 = self._quant_experts(pkg, h, i, 12)
        g = torch.Generator(device="cuda").manual_seed(1000 + self.rank)
        self.x = torch.randn(t, h, generator=g, device="cuda").to(torch.bfloat16)
        self.logits = torch.randn(t, e, generator=g, device="cuda")
        if self.kind == "decode" and self.rank == 0:
            n_hot = max(1, -(-self.tokens // 100))
            self.logits[:n_hot, 0] += 1e4
        self.out = torch.empty(t, h, dtype=torch.bfloat16, device="cuda")
        self.fc2_scale = torch.ones(1, device="cuda")
        # per-expert output rows between FC2 and the weighted f32 sum: bf16 (default) or f32
        self.slot_rows = torch.float32 if os.environ.get("B200FP4_SLOT_ROWS", "bf16") == "f32" else torch.bfloat16
        ids, _ = pkg.topk_route(self.logits, k)
        active = int(torch.unique(ids).numel())
        self.active_experts = active
        self.alg_bytes = min(active, self.local_experts) * self.expert_bytes + 2 * t * h * 2
        self.ep = None
        if self.world > 1:
            if os.environ.get("B200FP4_EP", "peer") == "collective":
                self.ep = pkg.parallel.ExpertParallelMoE(e, k)
            else:
                self.ep = pkg.parallel.PeerExpertParallelMoE(e, k, t, h, i)
            self.weights = {"w1": self.w1, "w1_sf": self.w1_sf, "w2": self.w2, "w2_sf": self.w2_sf,
                            "w1_alpha": self.a1, "w2_alpha": self.a2, "fc2_input_scale": self.fc2_scale}
        # L2 flush buffer: the weights of the prefill case (340 MB) exceed L2 by themselves; the decode
        # cases touch as little as 0.2 GB, so a 256 MB buffer is rewritten between steps (untimed)
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if self.alg_bytes < (400 << 20) else None

    def restore(self):
        if self.flush is not None:
            self.flush.zero_()

    def step(self):
        ids, wts = self.pkg.topk_route(self.logits, self.top_k)
        if self.ep is not None:
            self.ep.forward(self.x, ids, wts, self.weights, out=self.out)
            return
        self.pkg.b12x_fused_moe(self.x, self.w1, self.w1_sf, self.w2, self.w2_sf, ids, wts, self.experts, self.top_k,
                                w1_alpha=self.a1, w2_alpha=self.a2, fc2_input_scale=self.fc2_scale, output=self.out,
                                slot_rows_dtype=self.slot_rows)

    def config(self, world):
        return {"workload": self.name, "tokens": self.tokens, "hidden": self.hidden, "experts": self.experts,
                "top_k": self.top_k, "intermediate": self.inter, "active_experts": self.active_experts,
                "slot_rows": "bf16" if world > 1 or self.slot_rows is not None and "bfloat16" in str(self.slot_rows)
                else "f32",
                "parallelism": (f"experts x{world}, tokens x{world}; " + (
                    "NCCL all-gather of tokens + routing, reduce-scatter of f32 partial outputs"
                    if os.environ.get("B200FP4_EP", "peer") == "collective" else
                    "dispatch / combine as NVLink peer loads inside the kernels, two barriers per step")
                ) if world > 1 else "single GPU",
                "l2": "weights streamed per step exceed the 126 MB L2" if self.flush is None else
                      "a 256 MB buffer is rewritten (untimed) between steps to flush the 126 MB L2"}

    def setup_e2e(self):
        import torch
        self.hx = self.x.cpu().pin_memory()
        self.hl = self.logits.cpu().pin_memory()
        self.ho = torch.empty(self.out.shape, dtype=torch.bfloat16).pin_memory()
        self.h2d = self.hx.numel() * 2 + self.hl.numel() * 4
        self.d2h = self.ho.numel() * 2

    def step_e2e(self):
        self.x.copy_(self.hx, non_blocking=True)
        self.logits.copy_(self.hl, non_blocking=True)
        self.step()
        self.ho.copy_(self.out, non_blocking=True)

    def cpu_run(self, threads: int):
        import numpy as np
        import torch
        from oracle import nvfp4_oracle as O
        torch.set_num_threads(threads)
        t = min(self.tokens, 64)
        e = 8                                   # a bounded sample: 64 tokens routed over 8 experts of the same shape
        rng = np.random.default_rng(0)
        w1c = rng.integers(0, 16, size=(e, 2 * self.inter, self.hidden), dtype=np.uint8)
        w2c = rng.integers(0, 16, size=(e, self.hidden, self.inter), dtype=np.uint8)
        w1s = rng.integers(0x18, 0x30, size=(e, 2 * self.inter, self.hidden // 16), dtype=np.uint8)
        w2s = rng.integers(0x18, 0x30, size=(e, self.hidden, self.inter // 16), dtype=np.uint8)
        x = torch.randn(t, self.hidden).to(torch.bfloat16)
        ids, wts = O.route_topk_ref(torch.randn(t, e), min(self.top_k, e))
        t0 = time.perf_counter()
        O.moe_ref(x, w1c, w1s, w2c, w2s, ids, wts)
        dt = time.perf_counter() - t0
        return t / dt, dt, (f"{t} tokens over {e} experts of this shape, top-{min(self.top_k, e)}: oracle port "
                            f"(numpy+torch), {threads} threads")


WORKLOADS = {"add_rmsnorm": AddRmsNormWorkload, "gemm": GemmWorkload, "moe_prefill": MoeWorkload,
             "moe_decode": MoeWorkload}


# ---------------------------------------------------------------------------
def host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def run_reference_arm(args, wl):
    """The reference's CPU golden path for this workload (restated in oracle/), timed on the host cores."""
    threads = host_threads()
    vals = []
    for _ in range(max(0, min(args.warmup, 1))):
        wl.cpu_run(threads)
    t_total = 0.0
    for _ in range(max(1, min(args.steps, 3))):
        v, dt, sample = wl.cpu_run(threads)
        vals.append(v)
        t_total += dt
    value = statistics.median(vals)
    line = {
        "impl": "reference", "metric": wl.metric, "value": round(value, 4), "unit": wl.unit, "n_gpus": args.gpus,
        "steps": len(vals), "warmup": min(args.warmup, 1), "ms_per_step": round(1e3 * t_total / len(vals), 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
        "config": {"workload": wl.name, "device": "host cpu"},
        "cpu_baseline": {"value": round(value, 4), "unit": wl.unit, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": round(value, 4), "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="add_rmsnorm", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU arm inside the GPU run")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--rows", type=int, default=None, help="override the row count (small profiling cases)")
    ap.add_argument("--m", type=int, default=None, help="gemm: override M (M-sweep 128 / 1024 / 8192)")
    ap.add_argument("--nk", type=int, default=None, help="gemm: override N = K (small profiling cases)")
    ap.add_argument("--tile-n", type=int, default=0, help="gemm: force the 128- or 256-wide tile")
    ap.add_argument("--cuda-graph", action="store_true",
                    help="moe, gemm: capture a step in a CUDA graph after warm-up and replay it in the timed region")
    ap.add_argument("--tokens", type=int, default=None, help="moe: override the token count (decode: 1 / 8 / 64)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.workload == "gemm":
        nk = args.nk or 8192
        wl = GemmWorkload(rank, args.m or 8192, nk, nk)
        wl.tile_n = args.tile_n
        wl.kernel = {0: "nvfp4_gemm_pair_kernel (256x256 tiles on CTA pairs) for a full wave of such tiles, "
                        "else nvfp4_gemm_kernel<256|128|64>",
                     512: "nvfp4_gemm_pair_kernel (256x256 tiles on CTA pairs)"}.get(
                         args.tile_n, f"nvfp4_gemm_kernel<{args.tile_n}>")
    elif args.workload.startswith("moe_"):
        wl = MoeWorkload(rank, args.workload[4:], args.tokens, world)
    else:
        wl = WORKLOADS[args.workload](rank)
    if args.rows and args.workload == "add_rmsnorm":
        wl.rows = args.rows
        wl.name += f"_rows{args.rows}"
        wl.alg_bytes = int(wl.rows * wl.hidden * wl.bytes_per_element)

    if args.impl == "reference":
        if rank == 0:
            run_reference_arm(args, wl)
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
    wl.setup(pkg)
    warmup = max(3, args.warmup)
    steps = max(1, args.steps)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-timed steps (inputs resident in HBM)
    for _ in range(warmup):
        wl.restore()
        wl.step()
    step_fn, launch_mode = wl.step, "eager"
    if args.cuda_graph and args.workload.startswith("moe_") and (
            world == 1 or os.environ.get("B200FP4_EP", "peer") != "collective"):
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            wl.step()
        step_fn, launch_mode = graph.replay, "cuda graph replay"
    elif args.cuda_graph and args.workload == "gemm":
        # one graph per rotating operand set (a graph pins its pointers)
        torch.cuda.synchronize()
        graphs = []
        for i in range(wl.sets):
            wl.i = i
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                wl.step()
            graphs.append(g)
        turn = [0]

        def replay_next():
            graphs[turn[0] % len(graphs)].replay()
            turn[0] += 1
        step_fn, launch_mode = replay_next, "cuda graph replay"
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    barrier()
    # three untimed pre-roll steps are queued right behind the barrier so that the timed steps do not
    # start on a GPU that idled (and clocked down) while the ranks met; only the K steps below are timed
    for _ in range(3):
        wl.restore()
        step_fn()
    t_wall0 = time.time()
    for a, b in ev:
        wl.restore()
        a.record()
        step_fn()
        b.record()
    barrier()
    t_wall1 = time.time()
    step_ms = [a.elapsed_time(b) for a, b in ev]
    total_ms = sum(step_ms)
    clocks = sampler.stop(t_wall0, t_wall1) if rank == 0 else None

    # ---- end to end: host buffers in, host buffers out, copies inside the timed region
    e2e_steps = min(steps, 10)
    e2e_ms = float("nan")
    if not args.no_e2e:
        wl.setup_e2e()
        for _ in range(3):
            wl.step_e2e()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(e2e_steps):
            wl.step_e2e()
        e1.record()
        barrier()
        e2e_ms = e0.elapsed_time(e1)

    t = torch.tensor([total_ms, e2e_ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms = (float(v) for v in t.cpu())

    if rank == 0:
        ms_per_step = total_ms / steps
        scale = {"GB/s": 1e9, "TFLOP/s": 1e12}.get(wl.unit, 1.0)
        value = wl.work * world / (ms_per_step * 1e-3) / scale
        e2e_value = wl.work * world / (e2e_ms / e2e_steps * 1e-3) / scale
        # roofline of the dominant kernel: rank 0's own launches, averaged over the timed region
        k_ms = statistics.mean(step_ms)
        achieved = wl.work / (k_ms * 1e-3) / scale
        roof_unit = wl.unit
        if wl.unit == "tokens/s":          # roofline of the whole step in bytes streamed from HBM
            achieved, roof_unit = wl.alg_bytes / (k_ms * 1e-3) / 1e9, "GB/s"
        if wl.bound == "hbm":
            peak, peak_src = peaks["hbm_gbs"], peaks["source"]
        else:
            peak, peak_src = wl.FP4_NOMINAL_TFLOPS, "nominal dense FP4 (no measured FP4 peak; 4x measured bf16 burst = %.0f)" % (4 * peaks["bf16_tflops"])
        line = {
            "metric": wl.metric, "value": round(value, 2), "unit": wl.unit, "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": round(ms_per_step, 5), "higher_is_better": True,
            "scaling": getattr(wl, "scaling", "weak"),
            "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
            "config": dict(wl.config(world), launch=launch_mode),
            "e2e": None if args.no_e2e else {
                "value": round(e2e_value, 3), "unit": wl.unit, "h2d_bytes_per_step": wl.h2d * world,
                "d2h_bytes_per_step": wl.d2h * world, "steps": e2e_steps},
            "gpu_launches": wl.launches_per_step * steps * world,
            "roofline": {"bound": wl.bound, "kernel": wl.kernel, "achieved": round(achieved, 1),
                         "peak": peak, "peak_source": peak_src, "unit": roof_unit,
                         "frac": round(achieved / peak, 4),
                         "traffic": (int(wl.traffic_per_element * wl.rows * wl.hidden)
                                     if hasattr(wl, "traffic_per_element") else None),
                         "algorithmic_bytes_per_launch": wl.alg_bytes,
                         "kernel_us": round(k_ms * 1e3, 2), "kernel_us_min": round(min(step_ms) * 1e3, 2)},
            "clocks": clocks,
        }
        if not args.no_cpu_baseline and world == 1:
            threads = host_threads()
            vals, spent = [], 0.0
            while spent < 8.0 and len(vals) < 50:          # a bounded sample: about 8 s of wall time on all cores
                v, dt, sample = wl.cpu_run(threads)
                vals.append(v)
                spent += dt
            line["cpu_baseline"] = {"value": round(statistics.median(vals), 4), "unit": wl.unit, "cores": threads,
                                    "kind": "port", "sample": f"{sample}; median of {len(vals)} runs",
                                    "seconds": round(spent, 2)}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
