"""Benchmark of the block-scaled GEMM hot path (one JSON line on stdout).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--all-configs]
                    [--only all|gemm|mega_moe] [--moe-tokens T] [--moe-experts E]

A step is one pass of the hot path over one batch of synthetic input.  The headline workload is
the contiguous M-grouped FP8 GEMM (8 experts, N=4096, K=7168, rows per expert uniform in
[0.7, 1.3] x 8192 padded to 128): seeded BF16 normal tensors quantised 1x128 (activations) and
128x128 (weights) to E4M3 with UE8M0 scales, scale factors pre-packed.  Inputs (about 1.2 GB)
are larger than L2, so consecutive timed steps do not find their operands cached.

`value`   : TFLOPS of the kernel with inputs resident in HBM (CUDA events on the launch stream).
`e2e`     : the same metric through the public operator with HOST buffers: pinned activations,
            scales and layout are copied in, the BF16 result is copied out, every step.
`roofline`: tensor-core bound; achieved = 2 * M_valid * N * K / kernel time; peak = 2 x the
            measured dense BF16 figure of MEASURED_PEAKS.json (FP8 UMMA issues at twice the BF16
            rate), fallback 2 x 1590 TFLOPS when that file is absent.
`cpu_baseline`: the CPU oracle (dequantise + float32 BLAS matmul) timed on a bounded sample.

With --gpus N > 1 the GEMM does not shard (no exchange step): N independent replicas run, one
per GPU, and `value` is the aggregate.  --impl reference times the reference's only CPU-runnable
formulation of this path (dequantise-then-matmul, here the oracle port) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import random
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# DRAM traffic of one launch of the headline kernel, from one ncu capture (not measured live: ncu is not part of a run)
NCU_TRAFFIC_BYTES_PER_LAUNCH = 1.996e9
NOMINAL_FP8_TFLOPS = 4500.0


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return dict(bf16=float(p["bf16_tflops"]), bf16_sustained=float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                    hbm=float(p["hbm_gbs"]), source="measured")
    except Exception:
        return dict(bf16=1590.0, bf16_sustained=1400.0, hbm=6650.0, source="fallback")


class ClockSampler:
    """SM clock and clock-event (throttle) reasons of one GPU, polled through NVML every 2 ms by a thread while the
    timed region runs (read-only queries; nvidia-smi's fastest loop is too slow for a region of a few tens of ms)."""

    def __init__(self, device):
        self.samples, self.thread, self.stop_flag, self.handle, self.nv, self.error = [], None, False, None, None, None
        try:
            import pynvml as nv
            import torch
            nv.nvmlInit()
            prop = torch.cuda.get_device_properties(device)
            try:
                bus = f"{prop.pci_domain_id:08x}:{prop.pci_bus_id:02x}:{prop.pci_device_id:02x}.0"
                self.handle = nv.nvmlDeviceGetHandleByPciBusId(bus.encode())
            except Exception:
                self.handle = nv.nvmlDeviceGetHandleByIndex(device.index or 0)
            self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(self.handle, nv.NVML_CLOCK_SM))
            self.nv = nv
        except Exception as exc:
            self.error = f"NVML unavailable: {type(exc).__name__}"

    def _poll(self):
        nv = self.nv
        while not self.stop_flag:
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)
                try:
                    reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                except Exception:
                    reasons = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                self.samples.append((float(mhz), int(reasons)))
            except Exception as exc:
                self.error = f"NVML query failed: {type(exc).__name__}"
                return
            time.sleep(0.002)

    def start(self):
        if self.nv is None:
            return
        self.stop_flag = False
        self.thread = threading.Thread(target=self._poll, daemon=True)
        self.thread.start()

    def stop(self):
        if self.nv is None or self.thread is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [self.error or "not started"], "samples": 0}
        self.stop_flag = True
        self.thread.join(timeout=1.0)
        nv = self.nv
        bits = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40,
                "hw_power_brake_slowdown": 0x80}
        mhz = sorted(m for m, _ in self.samples)
        seen = 0
        for _, r in self.samples:
            seen |= r
        reasons = sorted(name for name, bit in bits.items() if seen & bit)
        out = {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_min_mhz": mhz[0] if mhz else None,
               "sm_max_mhz": self.max_mhz, "reasons": reasons, "samples": len(mhz)}
        if self.error:
            out["note"] = self.error
        return out


# --------------------------------------------------------------------------- workloads
def make_c2(device, seed=0):
    """Contiguous M-grouped FP8 GEMM of BASELINE config 2 (tests/generators.py:378-419 of the reference)."""
    import torch
    import deepgemm_b200 as dg
    rnd = random.Random(seed)
    torch.manual_seed(seed)
    groups, n, k, alignment = 8, 4096, 7168, 128
    actual = [int(8192 * rnd.uniform(0.7, 1.3)) for _ in range(groups)]
    aligned = [(x + alignment - 1) // alignment * alignment for x in actual]
    m = sum(aligned)
    layout = torch.full((m,), -1, dtype=torch.int32)
    start = 0
    for i, (am, al) in enumerate(zip(actual, aligned)):
        layout[start:start + am] = i
        start += al
    a_q = torch.empty((m, k), dtype=torch.float8_e4m3fn, device=device)
    a_sf = torch.empty((m, k // 128), dtype=torch.float32, device=device)
    start = 0
    for am, al in zip(actual, aligned):                       # quantise per group to bound temporaries
        x = torch.randn((al, k), device=device, dtype=torch.bfloat16)
        x[am:] = 0
        q, s = dg.utils.per_token_cast_to_fp8(x, True, 128)
        a_q[start:start + al], a_sf[start:start + al] = q, s
        start += al
    b_q = torch.empty((groups, n, k), dtype=torch.float8_e4m3fn, device=device)
    b_sf = torch.empty((groups, n // 128, k // 128), dtype=torch.float32, device=device)
    for g in range(groups):
        w = torch.randn((n, k), device=device, dtype=torch.bfloat16)
        b_q[g], b_sf[g] = dg.utils.per_block_cast_to_fp8(w, True, 128)
    sfa = dg.transform_sf_into_required_layout(a_sf, m, k, (1, 128))
    sfb = dg.transform_sf_into_required_layout(b_sf, n, k, (128, 128), num_groups=groups)
    layout = layout.to(device)
    d = torch.empty((m, n), dtype=torch.bfloat16, device=device)
    flops = 2.0 * sum(actual) * n * k
    nbytes = m * k + groups * n * k + m * n * 2
    cfg = dict(workload="m_grouped_fp8_gemm_nt_contiguous (BASELINE config 2)", groups=groups, m=m,
               m_valid=sum(actual), n=n, k=k, alignment=alignment, a="e4m3 1x128 UE8M0", b="e4m3 128x128 UE8M0",
               out="bf16", sf="pre-packed int32", l2="inputs (1.2 GB) larger than L2")
    return dict(a=(a_q, sfa), b=(b_q, sfb), a_fp32_sf=a_sf, b_fp32_sf=b_sf, layout=layout, d=d, flops=flops, cfg=cfg,
                actual=actual, aligned=aligned, bytes=nbytes)


def run_c2(w):
    import deepgemm_b200 as dg
    dg.m_grouped_fp8_gemm_nt_contiguous(w["a"], w["b"], w["d"], w["layout"], recipe_a=(1, 128), recipe_b=(1, 128))


def time_steps(fn, steps, warmup, flush=None):
    """Per-step device times (ms) with CUDA events on the current stream."""
    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(steps):
        if flush is not None:
            flush.zero_()
        torch.cuda._sleep(200000)          # cover the host's enqueue latency: time the kernel, not the launch
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        e.synchronize()
        times.append(s.elapsed_time(e))
    return times


def other_configs(device, steps, warmup):
    """Kernel-only TFLOPS of the other single-GPU BASELINE configs (dense FP8, masked, FP8xFP4)."""
    import torch
    import deepgemm_b200 as dg
    out = {}
    flush = torch.empty(int(256e6), dtype=torch.int8, device=device)
    torch.manual_seed(0)
    # C1 dense 4096 x 4096 x 7168
    m, n, k = 4096, 4096, 7168
    a = dg.utils.per_token_cast_to_fp8(torch.randn((m, k), device=device, dtype=torch.bfloat16), True, 128)
    b = dg.utils.per_block_cast_to_fp8(torch.randn((n, k), device=device, dtype=torch.bfloat16), True, 128)
    sfa = dg.transform_sf_into_required_layout(a[1], m, k, (1, 128))
    sfb = dg.transform_sf_into_required_layout(b[1], n, k, (128, 128))
    d = torch.empty((m, n), dtype=torch.bfloat16, device=device)
    t = time_steps(lambda: dg.fp8_gemm_nt((a[0], sfa), (b[0], sfb), d, recipe_a=(1, 128), recipe_b=(1, 128)),
                   steps, warmup, flush)
    ms = sorted(t)[len(t) // 2]
    out["c1_dense_fp8_4096x4096x7168"] = dict(ms=ms, tflops=2.0 * m * n * k / ms / 1e9)
    # C4 FP8 x FP4 8192 x 7168 x 2048
    m, n, k = 8192, 7168, 2048
    a = dg.utils.per_token_cast_to_fp8(torch.randn((m, k), device=device, dtype=torch.bfloat16), True, 128)
    b = dg.utils.per_token_cast_to_fp4(torch.randn((n, k), device=device, dtype=torch.bfloat16) * 0.02, True, 32)
    sfa = dg.transform_sf_into_required_layout(a[1], m, k, (1, 128))
    sfb = dg.transform_sf_into_required_layout(b[1], n, k, (1, 32))
    d = torch.empty((m, n), dtype=torch.bfloat16, device=device)
    t = time_steps(lambda: dg.fp8_fp4_gemm_nt((a[0], sfa), (b[0], sfb), d, recipe_a=(1, 128), recipe_b=(1, 32)),
                   steps, warmup, flush)
    ms = sorted(t)[len(t) // 2]
    out["c4_fp8xfp4_8192x7168x2048"] = dict(ms=ms, tflops=2.0 * m * n * k / ms / 1e9)
    # C3 masked: 16 experts, max_m 1024, expected 256
    g, max_m, n, k = 16, 1024, 4096, 7168
    rnd = random.Random(0)
    masked = [min(max_m, int(256 * rnd.uniform(0.5, 1.5))) for _ in range(g)]
    a_q = torch.empty((g, max_m, k), dtype=torch.float8_e4m3fn, device=device)
    a_s = torch.empty((g, max_m, k // 128), dtype=torch.float32, device=device)
    b_q = torch.empty((g, n, k), dtype=torch.float8_e4m3fn, device=device)
    b_s = torch.empty((g, n // 128, k // 128), dtype=torch.float32, device=device)
    for i in range(g):
        a_q[i], a_s[i] = dg.utils.per_token_cast_to_fp8(torch.randn((max_m, k), device=device, dtype=torch.bfloat16), True, 128)
        a_s[i, masked[i]:] = 0
        b_q[i], b_s[i] = dg.utils.per_block_cast_to_fp8(torch.randn((n, k), device=device, dtype=torch.bfloat16), True, 128)
    sfa = dg.transform_sf_into_required_layout(a_s, max_m, k, (1, 128), num_groups=g)
    sfb = dg.transform_sf_into_required_layout(b_s, n, k, (128, 128), num_groups=g)
    mm = torch.tensor(masked, dtype=torch.int32, device=device)
    d = torch.empty((g, max_m, n), dtype=torch.bfloat16, device=device)
    t = time_steps(lambda: dg.m_grouped_fp8_gemm_nt_masked((a_q, sfa), (b_q, sfb), d, mm, 256, recipe_a=(1, 128),
                                                           recipe_b=(1, 128)), steps, warmup, flush)
    ms = sorted(t)[len(t) // 2]
    valid = sum(masked)
    nbytes = (a_q.numel() + d.numel() * 2) * valid / (g * max_m) + b_q.numel()
    out["c3_masked_16x(256 of 1024)x4096x7168"] = dict(ms=ms, tflops=2.0 * valid * n * k / ms / 1e9,
                                                       gbs=nbytes / ms / 1e6)
    del a_q, a_s, b_q, b_s, d
    # K-grouped TN (weight-gradient shape of the reference's tests, tests/generators.py:251-254): 4 groups,
    # D[g] = A[k_g, :]^T B[k_g, :], m 4096, n 7168, k 8192 per group, FP32 accumulate into D
    g, m, n, kk = 4, 4096, 7168, 8192
    ks = [kk] * g
    a = torch.empty((g * kk, m), dtype=torch.float8_e4m3fn, device=device)
    b = torch.empty((g * kk, n), dtype=torch.float8_e4m3fn, device=device)
    sa = torch.empty((g * kk // 128, m), dtype=torch.float32, device=device)
    sb = torch.empty((g * kk // 128, n), dtype=torch.float32, device=device)
    for i in range(g):
        r = slice(i * kk, (i + 1) * kk)
        rs = slice(i * kk // 128, (i + 1) * kk // 128)
        a[r], sa[rs] = dg.utils.per_channel_cast_to_fp8(torch.randn((kk, m), device=device, dtype=torch.bfloat16), True, 128)
        b[r], sb[rs] = dg.utils.per_channel_cast_to_fp8(torch.randn((kk, n), device=device, dtype=torch.bfloat16), True, 128)
    layout = torch.tensor(ks, dtype=torch.int32, device=device)
    d = torch.zeros((g, m, n), dtype=torch.float32, device=device)
    t = time_steps(lambda: dg.k_grouped_fp8_gemm_tn_contiguous((a, sa), (b, sb), d, ks, layout, c=d), steps, warmup, flush)
    ms = sorted(t)[len(t) // 2]
    out["k_grouped_tn_4x4096x7168x8192_fp32_accumulate"] = dict(ms=ms, tflops=2.0 * g * m * n * kk / ms / 1e9,
                                                                note="includes packing the FP32 scales (2 launches)")
    del a, b, sa, sb, d
    # Fused activation cast (BF16 -> E4M3 + UE8M0 scales in GEMM-ready layout): HBM bound, 3 + 1/gran bytes per element
    for rows, cols, gran in ((4096, 7168, 32), (65536, 7168, 128)):
        x = torch.randn((rows, cols), device=device, dtype=torch.bfloat16)
        q = torch.empty((rows, cols), dtype=torch.float8_e4m3fn, device=device)
        _, sf = dg.per_token_cast_to_fp8_fused(x, gran, "gemm", out=q)
        t = time_steps(lambda: dg.per_token_cast_to_fp8_fused(x, gran, "gemm", out=q, sf_out=sf), steps, warmup, flush)
        ms = sorted(t)[len(t) // 2]
        nbytes = rows * cols * (3.0 + 1.0 / gran)
        out[f"cast_bf16_to_fp8_1x{gran}_{rows}x{cols}"] = dict(ms=ms, gbs=nbytes / ms / 1e6)
        del x, q, sf
    return out



def mega_moe_bench(device, group, rank, world, steps, warmup, tokens=4096, experts_per_rank=32, topk=8, hidden=7168,
                   inter=2048, check_tokens=512, check_experts=2):
    """Mega MoE forward of BASELINE config 5 under weak scaling: 32 experts and 4096 tokens per GPU, top-8,
    hidden 7168, intermediate 2048; activations E4M3 with per-32 UE8M0 scales, expert weights MXFP4."""
    import torch
    import deepgemm_b200 as dg
    experts = experts_per_rank * world
    torch.manual_seed(1000 + rank)

    raw = []                     # (codes, FP32 scales) as quantised, kept for the CPU check

    def fp4(n, k, scale):
        q = torch.empty((experts_per_rank, n, k // 2), dtype=torch.int8, device=device)
        sf = torch.empty((experts_per_rank, n, k // 32), dtype=torch.float32, device=device)
        for e in range(experts_per_rank):
            q[e], sf[e] = dg.utils.per_token_cast_to_fp4(torch.randn((n, k), device=device, dtype=torch.bfloat16) * scale,
                                                         True, 32)
        raw.append((q, sf))
        return q, dg.transform_sf_into_required_layout(sf, n, k, (1, 32), experts_per_rank)

    l1, l2 = dg.transform_weights_for_mega_moe(fp4(2 * inter, hidden, 0.02), fp4(hidden, inter, 0.02))
    x = torch.randn((tokens, hidden), device=device, dtype=torch.bfloat16)
    x_fp8, x_sf = dg.utils.per_token_cast_to_fp8(x, True, 32, use_packed_ue8m0=True)
    w, idx = torch.topk(torch.randn((tokens, experts), device=device).softmax(-1), topk, dim=-1, sorted=False)
    w = (w / w.sum(-1, keepdim=True)).float()
    buf = dg.get_symm_buffer_for_mega_moe(group, experts, tokens, topk, hidden, inter)
    buf.x[:tokens].copy_(x_fp8), buf.x_sf[:tokens].copy_(x_sf)
    buf.topk_idx[:tokens].copy_(idx), buf.topk_weights[:tokens].copy_(w)
    y = torch.empty((tokens, hidden), dtype=torch.bfloat16, device=device)
    stats = torch.zeros(experts_per_rank, dtype=torch.int32, device=device)

    def step():
        dg.fp8_fp4_mega_moe(y, l1, l2, buf, cumulative_local_expert_recv_stats=stats)

    def barrier():
        if world > 1:
            group.barrier()
        torch.cuda.synchronize()

    def timed(fused):
        dg.mega.set_fused(fused)
        for _ in range(warmup):
            step()
        barrier()
        stats.zero_()
        times = []
        for _ in range(steps):
            barrier()
            # a ~0.5 ms device-side spin first: the host enqueues the events and the call while the GPU is still
            # busy, so the interval holds GPU time only, and the ranks' kernels start together
            # (deep_gemm/testing/bench.py:109-113 of the reference aligns ranks the same way)
            torch.cuda._sleep(1_000_000)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            step()
            e.record()
            e.synchronize()
            times.append(s.elapsed_time(e))
        barrier()
        dg.check_status()
        t = torch.tensor([sorted(times)[len(times) // 2]], device=device, dtype=torch.float64)
        rows = stats.sum().to(torch.float64) / steps
        if world > 1:
            import torch.distributed as dist
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dist.all_reduce(rows, op=dist.ReduceOp.MAX)
        return float(t.item()), float(rows.item())

    ms_phase, _ = timed(False)            # one launch per phase (7 kernels)
    y_phase = y.clone()
    ms, rows = timed(True)                # the library's default: one persistent kernel
    # full-size property: the two paths sum in the same order, so their outputs agree bit for bit on every rank
    agree = torch.tensor([1.0 if torch.equal(y, y_phase) and bool(torch.isfinite(y.float()).all()) else 0.0],
                         device=device, dtype=torch.float64)
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(agree, op=dist.ReduceOp.MIN)
    del y_phase
    # full-size parity sample against the CPU oracle (one GPU only): the contributions of the first `check_experts`
    # experts to the first `check_tokens` tokens, taken from the combine planes (one BF16 row per token and slot)
    # before the top-k reduction; those experts' weights are dequantised on the host
    parity = None
    if world == 1 and check_tokens > 0:
        import numpy as np
        from oracle import mega_moe as OM
        from oracle import quant as OQ

        class LazyDeq:
            def __init__(self, q, sf):
                self.q, self.sf, self.shape = q, sf, (q.size(0), q.size(1), q.size(2) * 2)

            def __getitem__(self, e):
                return OQ.cast_back_from_fp4(self.q[e].cpu().view(torch.uint8).numpy(), self.sf[e].cpu().numpy(), 32)

        n_chk = min(check_tokens, tokens)
        idx_sub = idx[:n_chk].clone()
        idx_sub[idx_sub >= check_experts] = -1                       # the oracle skips negative slots
        x_deq = OQ.cast_back_from_fp8(buf.x[:n_chk].cpu().view(torch.uint8).numpy(), buf.x_sf[:n_chk].cpu().numpy(), 32,
                                      use_packed_ue8m0=True)
        ref, counts = OM.mega_moe_reference(x_deq, idx_sub.cpu().numpy(), w[:n_chk].cpu().numpy(), LazyDeq(*raw[0]),
                                            LazyDeq(*raw[1]))
        mask = (idx_sub >= 0).t().unsqueeze(-1)                      # [topk, tokens, 1]
        got = (buf.combine[:, :n_chk].float() * mask).sum(0).to(torch.bfloat16).float().cpu().numpy()
        parity = dict(tokens=n_chk, experts=check_experts, rows=int(counts.sum()),
                      calc_diff=float(OQ.calc_diff(got, ref)), tolerance=2e-4)
    flops = 2.0 * rows * hidden * inter * 3
    buf.destroy()
    return dict(ep=world, tokens_per_rank=tokens, experts=experts, topk=topk, hidden=hidden, intermediate=inter,
                ms_per_step=ms, tokens_per_s=world * tokens / ms * 1e3, rows_per_rank_max=rows,
                tflops_per_gpu=flops / ms / 1e9, gpu_launches_per_step=1,
                paths_agree_bitwise=bool(agree.item() == 1.0), parity_vs_cpu_oracle=parity,
                per_phase_path=dict(ms_per_step=ms_phase, tokens_per_s=world * tokens / ms_phase * 1e3,
                                    gpu_launches_per_step=7),
                note="x: 1x32 UE8M0 E4M3 (the kernel's only recipe); weights MXFP4 ~N(0, 0.02); time = max over ranks, "
                     "median of per-step CUDA-event times; before each step a cross-rank barrier and a 0.5 ms device spin "
                     "that hides the host's enqueue latency")


def cpu_baseline_sample(w, budget_s=12.0, max_experts=6):
    """Oracle port on the host: whole experts of the workload (all valid rows of expert 0, 1, ...), each dequantised
    and multiplied in float32, until about `budget_s` seconds of CPU work are done.  Returns the baseline record,
    expert 0's result (the parity sample) and its row count."""
    import numpy as np
    import torch
    from oracle import gemm as OG
    n, k = w["cfg"]["n"], w["cfg"]["k"]
    threads = torch.get_num_threads()
    starts = np.concatenate([[0], np.cumsum(w["aligned"])])[:-1] if "aligned" in w else None
    a_all, sf_all = w["a"][0].view(torch.uint8), w["a_fp32_sf"]
    d0, rows0, done_rows, spent, used = None, 0, 0, 0.0, 0
    for g in range(min(max_experts, len(w["actual"]))):
        lo = int(starts[g]) if starts is not None else 0
        rows = int(w["actual"][g])
        a_bits, a_sf = a_all[lo:lo + rows].cpu().numpy(), sf_all[lo:lo + rows].cpu().numpy()
        b_bits, b_sf = w["b"][0][g].cpu().view(torch.uint8).numpy(), w["b_fp32_sf"][g].cpu().numpy()
        t0 = time.perf_counter()
        a = OG.dequant_operand(a_bits, a_sf, 1, 128, False)
        b = OG.dequant_operand(b_bits, b_sf, 128, 128, False)
        d = OG.gemm_nt_f32(a, b)
        spent += time.perf_counter() - t0
        done_rows += rows
        used += 1
        if g == 0:
            d0, rows0 = d, rows
        if spent >= budget_s or starts is None:
            break
    flops = 2.0 * done_rows * n * k
    return dict(value=flops / spent / 1e12, unit="TFLOPS", cores=threads, kind="port",
                sample=f"experts 0..{used - 1} of the workload, {done_rows} rows x N={n} x K={k}: dequantise + float32 "
                       f"BLAS matmul, {spent:.1f} s of host work"), d0, rows0


_JSON_FD = None


def keep_stdout_for_json():
    """Libraries (NCCL's version banner, torchrun's notices) print to file descriptor 1; the one JSON line must stand
    alone there, so everything else is sent to stderr and the line goes to a private copy of the descriptor."""
    global _JSON_FD
    sys.stdout.flush()
    _JSON_FD = os.dup(1)
    os.dup2(2, 1)


def emit(line):
    data = (json.dumps(line) + "\n").encode()
    sys.stdout.flush()
    if _JSON_FD is None:
        sys.stdout.write(data.decode()), sys.stdout.flush()
    else:
        os.write(_JSON_FD, data)


def main():
    keep_stdout_for_json()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--all-configs", action="store_true", help="also time the other single-GPU configs")
    ap.add_argument("--only", default="all", choices=["all", "gemm", "mega_moe"],
                    help="profiling aid: `gemm` runs the headline GEMM alone (no other configs, no Mega MoE, no CPU "
                         "baseline); `mega_moe` runs the Mega MoE forward alone and prints its record")
    ap.add_argument("--moe-tokens", type=int, default=4096, help="tokens per rank of the Mega MoE run")
    ap.add_argument("--moe-experts", type=int, default=32, help="experts per rank of the Mega MoE run")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        if rank != 0:
            return
        return reference_arm(args)

    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    import deepgemm_b200 as dg

    if args.only == "mega_moe":
        moe = mega_moe_bench(device, dist.group.WORLD if world > 1 else None, rank, world, max(1, min(args.steps, 10)),
                             args.warmup, tokens=args.moe_tokens, experts_per_rank=args.moe_experts)
        if rank == 0:
            emit({"mega_moe": moe})
        if world > 1:
            dist.destroy_process_group()
        return

    w = make_c2(device, seed=0)
    peaks = measured_peaks()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- kernel-only: inputs resident in HBM
    sampler = ClockSampler(device)
    for _ in range(args.warmup):
        run_c2(w)
    barrier()
    sampler.start()
    times = time_steps(lambda: run_c2(w), args.steps, 0)
    barrier()
    clocks = sampler.stop()
    dg.check_status()
    total_ms = sum(times)
    t = torch.tensor([total_ms], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = float(t.item()) / args.steps
    value = world * w["flops"] / ms_per_step / 1e9

    # ---- end to end through the public operator with host buffers
    a_host = w["a"][0].view(torch.uint8).cpu().pin_memory()
    sfa_store = torch.empty(w["a"][1].size(1) * w["a"][1].stride(1), dtype=torch.int32, device=device)
    sfa_dev = sfa_store.as_strided(w["a"][1].shape, w["a"][1].stride())
    sfa_dev.copy_(w["a"][1])
    sfa_host = sfa_store.cpu().pin_memory()
    layout_host = w["layout"].cpu().pin_memory()
    d_host = torch.empty(w["d"].shape, dtype=torch.bfloat16).pin_memory()
    a_dev = torch.empty_like(w["a"][0])
    layout_dev = torch.empty_like(w["layout"])

    # One expert's rows at a time on three streams (copy in, GEMM through the public operator, copy out), so that the
    # two PCIe directions and the GPU overlap; the scales and the layout (3 % of the bytes) go first in one piece.
    bounds, start = [], 0
    for al in w["aligned"]:
        bounds.append((start, start + al))
        start += al
    st_in, st_run, st_out = torch.cuda.Stream(device), torch.cuda.Stream(device), torch.cuda.Stream(device)
    ev_in = [torch.cuda.Event() for _ in bounds]
    ev_run = [torch.cuda.Event() for _ in bounds]
    ev_out = [torch.cuda.Event() for _ in bounds]
    ev_sf = torch.cuda.Event()
    a_dev8, d_dev = a_dev.view(torch.uint8), w["d"]
    d_one_piece = w["d"].clone()                     # the timed kernel-only run's result
    first = [True]

    def e2e_step():
        cur = torch.cuda.current_stream(device)
        for st in (st_in, st_run, st_out):
            st.wait_stream(cur)
        with torch.cuda.stream(st_in):
            if not first[0]:
                st_in.wait_event(ev_run[-1])            # the previous step's last GEMM has read the scales / layout
            sfa_store.copy_(sfa_host, non_blocking=True)
            layout_dev.copy_(layout_host, non_blocking=True)
            ev_sf.record(st_in)
            for i, (r0, r1) in enumerate(bounds):
                if not first[0]:
                    st_in.wait_event(ev_run[i])         # the previous step's GEMM has read these rows
                a_dev8[r0:r1].copy_(a_host[r0:r1], non_blocking=True)
                ev_in[i].record(st_in)
        with torch.cuda.stream(st_run):
            st_run.wait_event(ev_sf)
            for i, (r0, r1) in enumerate(bounds):
                st_run.wait_event(ev_in[i])
                if not first[0]:
                    st_run.wait_event(ev_out[i])        # the previous step's result rows have left
                dg.m_grouped_fp8_gemm_nt_contiguous((a_dev[r0:r1], sfa_dev[r0:r1]), w["b"], d_dev[r0:r1],
                                                    layout_dev[r0:r1], recipe_a=(1, 128), recipe_b=(1, 128))
                ev_run[i].record(st_run)
        with torch.cuda.stream(st_out):
            for i, (r0, r1) in enumerate(bounds):
                st_out.wait_event(ev_run[i])
                d_host[r0:r1].copy_(d_dev[r0:r1], non_blocking=True)
                ev_out[i].record(st_out)
        for st in (st_in, st_run, st_out):
            cur.wait_stream(st)
        first[0] = False

    e2e_steps = max(3, min(args.steps, 5))
    e2e_step()
    barrier()
    dg.check_status()
    e2e_parity = bool(torch.equal(d_host.to(device), d_one_piece))
    del d_one_piece
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(e2e_steps):
        e2e_step()
    e.record()
    barrier()
    e2e_ms = torch.tensor([s.elapsed_time(e) / e2e_steps], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
    e2e_value = world * w["flops"] / float(e2e_ms.item()) / 1e9
    h2d = a_host.numel() + sfa_host.numel() * 4 + layout_host.numel() * 4
    d2h = d_host.numel() * 2

    # ---- Mega MoE forward at EP = world (every rank takes part)
    del a_host, sfa_host, d_host, a_dev
    moe = None
    try:
        if args.only == "gemm":
            raise RuntimeError("skipped (--only gemm)")
        moe = mega_moe_bench(device, dist.group.WORLD if world > 1 else None, rank, world, max(3, min(args.steps, 10)),
                             args.warmup, tokens=args.moe_tokens, experts_per_rank=args.moe_experts)
        peak_fp8 = 2.0 * peaks["bf16"]
        moe["roofline_frac_of_2x_measured_bf16"] = moe["tflops_per_gpu"] / peak_fp8
        moe["roofline_frac_of_nominal_4500"] = moe["tflops_per_gpu"] / NOMINAL_FP8_TFLOPS
    except Exception as exc:   # reported, not hidden
        moe = {"error": f"{type(exc).__name__}: {exc}"}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- checks and baselines (rank 0)
    cpu, d_cpu, rows = cpu_baseline_sample(w) if (world == 1 and args.only == "all") else (None, None, 0)
    parity = None
    if d_cpu is not None:
        from oracle.quant import calc_diff
        parity = calc_diff(w["d"][:rows].float().cpu().numpy(), d_cpu)
    kernel_ms = sorted(times)[len(times) // 2]
    achieved = w["flops"] / kernel_ms / 1e9
    peak = 2.0 * peaks["bf16"]
    extra = other_configs(device, min(args.steps, 10), args.warmup) \
        if (args.all_configs or (world == 1 and args.only == "all")) else {}
    line = {
        "metric": "fp8_fp4_gemm_tflops", "value": value, "unit": "TFLOPS", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp8_e4m3 (fp32 accumulate, bf16 out)", "data": "synthetic",
        "config": dict(w["cfg"], replicas=world, parallelism="replicas only (no exchange step)"),
        "e2e": {"value": e2e_value, "unit": "TFLOPS", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "pipeline": "per-expert row blocks on 3 streams",
                "result_matches_device_run": e2e_parity,
                "ms_per_step": float(e2e_ms.item())},
        "gpu_launches": args.steps,
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                     "peak_source": f"2 x bf16_tflops of MEASURED_PEAKS.json ({peaks['source']}); FP8 UMMA issues at twice the BF16 rate",
                     "frac_of_nominal_4500": achieved / NOMINAL_FP8_TFLOPS,
                     "frac_of_2x_bf16_sustained": achieved / (2.0 * peaks["bf16_sustained"]),
                     "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH, "traffic_unit": "bytes per launch",
                     "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of this "
                                       "workload (profiles/gemm_bs_kernel_c2_grouped_contiguous.md)",
                     "algorithmic_bytes": w["bytes"], "kernel_ms": kernel_ms},
        "cpu_baseline": cpu,
        "clocks": clocks,
        "parity_calc_diff_vs_cpu_oracle": parity,
        "other_configs": extra,
        "mega_moe": moe,
    }
    emit(line)
    if world > 1:
        dist.destroy_process_group()


def reference_arm(args):
    """The reference's CPU-runnable formulation of the path (dequantise, then matmul) on the host cores."""
    import numpy as np
    import torch
    from oracle import gemm as OG
    from oracle import quant as OQ
    groups, n, k = 8, 4096, 7168
    rows = 2048
    rng = np.random.default_rng(0)
    x = OQ.bf16_round(rng.standard_normal((rows, k), dtype=np.float32))
    wt = OQ.bf16_round(rng.standard_normal((n, k), dtype=np.float32))
    a_bits, a_sf = OQ.per_token_cast_to_fp8(x, True, 128)
    b_bits, b_sf = OQ.per_block_cast_to_fp8(wt, True, 128)
    threads = torch.get_num_threads()

    def step():
        a = OG.dequant_operand(a_bits, a_sf, 1, 128, False)
        b = OG.dequant_operand(b_bits, b_sf, 128, 128, False)
        return OG.gemm_nt_f32(a, b)

    for _ in range(min(args.warmup, 1)):
        step()
    steps = max(1, min(args.steps, 5))
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    value = 2.0 * rows * n * k / dt / 1e12
    sample = f"{rows} rows of one expert x N={n} x K={k} per step (dequantise + float32 BLAS matmul), {steps} steps"
    line = {
        "impl": "reference", "metric": "fp8_fp4_gemm_tflops", "value": value, "unit": "TFLOPS", "n_gpus": args.gpus,
        "steps": steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "float32 on host", "data": "synthetic",
        "config": dict(workload="m_grouped_fp8_gemm_nt_contiguous (BASELINE config 2)", groups=groups, n=n, k=k,
                       note="the reference has no CPU GEMM; this is its tests' dequantise-then-matmul on a bounded sample"),
        "cpu_baseline": {"value": value, "unit": "TFLOPS", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    emit(line)


if __name__ == "__main__":
    main()
