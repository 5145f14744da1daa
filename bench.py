"""Benchmark of the block-scaled GEMM hot path (one JSON line on stdout).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--all-configs]
                    [--only all|gemm|mega_moe|c1|c3|c4] [--tile CTA,BN,SWAP] [--moe-tokens T] [--moe-experts E]

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
`other_configs`: the other single-GPU configurations (dense FP8, masked grouped, FP8 x FP4, K-grouped), each timed
            alone and compared with the CPU oracle on a sample (`calc_diff`).
`mega_moe`: the Mega MoE forward at expert parallelism N with its own roofline, CPU-oracle parity on every rank
            and an end-to-end figure with host buffers.

With --gpus N > 1 the GEMM does not shard (no exchange step): N independent replicas run, one
per GPU, and `value` is the aggregate.  --impl reference times the reference's only CPU-runnable
formulation of this path (dequantise-then-matmul, here the oracle port) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import random
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

NOMINAL_FP8_TFLOPS = 4500.0
NVLINK_NOMINAL_GBS = 900.0
# DRAM traffic of one launch of the headline kernel: `dram__bytes_read.sum + dram__bytes_write.sum` of the ncu
# capture summarised in the named profile (ncu is not part of a run, so this is read from that file's table)
TRAFFIC_PROFILE = os.path.join("profiles", "gemm_bs_kernel_c2_grouped_contiguous.md")


def profile_traffic_bytes():
    """The `dram bytes per launch` figure of the committed ncu summary, or None when the file has no such line."""
    try:
        with open(os.path.join(ROOT, TRAFFIC_PROFILE)) as f:
            for line in f:
                if line.lower().startswith("dram_bytes_per_launch:"):
                    return float(line.split(":", 1)[1].split()[0])
    except OSError:
        pass
    return None


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
C2_GROUPS, C2_N, C2_K, C2_ALIGN = 8, 4096, 7168, 128


def c2_sizes(seed=0):
    """Rows per expert of BASELINE config 2 (tests/generators.py:383-408 of the reference): needs no GPU."""
    rnd = random.Random(seed)
    actual = [int(8192 * rnd.uniform(0.7, 1.3)) for _ in range(C2_GROUPS)]
    aligned = [(x + C2_ALIGN - 1) // C2_ALIGN * C2_ALIGN for x in actual]
    return actual, aligned


def c2_config(world):
    actual, aligned = c2_sizes()
    return dict(workload="m_grouped_fp8_gemm_nt_contiguous (BASELINE config 2)", groups=C2_GROUPS, m=sum(aligned),
                m_valid=sum(actual), n=C2_N, k=C2_K, alignment=C2_ALIGN, a="e4m3 1x128 UE8M0",
                b="e4m3 128x128 UE8M0", out="bf16", sf="pre-packed int32", l2="inputs (1.2 GB) larger than L2",
                replicas=world, parallelism="replicas only (no exchange step)")


def make_c2(device, seed=0):
    """Contiguous M-grouped FP8 GEMM of BASELINE config 2 (tests/generators.py:378-419 of the reference)."""
    import torch
    import deepgemm_b200 as dg
    torch.manual_seed(seed)
    groups, n, k = C2_GROUPS, C2_N, C2_K
    actual, aligned = c2_sizes(seed)
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
    return dict(a=(a_q, sfa), b=(b_q, sfb), a_fp32_sf=a_sf, b_fp32_sf=b_sf, layout=layout, d=d, flops=flops,
                actual=actual, aligned=aligned, bytes=nbytes, n=n, k=k)


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


def median(xs):
    return sorted(xs)[len(xs) // 2]


def np_of(t):
    import torch
    t = t.detach().cpu()
    if t.dtype in (torch.float8_e4m3fn, torch.int8):
        return t.contiguous().view(torch.uint8).numpy()
    return t.float().numpy() if t.dtype == torch.bfloat16 else t.numpy()


# ---- the other single-GPU configurations: each returns {ms, tflops, ..., calc_diff vs the CPU oracle on a sample}
def config_c1(device, steps, warmup, flush):
    """C1 dense FP8 4096 x 4096 x 7168; parity: the first 1024 rows against dequantise + float32 matmul."""
    import torch
    import deepgemm_b200 as dg
    from oracle import gemm as OG
    from oracle.quant import calc_diff
    torch.manual_seed(0)
    m, n, k = 4096, 4096, 7168
    a = dg.utils.per_token_cast_to_fp8(torch.randn((m, k), device=device, dtype=torch.bfloat16), True, 128)
    b = dg.utils.per_block_cast_to_fp8(torch.randn((n, k), device=device, dtype=torch.bfloat16), True, 128)
    sfa = dg.transform_sf_into_required_layout(a[1], m, k, (1, 128))
    sfb = dg.transform_sf_into_required_layout(b[1], n, k, (128, 128))
    d = torch.empty((m, n), dtype=torch.bfloat16, device=device)
    t = time_steps(lambda: dg.fp8_gemm_nt((a[0], sfa), (b[0], sfb), d, recipe_a=(1, 128), recipe_b=(1, 128)),
                   steps, warmup, flush)
    ms = median(t)
    rows = 1024
    ref = OG.gemm_nt_f32(OG.dequant_operand(np_of(a[0][:rows]), np_of(a[1][:rows]), 1, 128, False),
                         OG.dequant_operand(np_of(b[0]), np_of(b[1]), 128, 128, False))
    return dict(ms=ms, tflops=2.0 * m * n * k / ms / 1e9, calc_diff=float(calc_diff(np_of(d[:rows]), ref)),
                tolerance=1e-3, parity_sample=f"rows 0..{rows - 1}")


def config_c4(device, steps, warmup, flush):
    """C4 FP8 x FP4 8192 x 7168 x 2048; parity: the first 2048 rows."""
    import torch
    import deepgemm_b200 as dg
    from oracle import gemm as OG
    from oracle.quant import calc_diff
    torch.manual_seed(4)
    m, n, k = 8192, 7168, 2048
    a = dg.utils.per_token_cast_to_fp8(torch.randn((m, k), device=device, dtype=torch.bfloat16), True, 128)
    b = dg.utils.per_token_cast_to_fp4(torch.randn((n, k), device=device, dtype=torch.bfloat16) * 0.02, True, 32)
    sfa = dg.transform_sf_into_required_layout(a[1], m, k, (1, 128))
    sfb = dg.transform_sf_into_required_layout(b[1], n, k, (1, 32))
    d = torch.empty((m, n), dtype=torch.bfloat16, device=device)
    t = time_steps(lambda: dg.fp8_fp4_gemm_nt((a[0], sfa), (b[0], sfb), d, recipe_a=(1, 128), recipe_b=(1, 32)),
                   steps, warmup, flush)
    ms = median(t)
    rows = 2048
    ref = OG.gemm_nt_f32(OG.dequant_operand(np_of(a[0][:rows]), np_of(a[1][:rows]), 1, 128, False),
                         OG.dequant_operand(np_of(b[0]), np_of(b[1]), 1, 32, True))
    return dict(ms=ms, tflops=2.0 * m * n * k / ms / 1e9, calc_diff=float(calc_diff(np_of(d[:rows]), ref)),
                tolerance=5e-3, parity_sample=f"rows 0..{rows - 1}")


def config_c3(device, steps, warmup, flush):
    """C3 masked grouped FP8: 16 experts, max_m 1024, expected_m 256; HBM bound (470 MB of weights stream once).
    Parity: the valid rows of the shortest and the longest group."""
    import torch
    import deepgemm_b200 as dg
    from oracle import gemm as OG
    from oracle.quant import calc_diff
    torch.manual_seed(3)
    g, max_m, n, k = 16, 1024, 4096, 7168
    rnd = random.Random(0)
    masked = [min(max_m, int(256 * rnd.uniform(0.5, 1.5))) for _ in range(g)]
    if MASKED_ROWS_OVERRIDE:
        masked = [MASKED_ROWS_OVERRIDE] * g          # tuning aid: every group with the same number of rows
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
    ms = median(t)
    valid = sum(masked)
    nbytes = (a_q.numel() + d.numel() * 2) * valid / (g * max_m) + b_q.numel()
    worst = 0.0
    picks = sorted({masked.index(min(masked)), masked.index(max(masked))})
    for i in picks:
        r = masked[i]
        ref = OG.gemm_nt_f32(OG.dequant_operand(np_of(a_q[i, :r]), np_of(a_s[i, :r]), 1, 128, False),
                             OG.dequant_operand(np_of(b_q[i]), np_of(b_s[i]), 128, 128, False))
        worst = max(worst, float(calc_diff(np_of(d[i, :r]), ref)))
    peaks = measured_peaks()
    hbm_ms, tensor_ms = nbytes / peaks["hbm"] / 1e6, 2.0 * valid * n * k / (2.0 * peaks["bf16"]) / 1e9
    return dict(ms=ms, tflops=2.0 * valid * n * k / ms / 1e9, gbs=nbytes / ms / 1e6, valid_rows=valid, masked_m=masked,
                algorithmic_bytes=nbytes, roofline_ms=max(hbm_ms, tensor_ms), roofline_bound="hbm" if hbm_ms > tensor_ms else "tensor",
                roofline_frac=max(hbm_ms, tensor_ms) / ms, calc_diff=worst, tolerance=1e-3,
                parity_sample=f"valid rows of groups {picks}")


def config_k_grouped(device, steps, warmup, flush):
    """K-grouped TN (weight-gradient shape of the reference's tests, tests/generators.py:251-254): 4 groups,
    D[g] += A[k_g, :]^T B[k_g, :], m 4096, n 7168, k 8192 per group, FP32 accumulate into D."""
    import torch
    import deepgemm_b200 as dg
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
    ms = median(t)
    return dict(ms=ms, tflops=2.0 * g * m * n * kk / ms / 1e9, note="includes packing the FP32 scales (2 launches)")


def config_cast(device, steps, warmup, flush):
    """Fused activation cast (BF16 -> E4M3 + UE8M0 scales in GEMM-ready layout): HBM bound, 3 + 1/gran bytes/element."""
    import torch
    import deepgemm_b200 as dg
    out = {}
    for rows, cols, gran in ((4096, 7168, 32), (65536, 7168, 128)):
        x = torch.randn((rows, cols), device=device, dtype=torch.bfloat16)
        q = torch.empty((rows, cols), dtype=torch.float8_e4m3fn, device=device)
        _, sf = dg.per_token_cast_to_fp8_fused(x, gran, "gemm", out=q)
        t = time_steps(lambda: dg.per_token_cast_to_fp8_fused(x, gran, "gemm", out=q, sf_out=sf), steps, warmup, flush)
        ms = median(t)
        out[f"cast_bf16_to_fp8_1x{gran}_{rows}x{cols}"] = dict(ms=ms, gbs=rows * cols * (3.0 + 1.0 / gran) / ms / 1e6)
        del x, q, sf
    return out


def config_fp4(device, steps, warmup, flush):
    """FP4 x FP4 (kind::mxf4, twice the FP8 rate) 8192 x 7168 x 4096, MXFP4 1x32 on both sides; parity: 1024 rows."""
    import torch
    import deepgemm_b200 as dg
    from oracle import gemm as OG
    from oracle.quant import calc_diff
    torch.manual_seed(5)
    m, n, k = 8192, 7168, 4096
    a = dg.utils.per_token_cast_to_fp4(torch.randn((m, k), device=device, dtype=torch.bfloat16), True, 32)
    b = dg.utils.per_token_cast_to_fp4(torch.randn((n, k), device=device, dtype=torch.bfloat16) * 0.02, True, 32)
    sfa = dg.transform_sf_into_required_layout(a[1], m, k, (1, 32))
    sfb = dg.transform_sf_into_required_layout(b[1], n, k, (1, 32))
    d = torch.empty((m, n), dtype=torch.bfloat16, device=device)
    t = time_steps(lambda: dg.fp4_gemm_nt((a[0], sfa), (b[0], sfb), d, recipe_a=(1, 32), recipe_b=(1, 32)),
                   steps, warmup, flush)
    ms = median(t)
    rows = 1024
    ref = OG.gemm_nt_f32(OG.dequant_operand(np_of(a[0][:rows]), np_of(a[1][:rows]), 1, 32, True),
                         OG.dequant_operand(np_of(b[0]), np_of(b[1]), 1, 32, True))
    peak = 4.0 * measured_peaks()["bf16"]
    tf = 2.0 * m * n * k / ms / 1e9
    return dict(ms=ms, tflops=tf, frac_of_4x_measured_bf16=tf / peak, frac_of_nominal_9000=tf / 9000.0,
                calc_diff=float(calc_diff(np_of(d[:rows]), ref)), tolerance=5e-3, parity_sample=f"rows 0..{rows - 1}")


def config_bf16(device, steps, warmup, flush):
    """BF16 x BF16 (kind::f16, no scale factors) 4096 x 4096 x 7168 and the grouped form 8 x 8192 x 4096 x 7168's first
    expert shape 8192 x 4096 x 7168; parity: 1024 rows against a float64 matmul of the same BF16 values.  The fraction is
    against the measured cuBLAS BF16 figure itself."""
    import torch
    import deepgemm_b200 as dg
    from oracle.quant import calc_diff
    torch.manual_seed(6)
    peak = measured_peaks()["bf16"]
    out = {}
    for m, n, k in ((4096, 4096, 7168), (8192, 4096, 7168)):
        a = torch.randn((m, k), device=device, dtype=torch.bfloat16)
        b = torch.randn((n, k), device=device, dtype=torch.bfloat16)
        d = torch.empty((m, n), dtype=torch.bfloat16, device=device)
        ms = median(time_steps(lambda: dg.bf16_gemm_nt(a, b, d), steps, warmup, flush))
        rows = 1024
        ref = np_of(a[:rows]).astype("float64") @ np_of(b).astype("float64").T
        tf = 2.0 * m * n * k / ms / 1e9
        out[f"{m}x{n}x{k}"] = dict(ms=ms, tflops=tf, frac_of_measured_bf16=tf / peak, frac_of_nominal_2250=tf / 2250.0,
                                   calc_diff=float(calc_diff(np_of(d[:rows]), ref)), tolerance=1e-5,
                                   parity_sample=f"rows 0..{rows - 1}")
    return out


MASKED_ROWS_OVERRIDE = 0

CONFIGS = {"c1": ("c1_dense_fp8_4096x4096x7168", config_c1), "c4": ("c4_fp8xfp4_8192x7168x2048", config_c4),
           "c3": ("c3_masked_16x(256 of 1024)x4096x7168", config_c3),
           "kg": ("k_grouped_tn_4x4096x7168x8192_fp32_accumulate", config_k_grouped),
           "fp4": ("fp4xfp4_mxf4_8192x7168x4096", config_fp4), "bf16": ("bf16_dense", config_bf16)}


def other_configs(device, steps, warmup, which=("c1", "c4", "c3", "kg", "fp4", "bf16", "cast")):
    """Kernel-only figures of the other single-GPU configurations, each with its parity sample."""
    import gc
    import torch
    out = {}
    flush = torch.empty(int(256e6), dtype=torch.int8, device=device)
    peak = 2.0 * measured_peaks()["bf16"]
    for key in which:
        try:
            if key == "cast":
                out.update(config_cast(device, steps, warmup, flush))
                continue
            name, fn = CONFIGS[key]
            rec = fn(device, steps, warmup, flush)
            if "tflops" in rec and key not in ("fp4", "bf16"):
                rec["frac_of_2x_measured_bf16"] = rec["tflops"] / peak
                rec["frac_of_nominal_4500"] = rec["tflops"] / NOMINAL_FP8_TFLOPS
            out[name] = rec
        except Exception as exc:      # reported, not hidden
            out[CONFIGS.get(key, (key,))[0]] = {"error": f"{type(exc).__name__}: {exc}"}
        gc.collect()
        torch.cuda.empty_cache()
    return out


# --------------------------------------------------------------------------- Mega MoE
def nvlink_probe(device, group, rank, world, buf, nbytes=256 << 20):
    """Inbound NVLink bandwidth seen by this GPU with the access pattern the forward uses: a kernel of this library
    reads `nbytes` of the next rank's symmetric buffer with plain 16-byte loads into local memory, all ranks at once.
    Returns GB/s (max time over ranks), or None with one rank."""
    import torch
    import torch.distributed as dist
    from deepgemm_b200 import _lib
    if world == 1:
        return None
    nbytes = min(nbytes, buf.buffer.numel() // 2 // 256 * 256)
    peer = int(buf.handle.buffer_ptrs[(rank + 1) % world])
    dst = torch.empty(nbytes, dtype=torch.int8, device=device)
    stream = torch.cuda.current_stream(device).cuda_stream
    best = None
    for it in range(4):
        group.barrier()
        torch.cuda.synchronize()
        torch.cuda._sleep(1_000_000)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        _lib.check(_lib.lib().dg_debug_copy(dst.data_ptr(), peer, nbytes, stream))
        e.record()
        e.synchronize()
        ms = s.elapsed_time(e)
        if it > 0:
            best = ms if best is None else min(best, ms)
    t = torch.tensor([best], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return nbytes / float(t.item()) / 1e6


def moe_trace_summary(t, num_ctas, ms):
    """Text summary of the time stamps a -DDG_TRACE build of the single-kernel Mega MoE forward leaves per CTA and warp:
    [cta][warp or 18 (epilogue cycles) or 19 (clock64 at the stamps)][slot]; slots 0-4 = %globaltimer at kernel start,
    roles begin, roles end, reduce begin, end; 5-7 = cycles spent in that warp's waits."""
    import numpy as np
    t = t.reshape(-1, 20, 8).astype(np.float64)[:num_ctas]
    starts = t[:, :17, 0]          # rows 17-19 hold other things than the warps' stamps
    t0 = starts[starts > 0].min()
    out = ["event-timed step: %.1f us; %d CTAs; times in us after the first CTA's start (min / median / max over CTAs)" % (ms * 1e3, num_ctas)]
    names = ["kernel start", "roles begin (scatter, exchange, layout done)", "roles end", "reduce begin (barriers passed)", "end"]
    for w, role in ((0, "weight-copy warp"), (1, "UMMA warp"), (4, "epilogue warp 4"), (2, "pull warp 2")):
        for s in range(5):
            v = t[:, w, s]
            v = v[v > 0]
            if len(v):
                out.append("%-17s %-45s %8.1f %8.1f %8.1f" % (role, names[s], (v.min() - t0) / 1e3, (np.median(v) - t0) / 1e3, (v.max() - t0) / 1e3))
    waits = {0: ("weight-copy warp", ("pulled / l1_done counters", "stage empty", "-")),
             3: ("scale-copy warp", ("pulled / l1_done counters", "stage empty", "-")),
             1: ("UMMA warp", ("accumulator empty", "stage full", "-")),
             4: ("epilogue warp 4", ("accumulator full", "staging buffer", "pulled / l1_done counters")),
             13: ("epilogue warp 13", ("accumulator full", "staging buffer", "pulled / l1_done counters"))}
    out.append("cycles spent waiting, thousands (min / median / max over CTAs):")
    for w, (role, what) in waits.items():
        for i, s in enumerate((5, 6, 7)):
            v = t[:, w, s][0::2] if w == 1 else t[:, w, s]      # the leader CTA of a pair issues the UMMAs
            if what[i] != "-":
                out.append("%-17s %-28s %9.1f %9.1f %9.1f" % (role, what[i], v.min() / 1e3, np.median(v) / 1e3, v.max() / 1e3))
    out.append("epilogue warp 4, cycles per part, thousands (median): per-token table %.1f, tcgen05.ld %.1f, staging %.1f, "
               "layer-1 chunks %.1f, layer-2 chunks %.1f, layer-1 fence + counter %.1f"
               % tuple(np.median(t[:, 18, s]) / 1e3 for s in range(6)))
    fine = ("scatter done", "grid barrier 1 passed", "exchange done (CTA 0: counts out, cross-rank barrier 1, layout, tile table)",
            "layout seen", "grid barrier 2 passed", "cross-rank barrier 2 passed (CTA 0)")
    out.append("thread 0 of every CTA, us after the first CTA's start (min / median / max):")
    for s, name in enumerate(fine):
        v = t[:, 17, s]
        v = v[v > 0]
        if len(v):
            out.append("  %-88s %8.1f %8.1f %8.1f" % (name, (v.min() - t0) / 1e3, (np.median(v) - t0) / 1e3, (v.max() - t0) / 1e3))
    cyc, ns = t[:, 19, :5], t[:, 0, :5]
    for a, b, name in ((0, 1, "prologue"), (1, 2, "roles"), (3, 4, "reduce")):
        d = ns[:, b] - ns[:, a]
        f = (cyc[:, b] - cyc[:, a]) / np.maximum(d, 1.0)
        out.append("%-8s median %7.1f us, SM clock %.3f GHz (clock64 / %%globaltimer), %.0f k cycles"
                   % (name, np.median(d) / 1e3, np.median(f), np.median(cyc[:, b] - cyc[:, a]) / 1e3))
    return "\n".join(out) + "\n"


def mega_moe_bench(device, group, rank, world, steps, warmup, tokens=4096, experts_per_rank=32, topk=8, hidden=7168,
                   inter=2048, check_tokens=2048, trace_path=None):
    """Mega MoE forward of BASELINE config 5 under weak scaling: 32 experts and 4096 tokens per GPU, top-8,
    hidden 7168, intermediate 2048; activations E4M3 with per-32 UE8M0 scales, expert weights MXFP4."""
    import torch
    import torch.distributed as dist
    import deepgemm_b200 as dg
    experts = experts_per_rank * world

    def raw_expert(e, layer):
        """MXFP4 codes and FP32 scales of global expert e; its own seed, so that any rank can rebuild any expert."""
        g = torch.Generator(device=device)
        g.manual_seed(7000 + 2 * e + layer)
        n, k = (2 * inter, hidden) if layer == 0 else (hidden, inter)
        return dg.utils.per_token_cast_to_fp4(torch.randn((n, k), device=device, dtype=torch.bfloat16, generator=g) * 0.02,
                                              True, 32)

    def local_weights(layer):
        n, k = (2 * inter, hidden) if layer == 0 else (hidden, inter)
        q = torch.empty((experts_per_rank, n, k // 2), dtype=torch.int8, device=device)
        sf = torch.empty((experts_per_rank, n, k // 32), dtype=torch.float32, device=device)
        for e in range(experts_per_rank):
            q[e], sf[e] = raw_expert(rank * experts_per_rank + e, layer)
        return q, dg.transform_sf_into_required_layout(sf, n, k, (1, 32), experts_per_rank)

    l1, l2 = dg.transform_weights_for_mega_moe(local_weights(0), local_weights(1))
    torch.manual_seed(1000 + rank)
    x = torch.randn((tokens, hidden), device=device, dtype=torch.bfloat16)
    w, idx = torch.topk(torch.randn((tokens, experts), device=device).softmax(-1), topk, dim=-1, sorted=False)
    w = (w / w.sum(-1, keepdim=True)).float()
    buf = dg.get_symm_buffer_for_mega_moe(group, experts, tokens, topk, hidden, inter)
    buf.load_tokens(x, idx, w)           # fused cast to E4M3 + per-32 UE8M0 straight into the buffer
    y = torch.empty((tokens, hidden), dtype=torch.bfloat16, device=device)
    stats = torch.zeros(experts_per_rank, dtype=torch.int32, device=device)

    def step():
        dg.fp8_fp4_mega_moe(y, l1, l2, buf, cumulative_local_expert_recv_stats=stats)

    def barrier():
        if world > 1:
            group.barrier()
        torch.cuda.synchronize()

    def reduce(value, op):
        t = torch.tensor([value], device=device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=op)
        return float(t.item())

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
        rows = float(stats.sum().item()) / steps
        return reduce(median(times), dist.ReduceOp.MAX), reduce(rows, dist.ReduceOp.MAX), stats.clone()

    ms_phase, _, _ = timed(False)            # one launch per phase (7 kernels)
    y_phase = y.clone()
    ms, rows, stats_fused = timed(True)      # the library's default: one persistent kernel
    if trace_path:
        # one more step of the single kernel with its time stamps switched on (needs the -DDG_TRACE build:
        # python -m deepgemm_b200.build --trace, DEEPGEMM_B200_LIB=deepgemm_b200/lib/libdeepgemm_b200_trace.so)
        import ctypes
        from deepgemm_b200 import _lib
        if not hasattr(_lib.lib(), "dg_debug_set_trace"):
            raise RuntimeError("--trace needs the library built with -DDG_TRACE (python -m deepgemm_b200.build --trace)")
        set_trace = _lib.lib().dg_debug_set_trace
        set_trace.argtypes, set_trace.restype = [ctypes.c_void_p], None
        trace = torch.zeros(256 * 20 * 8, dtype=torch.int64, device=device)
        barrier()
        set_trace(trace.data_ptr())
        torch.cuda._sleep(1_000_000)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        step()
        e.record()
        e.synchronize()
        set_trace(None)
        barrier()
        with open("%s.ep%d.rank%d.txt" % (trace_path, world, rank), "w") as f:
            f.write(moe_trace_summary(trace.cpu().numpy(), _lib.lib().dg_get_mega_moe_num_sms() // 2 * 2, s.elapsed_time(e)))
    # full-size property: the two paths sum in the same order, so their outputs agree bit for bit on every rank
    agree = reduce(1.0 if torch.equal(y, y_phase) and bool(torch.isfinite(y.float()).all()) else 0.0, dist.ReduceOp.MIN)
    del y_phase

    # integer-exact: rows received per local expert == histogram of every rank's routing, once per timed step
    if world > 1:
        all_idx = [torch.empty_like(idx) for _ in range(world)]
        dist.all_gather(all_idx, idx.contiguous())
        all_idx = torch.cat(all_idx)
    else:
        all_idx = idx
    lo = rank * experts_per_rank
    hist = torch.bincount(all_idx.flatten(), minlength=experts)[lo:lo + experts_per_rank].to(torch.int32)
    stats_exact = reduce(1.0 if torch.equal(stats_fused, hist * steps) else 0.0, dist.ReduceOp.MIN) == 1.0

    # parity against the CPU oracle on EVERY rank: the contributions of the first expert of rank 0 and the last expert
    # of the last rank (local for one rank, across NVLink for the others) to this rank's first `check_tokens` tokens,
    # read from the combine planes (one BF16 row per token and slot) before the top-k reduction.  Every rank rebuilds
    # those two experts from their seeds and dequantises them on the host.
    parity = None
    if check_tokens > 0:
        from oracle import mega_moe as OM
        from oracle import quant as OQ
        check_experts = sorted({0, experts - 1})

        class LazyDeq:
            def __init__(self, layer):
                self.layer = layer
                n, k = (2 * inter, hidden) if layer == 0 else (hidden, inter)
                self.shape = (experts, n, k)

            def __getitem__(self, e):
                q, sf = raw_expert(int(e), self.layer)
                return OQ.cast_back_from_fp4(np_of(q), np_of(sf), 32)

        n_chk = min(check_tokens, tokens)
        idx_sub = idx[:n_chk].clone()
        keep = torch.zeros_like(idx_sub, dtype=torch.bool)
        for e in check_experts:
            keep |= idx_sub == e
        idx_sub[~keep] = -1                                           # the oracle skips negative slots
        x_deq = OQ.cast_back_from_fp8(np_of(buf.x[:n_chk]), buf.x_sf[:n_chk].cpu().numpy(), 32, use_packed_ue8m0=True)
        ref, counts = OM.mega_moe_reference(x_deq, idx_sub.cpu().numpy(), w[:n_chk].cpu().numpy(), LazyDeq(0), LazyDeq(1))
        mask = keep.t().unsqueeze(-1)                                 # [topk, tokens, 1]
        got = (buf.combine[:, :n_chk].float() * mask).sum(0).to(torch.bfloat16).float().cpu().numpy()
        diff = float(OQ.calc_diff(got, ref)) if counts.sum() > 0 else 0.0
        parity = dict(tokens_per_rank=n_chk, experts=check_experts, rows_min_over_ranks=int(reduce(float(counts.sum()), dist.ReduceOp.MIN)),
                      calc_diff=reduce(diff, dist.ReduceOp.MAX), tolerance=2e-4, stats_exact=stats_exact,
                      ranks_checked=world)

    # end to end through the public API with HOST buffers: pinned BF16 tokens + routing in, load_tokens (fused cast),
    # forward, y out to pinned memory, every step
    x_host, idx_host, w_host = x.cpu().pin_memory(), idx.cpu().pin_memory(), w.cpu().pin_memory()
    y_host = torch.empty(y.shape, dtype=y.dtype).pin_memory()
    x_dev, idx_dev, w_dev = torch.empty_like(x), torch.empty_like(idx), torch.empty_like(w)

    def e2e_step():
        x_dev.copy_(x_host, non_blocking=True), idx_dev.copy_(idx_host, non_blocking=True), w_dev.copy_(w_host, non_blocking=True)
        buf.load_tokens(x_dev, idx_dev, w_dev)
        step()
        y_host.copy_(y, non_blocking=True)

    e2e_step()
    barrier()
    e2e_n = max(3, min(steps, 5))
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    s.record()
    for _ in range(e2e_n):
        e2e_step()
    e.record()
    barrier()
    dg.check_status()
    e2e_ms = reduce(s.elapsed_time(e) / e2e_n, dist.ReduceOp.MAX)
    e2e_ok = bool(torch.equal(y_host.to(device), y))

    nvlink = nvlink_probe(device, group, rank, world, buf)
    flops = 2.0 * rows * hidden * inter * 3
    peaks = measured_peaks()
    compute_ms = flops / (2.0 * peaks["bf16"]) / 1e9
    remote = (world - 1) / world
    bytes_in = remote * rows * (hidden + hidden // 32 + 4) + remote * rows * hidden * 2   # pulled rows + pushed results
    nvlink_ms = bytes_in / nvlink / 1e6 if nvlink else 0.0
    bound_ms = max(compute_ms, nvlink_ms)
    buf.destroy()
    return dict(ep=world, tokens_per_rank=tokens, experts=experts, topk=topk, hidden=hidden, intermediate=inter,
                ms_per_step=ms, tokens_per_s=world * tokens / ms * 1e3, rows_per_rank_max=rows,
                tflops_per_gpu=flops / ms / 1e9, gpu_launches_per_step=1,
                roofline=dict(compute_ms=compute_ms, nvlink_ms=nvlink_ms, bound="nvlink" if nvlink_ms > compute_ms else "tensor",
                              frac=bound_ms / ms, nvlink_in_bytes_per_rank=bytes_in, nvlink_measured_gbs=nvlink,
                              nvlink_nominal_gbs=NVLINK_NOMINAL_GBS,
                              compute_peak="2 x bf16_tflops of MEASURED_PEAKS.json (%s)" % peaks["source"],
                              frac_of_nominal_4500=flops / NOMINAL_FP8_TFLOPS / 1e9 / ms),
                paths_agree_bitwise=bool(agree == 1.0), parity_vs_cpu_oracle=parity,
                e2e=dict(ms_per_step=e2e_ms, tokens_per_s=world * tokens / e2e_ms * 1e3,
                         h2d_bytes_per_step=x_host.numel() * 2 + idx_host.numel() * 8 + w_host.numel() * 4,
                         d2h_bytes_per_step=y_host.numel() * 2, result_matches_device_run=e2e_ok,
                         path="pinned BF16 tokens -> load_tokens (fused FP8 cast) -> forward -> y to pinned host"),
                per_phase_path=dict(ms_per_step=ms_phase, tokens_per_s=world * tokens / ms_phase * 1e3,
                                    gpu_launches_per_step=7),
                note="x: 1x32 UE8M0 E4M3 (the kernel's only recipe); weights MXFP4 ~N(0, 0.02); time = max over ranks, "
                     "median of per-step CUDA-event times; before each step a cross-rank barrier and a 0.5 ms device spin "
                     "that hides the host's enqueue latency")


# --------------------------------------------------------------------------- CPU side
def host_threads():
    """All the host cores, whatever OMP_NUM_THREADS says (torchrun sets it to 1 for its children)."""
    n = os.cpu_count() or 1
    try:
        n = len(os.sched_getaffinity(0))
    except Exception:
        pass
    return n


class cpu_sample:
    """The CPU oracle on a bounded sample of config 2: `rows` rows of one expert against that expert's 4096 x 7168
    weight, both dequantised ONCE (outside the timed step), the float32 BLAS contraction timed per step."""

    def __init__(self, rows=2048, seed=0):
        import numpy as np
        from oracle import gemm as OG
        from oracle import quant as OQ
        rng = np.random.default_rng(seed)
        x = OQ.bf16_round(rng.standard_normal((rows, C2_K), dtype=np.float32))
        wt = OQ.bf16_round(rng.standard_normal((C2_N, C2_K), dtype=np.float32))
        a_bits, a_sf = OQ.per_token_cast_to_fp8(x, True, 128)
        b_bits, b_sf = OQ.per_block_cast_to_fp8(wt, True, 128)
        self.a = OG.dequant_operand(a_bits, a_sf, 1, 128, False)
        self.b = OG.dequant_operand(b_bits, b_sf, 128, 128, False)
        self.rows, self.flops, self.OG = rows, 2.0 * rows * C2_N * C2_K, OG
        self.sample = (f"{rows} rows of one expert x N={C2_N} x K={C2_K} per step: float32 BLAS matmul of the dequantised "
                       "operands (dequantised once, outside the step)")

    def step(self):
        return self.OG.gemm_nt_f32(self.a, self.b)


def run_cpu_sample(steps, warmup, budget_s=30.0):
    from threadpoolctl import threadpool_limits
    threads = host_threads()
    with threadpool_limits(limits=threads):
        smp = cpu_sample()
        for _ in range(max(1, min(warmup, 2))):
            smp.step()
        times = []
        t_all = time.perf_counter()
        for _ in range(steps):
            t0 = time.perf_counter()
            smp.step()
            times.append(time.perf_counter() - t0)
            if time.perf_counter() - t_all > budget_s * 4:
                break
    dt = sum(times) / len(times)
    return smp, dt, len(times), threads


def cpu_parity_c2(w):
    """Expert 0's valid rows of the timed workload against the CPU oracle (dequantise + float32 matmul)."""
    import numpy as np
    import torch
    from oracle import gemm as OG
    from oracle.quant import calc_diff
    rows = int(w["actual"][0])
    a = OG.dequant_operand(np_of(w["a"][0][:rows]), w["a_fp32_sf"][:rows].cpu().numpy(), 1, 128, False)
    b = OG.dequant_operand(np_of(w["b"][0][0]), w["b_fp32_sf"][0].cpu().numpy(), 128, 128, False)
    return float(calc_diff(np_of(w["d"][:rows]), OG.gemm_nt_f32(a, b))), rows


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
    ap.add_argument("--all-configs", action="store_true", help="also time the other single-GPU configs at N > 1")
    ap.add_argument("--only", default="all", choices=["all", "gemm", "mega_moe"] + sorted(CONFIGS),
                    help="profiling aid: `gemm` runs the headline GEMM alone (no other configs, no Mega MoE, no CPU "
                         "baseline); `mega_moe` the Mega MoE forward alone; c1 / c3 / c4 / kg / fp4 one other config alone")
    ap.add_argument("--tile", default="", help="tuning aid: cta_group,block_n,swap (0 = automatic) pinned for every GEMM")
    ap.add_argument("--trace", default="", help="with --only mega_moe and a -DDG_TRACE build of the library: write the single "
                                                "kernel's per-CTA time stamps, summarised, to <this>.ep<N>.rank<r>.txt")
    ap.add_argument("--masked-rows", type=int, default=0, help="tuning aid: config c3 with this many rows in every group")
    ap.add_argument("--moe-tokens", type=int, default=4096, help="tokens per rank of the Mega MoE run")
    ap.add_argument("--moe-experts", type=int, default=32, help="experts per rank of the Mega MoE run")
    ap.add_argument("--sustained-s", type=float, default=1.0, help="length of the back-to-back loop of the headline kernel")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        if rank != 0:
            return
        return reference_arm(args, world)

    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    import deepgemm_b200 as dg
    from deepgemm_b200 import _lib
    if args.tile:
        cta, bn, swap = (int(v) for v in args.tile.split(","))
        _lib.check(_lib.lib().dg_debug_set_tile_override(cta, bn, swap))
    global MASKED_ROWS_OVERRIDE
    MASKED_ROWS_OVERRIDE = args.masked_rows

    if args.only == "mega_moe":
        moe = mega_moe_bench(device, dist.group.WORLD if world > 1 else None, rank, world, max(1, min(args.steps, 10)),
                             args.warmup, tokens=args.moe_tokens, experts_per_rank=args.moe_experts,
                             trace_path=args.trace or None)
        if rank == 0:
            emit({"mega_moe": moe})
        if world > 1:
            dist.destroy_process_group()
        return
    if args.only in CONFIGS:
        out = other_configs(device, max(1, min(args.steps, 10)), args.warmup, which=(args.only,))
        if rank == 0:
            emit({"other_configs": out, "tile": args.tile or "automatic", "masked_rows": args.masked_rows or "config"})
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
    d_one_piece = w["d"].clone()                     # the timed kernel-only run's result

    # ---- the same kernel back to back for >= 1 s (no sleeps, no host syncs): the figure under the power cap,
    # with the SM clock NVML reports while it runs
    sustained = None
    if args.sustained_s > 0 and args.only != "gemm":
        n_loop = max(10, int(args.sustained_s * 1e3 / median(times)))
        sampler2 = ClockSampler(device)
        barrier()
        sampler2.start()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(n_loop):
            run_c2(w)
        e.record()
        barrier()
        clk = sampler2.stop()
        loop_ms = torch.tensor([s.elapsed_time(e) / n_loop], device=device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(loop_ms, op=dist.ReduceOp.MAX)
        v = world * w["flops"] / float(loop_ms.item()) / 1e9
        sustained = dict(value=v, unit="TFLOPS", launches=n_loop, ms_per_launch=float(loop_ms.item()),
                         frac_of_2x_bf16_sustained=v / world / (2.0 * peaks["bf16_sustained"]), clocks=clk,
                         ms_x_mhz=(float(loop_ms.item()) * clk["sm_mhz"]) if clk.get("sm_mhz") else None,
                         isolated_ms_x_mhz=(median(times) * clocks["sm_mhz"]) if clocks.get("sm_mhz") else None)

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
    del a_host, sfa_host, d_host, a_dev

    # ---- parity of the timed workload against the CPU oracle, on every run (rank 0; the replicas compute the same)
    parity, parity_rows = (None, 0)
    if rank == 0 and args.only == "all":
        run_c2(w)
        torch.cuda.synchronize()
        parity, parity_rows = cpu_parity_c2(w)

    # ---- Mega MoE forward at EP = world (every rank takes part)
    moe = None
    try:
        if args.only == "gemm":
            raise RuntimeError("skipped (--only gemm)")
        moe = mega_moe_bench(device, dist.group.WORLD if world > 1 else None, rank, world, max(3, min(args.steps, 10)),
                             args.warmup, tokens=args.moe_tokens, experts_per_rank=args.moe_experts)
    except Exception as exc:   # reported, not hidden
        moe = {"error": f"{type(exc).__name__}: {exc}"}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- baselines (rank 0)
    cpu = None
    if world == 1 and args.only == "all":
        smp, dt, n_done, threads = run_cpu_sample(steps=10, warmup=1)
        cpu = dict(value=smp.flops / dt / 1e12, unit="TFLOPS", cores=threads, kind="port",
                   sample=f"{smp.sample}; {n_done} steps, {dt * 1e3:.0f} ms each")
    kernel_ms = median(times)
    achieved = w["flops"] / kernel_ms / 1e9
    peak = 2.0 * peaks["bf16"]
    extra = other_configs(device, min(args.steps, 10), args.warmup) \
        if (args.all_configs or (world == 1 and args.only == "all")) else {}
    traffic = profile_traffic_bytes()
    line = {
        "metric": "fp8_fp4_gemm_tflops", "value": value, "unit": "TFLOPS", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp8_e4m3 (fp32 accumulate, bf16 out)", "data": "synthetic",
        "config": c2_config(world),
        "value_sustained": sustained,
        "e2e": {"value": e2e_value, "unit": "TFLOPS", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "pipeline": "per-expert row blocks on 3 streams", "result_matches_device_run": e2e_parity,
                "ms_per_step": float(e2e_ms.item()),
                "bound": "PCIe: the BF16 result (d2h bytes) leaves at the host link's rate; with N replicas on one host "
                         "the ranks share the host's copy bandwidth, so this figure does not scale with N"},
        "gpu_launches": args.steps,
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                     "peak_source": f"2 x bf16_tflops of MEASURED_PEAKS.json ({peaks['source']}); FP8 UMMA issues at twice the BF16 rate",
                     "frac_of_nominal_4500": achieved / NOMINAL_FP8_TFLOPS,
                     "frac_of_2x_bf16_sustained": achieved / (2.0 * peaks["bf16_sustained"]),
                     "traffic": traffic, "traffic_unit": "bytes per launch",
                     "traffic_source": f"dram_bytes_per_launch of {TRAFFIC_PROFILE} (dram__bytes_read.sum + "
                                       "dram__bytes_write.sum of one ncu capture of this workload)",
                     "algorithmic_bytes": w["bytes"], "kernel_ms": kernel_ms},
        "cpu_baseline": cpu,
        "clocks": clocks,
        "parity_calc_diff_vs_cpu_oracle": parity,
        "parity_sample": f"expert 0's {parity_rows} valid rows" if parity is not None else None,
        "other_configs": extra,
        "mega_moe": moe,
    }
    emit(line)
    if world > 1:
        dist.destroy_process_group()


def reference_arm(args, world):
    """The reference's CPU-runnable formulation of the path (its tests' dequantise-then-matmul; the reference has no
    CPU GEMM and cannot be built here) on all the host cores: the same bounded sample of config 2 as the
    `cpu_baseline` leg of the other arm, the same number of steps as asked for."""
    smp, dt, n_done, threads = run_cpu_sample(steps=max(1, args.steps), warmup=args.warmup)
    value = smp.flops / dt / 1e12
    line = {
        "impl": "reference", "metric": "fp8_fp4_gemm_tflops", "value": value, "unit": "TFLOPS", "n_gpus": args.gpus,
        "steps": n_done, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "float32 on host", "data": "synthetic",
        "config": c2_config(world),
        "cpu_baseline": {"value": value, "unit": "TFLOPS", "cores": threads, "kind": "port", "sample": smp.sample},
        "e2e": {"value": value, "unit": "TFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "each step is a bounded sample of the workload (the whole of config 2 is 3.85 TFLOP, about 10 s on these "
                "cores); TFLOPS does not depend on the sample's size",
    }
    emit(line)


if __name__ == "__main__":
    main()
