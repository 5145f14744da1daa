"""GPU parity of the BF16 GEMM family (tcgen05 kind::f16 through the block-scaled kernel's layouts) against a float64
matmul of the same BF16 values, through the C ABI.

Cases after the reference's tests/test_bf16.py:23-196 (dense in all four majors with BF16 / FP32 output, accumulation
and alpha; M-grouped contiguous and PSUM; masked; K-grouped with empty groups, PSUM layout and accumulation) with its
bound `calc_diff < 1e-5`, plus the identities of tests/utils.py:20-79 (direct BF16 output == FP32 accumulation then
cast; stochastic rounding is a function of the FP32 result).
"""
from __future__ import annotations

import random

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

import deepgemm_b200 as dg
import helpers as H
from oracle import gemm as OG
from test_fp4_einsum_gpu import stochastic_expected

BF16_TOL = 1e-5


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    dg.check_status()


def T(c, bn, sw=1):
    return dict(cta_group=c, block_n=bn, swap=sw)


def randn(shape, seed, scale=1.0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(torch.bfloat16).cuda()


def f64(t):
    return t.float().cpu().numpy().astype(np.float64)


@pytest.mark.parametrize("tile", [None, T(1, 128), T(1, 256), T(2, 128), T(2, 256), T(2, 256, 2), T(2, 128, 2), T(1, 64, 2),
                                  T(1, 256, 2)])
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (300, 384, 200), (1000, 512, 1096), (4096, 256, 7168)])
def test_bf16_dense_nt(m, n, k, tile):
    a, b = randn((m, k), 1), randn((n, k), 2)
    d = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    if tile is None:
        dg.bf16_gemm_nt(a, b, d)
    else:
        if tile["swap"] == 2 and tile["cta_group"] == 2 and n % 256 != 0:
            pytest.skip("a CTA pair splits 256 weight rows")
        with H.force_tile(**tile):
            dg.bf16_gemm_nt(a, b, d)
    assert H.calc_diff(f64(d), OG.gemm_nt(f64(a), f64(b), cd_dtype="f32")) < BF16_TOL


@pytest.mark.parametrize("layout", ["nt", "nn", "tn", "tt"])
@pytest.mark.parametrize("out_dtype,accumulate,alpha", [(torch.bfloat16, False, None), (torch.float32, False, None),
                                                        (torch.float32, True, None), (torch.bfloat16, False, 0.37),
                                                        (torch.float32, False, -1.5)])
def test_bf16_dense_majors_outputs(layout, out_dtype, accumulate, alpha):
    m, n, k = 384, 640, 520
    a, b = randn((m, k), 3), randn((n, k), 4)
    ref = f64(a) @ f64(b).T * (1.0 if alpha is None else alpha)
    a_in = a if layout[0] == "n" else a.t().contiguous()            # given as [k, m] for t*
    b_in = b if layout[1] == "t" else b.t().contiguous()            # given as [k, n] for *n
    c = None
    d = torch.full((m, n), float("nan"), dtype=out_dtype, device="cuda")
    if accumulate:
        c = randn((m, n), 5).float()
        d = c.clone()
        ref = ref + f64(c)
        c = d
    getattr(dg, f"bf16_gemm_{layout}")(a_in, b_in, d, c=c, alpha=alpha)
    assert H.calc_diff(f64(d), ref) < BF16_TOL, (layout, out_dtype, accumulate, alpha)


def test_bf16_direct_output_is_fp32_accumulation_then_cast_and_stochastic_rounding():
    m, n, k = 300, 768, 1024
    a, b = randn((m, k), 6), randn((n, k), 7)
    acc = torch.zeros((m, n), dtype=torch.float32, device="cuda")
    dg.bf16_gemm_nt(a, b, acc, c=acc)
    d = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    dg.bf16_gemm_nt(a, b, d)
    dg.testing.assert_bitwise_equal(d, acc.to(torch.bfloat16), "direct BF16 output")
    sr = torch.empty_like(d)
    dg.bf16_gemm_nt(a, b, sr, epilogue=dg.epilogue.BF16StochasticRounding())
    dg.testing.assert_bitwise_equal(sr, stochastic_expected(acc), "stochastic rounding")
    assert not torch.equal(sr, d)
    for _ in range(5):                                   # bitwise determinism
        d2 = torch.empty_like(d)
        dg.bf16_gemm_nt(a, b, d2)
        assert torch.equal(d, d2)


def test_bf16_checks():
    a, b = randn((128, 64), 8), randn((128, 64), 9)
    d = torch.empty((128, 128), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="kBFloat16"):
        dg.bf16_gemm_nt(a.float(), b, d)
    with pytest.raises(RuntimeError, match="m == m_ and n == n_ and k == k_"):
        dg.bf16_gemm_nt(a, randn((128, 128), 1), d)
    with pytest.raises(RuntimeError, match="exclusive"):
        dg.bf16_gemm_nt(a, b, d, alpha=2.0, epilogue=dg.epilogue.Alpha(2.0))
    dg.bf16_gemm_nt(a[:0], b, d[:0])                     # empty problems return
    z = torch.full((128, 128), 3.0, dtype=torch.float32, device="cuda")
    dg.bf16_gemm_nt(a[:, :0], b[:, :0], z)               # k == 0: D = 0
    assert float(z.abs().max()) == 0.0


@pytest.mark.parametrize("use_psum", [False, True])
@pytest.mark.parametrize("major_b", ["k", "mn"])
def test_m_grouped_bf16_contiguous(use_psum, major_b):
    groups, n, k, align = 4, 512, 448, dg.get_mk_alignment_for_contiguous_layout()
    rnd = random.Random(11)
    sizes = [int(300 * rnd.uniform(0.7, 1.3)) for _ in range(groups)]
    aligned = [H.align_up(s, align) for s in sizes]
    m = sum(aligned)
    a = randn((m, k), 12)
    b = randn((groups, n, k), 13)
    layout = torch.full((m,), -1, dtype=torch.int32)
    ref = np.zeros((m, n))
    valid = np.zeros(m, dtype=bool)
    start, ends = 0, []
    for g, (s, al) in enumerate(zip(sizes, aligned)):
        layout[start:start + s] = g
        valid[start:start + s] = True
        ref[start:start + s] = f64(a[start:start + s]) @ f64(b[g]).T
        ends.append(start + s)
        start += al
    a[torch.from_numpy(~valid).cuda()] = 0
    d = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    gl = torch.tensor(ends, dtype=torch.int32).cuda() if use_psum else layout.cuda()
    if major_b == "k":
        dg.m_grouped_bf16_gemm_nt_contiguous(a, b, d, gl, use_psum_layout=use_psum)
    else:
        dg.m_grouped_bf16_gemm_nn_contiguous(a, b.transpose(1, 2).contiguous(), d, gl, use_psum_layout=use_psum)
    got = f64(d)
    assert H.calc_diff(got[valid], ref[valid]) < BF16_TOL
    if use_psum:
        assert not np.isnan(got).any() and np.all(got[~valid] == 0)     # ensure_zero_padding


def test_m_grouped_bf16_masked():
    groups, max_m, n, k = 6, 512, 768, 320
    rnd = random.Random(5)
    masked = [min(max_m, int(200 * rnd.uniform(0.3, 1.9))) for _ in range(groups)]
    a, b = randn((groups, max_m, k), 14), randn((groups, n, k), 15)
    d = torch.full((groups, max_m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    dg.m_grouped_bf16_gemm_nt_masked(a, b, d, torch.tensor(masked, dtype=torch.int32).cuda(), 200)
    ref = OG.m_grouped_masked(f64(a), f64(b), masked)
    for g in range(groups):
        assert H.calc_diff(f64(d[g, :masked[g]]), ref[g, :masked[g]]) < BF16_TOL, g


@pytest.mark.parametrize("use_psum", [False, True])
@pytest.mark.parametrize("accumulate,out_dtype", [(False, torch.bfloat16), (True, torch.float32), (False, torch.float32)])
def test_k_grouped_bf16_tn(use_psum, accumulate, out_dtype):
    m, n, k_align = 256, 384, dg.get_mk_alignment_for_contiguous_layout()
    real_ks = [256, 0, 384, 128] if not use_psum else [200, 0, 384, 77]
    if use_psum:
        ends, prev, bounds = [], 0, []
        for kk in real_ks:
            prev = H.align_up(prev, k_align) + kk
            ends.append(prev)
            bounds.append((prev - kk, prev))
        total = H.align_up(ends[-1], k_align)
        gl, ks_arg = torch.tensor(ends, dtype=torch.int32).cuda(), None
    else:
        bounds, pos = [], 0
        for kk in real_ks:
            bounds.append((pos, pos + kk))
            pos += kk
        total = pos
        gl, ks_arg = torch.tensor(real_ks, dtype=torch.int32).cuda(), real_ks
    a, b = torch.zeros((total, m), dtype=torch.bfloat16, device="cuda"), torch.zeros((total, n), dtype=torch.bfloat16, device="cuda")
    for i, (k0, k1) in enumerate(bounds):
        if k1 > k0:
            a[k0:k1], b[k0:k1] = randn((k1 - k0, m), 20 + i), randn((k1 - k0, n), 30 + i)
    g = len(real_ks)
    c = randn((g, m, n), 40).to(out_dtype) if accumulate else None
    d = c.clone() if accumulate else torch.full((g, m, n), float("nan"), dtype=out_dtype, device="cuda")
    dg.k_grouped_bf16_gemm_tn_contiguous(a, b, d, ks_arg, gl, c=d if accumulate else None, use_psum_layout=use_psum)
    for i, (k0, k1) in enumerate(bounds):
        ref = f64(a[k0:k1]).T @ f64(b[k0:k1]) + (f64(c[i]) if accumulate else 0.0)
        if k1 == k0 and not accumulate:
            assert float(d[i].float().abs().max()) == 0.0          # a group without K rows writes zeros
        else:
            assert H.calc_diff(f64(d[i]), ref) < BF16_TOL, (i, use_psum)
