"""GPU parity of the FP4 x FP4 (kind::mxf4) GEMMs, the batched FP8 GEMM behind fp8_einsum with its FP8-output and
stochastic-rounding epilogues, and programmatic dependent launch, all through the C ABI against the CPU oracle.

Mirrors the reference's tests/test_fp8_fp4.py (FP4 rows of enumerate_normal, the FP4 == FP8 identity :95-100, the
stochastic-rounding check :66-76), tests/test_einsum.py:128-265 and tests/utils.py:53-79.
Tolerances: calc_diff <= 5e-3 for FP4 operands and <= 1e-3 for FP8 against the dequantised oracle; quantised outputs
(E4M3 bytes, scale words, clamp counts) and stochastic rounding are bit-exact.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

import deepgemm_b200 as dg
import helpers as H
from deepgemm_b200.utils import math as M
from oracle import gemm as OG
from oracle import quant as OQ

FP8_TOL, FP4_TOL = 1e-3, 5e-3


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    dg.check_status()


def T(c, bn, sw=1):
    return dict(cta_group=c, block_n=bn, swap=sw)


def fp4_pair(rows, k, seed, scale=1.0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = (torch.randn((rows, k), generator=g) * scale).to(torch.bfloat16).cuda()
    q = M.per_token_cast_to_fp4(x, use_ue8m0=True, gran_k=32)
    return q, H.dequant(q[0], q[1], 1, 32)


def fp4_as_fp8(q):
    """The same values as E4M3 bytes (every E2M1 value is an E4M3 value; tests/utils.py:82-95 of the reference)."""
    codes = OQ.unpack_fp4_codes(H.to_np(q[0]))
    return torch.from_numpy(OQ.fp4_codes_to_e4m3_bits(codes)).cuda().view(torch.float8_e4m3fn), q[1]


# --------------------------------------------------------------------------- FP4 x FP4 dense
@pytest.mark.parametrize("m,n,k", [(256, 512, 1024), (300, 768, 2176), (128, 256, 128), (1000, 1280, 4096)])
@pytest.mark.parametrize("tile", [None, T(2, 256), T(2, 128), T(1, 256), T(1, 128), T(2, 256, 2), T(1, 64, 2)])
def test_fp4xfp4_dense(m, n, k, tile):
    (a, ref_a), (b, ref_b) = fp4_pair(m, k, m + k), fp4_pair(n, k, n + 3 * k, 0.02)
    d = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    with H.force_tile(**(tile or {})):
        dg.fp4_gemm_nt(a, b, d, recipe_a=(1, 32), recipe_b=(1, 32))
        again = torch.empty_like(d)
        dg.fp4_gemm_nt(a, b, again, recipe_a=(1, 32), recipe_b=(1, 32))
    got = H.to_np(d)
    assert not np.isnan(got).any()
    assert H.calc_diff(got, OG.gemm_nt(ref_a, ref_b)) < FP4_TOL
    assert torch.equal(d, again)


@pytest.mark.parametrize("out_dtype,accumulate", [(torch.float32, False), (torch.float32, True), (torch.bfloat16, False)])
def test_fp4xfp4_outputs_and_fp8_identity(out_dtype, accumulate):
    m, n, k = 512, 768, 2048
    (a, ref_a), (b, ref_b) = fp4_pair(m, k, 5), fp4_pair(n, k, 6, 0.02)
    d = torch.randn((m, n), device="cuda").to(out_dtype) if accumulate else \
        torch.full((m, n), float("nan"), dtype=out_dtype, device="cuda")
    c0 = H.to_np(d).astype(np.float32) if accumulate else None
    d8 = d.clone()
    dg.fp8_fp4_gemm_nt(a, b, d, c=d if accumulate else None, recipe_a=(1, 32), recipe_b=(1, 32))
    ref = OG.gemm_nt(ref_a, ref_b, c=c0, cd_dtype="f32" if out_dtype == torch.float32 else "bf16")
    assert H.calc_diff(H.to_np(d), ref) < FP4_TOL
    # the same values given as E4M3 bytes run on kind::mxf8f6f4 (UMMA K = 32 instead of 64): same result
    dg.fp8_fp4_gemm_nt(fp4_as_fp8(a), fp4_as_fp8(b), d8, c=d8 if accumulate else None, recipe_a=(1, 32), recipe_b=(1, 32))
    assert H.calc_diff(H.to_np(d), H.to_np(d8)) < 1e-14
    for _ in range(20):                                   # bitwise determinism (tests/test_fp8_fp4.py:78-82)
        again = torch.full((m, n), float("nan"), dtype=out_dtype, device="cuda")
        if accumulate:
            again.copy_(torch.from_numpy(c0).to(out_dtype))
        dg.fp8_fp4_gemm_nt(a, b, again, c=again if accumulate else None, recipe_a=(1, 32), recipe_b=(1, 32))
        assert torch.equal(again, d)


def test_fp4xfp4_known_answer_and_packed_scale_pitch():
    """All ones (E2M1 code 2 = 1.0, scale 1): every output is K.  Then pre-packed scales behind a padded, NaN-poisoned
    pitch give the same bits as compact ones (tests/utils.py:41-50 of the reference)."""
    m, n, k = 384, 512, 1536
    ones = torch.full((m, k // 2), 0x22, dtype=torch.int8, device="cuda")
    onesb = torch.full((n, k // 2), 0x22, dtype=torch.int8, device="cuda")
    d = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    dg.fp4_gemm_nt((ones, torch.ones((m, k // 32), device="cuda")), (onesb, torch.ones((n, k // 32), device="cuda")), d,
                   recipe_a=(1, 32), recipe_b=(1, 32))
    assert torch.equal(d, torch.full_like(d, k))
    (a, _), (b, _) = fp4_pair(m, k, 1), fp4_pair(n, k, 2, 0.02)
    sfa = dg.transform_sf_into_required_layout(a[1], m, k, (1, 32))
    sfb = dg.transform_sf_into_required_layout(b[1], n, k, (1, 32))
    want = torch.empty_like(d)
    dg.fp4_gemm_nt((a[0], sfa), (b[0], sfb), want, recipe_a=(1, 32), recipe_b=(1, 32))

    def padded(sf, mn):
        pitch = H.align_up(mn, 4) + 8
        store = torch.full((sf.size(1), pitch), -1, dtype=torch.int32, device="cuda")     # 0xFF bytes: UE8M0 NaN
        view = store.as_strided(sf.shape, (1, pitch))
        view.copy_(sf)
        return view

    dg.fp4_gemm_nt((a[0], padded(sfa, m)), (b[0], padded(sfb, n)), d, recipe_a=(1, 32), recipe_b=(1, 32))
    assert torch.equal(d, want)


# --------------------------------------------------------------------------- FP4 x FP4 grouped
@pytest.mark.parametrize("use_psum", [False, True])
def test_m_grouped_fp4_contiguous(use_psum):
    import random
    groups, n, k, alignment = 4, 512, 1024, 128
    rnd = random.Random(7)
    actual = [int(300 * rnd.uniform(0.7, 1.3)) for _ in range(groups)]
    aligned = [H.align_up(x, alignment) for x in actual]
    m = sum(aligned)
    g = torch.Generator(device="cpu").manual_seed(11)
    x = torch.randn((m, k), generator=g).to(torch.bfloat16)
    layout = torch.empty(groups if use_psum else m, dtype=torch.int32)
    ids = np.full(m, -1, dtype=np.int64)
    start = 0
    for i, (am, al) in enumerate(zip(actual, aligned)):
        x[start + am:start + al] = 0
        ids[start:start + am] = i
        if use_psum:
            layout[i] = start + am
        else:
            layout[start:start + am], layout[start + am:start + al] = i, -1
        start += al
    a = M.per_token_cast_to_fp4(x.cuda(), True, 32)
    bs = [fp4_pair(n, k, 20 + i, 0.02) for i in range(groups)]
    b = (torch.stack([q[0][0] for q in bs]), torch.stack([q[0][1] for q in bs]))
    d = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    dg.m_grouped_fp4_gemm_nt_contiguous(a, b, d, layout.cuda(), recipe_a=(1, 32), recipe_b=(1, 32), use_psum_layout=use_psum)
    ref = OG.m_grouped_contiguous(H.dequant(a[0], a[1], 1, 32), np.stack([q[1] for q in bs]), ids)
    got = H.to_np(d)
    assert H.calc_diff(got[ids >= 0], ref[ids >= 0]) < FP4_TOL


def test_m_grouped_fp4_masked():
    import random
    groups, max_m, n, k = 5, 512, 512, 1024
    rnd = random.Random(3)
    masked = [min(max_m, int(200 * rnd.uniform(0.5, 1.5))) for _ in range(groups)]
    qa = [fp4_pair(max_m, k, 40 + i) for i in range(groups)]
    qb = [fp4_pair(n, k, 60 + i, 0.02) for i in range(groups)]
    a = (torch.stack([q[0][0] for q in qa]), torch.stack([q[0][1] for q in qa]))
    b = (torch.stack([q[0][0] for q in qb]), torch.stack([q[0][1] for q in qb]))
    d = torch.full((groups, max_m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    dg.m_grouped_fp4_gemm_nt_masked(a, b, d, torch.tensor(masked, dtype=torch.int32, device="cuda"), 200,
                                    recipe_a=(1, 32), recipe_b=(1, 32))
    got = H.to_np(d)
    for i, mm in enumerate(masked):
        assert H.calc_diff(got[i, :mm], OG.gemm_nt(qa[i][1][:mm], qb[i][1])) < FP4_TOL, i


@pytest.mark.parametrize("use_psum", [False, True])
@pytest.mark.parametrize("accumulate,out_dtype", [(True, torch.float32), (False, torch.bfloat16)])
def test_k_grouped_fp4_nt(use_psum, accumulate, out_dtype):
    """k_grouped_fp4_gemm_nt_contiguous (tests/generators.py:488-520 of the reference): K-major packed operands with
    the groups along K, K alignment 256, scales compact by group [sum(k_g / 32), mn]; empty groups included."""
    old = dg.get_mk_alignment_for_contiguous_layout()
    try:
        dg.set_mk_alignment_for_contiguous_layout(256)
        m, n = 256, 512
        real_ks = [300, 0, 1024, 256, 0] if use_psum else [512, 0, 1024, 256, 0]
        aligned = [H.align_up(kk, 256) for kk in real_ks]
        ends, prev = [], 0
        for kk in real_ks:
            prev = H.align_up(prev, 256) + kk
            ends.append(prev)
        total = sum(aligned)
        g = torch.Generator(device="cpu").manual_seed(13)
        xa = torch.zeros((total, m), dtype=torch.bfloat16)
        xb = torch.zeros((total, n), dtype=torch.bfloat16)
        bounds = []
        for kk, end in zip(real_ks, ends):
            xa[end - kk:end] = torch.randn((kk, m), generator=g).to(torch.bfloat16)
            xb[end - kk:end] = (torch.randn((kk, n), generator=g) * 0.02).to(torch.bfloat16)
            bounds.append((end - kk, end))

        def cast(x):
            mn = x.size(1)
            data = torch.zeros((mn, total // 2), dtype=torch.int8, device="cuda")
            sfs, deq = [], np.zeros((mn, total), dtype=np.float32)
            for (k0, _), al in zip(bounds, aligned):
                if al == 0:
                    continue
                q, sf = M.per_token_cast_to_fp4(x[k0:k0 + al].t().contiguous().cuda(), True, 32)   # zero padding included
                data[:, k0 // 2:(k0 + al) // 2] = q
                sfs.append(sf.t().contiguous())
                deq[:, k0:k0 + al] = H.dequant(q, sf, 1, 32)
            return (data, torch.cat(sfs)), deq

        (qa, ref_a), (qb, ref_b) = cast(xa), cast(xb)
        groups = len(real_ks)
        d = torch.randn((groups, m, n), device="cuda").to(out_dtype) * 8 if accumulate else \
            torch.full((groups, m, n), float("nan"), dtype=out_dtype, device="cuda")
        c0 = H.to_np(d).astype(np.float32) if accumulate else None
        layout = torch.tensor(ends if use_psum else aligned, dtype=torch.int32, device="cuda")
        dg.k_grouped_fp4_gemm_nt_contiguous(qa, qb, d, aligned, layout, c=d if accumulate else None,
                                            use_psum_layout=use_psum)
        torch.cuda.synchronize()
        dg.check_status()
        got = H.to_np(d)
        assert not np.isnan(got).any()
        for i, (k0, k1) in enumerate(bounds):
            acc = ref_a[:, k0:k1].astype(np.float64) @ ref_b[:, k0:k1].astype(np.float64).T
            if accumulate:
                acc = acc + c0[i]
            want = OG.to_cd(acc, "f32" if out_dtype == torch.float32 else "bf16")
            if k1 == k0:
                assert np.array_equal(got[i], want), f"empty group {i}"
            else:
                assert H.calc_diff(got[i], want) < FP4_TOL, i
    finally:
        dg.set_mk_alignment_for_contiguous_layout(old)


# --------------------------------------------------------------------------- fp8_einsum
def stochastic_expected(fp32: torch.Tensor) -> torch.Tensor:
    """BF16 bits that stochastic rounding must give for these FP32 results (tests/utils.py:53-79 of the reference): the
    random 16 bits of each value come from a hash of its column quartet's four FP32 bit patterns and the quartet's
    index along the last axis."""
    v = fp32.contiguous().view(torch.int32).to(torch.int64) & 0xffffffff
    shape = fp32.shape
    v = v.view(*shape[:-1], -1, 4)
    q = torch.arange(shape[-1] // 4, device=fp32.device, dtype=torch.int64)
    h = (v[..., 0] * 0x5671d42b + v[..., 1] * 0x9995e499 + v[..., 2] * 0xace1b8a5 + v[..., 3] * 0xe153538d + q) & 0xffffffff
    h = (h ^ (h >> 23)) * 0x7feb352d & 0xffffffff
    h ^= h >> 16
    h1, h2 = h * 0x846ca68b & 0xffffffff, h * 0xd35a2d97 & 0xffffffff
    h1 ^= h1 >> 11
    h2 ^= h2 >> 11
    bits = torch.stack((h1 & 0xffff, h1 >> 16, h2 & 0xffff, h2 >> 16), dim=-1)
    rounded = ((v >> 16) + (((v & 0xffff) + bits) >> 16)) & 0xffff
    return rounded.to(torch.uint16).view(torch.bfloat16).view(shape)


def quant_bhx(x, gran=128):
    b, h, r = x.shape
    q, sf = M.per_token_cast_to_fp8(x.view(-1, r), use_ue8m0=True, gran_k=gran)
    return q.view(b, h, r), sf.view(b, h, -1)


def quant_hdr(y):
    h, d, r = y.shape
    q = torch.empty_like(y, dtype=torch.float8_e4m3fn)
    sf = torch.empty((h, (d + 127) // 128, (r + 127) // 128), device="cuda", dtype=torch.float32)
    for i in range(h):
        q[i], sf[i] = M.per_block_cast_to_fp8(y[i], use_ue8m0=True, gran_k=128)
    return q, sf


def deq_hdr(q, sf):
    return np.stack([H.dequant(q[i], sf[i], 128, 128) for i in range(q.size(0))])


@pytest.mark.parametrize("b", [4, 130, 512])
def test_fp8_einsum_bhr_hdr_bhd(b):
    h, r, d = 4, 512, 256
    torch.manual_seed(b)
    x = torch.randn((b, h, r), device="cuda", dtype=torch.bfloat16)
    y = torch.randn((h, d, r), device="cuda", dtype=torch.bfloat16)
    xq, yq = quant_bhx(x), quant_hdr(y)
    x_deq = H.dequant(xq[0].view(-1, r), xq[1].view(b * h, -1), 1, 128).reshape(b, h, r)
    ref = np.einsum("bhr,hdr->bhd", x_deq.astype(np.float64), deq_hdr(*yq).astype(np.float64))
    z = torch.full((b, h, d), float("nan"), dtype=torch.bfloat16, device="cuda")
    dg.fp8_einsum("bhr,hdr->bhd", xq, yq, z)
    assert H.calc_diff(H.to_np(z), ref) < FP8_TOL
    # FP32 accumulation into a permuted zero tensor, then stochastic rounding must be a function of exactly that
    tmp = torch.zeros((h, b, d), device="cuda", dtype=torch.float32).permute(1, 0, 2)
    dg.fp8_einsum("bhr,hdr->bhd", xq, yq, tmp, c=tmp)
    assert H.calc_diff(H.to_np(tmp), ref) < FP8_TOL
    z_sr = torch.empty_like(z)
    dg.fp8_einsum("bhr,hdr->bhd", xq, yq, z_sr, epilogue=dg.epilogue.BF16StochasticRounding())
    dg.testing.assert_bitwise_equal(z_sr, stochastic_expected(tmp.contiguous()), f"stochastic rounding b={b}")
    # FP8 output: bytes, packed scales and clamp count equal a BF16 D followed by the per-token cast
    out = torch.empty((b, h, d), dtype=torch.float8_e4m3fn, device="cuda")
    sfd = torch.empty_strided((b, (h * d + 127) // 128), (1, H.align_up(b, 4)), dtype=torch.int32, device="cuda")
    count = torch.empty(1, device="cuda", dtype=torch.uint32)
    for clamp in (None, 2.576 * r ** 0.5):
        expect = z if clamp is None else z.clamp(-clamp, clamp)
        ref_q, ref_sf = M.per_token_cast_to_fp8(expect.view(b, h * d), use_ue8m0=True, gran_k=32, use_packed_ue8m0=True)
        o_q, o_sf = OQ.per_token_cast_to_fp8(H.to_np(expect.view(b, h * d)), True, 32, use_packed_ue8m0=True)
        ref_count = 0 if clamp is None else int((z.abs() > clamp).sum().item())
        for counter in (None, count):
            if counter is not None:
                counter.fill_(0xffffffff)
            out.view(torch.uint8).fill_(0xAA)
            sfd.fill_(-1)
            if clamp is None and counter is None:
                dg.fp8_einsum("bhr,hdr->bhd", xq, yq, (out, sfd))
            else:
                dg.fp8_einsum("bhr,hdr->bhd", xq, yq, out,
                              epilogue=dg.epilogue.FP8CastWithClamp(sfd=sfd, clamp_value=clamp, clamped_count=counter))
            torch.cuda.synchronize()
            if counter is not None:
                assert int(counter.item()) == ref_count, (b, clamp)
            assert torch.equal(out.view(b, h * d).view(torch.uint8), ref_q.view(torch.uint8)), (b, clamp)
            assert torch.equal(sfd.contiguous(), ref_sf), (b, clamp)
            assert np.array_equal(H.to_np(out.view(b, h * d)), o_q) and np.array_equal(sfd.contiguous().cpu().numpy(), o_sf)
    if clamp is not None:
        assert ref_count > 0


@pytest.mark.parametrize("b", [4, 300])
def test_fp8_einsum_bhd_hdr_bhr(b):
    h, r, d = 4, 512, 256
    torch.manual_seed(b + 1)
    x = torch.randn((b, h, d), device="cuda", dtype=torch.bfloat16)
    y = torch.randn((h, d, r), device="cuda", dtype=torch.bfloat16)
    xq, yq = quant_bhx(x), quant_hdr(y)
    x_deq = H.dequant(xq[0].view(-1, d), xq[1].view(b * h, -1), 1, 128).reshape(b, h, d)
    ref = np.einsum("bhd,hdr->bhr", x_deq.astype(np.float64), deq_hdr(*yq).astype(np.float64))
    z = torch.full((b, h, r), float("nan"), dtype=torch.bfloat16, device="cuda")
    dg.fp8_einsum("bhd,hdr->bhr", xq, yq, z)
    assert H.calc_diff(H.to_np(z), ref) < FP8_TOL
    tmp = torch.zeros((h, b, r), device="cuda", dtype=torch.float32).permute(1, 0, 2)
    dg.fp8_einsum("bhd,hdr->bhr", xq, yq, tmp, c=tmp)
    z_sr = torch.empty_like(z)
    dg.fp8_einsum("bhd,hdr->bhr", xq, yq, z_sr, epilogue=dg.epilogue.BF16StochasticRounding())
    dg.testing.assert_bitwise_equal(z_sr, stochastic_expected(tmp.contiguous()), f"stochastic rounding b={b}")


def test_fp8_einsum_bhd_bhr_hdr():
    h, r, d, b = 4, 512, 256, 1024
    torch.manual_seed(9)
    x = torch.randn((b, h, d), device="cuda", dtype=torch.bfloat16)
    y = torch.randn((b, h, r), device="cuda", dtype=torch.bfloat16)
    z0 = torch.randn((h, d, r), device="cuda", dtype=torch.float32) * 10
    xq = M.per_channel_cast_to_fp8(x.view(b, -1), use_ue8m0=True, gran_k=128)
    yq = M.per_channel_cast_to_fp8(y.view(b, -1), use_ue8m0=True, gran_k=128)

    def deq(q, sf):
        return OQ.e4m3_bits_to_f32(H.to_np(q)) * np.repeat(H.to_np(sf), 128, axis=0)[:b]

    ref = H.to_np(z0).astype(np.float64) + np.einsum(
        "bhd,bhr->hdr", deq(*xq).reshape(b, h, d).astype(np.float64), deq(*yq).reshape(b, h, r).astype(np.float64))
    xq = (xq[0].view(b, h, d), xq[1].view(-1, h, d))
    yq = (yq[0].view(b, h, r), yq[1].view(-1, h, r))
    z = z0.clone()
    dg.fp8_einsum("bhd,bhr->hdr", xq, yq, z, c=z, recipe=(1, 1, 128))
    assert H.calc_diff(H.to_np(z), ref) < FP8_TOL
    with pytest.raises(RuntimeError, match="Unsupported einsum"):
        dg.fp8_einsum("bh,hr->br", xq, yq, z)


def test_dense_stochastic_rounding_epilogue():
    """tests/test_fp8_fp4.py:66-76 of the reference: the dense GEMM with BF16StochasticRounding equals the stochastic
    rounding of its own FP32-accumulated result."""
    m, n, k = 300, 768, 1024
    qa, qb, (ga, gmb, gb), _, _ = H.make_dense(m, n, k, seed=77)
    acc = torch.zeros((m, n), device="cuda", dtype=torch.float32)
    dg.fp8_gemm_nt(qa, qb, acc, c=acc)
    d = torch.empty((m, n), device="cuda", dtype=torch.bfloat16)
    dg.fp8_gemm_nt(qa, qb, d, epilogue=dg.epilogue.BF16StochasticRounding())
    dg.testing.assert_bitwise_equal(d, stochastic_expected(acc), "dense stochastic rounding")
    rn = torch.empty_like(d)
    dg.fp8_gemm_nt(qa, qb, rn)
    assert not torch.equal(rn, d) and (rn.float() - d.float()).abs().max() <= (rn.float().abs().max() * 2 ** -7)


# --------------------------------------------------------------------------- programmatic dependent launch
def test_pdl_gives_the_same_bits():
    """With set_pdl(True) the pack kernels and the GEMM of an FP32-scale call are launched with programmatic stream
    serialisation and wait in-kernel; results equal those of ordinary launches, call after call."""
    m, n, k = 1024, 2048, 2048
    qa, qb, _, ref_a, ref_b = H.make_dense(m, n, k, seed=5)
    want = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    dg.fp8_gemm_nt(qa, qb, want)
    x = torch.randn((m, k), device="cuda", dtype=torch.bfloat16)
    case = H.make_masked(4, 512, 200, 512, 1024, seed=4)
    dm = torch.zeros((4, 512, 512), dtype=torch.bfloat16, device="cuda")
    dg.m_grouped_fp8_fp4_gemm_nt_masked(case["a"], case["b"], dm, case["masked"], 200)
    try:
        assert not dg.get_pdl()
        dg.set_pdl(True)
        assert dg.get_pdl()
        for _ in range(10):
            got = torch.full_like(want, float("nan"))
            dg.fp8_gemm_nt(qa, qb, got)                       # pack A, pack B, GEMM: three dependent launches
            assert torch.equal(got, want)
            d2 = torch.zeros_like(dm)
            dg.m_grouped_fp8_fp4_gemm_nt_masked(case["a"], case["b"], d2, case["masked"], 200)
            for g_, mm in enumerate(case["masked_cpu"]):
                assert torch.equal(d2[g_, :mm], dm[g_, :mm])
            # a producer kernel right before its consumer: the fused cast feeding a GEMM
            q = dg.per_token_cast_to_fp8_fused(x, 128, "gemm")
            d3 = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
            dg.fp8_gemm_nt(q, qb, d3, recipe_a=(1, 128), recipe_b=(128, 128))
        torch.cuda.synchronize()
        dg.check_status()
    finally:
        dg.set_pdl(False)
    d4 = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    dg.fp8_gemm_nt(dg.per_token_cast_to_fp8_fused(x, 128, "gemm"), qb, d4, recipe_a=(1, 128), recipe_b=(128, 128))
    assert torch.equal(d3, d4)
