"""GPU parity tests: the CUDA path (through the C ABI) against the CPU oracle.

Tolerances: scale packing, layouts and routing are bit-exact; GEMM outputs must reach
calc_diff <= 1e-3 (FP8) and <= 5e-3 (FP8 x FP4) against the dequantise-then-matmul oracle.
The cases mirror the reference's tests/test_fp8_fp4.py and tests/test_layout.py.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

import deepgemm_b200 as dg
import helpers as H
from oracle import gemm as OG
from oracle import layout as OL
from oracle import quant as OQ

FP8_TOL, FP4_TOL = 1e-3, 5e-3


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    dg.check_status()


def T(c, bn, sw=1):
    return dict(cta_group=c, block_n=bn, swap=sw)


# --------------------------------------------------------------------------- SF layout kernels (bit-exact)
@pytest.mark.parametrize("mn,k,gran,batches", [(128, 512, 128, 1), (4097, 7168, 128, 1), (4096, 7296, 32, 2),
                                                 (64, 128, 128, 4), (333, 1211 * 32, 32, 1), (1, 7168, 128, 1)])
def test_sf_pack_matches_oracle(mn, k, gran, batches):
    g = torch.Generator().manual_seed(mn + k)
    e = torch.randint(1, 254, (batches, mn, (k + gran - 1) // gran), generator=g, dtype=torch.int32)
    sf = (e << 23).view(torch.float32)
    sf = sf[0] if batches == 1 else sf
    for transposed_input in (False, True):
        src = sf.cuda()
        if transposed_input:
            src = src.transpose(-1, -2).contiguous().transpose(-1, -2)
        out = dg.get_mn_major_tma_aligned_packed_ue8m0_tensor(src)
        ref = OL.packed_ue8m0_mn_major(sf.numpy())
        assert np.array_equal(out.cpu().numpy(), np.ascontiguousarray(ref))
        amn, pk = (mn + 3) // 4 * 4, out.size(-1)
        assert tuple(out.stride()) == ((1, amn) if out.dim() == 2 else (pk * amn, 1, amn))


def test_sf_pack_block_broadcast_and_transform():
    n, k = 4096, 7168
    g = torch.Generator().manual_seed(3)
    e = torch.randint(100, 140, (n // 128, k // 128), generator=g, dtype=torch.int32)
    sf = (e << 23).view(torch.float32)
    out = dg.transform_sf_into_required_layout(sf.cuda(), n, k, (1, 128, 128), is_sfa=False)
    ref = OL.packed_ue8m0_mn_major(OL.broadcast_block_sf(sf.numpy(), n, 128))
    assert np.array_equal(out.cpu().numpy(), np.ascontiguousarray(ref))


def test_sf_pack_psum_gap_rows_are_zero():
    old = dg.get_mk_alignment_for_contiguous_layout()
    try:
        for alignment, counts, sf_k in ((128, [64, 64], 2), (128, [5, 0, 129, 17], 3), (256, [255, 1, 257, 0, 33], 7)):
            dg.set_mk_alignment_for_contiguous_layout(alignment)
            ends, mn = [], 0
            for c in counts:
                ends.append(mn + c)
                mn += H.align_up(c, alignment)
            g = torch.Generator().manual_seed(mn)
            e = torch.randint(1, 240, (mn, sf_k), generator=g, dtype=torch.int32)
            sf = (e << 23).view(torch.float32)
            valid = OL.psum_valid_rows(ends, alignment, mn)
            poisoned = sf.clone()
            poisoned[torch.from_numpy(~valid)] = float("nan")
            layout = torch.tensor(ends, dtype=torch.int32, device="cuda")
            out = dg.get_mn_major_tma_aligned_packed_ue8m0_tensor(poisoned.cuda(), layout)
            ref = OL.packed_ue8m0_mn_major_psum(sf.numpy(), ends, alignment)
            assert np.array_equal(out.cpu().numpy(), np.ascontiguousarray(ref))
            strided = poisoned.cuda().t().contiguous().t()
            with pytest.raises(RuntimeError, match="allow_strided_psum_scales"):
                dg.get_mn_major_tma_aligned_packed_ue8m0_tensor(strided, layout)
            out2 = dg.get_mn_major_tma_aligned_packed_ue8m0_tensor(strided, layout, allow_strided_psum_scales=True)
            assert torch.equal(out, out2)
    finally:
        dg.set_mk_alignment_for_contiguous_layout(old)


@pytest.mark.parametrize("gran_k,k_alignment", [(32, 128), (128, 128), (128, 256), (32, 384)])
def test_sf_pack_k_grouped(gran_k, k_alignment):
    import random
    rnd = random.Random(gran_k + k_alignment)
    mn = 4096
    ks = [H.align_up(int(rnd.uniform(0.7, 1.3) * 1024), k_alignment) for _ in range(9)]
    ks[3] = 0
    rows = sum(k // gran_k for k in ks)
    g = torch.Generator().manual_seed(rows)
    sf = (torch.randint(1, 254, (rows, mn), generator=g, dtype=torch.int32) << 23).view(torch.float32)
    layout = torch.tensor(ks, dtype=torch.int32, device="cuda")
    out = dg.get_k_grouped_mn_major_tma_aligned_packed_ue8m0_tensor(sf.cuda(), layout, ks, gran_k, k_alignment)
    ref = OL.k_grouped_packed_ue8m0(sf.numpy(), ks, gran_k)
    assert out.shape == ref.shape and np.array_equal(out.cpu().numpy(), ref)


@pytest.mark.parametrize("gran_k,k_alignment", [(128, 128), (32, 128), (128, 256), (32, 384)])
def test_sf_pack_k_grouped_psum(gran_k, k_alignment):
    """The PSUM form (tests/test_layout.py:268-304 of the reference): the layout holds cumulative un-aligned K ends,
    every group's scale rows cover its aligned extent; with and without the host-side list of aligned sizes."""
    mn = 1024
    real_ks = [200, 0, 1000, 128, 513, 0, 77, 640]
    aligned = [H.align_up(k, k_alignment) for k in real_ks]
    ends, prev = [], 0
    for k in real_ks:
        prev = H.align_up(prev, k_alignment) + k
        ends.append(prev)
    rows = sum(al // gran_k for al in aligned)
    g = torch.Generator().manual_seed(rows)
    sf = (torch.randint(1, 254, (rows, mn), generator=g, dtype=torch.int32) << 23).view(torch.float32)
    layout = torch.tensor(ends, dtype=torch.int32, device="cuda")
    ref = OL.k_grouped_packed_ue8m0(sf.numpy(), aligned, gran_k)
    out = dg.get_k_grouped_mn_major_tma_aligned_packed_ue8m0_tensor(sf.cuda(), layout, aligned, gran_k, k_alignment,
                                                                    use_psum_layout=True)
    assert out.shape == ref.shape and np.array_equal(out.cpu().numpy(), ref)
    for ks_cpu in (None, []):                      # sizes not known on the host: a safe upper bound of rows
        out2 = dg.get_k_grouped_mn_major_tma_aligned_packed_ue8m0_tensor(sf.cuda(), layout, ks_cpu, gran_k,
                                                                         k_alignment, use_psum_layout=True)
        assert out2.size(0) >= ref.shape[0] and np.array_equal(out2[:ref.shape[0]].cpu().numpy(), ref)


# --------------------------------------------------------------------------- dense GEMM
def run_dense(m, n, k, *, gran_a=128, b_kind="fp8_block", tile=None, out_dtype=torch.bfloat16, packed=False,
              accumulate=False, alpha=None, mn_major=(False, False), alias=False, scale_b=1.0):
    qa, qb, (ga, gmb, gb), ref_a, ref_b = H.make_dense(m, n, k, gran_a=gran_a, b_kind=b_kind, seed=m + 3 * n + 7 * k,
                                                       scale_b=scale_b)
    (a_data, a_sf), (b_data, b_sf) = qa, qb
    rec = dict(recipe_a=(1, ga), recipe_b=(gmb, gb))
    if packed:
        a_sf = dg.transform_sf_into_required_layout(a_sf, m, k, (1, ga))
        b_sf = dg.transform_sf_into_required_layout(b_sf, n, k, (gmb, gb))
        rec = dict(recipe_a=(1, ga), recipe_b=(1, gb))
    if mn_major[0]:
        a_data = a_data.t().contiguous().t()
    if mn_major[1]:
        b_data = b_data.t().contiguous().t()
    d = torch.full((m, n), float("nan"), dtype=out_dtype, device="cuda")
    c = cref = None
    if accumulate:
        c = torch.randn((m, n), dtype=out_dtype, device="cuda") * 32
        cref = H.to_np(c).astype(np.float32)
        d = c
    fn, a_arg, b_arg = dg.fp8_fp4_gemm_nt, (a_data, a_sf), (b_data, b_sf)
    if alias:
        name = "fp8_fp4_gemm_" + ("t" if mn_major[0] else "n") + ("n" if mn_major[1] else "t")
        fn = getattr(dg, name)
        if mn_major[0]:
            a_arg = (a_data.t(), a_sf.t())
        if mn_major[1]:
            b_arg = (b_data.t(), b_sf.t())
    with H.force_tile(**(tile or {})):
        fn(a_arg, b_arg, d, c=c, alpha=alpha, **rec)
    torch.cuda.synchronize()
    ref = OG.gemm_nt(ref_a, ref_b, c=cref, alpha=1.0 if alpha is None else alpha,
                     cd_dtype="bf16" if out_dtype == torch.bfloat16 else "f32")
    return H.to_np(d), ref


@pytest.mark.parametrize("tile", [T(1, 128), T(1, 256), T(2, 128), T(2, 256), T(1, 128, 2), T(2, 128, 2),
                                  T(2, 256, 2), T(1, 64, 2), T(2, 64, 2), None])
@pytest.mark.parametrize("shape", [(128, 128, 128), (256, 512, 1024), (200, 328, 640), (1, 256, 512),
                                   (1024, 1024, 7168)])
def test_dense_fp8_all_tiles(tile, shape):
    m, n, k = shape
    d, ref = run_dense(m, n, k, tile=tile)
    assert not np.isnan(d).any()
    assert H.calc_diff(d, ref) < FP8_TOL


@pytest.mark.parametrize("gran_a,b_kind,tol", [(128, "fp8_row128", FP8_TOL), (32, "fp8_row32", FP8_TOL),
                                               (32, "fp8_block", FP8_TOL), (128, "fp4", FP4_TOL), (32, "fp4", FP4_TOL)])
@pytest.mark.parametrize("tile", [T(1, 128), T(2, 256), T(2, 128, 2)])
def test_dense_recipes(gran_a, b_kind, tol, tile):
    d, ref = run_dense(384, 512, 2048, gran_a=gran_a, b_kind=b_kind, tile=tile, packed=(b_kind != "fp8_block"),
                       scale_b=0.02 if b_kind == "fp4" else 1.0)
    assert H.calc_diff(d, ref) < tol


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("accumulate", [False, True])
@pytest.mark.parametrize("tile", [T(1, 128), T(2, 256)])
def test_dense_output_modes(out_dtype, accumulate, tile):
    d, ref = run_dense(256, 384, 1024, out_dtype=out_dtype, accumulate=accumulate, tile=tile, b_kind="fp8_row128")
    assert H.calc_diff(d, ref) < FP8_TOL
    d, ref = run_dense(256, 384, 1024, out_dtype=out_dtype, alpha=-0.37, tile=tile)
    assert H.calc_diff(d, ref) < FP8_TOL


@pytest.mark.parametrize("mn_major", [(True, False), (False, True), (True, True)])
@pytest.mark.parametrize("alias", [False, True])
def test_dense_mn_major_and_aliases(mn_major, alias):
    for tile in (T(1, 128), T(2, 256)):
        d, ref = run_dense(512, 512, 1024, mn_major=mn_major, alias=alias, tile=tile, b_kind="fp8_row128")
        assert H.calc_diff(d, ref) < FP8_TOL


def test_direct_output_equals_fp32_accumulation_then_cast():
    """BF16 direct output == FP32 accumulate-from-zero then one cast (tests/utils.py:20-38 of the reference)."""
    qa, qb, (ga, gmb, gb), _, _ = H.make_dense(256, 512, 2048, seed=11)
    rec = dict(recipe_a=(1, ga), recipe_b=(gmb, gb))
    direct = torch.empty((256, 512), dtype=torch.bfloat16, device="cuda")
    dg.fp8_gemm_nt(qa, qb, direct, **rec)
    acc = torch.zeros((256, 512), dtype=torch.float32, device="cuda")
    dg.fp8_gemm_nt(qa, qb, acc, c=acc, **rec)
    dg.testing.assert_bitwise_equal(direct, acc.to(torch.bfloat16), "direct vs fp32 accumulation")


def test_known_answer_all_ones():
    """All-ones E4M3 operands with unit scales: every output equals K (tests/test_layout.py:182-230)."""
    m, n, k = 300, 384, 256
    a = torch.ones((m, k), device="cuda").to(torch.float8_e4m3fn)
    b = torch.ones((n, k), device="cuda").to(torch.float8_e4m3fn)
    sfa = torch.ones((m, k // 128), device="cuda")
    sfb = torch.ones((n // 128, k // 128), device="cuda")
    d = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    dg.fp8_gemm_nt((a, sfa), (b, sfb), d)
    assert torch.equal(d, torch.full_like(d, k))


def test_bitwise_determinism_and_poisoned_sf_stride():
    """20 reruns are bitwise identical; packed scales with a padded, NaN-poisoned K pitch give the
    same bits (tests/test_fp8_fp4.py:78-94, tests/utils.py:41-50 of the reference)."""
    m, n, k = 512, 768, 2048
    qa, qb, (ga, gmb, gb), _, _ = H.make_dense(m, n, k, seed=5)
    d0 = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    dg.fp8_gemm_nt(qa, qb, d0)
    for _ in range(20):
        d = torch.empty_like(d0)
        dg.fp8_gemm_nt(qa, qb, d)
        assert torch.equal(d, d0)
    pa = dg.transform_sf_into_required_layout(qa[1], m, k, (1, ga))
    pb = dg.transform_sf_into_required_layout(qb[1], n, k, (gmb, gb))

    def poison(sf):
        mn = sf.size(-2)
        pitch = (mn + 3) // 4 * 4 + 4
        store = sf.new_full((sf.numel() // mn, pitch), -1)
        return store.as_strided(sf.shape, (1, pitch)).copy_(sf)

    d = torch.empty_like(d0)
    dg.fp8_gemm_nt((qa[0], poison(pa)), (qb[0], poison(pb)), d, recipe_a=(1, ga), recipe_b=(1, gb))
    dg.testing.assert_bitwise_equal(d, d0, "poisoned SF pitch")


def test_fp4_equals_same_values_as_fp8():
    """E2M1 weights re-encoded as E4M3 bytes give the same output (tests/test_fp8_fp4.py:95-100)."""
    m, n, k = 256, 512, 1024
    qa, qb, (ga, gmb, gb), _, _ = H.make_dense(m, n, k, b_kind="fp4", scale_b=0.02, seed=9)
    d4 = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    dg.fp8_fp4_gemm_nt(qa, qb, d4, recipe_a=(1, ga), recipe_b=(1, gb))
    codes = OQ.unpack_fp4_codes(H.to_np(qb[0]))
    as_fp8 = torch.from_numpy(OQ.fp4_codes_to_e4m3_bits(codes)).cuda().view(torch.float8_e4m3fn)
    d8 = torch.empty_like(d4)
    dg.fp8_fp4_gemm_nt(qa, (as_fp8, qb[1]), d8, recipe_a=(1, ga), recipe_b=(1, gb))
    assert H.calc_diff(H.to_np(d4), H.to_np(d8)) < 1e-14


def test_empty_and_k_zero():
    a = (torch.empty((0, 256), device="cuda").to(torch.float8_e4m3fn), torch.empty((0, 2), device="cuda"))
    b = (torch.ones((128, 256), device="cuda").to(torch.float8_e4m3fn), torch.ones((1, 2), device="cuda"))
    d = torch.empty((0, 128), dtype=torch.bfloat16, device="cuda")
    dg.fp8_gemm_nt(a, b, d)       # m == 0: nothing to do
    with pytest.raises(RuntimeError):
        dg.fp8_gemm_nt(b, b, torch.empty((128, 64), dtype=torch.bfloat16, device="cuda"))   # shape mismatch


# --------------------------------------------------------------------------- M-grouped
@pytest.mark.parametrize("use_psum", [False, True])
@pytest.mark.parametrize("b_kind,tol", [("fp8_block", FP8_TOL), ("fp4", FP4_TOL)])
@pytest.mark.parametrize("tile", [None, T(1, 128, 2), T(2, 128, 2), T(1, 64, 2), T(2, 256, 2), T(1, 256, 2)])
def test_m_grouped_contiguous(use_psum, b_kind, tol, tile):
    case = H.make_m_grouped_contiguous(5, 300, 512, 1024, use_psum=use_psum, b_kind=b_kind,
                                       scale_b=0.02 if b_kind == "fp4" else 1.0, seed=21)
    ga, gmb, gb = case["grans"]
    d = torch.full((case["m"], 512), float("nan"), dtype=torch.bfloat16, device="cuda")
    with H.force_tile(**(tile or {})):
        dg.m_grouped_fp8_fp4_gemm_nt_contiguous(case["a"], case["b"], d, case["layout"], recipe_a=(1, ga),
                                                recipe_b=(gmb, gb), use_psum_layout=use_psum)
    ref = H.ref_m_grouped(case)
    dn = H.to_np(d)
    v = case["valid"]
    assert H.calc_diff(dn[v], ref[v]) < tol
    if use_psum:
        assert np.array_equal(dn[~v], np.zeros_like(dn[~v]))     # zero input padding -> zero output padding


@pytest.mark.parametrize("tile", [None, T(2, 128, 2)])
def test_m_grouped_psum_without_zero_padding(tile):
    """ensure_zero_padding=False (scheduler/gemm.cuh:178-184 of the reference): only a group's valid rows, rounded up
    to 16, are computed (zero input rows give zero output rows there); rows of d beyond the 32-row store granule keep
    what they held, the rows in between are unspecified."""
    case = H.make_m_grouped_contiguous(5, 300, 512, 1024, use_psum=True, seed=22)
    ga, gmb, gb = case["grans"]
    d = torch.full((case["m"], 512), 7.0, dtype=torch.bfloat16, device="cuda")
    with H.force_tile(**(tile or {})):
        dg.m_grouped_fp8_fp4_gemm_nt_contiguous(case["a"], case["b"], d, case["layout"], recipe_a=(1, ga),
                                                recipe_b=(gmb, gb), use_psum_layout=True, ensure_zero_padding=False,
                                                expected_m_for_psum_layout=300)
    ref, dn, v = H.ref_m_grouped(case), H.to_np(d), case["valid"]
    assert H.calc_diff(dn[v], ref[v]) < FP8_TOL
    start = 0
    for am, al in zip(case["actual"], case["aligned"]):
        computed = min(al, H.align_up(am, 16))
        assert np.array_equal(dn[start + am:start + computed], np.zeros_like(dn[start + am:start + computed]))
        untouched = min(al, H.align_up(am, 32))
        assert (dn[start + untouched:start + al] == 7.0).all()
        start += al


def test_m_grouped_contiguous_nn_alias():
    case = H.make_m_grouped_contiguous(3, 200, 512, 1024, seed=4)
    ga, gmb, gb = case["grans"]
    b_data, b_sf = case["b"]
    b_kn = b_data.transpose(1, 2).contiguous()              # [G, K, N] storage
    sf_kn = b_sf.transpose(1, 2).contiguous()
    d = torch.empty((case["m"], 512), dtype=torch.bfloat16, device="cuda")
    dg.m_grouped_fp8_fp4_gemm_nn_contiguous(case["a"], (b_kn, sf_kn), d, case["layout"], recipe_a=(1, ga),
                                            recipe_b=(gmb, gb))
    ref = H.ref_m_grouped(case)
    v = case["valid"]
    assert H.calc_diff(H.to_np(d)[v], ref[v]) < FP8_TOL


@pytest.mark.parametrize("b_kind,tol", [("fp8_block", FP8_TOL), ("fp4", FP4_TOL)])
@pytest.mark.parametrize("groups,max_m,expected", [(4, 512, 150), (6, 256, 20), (3, 1024, 700)])
@pytest.mark.parametrize("tile", [None, T(2, 256, 2), T(2, 128, 2), T(1, 64, 2)])
def test_m_grouped_masked(b_kind, tol, groups, max_m, expected, tile):
    case = H.make_masked(groups, max_m, expected, 512, 1024, b_kind=b_kind, scale_b=0.02 if b_kind == "fp4" else 1.0,
                         seed=groups)
    ga, gmb, gb = case["grans"]
    d = torch.full((groups, max_m, 512), float("nan"), dtype=torch.bfloat16, device="cuda")
    with H.force_tile(**(tile or {})):
        dg.m_grouped_fp8_fp4_gemm_nt_masked(case["a"], case["b"], d, case["masked"], expected, recipe_a=(1, ga),
                                            recipe_b=(gmb, gb))
    ref = OG.m_grouped_masked(case["ref_a"], case["ref_b"], case["masked_cpu"])
    dn = H.to_np(d)
    for g in range(groups):
        mm = int(case["masked_cpu"][g])
        if mm:
            assert H.calc_diff(dn[g, :mm], ref[g, :mm]) < tol, g


# --------------------------------------------------------------------------- K-grouped
@pytest.mark.parametrize("gran_k", [128, 32])
@pytest.mark.parametrize("accumulate,out_dtype", [(True, torch.float32), (False, torch.float32), (False, torch.bfloat16)])
def test_k_grouped_tn(gran_k, accumulate, out_dtype):
    old = dg.get_mk_alignment_for_contiguous_layout()
    try:
        dg.set_mk_alignment_for_contiguous_layout(128)
        ks = [512, 256, 1024, 128]
        m, n = 256, 512
        case = H.make_k_grouped(len(ks), m, n, ks, gran_k=gran_k, seed=gran_k)
        d = torch.randn((len(ks), m, n), dtype=out_dtype, device="cuda") * 32 if accumulate else \
            torch.full((len(ks), m, n), float("nan"), dtype=out_dtype, device="cuda")
        c = d if accumulate else None
        cref = H.to_np(d).astype(np.float32) if accumulate else None
        layout = torch.tensor(ks, dtype=torch.int32, device="cuda")
        dg.k_grouped_fp8_gemm_tn_contiguous(case["a"], case["b"], d, ks, layout, c=c, recipe=(1, 1, gran_k))
        ref = OG.k_grouped_tn(case["ref_a"], case["ref_b"], case["bounds"], c=cref,
                              cd_dtype="f32" if out_dtype == torch.float32 else "bf16")
        assert H.calc_diff(H.to_np(d), ref) < FP8_TOL
    finally:
        dg.set_mk_alignment_for_contiguous_layout(old)


@pytest.mark.parametrize("accumulate,out_dtype", [(True, torch.float32), (False, torch.float32), (False, torch.bfloat16)])
@pytest.mark.parametrize("ks", [[0, 256, 0, 512, 128, 0], [0, 0, 384, 0]])
def test_k_grouped_tn_empty_groups(ks, accumulate, out_dtype):
    """Groups without K rows give D = 0 (or leave C alone), first, last and in between: the variants of
    tests/generators.py:265-273."""
    old = dg.get_mk_alignment_for_contiguous_layout()
    try:
        dg.set_mk_alignment_for_contiguous_layout(128)
        m, n = 256, 512
        case = H.make_k_grouped(len(ks), m, n, ks, gran_k=128, seed=len(ks))
        d = torch.randn((len(ks), m, n), dtype=out_dtype, device="cuda") * 32 if accumulate else \
            torch.full((len(ks), m, n), float("nan"), dtype=out_dtype, device="cuda")
        c = d if accumulate else None
        cref = H.to_np(d).astype(np.float32) if accumulate else None
        layout = torch.tensor(ks, dtype=torch.int32, device="cuda")
        dg.k_grouped_fp8_gemm_tn_contiguous(case["a"], case["b"], d, ks, layout, c=c, recipe=(1, 1, 128))
        torch.cuda.synchronize()
        dg.check_status()
        ref = OG.k_grouped_tn(case["ref_a"], case["ref_b"], case["bounds"], c=cref,
                              cd_dtype="f32" if out_dtype == torch.float32 else "bf16")
        got = H.to_np(d)
        assert not np.isnan(got).any()
        for g, kk in enumerate(ks):
            if kk == 0:
                assert np.array_equal(got[g], ref[g]), f"empty group {g}"
        assert H.calc_diff(got, ref) < FP8_TOL
    finally:
        dg.set_mk_alignment_for_contiguous_layout(old)


@pytest.mark.parametrize("gran_k", [128, 32])
@pytest.mark.parametrize("accumulate,out_dtype", [(True, torch.float32), (False, torch.bfloat16)])
@pytest.mark.parametrize("synced", [True, False])
def test_k_grouped_tn_psum(gran_k, accumulate, out_dtype, synced):
    """K-grouped GEMM over the PSUM layout (tests/generators.py:540-608 of the reference): un-aligned K ends, a group's
    last K block stops inside the zero padding before the next group; empty groups first, last and in between; with the
    aligned sizes known on the host and without."""
    old = dg.get_mk_alignment_for_contiguous_layout()
    try:
        dg.set_mk_alignment_for_contiguous_layout(128)
        real_ks = [0, 200, 0, 1000, 128, 513, 0]
        m, n = 256, 512
        case = H.make_k_grouped_psum(m, n, real_ks, 128, gran_k=gran_k, seed=gran_k + 1)
        g = len(real_ks)
        d = torch.randn((g, m, n), dtype=out_dtype, device="cuda") * 32 if accumulate else \
            torch.full((g, m, n), float("nan"), dtype=out_dtype, device="cuda")
        c = d if accumulate else None
        cref = H.to_np(d).astype(np.float32) if accumulate else None
        layout = torch.tensor(case["ends"], dtype=torch.int32, device="cuda")
        dg.k_grouped_fp8_gemm_tn_contiguous(case["a"], case["b"], d, case["aligned"] if synced else None, layout, c=c,
                                            recipe=(1, 1, gran_k), use_psum_layout=True)
        torch.cuda.synchronize()
        dg.check_status()
        ref = OG.k_grouped_tn(case["ref_a"], case["ref_b"], case["bounds"], c=cref,
                              cd_dtype="f32" if out_dtype == torch.float32 else "bf16")
        got = H.to_np(d)
        assert not np.isnan(got).any()
        for i, kk in enumerate(real_ks):
            if kk == 0:
                assert np.array_equal(got[i], ref[i]), f"empty group {i}"
        assert H.calc_diff(got, ref) < FP8_TOL
    finally:
        dg.set_mk_alignment_for_contiguous_layout(old)


# --------------------------------------------------------------------------- full-size properties
def test_full_size_dense_known_answer_and_torch_reference():
    """4096 x 4096 x 7168 (the dense headline shape): all-ones known answer, then seeded inputs against a
    float32 torch matmul of the dequantised operands on the same device."""
    m, n, k = 4096, 4096, 7168
    a = torch.ones((m, k), device="cuda").to(torch.float8_e4m3fn)
    b = torch.ones((n, k), device="cuda").to(torch.float8_e4m3fn)
    d = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    dg.fp8_gemm_nt((a, torch.ones((m, k // 128), device="cuda")), (b, torch.ones((n // 128, k // 128), device="cuda")), d)
    assert torch.equal(d, torch.full_like(d, k))
    torch.manual_seed(0)
    x = torch.randn((m, k), device="cuda", dtype=torch.bfloat16)
    w = torch.randn((n, k), device="cuda", dtype=torch.bfloat16)
    qa = dg.utils.per_token_cast_to_fp8(x, True, 128)
    qb = dg.utils.per_block_cast_to_fp8(w, True, 128)
    dg.fp8_gemm_nt(qa, qb, d)
    ref_a = dg.utils.cast_back_from_fp8(qa[0], qa[1], 128)
    ref_b = qb[0].float() * qb[1].repeat_interleave(128, 0)[:n].repeat_interleave(128, 1)[:, :k]
    ref = ref_a @ ref_b.t()
    assert dg.testing.calc_diff(d, ref) < FP8_TOL
    assert dg.testing.calc_diff(d, x.float() @ w.float().t()) < 1e-3     # the reference tests' own criterion
