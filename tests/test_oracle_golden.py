"""The numpy oracle against vectors produced by the reference's own CPU code.

The vectors in tests/golden/quant_golden.npz were written by
tests/golden/make_golden.py from the reference's deep_gemm/utils/math.py and
deep_gemm/testing/numeric.py.  Everything here is bit-exact except calc_diff.
"""
import numpy as np

from oracle import layout as L
from oracle import quant as Q


def eq(a, b):
    a, b = np.asarray(a), np.asarray(b)
    assert a.shape == b.shape, (a.shape, b.shape)
    if a.dtype.kind == "f":
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    else:
        assert np.array_equal(a, b)


def test_per_token_fp8(golden):
    for tag, g in (("pt128", 128), ("pt32", 32), ("pt128_ragged", 128)):
        for ue in (0, 1):
            x = golden[f"{tag}_ue{ue}_x"]
            q, sf = Q.per_token_cast_to_fp8(x, bool(ue), g)
            eq(q, golden[f"{tag}_ue{ue}_q"])
            eq(sf, golden[f"{tag}_ue{ue}_sf"])
        q, psf = Q.per_token_cast_to_fp8(x, True, g, use_packed_ue8m0=True)
        eq(psf, golden[f"{tag}_packed_sf"])
        eq(Q.cast_back_from_fp8(q, psf, g, use_packed_ue8m0=True), golden[f"{tag}_back"])


def test_per_block_and_channel_fp8(golden):
    for ue in (0, 1):
        q, sf = Q.per_block_cast_to_fp8(golden["pb_x"], bool(ue), 128)
        eq(q, golden[f"pb_ue{ue}_q"])
        eq(sf, golden[f"pb_ue{ue}_sf"])
    for g in (32, 128):
        q, sf = Q.per_channel_cast_to_fp8(golden["pc_x"], True, g)
        eq(q, golden[f"pc{g}_q"])
        eq(sf, golden[f"pc{g}_sf"])


def test_fp4(golden):
    x = golden["fp4_x"]
    for ue in (0, 1):
        p, sf = Q.per_token_cast_to_fp4(x, bool(ue), 32)
        eq(p, golden[f"fp4_ue{ue}_p"])
        eq(sf, golden[f"fp4_ue{ue}_sf"])
    p, psf = Q.per_token_cast_to_fp4(x, True, 32, use_packed_ue8m0=True)
    eq(psf, golden["fp4_packed_sf"])
    eq(Q.cast_back_from_fp4(p, psf, 32, use_packed_ue8m0=True), golden["fp4_back"])
    eq(Q.transpose_packed_fp4(golden["fp4_t_in"]), golden["fp4_t_out"])


def test_fp4_reencoded_as_fp8_is_exact():
    codes = np.arange(16, dtype=np.uint8)
    eq(Q.e4m3_bits_to_f32(Q.fp4_codes_to_e4m3_bits(codes)), Q.fp4_codes_to_f32(codes))
    # e2m1 value table of the reference (deep_gemm/utils/math.py:145)
    eq(Q.fp4_codes_to_f32(np.arange(8, dtype=np.uint8)),
       np.array([0, .5, 1, 1.5, 2, 3, 4, 6], dtype=np.float32))


def test_ceil_to_ue8m0(golden):
    eq(Q.ceil_to_ue8m0(golden["ceil_in"]), golden["ceil_out"])


def test_e4m3_codec_roundtrip():
    codes = np.arange(256, dtype=np.uint8)
    vals = Q.e4m3_bits_to_f32(codes)
    ok = ~np.isnan(vals)
    back = Q.f32_to_e4m3_bits(vals[ok])
    # -0 and +0 keep their sign bit
    assert np.array_equal(back, codes[ok])
    # ties round to even mantissa
    assert Q.f32_to_e4m3_bits(np.array([17.0], np.float32))[0] == Q.f32_to_e4m3_bits(np.array([16.0], np.float32))[0]
    assert Q.f32_to_e4m3_bits(np.array([19.0], np.float32))[0] == Q.f32_to_e4m3_bits(np.array([20.0], np.float32))[0]


def test_packed_layout(golden):
    for tag in ("lay2d", "lay2d_al", "lay3d"):
        out = L.packed_ue8m0_mn_major(golden[f"{tag}_sf"])
        eq(np.ascontiguousarray(out), golden[f"{tag}_out"])
        assert L.element_strides(out) == tuple(int(s) for s in golden[f"{tag}_strides"])


def test_calc_diff(golden):
    assert abs(Q.calc_diff(golden["diff_a"], golden["diff_b"]) - float(golden["diff_val"])) < 1e-12
    assert Q.calc_diff(np.zeros(4), np.zeros(4)) == 0.0


def test_k_grouped_packing_matches_per_group_layout():
    rng = np.random.default_rng(0)
    ks, gran = [256, 128, 0, 640], 128
    mn = 12
    rows = sum(k // gran for k in ks)
    sf = (rng.integers(1, 254, (rows, mn)).astype(np.int32) << 23).view(np.float32)
    packed = L.k_grouped_packed_ue8m0(sf, ks, gran)
    off = poff = 0
    for k in ks:
        n = k // gran
        if not n:
            continue
        ref = np.ascontiguousarray(L.packed_ue8m0_mn_major(np.ascontiguousarray(sf[off:off + n].T))).T
        pk = (n + 3) // 4
        eq(packed[poff:poff + pk], ref)
        off += n
        poff += pk


def test_mega_moe_weight_transforms():
    g, n, k = 2, 256, 3
    t = np.arange(g * n * k, dtype=np.int32).reshape(g, n, k)
    il = L.interleave_gate_up(t)
    # block b of 16 rows = gate rows 8b..8b+7 then up rows 8b..8b+7
    assert np.array_equal(il[:, 0:8], t[:, 0:8]) and np.array_equal(il[:, 8:16], t[:, 128:136])
    assert np.array_equal(il[:, 16:24], t[:, 8:16])
    tr = L.transpose_sf_for_utccp(t)
    i = np.arange(n)
    assert np.array_equal(tr[:, L.utccp_row_index(i)], t[:, i])


def test_mega_moe_oracle_matches_reference_baseline():
    """oracle/mega_moe.py against the output of the reference's own torch baseline
    (tests/test_mega_moe.py:466-480, run by tests/golden/make_mega_moe_golden.py): masked slots, an expert
    without tokens, 3 slots per token.  Bit for bit."""
    import os
    from oracle import mega_moe as OM
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "mega_moe_golden.npz"))
    y, counts = OM.mega_moe_reference(g["x_deq"], g["topk_idx"], g["topk_weights"], g["l1_deq"], g["l2_deq"])
    assert np.array_equal(y, g["y"])
    assert counts[5] == 0 and counts.sum() == (g["topk_idx"] >= 0).sum()
    # the other gated activations of the reference's test (tests/test_mega_moe.py:551-566)
    for tag, kw in (("y_geglu", dict(activation="geglu")),
                    ("y_situ_4_25", dict(activation="situ", situ_beta=4.0, situ_linear_beta=25.0)),
                    ("y_situ_4_none", dict(activation="situ", situ_beta=4.0)),
                    ("y_situ_2_3", dict(activation="situ", situ_beta=2.0, situ_linear_beta=3.0))):
        y, _ = OM.mega_moe_reference(g["x_deq"], g["topk_idx"], g["topk_weights"], g["l1_deq"], g["l2_deq"], **kw)
        assert np.array_equal(y, g[tag]), tag


def test_layout_oracle_matches_reference_text():
    """oracle/layout.py against outputs of the reference's own Python for the packed MN-major scale layout
    (tests/test_layout.py:24-46) and for the Mega MoE weight permutations (deep_gemm/mega/__init__.py:167-198), both
    run from the reference's text by tests/golden/make_layout_golden.py.  Values and strides, bit for bit."""
    import os
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "layout_golden.npz"))
    for tag in ("p2", "p2b", "p3", "p1row"):
        got = L.packed_ue8m0_mn_major(g[f"{tag}_sf"])
        assert np.array_equal(np.ascontiguousarray(got), g[f"{tag}_packed"]), tag
        mn = g[f"{tag}_sf"].shape[-2]
        if mn > 1:      # a one-row tensor's strides carry no information
            assert L.element_strides(got) == tuple(g[f"{tag}_strides"]), tag
    assert np.array_equal(L.interleave_gate_up(g["w"]), g["w_interleaved"])
    assert np.array_equal(L.interleave_gate_up(g["w2d"][None])[0], g["w2d_interleaved"])
    il = L.interleave_gate_up(g["wsf"])
    assert np.array_equal(il, g["wsf_interleaved"])
    assert np.array_equal(L.transpose_sf_for_utccp(il), g["wsf_utccp"])
    # the reference keeps the packed scales' MN-major strides through both permutations
    assert tuple(g["wsf_utccp_strides"]) == tuple(g["wsf_in_strides"])


def test_shipped_weight_transform_matches_reference_text():
    """transform_weights_for_mega_moe of the package (torch, CPU tensors) against the same reference outputs,
    strides included."""
    import os
    import torch
    import deepgemm_b200 as dg
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "layout_golden.npz"))
    w = torch.from_numpy(g["w"])
    sf = torch.from_numpy(np.ascontiguousarray(g["wsf"].transpose(0, 2, 1))).transpose(1, 2)   # MN-major [G, 2I, pk]
    assert tuple(sf.stride()) == tuple(g["wsf_in_strides"])
    w2 = torch.zeros((2, 128, 8), dtype=torch.int8)
    sf2 = torch.zeros((2, 1, 128), dtype=torch.int32).transpose(1, 2)
    (t1, tsf1), _ = dg.transform_weights_for_mega_moe((w, sf), (w2, sf2))
    assert np.array_equal(t1.numpy(), g["w_interleaved"])
    assert np.array_equal(tsf1.numpy(), g["wsf_utccp"])
    assert tuple(tsf1.stride()) == tuple(g["wsf_utccp_strides"])
