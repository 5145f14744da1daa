"""CPU checks of the shipped package: torch quantisation helpers against the reference-generated
golden vectors, the C ABI's exported symbols, and host-side argument validation."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

import deepgemm_b200 as dg
from deepgemm_b200 import _lib
from deepgemm_b200.utils import math as M

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def bits(t):
    return t.contiguous().view(torch.uint8).numpy()


def test_torch_quant_helpers_match_reference_vectors(golden):
    for tag, g in (("pt128", 128), ("pt32", 32), ("pt128_ragged", 128)):
        for ue in (0, 1):
            x = torch.from_numpy(golden[f"{tag}_ue{ue}_x"]).to(torch.bfloat16)
            q, sf = M.per_token_cast_to_fp8(x, bool(ue), g)
            assert np.array_equal(bits(q), golden[f"{tag}_ue{ue}_q"])
            assert np.array_equal(sf.numpy().view(np.uint32), golden[f"{tag}_ue{ue}_sf"].view(np.uint32))
        q, psf = M.per_token_cast_to_fp8(x, True, g, use_packed_ue8m0=True)
        assert np.array_equal(psf.numpy(), golden[f"{tag}_packed_sf"])
        back = M.cast_back_from_fp8(q, psf, g, use_packed_ue8m0=True)
        assert np.array_equal(back.numpy().view(np.uint32), golden[f"{tag}_back"].view(np.uint32))
    x = torch.from_numpy(golden["pb_x"]).to(torch.bfloat16)
    for ue in (0, 1):
        q, sf = M.per_block_cast_to_fp8(x, bool(ue), 128)
        assert np.array_equal(bits(q), golden[f"pb_ue{ue}_q"])
        assert np.array_equal(sf.numpy(), golden[f"pb_ue{ue}_sf"])
    x = torch.from_numpy(golden["pc_x"]).to(torch.bfloat16)
    for g in (32, 128):
        q, sf = M.per_channel_cast_to_fp8(x, True, g)
        assert np.array_equal(bits(q), golden[f"pc{g}_q"]) and np.array_equal(sf.numpy(), golden[f"pc{g}_sf"])
    x = torch.from_numpy(golden["fp4_x"]).to(torch.bfloat16)
    for ue in (0, 1):
        p, sf = M.per_token_cast_to_fp4(x, bool(ue), 32)
        assert np.array_equal(bits(p), golden[f"fp4_ue{ue}_p"]) and np.array_equal(sf.numpy(), golden[f"fp4_ue{ue}_sf"])
    p, psf = M.per_token_cast_to_fp4(x, True, 32, use_packed_ue8m0=True)
    assert np.array_equal(psf.numpy(), golden["fp4_packed_sf"])
    assert np.array_equal(M.cast_back_from_fp4(p, psf, 32, use_packed_ue8m0=True).numpy(), golden["fp4_back"])
    t_in = torch.from_numpy(golden["fp4_t_in"]).view(torch.int8)
    assert np.array_equal(bits(M.transpose_packed_fp4(t_in)), golden["fp4_t_out"])
    assert np.array_equal(M.ceil_to_ue8m0(torch.from_numpy(golden["ceil_in"])).numpy().view(np.uint32),
                          golden["ceil_out"].view(np.uint32))
    assert abs(dg.testing.calc_diff(torch.from_numpy(golden["diff_a"]), torch.from_numpy(golden["diff_b"]))
               - float(golden["diff_val"])) < 1e-12


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "deepgemm_b200.h")).read()
    declared = set(re.findall(r"\b(dg_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    lib = _lib.lib()
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert declared == set(_lib.EXPORTS)
    assert b"sm_100a" in lib.dg_version()


def test_knobs_roundtrip():
    old = dg.get_mk_alignment_for_contiguous_layout()
    try:
        dg.set_mk_alignment_for_contiguous_layout(256)
        assert dg.get_mk_alignment_for_contiguous_layout() == 256
        with pytest.raises(RuntimeError):
            dg.set_mk_alignment_for_contiguous_layout(7)
    finally:
        dg.set_mk_alignment_for_contiguous_layout(old)
    assert dg.get_tc_util() == 100
    dg.set_tc_util(80)
    assert dg.get_tc_util() == 80
    dg.set_tc_util(100)
    # 256 on sm_100 whatever the expected group size (csrc/jit_kernels/heuristics/runtime.hpp:57-64 of the reference)
    assert dg.get_theoretical_mk_alignment_for_contiguous_layout() == 256
    assert dg.get_theoretical_mk_alignment_for_contiguous_layout(64) == 256
    assert dg.utils.get_m_alignment_for_contiguous_layout() == old


def test_gemm_argument_checks_raise_runtime_error():
    lib = _lib.lib()
    args = _lib.GemmArgs()
    args.gemm_type, args.m, args.n, args.k = 0, 128, 128, 128
    assert lib.dg_gemm_bs(ctypes.byref(args)) != 0          # null tensors
    assert b"Assertion failed" in lib.dg_last_error()
    args.gemm_type = 99
    assert lib.dg_gemm_bs(ctypes.byref(args)) != 0
    args.gemm_type, args.m = 0, 0
    assert lib.dg_gemm_bs(ctypes.byref(args)) == 0          # empty problem: nothing to do


def test_bf16_family_surface_and_checks():
    """The BF16 operators exist under the reference's names (csrc/apis/gemm.hpp:938-985) and refuse wrong dtypes, shapes
    and mixed operand kinds before anything is launched."""
    for name in ("bf16_gemm_nt", "bf16_gemm_nn", "bf16_gemm_tn", "bf16_gemm_tt", "m_grouped_bf16_gemm_nt_contiguous",
                 "m_grouped_bf16_gemm_nn_contiguous", "m_grouped_bf16_gemm_nt_masked", "k_grouped_bf16_gemm_tn_contiguous"):
        assert callable(getattr(dg, name))
    a, b = torch.zeros((128, 64), dtype=torch.bfloat16), torch.zeros((128, 64), dtype=torch.bfloat16)
    d = torch.zeros((128, 128), dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="kBFloat16"):
        dg.bf16_gemm_nt(a.float(), b, d)
    with pytest.raises(RuntimeError, match="m == m_ and n == n_ and k == k_"):
        dg.bf16_gemm_nt(a, b[:, :32], d)
    with pytest.raises(RuntimeError, match="major_a == cute::UMMA::Major::K"):
        dg.m_grouped_bf16_gemm_nt_contiguous(a.t().contiguous().t(), b.unsqueeze(0), d, torch.zeros(128, dtype=torch.int32))
    lib = _lib.lib()
    args = _lib.GemmArgs()
    args.gemm_type, args.m, args.n, args.k = 0, 128, 128, 128
    args.a.data = args.b.data = args.d = 16                  # never dereferenced: the checks come first
    args.a.dtype, args.b.dtype = _lib.DG_BF16, _lib.DG_E4M3
    assert lib.dg_gemm_bs(ctypes.byref(args)) != 0 and b"both BF16" in lib.dg_last_error()


def test_sf_layout_validation_messages():
    sf = torch.zeros((64, 3), dtype=torch.int32)
    with pytest.raises(RuntimeError, match=r"sf\.size\(-1\)"):
        dg.transform_sf_into_required_layout(sf, 64, 128 * 4 * 2, (1, 128))
    good = torch.zeros((2, 64), dtype=torch.int32).t()     # MN-major [64, 2]
    out = dg.transform_sf_into_required_layout(good, 64, 1024, (1, 128))
    assert out.data_ptr() == good.data_ptr()
    bad = torch.zeros((64, 2), dtype=torch.int32)           # K-major packed scales are rejected
    with pytest.raises(RuntimeError, match=r"stride\(-2\) == 1"):
        dg.transform_sf_into_required_layout(bad, 64, 1024, (1, 128))
    with pytest.raises(RuntimeError, match="is_sfa"):
        dg.transform_sf_into_required_layout(good, 64, 1024, (1, 1, 128))


def test_mega_moe_weight_transform_matches_oracle_permutations():
    from oracle import layout as OL
    g, n, h = 2, 256, 512
    w = torch.randint(-128, 127, (g, n, h // 2), dtype=torch.int8)
    sf_store = torch.randint(0, 2 ** 31 - 1, (g, h // 128, n), dtype=torch.int32)
    sf = sf_store.transpose(1, 2)                              # [g, n, pk] with MN-major strides
    w2 = torch.randint(-128, 127, (g, h, n // 4), dtype=torch.int8)
    sf2 = torch.randint(0, 2 ** 31 - 1, (g, (n // 2) // 128, h), dtype=torch.int32).transpose(1, 2)
    (t1, tsf1), (t2, tsf2) = dg.transform_weights_for_mega_moe((w, sf), (w2, sf2))
    assert np.array_equal(t1.numpy(), OL.interleave_gate_up(w.numpy()))
    assert np.array_equal(tsf1.numpy(), OL.transpose_sf_for_utccp(OL.interleave_gate_up(sf.numpy())))
    assert np.array_equal(tsf2.numpy(), OL.transpose_sf_for_utccp(sf2.numpy()))
    assert t2.data_ptr() == w2.data_ptr()
    assert tsf1.stride() == sf.stride() and tsf2.stride() == sf2.stride()      # still MN-major


def test_mega_moe_buffer_layout_and_checks():
    cfg = _lib.MoeConfig(8, 256, 4096, 8, 7168, 2048)
    lay = _lib.MoeLayout()
    assert _lib.lib().dg_mega_moe_buffer_layout(ctypes.byref(cfg), ctypes.byref(lay)) == 0
    offs = [lay.off_x, lay.off_x_sf, lay.off_topk_idx, lay.off_topk_weights, lay.off_l1_acts, lay.off_l1_acts_sf,
            lay.off_l2_acts, lay.off_l2_acts_sf, lay.off_combine]
    assert all(o % 1024 == 0 for o in offs) and len(set(offs)) == len(offs) and lay.num_bytes > max(offs)
    assert lay.pool_rows >= 4096 * 8 * 8 and lay.pool_rows % 256 == 0
    bad = _lib.MoeConfig(3, 256, 4096, 8, 7168, 2048)
    assert _lib.lib().dg_mega_moe_buffer_layout(ctypes.byref(bad), ctypes.byref(lay)) != 0
    assert b"num_experts" in _lib.lib().dg_last_error()
    assert dg.get_token_alignment_for_mega_moe() == 128


def test_mega_moe_scale_rows_cover_every_tile():
    """The single-kernel forward gives every token tile 256 scale rows: whatever the split of the pool over the local
    experts, the tiles' scale rows fit `sf_rows`."""
    lay = _lib.MoeLayout()
    bm = dg.get_block_m_for_mega_moe(8, 256, 4096, 4096, 8)
    assert bm % 16 == 0 and 16 <= bm <= 256
    for ranks, experts, tokens, topk in ((8, 256, 4096, 8), (1, 48, 8192, 6), (2, 8, 128, 4), (8, 64, 128, 8)):
        cfg = _lib.MoeConfig(ranks, experts, tokens, topk, 1024, 512, 0, 0)
        assert _lib.lib().dg_mega_moe_buffer_layout(ctypes.byref(cfg), ctypes.byref(lay)) == 0
        local, rows = experts // ranks, min(ranks * tokens * topk, lay.pool_rows)
        assert lay.sf_rows >= lay.pool_rows and lay.sf_rows % 256 == 0
        for split in ([rows // local] * local, [1] * (local - 1) + [rows - (local - 1)],
                      [bm + 1] * min(local, rows // (bm + 1)) + [0] * (local - min(local, rows // (bm + 1)))):
            tiles = sum(-(-r // bm) for r in split)
            assert tiles * 256 <= lay.sf_rows, (ranks, experts, split[:3])


def test_mega_moe_sm_headroom_policy(monkeypatch):
    """The table of the reference's tests/test_mega_moe_headroom.py: the grid is num_sms minus the headroom rounded up to
    even; negative, all-consuming and odd results are refused."""
    lib = _lib.lib()
    try:
        for sms, env, want in ((148, None, 148), (148, "0", 148), (148, "2", 146), (148, "3", 144), (148, "8", 140),
                               (132, "1", 130), (148, "-1", -1), (148, "148", -1), (148, "147", -1), (147, "0", -1)):
            dg.set_num_sms(sms)
            if env is None:
                monkeypatch.delenv("DG_MEGA_MOE_SM_HEADROOM", raising=False)
            else:
                monkeypatch.setenv("DG_MEGA_MOE_SM_HEADROOM", env)
            assert lib.dg_get_mega_moe_num_sms() == want, (sms, env)
    finally:
        dg.set_num_sms(0)


def test_mega_moe_pool_capacity_and_control_block():
    """num_ring_tokens bounds the pool (and with it the buffer); the first view starts after the fixed 16 KiB control
    block whatever the configuration, which is what makes reusing a buffer for another configuration legal."""
    lay = _lib.MoeLayout()
    sizes = {}
    for cap in (0, 40000):
        cfg = _lib.MoeConfig(8, 256, 4096, 8, 7168, 2048, cap, 0)
        assert _lib.lib().dg_mega_moe_buffer_layout(ctypes.byref(cfg), ctypes.byref(lay)) == 0
        sizes[cap] = (lay.num_bytes, lay.pool_rows)
    assert sizes[0][1] >= 4096 * 8 * 8 and 40000 <= sizes[40000][1] < 40000 + 32 * 128 + 256
    assert sizes[40000][0] < sizes[0][0] / 2
    firsts = set()
    for experts, tokens, hidden in ((256, 4096, 7168), (8, 128, 1024), (64, 512, 2048)):
        cfg = _lib.MoeConfig(8, experts, tokens, 4, hidden, 512, 0, 0)
        assert _lib.lib().dg_mega_moe_buffer_layout(ctypes.byref(cfg), ctypes.byref(lay)) == 0
        firsts.add(min(lay.off_x, lay.off_x_sf, lay.off_topk_idx, lay.off_l1_acts, lay.off_combine) >= 16384)
    assert firsts == {True}
    too_many = _lib.MoeConfig(1, 8192, 128, 4, 1024, 512, 0, 0)
    assert _lib.lib().dg_mega_moe_buffer_layout(ctypes.byref(too_many), ctypes.byref(lay)) != 0


def test_header_is_plain_c_and_library_answers_without_gpu(tmp_path):
    """include/deepgemm_b200.h compiles as C; a C program dlopens the library, finds every exported symbol and gets
    answers from the entry points that touch no device (tests/c_abi/abi_check.c)."""
    import shutil
    import subprocess
    from deepgemm_b200 import _lib
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no gcc")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    exe = str(tmp_path / "abi_check")
    subprocess.run([gcc, "-std=c11", "-Wall", "-Werror", "-I", os.path.join(root, "include"),
                    os.path.join(root, "tests", "c_abi", "abi_check.c"), "-o", exe, "-ldl"], check=True)
    res = subprocess.run([exe, _lib.LIB_PATH, *_lib.EXPORTS], capture_output=True, text=True)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "align=128" in res.stdout and "bad_rc=" in res.stdout
