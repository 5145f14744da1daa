"""ctypes binding of the C ABI in include/deepgemm_b200.h.

There is no fallback: if the shared library is missing or a call fails, a RuntimeError is
raised (the reference raises RuntimeError from its DG_HOST_ASSERT, csrc/utils/exception.hpp:13-37).
"""
from __future__ import annotations

import ctypes as C
import os

from .build import LIB_PATH

DG_E4M3, DG_E2M1_PACKED, DG_BF16, DG_F32 = 0, 1, 2, 3
GEMM_NORMAL, GEMM_M_CONTIGUOUS, GEMM_M_MASKED, GEMM_M_PSUM, GEMM_K_GROUPED, GEMM_K_GROUPED_PSUM, GEMM_BATCHED = range(7)
EPILOGUE_STORE, EPILOGUE_STOCHASTIC_BF16, EPILOGUE_FP8_CAST = range(3)

EXPORTS = (
    "dg_gemm_bs", "dg_sf_pack_ue8m0", "dg_sf_pack_ue8m0_k_grouped", "dg_set_num_sms", "dg_get_num_sms",
    "dg_set_tc_util", "dg_get_tc_util", "dg_set_mk_alignment_for_contiguous_layout",
    "dg_get_mk_alignment_for_contiguous_layout", "dg_get_theoretical_mk_alignment_for_contiguous_layout",
    "dg_set_wait_timeout_ms", "dg_check_status", "dg_last_error", "dg_version",
    "dg_mega_moe_buffer_layout", "dg_get_token_alignment_for_mega_moe", "dg_mega_moe_forward", "dg_set_mega_moe_fused", "dg_gemm_fp8_fp32sf_noalloc", "dg_noalloc_scratch_bytes",
    "dg_per_token_cast_to_fp8", "dg_debug_set_tile_override", "dg_get_mega_moe_num_sms", "dg_debug_copy", "dg_set_pdl", "dg_get_pdl", "dg_get_block_m_for_mega_moe",
)


class Operand(C.Structure):
    _fields_ = [("data", C.c_void_p), ("sf", C.c_void_p), ("ld", C.c_int64), ("sf_ld", C.c_int64),
                ("dtype", C.c_int32), ("mn_major", C.c_int32), ("gran_k", C.c_int32), ("reserved", C.c_int32),
                ("batch_stride", C.c_int64), ("sf_k_rows", C.c_int64)]


class GemmArgs(C.Structure):
    _fields_ = [("gemm_type", C.c_int32), ("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32),
                ("num_groups", C.c_int32), ("alignment", C.c_int32),
                ("a", Operand), ("b", Operand),
                ("d", C.c_void_p), ("ldd", C.c_int64), ("d_dtype", C.c_int32), ("accumulate", C.c_int32),
                ("alpha", C.c_float), ("expected_m", C.c_int32),
                ("grouped_layout", C.c_void_p), ("stream", C.c_void_p),
                ("d_batch_stride", C.c_int64), ("epilogue", C.c_int32), ("clamp_value", C.c_float),
                ("sfd", C.c_void_p), ("sfd_ld", C.c_int64), ("clamped_count", C.c_void_p),
                ("skip_padding_rows", C.c_int32), ("reserved", C.c_int32)]


class MoeConfig(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("num_ranks", "num_experts", "num_max_tokens_per_rank", "num_topk", "hidden",
                                          "intermediate_hidden", "num_ring_tokens", "num_shared_experts")]


class MoeLayout(C.Structure):
    _fields_ = [(n, C.c_int64) for n in ("num_bytes", "pool_rows", "off_x", "off_x_sf", "off_topk_idx",
                                          "off_topk_weights", "off_l1_acts", "off_l1_acts_sf", "off_l2_acts",
                                          "off_l2_acts_sf", "off_token_src_metadata", "off_combine",
                                          "off_shared_l1_acts_sf", "off_shared_l2_acts", "off_shared_l2_acts_sf", "sf_rows")]


class MoeArgs(C.Structure):
    _fields_ = [("cfg", MoeConfig), ("buffer_ptrs", C.POINTER(C.c_void_p)), ("rank", C.c_int32),
                ("num_tokens", C.c_int32), ("y", C.c_void_p), ("ldy", C.c_int64),
                ("l1_w", C.c_void_p), ("l1_sf", C.c_void_p), ("l2_w", C.c_void_p), ("l2_sf", C.c_void_p),
                ("l1_sf_ld", C.c_int64), ("l2_sf_ld", C.c_int64), ("stats", C.c_void_p),
                ("activation_clamp", C.c_float), ("fast_math", C.c_int32), ("stream", C.c_void_p),
                ("activation", C.c_int32), ("situ_beta", C.c_float), ("situ_linear_beta", C.c_float),
                ("post_down", C.c_int32), ("weights_fp8", C.c_int32),
                ("shared_l1_w", C.c_void_p), ("shared_l1_sf", C.c_void_p), ("shared_l2_w", C.c_void_p),
                ("shared_l2_sf", C.c_void_p), ("shared_l1_sf_ld", C.c_int64), ("shared_l2_sf_ld", C.c_int64)]


class GemmNoAllocArgs(C.Structure):
    _fields_ = [("m", C.c_int32), ("n", C.c_int32), ("k", C.c_int32), ("gran_k", C.c_int32),
                ("gran_mn_b", C.c_int32), ("d_dtype", C.c_int32),
                ("a", C.c_void_p), ("sfa", C.c_void_p), ("b", C.c_void_p), ("sfb", C.c_void_p), ("d", C.c_void_p),
                ("lda", C.c_int64), ("ldb", C.c_int64), ("ldd", C.c_int64), ("stream", C.c_void_p)]


class CastArgs(C.Structure):
    _fields_ = [("x", C.c_void_p), ("ldx", C.c_int64), ("rows", C.c_int32), ("cols", C.c_int32), ("gran_k", C.c_int32),
                ("q", C.c_void_p), ("ldq", C.c_int64), ("sf", C.c_void_p), ("sf_mode", C.c_int32), ("sf_ld", C.c_int64),
                ("stream", C.c_void_p)]


CAST_SF_FLOAT, CAST_SF_PACKED_ROW_MAJOR, CAST_SF_PACKED_MN_MAJOR = 0, 1, 2

_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m deepgemm_b200.build` "
                "(there is no fallback path)")
        l = C.CDLL(LIB_PATH)
        l.dg_last_error.restype = C.c_char_p
        l.dg_version.restype = C.c_char_p
        l.dg_gemm_bs.argtypes = [C.POINTER(GemmArgs)]
        l.dg_sf_pack_ue8m0.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                       C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_int32, C.c_int32,
                                       C.c_void_p]
        l.dg_sf_pack_ue8m0_k_grouped.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32,
                                                 C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                                 C.c_void_p]
        l.dg_check_status.argtypes = [C.POINTER(C.c_uint32)]
        l.dg_mega_moe_buffer_layout.argtypes = [C.POINTER(MoeConfig), C.POINTER(MoeLayout)]
        l.dg_mega_moe_forward.argtypes = [C.POINTER(MoeArgs)]
        l.dg_gemm_fp8_fp32sf_noalloc.argtypes = [C.POINTER(GemmNoAllocArgs)]
        l.dg_per_token_cast_to_fp8.argtypes = [C.POINTER(CastArgs)]
        for name in ("dg_set_num_sms", "dg_set_tc_util", "dg_set_pdl", "dg_set_mk_alignment_for_contiguous_layout",
                     "dg_get_theoretical_mk_alignment_for_contiguous_layout", "dg_set_wait_timeout_ms",
                     "dg_set_mega_moe_fused"):
            getattr(l, name).argtypes = [C.c_int32]
        l.dg_debug_set_tile_override.argtypes = [C.c_int32, C.c_int32, C.c_int32]
        l.dg_debug_copy.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]
        _lib = l
    return _lib


def check(rc: int) -> None:
    if rc != 0:
        raise RuntimeError(lib().dg_last_error().decode())


def check_status():
    """Synchronise and raise if a kernel abandoned a bounded wait (see dg_check_status)."""
    info = (C.c_uint32 * 8)()
    check(lib().dg_check_status(info))
