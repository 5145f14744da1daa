"""GEMM operators behind the `deep_gemm` names.

Same names, positional order, keyword names and defaults as the reference's pybind surface
(csrc/apis/gemm.hpp:839-1001); argument checks follow csrc/apis/gemm.hpp:17-375 and raise
RuntimeError.  All arithmetic happens in the CUDA library through the C ABI (dg_gemm_bs);
tensors are borrowed, D is written in place on the current CUDA stream, nothing synchronises.
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch

from . import _lib
from .layout import (_require, _stream, get_k_grouped_mn_major_tma_aligned_packed_ue8m0_tensor,
                     get_mk_alignment_for_contiguous_layout, transform_sf_pair_into_required_layout)

PACKED_FP4 = torch.int8   # two E2M1 codes per byte (csrc/utils/math.hpp:11)
_K, _MN = 0, 1

class _Epilogue:
    pass


class Identity(_Epilogue):
    """D = acc."""


class Alpha(_Epilogue):
    """D = alpha * acc."""

    def __init__(self, alpha: float):
        self.alpha = float(alpha)


class FP8CastWithClamp(_Epilogue):
    """D as E4M3 with one UE8M0 scale per row and 32 columns, packed four to an int32 in the MN-major TMA-aligned
    layout (the layout accepted for SFA).  The accumulator is rounded to BF16 first, so the bytes equal a BF16 D
    followed by per_token_cast_to_fp8(gran_k=32, use_packed_ue8m0=True).  `clamp_value` clamps the BF16 values before
    scaling; `clamped_count` (a one-element CUDA uint32 tensor) receives how many exceeded it
    (csrc/jit_kernels/impls/epilogue_class.hpp:69-118 of the reference)."""

    def __init__(self, sfd: torch.Tensor, clamp_value: Optional[float] = None, clamped_count: Optional[torch.Tensor] = None):
        _require(clamp_value is None or clamp_value > 0.0, "not clamp_value.has_value() or clamp_value.value() > 0.0f")
        if clamped_count is not None:
            _require(clamped_count.dtype == torch.uint32 and clamped_count.numel() == 1,
                     "clamped_count->scalar_type() == torch::kUInt32 and clamped_count->numel() == 1")
        self.sfd, self.clamp_value, self.clamped_count = sfd, clamp_value, clamped_count

    def check(self, c, d):
        _require(c is None and d.dtype == torch.float8_e4m3fn,
                 "not c.has_value() and d.scalar_type() == torch::kFloat8_e4m3fn and \"FP8 quantization requires a direct E4M3 output\"")


class BF16StochasticRounding(_Epilogue):
    """BF16 D rounded stochastically; the random bits are a hash of the FP32 results themselves, so the output is a
    function of the FP32-accumulated result (csrc/jit_kernels/impls/epilogue_class.hpp:120-136 of the reference)."""

    def check(self, c, d):
        _require(c is None and d.dtype == torch.bfloat16,
                 "not c.has_value() and d.scalar_type() == torch::kBFloat16 and \"Stochastic rounding requires a direct BF16 output\"")


def _major(t: torch.Tensor) -> int:
    """K-major if the last axis is contiguous, else MN-major (csrc/utils/layout.hpp:18-33)."""
    _require(t.dim() in (2, 3), "dim == 2 or dim == 3")
    if t.dim() == 3:
        _require(t.stride(0) == t.size(-2) * t.size(-1), "t.stride(0) == t.size(-2) * t.size(-1)")
    _require(t.stride(-2) == 1 or t.stride(-1) == 1, "t.stride(-2) == 1 or t.stride(-1) == 1")
    return _K if t.stride(-1) == 1 else _MN


def _check_cd(t: torch.Tensor) -> None:
    _require(t.dim() in (2, 3), "dim == 2 or dim == 3")
    if t.dim() == 3:
        _require(t.stride(0) == t.size(-2) * t.size(-1), "t.stride(0) == t.size(-2) * t.size(-1)")
    _require(t.stride(-1) == 1, "t.stride(-1) == 1")


def _logical_mn_k(t: torch.Tensor, major: int) -> Tuple[int, int]:
    _require(t.is_cuda, "t.is_cuda()")
    mn, k = t.shape[-2], t.shape[-1]
    if t.dtype != torch.float8_e4m3fn:
        _require(t.dtype == PACKED_FP4, "ab.scalar_type() == kPackedFP4 and arch_major == 10")
        if major == _K:
            k *= 2
        else:
            mn *= 2
    return mn, k


def _operand(data: torch.Tensor, sf: Optional[torch.Tensor], major: int, gran_k: int, batched: bool = False) -> _lib.Operand:
    op = _lib.Operand()
    op.data = data.data_ptr()
    if sf is None:                      # BF16 operand: no scale factors
        op.ld = (data.stride(-2) if major == _K else data.stride(-1)) * data.element_size()
        op.dtype, op.mn_major = _lib.DG_BF16, int(major == _MN)
        return op
    op.sf = sf.data_ptr()
    op.ld = (data.stride(-2) if major == _K else data.stride(-1)) * data.element_size()
    op.batch_stride = data.stride(0) * data.element_size() if batched else 0
    op.sf_k_rows = getattr(sf, "k_rows", 0)
    op.sf_ld = sf.stride(-1)
    op.dtype = _lib.DG_E2M1_PACKED if data.dtype == PACKED_FP4 else _lib.DG_E4M3
    op.mn_major = int(major == _MN)
    op.gran_k = gran_k
    return op


def _resolve_alpha(alpha: Optional[float], epilogue, c=None, d=None, value_epilogues: bool = False) -> float:
    """The epilogue class, `alpha` and (einsum only) the FP8 output pair are exclusive
    (resolve_epilogue_class, csrc/jit_kernels/impls/epilogue_class.hpp:138-157 of the reference)."""
    _require(not (epilogue is not None and alpha is not None),
             "The epilogue class, `alpha` and the FP8 output pair are exclusive")
    if epilogue is None or isinstance(epilogue, Identity):
        return 1.0 if alpha is None else float(alpha)
    if isinstance(epilogue, Alpha):
        return epilogue.alpha
    if value_epilogues and isinstance(epilogue, (BF16StochasticRounding, FP8CastWithClamp)):
        epilogue.check(c, d)
        return 1.0
    raise RuntimeError(f"epilogue {type(epilogue).__name__} is not supported by this operator")


_D_DTYPES = {torch.float32: _lib.DG_F32, torch.bfloat16: _lib.DG_BF16, torch.float8_e4m3fn: _lib.DG_E4M3}


def _launch(gemm_type, m, n, k, a, sfa, major_a, gran_a, b, sfb, major_b, gran_b, d, *, num_groups=1, alignment=0,
            accumulate=False, alpha=1.0, expected_m=0, grouped_layout=None, epilogue=None, batched=False,
            skip_padding_rows=False) -> None:
    args = _lib.GemmArgs()
    args.gemm_type, args.m, args.n, args.k = gemm_type, m, n, k
    args.num_groups, args.alignment = num_groups, alignment
    args.a = _operand(a, sfa, major_a, gran_a, batched)
    args.b = _operand(b, sfb, major_b, gran_b, batched)
    args.d = d.data_ptr()
    args.ldd = d.stride(-2) * d.element_size()
    args.d_batch_stride = d.stride(0) * d.element_size() if batched else 0
    args.d_dtype = _D_DTYPES[d.dtype]
    args.skip_padding_rows = int(skip_padding_rows)
    args.epilogue = _lib.EPILOGUE_STORE
    if isinstance(epilogue, BF16StochasticRounding):
        args.epilogue = _lib.EPILOGUE_STOCHASTIC_BF16
    elif isinstance(epilogue, FP8CastWithClamp):
        args.epilogue = _lib.EPILOGUE_FP8_CAST
        args.sfd, args.sfd_ld = epilogue.sfd.data_ptr(), epilogue.sfd.stride(-1)
        args.clamp_value = float(epilogue.clamp_value or 0.0)
        args.clamped_count = epilogue.clamped_count.data_ptr() if epilogue.clamped_count is not None else None
    args.accumulate = int(accumulate)
    args.alpha = alpha
    args.expected_m = int(expected_m or 0)
    args.grouped_layout = grouped_layout.data_ptr() if grouped_layout is not None else None
    args.stream = _stream(d)
    _lib.check(_lib.lib().dg_gemm_bs(args))


def _early_return(m: int, n: int, k: int, d: torch.Tensor, c: Optional[torch.Tensor], allow_fp8: bool = False) -> bool:
    """Empty problems and the C != D copy (csrc/apis/gemm.hpp:17-53)."""
    if m == 0 or n == 0:
        return True
    same = c is not None and c.data_ptr() == d.data_ptr()
    if same:
        _require(c.shape == d.shape and c.stride() == d.stride(), "c->sizes() == d.sizes() and c->strides() == d.strides()")
    _require(d.dtype in (torch.bfloat16, torch.float32) or (allow_fp8 and d.dtype == torch.float8_e4m3fn),
             "d.scalar_type() == torch::kBFloat16 or d.scalar_type() == torch::kFloat")
    if c is not None:
        _check_cd(c)
        _require(d.dtype == c.dtype, "d.scalar_type() == c.value().scalar_type()")
    if k == 0:
        if not same:
            d.copy_(c) if c is not None else d.zero_()
        return True
    if c is not None and not same:
        d.copy_(c)
    return False


# --------------------------------------------------------------------------- dense
def fp8_fp4_gemm_nt(a, b, d, c=None, recipe=None, recipe_a=None, recipe_b=None, compiled_dims: str = "nk",
                    disable_ue8m0_cast: bool = False, alpha: Optional[float] = None, epilogue=None) -> None:
    """D = alpha * A @ B^T (+ C); a = (data [m,k], sf), b = (data [n,k], sf) (csrc/apis/gemm.hpp:78-133)."""
    (a_data, a_sf), (b_data, b_sf) = a, b
    major_a, major_b = _major(a_data), _major(b_data)
    if a_data.dtype == PACKED_FP4 and b_data.dtype == PACKED_FP4:
        _require(major_a == _K and major_b == _K, "major_a == cute::UMMA::Major::K and major_b == cute::UMMA::Major::K")
    _check_cd(d)
    m, k = _logical_mn_k(a_data, major_a)
    n, k_ = _logical_mn_k(b_data, major_b)
    _require(d.dim() == 2 and d.is_cuda, "t.dim() == N")
    _require(m == d.size(0) and n == d.size(1) and k == k_, "m == m_ and n == n_ and k == k_")
    _require(d.dtype in (torch.bfloat16, torch.float32), "d.scalar_type() == torch::kBFloat16 or d.scalar_type() == torch::kFloat")
    scale = _resolve_alpha(alpha, epilogue, c, d, value_epilogues=True)
    if _early_return(m, n, k, d, c):
        return
    sfa, sfb, gran_a, gran_b = transform_sf_pair_into_required_layout(
        a_sf, b_sf, m, n, k, recipe, recipe_a, recipe_b, None, None, disable_ue8m0_cast)
    _launch(_lib.GEMM_NORMAL, m, n, k, a_data, sfa, major_a, gran_a, b_data, sfb, major_b, gran_b, d,
            accumulate=c is not None, alpha=scale, epilogue=epilogue)


def _t(pair):
    return pair[0].transpose(0, 1), pair[1].transpose(0, 1)


def fp8_fp4_gemm_nn(a, b, d, c=None, recipe=None, recipe_a=None, recipe_b=None, compiled_dims: str = "nk",
                    disable_ue8m0_cast: bool = False, alpha=None, epilogue=None) -> None:
    """b given as [k, n] (csrc/apis/gemm.hpp:135-148)."""
    fp8_fp4_gemm_nt(a, _t(b), d, c, recipe, recipe_a, recipe_b, compiled_dims, disable_ue8m0_cast, alpha, epilogue)


def fp8_fp4_gemm_tn(a, b, d, c=None, recipe=None, recipe_a=None, recipe_b=None, compiled_dims: str = "mn",
                    disable_ue8m0_cast: bool = False, alpha=None, epilogue=None) -> None:
    """a given as [k, m], b as [k, n] (csrc/apis/gemm.hpp:150-164)."""
    fp8_fp4_gemm_nt(_t(a), _t(b), d, c, recipe, recipe_a, recipe_b, compiled_dims, disable_ue8m0_cast, alpha, epilogue)


def fp8_fp4_gemm_tt(a, b, d, c=None, recipe=None, recipe_a=None, recipe_b=None, compiled_dims: str = "mn",
                    disable_ue8m0_cast: bool = False, alpha=None, epilogue=None) -> None:
    """a given as [k, m] (csrc/apis/gemm.hpp:166-179)."""
    fp8_fp4_gemm_nt(_t(a), b, d, c, recipe, recipe_a, recipe_b, compiled_dims, disable_ue8m0_cast, alpha, epilogue)


# --------------------------------------------------------------------------- M-grouped
def m_grouped_fp8_fp4_gemm_nt_contiguous(a, b, d, grouped_layout, recipe=None, recipe_a=None, recipe_b=None,
                                         compiled_dims: str = "nk", disable_ue8m0_cast: bool = False,
                                         use_psum_layout: bool = False, ensure_zero_padding: bool = True,
                                         expected_m_for_psum_layout: Optional[int] = None,
                                         allow_strided_psum_scales: bool = False, epilogue=None) -> None:
    """Rows of A [m,k] are grouped by expert; B is [G,n,k] (csrc/apis/gemm.hpp:181-252).

    grouped_layout: int32[m] expert id per row (-1 = padding), or with use_psum_layout int32[G]
    cumulative row ends where group g starts at align(end[g-1], mk alignment).
    """
    (a_data, a_sf), (b_data, b_sf) = a, b
    major_a, major_b = _major(a_data), _major(b_data)
    _require(major_a == _K, "major_a == cute::UMMA::Major::K")
    if a_data.dtype == PACKED_FP4 and b_data.dtype == PACKED_FP4:
        _require(major_b == _K, "major_b == cute::UMMA::Major::K")
    _require(grouped_layout.is_contiguous(), "grouped_layout.is_contiguous()")
    _require(a_data.dim() == 2 and b_data.dim() == 3 and d.dim() == 2, "t.dim() == N")
    m, k = _logical_mn_k(a_data, major_a)
    n, k_ = _logical_mn_k(b_data, major_b)
    num_groups = b_data.size(0)
    _require(m == d.size(0) and n == d.size(1) and k == k_, "m == m_ and n == n_ and k == k_")
    _require(n > 0 and k > 0 and num_groups > 0, "n > 0 and k > 0 and num_groups > 0")
    _require(d.dtype == torch.bfloat16, "d.scalar_type() == torch::kBFloat16")
    _require(grouped_layout.dtype == torch.int32, "grouped_layout.scalar_type() == torch::kInt")
    if use_psum_layout:
        _require(grouped_layout.dim() == 1 and grouped_layout.numel() == num_groups, "num_groups == num_groups_")
    else:
        _require(grouped_layout.dim() == 1 and grouped_layout.numel() == m, "m == m__")
        _require(expected_m_for_psum_layout is None, "not expected_m_for_psum_layout.has_value()")
    _require(not allow_strided_psum_scales or use_psum_layout, "not allow_strided_psum_scales or use_psum_layout")
    _check_cd(d)
    _resolve_alpha(None, epilogue)
    if m == 0:
        return
    sfa, sfb, gran_a, gran_b = transform_sf_pair_into_required_layout(
        a_sf, b_sf, m, n, k, recipe, recipe_a, recipe_b, None, num_groups, disable_ue8m0_cast,
        grouped_layout if use_psum_layout else None, allow_strided_psum_scales)
    _launch(_lib.GEMM_M_PSUM if use_psum_layout else _lib.GEMM_M_CONTIGUOUS, m, n, k,
            a_data, sfa, major_a, gran_a, b_data, sfb, major_b, gran_b, d, num_groups=num_groups,
            alignment=get_mk_alignment_for_contiguous_layout(), expected_m=expected_m_for_psum_layout or 0,
            grouped_layout=grouped_layout, skip_padding_rows=use_psum_layout and not ensure_zero_padding)


def m_grouped_fp8_fp4_gemm_nn_contiguous(a, b, d, grouped_layout, recipe=None, recipe_a=None, recipe_b=None,
                                         compiled_dims: str = "nk", disable_ue8m0_cast: bool = False,
                                         use_psum_layout: bool = False, ensure_zero_padding: bool = True,
                                         allow_strided_psum_scales: bool = False, epilogue=None) -> None:
    """b given as [G, k, n] (csrc/apis/gemm.hpp:254-271)."""
    m_grouped_fp8_fp4_gemm_nt_contiguous(a, (b[0].transpose(1, 2), b[1].transpose(1, 2)), d, grouped_layout, recipe,
                                         recipe_a, recipe_b, compiled_dims, disable_ue8m0_cast, use_psum_layout,
                                         ensure_zero_padding, None, allow_strided_psum_scales, epilogue)


def m_grouped_fp8_fp4_gemm_nt_masked(a, b, d, masked_m, expected_m, recipe=None, recipe_a=None, recipe_b=None,
                                     compiled_dims: str = "nk", disable_ue8m0_cast: bool = False, epilogue=None) -> None:
    """a [G,max_m,k], b [G,n,k], d [G,max_m,n]; only the first masked_m[g] rows of group g are computed.

    masked_m is read on the device (csrc/apis/gemm.hpp:273-322).
    """
    (a_data, a_sf), (b_data, b_sf) = a, b
    _require(a_data.dim() == 3 and b_data.dim() == 3 and d.dim() == 3, "t.dim() == N")
    major_a, major_b = _major(a_data), _major(b_data)
    _require(major_a == _K and major_b == _K, "major_a == cute::UMMA::Major::K and major_b == cute::UMMA::Major::K")
    _require(masked_m.is_contiguous(), "masked_m.is_contiguous()")
    m, k = _logical_mn_k(a_data, major_a)
    n, k_ = _logical_mn_k(b_data, major_b)
    g = a_data.size(0)
    _require(g == b_data.size(0) and g == d.size(0) and g == masked_m.numel(),
             "num_groups == num_groups_ and num_groups == num_groups__ and num_groups == num_groups___")
    _require(m == d.size(1) and n == d.size(2) and k == k_, "m == m_ and n == n_ and k == k_")
    _require(expected_m > 0 and m > 0 and n > 0 and k > 0 and g > 0,
             "expected_m > 0 and m > 0 and n > 0 and k > 0 and num_groups > 0")
    _require(d.dtype == torch.bfloat16, "d.scalar_type() == torch::kBFloat16")
    _require(masked_m.dtype == torch.int32, "masked_m.scalar_type() == torch::kInt")
    _check_cd(d)
    _resolve_alpha(None, epilogue)
    sfa, sfb, gran_a, gran_b = transform_sf_pair_into_required_layout(
        a_sf, b_sf, m, n, k, recipe, recipe_a, recipe_b, g, g, disable_ue8m0_cast)
    _launch(_lib.GEMM_M_MASKED, m, n, k, a_data, sfa, major_a, gran_a, b_data, sfb, major_b, gran_b, d,
            num_groups=g, expected_m=expected_m, grouped_layout=masked_m)


# --------------------------------------------------------------------------- K-grouped
def k_grouped_fp8_gemm_tn_contiguous(a, b, d, ks_cpu: Optional[Sequence[int]], grouped_layout, c=None,
                                     recipe=(1, 1, 128), compiled_dims: str = "mn", use_psum_layout: bool = False,
                                     epilogue=None) -> None:
    """D[g] (+= C[g]) = A[k_g, :]^T @ B[k_g, :]; a [sum_k, m], b [sum_k, n] (csrc/apis/gemm.hpp:324-375)."""
    (a_data, a_sf), (b_data, b_sf) = a, b
    recipe = tuple(recipe)
    _require(recipe[0] == 1 and recipe[1] == 1, "std::get<0>(recipe) == 1 and std::get<1>(recipe) == 1")
    gran_k = recipe[2]
    k_alignment = get_mk_alignment_for_contiguous_layout()
    _require(gran_k in (32, 128), "gran_k == 32 or gran_k == 128")
    _require(k_alignment % 128 == 0, "k_alignment % 128 == 0")
    _require(d.dim() == 3 and a_data.dim() == 2 and b_data.dim() == 2, "t.dim() == N")
    g, m, n = d.shape
    sum_k, m_ = a_data.shape
    sum_k_, n_ = b_data.shape
    _require(grouped_layout.is_contiguous() and grouped_layout.dtype == torch.int32 and grouped_layout.numel() == g,
             "static_cast<int>(grouped_layout.numel()) == num_groups")
    if ks_cpu is not None and len(ks_cpu) > 0:
        _require(len(ks_cpu) == g, "ks_cpu.value().size() == num_groups")
        for kk in ks_cpu:
            _require(kk % k_alignment == 0, "k % k_alignment == 0")
        total = sum(ks_cpu)
    else:
        _require(use_psum_layout, "use_psum_layout")
        total = sum_k
    _require(m == m_ and n == n_ and total == sum_k and total == sum_k_, "m == m_ and n == n_ and sum_k == sum_k_ and sum_k == sum_k__")
    _require(a_data.is_contiguous() and b_data.is_contiguous() and d.is_contiguous(), "is_contiguous()")
    _require(c is None or c.is_contiguous(), "not c.has_value() or c.value().is_contiguous()")
    _require(a_data.dtype == torch.float8_e4m3fn and b_data.dtype == torch.float8_e4m3fn, "FP8 operands")
    _resolve_alpha(None, epilogue)
    if _early_return(m, n, total, d, c):
        return

    def sf_of(sf):
        if sf.dtype == torch.float32:
            return get_k_grouped_mn_major_tma_aligned_packed_ue8m0_tensor(sf, grouped_layout, ks_cpu, gran_k,
                                                                          k_alignment, use_psum_layout)
        _require(sf.dtype == torch.int32 and gran_k == 32, "pre-packed UE8M0 is only accepted for gran_k == 32")
        _require(sf.dim() == 2 and sf.size(1) % 4 == 0 and sf.stride(1) == 1 and sf.stride(0) % 4 == 0,
                 "sf.stride(0) >= mn and sf.stride(1) == 1")
        return sf

    sfa, sfb = sf_of(a_sf), sf_of(b_sf)
    # a / b are [sum_k, mn] row-major, i.e. MN-major operands; their scales are [packed_k, mn] with row pitch stride(0)
    args_a = (a_data.t(), _SfView(sfa), _MN, gran_k)
    args_b = (b_data.t(), _SfView(sfb), _MN, gran_k)
    _launch(_lib.GEMM_K_GROUPED_PSUM if use_psum_layout else _lib.GEMM_K_GROUPED, m, n, total, *args_a, *args_b, d,
            num_groups=g, alignment=k_alignment, accumulate=c is not None, grouped_layout=grouped_layout)


def k_grouped_fp4_gemm_nt_contiguous(a, b, d, ks_cpu: Optional[Sequence[int]], grouped_layout, c=None,
                                     recipe=(1, 1, 32), compiled_dims: str = "mn", use_psum_layout: bool = False,
                                     epilogue=None) -> None:
    """D[g] (+= C[g]) = A[:, k_g] @ B[:, k_g]^T over packed-FP4 operands a [m, sum_k / 2], b [n, sum_k / 2] (K-major,
    the groups laid along K), scales [sum_k / 32, mn] FP32 or packed int32 [., mn]; runs on kind::mxf4
    (csrc/apis/gemm.hpp:433-491).  The K alignment (get_mk_alignment_for_contiguous_layout) must be a multiple of 256;
    padding codes must be zero."""
    (a_data, a_sf), (b_data, b_sf) = a, b
    _require(tuple(recipe) == (1, 1, 32), "recipe == std::make_tuple(1, 1, 32)")
    _require(a_data.dtype == PACKED_FP4 and b_data.dtype == PACKED_FP4,
             "a.first.scalar_type() == kPackedFP4 and b.first.scalar_type() == kPackedFP4")
    _require(a_data.dim() == 2 and b_data.dim() == 2 and d.dim() == 3, "t.dim() == N")
    major_a, major_b = _major(a_data), _major(b_data)
    _require(major_a == _K and major_b == _K, "major_a == cute::UMMA::Major::K and major_b == cute::UMMA::Major::K")
    k_alignment = get_mk_alignment_for_contiguous_layout()
    _require(k_alignment % 256 == 0, "k_alignment % 256 == 0")
    g, m, n = d.shape
    m_, sum_k_ = _logical_mn_k(a_data, major_a)
    n_, sum_k__ = _logical_mn_k(b_data, major_b)
    _require(grouped_layout.is_contiguous() and grouped_layout.dtype == torch.int32 and grouped_layout.numel() == g,
             "static_cast<int>(grouped_layout.numel()) == num_groups")
    if ks_cpu is not None and len(ks_cpu) > 0:
        _require(len(ks_cpu) == g, "ks_cpu.value().size() == num_groups")
        for kk in ks_cpu:
            _require(kk % k_alignment == 0, "k % k_alignment == 0")
        total = sum(ks_cpu)
    else:
        _require(use_psum_layout, "use_psum_layout")
        total = sum_k_
    _require(m == m_ and n == n_ and total == sum_k_ and total == sum_k__, "m == m_ and n == n_ and sum_k == sum_k_ and sum_k == sum_k__")
    _require(a_data.is_contiguous() and b_data.is_contiguous() and d.is_contiguous(), "is_contiguous()")
    _require(c is None or c.is_contiguous(), "not c.has_value() or c.value().is_contiguous()")
    _resolve_alpha(None, epilogue)
    if _early_return(m, n, total, d, c):
        return

    def sf_of(sf):
        if sf.dtype == torch.float32:
            return get_k_grouped_mn_major_tma_aligned_packed_ue8m0_tensor(sf, grouped_layout, ks_cpu, 32, k_alignment,
                                                                          use_psum_layout)
        _require(sf.dtype == torch.int32 and sf.dim() == 2 and sf.stride(1) == 1 and sf.stride(0) % 4 == 0,
                 "sf.stride(0) >= mn and sf.stride(1) == 1")
        return sf

    sfa, sfb = sf_of(a_sf), sf_of(b_sf)
    _launch(_lib.GEMM_K_GROUPED_PSUM if use_psum_layout else _lib.GEMM_K_GROUPED, m, n, total,
            a_data, _SfView(sfa), _K, 32, b_data, _SfView(sfb), _K, 32, d,
            num_groups=g, alignment=k_alignment, accumulate=c is not None, grouped_layout=grouped_layout)


class _SfView:
    """Adapter: a [packed_k, mn] scale tensor seen through the (.., mn, packed_k) stride convention."""

    def __init__(self, t: torch.Tensor):
        self._t = t
        self.k_rows = t.size(0)      # the tensor map's real extent: reads past it are zero-filled, not made

    def data_ptr(self):
        return self._t.data_ptr()

    def stride(self, i):
        assert i == -1
        return self._t.stride(0)
