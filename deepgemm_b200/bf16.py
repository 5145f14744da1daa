"""BF16 GEMM family behind the reference's `bf16_gemm_*`, `m_grouped_bf16_gemm_*` and
`k_grouped_bf16_gemm_tn_contiguous` (csrc/apis/gemm.hpp:492-726): the block-scaled kernel's layouts and epilogues with
BF16 operands and no scale factors (tcgen05 kind::f16, FP32 accumulation).  Every call runs this library's own kernel
(the reference hands the plain dense case to cuBLASLt when it is available)."""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from . import _lib
from .layout import _require, get_mk_alignment_for_contiguous_layout
from .ops import _K, _MN, _check_cd, _early_return, _launch, _major, _resolve_alpha


def _check_bf16(a: torch.Tensor, b: torch.Tensor) -> None:
    _require(a.dtype == torch.bfloat16, "a.scalar_type() == torch::kBFloat16")
    _require(b.dtype == torch.bfloat16, "b.scalar_type() == torch::kBFloat16")


def bf16_gemm_nt(a: torch.Tensor, b: torch.Tensor, d: torch.Tensor, c: Optional[torch.Tensor] = None,
                 compiled_dims: str = "nk", alpha: Optional[float] = None, epilogue=None) -> None:
    """D = alpha * A @ B^T (+ C); a [m, k], b [n, k], either of them K-major or MN-major (csrc/apis/gemm.hpp:492-539)."""
    major_a, major_b = _major(a), _major(b)
    _check_cd(d)
    _require(a.dim() == 2 and b.dim() == 2 and d.dim() == 2, "t.dim() == N")
    (m, k), (n, k_) = a.shape, b.shape
    _require(m == d.size(0) and n == d.size(1) and k == k_, "m == m_ and n == n_ and k == k_")
    _check_bf16(a, b)
    _require(d.dtype in (torch.bfloat16, torch.float32), "d.scalar_type() == torch::kBFloat16 or d.scalar_type() == torch::kFloat")
    scale = _resolve_alpha(alpha, epilogue, c, d, value_epilogues=True)
    if _early_return(m, n, k, d, c):
        return
    _launch(_lib.GEMM_NORMAL, m, n, k, a, None, major_a, 0, b, None, major_b, 0, d, accumulate=c is not None,
            alpha=scale, epilogue=epilogue)


def bf16_gemm_nn(a, b, d, c=None, compiled_dims: str = "nk", alpha=None, epilogue=None) -> None:
    """b given as [k, n] (csrc/apis/gemm.hpp:541-549)."""
    bf16_gemm_nt(a, b.transpose(0, 1), d, c, compiled_dims, alpha, epilogue)


def bf16_gemm_tn(a, b, d, c=None, compiled_dims: str = "mn", alpha=None, epilogue=None) -> None:
    """a given as [k, m], b as [k, n] (csrc/apis/gemm.hpp:551-559)."""
    bf16_gemm_nt(a.transpose(0, 1), b.transpose(0, 1), d, c, compiled_dims, alpha, epilogue)


def bf16_gemm_tt(a, b, d, c=None, compiled_dims: str = "mn", alpha=None, epilogue=None) -> None:
    """a given as [k, m] (csrc/apis/gemm.hpp:561-569)."""
    bf16_gemm_nt(a.transpose(0, 1), b, d, c, compiled_dims, alpha, epilogue)


def m_grouped_bf16_gemm_nt_contiguous(a: torch.Tensor, b: torch.Tensor, d: torch.Tensor, grouped_layout: torch.Tensor,
                                      compiled_dims: str = "nk", use_psum_layout: bool = False,
                                      ensure_zero_padding: bool = True,
                                      expected_m_for_psum_layout: Optional[int] = None, epilogue=None) -> None:
    """Rows of A [m, k] are grouped by expert; B is [G, n, k] (csrc/apis/gemm.hpp:571-627)."""
    major_a, major_b = _major(a), _major(b)
    _require(major_a == _K, "major_a == cute::UMMA::Major::K")
    _require(grouped_layout.is_contiguous(), "grouped_layout.is_contiguous()")
    _require(a.dim() == 2 and b.dim() == 3 and d.dim() == 2, "t.dim() == N")
    (m, k), (num_groups, n, k_) = a.shape, b.shape
    _require(m == d.size(0) and n == d.size(1) and k == k_, "m == m_ and n == n_ and k == k_")
    _require(n > 0 and k > 0 and num_groups > 0, "n > 0 and k > 0 and num_groups > 0")
    _check_bf16(a, b)
    _require(d.dtype == torch.bfloat16, "d.scalar_type() == torch::kBFloat16")
    _require(grouped_layout.dtype == torch.int32, "grouped_layout.scalar_type() == torch::kInt")
    if use_psum_layout:
        _require(grouped_layout.dim() == 1 and grouped_layout.numel() == num_groups, "num_groups == num_groups_")
    else:
        _require(grouped_layout.dim() == 1 and grouped_layout.numel() == m, "m == m__")
        _require(expected_m_for_psum_layout is None, "not expected_m_for_psum_layout.has_value()")
    _check_cd(d)
    _resolve_alpha(None, epilogue)
    if m == 0:
        return
    _launch(_lib.GEMM_M_PSUM if use_psum_layout else _lib.GEMM_M_CONTIGUOUS, m, n, k, a, None, major_a, 0,
            b, None, major_b, 0, d, num_groups=num_groups, alignment=get_mk_alignment_for_contiguous_layout(),
            expected_m=expected_m_for_psum_layout or 0, grouped_layout=grouped_layout,
            skip_padding_rows=use_psum_layout and not ensure_zero_padding)


def m_grouped_bf16_gemm_nn_contiguous(a, b, d, grouped_layout, compiled_dims: str = "nk", use_psum_layout: bool = False,
                                      ensure_zero_padding: bool = True, epilogue=None) -> None:
    """b given as [G, k, n] (csrc/apis/gemm.hpp:629-637)."""
    m_grouped_bf16_gemm_nt_contiguous(a, b.transpose(1, 2), d, grouped_layout, compiled_dims, use_psum_layout,
                                      ensure_zero_padding, None, epilogue)


def m_grouped_bf16_gemm_nt_masked(a: torch.Tensor, b: torch.Tensor, d: torch.Tensor, masked_m: torch.Tensor,
                                  expected_m: int, compiled_dims: str = "nk", epilogue=None) -> None:
    """a [G, m, k], b [G, n, k], d [G, m, n]; only the first masked_m[g] rows of group g are computed
    (csrc/apis/gemm.hpp:639-678)."""
    major_a, major_b = _major(a), _major(b)
    _require(major_a == _K and major_b == _K, "major_a == cute::UMMA::Major::K and major_b == cute::UMMA::Major::K")
    _require(masked_m.is_contiguous(), "masked_m.is_contiguous()")
    _require(a.dim() == 3 and b.dim() == 3 and d.dim() == 3, "t.dim() == N")
    (g, m, k), (g_, n, k_), (g__, m_, n_) = a.shape, b.shape, d.shape
    _require(g == g_ and g == g__ and g == masked_m.numel(),
             "num_groups == num_groups_ and num_groups == num_groups__ and num_groups == num_groups___")
    _require(m == m_ and n == n_ and k == k_, "m == m_ and n == n_ and k == k_")
    _require(expected_m > 0 and m > 0 and n > 0 and k > 0 and g > 0,
             "expected_m > 0 and m > 0 and n > 0 and k > 0 and num_groups > 0")
    _check_bf16(a, b)
    _require(d.dtype == torch.bfloat16, "d.scalar_type() == torch::kBFloat16")
    _require(masked_m.dtype == torch.int32, "masked_m.scalar_type() == torch::kInt")
    _require(a.is_contiguous() and b.is_contiguous() and d.is_contiguous(), "is_contiguous()")
    _check_cd(d)
    _resolve_alpha(None, epilogue)
    _launch(_lib.GEMM_M_MASKED, m, n, k, a, None, major_a, 0, b, None, major_b, 0, d, num_groups=g,
            expected_m=expected_m, grouped_layout=masked_m)


def k_grouped_bf16_gemm_tn_contiguous(a: torch.Tensor, b: torch.Tensor, d: torch.Tensor,
                                      ks_cpu: Optional[Sequence[int]], grouped_layout: torch.Tensor,
                                      c: Optional[torch.Tensor] = None, compiled_dims: str = "mn",
                                      use_psum_layout: bool = False, epilogue=None) -> None:
    """D[g] (+= C[g]) = A[k_g, :]^T @ B[k_g, :]; a [sum_k, m], b [sum_k, n], d [G, m, n] (csrc/apis/gemm.hpp:680-725)."""
    _require(d.dim() == 3 and a.dim() == 2 and b.dim() == 2, "t.dim() == N")
    g, m, n = d.shape
    (sum_k, m_), (sum_k_, n_) = a.shape, b.shape
    k_alignment = get_mk_alignment_for_contiguous_layout()
    _require(k_alignment % 128 == 0, "k_alignment % 128 == 0")
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
    _require(m == m_ and n == n_ and total == sum_k and total == sum_k_,
             "m == m_ and n == n_ and sum_k == sum_k_ and sum_k == sum_k__")
    _require(a.is_contiguous() and b.is_contiguous() and d.is_contiguous(), "is_contiguous()")
    _require(c is None or c.is_contiguous(), "not c.has_value() or c.value().is_contiguous()")
    _check_bf16(a, b)
    _resolve_alpha(None, epilogue, c, d, value_epilogues=True)
    if _early_return(m, n, total, d, c):
        return
    # a / b are [sum_k, mn] row-major, i.e. MN-major operands
    _launch(_lib.GEMM_K_GROUPED_PSUM if use_psum_layout else _lib.GEMM_K_GROUPED, m, n, total, a.t(), None, _MN, 0,
            b.t(), None, _MN, 0, d, num_groups=g, alignment=k_alignment, accumulate=c is not None,
            grouped_layout=grouped_layout, epilogue=epilogue)
