"""Scale-factor layout transforms behind the `deep_gemm` names.

Mirrors the reference's layout API (csrc/apis/layout.hpp:11-147, csrc/utils/layout.hpp:85-140,
csrc/jit_kernels/impls/smxx_layout.hpp:60-347): same argument names, defaults and failure
behaviour (RuntimeError whose text names the failed condition).  The packing itself runs in the
CUDA library (dg_sf_pack_ue8m0*); nothing here computes on the host.
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple, Union

import torch

from . import _lib
from .utils.math import align, ceil_div


def _require(cond: bool, text: str) -> None:
    if not cond:
        raise RuntimeError(f"Assertion failed: {text}")


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def get_tma_aligned_size(x: int, element_size: int) -> int:
    """Rows padded so that a column starts on a 16-byte boundary (csrc/utils/math.hpp:23-27)."""
    _require(16 % element_size == 0, "kNumTMAAlignmentBytes % element_size == 0")
    return align(x, 16 // element_size)


def set_mk_alignment_for_contiguous_layout(new_value: int) -> None:
    _lib.check(_lib.lib().dg_set_mk_alignment_for_contiguous_layout(int(new_value)))


def get_mk_alignment_for_contiguous_layout() -> int:
    return int(_lib.lib().dg_get_mk_alignment_for_contiguous_layout())


def get_theoretical_mk_alignment_for_contiguous_layout(expected_m: Optional[int] = None) -> int:
    return int(_lib.lib().dg_get_theoretical_mk_alignment_for_contiguous_layout(int(expected_m or 0)))


def get_mn_major_tma_aligned_tensor(sf: torch.Tensor) -> torch.Tensor:
    """FP32 scales [(b,) mn, k] -> same values with MN contiguous and 16-byte-aligned columns.

    Only the legacy FP32-scale recipes use this (smxx_layout.hpp:60-106); it is a strided copy.
    """
    _require(sf.dim() in (2, 3) and sf.dtype == torch.float32, "sf.dim() in (2, 3) and sf.dtype == float32")
    batched = sf.unsqueeze(0) if sf.dim() == 2 else sf
    b, mn, k = batched.shape
    amn = get_tma_aligned_size(mn, 4)
    if (batched.stride(0) == amn * k or sf.dim() == 2) and batched.stride(1) == 1 and batched.stride(2) == amn:
        return sf
    out = torch.empty_strided((b, mn, k), (amn * k, 1, amn), dtype=sf.dtype, device=sf.device)
    out.copy_(batched)
    return out.squeeze(0) if sf.dim() == 2 else out


def _pack(sf: torch.Tensor, mn: int, gran_mn: int, psum_layout: Optional[torch.Tensor], psum_alignment: int):
    """Launch the pack kernel for FP32 scales [(b,) ceil(mn / gran_mn), k]."""
    batched = sf.unsqueeze(0) if sf.dim() == 2 else sf
    b, _, sf_k = batched.shape
    pk = ceil_div(sf_k, 4)
    amn = get_tma_aligned_size(mn, 4)
    out = torch.empty_strided((b, mn, pk), (pk * amn, 1, amn), dtype=torch.int32, device=sf.device)
    if b * mn * sf_k:
        _lib.check(_lib.lib().dg_sf_pack_ue8m0(
            batched.data_ptr(), out.data_ptr(), b, mn, sf_k, gran_mn,
            batched.stride(0), batched.stride(1), batched.stride(2),
            psum_layout.data_ptr() if psum_layout is not None else None,
            psum_layout.numel() if psum_layout is not None else 0, psum_alignment, _stream(sf)))
    return out.squeeze(0) if sf.dim() == 2 else out


def get_mn_major_tma_aligned_packed_ue8m0_tensor(sf: torch.Tensor, psum_layout: Optional[torch.Tensor] = None,
                                                 allow_strided_psum_scales: bool = False) -> torch.Tensor:
    """FP32 power-of-two scales [(b,) mn, k] -> int32 [(b,) mn, ceil(k/4)], strides (.., 1, align(mn, 4)).

    With `psum_layout` (int32 cumulative row ends) rows in the gaps between groups come out zero
    (smxx_layout.hpp:133-246).
    """
    _require(sf.dim() in (2, 3), "dim == 2 or dim == 3")
    _require(sf.dtype == torch.float32, "sf.scalar_type() == torch::kFloat")
    _require(sf.is_cuda, "t.is_cuda()")
    use_psum = psum_layout is not None
    if use_psum:
        _require(sf.dim() == 2, "dim == 2 and num_sf_batches == 1")
        _require(sf.stride(0) > 0 and sf.stride(1) > 0, "batched_sf.stride(1) > 0 and batched_sf.stride(2) > 0")
        _require(psum_layout.dtype == torch.int32 and psum_layout.is_contiguous(),
                 "psum_layout->scalar_type() == torch::kInt and psum_layout->is_contiguous()")
        _require(psum_layout.numel() > 0, "psum_layout->numel() > 0")
    _require(not allow_strided_psum_scales or use_psum, "not allow_strided_psum_scales or use_psum_layout")
    _require(not (use_psum and not sf.is_contiguous()) or allow_strided_psum_scales,
             "not use_strided_psum_scales or allow_strided_psum_scales")
    alignment = get_mk_alignment_for_contiguous_layout() if use_psum else 0
    return _pack(sf, sf.size(-2), 1, psum_layout, alignment)


def get_k_grouped_mn_major_tma_aligned_packed_ue8m0_tensor(sf: torch.Tensor, grouped_layout: torch.Tensor,
                                                           ks_cpu: Optional[Sequence[int]], gran_k: int,
                                                           k_alignment: int, use_psum_layout: bool = False):
    """K-grouped FP32 scales [sum(k_g / gran_k), mn] -> int32 [sum(ceil(k_g / gran_k / 4)), mn].

    Every group starts a new packed row (smxx_layout.hpp:248-313).
    """
    _require(gran_k in (32, 128) and k_alignment % 128 == 0, "(gran_k == 32 or gran_k == 128) and k_alignment % 128 == 0")
    _require(sf.dim() == 2 and sf.is_cuda, "t.dim() == N")
    sf_k, mn = sf.shape
    num_groups = grouped_layout.numel()
    _require(sf.is_contiguous(), "sf.is_contiguous()")
    _require(num_groups <= 128 and mn % 4 == 0, "num_groups <= 128 and mn % 4 == 0")
    _require(grouped_layout.is_contiguous() and grouped_layout.dtype == torch.int32,
             "grouped_layout.is_contiguous() and grouped_layout.scalar_type() == torch::kInt")
    synced = ks_cpu is not None and len(ks_cpu) > 0
    if synced:
        _require(len(ks_cpu) == num_groups, "ks_cpu.value().size() == num_groups")
        ref_sf_k = packed = 0
        for k in ks_cpu:
            _require(k % k_alignment == 0 and k % gran_k == 0, "k % k_alignment == 0 and k % gran_k == 0")
            ref_sf_k += k // gran_k
            packed += ceil_div(k // gran_k, 4)
        _require(ref_sf_k == sf_k, "ref_sf_k == sf_k")
    else:
        _require(use_psum_layout, "use_psum_layout")
        packed = (sf_k + num_groups * 3) // 4
    out = torch.empty((packed, mn), dtype=torch.int32, device=sf.device)
    if packed:
        _lib.check(_lib.lib().dg_sf_pack_ue8m0_k_grouped(
            sf.data_ptr(), out.data_ptr(), grouped_layout.data_ptr(), num_groups, mn, sf_k, packed,
            gran_k, k_alignment, int(use_psum_layout), _stream(sf)))
    return out


def check_sf_layout(sf: torch.Tensor, mn: int, k: int, gran_mn: int, gran_k: int, num_groups: Optional[int],
                    tma_stride_check: bool = False, type_check: Optional[torch.dtype] = None) -> torch.Tensor:
    """Shape / stride validation of a scale tensor (csrc/utils/layout.hpp:101-140)."""
    if type_check is not None:
        _require(sf.dtype == type_check, "sf.scalar_type() == type_check.value()")
    _require(sf.dtype in (torch.float32, torch.int32), "sf_dtype == torch::kFloat or sf_dtype == torch::kInt")
    _require(sf.dim() == int(num_groups is not None) + 2, "sf.dim() == static_cast<int>(num_groups.has_value()) + 2")
    if num_groups is not None:
        _require(sf.size(-3) == num_groups, "sf.size(-3) == num_groups.value()")
    _require(sf.size(-2) == ceil_div(mn, gran_mn), "sf.size(-2) == ceil_div(mn, gran_mn)")
    _require(sf.size(-1) == ceil_div(k, gran_k * (1 if sf.dtype == torch.float32 else 4)),
             "sf.size(-1) == ceil_div(k, gran_k * (sf_dtype == torch::kFloat ? 1 : 4))")
    if tma_stride_check:
        if num_groups is not None:
            _require(sf.stride(-3) == sf.stride(-1) * sf.size(-1), "sf.stride(-3) == sf.stride(-1) * sf.size(-1)")
        _require(sf.stride(-2) == 1 or mn == 1, "sf.stride(-2) == 1 or mn == 1")
        _require(sf.stride(-1) >= get_tma_aligned_size(mn, sf.element_size()), "sf.stride(-1) >= compact_stride")
        _require(sf.stride(-1) % 4 == 0, "sf.stride(-1) % 4 == 0")
    return sf


def get_default_recipe(sfa_dtype: torch.dtype, sfb_dtype: torch.dtype) -> Tuple[int, int, int]:
    """(1, 128, 128) for FP32 weight scales, (1, 1, 128) for packed ones (csrc/utils/layout.hpp:85-98)."""
    _require(sfb_dtype in (torch.float32, torch.int32), "sfb_dtype == torch::kFloat or sfb_dtype == torch::kInt")
    return (1, 128, 128) if sfb_dtype == torch.float32 else (1, 1, 128)


def transform_sf_into_required_layout(sf: torch.Tensor, mn: int, k: int,
                                      recipe: Union[Tuple[int, int, int], Tuple[int, int]],
                                      num_groups: Optional[int] = None, is_sfa: Optional[bool] = None,
                                      disable_ue8m0_cast: bool = False,
                                      psum_layout: Optional[torch.Tensor] = None,
                                      allow_strided_psum_scales: bool = False) -> torch.Tensor:
    """Bring one scale tensor into the packed, MN-major layout the kernels read (csrc/apis/layout.hpp:11-60)."""
    recipe = tuple(recipe)
    if len(recipe) == 3:
        _require(is_sfa is not None, "is_sfa.has_value()")
        gran_mn, gran_k = (recipe[0] if is_sfa else recipe[1]), recipe[2]
    elif len(recipe) == 2:
        _require(is_sfa is None, "not is_sfa.has_value()")
        gran_mn, gran_k = recipe
    else:
        raise RuntimeError("Invalid recipe")
    check_sf_layout(sf, mn, k, gran_mn, gran_k, num_groups)
    if sf.dtype == torch.float32 and gran_k in (32, 128):
        # Blackwell consumes UE8M0 only: the FP32-scale kernels of older parts have no counterpart here
        _require(not disable_ue8m0_cast, "not disable_ue8m0_cast")
        use_psum = psum_layout is not None
        _require(not allow_strided_psum_scales or use_psum, "not allow_strided_psum_scales or use_psum_layout")
        if use_psum:
            _require(sf.dim() == 2, "dim == 2 and num_sf_batches == 1")
            _require(sf.is_contiguous() or allow_strided_psum_scales,
                     "not use_strided_psum_scales or allow_strided_psum_scales")
        alignment = get_mk_alignment_for_contiguous_layout() if use_psum else 0
        return _pack(sf, mn, gran_mn, psum_layout, alignment)
    if sf.dtype == torch.int32 and gran_mn == 1 and gran_k in (32, 128):
        return check_sf_layout(sf, mn, k, gran_mn, gran_k, num_groups, tma_stride_check=True, type_check=torch.int32)
    raise RuntimeError("Unknown SF transformation")


def transform_sf_pair_into_required_layout(sfa, sfb, m, n, k, recipe, recipe_a, recipe_b, num_groups_a, num_groups_b,
                                           disable_ue8m0_cast=False, psum_layout=None,
                                           allow_strided_psum_scales=False):
    """Both operands' scales + their K granularities (csrc/apis/layout.hpp:62-90)."""
    if recipe_a is None and recipe is None:
        recipe = get_default_recipe(sfa.dtype, sfb.dtype)
    _require((recipe_a is None) == (recipe_b is None), "recipe_a.has_value() == recipe_b.has_value()")
    _require((recipe_a is None) != (recipe is None), "recipe_a.has_value() != recipe.has_value()")
    if recipe is not None:
        ta = transform_sf_into_required_layout(sfa, m, k, recipe, num_groups_a, True, disable_ue8m0_cast,
                                               psum_layout, allow_strided_psum_scales)
        tb = transform_sf_into_required_layout(sfb, n, k, recipe, num_groups_b, False, disable_ue8m0_cast)
        return ta, tb, recipe[2], recipe[2]
    ta = transform_sf_into_required_layout(sfa, m, k, recipe_a, num_groups_a, None, disable_ue8m0_cast,
                                           psum_layout, allow_strided_psum_scales)
    tb = transform_sf_into_required_layout(sfb, n, k, recipe_b, num_groups_b, None, disable_ue8m0_cast)
    return ta, tb, recipe_a[1], recipe_b[1]
