"""Fused activation cast: BF16 -> E4M3 with per-group UE8M0 scales in one CUDA kernel.

The arithmetic is the reference helper per_token_cast_to_fp8(use_ue8m0=True) (deep_gemm/utils/math.py:13-49), which
the reference runs as torch eager code and recommends fusing into the producer (README.md:71,133-138;
docs/scaling-factor-format.md:44-48).  The kernel writes the scales in the layout the consumer reads, so neither
transform_sf_into_required_layout nor a copy into the Mega MoE buffer runs afterwards.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch

from . import _lib
from .utils.math import align, ceil_div

_MODES = {"float": _lib.CAST_SF_FLOAT, "packed": _lib.CAST_SF_PACKED_ROW_MAJOR, "gemm": _lib.CAST_SF_PACKED_MN_MAJOR}


def _require(cond: bool, text: str) -> None:
    if not cond:
        raise RuntimeError(f"Assertion failed: {text}")


def per_token_cast_to_fp8_fused(x: torch.Tensor, gran_k: int = 128, sf_layout: str = "gemm",
                                out: Optional[torch.Tensor] = None,
                                sf_out: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """x: CUDA BF16 [rows, cols] with unit column stride.  Returns (E4M3 [rows, cols], scales) where the scales are

    * sf_layout "float":  float32 [rows, ceil(cols / gran_k)] powers of two (what the reference helper returns),
    * sf_layout "packed": int32 [rows, ceil(groups / 4)] (the helper's use_packed_ue8m0 form),
    * sf_layout "gemm":   int32 [rows, ceil(groups / 4)] with strides (1, align(rows, 4)): ready to be passed to the
      GEMMs as a pre-packed scale tensor (check_sf_layout of csrc/utils/layout.hpp:101-140 accepts it as is).

    `out` / `sf_out` let the caller have the results written in place (for instance into the x / x_sf views of a Mega
    MoE buffer, sf_layout "packed").
    """
    _require(x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2, "x is a 2-D CUDA BF16 tensor")
    _require(gran_k in (32, 128), "gran_k in (32, 128)")
    _require(sf_layout in _MODES, "sf_layout in ('float', 'packed', 'gemm')")
    rows, cols = x.shape
    _require(x.stride(1) == 1 and cols % 8 == 0 and x.stride(0) % 8 == 0, "x.stride(1) == 1 and cols % 8 == 0")
    groups = ceil_div(cols, gran_k)
    words = ceil_div(groups, 4)
    if out is None:
        out = torch.empty((rows, cols), dtype=torch.float8_e4m3fn, device=x.device)
    _require(out.dtype == torch.float8_e4m3fn and out.shape == x.shape and out.stride(1) == 1, "out matches x")
    if sf_layout == "float":
        if sf_out is None:
            sf_out = torch.empty((rows, groups), dtype=torch.float32, device=x.device)
        _require(sf_out.dtype == torch.float32 and tuple(sf_out.shape) == (rows, groups) and sf_out.stride(1) == 1,
                 "sf_out is float32 [rows, groups]")
        sf_ld = sf_out.stride(0)
    elif sf_layout == "packed":
        if sf_out is None:
            sf_out = torch.empty((rows, words), dtype=torch.int32, device=x.device)
        _require(sf_out.dtype == torch.int32 and tuple(sf_out.shape) == (rows, words) and sf_out.stride(1) == 1,
                 "sf_out is int32 [rows, ceil(groups / 4)]")
        sf_ld = sf_out.stride(0)
    else:
        if sf_out is None:
            pitch = align(rows, 4)
            sf_out = torch.empty(words * pitch, dtype=torch.int32, device=x.device).as_strided((rows, words), (1, pitch))
        _require(sf_out.dtype == torch.int32 and tuple(sf_out.shape) == (rows, words) and sf_out.stride(0) == 1,
                 "sf_out is int32 [rows, ceil(groups / 4)] with unit row stride")
        sf_ld = sf_out.stride(1) if words > 1 else max(align(rows, 4), rows)
    if rows == 0 or cols == 0:
        return out, sf_out
    args = _lib.CastArgs(x.data_ptr(), x.stride(0), rows, cols, gran_k, out.data_ptr(), out.stride(0), sf_out.data_ptr(),
                         _MODES[sf_layout], sf_ld, torch.cuda.current_stream(x.device).cuda_stream)
    _lib.check(_lib.lib().dg_per_token_cast_to_fp8(C.byref(args)))
    return out, sf_out
