"""Torch helpers for block-scaled quantisation (device-agnostic: run on CUDA or CPU tensors).

Same names, arguments and bit-exact results as the reference's ``deep_gemm/utils/math.py``
(line ranges per function); they are the quantisation contract of the GEMM operands:
power-of-two (UE8M0) scales per 1 x gran_k group or per 128 x 128 block, E4M3 / E2M1 codes.
"""
from __future__ import annotations

from typing import Tuple

import torch

E4M3_MAX = 448.0
E2M1_MAX = 6.0
_E2M1_MAGNITUDES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
# Decision thresholds between neighbouring E2M1 magnitudes; True = the threshold itself rounds up.
_E2M1_THRESHOLDS = ((0.25, False), (0.75, True), (1.25, False), (1.75, True), (2.5, False), (3.5, True), (5.0, False))


def ceil_div(x: int, y: int) -> int:
    return -(-x // y)


def align(x: int, y: int) -> int:
    return ceil_div(x, y) * y


def ceil_to_ue8m0(x: torch.Tensor) -> torch.Tensor:
    """|x| rounded up to a power of two with biased exponent in [1, 254] (math.py:13-16)."""
    raw = x.abs().float().view(torch.int32)
    biased = (raw >> 23) & 0xFF
    biased = biased + ((raw & 0x7FFFFF) != 0).to(torch.int32)
    return (biased.clamp(1, 254) << 23).view(torch.float32)


def pack_ue8m0_to_int(x: torch.Tensor) -> torch.Tensor:
    """Four power-of-two float32 scales -> one int32 of exponent bytes, first scale lowest (math.py:19-23)."""
    assert x.dtype == torch.float32 and x.size(-1) % 4 == 0
    raw = x.view(torch.int32)
    assert bool((raw >= 0).all()) and bool(((raw & 0x7FFFFF) == 0).all()), "scales must be positive powers of two"
    return (raw >> 23).to(torch.uint8).view(torch.int32)


def unpack_ue8m0_from_int(packed_sf: torch.Tensor) -> torch.Tensor:
    """Inverse of pack_ue8m0_to_int (math.py:151-152)."""
    return (packed_sf.view(torch.uint8).to(torch.int32) << 23).view(torch.float32)


def _scale_of(amax: torch.Tensor, qmax: float, use_ue8m0: bool) -> torch.Tensor:
    sf = amax.clamp(1e-4) / qmax
    return ceil_to_ue8m0(sf) if use_ue8m0 else sf


def _pad_and_pack(sf: torch.Tensor) -> torch.Tensor:
    # Pad the scale count to a multiple of four with 1.0 (exponent byte 127); the pad covers no data.
    extra = (-sf.size(-1)) % 4
    if extra:
        sf = torch.nn.functional.pad(sf, (0, extra), value=1.0)
    return pack_ue8m0_to_int(sf)


def per_token_cast_to_fp8(x: torch.Tensor, use_ue8m0: bool, gran_k: int = 128,
                          use_packed_ue8m0: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """1 x gran_k groups along the last axis of a 2-D tensor (math.py:26-49)."""
    assert x.dim() == 2 and (use_ue8m0 or not use_packed_ue8m0)
    m, n = x.shape
    groups = ceil_div(n, gran_k)
    xp = torch.zeros((m, groups * gran_k), dtype=torch.float32, device=x.device)
    xp[:, :n] = x
    xg = xp.view(m, groups, gran_k)
    sf = _scale_of(xg.abs().amax(dim=2), E4M3_MAX, use_ue8m0)
    q = (xg * (1.0 / sf).unsqueeze(2)).to(torch.float8_e4m3fn).view(m, groups * gran_k)[:, :n].contiguous()
    return q, (_pad_and_pack(sf) if use_packed_ue8m0 else sf)


def per_channel_cast_to_fp8(x: torch.Tensor, use_ue8m0: bool, gran_k: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """gran_k x 1 groups along the first axis (math.py:52-59)."""
    assert x.dim() == 2 and x.size(0) % gran_k == 0
    m, n = x.shape
    xg = x.float().view(m // gran_k, gran_k, n)
    sf = _scale_of(xg.abs().amax(dim=1), E4M3_MAX, use_ue8m0)
    return (xg * (1.0 / sf).unsqueeze(1)).to(torch.float8_e4m3fn).view(m, n), sf


def per_block_cast_to_fp8(x: torch.Tensor, use_ue8m0: bool, gran_k: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """gran_k x gran_k blocks (math.py:62-72)."""
    assert x.dim() == 2
    m, n = x.shape
    bm, bn = ceil_div(m, gran_k), ceil_div(n, gran_k)
    xp = torch.zeros((bm * gran_k, bn * gran_k), dtype=torch.float32, device=x.device)
    xp[:m, :n] = x
    xb = xp.view(bm, gran_k, bn, gran_k)
    sf = _scale_of(xb.abs().amax(dim=(1, 3), keepdim=True), E4M3_MAX, use_ue8m0)
    q = (xb * (1.0 / sf)).to(torch.float8_e4m3fn).view(bm * gran_k, bn * gran_k)[:m, :n].contiguous()
    return q, sf.view(bm, bn)


def per_custom_dims_cast_to_fp8(x: torch.Tensor, dims: Tuple, use_ue8m0: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    """One scale per index of `dims`, shared over all other axes (math.py:75-81)."""
    reduce_over = tuple(i for i in range(x.dim()) if i not in set(dims))
    sf = _scale_of(x.abs().float().amax(dim=reduce_over, keepdim=True), E4M3_MAX, use_ue8m0)
    return (x * (1.0 / sf)).to(torch.float8_e4m3fn), sf.squeeze()


def _quantize_to_fp4_e2m1(x: torch.Tensor) -> torch.Tensor:
    """Nearest E2M1 code; ties go to the neighbour with an even mantissa (math.py:84-96)."""
    mag = x.abs()
    code = torch.zeros_like(x, dtype=torch.uint8)
    for threshold, inclusive in _E2M1_THRESHOLDS:
        code += (mag >= threshold if inclusive else mag > threshold).to(torch.uint8)
    negative = (x < 0) & (code != 0)
    return (code | (negative.to(torch.uint8) << 3)).view(torch.int8)


def per_token_cast_to_fp4(x: torch.Tensor, use_ue8m0: bool, gran_k: int = 128,
                          use_packed_ue8m0: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """1 x gran_k MXFP4: E2M1 codes, two per int8 byte with the even element in the low nibble (math.py:99-125)."""
    m, n = x.shape
    assert n % 2 == 0 and (use_ue8m0 or not use_packed_ue8m0)
    groups = ceil_div(n, gran_k)
    xp = torch.zeros((m, groups * gran_k), dtype=torch.float32, device=x.device)
    xp[:, :n] = x
    xg = xp.view(m, groups, gran_k)
    sf = _scale_of(xg.abs().amax(dim=2), E2M1_MAX, use_ue8m0)
    codes = _quantize_to_fp4_e2m1(xg * (1.0 / sf).unsqueeze(2)).view(m, groups * gran_k // 2, 2)
    packed = ((codes[:, :, 0] & 0x0F) | ((codes[:, :, 1] & 0x0F) << 4))[:, : n // 2].contiguous()
    return packed, (_pad_and_pack(sf) if use_packed_ue8m0 else sf)


def _unpack_fp4(packed: torch.Tensor) -> torch.Tensor:
    codes = torch.empty(packed.shape[:-1] + (packed.shape[-1] * 2,), dtype=torch.int8, device=packed.device)
    codes[..., 0::2] = packed & 0x0F
    codes[..., 1::2] = (packed >> 4) & 0x0F
    return codes


def transpose_packed_fp4(a: torch.Tensor) -> torch.Tensor:
    """[m, n/2] packed codes -> [n, m/2] packed codes (math.py:128-141)."""
    assert a.dtype == torch.int8 and a.dim() == 2 and a.size(0) % 2 == 0
    t = _unpack_fp4(a).t().contiguous()
    pairs = t.view(t.size(0), t.size(1) // 2, 2)
    return ((pairs[:, :, 0] & 0x0F) | ((pairs[:, :, 1] & 0x0F) << 4)).contiguous()


def _dequantize_from_fp4_e2m1(codes: torch.Tensor) -> torch.Tensor:
    table = torch.tensor(_E2M1_MAGNITUDES, dtype=torch.float32, device=codes.device)
    mag = table[(codes & 0x07).to(torch.int64)]
    return torch.where((codes & 0x08) != 0, -mag, mag)


def cast_back_from_fp4(packed: torch.Tensor, sf: torch.Tensor, gran_k: int = 128,
                       use_packed_ue8m0: bool = False) -> torch.Tensor:
    """Dequantise packed E2M1 with 1 x gran_k scales (math.py:155-166)."""
    if use_packed_ue8m0:
        sf = unpack_ue8m0_from_int(sf)
    values = _dequantize_from_fp4_e2m1(_unpack_fp4(packed))
    group = torch.arange(values.size(-1), device=packed.device) // gran_k
    return values * sf[:, group]


def cast_back_from_fp8(x_fp8: torch.Tensor, sf: torch.Tensor, gran_k: int = 128,
                       use_packed_ue8m0: bool = False) -> torch.Tensor:
    """Dequantise E4M3 with 1 x gran_k scales (math.py:169-176)."""
    if use_packed_ue8m0:
        sf = unpack_ue8m0_from_int(sf)
    group = torch.arange(x_fp8.size(-1), device=x_fp8.device) // gran_k
    return x_fp8.float() * sf[:, group]
