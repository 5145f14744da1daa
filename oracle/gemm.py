"""CPU oracle: the block-scaled GEMM family, as "dequantise, then matmul".

TEST INFRASTRUCTURE ONLY (see oracle/quant.py).  The reference has no CPU GEMM; its
tests compare the GPU kernels with torch matmuls of the un-quantised inputs
(tests/generators.py:350-375, 378-419, 446-485, 488-608).  The functions here are the
dequantised variant of the same contractions: they take exactly the tensors the
kernels take (quantised data + scales) and accumulate in float32 / float64 on the
host, so that any difference from the kernel output is kernel error, not
quantisation error.

The BF16 family (tests/test_bf16.py:23-196 of the reference: torch matmuls of the same BF16 tensors) uses the same
contractions on the operands' float values; there is nothing to dequantise.

Data conventions: FP8 operands are uint8 arrays of E4M3 bit patterns, FP4 operands
are uint8 arrays with two E2M1 codes per byte (low nibble first); scales are either
float32 power-of-two arrays or packed int32 (four UE8M0 bytes per word, K order).
"""
from __future__ import annotations

from typing import Optional, Sequence

import numpy as np

from .quant import (align, bf16_round, cast_back_from_fp4, cast_back_from_fp8,
                    unpack_ue8m0_from_int)


def dequant_operand(data: np.ndarray, sf: np.ndarray, gran_mn: int, gran_k: int,
                    is_fp4: bool) -> np.ndarray:
    """Dequantise one [.., mn, k] K-major operand to float32.

    `sf` is float32 [.., ceil(mn/gran_mn), ceil(k/gran_k)] or packed int32
    [.., mn, ceil(k/(4*gran_k))] (then gran_mn must be 1).
    """
    packed = sf.dtype == np.int32
    if packed:
        assert gran_mn == 1
        sf = unpack_ue8m0_from_int(np.ascontiguousarray(sf))
    mn = data.shape[-2]
    if gran_mn != 1:
        sf = np.take(sf, np.arange(mn) // gran_mn, axis=-2)
    if is_fp4:
        return cast_back_from_fp4(data, sf, gran_k)
    return cast_back_from_fp8(data, sf, gran_k)


def to_cd(acc: np.ndarray, cd_dtype: str) -> np.ndarray:
    acc = acc.astype(np.float32)
    return bf16_round(acc) if cd_dtype == "bf16" else acc


def gemm_nt(a: np.ndarray, b: np.ndarray, c: Optional[np.ndarray] = None,
            alpha: float = 1.0, cd_dtype: str = "bf16") -> np.ndarray:
    """D = alpha * A @ B^T (+ C) on dequantised float32 operands, float64 accumulate."""
    acc = a.astype(np.float64) @ b.astype(np.float64).T
    acc = np.float32(alpha) * acc.astype(np.float32) if alpha != 1.0 else acc
    if c is not None:
        acc = acc + c.astype(np.float64)
    return to_cd(acc, cd_dtype)


def m_grouped_contiguous(a: np.ndarray, b: np.ndarray, grouped_layout: np.ndarray) -> np.ndarray:
    """Rows of A pick B[g] by their entry in `grouped_layout` (-1 rows are left zero).

    tests/generators.py:378-419 of the reference.
    """
    m = a.shape[0]
    n = b.shape[1]
    d = np.zeros((m, n), dtype=np.float32)
    for g in range(b.shape[0]):
        rows = np.nonzero(grouped_layout == g)[0]
        if rows.size:
            d[rows] = a[rows].astype(np.float64) @ b[g].astype(np.float64).T
    return bf16_round(d)


def m_grouped_psum(a: np.ndarray, b: np.ndarray, psum_layout: Sequence[int], alignment: int) -> np.ndarray:
    """PSUM layout: group g owns rows [align(end[g-1], alignment), end[g])."""
    m = a.shape[0]
    d = np.zeros((m, b.shape[1]), dtype=np.float32)
    prev = 0
    for g, end in enumerate(psum_layout):
        start = align(prev, alignment)
        if end > start:
            d[start:end] = a[start:end].astype(np.float64) @ b[g].astype(np.float64).T
        prev = end
    return bf16_round(d)


def m_grouped_masked(a: np.ndarray, b: np.ndarray, masked_m: Sequence[int]) -> np.ndarray:
    """a [G, max_m, K], b [G, N, K]; only the first masked_m[g] rows of each group are defined.

    tests/generators.py:446-485 of the reference.
    """
    g_, max_m, _ = a.shape
    d = np.zeros((g_, max_m, b.shape[1]), dtype=np.float32)
    for g in range(g_):
        mm = int(masked_m[g])
        if mm:
            d[g, :mm] = a[g, :mm].astype(np.float64) @ b[g].astype(np.float64).T
    return bf16_round(d)


def k_grouped_tn(a: np.ndarray, b: np.ndarray, group_bounds: Sequence[tuple],
                 c: Optional[np.ndarray] = None, cd_dtype: str = "f32") -> np.ndarray:
    """D[g] = A[k0:k1, :]^T @ B[k0:k1, :] (+ C[g]); a [sum_k, M], b [sum_k, N] dequantised.

    tests/generators.py:527-608 of the reference.
    """
    m, n = a.shape[1], b.shape[1]
    out = np.zeros((len(group_bounds), m, n), dtype=np.float32)
    for g, (k0, k1) in enumerate(group_bounds):
        acc = a[k0:k1].astype(np.float64).T @ b[k0:k1].astype(np.float64)
        if c is not None:
            acc = acc + c[g].astype(np.float64)
        out[g] = acc
    return to_cd(out, cd_dtype)


def gemm_nt_f32(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """float32 BLAS contraction of dequantised operands: the timed CPU baseline (the reference's
    tests contract in float32 too, tests/generators.py:363); BF16-rounded like the kernels' output."""
    return bf16_round(np.asarray(a, dtype=np.float32) @ np.asarray(b, dtype=np.float32).T)
