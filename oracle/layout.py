"""CPU oracle: scale-factor layouts the block-scaled GEMMs consume.

TEST INFRASTRUCTURE ONLY (see oracle/quant.py).  Integer-exact restatements of

* the packed-UE8M0, MN-major, TMA-aligned scale tensor
  (reference: csrc/jit_kernels/impls/smxx_layout.hpp:108-131 and the pure-torch
  construction in tests/test_layout.py:24-46; prose in docs/scaling-factor-format.md);
* the per-row broadcast of 128x128 block scales (csrc/apis/layout.hpp:47-50);
* PSUM gap-row zeroing (tests/test_layout.py:110-179);
* the K-grouped packed layout (tests/test_layout.py:233-265);
* the Mega MoE weight / scale permutations (deep_gemm/mega/__init__.py:167-220).

Pinned: tests/golden/layout_golden.npz holds outputs of the reference's own Python for the packed layout
(tests/test_layout.py:24-46) and for both permutations (deep_gemm/mega/__init__.py:167-198), produced by running those
functions from the reference's text (tests/golden/make_layout_golden.py); tests/test_oracle_golden.py requires bit
equality, strides included.
"""
from __future__ import annotations

import numpy as np

from .quant import align, ceil_div, ue8m0_bytes


def tma_aligned_size(x: int, element_size: int) -> int:
    """csrc/utils/math.hpp:23-27."""
    assert 16 % element_size == 0
    return align(x, 16 // element_size)


def packed_ue8m0_mn_major(sf: np.ndarray) -> np.ndarray:
    """float32 power-of-two scales [(b,) mn, k] -> int32 [(b,) mn, ceil(k/4)].

    The result is a strided *view*: element strides are
    (ceil(k/4) * align(mn,4), 1, align(mn,4)), i.e. MN is the contiguous axis and
    each packed-K column is padded to a multiple of four rows (16 bytes).  Padding
    bytes inside a packed word (K not a multiple of 4) are zero.
    """
    squeeze = sf.ndim == 2
    if squeeze:
        sf = sf[None]
    b, mn, k = sf.shape
    amn, ak = tma_aligned_size(mn, 4), align(k, 4)
    by = np.zeros((b, amn, ak), dtype=np.uint8)
    by[:, :mn, :k] = ue8m0_bytes(sf)
    words = by.reshape(b, amn, ak // 4, 4).view(np.int32).reshape(b, amn, ak // 4)
    storage = np.ascontiguousarray(words.transpose(0, 2, 1))        # [b, pk, amn]
    out = storage.transpose(0, 2, 1)[:, :mn, :]                     # view: [b, mn, pk]
    return out[0] if squeeze else out


def element_strides(a: np.ndarray):
    return tuple(s // a.itemsize for s in a.strides)


def broadcast_block_sf(sf: np.ndarray, mn: int, gran_mn: int) -> np.ndarray:
    """Row-broadcast of [.., ceil(mn/gran_mn), k] scales to per-row [.., mn, k]."""
    idx = np.arange(mn) // gran_mn
    return np.take(sf, idx, axis=-2)


def psum_valid_rows(psum_layout, alignment: int, mn: int) -> np.ndarray:
    """Row mask of a PSUM layout: group g occupies [align(end[g-1], alignment), end[g])."""
    valid = np.zeros(mn, dtype=bool)
    prev = 0
    for end in psum_layout:
        start = align(prev, alignment)
        valid[start:end] = True
        prev = end
    return valid


def packed_ue8m0_mn_major_psum(sf: np.ndarray, psum_layout, alignment: int) -> np.ndarray:
    """Packed layout where rows in the gaps between groups come out as zero words."""
    valid = psum_valid_rows(psum_layout, alignment, sf.shape[0])
    clean = np.where(valid[:, None], sf, np.float32(0)).astype(np.float32)
    # zero float has exponent byte 0
    return packed_ue8m0_mn_major(clean)


def k_grouped_packed_ue8m0(sf: np.ndarray, ks, gran_k: int) -> np.ndarray:
    """K-grouped packing: sf [sum(k_g/gran_k), mn] -> int32 [sum(ceil(k_g/gran_k/4)), mn].

    Every group starts a fresh packed row and zero-fills the unused byte slots of
    its last row.
    """
    rows = []
    off = 0
    mn = sf.shape[1]
    for k in ks:
        n = k // gran_k
        if n == 0:
            continue
        g = sf[off: off + n]
        off += n
        pk = ceil_div(n, 4)
        by = np.zeros((pk * 4, mn), dtype=np.uint8)
        by[:n] = ue8m0_bytes(g)
        w = by.reshape(pk, 4, mn).transpose(0, 2, 1).copy().view(np.int32).reshape(pk, mn)
        rows.append(w)
    if not rows:
        return np.zeros((0, mn), dtype=np.int32)
    return np.concatenate(rows, axis=0)


# --------------------------------------------------------------------------- Mega MoE weight transforms
def interleave_gate_up(t: np.ndarray, gran: int = 8) -> np.ndarray:
    """[G, 2*I, ...] with gate rows then up rows -> blocks of `gran` gate rows, `gran` up rows, ...

    deep_gemm/mega/__init__.py:167-181.
    """
    g, n2 = t.shape[:2]
    rest = t.shape[2:]
    half = n2 // 2
    gate, up = t[:, :half], t[:, half:]
    gate = gate.reshape(g, half // gran, gran, *rest)
    up = up.reshape(g, half // gran, gran, *rest)
    return np.stack([gate, up], axis=2).reshape(g, n2, *rest)


def transpose_sf_for_utccp(sf: np.ndarray) -> np.ndarray:
    """Per 128 rows reorder row i -> (i%32)*4 + i//32.  deep_gemm/mega/__init__.py:184-198."""
    g, mn, pk = sf.shape
    assert mn % 128 == 0
    v = sf.reshape(g, mn // 128, 4, 32, pk).transpose(0, 1, 3, 2, 4)
    return np.ascontiguousarray(v).reshape(g, mn, pk)


def utccp_row_index(i: np.ndarray) -> np.ndarray:
    """Position of logical row i after transpose_sf_for_utccp (within its 128-row group)."""
    return (i & ~127) + (i & 31) * 4 + ((i >> 5) & 3)
