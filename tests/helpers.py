"""Shared input generators and oracle glue for the GPU parity tests.

Inputs follow the reference's generators (tests/generators.py:350-485): seeded BF16 normal
matrices, quantised per token (1 x gran_k) for activations and per 128 x 128 block (FP8) or
1 x 32 (FP4) for weights, power-of-two scales.  Expected values come from the numpy oracle
(oracle/), which dequantises exactly what the kernel is given.
"""
from __future__ import annotations

import numpy as np
import torch

from oracle import gemm as OG
from oracle import layout as OL
from oracle import quant as OQ

import deepgemm_b200 as dg
from deepgemm_b200.utils import math as M


def to_np(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu()
    if t.dtype == torch.float8_e4m3fn or t.dtype == torch.int8:
        return t.contiguous().view(torch.uint8).numpy()
    if t.dtype == torch.bfloat16:
        return t.float().numpy()
    return t.numpy()


def packed_sf_to_torch(view: np.ndarray, device="cuda") -> torch.Tensor:
    """Upload an oracle packed-SF strided view keeping its MN-major strides."""
    shape = view.shape
    # numpy may report anything for size-1 axes; rebuild the canonical MN-major strides
    amn = (shape[-2] + 3) // 4 * 4
    strides = (1, amn) if view.ndim == 2 else (shape[-1] * amn, 1, amn)
    n_store = sum((s - 1) * st for s, st in zip(shape, strides)) + 1
    # rebuild the storage in the same order
    storage = np.zeros(n_store, dtype=np.int32)
    np.lib.stride_tricks.as_strided(storage, shape=shape, strides=[s * 4 for s in strides])[...] = view
    t = torch.from_numpy(storage).to(device)
    return t.as_strided(shape, strides)


def quant_act(x: torch.Tensor, gran_k: int):
    """Per-token FP8 (activations): returns (e4m3 tensor, fp32 scales)."""
    return M.per_token_cast_to_fp8(x, use_ue8m0=True, gran_k=gran_k)


def quant_weight_fp8_block(w: torch.Tensor):
    return M.per_block_cast_to_fp8(w, use_ue8m0=True, gran_k=128)


def quant_weight_fp4(w: torch.Tensor):
    return M.per_token_cast_to_fp4(w, use_ue8m0=True, gran_k=32)


def dequant(data: torch.Tensor, sf: torch.Tensor, gran_mn: int, gran_k: int) -> np.ndarray:
    """Oracle dequantisation of one [.., mn, k] operand given exactly as the kernel gets it."""
    is_fp4 = data.dtype == torch.int8
    return OG.dequant_operand(to_np(data), to_np(sf), gran_mn, gran_k, is_fp4)


def calc_diff(x, y) -> float:
    return OQ.calc_diff(np.asarray(x, dtype=np.float64), np.asarray(y, dtype=np.float64))


def make_dense(m, n, k, *, gran_a=128, b_kind="fp8_block", seed=0, device="cuda", scale_b=1.0):
    """A per-token FP8; B 128x128-block FP8 ('fp8_block'), per-row FP8 ('fp8_row', gran from b_gran)
    or MXFP4 1x32 ('fp4')."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    a = torch.randn((m, k), generator=g, dtype=torch.float32).to(torch.bfloat16).to(device)
    b = (torch.randn((n, k), generator=g, dtype=torch.float32) * scale_b).to(torch.bfloat16).to(device)
    qa = quant_act(a, gran_a)
    if b_kind == "fp8_block":
        qb, gran_mn_b, gran_b = quant_weight_fp8_block(b), 128, 128
    elif b_kind == "fp8_row128":
        qb, gran_mn_b, gran_b = M.per_token_cast_to_fp8(b, True, 128), 1, 128
    elif b_kind == "fp8_row32":
        qb, gran_mn_b, gran_b = M.per_token_cast_to_fp8(b, True, 32), 1, 32
    elif b_kind == "fp4":
        qb, gran_mn_b, gran_b = quant_weight_fp4(b), 1, 32
    else:
        raise ValueError(b_kind)
    ref_a = dequant(qa[0], qa[1], 1, gran_a)
    ref_b = dequant(qb[0], qb[1], gran_mn_b, gran_b)
    return qa, qb, (gran_a, gran_mn_b, gran_b), ref_a, ref_b


def recipes(gran_a, gran_mn_b, gran_b):
    return dict(recipe_a=(1, gran_a), recipe_b=(gran_mn_b, gran_b))


class force_tile:
    """Context manager: pin the tile the library picks (tests only)."""

    def __init__(self, **kw):
        self.kw = kw

    def __enter__(self):
        from deepgemm_b200 import _lib
        kw = self.kw
        _lib.check(_lib.lib().dg_debug_set_tile_override(kw.get("cta_group") or 0, kw.get("block_n") or 0,
                                                         kw.get("swap") or 0))

    def __exit__(self, *exc):
        from deepgemm_b200 import _lib
        _lib.check(_lib.lib().dg_debug_set_tile_override(0, 0, 0))


# --------------------------------------------------------------------------- grouped generators
def align_up(x, a):
    return (x + a - 1) // a * a


def make_m_grouped_contiguous(num_groups, expected_m, n, k, *, alignment=128, use_psum=False, b_kind="fp8_block",
                              gran_a=128, seed=0, device="cuda", scale_b=1.0):
    """tests/generators.py:378-419 of the reference: ragged groups padded to `alignment` rows,
    padding rows zero, layout either per-row expert ids (-1 = padding) or cumulative row ends."""
    import random
    rnd = random.Random(seed)
    g = torch.Generator(device="cpu").manual_seed(seed)
    actual = [int(expected_m * rnd.uniform(0.7, 1.3)) for _ in range(num_groups)]
    aligned = [align_up(x, alignment) for x in actual]
    m = sum(aligned)
    a = torch.randn((m, k), generator=g).to(torch.bfloat16)
    b = (torch.randn((num_groups, n, k), generator=g) * scale_b).to(torch.bfloat16)
    layout = torch.empty(num_groups if use_psum else m, dtype=torch.int32)
    valid = torch.zeros(m, dtype=torch.bool)
    start = 0
    for i, (am, al) in enumerate(zip(actual, aligned)):
        if use_psum:
            layout[i] = start + am
        else:
            layout[start:start + am] = i
            layout[start + am:start + al] = -1
        valid[start:start + am] = True
        a[start + am:start + al] = 0
        start += al
    a, b = a.to(device), b.to(device)
    qa = quant_act(a, gran_a)
    if b_kind == "fp8_block":
        qb_list = [quant_weight_fp8_block(b[i]) for i in range(num_groups)]
        gran_mn_b, gran_b = 128, 128
    else:
        qb_list = [quant_weight_fp4(b[i]) for i in range(num_groups)]
        gran_mn_b, gran_b = 1, 32
    qb = (torch.stack([q[0] for q in qb_list]), torch.stack([q[1] for q in qb_list]))
    ref_a = dequant(qa[0], qa[1], 1, gran_a)
    ref_b = np.stack([dequant(qb_list[i][0], qb_list[i][1], gran_mn_b, gran_b) for i in range(num_groups)])
    return dict(m=m, a=qa, b=qb, layout=layout.to(device), valid=valid.numpy(), actual=actual, aligned=aligned,
                grans=(gran_a, gran_mn_b, gran_b), ref_a=ref_a, ref_b=ref_b)


def ref_m_grouped(case) -> np.ndarray:
    """Oracle output on the valid rows' groups (padding rows stay zero)."""
    ids = np.full(case["m"], -1, dtype=np.int64)
    start = 0
    for i, (am, al) in enumerate(zip(case["actual"], case["aligned"])):
        ids[start:start + am] = i
        start += al
    return OG.m_grouped_contiguous(case["ref_a"], case["ref_b"], ids)


def make_masked(num_groups, max_m, expected_m, n, k, *, b_kind="fp8_block", gran_a=128, seed=0, device="cuda",
                scale_b=1.0):
    """tests/generators.py:446-485 of the reference."""
    import random
    rnd = random.Random(seed)
    g = torch.Generator(device="cpu").manual_seed(seed)
    a = torch.randn((num_groups, max_m, k), generator=g).to(torch.bfloat16).to(device)
    b = (torch.randn((num_groups, n, k), generator=g) * scale_b).to(torch.bfloat16).to(device)
    masked = torch.tensor([min(max_m, int(expected_m * rnd.uniform(0.5, 1.5))) for _ in range(num_groups)],
                          dtype=torch.int32)
    qa_list = [quant_act(a[i], gran_a) for i in range(num_groups)]
    qa = (torch.stack([q[0] for q in qa_list]), torch.stack([q[1] for q in qa_list]))
    for i in range(num_groups):
        qa[1][i, int(masked[i]):] = 0          # scale rows beyond the valid count are zero
    if b_kind == "fp8_block":
        qb_list = [quant_weight_fp8_block(b[i]) for i in range(num_groups)]
        gran_mn_b, gran_b = 128, 128
    else:
        qb_list = [quant_weight_fp4(b[i]) for i in range(num_groups)]
        gran_mn_b, gran_b = 1, 32
    qb = (torch.stack([q[0] for q in qb_list]), torch.stack([q[1] for q in qb_list]))
    ref_a = np.stack([dequant(qa_list[i][0], qa_list[i][1], 1, gran_a) for i in range(num_groups)])
    ref_b = np.stack([dequant(qb_list[i][0], qb_list[i][1], gran_mn_b, gran_b) for i in range(num_groups)])
    return dict(a=qa, b=qb, masked=masked.to(device), masked_cpu=masked.numpy(), grans=(gran_a, gran_mn_b, gran_b),
                ref_a=ref_a, ref_b=ref_b)


def make_k_grouped(num_groups, m, n, ks, *, gran_k=128, seed=0, device="cuda"):
    """tests/generators.py:527-608 of the reference (non-psum): A [sum_k, m], B [sum_k, n], per-channel scales."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    total = sum(ks)
    a = torch.randn((total, m), generator=g).to(torch.bfloat16).to(device)
    b = torch.randn((total, n), generator=g).to(torch.bfloat16).to(device)
    qa_d, qa_s, qb_d, qb_s = [], [], [], []
    off = 0
    for kk in ks:
        if kk == 0:
            continue
        da, sa = M.per_channel_cast_to_fp8(a[off:off + kk], True, gran_k)
        db, sb = M.per_channel_cast_to_fp8(b[off:off + kk], True, gran_k)
        qa_d.append(da), qa_s.append(sa), qb_d.append(db), qb_s.append(sb)
        off += kk
    qa = (torch.cat(qa_d), torch.cat(qa_s))
    qb = (torch.cat(qb_d), torch.cat(qb_s))

    def deq(d, s):
        # per-channel: scale row r covers K rows [r*gran_k, (r+1)*gran_k)
        dn = OQ.e4m3_bits_to_f32(to_np(d))
        sn = to_np(s)
        return dn * np.repeat(sn, gran_k, axis=0)

    bounds, off = [], 0
    for kk in ks:
        bounds.append((off, off + kk))
        off += kk
    return dict(a=qa, b=qb, ref_a=deq(*qa), ref_b=deq(*qb), bounds=bounds)


def make_k_grouped_psum(m, n, real_ks, k_alignment, *, gran_k=128, seed=0, device="cuda"):
    """tests/generators.py:540-608 of the reference with use_psum_layout: group g owns the K rows
    [align(end[g-1], k_alignment), end[g]); the rows up to the next boundary are zero; every group is quantised over
    its aligned extent, so its scale rows cover align(k_g, k_alignment) / gran_k rows.  Returns the quantised operands,
    the cumulative ends, the aligned sizes and dequantised copies with the groups' real K ranges."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    aligned = [align_up(k, k_alignment) for k in real_ks]
    ends, prev = [], 0
    for k in real_ks:
        prev = align_up(prev, k_alignment) + k
        ends.append(prev)
    total = sum(aligned)
    a = torch.zeros((total, m), dtype=torch.bfloat16)
    b = torch.zeros((total, n), dtype=torch.bfloat16)
    bounds = []
    for k, end in zip(real_ks, ends):
        a[end - k:end] = torch.randn((k, m), generator=g).to(torch.bfloat16)
        b[end - k:end] = torch.randn((k, n), generator=g).to(torch.bfloat16)
        bounds.append((end - k, end))
    a, b = a.to(device), b.to(device)

    def cast(x):
        data = torch.zeros(x.shape, dtype=torch.float8_e4m3fn, device=device)
        sfs = []
        for (k0, k1), al in zip(bounds, aligned):
            if al == 0:
                continue
            q, sf = M.per_channel_cast_to_fp8(x[k0:k0 + al], True, gran_k)    # rows past k1 are the zero padding
            data[k0:k0 + al] = q
            sfs.append(sf)
        return data, torch.cat(sfs)

    qa, qb = cast(a), cast(b)

    def deq(d, s):
        return OQ.e4m3_bits_to_f32(to_np(d)) * np.repeat(to_np(s), gran_k, axis=0)

    return dict(a=qa, b=qb, ref_a=deq(*qa), ref_b=deq(*qb), bounds=bounds, ends=ends, aligned=aligned)
