"""CPU oracle: Mega MoE forward for one rank's tokens.

TEST INFRASTRUCTURE ONLY (see oracle/quant.py).  Restates the reference's torch formulation
`_mega_moe_reference` (tests/test_mega_moe.py:466-480) with its numeric boundaries (:443-450): exact
dequantisation, float GEMMs, BF16 rounding of the first GEMM's output, optional clamp,
gate * sigmoid(gate) * up, times the route weight, per-32 UE8M0 E4M3 requantisation, BF16 rounding of the
second GEMM's output per (token, expert), float32 sum over the slots in slot order, BF16.
"""
from __future__ import annotations

import numpy as np

from .quant import bf16_round, cast_back_from_fp8, per_token_cast_to_fp8


def swiglu(gate: np.ndarray, up: np.ndarray, clamp=None) -> np.ndarray:
    if clamp is not None:
        gate = np.minimum(gate, np.float32(clamp))
        up = np.clip(up, -np.float32(clamp), np.float32(clamp))
    g = gate.astype(np.float32)
    return (g / (np.float32(1) + np.exp(-g, dtype=np.float32))) * up.astype(np.float32)


def mega_moe_reference(x_deq, topk_idx, topk_weights, l1_deq, l2_deq, clamp=None):
    """x_deq [T, H]; topk_idx [T, K] (entries < 0 are skipped); l1_deq [E, 2I, H] (gate rows then up rows);
    l2_deq [E, H, I].  Returns BF16-valued float32 [T, H] and the per-expert row counts."""
    t, h = x_deq.shape
    inter = l2_deq.shape[2]
    k = topk_idx.shape[1]
    per_slot = np.zeros((k, t, h), dtype=np.float32)
    counts = np.zeros(l1_deq.shape[0], dtype=np.int64)
    for e in range(l1_deq.shape[0]):
        rows, slots = np.nonzero(topk_idx == e)
        counts[e] = rows.size
        if rows.size == 0:
            continue
        l1 = bf16_round((x_deq[rows].astype(np.float64) @ l1_deq[e].astype(np.float64).T).astype(np.float32))
        act = swiglu(l1[:, :inter], l1[:, inter:], clamp) * topk_weights[rows, slots][:, None].astype(np.float32)
        q, sf = per_token_cast_to_fp8(act.astype(np.float32), True, 32)
        l2 = bf16_round((cast_back_from_fp8(q, sf, 32).astype(np.float64) @ l2_deq[e].astype(np.float64).T).astype(np.float32))
        per_slot[slots, rows] = l2
    y = np.zeros((t, h), dtype=np.float32)
    for s in range(k):                     # float32 accumulation in slot order
        y += per_slot[s]
    return bf16_round(y), counts
