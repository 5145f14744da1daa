"""Batched FP8 GEMM behind the reference's `fp8_einsum` (csrc/apis/einsum.hpp:182-304).

Three expressions, each mapped onto `[B, M, K] @ [B, N, K]^T` by permuting views (no data moves):

    "bhr,hdr->bhd"   (batch, m, n, k) = (h, b, d, r)   K-major operands; D may be an FP8 (d, sfd) pair
    "bhd,hdr->bhr"   (batch, m, n, k) = (h, b, r, d)   the weight is read MN-major
    "bhd,bhr->hdr"   (batch, m, n, k) = (h, d, r, b)   both operands MN-major, per-channel scales, recipe (1, 1, 128)

The batches become the group axis of the block-scaled GEMM kernel (a batch owns a full m x n tile grid); operands and D
carry their own batch strides, so permuted views are passed as they are.
"""
from __future__ import annotations

from typing import Optional, Tuple, Union

import torch

from . import _lib
from .layout import _require, check_sf_layout, transform_sf_pair_into_required_layout
from .ops import (_K, _MN, Alpha, BF16StochasticRounding, FP8CastWithClamp, Identity, _early_return, _launch)

Pair = Tuple[torch.Tensor, torch.Tensor]


def _bmm_major(t: torch.Tensor) -> int:
    _require(t.stride(-1) == 1 or t.stride(-2) == 1, "a.stride(-1) == 1 or a.stride(-2) == 1")
    return _K if t.stride(-1) == 1 else _MN


def fp8_bmm(a: torch.Tensor, sfa: torch.Tensor, b: torch.Tensor, sfb: torch.Tensor,
            d: Union[torch.Tensor, Pair], c: Optional[torch.Tensor], recipe, compiled_dims: str = "nk",
            epilogue=None) -> None:
    """D[i] = A[i] @ B[i]^T (+ C[i]) for every batch i; a [B, M, K], b [B, N, K], d [B, M, N], any of them a strided
    view whose innermost or second-innermost stride is 1 (csrc/apis/einsum.hpp:182-249)."""
    sfd = None
    if isinstance(d, tuple):
        # the FP8 output pair is shorthand for FP8CastWithClamp without clamping
        _require(epilogue is None, "epilogue_class == nullptr and \"The FP8 output pair supports no other epilogue\"")
        d, sfd = d
        epilogue = FP8CastWithClamp(sfd)
    elif isinstance(epilogue, FP8CastWithClamp):
        sfd = epilogue.sfd
    major_a, major_b = _bmm_major(a), _bmm_major(b)
    _require(d.stride(-1) == 1, "d_tensor.stride(-1) == 1")
    _require(a.dim() == 3 and b.dim() == 3 and d.dim() == 3, "t.dim() == N")
    batch, m, k = a.shape
    batch_, n, k_ = b.shape
    batch__, m_, n_ = d.shape
    _require(batch == batch_ and batch == batch__, "batch_size == batch_size_ and batch_size == batch_size__")
    _require(m == m_ and n == n_ and k == k_, "m == m_ and n == n_ and k == k_")
    _require(a.dtype == torch.float8_e4m3fn and b.dtype == torch.float8_e4m3fn,
             "a.scalar_type() == torch::kFloat8_e4m3fn and b.scalar_type() == torch::kFloat8_e4m3fn")
    if sfd is not None:
        # the scales match a per-token cast of D seen as [m, batch * n]: the batches must be adjacent along the
        # columns of that view, and neither a 32-column group nor a packed word may straddle two batches
        _require(d.stride(0) == n and n % 128 == 0, "d_tensor.stride(0) == n and n % 128 == 0")
        check_sf_layout(sfd, m, batch * n, 1, 32, None, tma_stride_check=True, type_check=torch.int32)
    if epilogue is not None and not isinstance(epilogue, (Identity, Alpha)):
        epilogue.check(c, d)
    else:
        _require(d.dtype in (torch.bfloat16, torch.float32), "d.scalar_type() == torch::kBFloat16 or d.scalar_type() == torch::kFloat")
    if batch == 0:
        return
    if (m == 0 or n == 0 or k == 0) and sfd is not None:
        sfd.zero_()          # an empty problem zeroes the scales it would have produced
    if _early_return(m, n, k, d, c, allow_fp8=sfd is not None):
        return
    ta, tb, gran_a, gran_b = transform_sf_pair_into_required_layout(sfa, sfb, m, n, k, recipe, None, None, batch, batch)
    alpha = epilogue.alpha if isinstance(epilogue, Alpha) else 1.0
    _launch(_lib.GEMM_BATCHED, m, n, k, a, ta, major_a, gran_a, b, tb, major_b, gran_b, d, num_groups=batch,
            accumulate=c is not None, alpha=alpha, epilogue=epilogue, batched=True)


def fp8_einsum(expr: str, a: Pair, b: Pair, d: Union[torch.Tensor, Pair], c: Optional[torch.Tensor] = None,
               recipe: Tuple[int, int, int] = (1, 128, 128), epilogue=None) -> None:
    """The reference's hard-coded Einstein sums over quantised operands (csrc/apis/einsum.hpp:251-297).  Only
    "bhr,hdr->bhd" takes an FP8 (d, sfd) output pair."""
    def perm(t, order):
        return None if t is None else t.permute(*order)

    if expr == "bhr,hdr->bhd":
        # the FP8 output scales are flattened over D's last two dims, so they are unchanged by the (b, h) permutation
        d_perm = (perm(d[0], (1, 0, 2)), d[1]) if isinstance(d, tuple) else perm(d, (1, 0, 2))
        fp8_bmm(perm(a[0], (1, 0, 2)), perm(a[1], (1, 0, 2)), b[0], b[1], d_perm, perm(c, (1, 0, 2)), recipe, "nk", epilogue)
    elif expr == "bhd,hdr->bhr":
        _require(not isinstance(d, tuple), "std::holds_alternative<torch::Tensor>(d)")
        fp8_bmm(perm(a[0], (1, 0, 2)), perm(a[1], (1, 0, 2)), perm(b[0], (0, 2, 1)), perm(b[1], (0, 2, 1)),
                perm(d, (1, 0, 2)), perm(c, (1, 0, 2)), recipe, "nk", epilogue)
    elif expr == "bhd,bhr->hdr":
        _require(not isinstance(d, tuple), "std::holds_alternative<torch::Tensor>(d)")
        fp8_bmm(perm(a[0], (1, 2, 0)), perm(a[1], (1, 2, 0)), perm(b[0], (1, 2, 0)), perm(b[1], (1, 2, 0)), d, c, recipe,
                "mn", epilogue)
    else:
        raise RuntimeError(f"Unsupported einsum expression: {expr}")
