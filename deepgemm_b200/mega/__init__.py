"""Mega MoE forward behind the reference's `deep_gemm.mega` names.

SymmBuffer / get_symm_buffer_for_mega_moe / transform_weights_for_mega_moe / fp8_fp4_mega_moe keep the
signatures of deep_gemm/mega/__init__.py:32-348.  The buffer's byte layout is this library's own
(dg_mega_moe_buffer_layout); the views the caller fills (x, x_sf, topk_idx, topk_weights) have the
reference's shapes and dtypes.  NCCL is used only by torch's symmetric-memory rendezvous; all data
movement happens in the library's kernels through peer loads / stores.
"""
from __future__ import annotations

import ctypes as C
import enum
import math
import types
from typing import Optional, Tuple

import torch

from .. import _lib
from ..layout import _require, _stream
from ..utils.math import align


def set_fused(enable: bool) -> None:
    """Run the forward as one persistent kernel (default) or as one kernel per phase; same results."""
    _lib.check(_lib.lib().dg_set_mega_moe_fused(int(bool(enable))))


def get_token_alignment_for_mega_moe() -> int:
    return int(_lib.lib().dg_get_token_alignment_for_mega_moe())


def get_block_m_for_mega_moe(num_ranks: int, num_experts: int, num_max_tokens_per_rank: int, num_tokens: int,
                             num_topk: int, mma_type: str = "fp8xfp4") -> int:
    """Token rows per expert tile; tiles shrink at run time for short experts (csrc/apis/mega_moe.hpp:38-47)."""
    return int(_lib.lib().dg_get_block_m_for_mega_moe())


_ACTIVATIONS = {"swiglu": 0, "geglu": 1, "situ": 2}


class RouteWeightMode(enum.Enum):
    """Where the route weight enters (deep_gemm/mega/__init__.py RouteWeightMode): before the second GEMM's input is
    quantised, or on the second GEMM's BF16 output at the combine write."""
    PRE_DOWN = "pre_down"
    POST_DOWN = "post_down"


class SymmBuffer:
    """One symmetric buffer per rank plus the views user code fills (deep_gemm/mega/__init__.py:32-134)."""

    def __init__(self, group, num_experts: int, num_max_tokens_per_rank: int, num_topk: int, hidden: int,
                 intermediate_hidden: int, num_ring_tokens: Optional[int] = None, mma_type: str = "fp8xfp4",
                 activation: str = "swiglu", base: Optional["SymmBuffer"] = None, num_shared_experts: int = 0,
                 side_lora: bool = False):
        if mma_type not in ("fp8xfp4", "fp8xfp8") or side_lora:
            raise NotImplementedError("the forward with FP8 activations and MXFP4 or FP8 expert weights (with or without "
                                      "shared experts) is what this build holds; BF16 and side-LoRA variants are not")
        _require(num_shared_experts >= 0, "num_shared_experts >= 0")
        if activation not in _ACTIVATIONS:
            raise NotImplementedError(f"activation `{activation}` is not part of this build")
        num_max_tokens_per_rank = align(num_max_tokens_per_rank, get_token_alignment_for_mega_moe())
        self.group = group
        self.num_ranks = 1 if group is None else group.size()
        self.rank = 0 if group is None else group.rank()
        self.num_experts, self.num_max_tokens_per_rank, self.num_topk = num_experts, num_max_tokens_per_rank, num_topk
        self.hidden, self.intermediate_hidden = hidden, intermediate_hidden
        self.num_shared_experts, self.mma_type, self.activation = int(num_shared_experts), mma_type, activation
        # `num_ring_tokens` bounds the rows of the expert-sorted pool (None / 0: the worst case, every token of every
        # rank routed here); a call that receives more is abandoned and reported by check_status()
        _require(num_ring_tokens is None or num_ring_tokens >= 0, "num_ring_tokens >= 0")
        self.config = _lib.MoeConfig(self.num_ranks, num_experts, num_max_tokens_per_rank, num_topk, hidden,
                                     intermediate_hidden, int(num_ring_tokens or 0), int(num_shared_experts))
        lay = _lib.MoeLayout()
        _lib.check(_lib.lib().dg_mega_moe_buffer_layout(C.byref(self.config), C.byref(lay)))
        self.layout = lay
        device = torch.device("cuda", torch.cuda.current_device())
        if base is None:
            if self.num_ranks == 1:
                self.buffer = torch.empty(lay.num_bytes, dtype=torch.int8, device=device)
                self.handle = types.SimpleNamespace(buffer_ptrs=[self.buffer.data_ptr()])
            else:
                import torch.distributed._symmetric_memory as symm_mem
                self.buffer = symm_mem.empty(lay.num_bytes, dtype=torch.int8, device=device)
                self.handle = symm_mem.rendezvous(self.buffer, group=group)
            self.buffer.zero_()
            if group is not None:
                group.barrier()
            torch.cuda.synchronize()
        else:
            # Another configuration on the memory of `base` (deep_gemm/mega/__init__.py:80-92).  Legal between calls:
            # the words that live across calls (barrier epochs, grid barrier, send counters) sit in a control block
            # whose place does not depend on the configuration, everything else is rewritten by each call.
            _require(base.buffer is not None and base.group is group, "cannot reuse an invalid symmetric buffer")
            _require(lay.num_bytes <= base.buffer.nbytes, "the reused buffer is too small for this configuration")
            self.buffer, self.handle = base.buffer, base.handle

        def view(off, dtype, shape, strides=None):
            n = math.prod(shape) * torch.empty((), dtype=dtype).element_size()
            flat = self.buffer[off:off + n].view(dtype)
            return flat.view(shape) if strides is None else flat.as_strided(shape, strides)

        t, k, h, i, p, q = num_max_tokens_per_rank, num_topk, hidden, intermediate_hidden, lay.pool_rows, lay.sf_rows
        self.x = view(lay.off_x, torch.float8_e4m3fn, (t, h))
        self.x_sf = view(lay.off_x_sf, torch.int32, (t, h // 128))
        self.topk_idx = view(lay.off_topk_idx, torch.int64, (t, k))
        self.topk_weights = view(lay.off_topk_weights, torch.float32, (t, k))
        self.l1_acts = view(lay.off_l1_acts, torch.float8_e4m3fn, (p, h))
        self.l1_acts_sf = view(lay.off_l1_acts_sf, torch.int32, (q, h // 128), (1, q))
        self.l2_acts = view(lay.off_l2_acts, torch.float8_e4m3fn, (p, i))
        self.l2_acts_sf = view(lay.off_l2_acts_sf, torch.int32, (q, i // 128), (1, q))
        self.token_src_metadata = view(lay.off_token_src_metadata, torch.int32, (p, 3))
        self.combine = view(lay.off_combine, torch.bfloat16, (k + (1 if num_shared_experts else 0), t, h))
        # Shared experts (deep_gemm/mega/__init__.py:107-123): their first GEMM reads x itself; its scales are needed
        # once more, MN-major and in the row order tcgen05.cp consumes (row i of every 128 at (i % 32) * 4 + i // 32)
        self.shared_l1_acts = self.shared_l1_acts_sf = self.shared_l2_acts = self.shared_l2_acts_sf = None
        if num_shared_experts:
            ta, i_s = align(t, 128), i * num_shared_experts
            self.shared_l1_acts = self.x
            self.shared_l1_acts_sf = view(lay.off_shared_l1_acts_sf, torch.int32, (ta, h // 128), (1, ta))
            self.shared_l2_acts = view(lay.off_shared_l2_acts, torch.float8_e4m3fn, (ta, i_s))
            self.shared_l2_acts_sf = view(lay.off_shared_l2_acts_sf, torch.int32, (ta, i_s // 128), (1, ta))
        self.num_ring_tokens = p
        self.num_sf_ring_tokens = q

    def load_tokens(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_weights: torch.Tensor) -> int:
        """Fill the input views from BF16 activations: one fused kernel casts x to E4M3 with per-32 UE8M0 scales
        straight into `self.x` / `self.x_sf` (the recipe the forward consumes), the routing tensors are copied.
        Returns the number of tokens, i.e. the row count to give `y`."""
        from ..cast import per_token_cast_to_fp8_fused
        n = x.size(0)
        _require(n <= self.num_max_tokens_per_rank and x.size(1) == self.hidden, "x fits the buffer")
        _require(tuple(topk_idx.shape) == (n, self.num_topk) and tuple(topk_weights.shape) == (n, self.num_topk),
                 "topk_idx / topk_weights are [num_tokens, num_topk]")
        per_token_cast_to_fp8_fused(x, 32, "packed", out=self.x[:n], sf_out=self.x_sf[:n])
        if self.num_shared_experts:
            self.fill_shared_scales(n)
        self.topk_idx[:n].copy_(topk_idx)
        self.topk_weights[:n].copy_(topk_weights)
        return n

    def fill_shared_scales(self, num_tokens: int) -> None:
        """Copy the first `num_tokens` rows of x_sf into shared_l1_acts_sf (the layout the shared experts' first GEMM
        reads: MN-major, rows of every 128 in tcgen05.cp order).  Call after writing x_sf by hand; load_tokens does it."""
        i = torch.arange(num_tokens, device=self.x_sf.device)
        dst = (i // 128) * 128 + (i % 32) * 4 + (i % 128) // 32
        self.shared_l1_acts_sf[dst] = self.x_sf[:num_tokens]

    def reset(self) -> None:
        """Make the buffer usable again after a call that gave up on a wait (check_status() raised): such a call
        leaves barrier arrivals and epochs behind that the next call would trip over.  Every rank of the group must
        call this, with no forward in flight on any of them: the ranks meet, each clears its whole buffer (control
        block included), and they meet again.  The inputs (x, x_sf, topk_idx, topk_weights) must be refilled."""
        torch.cuda.synchronize()
        if self.group is not None:
            self.group.barrier()
        self.buffer.zero_()
        torch.cuda.synchronize()
        if self.group is not None:
            self.group.barrier()
        try:
            _lib.check_status()      # drop a stale record of the abandoned wait
        except RuntimeError:
            pass

    def destroy(self):
        self.handle = self.buffer = self.group = None
        self.x = self.x_sf = self.topk_idx = self.topk_weights = None
        self.l1_acts = self.l1_acts_sf = self.l2_acts = self.l2_acts_sf = self.token_src_metadata = self.combine = None
        self.shared_l1_acts = self.shared_l1_acts_sf = self.shared_l2_acts = self.shared_l2_acts_sf = None


def get_symm_buffer_for_mega_moe(group, num_experts: int, num_max_tokens_per_rank: int, num_topk: int, hidden: int,
                                 intermediate_hidden: int, use_fp8_dispatch: Optional[bool] = None,
                                 mma_type: str = "fp8xfp4", activation: str = "swiglu",
                                 num_ring_tokens: Optional[int] = None, num_shared_experts: int = 0,
                                 side_lora: bool = False) -> SymmBuffer:
    """deep_gemm/mega/__init__.py:138-164."""
    if use_fp8_dispatch is not None:
        assert use_fp8_dispatch == (mma_type.split("x")[0] == "fp8")
    return SymmBuffer(group, num_experts, num_max_tokens_per_rank, num_topk, hidden, intermediate_hidden,
                      num_ring_tokens, mma_type=mma_type, activation=activation,
                      num_shared_experts=num_shared_experts, side_lora=side_lora)


def _permute_rows(t: torch.Tensor, perm: torch.Tensor) -> torch.Tensor:
    """Row permutation of a [G, rows, ...] tensor that keeps the input's strides (packed scales are MN-major)."""
    out = torch.empty_like(t)
    out.copy_(t.index_select(1, perm))
    return out


def transform_weights_for_mega_moe(l1_weights, l2_weights, activation: str = "swiglu"):
    """Weight layout the fused kernels read (deep_gemm/mega/__init__.py:167-220): W13 rows (data and scales) as
    alternating blocks of 8 gate rows and 8 up rows; both scale tensors with every 128 rows reordered so that row
    i sits at (i % 32) * 4 + i // 32, the order tcgen05.cp copies into TMEM.  Pure permutations."""
    assert activation in ("swiglu", "geglu", "situ"), f"Unsupported activation: `{activation}`"
    _require(isinstance(l1_weights, tuple) and isinstance(l2_weights, tuple), "FP8 x FP4 weights are (data, sf) pairs")
    (w1, sf1), (w2, sf2) = l1_weights, l2_weights
    if w1.dim() == 2:
        # one expert without a group axis (the shared experts' weights): same permutations
        (t1, ts1), (t2, ts2) = transform_weights_for_mega_moe((w1.unsqueeze(0), sf1.unsqueeze(0)),
                                                              (w2.unsqueeze(0), sf2.unsqueeze(0)), activation)
        return (t1.squeeze(0), ts1.squeeze(0)), (t2.squeeze(0), ts2.squeeze(0))
    dev = w1.device
    n1 = w1.size(1)
    half = n1 // 2
    r = torch.arange(n1, device=dev)
    blk, within = r // 16, r % 16
    interleave = torch.where(within < 8, blk * 8 + within, half + blk * 8 + (within - 8))

    def utccp_perm(rows):
        i = torch.arange(rows, device=dev)
        dst = (i // 128) * 128 + (i % 32) * 4 + (i % 128) // 32
        src = torch.empty_like(i)
        src[dst] = i
        return src

    _require(n1 % 128 == 0 and w2.size(1) % 128 == 0, "mn % 128 == 0")
    l1 = (_permute_rows(w1, interleave), _permute_rows(_permute_rows(sf1, interleave), utccp_perm(n1)))
    l2 = (w2, _permute_rows(sf2, utccp_perm(w2.size(1))))
    return l1, l2


def fp8_fp4_mega_moe(y: torch.Tensor, l1_weights: Tuple[torch.Tensor, torch.Tensor],
                     l2_weights: Tuple[torch.Tensor, torch.Tensor], sym_buffer: SymmBuffer,
                     cumulative_local_expert_recv_stats: Optional[torch.Tensor] = None,
                     recipe: Tuple[int, int, int] = (1, 1, 32), activation: str = "swiglu",
                     activation_clamp: Optional[float] = None, fast_math: bool = True, *,
                     situ_beta: Optional[float] = None, situ_linear_beta: Optional[float] = None,
                     shared_l1_weights: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
                     shared_l2_weights: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
                     **unsupported) -> None:
    """Fused expert-parallel MoE forward into y [num_tokens, hidden] (deep_gemm/mega/__init__.py:273-348).

    The caller has filled sym_buffer.x / x_sf / topk_idx / topk_weights for its num_tokens = y.size(0) tokens;
    every rank of the group calls this.  No host synchronisation, no collective.
    """
    for name, val in unsupported.items():
        # saved_* tensors belong to the training path (activations kept for the backward pass), which is not built
        if val is not None and name not in ("route_weight_mode", "num_config_tokens"):
            raise NotImplementedError(f"`{name}` is not part of this build")
    mode = unsupported.get("route_weight_mode", "pre_down")
    mode = (mode.value if isinstance(mode, RouteWeightMode) else str(mode).split(".")[-1]).lower()
    _require(mode in ("pre_down", "post_down"), "route_weight_mode in ('pre_down', 'post_down')")
    _require(tuple(recipe) == (1, 1, 32), "recipe == (1, 1, 32)")
    _require(activation in _ACTIVATIONS, "activation in ('swiglu', 'geglu', 'situ')")
    b = sym_buffer
    (w1, sf1), (w2, sf2) = l1_weights, l2_weights
    el, h, i = b.num_experts // b.num_ranks, b.hidden, b.intermediate_hidden
    _require(y.dim() == 2 and y.size(1) == h and y.dtype == torch.bfloat16 and y.stride(1) == 1, "y is [num_tokens, hidden] bf16")
    _require(y.size(0) <= b.num_max_tokens_per_rank, "num_tokens <= num_max_tokens_per_rank")
    # MXFP4 weights (int8, two codes per byte) or E4M3 weights (the reference's "fp8xfp8", csrc/apis/mega_moe.hpp:374-377)
    _require(w1.dtype in (torch.int8, torch.float8_e4m3fn) and w2.dtype == w1.dtype,
             "weight_dtype == torch::kFloat8_e4m3fn or weight_dtype == kPackedFP4")
    wdiv = 2 if w1.dtype == torch.int8 else 1
    _require(tuple(w1.shape) == (el, 2 * i, h // wdiv) and w1.is_contiguous(), "l1 weights [E_local, 2I, H] (E4M3) or [E_local, 2I, H/2] (packed FP4)")
    _require(tuple(w2.shape) == (el, h, i // wdiv) and w2.is_contiguous(), "l2 weights [E_local, H, I] (E4M3) or [E_local, H, I/2] (packed FP4)")
    for sf, mn, k in ((sf1, 2 * i, h), (sf2, h, i)):
        _require(sf.dtype == torch.int32 and tuple(sf.shape) == (el, mn, k // 128), "packed weight scales [E_local, mn, k/128] int32")
        _require(sf.stride(-2) == 1 and sf.stride(-1) % 4 == 0 and sf.stride(-1) >= mn and
                 sf.stride(0) == sf.stride(-1) * sf.size(-1), "weight scales are MN-major and TMA-aligned")
    stats = cumulative_local_expert_recv_stats
    if stats is not None:
        _require(stats.dtype == torch.int32 and stats.numel() == el and stats.is_contiguous(), "stats int32 [E_local]")
    args = _lib.MoeArgs()
    args.cfg = b.config
    ptrs = (C.c_void_p * b.num_ranks)(*[int(p) for p in b.handle.buffer_ptrs])
    args.buffer_ptrs = C.cast(ptrs, C.POINTER(C.c_void_p))
    args.rank, args.num_tokens = b.rank, y.size(0)
    args.y, args.ldy = y.data_ptr(), y.stride(0)
    args.l1_w, args.l1_sf, args.l2_w, args.l2_sf = w1.data_ptr(), sf1.data_ptr(), w2.data_ptr(), sf2.data_ptr()
    args.l1_sf_ld, args.l2_sf_ld = sf1.stride(-1), sf2.stride(-1)
    args.stats = stats.data_ptr() if stats is not None else None
    args.activation_clamp = float("inf") if activation_clamp is None else float(activation_clamp)
    args.fast_math = int(bool(fast_math))
    # SiTU parameters are ignored by the other activations (tests/test_mega_moe.py:551-559 of the reference)
    args.activation = _ACTIVATIONS[activation]
    args.post_down = int(mode == "post_down")
    args.weights_fp8 = int(w1.dtype == torch.float8_e4m3fn)
    _require((shared_l1_weights is None) == (shared_l2_weights is None),
             "shared_l1_weights_tuple_opt.has_value() == shared_l2_weights_tuple_opt.has_value()")
    _require((shared_l1_weights is not None) == (b.num_shared_experts > 0),
             "shared expert weights are given exactly when the buffer was sized for shared experts")
    if shared_l1_weights is not None:
        (sw1, ssf1), (sw2, ssf2) = shared_l1_weights, shared_l2_weights
        i_s = i * b.num_shared_experts
        _require(mode == "pre_down", "route_weight_mode == \"pre_down\"")
        _require(sw1.dtype == torch.float8_e4m3fn and sw2.dtype == torch.float8_e4m3fn,
                 "shared_l1_weights.scalar_type() == torch::kFloat8_e4m3fn")
        _require(tuple(sw1.shape) == (2 * i_s, h) and tuple(sw2.shape) == (h, i_s) and sw1.is_contiguous() and sw2.is_contiguous(),
                 "shared_l1_n == shared_intermediate_hidden * 2 and shared_l1_k == hidden and shared_l2_n == hidden")
        for sf, mn, k in ((ssf1, 2 * i_s, h), (ssf2, h, i_s)):
            _require(sf.dtype == torch.int32 and tuple(sf.shape) == (mn, k // 128) and sf.stride(0) == 1 and
                     sf.stride(1) % 4 == 0 and sf.stride(1) >= mn, "shared weight scales are packed, MN-major and TMA-aligned")
        args.shared_l1_w, args.shared_l1_sf, args.shared_l2_w, args.shared_l2_sf = (
            sw1.data_ptr(), ssf1.data_ptr(), sw2.data_ptr(), ssf2.data_ptr())
        args.shared_l1_sf_ld, args.shared_l2_sf_ld = ssf1.stride(1), ssf2.stride(1)
    args.situ_beta = 0.0 if situ_beta is None else float(situ_beta)
    args.situ_linear_beta = 0.0 if situ_linear_beta is None else float(situ_linear_beta)
    args.stream = _stream(y)
    _lib.check(_lib.lib().dg_mega_moe_forward(C.byref(args)))
