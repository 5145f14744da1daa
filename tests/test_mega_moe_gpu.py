"""GPU parity of the Mega MoE forward against the CPU oracle (oracle/mega_moe.py).

Bit-exact: dispatched token rows / scales, routing metadata (as sets per local expert), received-row
statistics.  Floating point: calc_diff <= 2e-4 against the dequantised reference, the bound the
reference's own test uses (tests/test_mega_moe.py:540-549).
"""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

import deepgemm_b200 as dg
import helpers as H
from oracle import mega_moe as OM
from oracle import quant as OQ

MOE_TOL = 2e-4


def make_weights(num_experts, hidden, inter, seed=1234, device="cuda"):
    """All experts from one seed (tests/test_mega_moe.py:490-511): MXFP4 1x32, dequantised copies for the oracle."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    l1 = (torch.randn((num_experts, 2 * inter, hidden), generator=g) * (2 / hidden ** 0.5)).to(torch.bfloat16)
    l2 = (torch.randn((num_experts, hidden, inter), generator=g) * (1 / inter ** 0.5)).to(torch.bfloat16)

    def cast(w):
        q, sf = [], []
        for i in range(w.shape[0]):
            a, b = dg.utils.per_token_cast_to_fp4(w[i].to(device), use_ue8m0=True, gran_k=32)
            q.append(a), sf.append(b)
        q, sf = torch.stack(q), torch.stack(sf)
        deq = np.stack([OQ.cast_back_from_fp4(H.to_np(q[i]), H.to_np(sf[i]), 32) for i in range(w.shape[0])])
        return q, sf, deq

    return cast(l1), cast(l2)


def make_inputs(num_tokens, hidden, num_experts, topk, seed, device="cuda", drop=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn((num_tokens, hidden), generator=g).to(torch.bfloat16).to(device)
    scores = torch.randn((num_tokens, num_experts), generator=g).to(device)
    w, idx = torch.topk(scores.softmax(dim=-1), topk, dim=-1, sorted=False)
    w = w / w.sum(dim=-1, keepdim=True)
    if drop:
        idx[::drop, 0] = -1                                    # masked slots are skipped
    x_fp8, x_sf = dg.utils.per_token_cast_to_fp8(x, use_ue8m0=True, gran_k=32, use_packed_ue8m0=True)
    x_deq = OQ.cast_back_from_fp8(H.to_np(x_fp8), H.to_np(x_sf), 32, use_packed_ue8m0=True)
    return x_fp8, x_sf, idx, w.float(), x_deq


def run_rank(group, rank, ranks, cfg, results=None):
    hidden, inter, experts, topk, tokens, clamp, drop = cfg
    el = experts // ranks
    (q1, sf1, deq1), (q2, sf2, deq2) = make_weights(experts, hidden, inter)
    lo = rank * el
    l1 = (q1[lo:lo + el].contiguous(),
          dg.transform_sf_into_required_layout(sf1[lo:lo + el].contiguous(), 2 * inter, hidden, (1, 32), el))
    l2 = (q2[lo:lo + el].contiguous(),
          dg.transform_sf_into_required_layout(sf2[lo:lo + el].contiguous(), hidden, inter, (1, 32), el))
    l1, l2 = dg.transform_weights_for_mega_moe(l1, l2)
    x_fp8, x_sf, idx, w, x_deq = make_inputs(tokens, hidden, experts, topk, 100 + rank, drop=drop)
    buf = dg.get_symm_buffer_for_mega_moe(group, experts, tokens, topk, hidden, inter)
    stats = torch.zeros(el, dtype=torch.int32, device="cuda")
    y = None
    for it in range(4):              # repeated calls: epochs and counters must reset; fused and per-phase paths alternate
        dg.mega.set_fused(it % 2 == 0)
        buf.x[:tokens].copy_(x_fp8)
        buf.x_sf[:tokens].copy_(x_sf)
        buf.topk_idx[:tokens].copy_(idx)
        buf.topk_weights[:tokens].copy_(w)
        y_it = torch.full((tokens, hidden), float("nan"), dtype=torch.bfloat16, device="cuda")
        dg.fp8_fp4_mega_moe(y_it, l1, l2, buf, cumulative_local_expert_recv_stats=stats, activation_clamp=clamp)
        torch.cuda.synchronize()
        dg.check_status()
        if group is not None:
            group.barrier()
        if y is not None:
            assert torch.equal(y, y_it), f"call {it} (fused={it % 2 == 0}) differs from the first"
        y = y_it
    ref, counts = OM.mega_moe_reference(x_deq, idx.cpu().numpy(), w.cpu().numpy(), deq1, deq2, clamp)
    diff = H.calc_diff(H.to_np(y), ref)
    assert not np.isnan(H.to_np(y)).any()
    assert diff < MOE_TOL, f"rank {rank}: calc_diff {diff}"
    # Integer-exact side: rows received per local expert (over all ranks' tokens) and the pool's routing metadata
    all_idx = [make_inputs(tokens, hidden, experts, topk, 100 + r, drop=drop)[2].cpu().numpy() for r in range(ranks)]
    expect = np.array([sum(int((a == lo + e).sum()) for a in all_idx) for e in range(el)])
    assert np.array_equal(stats.cpu().numpy(), 4 * expect)
    dg.mega.set_fused(True)
    meta = buf.token_src_metadata.cpu().numpy()
    l1_acts = buf.l1_acts.view(torch.uint8)
    start = 0
    for e in range(el):
        rows = meta[start:start + expect[e]]
        got = {tuple(r) for r in rows}
        want = {(r, int(t), int(s)) for r in range(ranks) for t, s in zip(*np.nonzero(all_idx[r] == lo + e))}
        assert got == want, f"expert {e}"
        mine = [(i, t) for i, (r, t, s) in enumerate(rows) if r == rank][:8]
        for i, t in mine:                                      # dispatched rows are byte copies of the source rows
            assert torch.equal(l1_acts[start + i], x_fp8.view(torch.uint8)[t])
        start = (start + expect[e] + 127) // 128 * 128
    buf.destroy()
    if results is not None:
        results[rank] = diff
    return diff


@pytest.mark.parametrize("cfg", [
    (1024, 512, 8, 4, 96, None, 0),          # hidden, inter, experts, topk, tokens, clamp, drop
    (2048, 1024, 16, 4, 700, 10.0, 5),
    (4096, 1536, 16, 4, 96, None, 0),        # the reference's own activation-test shape
    (7168, 2048, 8, 8, 1000, None, 0),       # production hidden / intermediate, few experts
])
def test_mega_moe_single_rank(cfg):
    run_rank(None, 0, 1, cfg)


def test_mega_moe_gated_activations():
    """The reference's test_mega_moe_gated_activations (tests/test_mega_moe.py:484-566) on one GPU: SwiGLU, GeGLU and
    SiTU against the dequantised reference at its shape; SiTU parameters are ignored by the other two; SiTU is far
    from SwiGLU (so the check has teeth)."""
    hidden, inter, experts, topk, tokens = 4096, 1536, 16, 4, 96
    (q1, sf1, deq1), (q2, sf2, deq2) = make_weights(experts, hidden, inter)
    l1 = (q1, dg.transform_sf_into_required_layout(sf1, 2 * inter, hidden, (1, 32), experts))
    l2 = (q2, dg.transform_sf_into_required_layout(sf2, hidden, inter, (1, 32), experts))
    x_fp8, x_sf, idx, w, x_deq = make_inputs(tokens, hidden, experts, topk, 100)

    def run(activation, **kw):
        buf = dg.get_symm_buffer_for_mega_moe(None, experts, tokens, topk, hidden, inter, use_fp8_dispatch=True,
                                              activation=activation)
        a1, a2 = dg.transform_weights_for_mega_moe(l1, l2, activation=activation)
        buf.x[:tokens].copy_(x_fp8), buf.x_sf[:tokens].copy_(x_sf)
        buf.topk_idx[:tokens].copy_(idx), buf.topk_weights[:tokens].copy_(w)
        y = torch.empty((tokens, hidden), dtype=torch.bfloat16, device="cuda")
        dg.fp8_fp4_mega_moe(y, a1, a2, buf, recipe=(1, 1, 32), activation=activation, activation_clamp=None,
                            fast_math=True, **kw)
        torch.cuda.synchronize()
        dg.check_status()
        buf.destroy()
        return y

    def reference(activation, **kw):
        return OM.mega_moe_reference(x_deq, idx.cpu().numpy(), w.cpu().numpy(), deq1, deq2, None, activation, **kw)[0]

    swiglu_ref = reference("swiglu")
    for activation in ("swiglu", "geglu"):
        y = run(activation)
        assert H.calc_diff(H.to_np(y), reference(activation)) < MOE_TOL, activation
        assert torch.equal(y, run(activation, situ_beta=None, situ_linear_beta=None)), activation
        assert torch.equal(y, run(activation, situ_beta=4.0, situ_linear_beta=25.0)), activation
    for beta, lin in ((4.0, 25.0), (4.0, None), (2.0, 3.0)):
        y = H.to_np(run("situ", situ_beta=beta, situ_linear_beta=lin))
        assert H.calc_diff(y, reference("situ", situ_beta=beta, situ_linear_beta=lin)) < MOE_TOL, (beta, lin)
        assert H.calc_diff(y, swiglu_ref) > 50 * MOE_TOL, (beta, lin)


@pytest.mark.parametrize("fused", [True, False])
def test_mega_moe_post_down_route_weights(fused):
    """route_weight_mode='post_down': the gated activation is requantised unweighted and the BF16 row of the second
    GEMM is multiplied by its route weight (and rounded again) at the combine write
    (impls/sm100_fp8_fp4_mega_moe.cuh:1538-1566 of the reference).  Against the oracle's statement of that boundary;
    the result must differ from the pre-down one (the two modes round at different places)."""
    hidden, inter, experts, topk, tokens = 2048, 1024, 16, 4, 300
    (q1, sf1, deq1), (q2, sf2, deq2) = make_weights(experts, hidden, inter)
    l1 = (q1, dg.transform_sf_into_required_layout(sf1, 2 * inter, hidden, (1, 32), experts))
    l2 = (q2, dg.transform_sf_into_required_layout(sf2, hidden, inter, (1, 32), experts))
    l1, l2 = dg.transform_weights_for_mega_moe(l1, l2)
    x_fp8, x_sf, idx, w, x_deq = make_inputs(tokens, hidden, experts, topk, 321, drop=9)
    buf = dg.get_symm_buffer_for_mega_moe(None, experts, tokens, topk, hidden, inter)
    dg.mega.set_fused(fused)
    try:
        outs = {}
        for mode in (dg.RouteWeightMode.POST_DOWN, "pre_down"):
            buf.x[:tokens].copy_(x_fp8), buf.x_sf[:tokens].copy_(x_sf)
            buf.topk_idx[:tokens].copy_(idx), buf.topk_weights[:tokens].copy_(w)
            y = torch.full((tokens, hidden), float("nan"), dtype=torch.bfloat16, device="cuda")
            dg.fp8_fp4_mega_moe(y, l1, l2, buf, route_weight_mode=mode)
            torch.cuda.synchronize()
            dg.check_status()
            outs[str(mode)] = H.to_np(y)
        ref = OM.mega_moe_reference(x_deq, idx.cpu().numpy(), w.cpu().numpy(), deq1, deq2,
                                    route_weight_mode="post_down")[0]
        got = outs[str(dg.RouteWeightMode.POST_DOWN)]
        assert not np.isnan(got).any()
        assert H.calc_diff(got, ref) < MOE_TOL
        assert not np.array_equal(got, outs["pre_down"])
    finally:
        dg.mega.set_fused(True)
        buf.destroy()


def _single_rank_case(hidden, inter, experts, topk, tokens, seed=100):
    (q1, sf1, deq1), (q2, sf2, deq2) = make_weights(experts, hidden, inter)
    l1 = (q1, dg.transform_sf_into_required_layout(sf1, 2 * inter, hidden, (1, 32), experts))
    l2 = (q2, dg.transform_sf_into_required_layout(sf2, hidden, inter, (1, 32), experts))
    l1, l2 = dg.transform_weights_for_mega_moe(l1, l2)
    x_fp8, x_sf, idx, w, x_deq = make_inputs(tokens, hidden, experts, topk, seed)
    ref = OM.mega_moe_reference(x_deq, idx.cpu().numpy(), w.cpu().numpy(), deq1, deq2)[0]

    def fill(buf):
        buf.x[:tokens].copy_(x_fp8), buf.x_sf[:tokens].copy_(x_sf)
        buf.topk_idx[:tokens].copy_(idx), buf.topk_weights[:tokens].copy_(w)

    def forward(buf):
        fill(buf)
        y = torch.full((tokens, hidden), float("nan"), dtype=torch.bfloat16, device="cuda")
        dg.fp8_fp4_mega_moe(y, l1, l2, buf)
        return y

    return forward, ref


@pytest.mark.parametrize("fused", [True, False])
def test_mega_moe_fp8_weights(fused):
    """Routed experts with E4M3 weights and 1 x 32 UE8M0 scales (the reference's mma_type "fp8xfp8",
    csrc/apis/mega_moe.hpp:374-377): same forward, the weight operand read as bytes instead of packed nibbles."""
    hidden, inter, experts, topk, tokens = 2048, 1024, 8, 4, 500
    g = torch.Generator(device="cpu").manual_seed(99)
    w1 = (torch.randn((experts, 2 * inter, hidden), generator=g) * (2 / hidden ** 0.5)).to(torch.bfloat16).cuda()
    w2 = (torch.randn((experts, hidden, inter), generator=g) * (1 / inter ** 0.5)).to(torch.bfloat16).cuda()

    def cast(w):
        q, sf = zip(*[dg.utils.per_token_cast_to_fp8(w[e], use_ue8m0=True, gran_k=32) for e in range(w.size(0))])
        q, sf = torch.stack(q), torch.stack(sf)
        deq = np.stack([OQ.cast_back_from_fp8(H.to_np(q[e]), H.to_np(sf[e]), 32) for e in range(w.size(0))])
        return q, sf, deq

    (q1, sf1, deq1), (q2, sf2, deq2) = cast(w1), cast(w2)
    l1 = (q1, dg.transform_sf_into_required_layout(sf1, 2 * inter, hidden, (1, 32), experts))
    l2 = (q2, dg.transform_sf_into_required_layout(sf2, hidden, inter, (1, 32), experts))
    l1, l2 = dg.transform_weights_for_mega_moe(l1, l2)
    x_fp8, x_sf, idx, w, x_deq = make_inputs(tokens, hidden, experts, topk, 55, drop=6)
    buf = dg.get_symm_buffer_for_mega_moe(None, experts, tokens, topk, hidden, inter, mma_type="fp8xfp8")
    dg.mega.set_fused(fused)
    try:
        buf.x[:tokens].copy_(x_fp8), buf.x_sf[:tokens].copy_(x_sf)
        buf.topk_idx[:tokens].copy_(idx), buf.topk_weights[:tokens].copy_(w)
        y = torch.full((tokens, hidden), float("nan"), dtype=torch.bfloat16, device="cuda")
        dg.fp8_fp4_mega_moe(y, l1, l2, buf)
        torch.cuda.synchronize()
        dg.check_status()
        ref = OM.mega_moe_reference(x_deq, idx.cpu().numpy(), w.cpu().numpy(), deq1, deq2)[0]
        assert not np.isnan(H.to_np(y)).any()
        assert H.calc_diff(H.to_np(y), ref) < MOE_TOL
    finally:
        dg.mega.set_fused(True)
        buf.destroy()


@pytest.mark.parametrize("fused", [True, False])
@pytest.mark.parametrize("num_shared,routed_fp8", [(1, False), (2, True)])
def test_mega_moe_shared_experts(fused, num_shared, routed_fp8):
    """Shared experts (csrc/apis/mega_moe.hpp:392-415 of the reference): E4M3 weights [2 S I, H] / [H, S I] applied to
    every token on its own rank, no route weight, their BF16 row first in the final sum.  Against the oracle's statement
    of the reference test's unfused baseline (tests/test_mega_moe.py:280-306); several calls with a changing token count."""
    hidden, inter, experts, topk, tokens = 2048, 512, 8, 4, 300
    g = torch.Generator(device="cpu").manual_seed(17)

    def cast_fp8(w):
        q, sf = dg.utils.per_token_cast_to_fp8(w.cuda(), use_ue8m0=True, gran_k=32)
        return q, sf, OQ.cast_back_from_fp8(H.to_np(q), H.to_np(sf), 32)

    i_s = inter * num_shared
    sq1, ssf1, sdeq1 = cast_fp8((torch.randn((2 * i_s, hidden), generator=g) * (2 / hidden ** 0.5)).to(torch.bfloat16))
    sq2, ssf2, sdeq2 = cast_fp8((torch.randn((hidden, i_s), generator=g) * (1 / i_s ** 0.5)).to(torch.bfloat16))
    s1 = (sq1, dg.transform_sf_into_required_layout(ssf1, 2 * i_s, hidden, (1, 32)))
    s2 = (sq2, dg.transform_sf_into_required_layout(ssf2, hidden, i_s, (1, 32)))
    s1, s2 = dg.transform_weights_for_mega_moe(s1, s2)
    if routed_fp8:
        r1 = (torch.randn((experts, 2 * inter, hidden), generator=g) * (2 / hidden ** 0.5)).to(torch.bfloat16)
        r2 = (torch.randn((experts, hidden, inter), generator=g) * (1 / inter ** 0.5)).to(torch.bfloat16)
        c1, c2 = [cast_fp8(r1[e]) for e in range(experts)], [cast_fp8(r2[e]) for e in range(experts)]
        q1, sf1, deq1 = (torch.stack([c[0] for c in c1]), torch.stack([c[1] for c in c1]), np.stack([c[2] for c in c1]))
        q2, sf2, deq2 = (torch.stack([c[0] for c in c2]), torch.stack([c[1] for c in c2]), np.stack([c[2] for c in c2]))
    else:
        (q1, sf1, deq1), (q2, sf2, deq2) = make_weights(experts, hidden, inter)
    l1 = (q1, dg.transform_sf_into_required_layout(sf1, 2 * inter, hidden, (1, 32), experts))
    l2 = (q2, dg.transform_sf_into_required_layout(sf2, hidden, inter, (1, 32), experts))
    l1, l2 = dg.transform_weights_for_mega_moe(l1, l2)
    buf = dg.get_symm_buffer_for_mega_moe(None, experts, tokens, topk, hidden, inter, num_shared_experts=num_shared,
                                          mma_type="fp8xfp8" if routed_fp8 else "fp8xfp4")
    assert buf.combine.size(0) == topk + 1 and buf.shared_l2_acts.size(1) == i_s
    dg.mega.set_fused(fused)
    try:
        for n_tok, seed in ((tokens, 1), (77, 2), (tokens, 3)):
            x_fp8, x_sf, idx, w, x_deq = make_inputs(n_tok, hidden, experts, topk, seed, drop=5)
            buf.x[:n_tok].copy_(x_fp8), buf.x_sf[:n_tok].copy_(x_sf)
            buf.fill_shared_scales(n_tok)
            buf.topk_idx[:n_tok].copy_(idx), buf.topk_weights[:n_tok].copy_(w)
            y = torch.full((n_tok, hidden), float("nan"), dtype=torch.bfloat16, device="cuda")
            dg.fp8_fp4_mega_moe(y, l1, l2, buf, shared_l1_weights=s1, shared_l2_weights=s2)
            torch.cuda.synchronize()
            dg.check_status()
            ref = OM.mega_moe_reference(x_deq, idx.cpu().numpy(), w.cpu().numpy(), deq1, deq2,
                                        shared_l1_deq=sdeq1, shared_l2_deq=sdeq2)[0]
            routed_only = OM.mega_moe_reference(x_deq, idx.cpu().numpy(), w.cpu().numpy(), deq1, deq2)[0]
            got = H.to_np(y)
            assert not np.isnan(got).any()
            assert H.calc_diff(got, ref) < MOE_TOL, (n_tok, seed)
            assert H.calc_diff(got, routed_only) > 50 * MOE_TOL      # the shared part is not small
        with pytest.raises(RuntimeError, match="shared expert weights"):
            dg.fp8_fp4_mega_moe(y, l1, l2, buf)
    finally:
        dg.mega.set_fused(True)
        buf.destroy()


def test_mega_moe_with_fewer_sms():
    """The persistent grid follows set_num_sms and DG_MEGA_MOE_SM_HEADROOM between calls on one buffer (its grid barrier
    does not remember earlier grids); a grouped GEMM runs under the same knob.  Results equal the full-grid ones bit
    for bit (the tiles' arithmetic does not depend on which CTA runs them)."""
    hidden, inter, experts, topk, tokens = 2048, 1024, 16, 4, 700
    forward, ref = _single_rank_case(hidden, inter, experts, topk, tokens)
    buf = dg.get_symm_buffer_for_mega_moe(None, experts, tokens, topk, hidden, inter)
    full = dg.get_num_sms()
    try:
        y_full = forward(buf)
        torch.cuda.synchronize()
        dg.check_status()
        assert H.calc_diff(H.to_np(y_full), ref) < MOE_TOL
        for sms, headroom in ((full - 2, None), (100, None), (full, "3"), (full + 40, None), (full, None)):
            dg.set_num_sms(sms)
            if headroom is None:
                os.environ.pop("DG_MEGA_MOE_SM_HEADROOM", None)
            else:
                os.environ["DG_MEGA_MOE_SM_HEADROOM"] = headroom
            y = forward(buf)
            torch.cuda.synchronize()
            dg.check_status()
            assert torch.equal(y, y_full), (sms, headroom)
        dg.set_num_sms(full - 2)
        case = H.make_m_grouped_contiguous(4, 300, 512, 1024, seed=9)
        d = torch.full((case["m"], 512), float("nan"), dtype=torch.bfloat16, device="cuda")
        ga, gmb, gb = case["grans"]
        dg.m_grouped_fp8_fp4_gemm_nt_contiguous(case["a"], case["b"], d, case["layout"], recipe_a=(1, ga), recipe_b=(gmb, gb))
        torch.cuda.synchronize()
        dg.check_status()
        from oracle import gemm as OG
        assert H.calc_diff(H.to_np(d)[case["valid"]], H.ref_m_grouped(case)[case["valid"]]) < 1e-3
    finally:
        os.environ.pop("DG_MEGA_MOE_SM_HEADROOM", None)
        dg.set_num_sms(0)
        buf.destroy()


def test_mega_moe_buffer_reused_for_another_configuration():
    """SymmBuffer(base=...) runs a second configuration on the first one's memory (deep_gemm/mega/__init__.py:80-92),
    then the first again: the words that live across calls keep their place, everything else is rewritten."""
    big = (2048, 1024, 16, 4, 700)
    small = (1024, 512, 8, 4, 96)
    fwd_big, ref_big = _single_rank_case(*big)
    fwd_small, ref_small = _single_rank_case(*small, seed=7)
    buf = dg.get_symm_buffer_for_mega_moe(None, big[2], big[4], big[3], big[0], big[1])
    assert H.calc_diff(H.to_np(fwd_big(buf)), ref_big) < MOE_TOL
    view = dg.SymmBuffer(None, small[2], small[4], small[3], small[0], small[1], base=buf)
    assert view.buffer.data_ptr() == buf.buffer.data_ptr()
    for fused in (True, False, True):
        dg.mega.set_fused(fused)
        assert H.calc_diff(H.to_np(fwd_small(view)), ref_small) < MOE_TOL
        assert H.calc_diff(H.to_np(fwd_big(buf)), ref_big) < MOE_TOL
        torch.cuda.synchronize()
        dg.check_status()
    dg.mega.set_fused(True)
    buf.destroy()


def test_mega_moe_pool_smaller_than_the_rows_is_reported():
    """num_ring_tokens below what arrives: the call is abandoned and reported (no write past the pool, no hang), and a
    later call that fits runs normally on the same buffer."""
    hidden, inter, experts, topk, tokens = 1024, 512, 8, 4, 512
    forward, ref = _single_rank_case(hidden, inter, experts, topk, tokens)
    buf = dg.get_symm_buffer_for_mega_moe(None, experts, tokens, topk, hidden, inter, num_ring_tokens=512)
    assert buf.layout.pool_rows < tokens * topk
    for fused in (True, False):
        dg.mega.set_fused(fused)
        forward(buf)
        with pytest.raises(RuntimeError, match="pool"):
            dg.check_status()
    dg.mega.set_fused(True)
    roomy = dg.get_symm_buffer_for_mega_moe(None, experts, tokens, topk, hidden, inter, num_ring_tokens=tokens * topk)
    assert H.calc_diff(H.to_np(forward(roomy)), ref) < MOE_TOL
    dg.check_status()
    buf.destroy(), roomy.destroy()


def _worker(local_rank, ranks, cfg, port, results):
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", world_size=ranks, rank=local_rank)
    try:
        run_rank(dist.group.WORLD, local_rank, ranks, cfg, results)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("ranks", [2, 4, 8])
def test_mega_moe_expert_parallel(ranks):
    if torch.cuda.device_count() < ranks:
        pytest.skip(f"needs {ranks} GPUs")
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import torch.multiprocessing as mp
    results = mp.get_context("spawn").Manager().dict()
    cfg = (2048, 1024, 8 * ranks, 4, 300, None, 7)
    mp.spawn(_worker, args=(ranks, cfg, 29531 + ranks, results), nprocs=ranks, join=True)
    assert len(results) == ranks and all(v < MOE_TOL for v in results.values())
