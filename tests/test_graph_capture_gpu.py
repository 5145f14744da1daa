"""The operators read their sizes on the device and do no host synchronisation: they can be captured in a CUDA graph
and replayed with other contents in the same buffers (the masked GEMM is the reference's CUDA-graph decode path,
csrc/apis/gemm.hpp:273-322; its Mega MoE forward has the same requirement, tests/test_mega_moe_compat.py:35-51)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

import deepgemm_b200 as dg
import helpers as H


def test_masked_gemm_replays_with_new_masks():
    g, max_m, n, k = 4, 512, 512, 1024
    case = H.make_masked(g, max_m, 2 * max_m, n, k, seed=3)       # every row quantised: any mask is valid later
    sfa = dg.transform_sf_into_required_layout(case["a"][1], max_m, k, (1, 128), num_groups=g)
    sfb = dg.transform_sf_into_required_layout(case["b"][1], n, k, (128, 128), num_groups=g)
    masked = case["masked"].clone()
    d = torch.zeros((g, max_m, n), dtype=torch.bfloat16, device="cuda")

    def run():
        dg.m_grouped_fp8_gemm_nt_masked((case["a"][0], sfa), (case["b"][0], sfb), d, masked, 200,
                                        recipe_a=(1, 128), recipe_b=(1, 128))

    run()                                                  # first call outside the capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        run()
    for new in ([17, 512, 0, 130], [256, 1, 300, 511]):
        masked.copy_(torch.tensor(new, dtype=torch.int32))
        d.zero_()
        graph.replay()
        torch.cuda.synchronize()
        dg.check_status()
        got = d.clone()
        d.zero_()
        run()
        torch.cuda.synchronize()
        for i, mm in enumerate(new):
            assert torch.equal(got[i, :mm], d[i, :mm]), (new, i)
            ref = case["ref_a"][i, :mm] @ case["ref_b"][i].T if mm else None
            if mm:
                assert H.calc_diff(H.to_np(got[i, :mm]), ref) < 1e-3


@pytest.mark.parametrize("fused", [True, False])
def test_mega_moe_forward_replays(fused):
    from test_mega_moe_gpu import make_inputs, make_weights
    hidden, inter, experts, topk, tokens = 1024, 512, 8, 4, 128
    (q1, sf1, _), (q2, sf2, _) = make_weights(experts, hidden, inter)
    l1 = (q1, dg.transform_sf_into_required_layout(sf1, 2 * inter, hidden, (1, 32), experts))
    l2 = (q2, dg.transform_sf_into_required_layout(sf2, hidden, inter, (1, 32), experts))
    l1, l2 = dg.transform_weights_for_mega_moe(l1, l2)
    buf = dg.get_symm_buffer_for_mega_moe(None, experts, tokens, topk, hidden, inter)
    y = torch.zeros((tokens, hidden), dtype=torch.bfloat16, device="cuda")
    dg.mega.set_fused(fused)
    try:
        def fill(seed):
            x_fp8, x_sf, idx, w, _ = make_inputs(tokens, hidden, experts, topk, seed)
            buf.x[:tokens].copy_(x_fp8), buf.x_sf[:tokens].copy_(x_sf)
            buf.topk_idx[:tokens].copy_(idx), buf.topk_weights[:tokens].copy_(w)

        fill(1)
        dg.fp8_fp4_mega_moe(y, l1, l2, buf)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            dg.fp8_fp4_mega_moe(y, l1, l2, buf)
        for seed in (2, 3):
            fill(seed)
            y.zero_()
            graph.replay()
            torch.cuda.synchronize()
            dg.check_status()
            got = y.clone()
            y.zero_()
            dg.fp8_fp4_mega_moe(y, l1, l2, buf)
            torch.cuda.synchronize()
            assert torch.equal(got, y), seed
            assert got.abs().sum() > 0
    finally:
        dg.mega.set_fused(True)
        buf.destroy()
