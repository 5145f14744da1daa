"""GPU parity of the fused BF16 -> E4M3 + UE8M0 cast kernel: bit for bit against the CPU oracle (oracle/quant.py,
which tests/test_oracle_golden.py pins to outputs of the reference's deep_gemm/utils/math.py:26-49), against the shipped
torch helper, and against the packed MN-major layout the SF transform produces."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

import deepgemm_b200 as dg
from oracle import quant as OQ


def make_x(rows, cols, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn((rows, cols), generator=g) * torch.exp(torch.randn((rows, 1), generator=g) * 3)
    if rows >= 8:
        x[0] = 0                                   # amax below the 1e-4 clamp
        x[1] = 1e-6
        x[2, :] = 448.0 * 2.0 ** -3                # amax / 448 an exact power of two
        x[3, ::2] = 449.0                          # just above one
        x[4] = 3.0e38                              # huge
        x[5, 5] = -7.0                             # a single non-zero per row
        x[5, :5] = 0
    return x.to(torch.bfloat16).cuda()


@pytest.mark.parametrize("gran_k", [32, 128])
@pytest.mark.parametrize("shape", [(64, 7168), (300, 2048), (17, 200), (9, 40), (1, 8), (128, 1024 + 64)])
def test_cast_matches_reference_helper(shape, gran_k):
    x = make_x(*shape, seed=shape[0] * 7 + gran_k)
    q_ref, sf_ref = dg.utils.per_token_cast_to_fp8(x, True, gran_k)
    _, packed_ref = dg.utils.per_token_cast_to_fp8(x, True, gran_k, use_packed_ue8m0=True)
    q, sf = dg.per_token_cast_to_fp8_fused(x, gran_k, "float")
    # the CPU oracle on the same BF16 values: E4M3 bytes, scale bits and packed words, bit for bit
    o_q, o_sf = OQ.per_token_cast_to_fp8(x.float().cpu().numpy(), True, gran_k)
    _, o_packed = OQ.per_token_cast_to_fp8(x.float().cpu().numpy(), True, gran_k, use_packed_ue8m0=True)
    assert np.array_equal(q.view(torch.uint8).cpu().numpy(), o_q)
    assert np.array_equal(sf.cpu().numpy().view(np.uint32), o_sf.view(np.uint32))
    assert torch.equal(q.view(torch.uint8), q_ref.view(torch.uint8))
    assert torch.equal(sf, sf_ref)
    q2, packed = dg.per_token_cast_to_fp8_fused(x, gran_k, "packed")
    assert np.array_equal(packed.cpu().numpy(), o_packed)
    assert torch.equal(q2.view(torch.uint8), q_ref.view(torch.uint8))
    assert torch.equal(packed, packed_ref)
    # GEMM-ready layout == what the SF transform makes of the FP32 scales, strides included
    q3, gemm_sf = dg.per_token_cast_to_fp8_fused(x, gran_k, "gemm")
    want = dg.transform_sf_into_required_layout(sf_ref, shape[0], shape[1], (1, gran_k))
    assert torch.equal(q3.view(torch.uint8), q_ref.view(torch.uint8))
    assert gemm_sf.shape == want.shape and gemm_sf.stride(0) == 1
    assert want.size(1) == 1 or gemm_sf.stride() == want.stride()
    # words that cover data must agree; a partly covered word's padding bytes are 127 here, 0 in the transform
    groups = (shape[1] + gran_k - 1) // gran_k
    full = groups // 4
    assert torch.equal(gemm_sf[:, :full], want[:, :full])
    if groups % 4:
        mask = (1 << (8 * (groups % 4))) - 1
        assert torch.equal(gemm_sf[:, full] & mask, want[:, full] & mask)


def test_strided_input_and_in_place_outputs():
    big = make_x(256, 4096, seed=5)
    x = big[:, 1024:3072]                                        # row stride 4096, offset columns
    q_ref, packed_ref = dg.utils.per_token_cast_to_fp8(x.contiguous(), True, 32, use_packed_ue8m0=True)
    q_store = torch.zeros((256, 4096), dtype=torch.uint8, device="cuda").view(torch.float8_e4m3fn)
    sf_store = torch.full((256, 32), -1, dtype=torch.int32, device="cuda")
    dg.per_token_cast_to_fp8_fused(x, 32, "packed", out=q_store[:, :2048], sf_out=sf_store[:, :16])
    assert torch.equal(q_store[:, :2048].view(torch.uint8), q_ref.view(torch.uint8))
    assert (q_store[:, 2048:].view(torch.uint8) == 0).all()
    assert torch.equal(sf_store[:, :16], packed_ref) and (sf_store[:, 16:] == -1).all()


def test_gemm_takes_the_fused_cast_output():
    torch.manual_seed(0)
    m, n, k = 512, 1024, 2048
    a = torch.randn((m, k), device="cuda", dtype=torch.bfloat16)
    b = torch.randn((n, k), device="cuda", dtype=torch.bfloat16)
    b_q = dg.utils.per_block_cast_to_fp8(b, True, 128)
    d_ref = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    dg.fp8_gemm_nt(dg.utils.per_token_cast_to_fp8(a, True, 128), b_q, d_ref)
    d = torch.empty_like(d_ref)
    dg.fp8_gemm_nt(dg.per_token_cast_to_fp8_fused(a, 128, "gemm"), b_q, d, recipe_a=(1, 128), recipe_b=(128, 128))
    torch.cuda.synchronize()
    dg.check_status()
    assert torch.equal(d, d_ref)


def test_argument_checks():
    x = torch.zeros((4, 12), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="cols % 8"):
        dg.per_token_cast_to_fp8_fused(x, 32)
    with pytest.raises(RuntimeError, match="gran_k"):
        dg.per_token_cast_to_fp8_fused(torch.zeros((4, 16), dtype=torch.bfloat16, device="cuda"), 64)


def test_mega_moe_buffer_load_tokens():
    tokens, hidden, inter, experts, topk = 96, 1024, 512, 8, 4
    buf = dg.get_symm_buffer_for_mega_moe(None, experts, tokens, topk, hidden, inter)
    x = make_x(tokens, hidden, seed=11)
    idx = torch.randint(0, experts, (tokens, topk), device="cuda")
    w = torch.rand((tokens, topk), device="cuda")
    assert buf.load_tokens(x, idx, w) == tokens
    q_ref, sf_ref = dg.utils.per_token_cast_to_fp8(x, True, 32, use_packed_ue8m0=True)
    assert torch.equal(buf.x[:tokens].view(torch.uint8), q_ref.view(torch.uint8))
    assert torch.equal(buf.x_sf[:tokens], sf_ref)
    assert torch.equal(buf.topk_idx[:tokens], idx) and torch.equal(buf.topk_weights[:tokens], w)
    buf.destroy()
