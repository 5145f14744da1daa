"""The allocation-free dense GEMM entry point against the ordinary one.

dg_gemm_fp8_fp32sf_noalloc exists for callers that may not allocate device memory around the GEMM (code that
runs inside another runtime's fixed memory plan, or between allocation-free phases of a serving loop): they
cannot create the temporary packed-scale tensors, so the library packs the FP32 scales into a scratch array
that is part of its own image.  Here it is called through the C ABI twice in a row, with different shapes, and
each result must equal bit for bit what dg_sf_pack_ue8m0 + dg_gemm_bs produce with caller-allocated scratch.
The file name sorts last so that a failure here cannot hide other tests in a run that stops at the first one.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

import deepgemm_b200 as dg
from deepgemm_b200 import _lib


def reference_path(qa, qb, m, n, k, gran_k, out_dtype):
    d = torch.empty((m, n), dtype=out_dtype, device="cuda")
    dg.fp8_gemm_nt(qa, qb, d, recipe_a=(1, gran_k), recipe_b=(qb_gran_mn(qb, n), gran_k))
    return d


def qb_gran_mn(qb, n):
    return 1 if qb[1].size(0) == n else 128


def call_noalloc(qa, qb, d, m, n, k, gran_k, out_dtype):
    args = _lib.GemmNoAllocArgs()
    args.m, args.n, args.k, args.gran_k = m, n, k, gran_k
    args.gran_mn_b = qb_gran_mn(qb, n)
    args.d_dtype = _lib.DG_F32 if out_dtype == torch.float32 else _lib.DG_BF16
    args.a, args.sfa, args.b, args.sfb, args.d = (qa[0].data_ptr(), qa[1].data_ptr(), qb[0].data_ptr(),
                                                  qb[1].data_ptr(), d.data_ptr())
    args.lda, args.ldb, args.ldd = qa[0].stride(0), qb[0].stride(0), d.stride(0) * d.element_size()
    args.stream = torch.cuda.current_stream().cuda_stream
    _lib.check(_lib.lib().dg_gemm_fp8_fp32sf_noalloc(C.byref(args)))
    return d


def test_noalloc_gemm_matches_ordinary_entry_point_twice_in_a_row():
    torch.manual_seed(0)
    cases = [(512, 768, 2048, 128, "block", torch.bfloat16), (300, 256, 1024, 32, "row", torch.float32)]
    prepared = []
    for m, n, k, gran_k, b_kind, out_dtype in cases:           # second call reuses the scratch with another shape
        x = torch.randn((m, k), device="cuda", dtype=torch.bfloat16)
        w = torch.randn((n, k), device="cuda", dtype=torch.bfloat16)
        qa = dg.utils.per_token_cast_to_fp8(x, True, gran_k)
        qb = dg.utils.per_block_cast_to_fp8(w, True, 128) if b_kind == "block" else \
            dg.utils.per_token_cast_to_fp8(w, True, gran_k)
        got = torch.full((m, n), float("nan"), dtype=out_dtype, device="cuda")
        call_noalloc(qa, qb, got, m, n, k, gran_k, out_dtype)
        want = reference_path(qa, qb, m, n, k, gran_k, out_dtype)
        torch.cuda.synchronize()
        dg.check_status()
        dg.testing.assert_bitwise_equal(got, want, f"noalloc vs ordinary ({m}x{n}x{k})")
        prepared.append((qa, qb, got, want, m, n, k, gran_k, out_dtype))
    # Nothing is allocated: with both kernels loaded by the calls above (the driver loads a kernel's code on first use),
    # the free device memory the DRIVER reports - which sees every cudaMalloc, not only torch's caching allocator -
    # must not move across further calls, and the results stay right.
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    torch_before = (torch.cuda.memory_allocated(), torch.cuda.memory_reserved())
    for qa, qb, got, want, m, n, k, gran_k, out_dtype in prepared + prepared[::-1]:
        got.fill_(float("nan"))
        call_noalloc(qa, qb, got, m, n, k, gran_k, out_dtype)
        torch.cuda.synchronize()
        dg.testing.assert_bitwise_equal(got, want, f"noalloc, repeated ({m}x{n}x{k})")
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, f"device memory moved by {free_before - free_after} bytes"
    assert (torch.cuda.memory_allocated(), torch.cuda.memory_reserved()) == torch_before


def test_noalloc_gemm_rejects_problems_beyond_the_scratch():
    limit = _lib.lib().dg_noalloc_scratch_bytes()
    m = n = 65536
    k = 16384
    assert (m + n) * (k // 512) * 4 > limit
    args = _lib.GemmNoAllocArgs()
    args.m, args.n, args.k, args.gran_k, args.gran_mn_b, args.d_dtype = m, n, k, 128, 1, _lib.DG_BF16
    one = torch.zeros(16, device="cuda")
    args.a = args.sfa = args.b = args.sfb = args.d = one.data_ptr()
    with pytest.raises(RuntimeError, match="scratch"):
        _lib.check(_lib.lib().dg_gemm_fp8_fp32sf_noalloc(C.byref(args)))
