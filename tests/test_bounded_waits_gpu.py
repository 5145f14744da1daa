"""A wait that cannot be satisfied ends with a status record, not with a hang or a trap.

Host-made failure: the Mega MoE forward is called for rank 0 of a two-rank configuration whose second rank never
runs (both ranks' buffers live on this GPU; nothing ever sets rank 1's barrier flag).  With the wait limit lowered to
200 ms the kernels give up at the cross-rank barrier, record where, and return; `check_status` reports it; the
context stays usable and the next operator runs normally.  Both forward paths are exercised.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

import deepgemm_b200 as dg
from deepgemm_b200 import _lib


def _forward_for_rank0_of_two(fused: bool):
    hidden, inter, experts, topk, tokens = 1024, 512, 8, 4, 128
    cfg = _lib.MoeConfig(2, experts, tokens, topk, hidden, inter)
    lay = _lib.MoeLayout()
    _lib.check(_lib.lib().dg_mega_moe_buffer_layout(C.byref(cfg), C.byref(lay)))
    bufs = [torch.zeros(lay.num_bytes, dtype=torch.int8, device="cuda") for _ in range(2)]
    el = experts // 2
    w1 = torch.zeros((el, 2 * inter, hidden // 2), dtype=torch.int8, device="cuda")
    w2 = torch.zeros((el, hidden, inter // 2), dtype=torch.int8, device="cuda")
    sf1 = torch.full((el, hidden // 128, 2 * inter), 0x7F7F7F7F, dtype=torch.int32, device="cuda")
    sf2 = torch.full((el, inter // 128, hidden), 0x7F7F7F7F, dtype=torch.int32, device="cuda")
    y = torch.zeros((tokens, hidden), dtype=torch.bfloat16, device="cuda")
    args = _lib.MoeArgs()
    args.cfg = cfg
    ptrs = (C.c_void_p * 2)(bufs[0].data_ptr(), bufs[1].data_ptr())
    args.buffer_ptrs = C.cast(ptrs, C.POINTER(C.c_void_p))
    args.rank, args.num_tokens = 0, tokens
    args.y, args.ldy = y.data_ptr(), y.stride(0)
    args.l1_w, args.l1_sf, args.l2_w, args.l2_sf = w1.data_ptr(), sf1.data_ptr(), w2.data_ptr(), sf2.data_ptr()
    args.l1_sf_ld, args.l2_sf_ld = 2 * inter, hidden
    args.stats = None
    args.activation_clamp, args.fast_math = float("inf"), 1
    args.stream = torch.cuda.current_stream().cuda_stream
    dg.mega.set_fused(fused)
    _lib.check(_lib.lib().dg_mega_moe_forward(C.byref(args)))
    return bufs, (w1, w2, sf1, sf2, y)


@pytest.mark.parametrize("fused", [False, True])
def test_missing_peer_times_out_and_context_survives(fused):
    lib = _lib.lib()
    dg.check_status()                                   # clean slate
    _lib.check(lib.dg_set_wait_timeout_ms(200))
    try:
        keep = _forward_for_rank0_of_two(fused)
        with pytest.raises(RuntimeError, match="abandoned a bounded wait"):
            dg.check_status()
        del keep
    finally:
        _lib.check(lib.dg_set_wait_timeout_ms(2000))
        dg.mega.set_fused(True)
    dg.check_status()                                   # the record was consumed
    # the context is intact: an ordinary GEMM runs and is right
    m = n = 256
    k = 512
    a = torch.ones((m, k), device="cuda").to(torch.float8_e4m3fn)
    b = torch.ones((n, k), device="cuda").to(torch.float8_e4m3fn)
    d = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    dg.fp8_gemm_nt((a, torch.ones((m, k // 128), device="cuda")), (b, torch.ones((n // 128, k // 128), device="cuda")), d)
    torch.cuda.synchronize()
    dg.check_status()
    assert torch.equal(d, torch.full_like(d, k))


def test_buffer_reset_after_an_abandoned_call():
    """A call that gives up on a wait leaves barrier arrivals behind; SymmBuffer.reset() makes the buffer usable again.
    The failure is made on the host: stale arrivals are written into the grid barrier's count (what an abandoned call
    leaves behind, exaggerated), so the count never equals the number of CTAs, nobody opens the barrier and every CTA
    waits for a generation that never comes; with the limit at 200 ms the call returns with a status record."""
    import test_mega_moe_gpu as T
    hidden, inter, experts, topk, tokens = 1024, 512, 8, 4, 96
    forward, ref = T._single_rank_case(hidden, inter, experts, topk, tokens)
    buf = dg.get_symm_buffer_for_mega_moe(None, experts, tokens, topk, hidden, inter)
    lib = _lib.lib()
    dg.check_status()
    try:
        y_good = forward(buf)
        torch.cuda.synchronize()
        dg.check_status()
        buf.buffer.view(torch.int32)[34] = 100000       # control word: arrivals of the grid barrier's generation
        _lib.check(lib.dg_set_wait_timeout_ms(200))
        forward(buf)
        with pytest.raises(RuntimeError, match="abandoned a bounded wait"):
            dg.check_status()
        _lib.check(lib.dg_set_wait_timeout_ms(2000))
        buf.reset()
        y = forward(buf)
        torch.cuda.synchronize()
        dg.check_status()
        assert torch.equal(y, y_good)
    finally:
        _lib.check(lib.dg_set_wait_timeout_ms(2000))
        buf.destroy()
