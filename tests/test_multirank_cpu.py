"""World-size-2 checks that need no GPU (gloo backend, spawned processes).

(a) The expert-parallel composition of the Mega MoE forward: every rank routes its tokens to the ranks that own the
    experts (expert e lives on rank e // experts_per_rank), the owners run their experts on the rows they receive and
    send each result back to the (rank, token, slot) it came from, the source sums its slots in slot order.  Built
    here from the oracle's single-rank pieces with gloo all_to_all exchanges, it must equal the oracle applied to each
    rank's tokens with all experts at hand, bit for bit, and the per-expert received-row counts must add up.  This is
    the host-side statement of what the kernels do over NVLink (dispatch = receiver pulls, combine = sender pushes).
(b) `bench.py --impl reference` under torchrun: rank 0 alone prints the one JSON line, the other rank exits 0.
"""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from oracle import mega_moe as OM          # noqa: E402
from oracle import quant as OQ             # noqa: E402


def _case(rank, experts, tokens=24, hidden=64, inter=32, topk=2):
    rng = np.random.default_rng(7)                      # weights: the same on every rank
    l1 = OQ.bf16_round(rng.standard_normal((experts, 2 * inter, hidden), dtype=np.float32) * 0.3)
    l2 = OQ.bf16_round(rng.standard_normal((experts, hidden, inter), dtype=np.float32) * 0.3)
    rng = np.random.default_rng(100 + rank)             # tokens and routing: per rank
    x = OQ.bf16_round(rng.standard_normal((tokens, hidden), dtype=np.float32))
    idx = np.stack([rng.permutation(experts)[:topk] for _ in range(tokens)]).astype(np.int64)
    idx[::5, 0] = -1                                    # masked slots
    w = rng.random((tokens, topk), dtype=np.float32)
    return x, idx, w, l1, l2


def _exchange(objs, world):
    out = [None] * world
    dist.all_to_all_object_list(out, objs) if hasattr(dist, "all_to_all_object_list") else None
    if out[0] is None:                                  # gloo builds without the object all-to-all
        gathered = [None] * world
        dist.all_gather_object(gathered, objs)
        out = [gathered[src][dist.get_rank()] for src in range(world)]
    return out


def _ep_worker(rank, world, port, results):
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", world_size=world, rank=rank)
    try:
        experts = 4 * world
        el = experts // world
        x, idx, w, l1, l2 = _case(rank, experts)
        tokens, topk = idx.shape
        # dispatch: rows grouped by owning rank, with where they came from
        send = [[] for _ in range(world)]
        for t in range(tokens):
            for s in range(topk):
                e = int(idx[t, s])
                if e >= 0:
                    send[e // el].append((e, t, s, x[t], w[t, s]))
        recv = _exchange(send, world)
        counts = np.zeros(el, dtype=np.int64)
        back = [[] for _ in range(world)]
        for src, rows in enumerate(recv):
            for e, t, s, xr, wr in rows:
                counts[e - rank * el] += 1
                # one (token, expert) row through this rank's expert e: the oracle with a single token and slot
                y, _ = OM.mega_moe_reference(xr[None, :], np.array([[0]]), np.array([[wr]], dtype=np.float32),
                                             l1[e][None], l2[e][None])
                back[src].append((t, s, y[0]))
        mine = _exchange(back, world)
        per_slot = np.zeros((topk, tokens, x.shape[1]), dtype=np.float32)
        for rows in mine:
            for t, s, y in rows:
                per_slot[s, t] = y
        acc = np.zeros((tokens, x.shape[1]), dtype=np.float32)
        for s in range(topk):                            # slot order, float32, as the reduce kernel sums
            acc += per_slot[s]
        got = OQ.bf16_round(acc)
        want, all_counts = OM.mega_moe_reference(x, idx, w, l1, l2)
        totals = torch.from_numpy(np.concatenate([np.zeros(rank * el, dtype=np.int64), counts,
                                                  np.zeros(experts - (rank + 1) * el, dtype=np.int64)]))
        sent = torch.from_numpy(all_counts.copy())
        dist.all_reduce(totals), dist.all_reduce(sent)
        results[rank] = (bool(np.array_equal(got, want)), bool(torch.equal(totals, sent)))
    finally:
        dist.destroy_process_group()


def test_expert_parallel_composition_gloo_world2():
    results = mp.get_context("spawn").Manager().dict()
    mp.spawn(_ep_worker, args=(2, 29641, results), nprocs=2, join=True)
    assert dict(results) == {0: (True, True), 1: (True, True)}


def test_reference_arm_under_torchrun_prints_one_line():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29643", os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2",
           "--steps", "1", "--warmup", "1"]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [l for l in res.stdout.splitlines() if l.strip()]
    assert len(lines) == 1, res.stdout
    rec = json.loads(lines[0])
    assert rec["impl"] == "reference" and rec["n_gpus"] == 2 and rec["value"] > 0
    assert rec["e2e"]["h2d_bytes_per_step"] == 0 and rec["cpu_baseline"]["kind"] == "port"
    # torchrun gives its children OMP_NUM_THREADS=1; the arm must use all the host cores anyway
    assert rec["cpu_baseline"]["cores"] == len(os.sched_getaffinity(0))
    assert rec["config"]["workload"].startswith("m_grouped_fp8_gemm_nt_contiguous") and rec["config"]["m"] == 67328
