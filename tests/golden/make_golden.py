"""Generate the golden quantisation / layout vectors from the reference's own CPU code.

Run once where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

It loads ``deep_gemm/utils/math.py`` and ``deep_gemm/testing/numeric.py`` of the
reference by file path (both import standalone on CPU), feeds them small seeded
inputs that include the edge cases the reference tests care about (tiny amax at
the 1e-4 clamp, exact powers of two, ties of the E2M1 rounding rule, K not a
multiple of the granularity) and stores inputs and outputs in ``quant_golden.npz``.
The layout vectors restate ``tests/test_layout.py:24-46`` of the reference (the
pure-torch construction of the packed, MN-major, TMA-aligned scale tensor) on the
same inputs.  The committed ``.npz`` is what the CPU tests compare the oracle
against; this script does not run in the test suite.
"""
import importlib.util
import os
import sys

import numpy as np
import torch


def load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def bf16_like(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16)


def packed_layout_torch(x: torch.Tensor, math) -> torch.Tensor:
    """tests/test_layout.py:24-46 of the reference, on CPU."""
    ue = (x.view(torch.int) >> 23).to(torch.uint8)
    mn, k = x.shape[-2], x.shape[-1]
    remove = x.dim() == 2
    if remove:
        x = x.unsqueeze(0)
        ue = ue.unsqueeze(0)
    b = x.shape[0]
    amn, ak = math.align(mn, 4), math.align(k, 4)
    padded = torch.zeros((b, amn, ak), dtype=torch.uint8)
    padded[:, :mn, :k] = ue
    padded = padded.view(-1).view(dtype=torch.int).view(b, amn, ak // 4)
    tr = torch.zeros((b, ak // 4, amn), dtype=torch.int).mT
    tr[:, :, :] = padded
    out = tr[:, :mn, :]
    return out.squeeze(0) if remove else out


def main(ref_root: str):
    math = load(os.path.join(ref_root, "deep_gemm/utils/math.py"), "ref_math")
    numeric = load(os.path.join(ref_root, "deep_gemm/testing/numeric.py"), "ref_numeric")
    out = {}
    torch.manual_seed(20251125)

    def edge_rows(n):
        """Rows exercising clamp / power-of-two / tie behaviour."""
        rows = [
            torch.zeros(n),                                   # all zero -> amax clamp 1e-4
            torch.full((n,), 1e-6),                           # below clamp
            torch.full((n,), 448.0 * 2.0 ** -22),             # exactly at the UE8M0 floor
            torch.full((n,), 448.0),                          # amax/448 == 1 exactly
            torch.full((n,), 449.0),                          # just above a power of two
            torch.full((n,), 224.0),
            torch.linspace(-6, 6, n),                         # dense E2M1 tie coverage after scaling
            torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0] * (n // 8)),
            -torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0] * (n // 8)),
            torch.randn(n) * 1e-3,
            torch.randn(n) * 300,
        ]
        return torch.stack(rows)

    # --- per-token FP8, gran 128 / 32, padded K
    for tag, (m, n, g) in {"pt128": (24, 384, 128), "pt32": (24, 160, 32), "pt128_ragged": (8, 200, 128)}.items():
        x = torch.cat([torch.randn(m, n), edge_rows(n) if n % 8 == 0 else torch.randn(2, n)]).to(torch.bfloat16)
        for ue in (False, True):
            q, sf = math.per_token_cast_to_fp8(x, use_ue8m0=ue, gran_k=g)
            out[f"{tag}_ue{int(ue)}_x"] = x.float().numpy()
            out[f"{tag}_ue{int(ue)}_q"] = q.view(torch.uint8).numpy()
            out[f"{tag}_ue{int(ue)}_sf"] = sf.numpy()
        q, psf = math.per_token_cast_to_fp8(x, use_ue8m0=True, gran_k=g, use_packed_ue8m0=True)
        out[f"{tag}_packed_sf"] = psf.numpy()
        back = math.cast_back_from_fp8(q, psf, gran_k=g, use_packed_ue8m0=True)
        out[f"{tag}_back"] = back.numpy()

    # --- per-block FP8
    x = (torch.randn(300, 260) * 3).to(torch.bfloat16)
    for ue in (False, True):
        q, sf = math.per_block_cast_to_fp8(x, use_ue8m0=ue, gran_k=128)
        out[f"pb_ue{int(ue)}_q"] = q.view(torch.uint8).numpy()
        out[f"pb_ue{int(ue)}_sf"] = sf.numpy()
    out["pb_x"] = x.float().numpy()

    # --- per-channel FP8
    x = torch.randn(256, 48).to(torch.bfloat16)
    for g in (32, 128):
        q, sf = math.per_channel_cast_to_fp8(x, use_ue8m0=True, gran_k=g)
        out[f"pc{g}_q"] = q.view(torch.uint8).numpy()
        out[f"pc{g}_sf"] = sf.numpy()
    out["pc_x"] = x.float().numpy()

    # --- FP4
    x = torch.cat([torch.randn(16, 128) * 0.02, edge_rows(128)]).to(torch.bfloat16)
    for ue in (False, True):
        p, sf = math.per_token_cast_to_fp4(x, use_ue8m0=ue, gran_k=32)
        out[f"fp4_ue{int(ue)}_p"] = p.view(torch.uint8).numpy()
        out[f"fp4_ue{int(ue)}_sf"] = sf.numpy()
    p, psf = math.per_token_cast_to_fp4(x, use_ue8m0=True, gran_k=32, use_packed_ue8m0=True)
    out["fp4_x"] = x.float().numpy()
    out["fp4_packed_sf"] = psf.numpy()
    out["fp4_back"] = math.cast_back_from_fp4(p, psf, gran_k=32, use_packed_ue8m0=True).numpy()
    xx = torch.randn(32, 64).to(torch.bfloat16)
    p2, _ = math.per_token_cast_to_fp4(xx, use_ue8m0=True, gran_k=32)
    out["fp4_t_in"] = p2.view(torch.uint8).numpy()
    out["fp4_t_out"] = math.transpose_packed_fp4(p2).view(torch.uint8).numpy()

    # --- ceil_to_ue8m0 on raw values
    v = torch.tensor([0.0, 1e-45, 1e-38, 2.0 ** -126, 0.75, 1.0, 1.0000001, 3.0, 4.0, 1e30, 3e38, float("inf")])
    out["ceil_in"] = v.numpy()
    out["ceil_out"] = math.ceil_to_ue8m0(v).numpy()

    # --- packed MN-major layout (with its element strides)
    for tag, shape in {"lay2d": (37, 7), "lay2d_al": (64, 8), "lay3d": (3, 21, 57)}.items():
        e = torch.randint(1, 254, shape, dtype=torch.int32)
        sf = (e << 23).view(torch.float)
        lay = packed_layout_torch(sf, math)
        out[f"{tag}_sf"] = sf.numpy()
        out[f"{tag}_out"] = lay.contiguous().numpy()
        out[f"{tag}_strides"] = np.array(lay.stride(), dtype=np.int64)

    # --- calc_diff
    a, b = torch.randn(64, 64), torch.randn(64, 64)
    out["diff_a"], out["diff_b"] = a.numpy(), (a + 0.01 * b).numpy()
    out["diff_val"] = np.array(float(numeric.calc_diff(a, a + 0.01 * b)))

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "quant_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main(sys.argv[1])
