"""Generate golden vectors for the scale-factor layout and the Mega MoE weight permutations from the reference's own
Python text.

    python tests/golden/make_layout_golden.py /path/to/reference

Three functions are taken out of the reference's files through the syntax tree and executed on CPU, unchanged:
``get_mn_major_tma_aligned_packed_ue8m0_tensor_torch_impl`` (tests/test_layout.py:24-46, the pure-torch statement of the
packed MN-major TMA-aligned layout) and ``_interleave_weights`` / ``_transpose_sf_for_utccp``
(deep_gemm/mega/__init__.py:167-198, the weight and scale permutations of transform_weights_for_mega_moe).  Neither
file can be imported without the compiled extension.  Seeded inputs and the functions' outputs (values and strides)
go to ``layout_golden.npz``; tests/test_oracle_golden.py holds ``oracle/layout.py`` to them bit for bit.  Nothing of
the reference is copied into this repository.
"""
import ast
import os
import sys

import numpy as np
import torch

from make_golden import load


def functions_from(path, wanted, namespace):
    text = open(path).read()
    pieces = [ast.get_source_segment(text, node) for node in ast.parse(text).body
              if isinstance(node, ast.FunctionDef) and node.name in wanted]
    assert len(pieces) == len(wanted), f"{wanted} not all found in {path}"
    exec(compile("\n\n".join(pieces), path, "exec"), namespace)
    return [namespace[name] for name in wanted]


def main(ref_root):
    math = load(os.path.join(ref_root, "deep_gemm/utils/math.py"), "ref_math")

    def get_tma_aligned_size(x, element_size):       # csrc/utils/math.hpp:23-27: rows padded to 16 bytes
        return math.align(x, 16 // element_size)

    (packed_impl,) = functions_from(os.path.join(ref_root, "tests/test_layout.py"),
                                    ["get_mn_major_tma_aligned_packed_ue8m0_tensor_torch_impl"],
                                    {"torch": torch, "align": math.align, "get_tma_aligned_size": get_tma_aligned_size})
    interleave, utccp = functions_from(os.path.join(ref_root, "deep_gemm/mega/__init__.py"),
                                       ["_interleave_weights", "_transpose_sf_for_utccp"], {"torch": torch})
    g = torch.Generator().manual_seed(20261125)
    out = {}
    # packed MN-major layout: 2-D and batched, ragged mn and k
    for tag, shape in (("p2", (133, 57)), ("p2b", (4, 7)), ("p3", (3, 130, 9)), ("p1row", (1, 56))):
        e = torch.randint(1, 254, shape, generator=g, dtype=torch.int32)
        sf = (e << 23).view(torch.float32)
        packed = packed_impl(sf)
        out[f"{tag}_sf"] = sf.numpy()
        out[f"{tag}_packed"] = np.ascontiguousarray(packed.numpy())
        out[f"{tag}_strides"] = np.array(packed.stride(), dtype=np.int64)
    # weight permutations: int8 data [G, 2I, H/2] and packed int32 scales [G, 2I, pk] kept MN-major
    w = torch.randint(-128, 127, (2, 256, 24), generator=g, dtype=torch.int8)
    sf_store = torch.randint(0, 2 ** 31 - 1, (2, 5, 256), generator=g, dtype=torch.int32)
    sf = sf_store.transpose(1, 2)
    out["w"], out["w_interleaved"] = w.numpy(), interleave(w).numpy()
    out["wsf"] = np.ascontiguousarray(sf.numpy())
    il_sf = interleave(sf)
    out["wsf_interleaved"] = np.ascontiguousarray(il_sf.numpy())
    t_sf = utccp(il_sf)
    out["wsf_utccp"] = np.ascontiguousarray(t_sf.numpy())
    out["wsf_utccp_strides"] = np.array(t_sf.stride(), dtype=np.int64)
    out["wsf_in_strides"] = np.array(sf.stride(), dtype=np.int64)
    w2d = torch.randint(-128, 127, (64, 12), generator=g, dtype=torch.int8)
    out["w2d"], out["w2d_interleaved"] = w2d.numpy(), interleave(w2d).numpy()
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "layout_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main(sys.argv[1])
