"""Generate the Mega MoE golden vector from the reference's own pure-torch baseline.

    python tests/golden/make_mega_moe_golden.py /path/to/reference

The reference's ``tests/test_mega_moe.py`` holds ``_mega_moe_reference`` (the dequantised torch formulation its
gated-activation tests compare the fused kernel with).  The test module itself cannot be imported without the
compiled extension, so this script parses the file, takes the two function definitions it needs
(``_gated_activation_reference`` and ``_mega_moe_reference``) out of the syntax tree, points their one device
literal at the CPU and executes them with the reference's own ``deep_gemm/utils/math.py`` quantisers (loaded by
path).  Inputs and the output of a small seeded case go to ``mega_moe_golden.npz``; the CPU tests compare
``oracle/mega_moe.py`` against it.  Nothing of the reference is copied into this repository.
"""
import ast
import os
import sys
from typing import Optional

import numpy as np
import torch

from make_golden import load


def reference_functions(ref_root, math):
    path = os.path.join(ref_root, "tests/test_mega_moe.py")
    text = open(path).read()
    wanted = {"_gated_activation_reference", "_mega_moe_reference"}
    pieces = [ast.get_source_segment(text, node) for node in ast.parse(text).body
              if isinstance(node, ast.FunctionDef) and node.name in wanted]
    assert len(pieces) == len(wanted), "reference baseline not found"
    ns = {"torch": torch, "Optional": Optional, "per_token_cast_to_fp8": math.per_token_cast_to_fp8,
          "cast_back_from_fp8": math.cast_back_from_fp8}
    exec(compile("\n\n".join(pieces).replace("device='cuda'", "device='cpu'"), path, "exec"), ns)
    return ns["_mega_moe_reference"]


def main(ref_root):
    math = load(os.path.join(ref_root, "deep_gemm/utils/math.py"), "ref_math")
    ref = reference_functions(ref_root, math)
    torch.manual_seed(20251126)
    tokens, hidden, inter, experts, topk = 40, 256, 128, 6, 3

    def fp4_deq(w):
        q, sf = math.per_token_cast_to_fp4(w, use_ue8m0=True, gran_k=32)
        return math.cast_back_from_fp4(q, sf, gran_k=32)

    l1 = torch.stack([fp4_deq((torch.randn(2 * inter, hidden) * (2 / hidden ** 0.5)).bfloat16()) for _ in range(experts)])
    l2 = torch.stack([fp4_deq((torch.randn(hidden, inter) * (1 / inter ** 0.5)).bfloat16()) for _ in range(experts)])
    x = torch.randn(tokens, hidden).bfloat16()
    x_q, x_sf = math.per_token_cast_to_fp8(x, use_ue8m0=True, gran_k=32)
    x_deq = math.cast_back_from_fp8(x_q, x_sf, gran_k=32)
    w, idx = torch.topk(torch.randn(tokens, experts).softmax(-1), topk, dim=-1, sorted=False)
    w = (w / w.sum(-1, keepdim=True)).float()
    idx[::7, 0] = -1                                   # masked slots; expert 5 gets no token at all
    idx[idx == 5] = -1
    y = ref(x_deq.float(), idx, w, l1.float(), l2.float(), "swiglu")
    out = dict(x_deq=x_deq.float().numpy(), topk_idx=idx.numpy(), topk_weights=w.numpy(), l1_deq=l1.float().numpy(),
               l2_deq=l2.float().numpy(), y=y.float().numpy())
    # the other gated activations of the reference's test (tests/test_mega_moe.py:551-566), same inputs
    out["y_geglu"] = ref(x_deq.float(), idx, w, l1.float(), l2.float(), "geglu").float().numpy()
    for tag, kw in (("situ_4_25", dict(situ_beta=4.0, situ_linear_beta=25.0)), ("situ_4_none", dict(situ_beta=4.0)),
                    ("situ_2_3", dict(situ_beta=2.0, situ_linear_beta=3.0))):
        out[f"y_{tag}"] = ref(x_deq.float(), idx, w, l1.float(), l2.float(), "situ", **kw).float().numpy()
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "mega_moe_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main(sys.argv[1])
