"""Comparison helpers under the reference's `deep_gemm.testing` names (deep_gemm/testing/numeric.py:5-44)."""
import torch


def calc_diff(x: torch.Tensor, y: torch.Tensor) -> float:
    """1 - 2<x,y> / (<x,x> + <y,y>) in float64; 0 for two all-zero tensors."""
    x, y = x.double(), y.double()
    den = (x * x + y * y).sum()
    if den == 0:
        return 0.0
    return float(1 - 2 * (x * y).sum() / den)


def count_bytes(*tensors) -> int:
    total = 0
    for t in tensors:
        if isinstance(t, (tuple, list)):
            total += count_bytes(*t)
        elif t is not None:
            total += t.numel() * t.element_size()
    return total


def assert_bitwise_equal(x: torch.Tensor, y: torch.Tensor, label: str = "") -> None:
    assert x.shape == y.shape and x.dtype == y.dtype, (x.shape, y.shape, x.dtype, y.dtype)
    xb, yb = x.contiguous().view(torch.uint8), y.contiguous().view(torch.uint8)
    if torch.equal(xb, yb):
        return
    bad = (xb != yb).flatten().nonzero()
    first = int(bad[0]) // x.element_size()
    raise AssertionError(f"bitwise mismatch ({label}): {bad.numel()} bytes differ, first element {first}: "
                         f"{x.flatten()[first].item()} vs {y.flatten()[first].item()}")
