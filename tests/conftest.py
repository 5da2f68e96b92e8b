import os
import sys
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parent.parent
if str(REPO) not in sys.path:
    sys.path.insert(0, str(REPO))

GOLDEN = REPO / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN


def rel_err(a, b):
    """max |a-b| divided by the RMS of the reference tensor b (scale-relative max error)."""
    import torch

    a = a.detach().double().cpu()
    b = b.detach().double().cpu()
    scale = b.pow(2).mean().sqrt().item()
    if scale == 0.0:
        scale = 1.0
    return (a - b).abs().max().item() / scale


def assert_close(a, b, rtol, name, max_bad_frac=0.0):
    """|a-b| <= rtol * (|b| + RMS(b)) elementwise: relative to each element plus the tensor's scale.

    `max_bad_frac` > 0 applies the criterion statistically (used for bfloat16 results, whose storage rounding alone
    reaches 5e-2 of the RMS on heavy-tailed tensors): at most that fraction of elements (at least one element) may lie outside, and the
    relative L2 error must stay below rtol / 2."""
    import torch

    a = a.detach().double().cpu()
    b = b.detach().double().cpu()
    assert a.shape == b.shape, f"{name}: shape {tuple(a.shape)} vs {tuple(b.shape)}"
    assert torch.isfinite(a).all(), f"{name}: non-finite values"
    scale = b.pow(2).mean().sqrt().item()
    tol = rtol * (b.abs() + scale)
    diff = (a - b).abs()
    bad = diff > tol
    if max_bad_frac > 0.0:
        rel_l2 = ((a - b).norm() / (b.norm() + 1e-300)).item()
        assert rel_l2 <= rtol / 2, f"{name}: relative L2 error {rel_l2:.3g} above {rtol / 2:g}"
        if int(bad.sum()) <= max(1, int(max_bad_frac * a.numel())):
            return
    if bad.any():
        idx = torch.argmax(diff - tol).item()
        raise AssertionError(
            f"{name}: {int(bad.sum())} of {a.numel()} elements outside rtol={rtol:g}; worst at flat index {idx}: "
            f"got {a.reshape(-1)[idx].item():.8g}, want {b.reshape(-1)[idx].item():.8g}, scale {scale:.3g}, "
            f"scale-relative max error {diff.max().item() / (scale or 1.0):.3g}")
