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


# Every comparison made through assert_close leaves a row here; the table is printed at the end of the run
# (pytest_terminal_summary), so the achieved errors are on record whether the run passes or fails.
PARITY_ROWS = []

# Absolute floor of the strict criterion |a-b| <= atol*RMS(b) + rtol*|b|, by relative tolerance class
# (1e-4 relative for float32 results, 2e-2 for bfloat16 results): 1e-6 and 1e-3 of the tensor's RMS.
STRICT_ATOL = {1e-4: 1e-6, 2e-4: 1e-6, 5e-4: 1e-6, 2e-2: 1e-3, 3e-2: 1e-3, 5e-2: 1e-3}


def parity_metrics(a, b, rtol):
    """Achieved errors of `a` against the reference `b`: scale-relative max error, relative L2 error, the fraction of
    elements outside |a-b| <= rtol*(|b| + RMS(b)) (the criterion asserted) and the fraction outside the strict form
    |a-b| <= atol*RMS(b) + rtol*|b| (reported beside it)."""
    import torch

    a = a.detach().double().cpu()
    b = b.detach().double().cpu()
    scale = b.pow(2).mean().sqrt().item()
    diff = (a - b).abs()
    n = max(1, a.numel())
    atol = STRICT_ATOL.get(rtol, rtol * 0.05)
    return {
        "max_rel": diff.max().item() / (scale or 1.0) if a.numel() else 0.0,
        "rel_l2": ((a - b).norm() / (b.norm() + 1e-300)).item(),
        "out": (diff > rtol * (b.abs() + scale)).sum().item() / n,
        "out_strict": (diff > atol * scale + rtol * b.abs()).sum().item() / n,
        "n": a.numel(),
    }


def assert_close(a, b, rtol, name, max_bad_frac=0.0):
    """|a-b| <= rtol * (|b| + RMS(b)) elementwise: relative to each element plus the tensor's scale.

    `max_bad_frac` > 0 applies the criterion statistically (bfloat16 results over long chains: rounding the float64
    reference itself to bfloat16 already leaves a few elements in 10^4 outside): at most that fraction of the
    elements (at least one element) may lie outside, and the relative L2 error must stay below rtol / 2.  The bounds
    passed by the tests are twice the fraction measured on B200 for that case, not round numbers.  The achieved
    figures of every call are recorded and printed at the end of the test run."""
    import torch

    a = a.detach().double().cpu()
    b = b.detach().double().cpu()
    assert a.shape == b.shape, f"{name}: shape {tuple(a.shape)} vs {tuple(b.shape)}"
    assert torch.isfinite(a).all(), f"{name}: non-finite values"
    m = parity_metrics(a, b, rtol)
    PARITY_ROWS.append((name, rtol, max_bad_frac, m))
    print(f"[parity] {name}: rtol={rtol:g} max/RMS={m['max_rel']:.3g} relL2={m['rel_l2']:.3g} "
          f"outside={m['out']:.3g} (allowed {max_bad_frac:g}) outside_strict={m['out_strict']:.3g} n={m['n']}")
    scale = b.pow(2).mean().sqrt().item()
    tol = rtol * (b.abs() + scale)
    diff = (a - b).abs()
    bad = diff > tol
    if max_bad_frac > 0.0:
        assert m["rel_l2"] <= rtol / 2, f"{name}: relative L2 error {m['rel_l2']:.3g} above {rtol / 2:g}"
        if int(bad.sum()) <= max(1, int(max_bad_frac * a.numel())):
            return
    if bad.any():
        idx = torch.argmax(diff - tol).item()
        raise AssertionError(
            f"{name}: {int(bad.sum())} of {a.numel()} elements ({m['out']:.3g}) outside rtol={rtol:g} "
            f"(allowed fraction {max_bad_frac:g}); worst at flat index {idx}: "
            f"got {a.reshape(-1)[idx].item():.8g}, want {b.reshape(-1)[idx].item():.8g}, scale {scale:.3g}, "
            f"scale-relative max error {m['max_rel']:.3g}, relative L2 {m['rel_l2']:.3g}")


def pytest_terminal_summary(terminalreporter, exitstatus, config):
    """Achieved parity figures of the run, worst first within each tolerance class (also written to the file named by
    TTT_PARITY_REPORT when that variable is set)."""
    if not PARITY_ROWS:
        return
    try:
        import torch
        on_gpu = torch.cuda.is_available()
    except Exception:
        on_gpu = False
    if not on_gpu and not os.environ.get("TTT_PARITY_REPORT"):
        return  # CPU runs compare the oracle with the golden vectors only: nothing of the GPU path to report
    worst = {}
    for name, rtol, allowed, m in PARITY_ROWS:
        key = (name, rtol)
        if key not in worst or m["max_rel"] > worst[key][1]["max_rel"]:
            worst[key] = (allowed, m)
    # loosest tolerance class (bfloat16 results) first, worst offenders first within a class
    rows = sorted(worst.items(), key=lambda kv: (-kv[0][1], -kv[1][1]["out"], -kv[1][1]["max_rel"]))
    lines = ["parity figures (GPU result vs oracle; worst call per name): rtol | max/RMS | rel L2 | outside (allowed) "
             "| outside strict | name"]
    for (name, rtol), (allowed, m) in rows:
        lines.append(f"  {rtol:g} | {m['max_rel']:.3g} | {m['rel_l2']:.3g} | {m['out']:.3g} ({allowed:g}) | "
                     f"{m['out_strict']:.3g} | {name}")
    terminalreporter.write_line("")
    shown = lines if len(lines) <= 90 else lines[:90] + [f"  ... {len(lines) - 90} more rows"]
    for ln in shown:
        terminalreporter.write_line(ln)
    path = os.environ.get("TTT_PARITY_REPORT")
    if path:
        Path(path).parent.mkdir(parents=True, exist_ok=True)
        Path(path).write_text("\n".join(lines) + "\n")
