import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), os.pardir))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_terminal_summary(terminalreporter):
    """The worst bfloat16 errors the run has seen, against the bounds of helpers.check_row."""
    try:
        import helpers
    except Exception:  # noqa: BLE001
        return
    w = helpers.worst_ratios
    if w["rows"]:
        terminalreporter.write_line(
            f"worst bfloat16 ratios over {w['rows']} rows: l2 {w['l2']:.4f} (bound {helpers.BF16_L2}), "
            f"largest entry {w['max']:.4f} (bound {helpers.BF16_MAX})"
        )
        top = sorted(helpers.worst_by_test.items(), key=lambda kv: -kv[1][0])[:8]
        for name, (l2, mx) in top:
            terminalreporter.write_line(f"  {l2:.4f} {mx:.4f}  {name}")
