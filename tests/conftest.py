"""Shared test set-up: markers, import path and small helpers."""

from __future__ import annotations

import sys
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parent.parent
for entry in (str(REPO), str(REPO / "tests")):
    if entry not in sys.path:
        sys.path.insert(0, entry)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def pytest_terminal_summary(terminalreporter):
    """How close the engine came to its error bounds, worst case per group of tests (so that drift is seen)."""
    import helpers

    if not helpers.WORST_RATIOS:
        return
    groups: dict[str, tuple[float, str]] = {}
    for case, ratio in helpers.WORST_RATIOS.items():
        group = case.split("[")[0] + ("/float32" if "float32" in case else "/bfloat16")
        if ratio >= groups.get(group, (0.0, ""))[0]:
            groups[group] = (ratio, case)
    terminalreporter.write_line("worst error / bound per group of tests:")
    for group, (ratio, case) in sorted(groups.items()):
        terminalreporter.write_line(f"  {ratio:6.3f}  {group}  ({case})")
