"""Shared pytest configuration: the ``gpu`` marker and import paths."""

from __future__ import annotations

import json
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

# The reference's pure-Python harness (registry, graph validation, A/B lifecycle), when a copy is at
# hand: an offline ``pip install --target baseline/_ref`` of the reference package, or a checkout next
# to this repository.  It has to be importable BEFORE ``fusedindextopk_b200.api`` is first imported,
# because that module adopts the reference's classes when it finds them.  Tests that need it skip
# themselves otherwise.
for candidate in (ROOT / "baseline" / "_ref", ROOT.parent / "reference" / "src"):
    if (candidate / "fused_index_topk" / "api.py").exists() and str(candidate) not in sys.path:
        sys.path.insert(1, str(candidate))
        break


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


@pytest.fixture(scope="session")
def golden() -> dict:
    """Fixtures recorded from the reference's Python host layer."""

    return json.loads((ROOT / "tests" / "golden" / "reference_golden.json").read_text())
