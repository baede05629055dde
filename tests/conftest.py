"""pytest configuration: the `gpu` marker and the shared golden-fixture loader."""
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="requires a CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def pytest_terminal_summary(terminalreporter):
    """Print the unscaled max-abs of every gradient check next to the flat 2e-2 bound."""
    from tests import _util
    if not _util.RECORDS:
        return
    worst = sorted(_util.RECORDS, key=lambda r: -r["max_abs"])
    over = [r for r in worst if r["dtype"] != "float32" and r["max_abs"] > _util.TOL_HALF_MAXABS]
    terminalreporter.write_line(
        f"gradient checks: {len(worst)}; unscaled max-abs above the flat {_util.TOL_HALF_MAXABS:.0e}: {len(over)}")
    for r in worst[:8]:
        terminalreporter.write_line(
            f"  {r['what'] or '?'} [{r['dtype']}]: max-abs {r['max_abs']:.3e} (max|expected| "
            f"{r['max_expected']:.2f}), rel-Frobenius {r['rel_fro']:.3e}")
