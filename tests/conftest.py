import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden_dir():
    return os.path.join(ROOT, "tests", "golden")


def pytest_terminal_summary(terminalreporter):
    """Worst measured error of every labelled parity check, against its bar (tests/util.py: PARITY_LOG)."""
    try:
        import util
    except ImportError:
        return
    if not util.PARITY_LOG:
        return
    terminalreporter.write_line("parity margins (worst relative error / bar):")
    for label, worst, tol in util.PARITY_LOG:
        terminalreporter.write_line(f"  {label}: {worst:.2e} / {tol:.0e}")
