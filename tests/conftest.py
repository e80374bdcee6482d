import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        have = torch.cuda.is_available()
    except Exception:
        have = False
    if have:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """Model folders of the tiny configurations, written once per session into a
    temporary folder: {name: path}."""
    from helpers import TINY, write_tiny

    root = tmp_path_factory.mktemp("models")
    return {name: write_tiny(name, str(root / name)) for name in TINY}


def pytest_terminal_summary(terminalreporter):
    import helpers
    if helpers.REPORT:
        terminalreporter.write_line("bfloat16 against what rounding alone costs (pooled rms ratio, bound %.2f; worst row, "
                                    "bound %.1f; worst single value, bound %.0f):"
                                    % (helpers.RMS_SLACK, helpers.ROW_SLACK, helpers.MAX_SLACK))
        for what, rows, ratio, row, value in helpers.REPORT:
            terminalreporter.write_line("  %-60s %6d rows  %.3f  %.2f  %.2f" % (what, rows, ratio, row, value))
