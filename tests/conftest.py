import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

os.environ.setdefault("AWEX_LOG_LEVEL", "WARNING")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200 box)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="module", autouse=True)
def _interpreter_paths_are_left_alone():
    """Ranks that later tests start with ``spawn`` inherit ``sys.path``: a test
    module that leaves one of this repository's directories behind (the stand-in
    packages under ``baseline/``, say) changes what those ranks import."""

    def ours():
        return [p for p in sys.path if os.path.abspath(p).startswith(ROOT)]

    before = ours()
    yield
    assert ours() == before, f"a test module left sys.path changed: {before} -> {ours()}"
