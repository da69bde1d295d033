import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def ext():
    from scalingcontrasts_b200 import _ext

    if not _ext.available():
        pytest.skip("native extension not built")
    return _ext.native()


def pytest_sessionfinish(session, exitstatus):
    """In the bounds-checked debug build (SC_NATIVE_VARIANT=bounds) every kernel compares its computed global indices with
    their limits and records the first miss; a session that ran the GPU tests under it must end with no miss recorded."""
    if os.environ.get("SC_NATIVE_VARIANT", "") != "bounds" or not torch.cuda.is_available():
        return
    from scalingcontrasts_b200 import _ext

    if not _ext.available():
        return
    records = _ext.native().bounds_records()
    if any(word != 0 for record in records for word in record):
        print(f"\nbounds-checked build recorded an out-of-range index: {records}")
        session.exitstatus = 1
