import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    # files named test_zz_* run last, whatever the collection order was
    items.sort(key=lambda it: 1 if os.path.basename(str(it.fspath)).startswith("test_zz_") else 0)


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """Model folders of the tiny configurations, written once with random weights."""
    import helpers

    out = {}
    for name in helpers.CONFIGS:
        d = tmp_path_factory.mktemp(f"model_{name}")
        helpers.write_model(str(d), helpers.CONFIGS[name], seed=helpers.SEEDS[name])
        out[name] = str(d)
    return out
