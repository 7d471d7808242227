import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# The reference package (installed under baseline/_ref) is the oracle of the parity tests; its
# compiled helpers are run eagerly.
os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")
REF = os.path.join(ROOT, "baseline", "_ref")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def ref_dion():
    """The reference ``dion`` package, or skip when it is not installed."""
    if not os.path.isdir(os.path.join(REF, "dion")):
        pytest.skip("reference package not installed under baseline/_ref")
    if REF not in sys.path:
        sys.path.insert(1, REF)
    import dion

    return dion
