import os
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
# the reference checkout used as an oracle: $GHB_REFERENCE_PATH, else a `reference` folder beside this repository
REFERENCE = Path(os.environ.get("GHB_REFERENCE_PATH") or ROOT.parent / "reference") / "code"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")
    config.addinivalue_line("markers", "multigpu: needs at least 2 CUDA devices")


def pytest_collection_modifyitems(config, items):
    have = torch.cuda.is_available()
    n = torch.cuda.device_count() if have else 0
    for item in items:
        if "gpu" in item.keywords and not have:
            item.add_marker(pytest.mark.skip(reason="no CUDA device"))
        if "multigpu" in item.keywords and n < 2:
            item.add_marker(pytest.mark.skip(reason="needs 2 CUDA devices"))


@pytest.fixture
def reference():
    """The mounted reference implementation as an importable oracle (skipped where it is not mounted)."""
    if not (REFERENCE / "ced").is_dir():
        pytest.skip("reference implementation not mounted")
    if str(REFERENCE) not in sys.path:
        sys.path.append(str(REFERENCE))
    import ced  # noqa: F401

    return ced


@pytest.fixture(autouse=True)
def _seed():
    torch.manual_seed(1234)
    yield
