import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
if str(ROOT / "tests") not in sys.path:
    sys.path.insert(0, str(ROOT / "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


@pytest.fixture(scope="session")
def tiny_models(tmp_path_factory):
    """Model folders with random weights for every tiny configuration, in a temporary folder."""
    from tiny_configs import SEED, TINY

    from cloud_inference_from_scratch_b200.weights import write_random_model

    root = tmp_path_factory.mktemp("models")
    return {
        name: write_random_model(root / name, config, SEED[name]) for name, config in TINY.items()
    }
