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


# Sharpened weights give attention scores a standard deviation of ``score_std`` instead of
# nearly zero.  The 32-bit runs use 3.0, where a wrong key or page changes logits by far more
# than the gate.  Keys, values and activations of the bfloat16 path carry a relative
# rounding error of 2^-9, and a score's absolute error grows with its size; those runs use 1.5
# so that honest bfloat16 rounding stays small while attention is still far from uniform.
SHARPNESS = {"float32": dict(score_std=3.0), "bfloat16": dict(score_std=1.5)}


class _Sharp:
    def __init__(self, tiny_models, root):
        self.tiny_models, self.root, self.made = tiny_models, root, {}

    def get(self, name, dtype):
        if (name, dtype) not in self.made:
            import helpers

            self.made[name, dtype] = helpers.sharpen(self.tiny_models[name], self.root / dtype / name,
                                                     **SHARPNESS[dtype])
        return self.made[name, dtype]


@pytest.fixture(scope="session")
def sharp_models(tiny_models, tmp_path_factory):
    return _Sharp(tiny_models, tmp_path_factory.mktemp("sharp"))


def pytest_terminal_summary(terminalreporter):
    """Worst logits error seen per configuration and dtype (in standard deviations of the reference
    logits): the figures the gates in helpers.py are set from."""
    import helpers

    if helpers.WORST:
        terminalreporter.write_line("worst logits error / std(reference logits):")
        for (label, dtype), error in sorted(helpers.WORST.items()):
            terminalreporter.write_line(f"  {label:24s} {dtype:9s} {error:.3e}  (gate {helpers.tolerance(dtype, label):.1e})")
