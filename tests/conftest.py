import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
for p in (str(ROOT), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a)")


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """Model folders (config.json, model.safetensors) of the tiny configurations with seeded
    random weights, made in a temporary folder."""
    from configs import CONFIGS, SEED
    from scratch_llm_b200.config import config_from_dict
    from scratch_llm_b200.weights import write_random_model

    out = {}
    for name, raw in CONFIGS.items():
        d = tmp_path_factory.mktemp(f"tiny_{name}")
        write_random_model(config_from_dict(raw), d, SEED[name])
        out[name] = d
    return out
