import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """name -> folder with config.json + model.safetensors (bfloat16 storage) for the tiny configs."""
    from pulse_infer_b200.weights import write_random_model
    from tiny_configs import CONFIGS, SEEDS
    out = {}
    for name, cfg in CONFIGS.items():
        folder = str(tmp_path_factory.mktemp(f"tiny_{name}"))
        write_random_model(cfg, SEEDS[name], folder, dtype="bfloat16")
        out[name] = folder
    return out
