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
    from tiny_configs import CONFIGS, QUERY_NORM_SCALE, SEEDS
    out = {}
    for name, cfg in CONFIGS.items():
        folder = str(tmp_path_factory.mktemp(f"tiny_{name}"))
        write_random_model(cfg, SEEDS[name], folder, dtype="bfloat16")
        if name in QUERY_NORM_SCALE:
            sharpen_queries(folder, QUERY_NORM_SCALE[name])
        out[name] = folder
    return out


def sharpen_queries(folder, scales):
    """Rewrite ``model.safetensors`` of ``folder`` with layer i's q_norm weight multiplied by ``scales[i]``."""
    import os
    from pulse_infer_b200.weights import SafetensorsFile, write_safetensors
    path = os.path.join(folder, "model.safetensors")
    f = SafetensorsFile(path)
    tensors = {n: f.tensor(n).clone() for n in f.names()}
    del f
    for layer, scale in enumerate(scales):
        name = f"model.layers.{layer}.self_attn.q_norm.weight"
        tensors[name] = (tensors[name].float() * scale).to(tensors[name].dtype)
    write_safetensors(path, tensors)
