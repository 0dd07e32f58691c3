import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
if os.path.dirname(os.path.abspath(__file__)) not in sys.path:
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """Model folders (config.json, model.safetensors) of the tiny configurations, made once a session
    in a temporary folder: {name: (folder, float32 folder, page size)}."""
    import torch
    from configs import CONFIGS
    from llmx_b200.config import Qwen3Config
    from llmx_b200.weights import write_random_model

    out = {}
    for name, (cfg, seed, page) in CONFIGS.items():
        c = Qwen3Config.from_dict(cfg)
        d16 = str(tmp_path_factory.mktemp(f"tiny_{name}_bf16"))
        d32 = str(tmp_path_factory.mktemp(f"tiny_{name}_f32"))
        write_random_model(d16, c, seed, dtype=torch.bfloat16)
        write_random_model(d32, c, seed, dtype=torch.float32)
        out[name] = (d16, d32, page)
    return out
