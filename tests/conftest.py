import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """name -> folder with config.json + model.safetensors for each tiny configuration."""
    import tiny_models
    base = tmp_path_factory.mktemp("models")
    return {name: tiny_models.make_model_dir(str(base / name), name) for name in tiny_models.CONFIGS}
