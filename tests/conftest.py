"""Shared fixtures.  Tests that need a GPU carry ``@pytest.mark.gpu``; all
others run on a machine without one."""
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """name -> folder of a tiny random model (bf16 safetensors), made once."""
    import tiny

    base = tmp_path_factory.mktemp("models")
    return {name: tiny.write(base / name, name) for name in tiny.CONFIGS}
