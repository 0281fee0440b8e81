import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """Model folders (config.json + model.safetensors, bfloat16-rounded values) of the tiny
    configurations, made once per session in a temporary folder."""
    import helpers
    root = tmp_path_factory.mktemp("models")
    return {name: helpers.make_folder(str(root / name), name) for name in helpers.TINY}


@pytest.fixture
def cpu_ops(monkeypatch):
    """The plain PyTorch operations in the place of the CUDA kernels (host-logic tests only)."""
    import ref_ops
    ref_ops.install(monkeypatch)
