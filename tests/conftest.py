import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")
    # the fp32 oracle's matmuls must stay fp32: no TF32, whatever the environment says
    import torch
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    os.environ.pop("NVIDIA_TF32_OVERRIDE", None)
    os.environ["TORCH_ALLOW_TF32_CUBLAS_OVERRIDE"] = "0"


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)


@pytest.fixture(scope="session")
def ext():
    """The in-tree CUDA extension; a GPU test that cannot load it fails (no PyTorch fallback)."""
    from ferrite_b200._ext import load
    return load()
