import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import gpt_fast_b200 as gf  # noqa: E402
from gpt_fast_b200 import ops  # noqa: E402
import plain_ops  # noqa: E402

# Two tiny configurations of the architecture that differ in every size and option.
TINY = {
    "tiny-a": dict(seed=11, vector_dtype="float32"),     # norm weights stored in 32-bit
    "tiny-b": dict(seed=12, vector_dtype="bfloat16"),
}


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def tiny_folders(tmp_path_factory):
    """Model folders (config.json + model.safetensors) of the tiny configurations,
    written by the library's random-weights mode into a temporary folder."""
    out = {}
    for name, kw in TINY.items():
        d = tmp_path_factory.mktemp(name.replace("-", "_"))
        gf.write_model_folder(str(d), name, kw["seed"], vector_dtype=kw["vector_dtype"])
        out[name] = str(d)
    return out


@pytest.fixture
def plain_kernels():
    """Run the library's host-side logic on the CPU against the plain statement of the kernels."""
    prev = ops.use_kernels(plain_ops.PlainOps())
    yield
    ops.use_kernels(prev)
