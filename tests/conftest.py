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


def rms(t) -> float:
    return float(torch.as_tensor(t).float().pow(2).mean().sqrt())


def assert_within_bf16_noise(got, want, emu, where="", rms_factor=1.5, max_factor=2.0):
    """Judge bfloat16 logits `got` against the 32-bit logits `want` of the plain implementation.

    How far may bfloat16 be from 32-bit?  As far as the plain implementation itself is when its activations
    are rounded to bfloat16 where the library stores them (`emu`, from `plain_llama.forward(..., act=torch.bfloat16)`
    or a test's own restatement): that is the noise of the format on this model, measured, not guessed.  The
    library's error must stay within rms_factor x that noise in the mean and max_factor x at the worst element.
    A wrong position, head, page or key shows as an error of the order of the logits' own scale, many times the
    noise.  All three are tensors of the same shape (one row of logits, or several)."""
    got, want, emu = (torch.as_tensor(t).float() for t in (got, want, emu))
    err, noise = got - want, emu - want
    assert rms(noise) > 0, f"{where}: the emulation shows no noise at all; the check would be empty"
    assert rms(err) <= rms_factor * rms(noise), \
        f"{where}: rms error {rms(err):.5f}, bfloat16 noise {rms(noise):.5f} (logit scale {rms(want):.4f})"
    assert float(err.abs().max()) <= max_factor * float(noise.abs().max()), \
        f"{where}: max error {float(err.abs().max()):.5f}, bfloat16 noise {float(noise.abs().max()):.5f}"
