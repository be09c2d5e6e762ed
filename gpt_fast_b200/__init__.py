"""gpt_fast_b200: a small single-GPU generation library for the Llama 2/3 dense
decoder on NVIDIA B200 (sm_100a), after what pytorch-labs/gpt-fast shows.

    import gpt_fast_b200 as gf
    model = gf.load("path/to/model_folder", dtype="bfloat16")
    sequences, stats = gf.generate(model, [[1, 5, 9], [1, 7]], max_new_tokens=32, temperature=0.0)
"""
from . import architectures  # noqa: F401  (registers the architectures)
from .config.args import ConfigError, ModelArgs
from .config.registry import architectures as architecture_names, config_from_name, named_configs
from .engine.generate import generate
from .engine.load import load
from .engine.model import Transformer
from .engine.step import DecodeBatch, Stepper
from .sampling import SamplingParams, sample
from .weights.loader import WeightError
from .weights.random_init import save_folder, write_model_folder

__all__ = ["load", "generate", "sample", "SamplingParams", "Transformer", "Stepper", "DecodeBatch", "ModelArgs",
           "ConfigError", "WeightError", "write_model_folder", "save_folder", "named_configs", "config_from_name",
           "architecture_names"]
