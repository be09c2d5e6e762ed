"""From a model folder (or a named size and a seed) to a model on the device.

gpt-fast's `_load_model` (generate.py:219-249) picks the size by the
checkpoint's directory name and loads a converted `model.pth`; here the
folder's config.json picks the architecture and the sizes, and the folder's
safetensors are read by name."""
import os
from typing import Optional, Union

import torch

from ..config.registry import architecture_for, config_from_name, read_config
from ..weights.loader import RandomCheckpoint, SafetensorsCheckpoint, load_parameters
from .model import Transformer, compute_dtype


def load(source: Union[str, os.PathLike, dict], dtype="bfloat16", device="cuda", *, random_weights: bool = False,
         seed: int = 0, n_layers: Optional[int] = None, progress=None) -> Transformer:
    """source: a model folder (config.json + safetensors), or, with
    random_weights=True, a folder with only config.json, a config dict, or the
    name of a named size (`config.registry.named_configs()`).
    n_layers: build only the first n layers (for measurements on less memory;
    only with random weights)."""
    if isinstance(source, dict):
        cfg, folder = dict(source), None
    elif os.path.isdir(os.fspath(source)):
        cfg, folder = read_config(source), os.fspath(source)
    elif random_weights:
        cfg, folder = config_from_name(os.fspath(source)), None
    else:
        raise FileNotFoundError(f"{source} is not a model folder")
    if n_layers is not None:
        if not random_weights:
            raise ValueError("n_layers needs random_weights=True")
        cfg["num_hidden_layers"] = n_layers
    arch = architecture_for(cfg)
    args = arch.parse(cfg)
    spec = arch.build_spec(args)
    plan = arch.weight_plan(args)
    dt = compute_dtype(dtype)
    model = Transformer(spec, dt, device)
    if random_weights:
        dev = torch.device(device)
        ckpt = RandomCheckpoint(plan, seed, gen_device=dev if dev.type == "cuda" else "cpu")
    else:
        ckpt = SafetensorsCheckpoint(folder)
    params = load_parameters(plan, ckpt, model.param_specs(), dt, device, progress)
    model.load_params(params)
    model.args = args
    model.config = cfg                     # the config.json it was built from
    model.weight_plan = plan
    return model
