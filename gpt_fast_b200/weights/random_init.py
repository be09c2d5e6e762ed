"""Random-weights mode: write a model folder (config.json, model.safetensors)
from a configuration and a seed.

gpt-fast has no such mode (it needs downloaded checkpoints,
scripts/download.py); tests and benchmarks here need models without a network.
The folder is an ordinary model folder: the loader reads it like any other.
"""
import json
import os
from typing import Any, Dict, Union

import torch

from ..config.registry import architecture_for, config_from_name
from .loader import RandomCheckpoint

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}


def write_model_folder(folder, config: Union[str, Dict[str, Any]], seed: int, *, std: float = 0.02,
                       jitter: float = 0.1, matrix_dtype="bfloat16", vector_dtype="bfloat16",
                       gen_device="cpu") -> str:
    """Write `folder/config.json` and `folder/model.safetensors`.

    config: a config.json dict, or the name of a named size.
    matrix_dtype / vector_dtype: storage of matrices / of norm weights
    ('bfloat16' or 'float32')."""
    from safetensors.torch import save_file
    cfg = config_from_name(config) if isinstance(config, str) else dict(config)
    arch = architecture_for(cfg)
    args = arch.parse(cfg)
    plan = arch.weight_plan(args)
    ckpt = RandomCheckpoint(plan, seed, std, jitter, _DTYPES[matrix_dtype], _DTYPES[vector_dtype], gen_device)
    os.makedirs(folder, exist_ok=True)
    tensors = {name: ckpt.get(name, "cpu").contiguous() for name in ckpt.shapes()}
    save_file(tensors, os.path.join(folder, "model.safetensors"), metadata={"format": "pt"})
    out = args.to_json() if hasattr(args, "to_json") else cfg
    out["torch_dtype"] = matrix_dtype
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(out, f, indent=1)
    return os.fspath(folder)


def save_folder(model, folder) -> str:
    """Write a loaded model back as a model folder: config.json and model.safetensors with the checkpoint's
    own tensor names and layouts (for Llama the q/k rows go back from interleaved to half-split rotary pairs,
    the inverse of what gpt-fast's converter does, scripts/convert_hf_checkpoint.py:75-81).  Loading the folder
    gives the same parameters bit for bit.  The model must come from `load` (it carries its config and plan)."""
    from safetensors.torch import save_file
    plan, cfg = getattr(model, "weight_plan", None), getattr(model, "config", None)
    if plan is None or cfg is None:
        raise ValueError("save_folder needs a model made by load(): it carries the weight plan and the configuration")
    params = model.export_params()
    tensors = {}
    for r in plan.recipes:
        t = params[r.target]
        if r.combine is None:
            pieces = [t]
        elif r.split is not None:
            pieces = r.split(t)
        else:
            raise ValueError(f"the weight plan combines tensors into {r.target} but names no way back (Recipe.split)")
        if len(pieces) != len(r.sources):
            raise ValueError(f"{r.target}: split gave {len(pieces)} tensors for {len(r.sources)} sources")
        for src, piece in zip(r.sources, pieces):
            if tuple(piece.shape) != tuple(src.shape):
                raise ValueError(f"{src.name}: split gave shape {tuple(piece.shape)}, the plan says {tuple(src.shape)}")
            tensors[src.name] = piece.detach().to("cpu").contiguous()
    os.makedirs(folder, exist_ok=True)
    save_file(tensors, os.path.join(folder, "model.safetensors"), metadata={"format": "pt"})
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(dict(cfg), f, indent=1)
    return os.fspath(folder)
