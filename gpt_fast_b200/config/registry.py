"""One registry from an architecture's name to what builds its model, and a
table of named sizes for runs without a model folder.

gpt-fast keeps a dict of named sizes and picks one by the checkpoint's
directory name (model.py:44-82).  Here config.json decides: its `model_type`
(or `architectures[0]`) names an `Architecture`; the named sizes are stored as
config.json files under `config/named/` and go through the same parser, so no
size stands in code.
"""
import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, List

from .args import ConfigError

NAMED_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "named")


@dataclass(frozen=True)
class Architecture:
    """What the library needs to know about one architecture.

    parse:        config.json dict -> typed configuration
    build_spec:   typed configuration -> config.spec.ModelSpec
    weight_plan:  typed configuration -> weights.plan.WeightPlan (tensor names)
    """
    name: str
    parse: Callable[[Dict[str, Any]], Any]
    build_spec: Callable[[Any], Any]
    weight_plan: Callable[[Any], Any]
    aliases: tuple = ()


_ARCHITECTURES: Dict[str, Architecture] = {}


def register_architecture(arch: Architecture) -> Architecture:
    for key in (arch.name,) + tuple(arch.aliases):
        if key in _ARCHITECTURES and _ARCHITECTURES[key] is not arch:
            raise ValueError(f"architecture name '{key}' is already registered")
        _ARCHITECTURES[key] = arch
    return arch


def architectures() -> List[str]:
    return sorted(_ARCHITECTURES)


def architecture_for(cfg: Dict[str, Any]) -> Architecture:
    """Choose the architecture a config.json dict names."""
    keys = []
    if cfg.get("model_type"):
        keys.append(cfg["model_type"])
    keys += list(cfg.get("architectures") or [])
    for k in keys:
        if k in _ARCHITECTURES:
            return _ARCHITECTURES[k]
    raise ConfigError(f"config.json names architecture {keys or '(none)'}; this library knows {architectures()}")


def read_config(folder_or_file) -> Dict[str, Any]:
    path = os.fspath(folder_or_file)
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json at {path}")
    with open(path) as f:
        cfg = json.load(f)
    if not isinstance(cfg, dict):
        raise ConfigError(f"{path} must hold one JSON object")
    return cfg


def named_configs() -> List[str]:
    return sorted(f[:-5] for f in os.listdir(NAMED_DIR) if f.endswith(".json"))


def config_from_name(name: str) -> Dict[str, Any]:
    """The config.json of a named size.  As gpt-fast's `ModelArgs.from_name`
    (model.py:44-57): an exact name wins; else every registered name that occurs
    in `name` (case-insensitive) is a candidate and the longest one wins; two
    longest candidates of equal length, or none at all, are an error."""
    names = named_configs()
    if name in names:
        chosen = name
    else:
        hits = sorted((n for n in names if n.lower() in str(name).lower()), key=len, reverse=True)
        if not hits:
            raise ConfigError(f"no named configuration matches '{name}'; known: {names}")
        if len(hits) > 1 and len(hits[0]) == len(hits[1]):
            raise ConfigError(f"'{name}' matches both '{hits[0]}' and '{hits[1]}'")
        chosen = hits[0]
    return read_config(os.path.join(NAMED_DIR, chosen + ".json"))
