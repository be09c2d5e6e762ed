"""Weights by tensor name, from safetensors or from a seed.

gpt-fast converts a checkpoint offline (scripts/convert_hf_checkpoint.py) and
then loads a flat state dict strictly (generate.py:238-241).  Here the model
folder's safetensors are read directly, by the names of an architecture's
`WeightPlan`; everything that is wrong with a checkpoint is reported in ONE
`WeightError` that lists missing tensors, unexpected tensors and wrong shapes.

Precision: a matrix is kept in the model's compute dtype (bfloat16 for
serving; a 32-bit run widens bfloat16 exactly).  A vector (norm weights) that
is stored in 32-bit stays 32-bit also in a bfloat16 model.  Integer tables
become int32.
"""
import json
import os
import re
import zlib
from dataclasses import dataclass
from typing import Dict, Tuple

import torch

from .plan import WeightPlan

ROLES = ("matrix", "vector", "table")


class WeightError(ValueError):
    """A checkpoint that does not fit the model.  `missing`, `unexpected` and
    `wrong_shape` hold the details that the message lists."""

    def __init__(self, where, missing=(), unexpected=(), wrong_shape=(), other=()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.other = list(other)
        lines = [f"weights at {where} do not fit the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, want, found in self.wrong_shape:
            lines.append(f"  wrong shape: {name} expected {tuple(want)}, found {tuple(found)}")
        lines += [f"  {o}" for o in self.other]
        super().__init__("\n".join(lines))


@dataclass(frozen=True)
class ParamSpec:
    """A model parameter as a part declares it."""
    shape: Tuple[int, ...]
    role: str = "matrix"


class SafetensorsCheckpoint:
    """The tensors of a model folder: `model.safetensors.index.json` with its
    shards if present, else the single `model.safetensors`."""

    def __init__(self, folder):
        from safetensors import safe_open
        self.where = os.fspath(folder)
        index = os.path.join(self.where, "model.safetensors.index.json")
        single = os.path.join(self.where, "model.safetensors")
        if os.path.isfile(index):
            with open(index) as f:
                files = sorted(set(json.load(f)["weight_map"].values()))
        elif os.path.isfile(single):
            files = ["model.safetensors"]
        else:
            raise WeightError(self.where, other=["no model.safetensors or model.safetensors.index.json in the folder"])
        self._file_of: Dict[str, str] = {}
        self._shapes: Dict[str, Tuple[int, ...]] = {}
        duplicates = []
        for fn in files:
            path = os.path.join(self.where, fn)
            if not os.path.isfile(path):
                raise WeightError(self.where, other=[f"the index names shard {fn}, which is not in the folder"])
            with safe_open(path, framework="pt") as f:
                for k in f.keys():
                    if k in self._file_of:
                        duplicates.append(f"{k} is in both {self._file_of[k]} and {fn}")
                    self._file_of[k] = path
                    self._shapes[k] = tuple(f.get_slice(k).get_shape())
        if duplicates:
            raise WeightError(self.where, other=duplicates)
        self._open = {}

    def shapes(self) -> Dict[str, Tuple[int, ...]]:
        return self._shapes

    def get(self, name: str, device="cpu") -> torch.Tensor:
        from safetensors import safe_open
        path = self._file_of[name]
        if path not in self._open:
            self._open[path] = safe_open(path, framework="pt")
        return self._open[path].get_tensor(name).to(device)


def _tensor_seed(seed: int, name: str) -> int:
    return (int(seed) * 1000003 + zlib.crc32(name.encode())) % (2 ** 63 - 1)


class RandomCheckpoint:
    """Seeded random tensors under the plan's checkpoint names: every matrix
    N(0, std), every norm weight 1 + N(0, jitter).  Each tensor has a random
    stream of its own, keyed by (seed, name), so the values do not depend on
    the order of reading.  Values are drawn in 32-bit on `gen_device` and
    rounded to the storage dtype."""

    def __init__(self, plan: WeightPlan, seed: int, std=0.02, jitter=0.1, matrix_dtype=torch.bfloat16,
                 vector_dtype=torch.bfloat16, gen_device="cpu"):
        self.where = f"random weights (seed {seed})"
        self._sources = plan.sources()
        self.seed, self.std, self.jitter = seed, std, jitter
        self.matrix_dtype, self.vector_dtype, self.gen_device = matrix_dtype, vector_dtype, gen_device

    def shapes(self):
        return {k: s.shape for k, s in self._sources.items()}

    def get(self, name: str, device="cpu") -> torch.Tensor:
        s = self._sources[name]
        g = torch.Generator(device=self.gen_device).manual_seed(_tensor_seed(self.seed, name))
        x = torch.randn(s.shape, generator=g, device=self.gen_device, dtype=torch.float32)
        if s.init == "norm":
            x = (1.0 + x * self.jitter).to(self.vector_dtype)
        else:
            x = (x * self.std).to(self.matrix_dtype)
        return x.to(device)


def check_plan(plan: WeightPlan, ckpt) -> None:
    """Raise one WeightError that lists everything wrong with `ckpt`."""
    have = ckpt.shapes()
    want = plan.sources()
    ignored = [re.compile(p) for p in plan.ignored]
    missing = [n for n in want if n not in have]
    wrong = [(n, want[n].shape, have[n]) for n in want if n in have and tuple(have[n]) != tuple(want[n].shape)]
    unexpected, other = [], []
    for n in have:
        if n in want or any(p.fullmatch(n) for p in ignored):
            continue
        if n in plan.forbidden:
            other.append(f"{n} is present, but {plan.forbidden[n]}")
        else:
            unexpected.append(n)
    if missing or wrong or unexpected or other:
        raise WeightError(ckpt.where, sorted(missing), sorted(unexpected), wrong, other)


def _store(t: torch.Tensor, role: str, dtype: torch.dtype) -> torch.Tensor:
    if role == "table":
        if t.dtype.is_floating_point:
            raise ValueError("an integer table is stored as floating point")
        return t.to(torch.int32)
    if not t.dtype.is_floating_point:
        raise ValueError(f"a floating-point parameter is stored as {t.dtype}")
    if role == "vector" and t.dtype == torch.float32:
        return t                       # stored in 32-bit: stays so
    return t.to(dtype)


def load_parameters(plan: WeightPlan, ckpt, specs: Dict[str, ParamSpec], dtype: torch.dtype,
                    device="cpu", progress=None) -> Dict[str, torch.Tensor]:
    """Build every model parameter the plan names.  `specs` are the model's own
    declarations (shape and role by parameter name): the plan must fill each of
    them, with the declared shape."""
    check_plan(plan, ckpt)
    targets = {r.target for r in plan.recipes} | set(plan.aliases)
    unfilled = sorted(set(specs) - targets)
    extra = sorted(targets - set(specs))
    if unfilled or extra:
        raise WeightError(ckpt.where, other=[f"the weight plan fills no model parameter {unfilled}" if unfilled else "",
                                             f"the weight plan names parameters the model lacks: {extra}" if extra else ""])
    out: Dict[str, torch.Tensor] = {}
    bad = []
    for i, r in enumerate(plan.recipes):
        parts = [ckpt.get(s.name, device) for s in r.sources]
        t = r.combine(*parts) if r.combine is not None else parts[0]
        spec = specs[r.target]
        if tuple(t.shape) != tuple(spec.shape):
            bad.append((r.target, spec.shape, t.shape))
            continue
        try:
            out[r.target] = _store(t, spec.role, dtype).contiguous()
        except ValueError as e:
            raise WeightError(ckpt.where, other=[f"{r.target}: {e}"]) from None
        if progress is not None:
            progress(i + 1, len(plan.recipes))
    if bad:
        raise WeightError(ckpt.where, wrong_shape=bad)
    for alias, target in plan.aliases.items():
        out[alias] = out[target]
    return out
