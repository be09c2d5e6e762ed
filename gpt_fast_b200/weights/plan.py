"""The plan that ties checkpoint tensor names to a model's parameters.

An architecture writes one `Recipe` per model parameter: which checkpoint
tensors it is made of (name, shape, how random weights are drawn for it) and
how they are combined.  The loader, the random-weights writer and the error
report all work from the plan, so none of them knows an architecture.
"""
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple


@dataclass(frozen=True)
class Source:
    """One tensor of the checkpoint.  `init` says how the random-weights mode
    draws it: 'normal' = N(0, std), 'norm' = 1 + N(0, jitter)."""
    name: str
    shape: Tuple[int, ...]
    init: str = "normal"


@dataclass(frozen=True)
class Recipe:
    """Model parameter `target` = combine(*sources).  `combine=None` takes the
    only source as it is.  `split` is the way back, for writing a model out:
    split(target tensor) -> the source tensors in order (None with `combine=None`:
    the tensor itself; a recipe with a `combine` and no `split` cannot be written)."""
    target: str
    sources: Sequence[Source]
    combine: Optional[Callable] = None
    split: Optional[Callable] = None


@dataclass
class WeightPlan:
    recipes: List[Recipe]
    # model parameters that are another parameter's storage (tied output):
    aliases: Dict[str, str] = field(default_factory=dict)
    # checkpoint names that may be present and are dropped (regular expressions)
    ignored: Tuple[str, ...] = ()
    # checkpoint names that must NOT be present, with the reason
    forbidden: Dict[str, str] = field(default_factory=dict)

    def sources(self) -> Dict[str, Source]:
        out = {}
        for r in self.recipes:
            for s in r.sources:
                if s.name in out and out[s.name].shape != s.shape:
                    raise ValueError(f"plan names '{s.name}' with two shapes")
                out[s.name] = s
        return out
