"""Data that describes a model to build: which parts, with which sizes and
constants, in which order.

Nothing here knows an architecture.  An architecture (see `registry.py`)
turns its typed configuration into a `ModelSpec`; `engine.model.Transformer`
builds itself from the spec alone.  Every size a part needs is in its
`PartSpec.params`; the order in which layers run is the `schedule` list.
"""
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


@dataclass(frozen=True)
class PartSpec:
    """One part: `kind` is a key of the matching registry in `parts`, `params`
    are the constructor's keyword arguments (sizes and constants only)."""
    kind: str
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One set of layer parameters.  `block` names the arrangement of the
    parts (for instance pre-norm residual); `parts` gives one `PartSpec` per
    role the arrangement declares (`parts.BLOCKS[block].roles`: for 'prenorm'
    mixer, feed_forward, mixer_norm, ffn_norm), so an arrangement with other
    roles (one shared norm, post-norms, no feed-forward) needs no change here.
    Each layer picks its own parts, so layers of one model may differ."""
    block: str
    parts: Dict[str, PartSpec]
    position: Optional[PartSpec] = None   # position encoding the layer's mixers apply


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  `layer` indexes `ModelSpec.layers` (a layer may be
    named by several entries: its weights are then shared).  `cache` is the id
    of the cache entry the run's mixer uses; with `owns_cache=False` the run
    appends nothing and reads what the entry's owner wrote earlier in the
    same step."""
    layer: int
    cache: int
    owns_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    dim: int
    vocab_size: int
    layers: List[LayerSpec]
    schedule: List[ScheduleEntry]
    final_norm: PartSpec
    tie_embeddings: bool = False
    max_position: int = 0                 # longest sequence the model allows
    stop_tokens: tuple = ()               # default stop tokens of generation
    bos_token: Optional[int] = None
    embed_scale: Optional[float] = None   # factor on the embedding rows (None: 1)
    logit_cap: Optional[float] = None     # soft cap on the logits, cap * tanh(logits / cap) (None: none)

    def validate(self) -> None:
        if self.logit_cap is not None and not self.logit_cap > 0:
            raise ValueError(f"ModelSpec.logit_cap = {self.logit_cap}: a soft cap must be positive")
        if self.embed_scale is not None and self.embed_scale != self.embed_scale:
            raise ValueError("ModelSpec.embed_scale is not a number")
        owners = {}
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"schedule[{i}] names layer {e.layer}, the model has {len(self.layers)}")
            if e.owns_cache:
                if e.cache in owners:
                    raise ValueError(f"cache entry {e.cache} has two owners: schedule[{owners[e.cache]}] and [{i}]")
                owners[e.cache] = i
            elif e.cache not in owners:
                raise ValueError(f"schedule[{i}] reads cache entry {e.cache} before any run wrote it")
