"""What a mixer asks of the cache for one run of its layer."""
from dataclasses import dataclass
from typing import Optional, Tuple

import torch


@dataclass(frozen=True)
class KVNeed:
    """Keys and values per token: n_kv heads of head_dim.  `window` (or None)
    is how many of the latest positions the mixer ever reads."""
    n_kv: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """Per-sequence state of fixed size, zero when a sequence starts."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass(frozen=True)
class CacheNeeds:
    kv: Optional[KVNeed] = None
    state: Optional[StateNeed] = None
