"""Choosing the next token from float32 logits, on the device.

gpt-fast's `sample` (generate.py:40-57): logits / max(temperature, 1e-5),
optional top-k by pivot (ties with the k-th value are kept), softmax, then the
exponential race argmax(p / q) with q ~ Exp(1), which needs no host
synchronisation.  gpt-fast has no exact greedy branch (temperature 0 means
"divide by 1e-5"); here temperature 0 is a plain argmax, lowest index on ties.
The noise is keyed by (seed, request id, token index), never by the row's
place in a batch, so a request draws the same tokens alone or in any batch.
"""
from dataclasses import dataclass
from typing import Optional

import torch

from .. import ops


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.8          # gpt-fast's command-line default (generate.py:457)
    top_k: Optional[int] = 200        # gpt-fast's command-line default (generate.py:456)
    seed: int = 1234                  # gpt-fast seeds the global generator with 1234 (generate.py:330)

    @property
    def greedy(self) -> bool:
        return self.temperature == 0


def sample(logits: torch.Tensor, temperature: float = 1.0, top_k: Optional[int] = None, *, seed: int = 0,
           request_ids: Optional[torch.Tensor] = None, token_index: Optional[torch.Tensor] = None,
           index_map: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
           seed_dev: Optional[torch.Tensor] = None) -> torch.Tensor:
    """logits float32 [B, V] -> token ids int32 [B].

    request_ids (int64 [B]) and token_index (int32; row b uses
    token_index[index_map[b]] if index_map is given, else token_index[b]) key
    the noise; without them rows use their index and 0."""
    if logits.dim() != 2:
        raise ValueError(f"logits must be [batch, vocab], got {tuple(logits.shape)}")
    if temperature < 0:
        raise ValueError("temperature must not be negative")
    if top_k is not None and top_k < 1:
        raise ValueError("top_k must be at least 1")
    if out is None:
        out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
    if temperature == 0:
        ops.argmax(logits, out)
    else:
        ops.sample(logits, out, temperature, top_k, seed, request_ids, token_index, index_map, seed_dev=seed_dev)
    return out
