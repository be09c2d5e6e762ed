"""Rotary position encoding: the frequencies (with the llama3 rescaling rule)
and the (cos, sin) table that the fused rotate-and-append kernel reads.

gpt-fast: model.py:266-278 (base frequencies, table), model.py:244-263
(llama3 rule), model.py:281-293 (rotation of interleaved pairs).  The table
is kept in 32-bit here also for a bfloat16 model (gpt-fast rounds it to the
model's dtype, model.py:278)."""
import math
from typing import Dict, Optional

import torch

from .. import ops
from . import register_position


def rope_frequencies(head_dim: int, base: float, scaling: Optional[Dict[str, float]]) -> torch.Tensor:
    """inv_freq[i] = base^(-2i/d) in 32-bit, i < d/2, then the llama3 rule:
    wavelengths shorter than original/high_freq_factor stay, longer than
    original/low_freq_factor are divided by `factor`, between them the two are
    blended linearly in original/wavelength."""
    exponent = torch.arange(0, head_dim, 2, dtype=torch.float32)[: head_dim // 2] / head_dim
    freqs = 1.0 / (base ** exponent)
    if scaling is None:
        return freqs
    factor, low, high = scaling["factor"], scaling["low_freq_factor"], scaling["high_freq_factor"]
    original = scaling["original_max_position_embeddings"]
    low_wavelen, high_wavelen = original / low, original / high
    out = torch.empty_like(freqs)
    for i in range(freqs.numel()):
        f = freqs[i]
        wavelen = 2 * math.pi / f
        if wavelen < high_wavelen:
            out[i] = f
        elif wavelen > low_wavelen:
            out[i] = f / factor
        else:
            smooth = (original / wavelen - low) / (high - low)
            out[i] = (1 - smooth) * f / factor + smooth * f
    return out


@register_position("rope")
class Rope:
    """pairing 'interleaved': pairs (2i, 2i+1); 'half': pairs (i, i + d/2)."""

    def __init__(self, head_dim: int, base: float, scaling: Optional[Dict[str, float]] = None,
                 pairing: str = "interleaved"):
        if head_dim % 2:
            raise ValueError(f"rotary pairs need an even head_dim, got {head_dim}")
        if pairing not in ("interleaved", "half"):
            raise ValueError(f"unknown rotary pairing '{pairing}'")
        self.head_dim, self.base, self.scaling, self.pairing = head_dim, float(base), scaling, pairing
        self.inv_freq = rope_frequencies(head_dim, self.base, scaling)
        self.table = None
        self._retired = []                 # earlier, shorter tables: captured decode steps may still point at them

    def prepare(self, max_positions: int, device) -> None:
        """Build the (cos, sin) table for positions 0 .. max_positions-1."""
        if self.table is not None and self.table.shape[0] >= max_positions and self.table.device == torch.device(device):
            return
        table = torch.empty(max_positions, self.head_dim // 2, 2, dtype=torch.float32, device=device)
        ops.rope_table(self.inv_freq.to(device), table)
        if self.table is not None:
            # a CUDA graph captured for an earlier cache has the old table's address and length in it; the old
            # table stays valid for as long as this part lives (a few KB to MB each, one per growth)
            self._retired.append(self.table)
        self.table = table
