"""Causal grouped-query attention with a fused q/k/v projection
(gpt-fast model.py:167-216).

Steps: qkv = h Wqkv^T; rotate q and k by each token's position, append k, v
to the sequence's place in the cache and attend over the cache (two kernels
for a prompt, one for a decode step); residual += y Wo^T.  Query head h reads key/value
head h // (n_head / n_kv); the scale is 1/sqrt(head_dim) unless given."""
import math
from typing import Optional

import torch

from .. import ops
from ..cache.needs import CacheNeeds, KVNeed
from ..weights.loader import ParamSpec
from . import register_mixer
from .residual import as_residual


@register_mixer("attention")
class Attention:
    def __init__(self, dim: int, n_head: int, n_kv: int, head_dim: int, dtype: torch.dtype, position,
                 window: Optional[int] = None, scale: Optional[float] = None):
        if n_head % n_kv:
            raise ValueError(f"{n_head} query heads do not divide into {n_kv} key/value heads")
        if position is None:
            raise ValueError("attention needs a position encoding")
        self.dim, self.n_head, self.n_kv, self.head_dim = dim, n_head, n_kv, head_dim
        self.window, self.dtype, self.position = window, dtype, position
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.wqkv = self.wo = None

    def param_specs(self):
        H, G, d, D = self.n_head, self.n_kv, self.head_dim, self.dim
        return {"wq": ParamSpec((H * d, D)), "wk": ParamSpec((G * d, D)), "wv": ParamSpec((G * d, D)),
                "wo": ParamSpec((D, H * d))}

    def load(self, tensors):
        # rows: q heads, then k heads, then v heads (gpt-fast model.py:184-189)
        self.wqkv = torch.cat([tensors["wq"], tensors["wk"], tensors["wv"]]).contiguous()
        self.wo = tensors["wo"]

    def export(self):
        """The parameters as `load` received them (the way back from the fused layout)."""
        H, G, d = self.n_head, self.n_kv, self.head_dim
        wq, wk, wv = self.wqkv.split([H * d, G * d, G * d])
        return {"wq": wq, "wk": wk, "wv": wv, "wo": self.wo}

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(kv=KVNeed(self.n_kv, self.head_dim, self.window))

    def forward(self, h, batch, view, residual, append: bool = True):
        T = batch.n_tokens
        H, G, d = self.n_head, self.n_kv, self.head_dim
        qkv = torch.empty(T, (H + 2 * G) * d, dtype=self.dtype, device=h.device)
        partials = ops.linear(h, self.wqkv, qkv, defer=True)      # a split sum is finished by the rotary kernel
        y = torch.empty(T, H * d, dtype=self.dtype, device=h.device)
        ops.rope_append_attention(qkv, partials, view.kv, batch, self.position.table, y, H, G, d, self.position.pairing,
                                  append, self.scale, self.window)
        as_residual(residual).add_linear(y, self.wo)
