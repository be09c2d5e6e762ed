"""Arrangements of a layer's parts.  'prenorm' is gpt-fast's TransformerBlock
(model.py:153-164): x += mixer(norm(x)); x += feed_forward(norm(x)), with the
residual stream x kept in 32-bit.

An arrangement declares `roles`: the names of the parts it is made of, each with
the kind of part that fills it ('mixer', 'feed_forward', 'norm': the registries of
`parts`).  The model builds one part per role from the layer's `LayerSpec.parts`
and hands them over as a dict; mixers also receive the layer's position encoding."""
import torch

from . import register_block
from .residual import as_residual


@register_block("prenorm")
class PreNormBlock:
    roles = {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm", "ffn_norm": "norm"}

    def __init__(self, parts: dict, dim: int, dtype: torch.dtype):
        self.mixer, self.feed_forward = parts["mixer"], parts["feed_forward"]
        self.mixer_norm, self.ffn_norm = parts["mixer_norm"], parts["ffn_norm"]
        self.dim, self.dtype = dim, dtype

    def parts(self):
        return {"mixer": self.mixer, "feed_forward": self.feed_forward,
                "mixer_norm": self.mixer_norm, "ffn_norm": self.ffn_norm}

    def cache_needs(self):
        """What one run of this layer keeps per sequence (its mixer's keys/values or state)."""
        return self.mixer.cache_needs()

    def forward(self, x, batch, view, append: bool = True):
        """x: the residual stream (`parts.residual.Residual`), updated in place."""
        x = as_residual(x)
        h = torch.empty(x.x.shape[0], self.dim, dtype=self.dtype, device=x.x.device)
        self.mixer_norm.forward(x, h)
        self.mixer.forward(h, batch, view, residual=x, append=append)
        self.ffn_norm.forward(x, h)
        self.feed_forward.forward(h, residual=x)
