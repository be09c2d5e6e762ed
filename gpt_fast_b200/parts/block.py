"""Arrangements of a layer's parts.  'prenorm' is gpt-fast's TransformerBlock
(model.py:153-164): x += mixer(norm(x)); x += feed_forward(norm(x)), with the
residual stream x kept in 32-bit."""
import torch

from . import register_block
from .residual import as_residual


@register_block("prenorm")
class PreNormBlock:
    def __init__(self, mixer, feed_forward, mixer_norm, ffn_norm, dim: int, dtype: torch.dtype):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.ffn_norm = mixer_norm, ffn_norm
        self.dim, self.dtype = dim, dtype

    def parts(self):
        return {"mixer": self.mixer, "feed_forward": self.feed_forward,
                "mixer_norm": self.mixer_norm, "ffn_norm": self.ffn_norm}

    def forward(self, x, batch, view, append: bool = True):
        """x: the residual stream (`parts.residual.Residual`), updated in place."""
        x = as_residual(x)
        h = torch.empty(x.x.shape[0], self.dim, dtype=self.dtype, device=x.x.device)
        self.mixer_norm.forward(x, h)
        self.mixer.forward(h, batch, view, residual=x, append=append)
        self.ffn_norm.forward(x, h)
        self.feed_forward.forward(h, residual=x)
