"""SwiGLU feed-forward (gpt-fast model.py:219-227): w2(silu(w1 x) * w3 x).

w1 (gate) and w3 (up) are stored as one matrix whose rows alternate gate, up,
so that one product yields both and its epilogue applies silu(gate) * up
before anything is written; the second product adds into the residual."""
import torch

from .. import ops
from ..weights.loader import ParamSpec
from . import register_feed_forward
from .residual import as_residual


@register_feed_forward("swiglu")
class SwiGLU:
    def __init__(self, dim: int, hidden: int, dtype: torch.dtype):
        self.dim, self.hidden, self.dtype = dim, hidden, dtype
        self.w13 = self.w2 = None

    def param_specs(self):
        return {"w1": ParamSpec((self.hidden, self.dim)), "w3": ParamSpec((self.hidden, self.dim)),
                "w2": ParamSpec((self.dim, self.hidden))}

    def load(self, tensors):
        self.w13 = torch.stack([tensors["w1"], tensors["w3"]], dim=1).reshape(2 * self.hidden, self.dim).contiguous()
        self.w2 = tensors["w2"]

    def export(self):
        """The parameters as `load` received them (gate and up rows taken apart again)."""
        w = self.w13.view(self.hidden, 2, self.dim)
        return {"w1": w[:, 0], "w3": w[:, 1], "w2": self.w2}

    def forward(self, h, residual):
        act = torch.empty(h.shape[0], self.hidden, dtype=self.dtype, device=h.device)
        ops.linear(h, self.w13, act, mode="swiglu")
        as_residual(residual).add_linear(act, self.w2)
