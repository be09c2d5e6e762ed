"""RMSNorm (gpt-fast model.py:230-241): x * rsqrt(mean(x^2) + eps) * weight,
with the statistics and the products in 32-bit."""
import torch

from .. import ops
from ..weights.loader import ParamSpec
from . import register_norm
from .residual import Residual


@register_norm("rmsnorm")
class RMSNorm:
    def __init__(self, dim: int, eps: float, dtype: torch.dtype):
        self.dim, self.eps, self.dtype = dim, float(eps), dtype
        self.weight = None

    def param_specs(self):
        return {"weight": ParamSpec((self.dim,), "vector")}

    def load(self, tensors):
        self.weight = tensors["weight"]

    def export(self):
        return {"weight": self.weight}

    def forward(self, x, out, rows=None):
        """x: the residual stream (a `Residual`, or a complete float32 tensor
        [T, dim]) -> out [R, dim] in the compute dtype; `rows` (int32 [R]) picks
        input rows, else R = T.  Partial sums pending on the stream are added
        by the same kernel."""
        if isinstance(x, Residual):
            ops.rmsnorm(x.x, self.weight, self.eps, out, rows, x.take_pending())
        else:
            ops.rmsnorm(x, self.weight, self.eps, out, rows)
        return out
