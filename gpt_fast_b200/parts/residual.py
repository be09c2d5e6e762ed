"""The residual stream of a step: the float32 running sum x [T, dim] plus,
possibly, partial sums that are still owed to it.

A product whose sum over K was split across blocks leaves its result as a few
partial sums.  Instead of a kernel that only adds them up, the stream keeps
them `pending` and the next kernel that reads x completes the sum on its way:
RMSNorm does (it reads every element of x anyway), so split reduction, residual
add and norm are one pass.  Parts use

    residual.add_linear(a, w)    x += a @ w.T   (fused into the product's epilogue, or deferred)
    residual.add(y)              x += y         (for parts that cannot fuse)
    residual.tensor()            x, complete
"""
import torch

from .. import ops


class Residual:
    def __init__(self, x: torch.Tensor):
        self.x = x
        self.pending = None

    def resolve(self) -> None:
        if self.pending is not None:
            ops.add_partials(self.x, self.pending)
            self.pending = None

    def tensor(self) -> torch.Tensor:
        self.resolve()
        return self.x

    def add_linear(self, a, w) -> None:
        self.resolve()
        self.pending = ops.linear(a, w, self.x, mode="add", defer=True)

    def add(self, y) -> None:
        self.resolve()
        ops.add_into(self.x, y)

    def take_pending(self):
        p, self.pending = self.pending, None
        return p


def as_residual(x) -> "Residual":
    return x if isinstance(x, Residual) else Residual(x)
