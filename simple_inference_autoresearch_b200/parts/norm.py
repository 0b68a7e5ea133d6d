"""RMSNorm, alone and fused with the residual add.

    y = x * rsqrt(mean(x^2) + eps) * w

with the square, mean, rsqrt and both scalings in 32-bit and one rounding on
store: the form of the reference's kernels (kernels/rmsnorm_kernel.py:99-107,
kernels/add_rmsnorm_kernel.py:86-103).  eps sits inside the square root, the
weight is used as it is (no ``1 + w``), and there is no bias.  The reference's
eager path rounds once more before the weight (ops/rmsnorm.py:41-46); that
variant is not reproduced.  Unlike the reference, the residual stream itself is
kept in 32-bit, so the fused add does not round.
"""

from __future__ import annotations

from typing import List, Mapping

import torch

from ..kernels import ops
from .base import NORMS, Norm, TensorSpec


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    def __init__(self, prefix: str, hidden_size: int, eps: float, weight_init: str = "ones",
                 weight_std: float = 0.02):
        super().__init__(prefix)
        self.hidden_size = int(hidden_size)
        self.eps = float(eps)
        self.weight_init, self.weight_std = weight_init, weight_std
        self.weight: torch.Tensor = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.prefix + "weight", (self.hidden_size,), role="vector",
                           init=self.weight_init, std=self.weight_std)]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[self.prefix + "weight"].contiguous()

    def extension_units(self, dtype=None):
        return ("elementwise",)

    def norm(self, ctx, residual: torch.Tensor) -> torch.Tensor:
        return ops.add_rmsnorm(residual, None, self.weight, self.eps, ctx.dtype)

    def add_norm(self, ctx, residual: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
        return ops.add_rmsnorm(residual, delta, self.weight, self.eps, ctx.dtype)

    def hint(self):
        return ops.NormHint(self.weight, self.eps)

    def deferred(self, ctx, residual: torch.Tensor, added):
        if added.scaled is None or added.weight is not self.weight:      # the product knew no norm, or another one
            return self.norm(ctx, residual)
        return ops.NormedResidual(residual, added.ss_parts, added.scaled, self.weight, self.eps, ctx.dtype)
