"""SwiGLU feed-forward.

    gu = x [W_gate; W_up]^T      (one product)
    f  = silu(gate) * up,  silu(g) = g * sigmoid(g)
    m  = f W_down^T

as the reference's MLP (ops/mlp.py:98-129,179-214; kernels/swiglu_kernel.py:139-140).  The
reference stacks the two weights as halves (rows [0, I) gate, [I, 2I) up); here their rows
alternate (gate_0, up_0, gate_1, up_1, ...), so that a tile of the product holds gate and up
of the same outputs and the activation can run in the product's epilogue, in 32-bit on the
accumulators, with one rounding of ``f`` (the reference's unfused path rounds ``gu`` first).
"""

from __future__ import annotations

from typing import List, Mapping

import torch

from ..kernels import ops
from .base import FEED_FORWARDS, FeedForward, TensorSpec


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    def __init__(self, prefix: str, hidden_size: int, intermediate_size: int, init_std: float = 0.02):
        super().__init__(prefix)
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.init_std = init_std
        self.w_gate_up: torch.Tensor = None
        self.w_down: torch.Tensor = None

    def tensor_specs(self) -> List[TensorSpec]:
        h, i, p, s = self.hidden_size, self.intermediate_size, self.prefix, self.init_std
        return [
            TensorSpec(p + "gate_proj.weight", (i, h), std=s),
            TensorSpec(p + "up_proj.weight", (i, h), std=s),
            TensorSpec(p + "down_proj.weight", (h, i), std=s),
        ]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        p = self.prefix
        gate, up = tensors[p + "gate_proj.weight"], tensors[p + "up_proj.weight"]
        self.w_gate_up = torch.stack([gate, up], dim=1).reshape(2 * gate.shape[0], gate.shape[1]).contiguous()
        self.w_down = tensors[p + "down_proj.weight"].contiguous()

    def extension_units(self, dtype=None):
        # the tcgen05 products are bfloat16 only; the CUDA-core product is the 32-bit path and the fallback
        return ("elementwise", "gemm_simt") + (() if dtype == torch.float32 else ("gemm_tc",))

    takes_deferred_norm = True

    def forward(self, ctx, x):
        f = ops.linear_swiglu(x, self.w_gate_up, options=ctx.options)
        return ops.linear(f, self.w_down, torch.float32, add_to=ctx.residual, next_norm=ctx.next_norm,
                          options=ctx.options)
