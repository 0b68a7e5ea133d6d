"""Grouped-query attention as a mixer.

In the reference's order (ops/attention.py:139-178,291-348):
one product with the stacked weight ``[Wq; Wk; Wv]`` (rows ``[0, Hq*D)`` are q,
the next ``Hkv*D`` are k, the rest v; the head index is the slow axis of each
slice), rotation of q and k by the tokens' positions, k and v written to the
cache (k is cached rotated), causal attention of each new token over keys
``[0, position]`` of its own sequence with scale ``1/sqrt(D)`` and query head
``hq`` reading kv head ``hq // (Hq/Hkv)``, and the output product with ``Wo``.
There are no biases (loader.py:74-93 reads none).

``window`` (not a Llama option; the reference has none, ops/attention.py:337-342) limits a
token to the last ``window`` keys, itself included; layers with a window get a cache group of
their own that gives pages back as they fall out of every later query's sight.
"""

from __future__ import annotations

import math
from typing import List, Mapping, Optional

import torch

from ..kernels import ops
from .base import KVNeed, MIXERS, Mixer, TensorSpec


@MIXERS.register("gqa_attention")
class GroupedQueryAttention(Mixer):
    def __init__(self, prefix: str, position, hidden_size: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 init_std: float = 0.02, window: Optional[int] = None):
        super().__init__(prefix)
        if window is not None and int(window) <= 0:
            raise ValueError(f"an attention window must be positive, got {window}")
        self.window = None if window is None else int(window)
        self.hidden_size, self.n_heads, self.n_kv_heads, self.head_dim = (
            int(hidden_size), int(n_heads), int(n_kv_heads), int(head_dim))
        ops.check_attention_sizes(self.n_heads, self.n_kv_heads, self.head_dim)
        self.scale = 1.0 / math.sqrt(self.head_dim)
        self.init_std = init_std
        self.position = position
        self.w_qkv: torch.Tensor = None
        self.w_o: torch.Tensor = None

    def tensor_specs(self) -> List[TensorSpec]:
        h, d = self.hidden_size, self.head_dim
        p, s = self.prefix, self.init_std
        return [
            TensorSpec(p + "q_proj.weight", (self.n_heads * d, h), std=s),
            TensorSpec(p + "k_proj.weight", (self.n_kv_heads * d, h), std=s),
            TensorSpec(p + "v_proj.weight", (self.n_kv_heads * d, h), std=s),
            TensorSpec(p + "o_proj.weight", (h, self.n_heads * d), std=s),
        ]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        p = self.prefix
        self.w_qkv = torch.cat([tensors[p + "q_proj.weight"], tensors[p + "k_proj.weight"],
                                tensors[p + "v_proj.weight"]], dim=0).contiguous()
        self.w_o = tensors[p + "o_proj.weight"].contiguous()

    def cache_need(self):
        return KVNeed(self.n_kv_heads, self.head_dim, self.window)

    def extension_units(self, dtype=None):
        units = ("elementwise", "attention", "gemm_simt")
        if dtype != torch.float32:            # the tensor-core units are bfloat16 only
            units += ("attention_mma", "gemm_tc")
            if self.head_dim in (64, 128) and self.n_heads // self.n_kv_heads <= 128:
                units += ("attention_tc",)    # prompts of bfloat16 models with these sizes
        return units

    takes_deferred_norm = True

    def forward(self, ctx, x, cache_entry, writes_cache: bool = True):
        qkv = ops.linear(x, self.w_qkv, ctx.dtype, options=ctx.options)
        rotary = self.position.rotary() if self.position is not None else None
        attn = ops.rope_and_attention(qkv, rotary, cache_entry, ctx.meta,
                                      self.n_heads, self.n_kv_heads, self.head_dim, self.scale,
                                      write_kv=writes_cache, window=self.window, options=ctx.options)
        return ops.linear(attn, self.w_o, torch.float32, add_to=ctx.residual, next_norm=ctx.next_norm,
                          options=ctx.options)
