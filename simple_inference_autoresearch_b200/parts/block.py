"""Pre-norm residual block: ``x += mixer(norm1(x)); x += ffn(norm2(x))``.

The adds are threaded the way the reference threads them (model/block.py:154-183):
each sublayer's output is left *pending* and added inside the next norm's kernel,
so no separate add is launched (for a few rows the products themselves add into the
residual and make the normed input of the next product: ``ops.Added``, ``ops.NormedResidual``); the last block's pending delta is resolved by the
model's final norm (model/llama.py:194).  A first block that receives no pending
delta only norms (model/block.py:164-166).
"""

from __future__ import annotations

from typing import List, Mapping

import torch

from ..kernels import ops
from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block, PartSpec, TensorSpec


def _units_of(part, dtype):
    """A part's units for ``dtype``; parts written before the argument existed take none."""
    try:
        return part.extension_units(dtype)
    except TypeError:
        return part.extension_units()


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    """``mixer``, ``feed_forward``, ``mixer_norm`` and ``ffn_norm`` are PartSpecs whose
    ``params`` may hold a ``prefix`` relative to this block's prefix."""

    def __init__(self, prefix: str, position, mixer: PartSpec, feed_forward: PartSpec, mixer_norm: PartSpec,
                 ffn_norm: PartSpec):
        super().__init__(prefix)

        def sub(registry, spec: PartSpec, **ctx):
            params = dict(spec.params)
            params["prefix"] = prefix + params.get("prefix", "")
            return registry.build(PartSpec(spec.kind, params), **ctx)

        self.mixer_norm = sub(NORMS, mixer_norm)
        self.mixer = sub(MIXERS, mixer, position=position)
        self.ffn_norm = sub(NORMS, ffn_norm)
        self.ffn = sub(FEED_FORWARDS, feed_forward)
        self._parts = [self.mixer_norm, self.mixer, self.ffn_norm, self.ffn]

    def tensor_specs(self) -> List[TensorSpec]:
        return [s for p in self._parts for s in p.tensor_specs()]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for p in self._parts:
            p.load(tensors)

    def extension_units(self, dtype=None):
        return tuple(u for p in self._parts for u in _units_of(p, dtype))

    def cache_need(self):
        return self.mixer.cache_need()

    @staticmethod
    def _normed(norm, consumer, ctx, residual, pending):
        """The consumer's input: norm(residual + pending), the add and the norm in one kernel, or
        left to the consumer's first product where the sublayer before already added itself."""
        if pending is None:
            return norm.norm(ctx, residual)
        if isinstance(pending, ops.Added):
            if consumer.takes_deferred_norm and pending.ss_parts is not None:
                return norm.deferred(ctx, residual, pending)
            return norm.norm(ctx, residual)
        return norm.add_norm(ctx, residual, pending)

    def first_norm_hint(self):
        return self.mixer_norm.hint() if self.mixer.takes_deferred_norm else None

    def forward(self, ctx, residual, pending, cache_entry, writes_cache: bool = True):
        ctx.residual = residual       # where a sublayer's last product may add its output itself
        h = self._normed(self.mixer_norm, self.mixer, ctx, residual, pending)
        # the norm that follows each sublayer, for a last product that can leave that norm's inputs behind
        ctx.next_norm = self.ffn_norm.hint() if self.ffn.takes_deferred_norm else None
        a = self.mixer.forward(ctx, h, cache_entry, writes_cache)
        h = self._normed(self.ffn_norm, self.ffn, ctx, residual, a)
        ctx.next_norm = getattr(ctx, "norm_after_block", None)
        m = self.ffn.forward(ctx, h)
        ctx.next_norm = None
        return residual, m
