"""Interfaces and registries of the parts a decoder layer is put together from.

A *part* is a mixer (attention here), a feed-forward, a norm, a position encoding
or a block (the arrangement of the first three around the residual stream).  Every
part receives its sizes and constants as constructor parameters, names the
checkpoint tensors it owns, and never learns which model it sits in.  A model is
data: a list of layer descriptions (``PartSpec`` trees) plus a run order.

The reference wires the same five things by hand inside ``TransformerBlock``
(model/block.py:56-100) and passes each constant as a constructor argument; the
registries below turn that wiring into a lookup by name so that another kind of
part can be added from outside the package (``MIXERS.register("my_kind")``).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Mapping, Optional, Sequence, Tuple

import torch


# --------------------------------------------------------------------------- specs
@dataclass(frozen=True)
class PartSpec:
    """``kind`` selects the class in the part's registry, ``params`` are its
    constructor arguments (plain numbers, strings, or nested ``PartSpec``)."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class TensorSpec:
    """One checkpoint tensor a part owns.

    ``role``:
      * ``"matrix"``  - operand of a matrix product or embedding table; held in
        the engine's compute dtype (bfloat16 or float32).
      * ``"vector"``  - small per-channel parameter (norm weights); a tensor the
        checkpoint stores in 32-bit stays 32-bit, otherwise compute dtype.
      * ``"int"``     - integer table, held as int32.
    ``init`` tells the random-weights writer how to draw it: ``"normal"`` (std),
    ``"ones"``, ``"ones_plus_normal"`` (1 + N(0, std)), ``"zeros"``.
    """

    name: str
    shape: Tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"
    std: float = 0.02


class PartRegistry:
    """Name -> class table for one family of parts."""

    def __init__(self, family: str):
        self.family = family
        self._classes: Dict[str, type] = {}

    def register(self, kind: str) -> Callable[[type], type]:
        def deco(cls: type) -> type:
            old = self._classes.get(kind)
            if old is not None and old is not cls:
                raise ValueError(f"{self.family} kind {kind!r} is already registered by {old.__name__}")
            self._classes[kind] = cls
            cls.kind = kind
            return cls
        return deco

    def unregister(self, kind: str) -> None:
        self._classes.pop(kind, None)

    def kinds(self) -> List[str]:
        return sorted(self._classes)

    def build(self, spec: PartSpec, **context) -> "Part":
        try:
            cls = self._classes[spec.kind]
        except KeyError:
            raise ValueError(
                f"unknown {self.family} kind {spec.kind!r}; registered: {', '.join(self.kinds()) or '(none)'}"
            ) from None
        return cls(**context, **dict(spec.params))


MIXERS = PartRegistry("mixer")
FEED_FORWARDS = PartRegistry("feed-forward")
NORMS = PartRegistry("norm")
POSITION_ENCODINGS = PartRegistry("position encoding")
BLOCKS = PartRegistry("block")


# --------------------------------------------------------------------------- cache needs
@dataclass(frozen=True)
class KVNeed:
    """A mixer that keeps keys and values of earlier tokens.  ``window`` = None
    keeps all of them; an integer keeps only that many most recent ones.  ``v_head_dim``:
    the width of a value when it differs from a key's (None: the same; the attention kernels of
    this library take equal widths only, a mixer with its own kernels may differ).  Layers
    whose needs compare equal share one storage group."""

    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    v_head_dim: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """A mixer with per-sequence state of fixed size (``shape`` per sequence)."""

    shape: Tuple[int, ...]
    dtype: str = "float32"


# --------------------------------------------------------------------------- parts
class Part:
    """Base of all parts.  ``prefix`` is the checkpoint name prefix of the part's
    tensors (for instance ``model.layers.3.self_attn.``)."""

    kind: str = "?"

    def __init__(self, prefix: str = ""):
        self.prefix = prefix

    def tensor_specs(self) -> List[TensorSpec]:
        return []

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        """Take ownership of the tensors named by ``tensor_specs`` (already on the
        device, already in the dtype their role asks for)."""

    def extension_units(self, dtype: Optional[torch.dtype] = None) -> Sequence[str]:
        """Names of the CUDA source units this part launches kernels from when the model computes
        in ``dtype`` (None: in any dtype)."""
        return ()


class Norm(Part):
    def norm(self, ctx, residual: torch.Tensor) -> torch.Tensor:
        """normed(residual) in the compute dtype; residual is float32 [N, H]."""
        raise NotImplementedError

    def add_norm(self, ctx, residual: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
        """residual += delta (in place, 32-bit), then return normed(residual)."""
        raise NotImplementedError

    def hint(self):
        """What the product in front of this norm may be told of it (``ops.NormHint``) so that it leaves
        the norm's inputs behind, or None for a norm the product kernels cannot take over."""
        return None

    def deferred(self, ctx, residual: torch.Tensor, added):
        """normed(residual) for a consumer that ``takes_deferred_norm``, after a sublayer whose
        output is already in ``residual`` (``added``: an ``ops.Added``).  A norm whose arithmetic
        the product kernels can take over returns an ``ops.NormedResidual``; the default computes."""
        return self.norm(ctx, residual)


class PositionEncoding(Part):
    def rotary(self):
        """Rotary parameters for a mixer that rotates queries and keys: an object with
        ``inv_freq`` (float32 [rotary_dim/2] on the device), ``rotary_dim`` (how many leading dims
        of a head are rotated) and ``interleaved`` (pairs (2i, 2i+1) instead of (i, i + rotary_dim/2)),
        see ``parts.rope.RotaryParams``; or None when positions enter the model elsewhere."""
        return None

    def at_embedding(self, ctx, residual: torch.Tensor) -> None:
        """Hook for encodings that add to the embedded tokens; default: nothing."""


class Mixer(Part):
    #: True when ``forward`` hands x to ``ops.linear`` / ``ops.linear_swiglu`` only, so that x may be
    #: an ``ops.NormedResidual`` instead of a tensor
    takes_deferred_norm = False

    def cache_need(self):
        """``KVNeed``, ``StateNeed`` or None."""
        return None

    def forward(self, ctx, x: torch.Tensor, cache_entry, writes_cache: bool) -> torch.Tensor:
        """x: normed activations [N, H] (compute dtype) -> float32 delta [N, H].  A part whose last
        step is ``ops.linear(..., torch.float32, add_to=ctx.residual)`` may return what that call
        returns: the delta, or the mark that it is already in the residual."""
        raise NotImplementedError


class FeedForward(Part):
    takes_deferred_norm = False       # as for Mixer

    def forward(self, ctx, x: torch.Tensor) -> torch.Tensor:
        """x: normed activations [N, H] (compute dtype) -> float32 delta [N, H] (or, as for a
        mixer, the result of ``ops.linear(..., add_to=ctx.residual)``)."""
        raise NotImplementedError


class Block(Part):
    """Arrangement of norm(s), mixer and feed-forward around the residual stream.

    The stream is the pair ``(residual, pending)``: ``residual`` float32 [N, H],
    ``pending`` a float32 delta not yet added (or None).  A block may leave its
    last delta pending so that the next norm fuses the add (the reference threads
    the residual the same way, model/block.py:120-183)."""

    def cache_need(self):
        return None

    def first_norm_hint(self):
        """``hint()`` of the norm this block applies first, when its consumer takes a deferred norm
        (the model tells the block in front, through ``ctx.norm_after_block``); None otherwise."""
        return None

    def forward(self, ctx, residual, pending, cache_entry, writes_cache: bool):
        raise NotImplementedError
