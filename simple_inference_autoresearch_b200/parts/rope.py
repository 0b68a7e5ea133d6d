"""Rotary position encoding with the llama3 frequency scaling.

Frequencies, as the reference builds them (ops/rope.py:97-105,128-163):

    inv_freq_i = 1 / theta^(2i / D),  i = 0 .. D/2 - 1        (float32, torch)

and for ``rope_type == "llama3"``, per frequency, in Python floats on the float32
value, the result stored back as float32:

    wavelen = 2 pi / f
    wavelen < orig / high_freq_factor            -> f
    wavelen > orig / low_freq_factor             -> f / factor
    otherwise  smooth = (orig / wavelen - low) / (high - low)
               f' = (1 - smooth) f / factor + smooth f

The rotation itself (pairs (x_i, x_{i+D/2}), angle = position * inv_freq_i formed
in float32, ops/rope.py:108-118, kernels/rope_kernel.py:143-152) happens inside
the mixer's fused rotate-and-cache-write kernel, which evaluates sin and cos of
the float32 angle on the fly; no table of ``max_position_embeddings`` rows is
kept (the reference keeps one and rounds it to bfloat16 on the bf16 path,
ops/rope.py:165-185; that rounding is not reproduced).
"""

from __future__ import annotations

import math
from typing import Optional

import torch

from .base import POSITION_ENCODINGS, PositionEncoding


def rotary_inv_freq(head_dim: int, theta: float, scaling: Optional[dict]) -> torch.Tensor:
    """``head_dim`` here is the width that is rotated (the whole head for Llama)."""
    idx = torch.arange(0, head_dim, 2, dtype=torch.float32)
    freqs = 1.0 / (theta ** (idx / head_dim))
    if scaling and scaling.get("rope_type", "default") == "llama3":
        factor = float(scaling["factor"])
        low, high = float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
        orig = int(scaling["original_max_position_embeddings"])
        low_wavelen, high_wavelen = orig / low, orig / high
        out = []
        for f in freqs.tolist():
            wavelen = 2 * math.pi / f
            if wavelen < high_wavelen:
                out.append(f)
            elif wavelen > low_wavelen:
                out.append(f / factor)
            else:
                smooth = (orig / wavelen - low) / (high - low)
                out.append((1 - smooth) * f / factor + smooth * f)
        freqs = torch.tensor(out, dtype=torch.float32)
    return freqs


class RotaryParams:
    """What a rotating mixer needs to know: the frequencies (float32 [rotary_dim / 2], on the
    device), how many leading dims of a head are rotated, and how they pair up: split-half
    (i, i + rotary_dim/2), the Llama way, or ``interleaved`` (2i, 2i+1)."""

    def __init__(self, inv_freq: torch.Tensor, rotary_dim: int, interleaved: bool = False):
        self.inv_freq, self.rotary_dim, self.interleaved = inv_freq, int(rotary_dim), bool(interleaved)


@POSITION_ENCODINGS.register("rotary")
class RotaryEncoding(PositionEncoding):
    """``scaling``: None or a dict with rope_type/factor/low_freq_factor/
    high_freq_factor/original_max_position_embeddings.  ``rotary_dim`` (default: the whole head)
    and ``interleaved`` (default: split-half pairs) are not Llama options (the reference's model
    always rotates the whole head in split-half pairs, ops/rope.py:188-203; its kernel also knows
    interleaved pairs, kernels/rope_kernel.py:139-152); they are here so that another architecture's
    rotary layout is a parameter, not another kernel."""

    def __init__(self, prefix: str = "", *, head_dim: int, theta: float, scaling: Optional[dict] = None,
                 rotary_dim: Optional[int] = None, interleaved: bool = False, device=None):
        super().__init__(prefix)
        self.head_dim, self.theta, self.scaling = int(head_dim), float(theta), scaling
        self.rotary_dim = int(rotary_dim) if rotary_dim else self.head_dim
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim must be even and within head_dim {self.head_dim}, got {rotary_dim}")
        inv = rotary_inv_freq(self.rotary_dim, self.theta, self.scaling)
        self._params = RotaryParams(inv.to(device) if device is not None else inv, self.rotary_dim, interleaved)

    def rotary(self) -> RotaryParams:
        return self._params


@POSITION_ENCODINGS.register("none")
class NoPositionEncoding(PositionEncoding):
    """Positions enter nowhere (a mixer with its own notion of order)."""

    def __init__(self, prefix: str = "", device=None):
        super().__init__(prefix)
