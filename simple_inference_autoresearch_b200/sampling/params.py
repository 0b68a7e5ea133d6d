"""Sampling options, with the names and meanings of the reference's ``sample()``
(sampling.py:151-236): ``temperature`` 0 means greedy and ignores the rest, a
negative one is an error (sampling.py:58-62); ``top_k`` <= 0 or >= vocab disables
top-k; ``top_p`` >= 1 disables the nucleus and <= 0 keeps only the top token.
``seed`` is per request: the reference draws from torch's global generator, so a
request's tokens depend on what else is in the batch; here the uniform for a
request's n-th token is a function of (seed, request id, n) alone, the request id being the
caller's (``Engine.generate(request_ids=...)``) or, by default, the prompt's index in the call.
"""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 1.0
    top_k: int = 0
    top_p: float = 1.0
    seed: int = 0

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError(f"temperature must be >= 0 (got {self.temperature}); 0 means greedy")
        if self.top_p != self.top_p:
            raise ValueError("top_p is NaN")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0


GREEDY = SamplingParams(temperature=0.0)

_MASK64 = (1 << 64) - 1


def request_seed(seed: int, request_id: int) -> int:
    """64-bit seed of one request: requests that share a user seed still draw
    different streams.  Returned as a signed 64-bit value (it travels in an int64 tensor)."""
    z = (int(seed) * 0x9E3779B97F4A7C15 + (int(request_id) + 1) * 0xD1B54A32D192ED03) & _MASK64
    z ^= z >> 32
    z = (z * 0xD6E8FEB86659FD93) & _MASK64
    z ^= z >> 32
    return z - (1 << 64) if z >= (1 << 63) else z


def uniform_from_counter(seed64: int, index: int) -> float:
    """The uniform in [0, 1) the sampling kernel uses for draw ``index`` of a
    request (same integer arithmetic, on the host)."""
    z = ((seed64 & _MASK64) + 0x9E3779B97F4A7C15 * (index + 1)) & _MASK64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK64
    z ^= z >> 31
    return (z >> 40) / 16777216.0
