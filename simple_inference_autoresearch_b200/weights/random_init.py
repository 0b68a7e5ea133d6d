"""Seeded random weights, and a writer that turns a configuration and a seed
into a model folder (``config.json`` + ``model.safetensors``).

The reference has no such mode (its benches load the real checkpoint).  Every
tensor is drawn on its own from ``(seed, tensor name)``, in float32, by a counter-based
generator whose arithmetic is the same on every device, so that any subset of the
tensors, in any order, on the CPU or on the GPU, reproduces the same bits:
matrices and embeddings N(0, std), norm weights 1 or 1 + N(0, std) as the part's
``TensorSpec`` says.
"""

from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Dict, Mapping, Optional, Sequence

import torch

from ..parts.base import TensorSpec


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{int(seed)}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


# ---- a counter-based normal generator that gives the same bits on the CPU and on the GPU
#
# Element i of a tensor is a function of (tensor key, i) alone: splitmix64 of the counter gives 64
# bits, of which two 24-bit fields become two uniforms, and Box-Muller turns those into one normal
# deviate.  Every step is a single torch operation that is exactly rounded on both devices (integer
# arithmetic, float32 add / multiply / divide / floor): the logarithm, the cosine and the square
# root are evaluated by series and iterations written out below, not by the devices' own
# libraries, which differ in the last bit (torch's float32 sqrt on the GPU is not exactly rounded:
# 0.7% of its results differ from the CPU's).  So ``random_tensor(spec, seed, dtype, "cpu")`` and ``(..., "cuda")`` hold identical bits,
# as do a tensor drawn whole and the same tensor drawn in pieces.

_CHUNK = 1 << 24        # elements drawn at a time (bounds the temporaries)


def _i64(x: int) -> int:
    """A 64-bit pattern as the signed integer torch's int64 holds."""
    x &= (1 << 64) - 1
    return x - (1 << 64) if x >= (1 << 63) else x


def _lshr(z: torch.Tensor, n: int) -> torch.Tensor:
    """Logical right shift of int64 (torch's shift is arithmetic)."""
    return (z >> n) & ((1 << (64 - n)) - 1)


def _splitmix64(counter: torch.Tensor, key: int) -> torch.Tensor:
    z = counter * _i64(0x9E3779B97F4A7C15) + _i64(key)
    z = (z ^ _lshr(z, 30)) * _i64(0xBF58476D1CE4E5B9)
    z = (z ^ _lshr(z, 27)) * _i64(0x94D049BB133111EB)
    return z ^ _lshr(z, 31)


def _horner(x: torch.Tensor, coeffs) -> torch.Tensor:
    """coeffs[0] + x (coeffs[1] + x (...)), one multiply and one add at a time (never fused)."""
    acc = torch.full_like(x, coeffs[-1])
    for c in reversed(coeffs[:-1]):
        acc = acc * x
        acc = acc + c
    return acc


_LN2_HI = 0.693145751953125          # the leading bits of ln 2: exact in float32, times |e| <= 24 exact too
_LN2_LO = 1.42860682030941723212e-6
_SQRT2 = 1.4142135381698608          # float32(sqrt 2)
# ln m = 2 s (1 + s^2/3 + s^4/5 + ...), s = (m - 1) / (m + 1), for m in [1/sqrt 2, sqrt 2]: s^2 <= 0.0295
_ATANH = [1.0, 1.0 / 3, 1.0 / 5, 1.0 / 7, 1.0 / 9, 1.0 / 11, 1.0 / 13]
# cos x and sin x / x in powers of x^2, for x in [0, pi/2]
_COS = [1.0, -1.0 / 2, 1.0 / 24, -1.0 / 720, 1.0 / 40320, -1.0 / 3628800, 1.0 / 479001600, -1.0 / 87178291200,
        1.0 / 20922789888000]
_SIN = [1.0, -1.0 / 6, 1.0 / 120, -1.0 / 5040, 1.0 / 362880, -1.0 / 39916800, 1.0 / 6227020800,
        -1.0 / 1307674368000, 1.0 / 355687428096000]
_HALF_PI = 1.5707963705062866        # float32(pi / 2)


def _neg_log(u: torch.Tensor) -> torch.Tensor:
    """-ln u for float32 u in (0, 1]."""
    bits = u.view(torch.int32)
    e = ((bits >> 23) & 0xFF) - 127
    m = ((bits & 0x7FFFFF) | 0x3F800000).view(torch.float32)          # in [1, 2)
    big = m > _SQRT2
    m = torch.where(big, m * 0.5, m)
    e = torch.where(big, e + 1, e).to(torch.float32)
    s = (m - 1.0) / (m + 1.0)
    ln_m = (s + s) * _horner(s * s, _ATANH)
    return -(e * _LN2_HI + (e * _LN2_LO + ln_m))


def _sqrt(y: torch.Tensor) -> torch.Tensor:
    """sqrt y for float32 y >= 0 to the last bit or two, from operations that round alike everywhere:
    a first guess from the bit pattern (halved exponent, 3.5% off at most), then Newton steps
    r <- (r + y / r) / 2, each of which squares the error."""
    r = ((y.view(torch.int32) >> 1) + 0x1FBD1DF5).view(torch.float32)
    for _ in range(4):
        r = (r + y / r) * 0.5
    return torch.where(y > 0, r, torch.zeros_like(y))


def _cos_turns(t: torch.Tensor) -> torch.Tensor:
    """cos(2 pi t) for float32 t in [0, 1) on a 2^-24 grid: the quadrant is split off exactly."""
    t4 = t * 4.0
    quad = torch.floor(t4)
    x = (t4 - quad) * _HALF_PI
    x2 = x * x
    c = _horner(x2, _COS)
    sn = x * _horner(x2, _SIN)
    return torch.where(quad == 0, c, torch.where(quad == 1, -sn, torch.where(quad == 2, -c, sn)))


def standard_normal(n: int, key: int, device="cpu", start: int = 0) -> torch.Tensor:
    """Elements ``start .. start + n - 1`` of the stream ``key``: float32 N(0, 1) deviates (to about
    1e-6; 24-bit uniforms, so |z| <= 5.8), bit-identical on every device."""
    dev = torch.device(device)
    counter = torch.arange(start + 1, start + n + 1, dtype=torch.int64, device=dev)
    z = _splitmix64(counter, key)
    u1 = (_lshr(z, 40) + 1).to(torch.float32) * (1.0 / 16777216.0)           # (0, 1]
    u2 = (_lshr(z, 16) & 0xFFFFFF).to(torch.float32) * (1.0 / 16777216.0)    # [0, 1)
    r = _sqrt(_neg_log(u1) * 2.0)
    return r * _cos_turns(u2)


def random_tensor(spec: TensorSpec, seed: int, dtype: torch.dtype, device="cpu") -> torch.Tensor:
    """The tensor ``spec`` names, drawn from ``(seed, spec.name)``: the same bits whatever the
    device, and whatever else is drawn before or after it."""
    dev = torch.device(device)
    shape = tuple(spec.shape)
    if spec.role == "int":
        return torch.zeros(shape, dtype=torch.int32, device=dev)
    if spec.init == "ones":
        return torch.ones(shape, dtype=dtype, device=dev)
    if spec.init == "zeros":
        return torch.zeros(shape, dtype=dtype, device=dev)
    if spec.init not in ("normal", "ones_plus_normal"):
        raise ValueError(f"unknown init {spec.init!r} for {spec.name}")
    n = 1
    for d in shape:
        n *= int(d)
    key = _tensor_seed(seed, spec.name)
    out = torch.empty(n, dtype=dtype, device=dev)
    for start in range(0, n, _CHUNK):
        m = min(_CHUNK, n - start)
        t = standard_normal(m, key, dev, start) * float(spec.std)
        if spec.init == "ones_plus_normal":
            t = t + 1.0
        out[start:start + m] = t.to(dtype)
    return out.view(shape)


def random_tensors(specs: Sequence[TensorSpec], seed: int, dtype: torch.dtype, device="cpu") -> Dict[str, torch.Tensor]:
    return {s.name: random_tensor(s, seed, dtype, device) for s in specs}


def write_model_folder(folder, config, seed: int, store_dtype: torch.dtype = torch.bfloat16,
                       vector_dtype: Optional[torch.dtype] = None, **spec_options) -> Path:
    """Writes ``config.json`` and ``model.safetensors`` for ``config`` (a typed
    configuration of a registered architecture) with weights drawn from ``seed``.
    ``vector_dtype`` stores the per-channel vectors (norm weights) in another
    dtype than the matrices, e.g. float32."""
    from safetensors.torch import save_file

    from .. import registry
    from ..engine.model import DecoderModel

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    raw = config.to_dict()
    raw["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32", torch.float16: "float16"}[store_dtype]
    arch = registry.resolve(raw)
    spec = arch.spec_builder(config, **spec_options)
    model = DecoderModel(spec, torch.float32, "cpu")
    tensors = {}
    for ts in model.tensor_specs():
        dt = vector_dtype if (vector_dtype is not None and ts.role == "vector") else store_dtype
        tensors[ts.name] = random_tensor(ts, seed, dt).contiguous()
    with open(folder / "config.json", "w") as f:
        json.dump(raw, f, indent=1)
    save_file(tensors, str(folder / "model.safetensors"), metadata={"format": "pt", "seed": str(seed)})
    return folder


def main(argv=None) -> int:
    """``python -m simple_inference_autoresearch_b200.weights.random_init --config config.json --out DIR --seed 0``"""
    import argparse

    from .. import registry

    ap = argparse.ArgumentParser(description="write a model folder with seeded random weights")
    ap.add_argument("--config", required=True, help="a config.json (or a folder holding one)")
    ap.add_argument("--out", required=True)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    args = ap.parse_args(argv)
    _, config = registry.resolve_path(args.config)
    folder = write_model_folder(args.out, config, args.seed, store_dtype=getattr(torch, args.dtype))
    print(folder)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
