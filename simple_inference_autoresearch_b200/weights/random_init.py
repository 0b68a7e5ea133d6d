"""Seeded random weights, and a writer that turns a configuration and a seed
into a model folder (``config.json`` + ``model.safetensors``).

The reference has no such mode (its benches load the real checkpoint).  Every
tensor is drawn on its own from ``(seed, tensor name)``, in float32, so that any
subset of the tensors, in any order, reproduces the same values:
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


def random_tensor(spec: TensorSpec, seed: int, dtype: torch.dtype, device="cpu") -> torch.Tensor:
    dev = torch.device(device)
    gen = torch.Generator(device=dev)
    gen.manual_seed(_tensor_seed(seed, spec.name))
    shape = tuple(spec.shape)
    if spec.role == "int":
        return torch.zeros(shape, dtype=torch.int32, device=dev)
    if spec.init == "ones":
        t = torch.ones(shape, dtype=torch.float32, device=dev)
    elif spec.init == "zeros":
        t = torch.zeros(shape, dtype=torch.float32, device=dev)
    elif spec.init == "normal":
        t = torch.randn(shape, generator=gen, dtype=torch.float32, device=dev) * spec.std
    elif spec.init == "ones_plus_normal":
        t = 1.0 + torch.randn(shape, generator=gen, dtype=torch.float32, device=dev) * spec.std
    else:
        raise ValueError(f"unknown init {spec.init!r} for {spec.name}")
    return t.to(dtype)


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
