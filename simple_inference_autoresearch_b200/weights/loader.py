"""Weights from safetensors, by tensor name.

File discovery is the reference's (loader.py:179-203): ``model.safetensors.index.json``
with its ``weight_map`` from tensor name to shard, else a single
``model.safetensors``, else ``FileNotFoundError``.  Unlike the reference, which
reports the first missing name as a ``KeyError`` (loader.py:218-226) and leaves
shape errors to ``copy_``, everything the model asks for is checked against the
files first and ONE ``WeightError`` lists all missing tensors, all unexpected
tensors and all wrong shapes.

Held dtype: matrices and embedding tables in the engine's compute dtype
(bfloat16, or float32 on the 32-bit path), integer tables as int32, and small
per-channel vectors that the file stores in 32-bit stay 32-bit.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Callable, Dict, Iterable, List, Mapping, Sequence

import torch

from ..parts.base import TensorSpec

INDEX_FILE = "model.safetensors.index.json"
SINGLE_FILE = "model.safetensors"


class WeightError(RuntimeError):
    """The checkpoint does not hold what the model needs; lists every fault."""

    def __init__(self, where, missing=(), unexpected=(), wrong_shape=(), wrong_kind=()):
        self.missing, self.unexpected = list(missing), list(unexpected)
        self.wrong_shape, self.wrong_kind = list(wrong_shape), list(wrong_kind)
        lines = [f"checkpoint {where} does not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(
                f"{n}: expected {tuple(e)}, file has {tuple(g)}" for n, e, g in self.wrong_shape))
        if self.wrong_kind:
            lines.append(f"  wrong dtypes ({len(self.wrong_kind)}): " + "; ".join(
                f"{n}: {why}" for n, why in self.wrong_kind))
        super().__init__("\n".join(lines))


def held_dtype(spec: TensorSpec, stored: torch.dtype, compute: torch.dtype) -> torch.dtype:
    if spec.role == "int":
        return torch.int32
    if spec.role == "vector" and stored in (torch.float32, torch.float64):
        return torch.float32
    return compute


def _shard_map(model_dir: Path) -> Dict[str, Path]:
    """tensor name -> file that holds it."""
    from safetensors import safe_open

    index = model_dir / INDEX_FILE
    if index.exists():
        with open(index) as f:
            weight_map = json.load(f)["weight_map"]
        files = {name: model_dir / shard for name, shard in weight_map.items()}
        absent = sorted({str(p) for p in files.values() if not p.exists()})
        if absent:
            raise FileNotFoundError(f"{index} names shard files that do not exist: {', '.join(absent)}")
        return files
    single = model_dir / SINGLE_FILE
    if single.exists():
        with safe_open(str(single), framework="pt", device="cpu") as f:
            return {name: single for name in f.keys()}
    raise FileNotFoundError(f"{model_dir} holds neither {INDEX_FILE} nor {SINGLE_FILE}")


def load_checkpoint(model_dir, specs: Sequence[TensorSpec], compute_dtype: torch.dtype, device,
                    ignorable: Iterable[str] = ()) -> Dict[str, torch.Tensor]:
    """Reads exactly the tensors ``specs`` name.  ``ignorable`` names (or, written ``*suffix``, every
    name that ends so) may be present in the files without being an error (a tied model's stored head)."""
    from safetensors import safe_open

    model_dir = Path(model_dir)
    files = _shard_map(model_dir)
    wanted = {s.name: s for s in specs}
    missing = sorted(n for n in wanted if n not in files)
    exact = {n for n in ignorable if not n.startswith("*")}
    suffixes = tuple(n[1:] for n in ignorable if n.startswith("*"))
    unexpected = sorted(n for n in files if n not in wanted and n not in exact and not (suffixes and n.endswith(suffixes)))
    wrong_shape, wrong_kind = [], []
    by_file: Dict[Path, List[str]] = {}
    for name in wanted:
        if name in files:
            by_file.setdefault(files[name], []).append(name)
    # first pass: shapes and dtypes from the headers only
    for path, names in by_file.items():
        with safe_open(str(path), framework="pt", device="cpu") as f:
            for name in names:
                sl = f.get_slice(name)
                shape = tuple(sl.get_shape())
                if shape != tuple(wanted[name].shape):
                    wrong_shape.append((name, wanted[name].shape, shape))
                stored = str(sl.get_dtype())
                is_int = stored.startswith(("I", "U")) or stored == "BOOL"
                if (wanted[name].role == "int") != is_int:
                    wrong_kind.append((name, f"role {wanted[name].role!r} but the file stores {stored}"))
    if missing or unexpected or wrong_shape or wrong_kind:
        raise WeightError(model_dir, missing, unexpected, wrong_shape, wrong_kind)
    out: Dict[str, torch.Tensor] = {}
    for path, names in by_file.items():
        with safe_open(str(path), framework="pt", device="cpu") as f:
            for name in names:
                t = f.get_tensor(name)
                out[name] = t.to(device=device, dtype=held_dtype(wanted[name], t.dtype, compute_dtype))
    return out


def check_tensors(tensors: Mapping[str, torch.Tensor], specs: Sequence[TensorSpec], where="(in memory)") -> None:
    """The same three checks for tensors that do not come from files."""
    wanted = {s.name: s for s in specs}
    missing = sorted(n for n in wanted if n not in tensors)
    unexpected = sorted(n for n in tensors if n not in wanted)
    wrong = [(n, wanted[n].shape, tuple(t.shape)) for n, t in tensors.items()
             if n in wanted and tuple(t.shape) != tuple(wanted[n].shape)]
    if missing or unexpected or wrong:
        raise WeightError(where, missing, unexpected, wrong)
