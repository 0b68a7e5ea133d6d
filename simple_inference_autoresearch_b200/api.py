"""Python entry points, in the manner of the reference's ``load_model`` /
``build_cache`` (model/registry.py:96-129) and ``generate`` /
``generate_with_stats`` (generate.py:50-238).

The reference downloads a checkpoint by its hub id and works on text through a
tokenizer; this library takes a local model folder and works on token ids.
"""

from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable, Iterator, Optional, Sequence, Tuple

import torch

from . import registry
from .engine.engine import Engine
from .engine.model import DecoderModel
from .kernels import build
from .kernels.options import DEFAULT as DEFAULT_OPTIONS, KernelOptions
from .sampling.params import SamplingParams
from .weights.loader import load_checkpoint
from .weights.random_init import random_tensors

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def as_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        return dtype
    try:
        return _DTYPES[str(dtype)]
    except KeyError:
        raise ValueError(f"dtype must be bfloat16 or float32, got {dtype!r}") from None


@dataclass(frozen=True)
class LoadedModel:
    model: DecoderModel
    config: Any
    architecture: registry.Architecture


def build_model(config, dtype=torch.bfloat16, device="cuda", **spec_options) -> LoadedModel:
    """A model of a typed configuration without weights (see ``load_model`` / ``init_random``)."""
    arch = registry.resolve(config.to_dict())
    model = DecoderModel(arch.spec_builder(config, **spec_options), as_dtype(dtype), device)
    if torch.device(device).type == "cuda":
        build.ensure_built([u for u in model.extension_units() if u in build.available_units()])
    return LoadedModel(model, config, arch)


def load_model(model_dir, device="cuda", dtype=torch.bfloat16) -> LoadedModel:
    """Builds the model that ``model_dir/config.json`` names and loads
    ``model_dir``'s safetensors into it by tensor name."""
    arch, config = registry.resolve_path(model_dir)
    loaded = build_model(config, dtype, device)
    m = loaded.model
    m.load(load_checkpoint(Path(model_dir), m.tensor_specs(), m.dtype, m.device, m.spec.ignorable_tensors))
    return loaded


def init_random(loaded: LoadedModel, seed: int) -> LoadedModel:
    """Fills a built model with seeded random weights drawn on its own device
    (for benchmarks of sizes one would not write to disk first)."""
    m = loaded.model
    store = torch.bfloat16
    tensors = random_tensors(m.tensor_specs(), seed, store, m.device)
    m.load({k: (v if m.dtype == store else v.to(m.dtype)) for k, v in tensors.items()})
    return loaded


def build_engine(loaded: LoadedModel, *, max_batch: int = 1, max_seq_len: Optional[int] = None,
                 max_tokens: Optional[int] = None, use_cuda_graph: bool = True,
                 options: KernelOptions = DEFAULT_OPTIONS) -> Engine:
    """The counterpart of the reference's ``build_cache``: cache and step function for a loaded model.
    ``options`` chooses kernels where there is a choice (``KernelOptions``)."""
    return Engine(loaded.model, max_batch=max_batch, max_seq_len=max_seq_len, max_tokens=max_tokens,
                  use_cuda_graph=use_cuda_graph, options=options)


def generate(prompt_ids: Sequence[int], engine: Engine, max_new_tokens: int = 256, temperature: float = 1.0,
             top_k: int = 50, top_p: float = 0.9, seed: int = 0, stop_token_ids=None,
             ignore_eos: bool = False, request_id: int = 0) -> Iterator[int]:
    """Yields the new token ids of one prompt, each as soon as it is drawn (defaults as generate.py:50-59).
    ``request_id`` keys the random stream together with ``seed`` (see ``Engine.generate``)."""
    for _index, tok in engine.stream([list(prompt_ids)], SamplingParams(temperature, top_k, top_p, seed),
                                     max_new_tokens, stop_token_ids=stop_token_ids, ignore_eos=ignore_eos,
                                     request_ids=[request_id]):
        yield tok


def generate_with_stats(prompt_ids: Sequence[int], engine: Engine, max_new_tokens: int = 256,
                        temperature: float = 1.0, top_k: int = 50, top_p: float = 0.9,
                        on_token: Optional[Callable[[int], None]] = None, seed: int = 0, stop_token_ids=None,
                        ignore_eos: bool = False, request_id: int = 0) -> Tuple[list, dict]:
    """(new token ids, stats) for one prompt; stats has the reference's keys (generate.py:227-237)."""
    cb = (lambda _i, tok: on_token(tok)) if on_token is not None else None
    outs, stats = engine.generate([list(prompt_ids)], SamplingParams(temperature, top_k, top_p, seed),
                                  max_new_tokens, stop_token_ids=stop_token_ids, ignore_eos=ignore_eos,
                                  on_token=cb, return_stats=True, request_ids=[request_id])
    return outs[0], stats
