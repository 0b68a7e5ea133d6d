"""A decoder model as data: parts, layers, and the order in which layers run.

``ModelSpec`` says which parts exist (embedding, position encoding, a list of
layer blocks, final norm, output head) and ``schedule`` says in which order the
layers run.  The schedule is a list because the order is data too: it may name a
layer twice (the same weights run again, with a cache entry of their own), and an
entry may read the cache that another entry writes instead of writing one.  The
Llama decoder's schedule is simply layer 0..L-1, each with its own entry, which is
the loop of the reference's forward (model/llama.py:170-199): embed, blocks with
the residual threaded through, final norm on the wanted rows only
(model/llama.py:189-194), output product with the tied or untied head
(ops/embedding.py:109-126).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Mapping, Optional, Sequence, Tuple

import torch

from ..kernels import ops
from ..kernels.options import DEFAULT, KernelOptions
from ..parts.base import BLOCKS, NORMS, POSITION_ENCODINGS, PartSpec, TensorSpec


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  ``cache_entry`` is the index of the cache entry the
    run uses; ``writes_cache`` False means it only reads that entry (which another
    run, earlier in the schedule, writes)."""

    layer: int
    cache_entry: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_position: int
    embedding_name: str
    head_name: Optional[str]           # None: the head is the embedding table (tied)
    position: PartSpec
    layers: Tuple[PartSpec, ...]       # block specs; params hold nested part specs
    final_norm: PartSpec
    schedule: Tuple[ScheduleEntry, ...] = ()
    stop_token_ids: Tuple[int, ...] = ()
    embedding_std: float = 0.02
    #: tensors a checkpoint of this architecture may hold beside the ones the model reads: exact names,
    #: or ``*suffix`` for every name that ends so (a tied model's stored head, buffers some writers save)
    ignorable_tensors: Tuple[str, ...] = ()

    def resolved_schedule(self) -> Tuple[ScheduleEntry, ...]:
        if self.schedule:
            return self.schedule
        return tuple(ScheduleEntry(i, i, True) for i in range(len(self.layers)))


class StepContext:
    """What parts see of a step: the compute dtype, the batch description and the kernel
    options of the engine that runs it (parts hand ``options`` on to the functions of ``ops``)."""

    def __init__(self, dtype: torch.dtype, meta, cache, options: KernelOptions = DEFAULT):
        self.dtype = dtype
        self.meta = meta
        self.cache = cache
        self.options = options
        self.residual = None      # set by a block: the stream a sublayer's last product may add into
        self.next_norm = None     # set by a block: ops.NormHint of the norm after the running sublayer
        self.norm_after_block = None      # set by the model: the hint of the norm the next block (or the model) applies first


class DecoderModel:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device):
        if dtype not in (torch.bfloat16, torch.float32):
            raise TypeError(f"compute dtype must be bfloat16 or float32, got {dtype}")
        self.spec, self.dtype, self.device = spec, dtype, torch.device(device)
        self.position = POSITION_ENCODINGS.build(spec.position, device=self.device)
        self.layers = [BLOCKS.build(ls, position=self.position) for ls in spec.layers]
        self.final_norm = NORMS.build(spec.final_norm)
        self.schedule = spec.resolved_schedule()
        for e in self.schedule:
            if not (0 <= e.layer < len(self.layers)):
                raise ValueError(f"schedule names layer {e.layer}; the model has {len(self.layers)}")
        n_entries = 1 + max((e.cache_entry for e in self.schedule), default=-1)
        writers: Dict[int, int] = {}
        for pos, e in enumerate(self.schedule):
            if e.writes_cache:
                if e.cache_entry in writers:
                    raise ValueError(f"cache entry {e.cache_entry} is written by two runs of the schedule")
                writers[e.cache_entry] = pos
        needs: List[object] = [None] * n_entries
        for pos, e in enumerate(self.schedule):
            need = self.layers[e.layer].cache_need()
            if e.writes_cache:
                needs[e.cache_entry] = need
            else:
                w = writers.get(e.cache_entry)
                if w is None or w > pos:
                    raise ValueError(f"run {pos} reads cache entry {e.cache_entry} before any run writes it")
                if self.layers[self.schedule[w].layer].cache_need() != need:
                    raise ValueError(f"run {pos} reads cache entry {e.cache_entry} whose layout differs from its own")
        self.cache_needs = needs
        self.embedding: torch.Tensor = None
        self.head: torch.Tensor = None
        self._weight_bytes = 0

    # ---- weights
    def tensor_specs(self) -> List[TensorSpec]:
        s = self.spec
        specs = [TensorSpec(s.embedding_name, (s.vocab_size, s.hidden_size), std=s.embedding_std)]
        specs += self.position.tensor_specs()
        for layer in self.layers:
            specs += layer.tensor_specs()
        specs += self.final_norm.tensor_specs()
        if s.head_name is not None:
            specs.append(TensorSpec(s.head_name, (s.vocab_size, s.hidden_size), std=s.embedding_std))
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        s = self.spec
        self.embedding = tensors[s.embedding_name].contiguous()
        self.head = self.embedding if s.head_name is None else tensors[s.head_name].contiguous()
        self.position.load(tensors)
        for layer in self.layers:
            layer.load(tensors)
        self.final_norm.load(tensors)
        seen, total = set(), 0
        for spec in self.tensor_specs():
            t = tensors[spec.name]
            if t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        self._weight_bytes = total

    def extension_units(self) -> List[str]:
        """The CUDA units a step of this model launches from: the model's own (embedding, head
        product, sampling) and what each part names for the compute dtype."""
        units = ["elementwise", "gemm_simt", "sampling"]
        if self.dtype == torch.bfloat16:
            units.append("gemm_tc")        # the head product
        for part in [self.position, self.final_norm] + self.layers:
            try:
                units += list(part.extension_units(self.dtype))
            except TypeError:              # a part written before the argument existed
                units += list(part.extension_units())
        return sorted(set(units))

    def weight_bytes(self) -> int:
        """Bytes of all tensors the model owns (what one decode step has to read)."""
        return self._weight_bytes

    # ---- forward
    def forward(self, meta, cache, options: KernelOptions = DEFAULT) -> torch.Tensor:
        """Runs the step's tokens through the schedule; returns float32 logits
        ``[len(want_rows), vocab]`` for the rows ``meta.want_rows`` names."""
        ctx = StepContext(self.dtype, meta, cache, options)
        residual = ops.embed(meta.tokens, self.embedding)
        self.position.at_embedding(ctx, residual)
        pending = None
        # the final norm's inputs can only come from the last block's product when every row is wanted
        last_hint = self.final_norm.hint() if (meta.want_is_identity and meta.n_want > 0) else None
        for i, e in enumerate(self.schedule):
            nxt = self.layers[self.schedule[i + 1].layer] if i + 1 < len(self.schedule) else None
            ctx.norm_after_block = last_hint if nxt is None else nxt.first_norm_hint()
            residual, pending = self.layers[e.layer].forward(ctx, residual, pending, cache.entry(e.cache_entry),
                                                             e.writes_cache)
        if meta.n_want == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=residual.device)
        if isinstance(pending, ops.Added):      # the last sublayer added itself
            if meta.want_is_identity and pending.ss_parts is not None:
                return ops.linear(self.final_norm.deferred(ctx, residual, pending), self.head, torch.float32,
                                  options=options)
            pending = None
        if not meta.want_is_identity:
            residual = ops.gather_rows(residual, meta.want_rows)
            if pending is not None:
                pending = ops.gather_rows(pending, meta.want_rows)
        if pending is None:
            h = self.final_norm.norm(ctx, residual)
        else:
            h = self.final_norm.add_norm(ctx, residual, pending)
        return ops.linear(h, self.head, torch.float32, options=options)
