"""The engine: a model, its cache, the step function and token sampling on one GPU.

``step`` is the one function everything else is built on: it takes a batch of
sequences with unequal numbers of new tokens (whole prompts, or one token each,
or any mix), runs exactly those tokens as one packed batch against the cache and
returns float32 logits at the wanted places.  The reference's counterpart is
``LlamaModel.forward(token_ids (B, T), start_pos)`` (model/llama.py:137-199),
which needs a rectangular batch at one shared position and returns the last
position only.

``run`` adds the draw of the next token for the generation loop; for steps of
one token per sequence it replays a captured CUDA graph that holds the whole
step, the sampling and the length bookkeeping (the reference captures its decode
forward the same way, model/cuda_graph_decode.py:118-143, with one position for
the whole batch and sampling outside the graph).
"""

from __future__ import annotations

import gc
import time
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.sequence_cache import DEFAULT_PAGE_TOKENS, SequenceCache, round_up
from ..kernels import ops
from ..kernels.options import DEFAULT, KernelOptions
from ..sampling.params import SamplingParams, request_seed
from . import generation
from .batch import BatchMeta, StepEntry
from .model import DecoderModel


#: captured decode steps an engine keeps (one per batch size and 512-key length bucket met)
MAX_CAPTURED_STEPS = 64


class Engine:
    def __init__(self, model: DecoderModel, max_batch: int = 8, max_seq_len: Optional[int] = None,
                 max_tokens: Optional[int] = None, max_slots: Optional[int] = None, page_tokens: int = DEFAULT_PAGE_TOKENS,
                 use_cuda_graph: bool = True, options: KernelOptions = DEFAULT,
                 beyond_trained_positions: bool = False):
        """``beyond_trained_positions``: let ``max_seq_len`` exceed the configuration's
        ``max_position_embeddings`` (nothing in the kernels depends on it: rotation angles are computed
        from the position; it is the length the model was trained for, and the default refuses more)."""
        self.model = model
        self.options = options        # which kernel runs where there is a choice (this engine's steps only)
        self.device = model.device
        self._cuda = self.device.type == "cuda"   # kernels refuse anything else at their first launch
        max_seq_len = int(max_seq_len or model.spec.max_position)
        if max_seq_len > model.spec.max_position and not beyond_trained_positions:
            raise ValueError(f"max_seq_len {max_seq_len} exceeds the model's max_position_embeddings "
                             f"{model.spec.max_position}")
        self.max_batch = int(max_batch)
        if max_tokens is None:
            max_tokens = self.max_batch * round_up(max_seq_len, page_tokens)
        self.cache = SequenceCache(model.cache_needs, int(max_tokens), int(max_slots or self.max_batch),
                                   max_seq_len, model.dtype, self.device, page_tokens)
        self.max_seq_len = self.cache.max_seq_len
        self.use_cuda_graph = bool(use_cuda_graph)
        self._graphs: Dict[Tuple[int, int], "_DecodeGraph"] = {}      # in order of last use
        self._graph_state: Optional[_GraphBuffers] = None
        self._graph_pool = None      # one memory pool for all captured steps: they never run at the same time
        self._last_logits: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------ slots
    def open(self) -> int:
        return self.cache.alloc()

    def close(self, slot: int) -> None:
        self.cache.free(slot)
        if self._graph_state is not None:
            self._graph_state.invalidate()

    def fits(self, token_counts: Sequence[int]) -> bool:
        c = self.cache
        free_pages = min(len(g.pages) for g in c.groups if hasattr(g, "pages")) if any(
            hasattr(g, "pages") for g in c.groups) else c.n_pages
        pages = sum(-(-n // c.page_tokens) for n in token_counts)
        return len(token_counts) <= len(c.slots) and pages <= free_pages

    # ------------------------------------------------------------------ the step function
    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Runs the entries' tokens as one batch from the cache; returns float32
        logits ``[sum(len(e.want)), vocab]`` in the order of the entries and of
        each entry's ``want``."""
        slots = [e.slot for e in entries]
        q_lens = [len(e.tokens) for e in entries]
        self.cache.reserve(slots, q_lens)
        base = [self.cache.length(s) for s in slots]
        meta = BatchMeta.build(entries, base, self.device)
        logits = self.model.forward(meta, self.cache, self.options)
        self.cache.commit(slots, q_lens)
        if self._graph_state is not None:
            self._graph_state.invalidate()
        return logits

    # ------------------------------------------------------------------ sampling
    def _sampling_arrays(self, requests: Sequence[generation.Request]):
        n = len(requests)
        f = np.empty(2 * n, dtype=np.float32)
        i = np.empty(2 * n, dtype=np.int32)
        s = np.empty(n, dtype=np.int64)
        for j, r in enumerate(requests):
            f[j], f[n + j] = r.params.temperature, r.params.top_p
            i[j], i[n + j] = r.params.top_k, len(r.output)
            s[j] = request_seed(r.params.seed, r.index if r.request_id is None else r.request_id)
        return f, i, s

    def _upload(self, array: np.ndarray) -> torch.Tensor:
        t = torch.from_numpy(array)
        return t.pin_memory().to(self.device, non_blocking=True) if self._cuda else t

    def sample(self, logits: torch.Tensor, requests: Sequence[generation.Request]) -> torch.Tensor:
        n = len(requests)
        f, i, s = self._sampling_arrays(requests)
        fd, idev, sd = self._upload(f), self._upload(i), self._upload(s)
        return ops.sample(logits, fd[:n], idev[:n], fd[n:], sd, idev[n:], advance_index=False)

    # ------------------------------------------------------------------ backend of the generation loop
    def run(self, requests: Sequence[generation.Request], new_tokens: Sequence[Sequence[int]]) -> List[int]:
        decode = all(len(t) == 1 for t in new_tokens)
        if decode and self.use_cuda_graph and self._cuda:
            return self._run_graph(requests, new_tokens)
        entries = [StepEntry(r.slot, t, [len(t) - 1]) for r, t in zip(requests, new_tokens)]
        logits = self.step(entries)
        self._last_logits = logits
        toks = self.sample(logits, requests)
        out = toks.cpu().tolist()
        ops.check_status(self.device)
        return out

    def _run_graph(self, requests, new_tokens) -> List[int]:
        slots = [r.slot for r in requests]
        b = len(slots)
        self.cache.reserve(slots, [1] * b)
        if self._graph_state is None:
            self._graph_state = _GraphBuffers(self, max(self.max_batch, b))
        st = self._graph_state
        if st.capacity < b:
            # the captured steps read the old buffers: they go with them
            self._graphs.clear()
            self._last_logits = None
            self._graph_state = st = _GraphBuffers(self, b)
        # A captured step serves lengths up to `bucket`; the attention grid and its chunking
        # are fixed by it, so buckets are kept fine (512 keys) and a new graph is captured
        # when the longest sequence crosses one.
        longest = max(self.cache.length(s) for s in slots) + 1
        bucket = min(-(-longest // 512) * 512, self.max_seq_len)
        if st.slots != slots or st.bucket != bucket:
            st.upload(requests, bucket)
        # the step's input tokens come from the host every step, as the caller gives them
        st.host_in_np[:b] = [t[0] for t in new_tokens]
        st.tokens[:b].copy_(st.host_in[:b], non_blocking=True)
        key = (b, bucket)
        g = self._graphs.pop(key, None)
        if g is None:
            while len(self._graphs) >= MAX_CAPTURED_STEPS:            # drop the step that was used longest ago
                del self._graphs[next(iter(self._graphs))]
            g = _DecodeGraph(self, st, b, bucket)
        self._graphs[key] = g
        g.replay()
        self._last_logits = g.logits
        # one synchronisation for both read-backs: the sampled tokens and the kernels' status word
        st.host_tokens[:b].copy_(st.tokens[:b], non_blocking=True)
        st.host_status.copy_(ops.status_word(self.device), non_blocking=True)
        torch.cuda.current_stream().synchronize()
        self.cache.commit(slots, [1] * b)
        out = st.host_tokens[:b].tolist()
        if int(st.host_status[0]):
            ops.check_status(self.device)      # raises with the kernels' message and clears the word
        return out

    def last_logits(self) -> Optional[torch.Tensor]:
        """float32 logits ``[sequences, vocab]`` that the last ``run`` drew its tokens from, in the
        order of its requests (None before the first ``run``).  After a captured step this is the
        step's own output buffer, which any later captured step overwrites; the reference's graph
        runner hands out its static logits the same way (model/cuda_graph_decode.py:134-143)."""
        return self._last_logits

    # ------------------------------------------------------------------ generation
    def _stop_set(self, stop_token_ids, ignore_eos: bool) -> set:
        stop = set() if ignore_eos else set(self.model.spec.stop_token_ids)
        if stop_token_ids is not None:
            stop |= {int(t) for t in stop_token_ids}
        return stop

    def stream(self, prompts: Sequence[Sequence[int]], params=SamplingParams(), max_new_tokens=128,
               stop_token_ids: Optional[Iterable[int]] = None, ignore_eos: bool = False,
               request_ids: Optional[Sequence[int]] = None):
        """``generate`` as a generator: yields ``(prompt index, token id)`` as soon as each token is drawn."""
        return generation.stream(self, prompts, params, max_new_tokens, self._stop_set(stop_token_ids, ignore_eos),
                                 request_ids=request_ids)

    def generate(self, prompts: Sequence[Sequence[int]], params=SamplingParams(), max_new_tokens=128,
                 stop_token_ids: Optional[Iterable[int]] = None, ignore_eos: bool = False,
                 on_token: Optional[Callable[[int, int], None]] = None, return_stats: bool = False,
                 request_ids: Optional[Sequence[int]] = None):
        """Generates for every prompt (lists of token ids); returns the new tokens
        of each, and with ``return_stats`` also a dict with the keys of the
        reference's stats (generate.py:227-237).  ``request_ids``: one integer per prompt that keys
        its random stream together with the seed (default: the prompt's index in this call), so
        that a request can be repeated alone, or at another place of another call, and draw the same tokens."""
        stop = self._stop_set(stop_token_ids, ignore_eos)
        timings: dict = {}
        if self._cuda:
            torch.cuda.reset_peak_memory_stats(self.device)
        t0 = time.perf_counter()
        reqs = generation.generate(self, prompts, params, max_new_tokens, stop, on_token, timings,
                                   request_ids=request_ids)
        if self._cuda:
            torch.cuda.synchronize(self.device)
        wall = time.perf_counter() - t0
        outs = [r.output for r in reqs]
        if not return_stats:
            return outs
        prefill = timings.get("prefill_s", [])
        decode = timings.get("decode_s", [])
        new = sum(len(o) for o in outs)
        tpot = (sum(decode) / len(decode)) if decode else 0.0
        stats = {
            "prompt_tokens": sum(len(p) for p in prompts),
            "new_tokens": new,
            "ttft_ms": round(1e3 * prefill[0], 2) if prefill else 0.0,
            "tpot_ms": round(1e3 * tpot, 3),
            "prefill_ms": round(1e3 * sum(prefill), 2),
            "decode_tok_s": round(sum(timings.get("decode_seqs", [])) / sum(decode), 1) if decode and sum(decode) > 0 else 0.0,
            "total_wall_ms": round(1e3 * wall, 2),
            "total_tok_s": round((sum(len(p) for p in prompts) + new) / wall, 1) if wall > 0 else 0.0,
            "peak_vram_gb": round(torch.cuda.max_memory_allocated(self.device) / 1e9, 2) if self._cuda else 0.0,
            "finish_reasons": [r.finish_reason for r in reqs],
            # median step time right after the prompts and at the end: after a long prefill at the
            # power cap the clocks take some tens of milliseconds to come back
            "tpot_ms_first16": round(1e3 * sorted(decode[:16])[len(decode[:16]) // 2], 3) if decode else 0.0,
            "tpot_ms_last16": round(1e3 * sorted(decode[-16:])[len(decode[-16:]) // 2], 3) if decode else 0.0,
        }
        return outs, stats


class _GraphBuffers:
    """Static device buffers the captured decode step reads and writes."""

    def __init__(self, engine: Engine, capacity: int):
        dev = engine.device
        self.capacity = capacity
        z = lambda n, dt: torch.zeros(n, dtype=dt, device=dev)  # noqa: E731
        self.tokens = z(capacity, torch.int32)
        self.slot_ids = z(capacity, torch.int32)
        self.q_start = torch.arange(capacity + 1, dtype=torch.int32, device=dev)
        self.base_len = z(capacity, torch.int32)
        self.want_rows = torch.arange(capacity, dtype=torch.int32, device=dev)
        self.temperature = z(capacity, torch.float32)
        self.top_p = z(capacity, torch.float32)
        self.top_k = z(capacity, torch.int32)
        self.draw_index = z(capacity, torch.int32)
        self.seeds = z(capacity, torch.int64)
        self.host_tokens = torch.zeros(capacity, dtype=torch.int32).pin_memory()
        self.host_in = torch.zeros(capacity, dtype=torch.int32).pin_memory()
        self.host_in_np = self.host_in.numpy()       # the same pinned memory, written without a torch call per token
        self.host_status = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.engine = engine
        self.slots: Optional[List[int]] = None
        self.bucket = 0

    def invalidate(self) -> None:
        self.slots = None

    def upload(self, requests, bucket: int) -> None:
        eng = self.engine
        b = len(requests)
        f, i, s = eng._sampling_arrays(requests)
        ints = np.concatenate([np.asarray([r.slot for r in requests], dtype=np.int32),
                               np.asarray([eng.cache.length(r.slot) for r in requests], dtype=np.int32), i])
        ints_d, f_d, s_d = eng._upload(ints), eng._upload(f), eng._upload(s)
        self.slot_ids[:b].copy_(ints_d[0:b])
        self.base_len[:b].copy_(ints_d[b:2 * b])
        self.top_k[:b].copy_(ints_d[2 * b:3 * b])
        self.draw_index[:b].copy_(ints_d[3 * b:4 * b])
        self.temperature[:b].copy_(f_d[:b])
        self.top_p[:b].copy_(f_d[b:])
        self.seeds[:b].copy_(s_d)
        self.slots = [r.slot for r in requests]
        self.bucket = bucket


class _DecodeGraph:
    """One captured decode step for ``b`` sequences and keys up to ``bucket``."""

    def __init__(self, engine: Engine, st: _GraphBuffers, b: int, bucket: int):
        self.engine, self.st, self.b = engine, st, b
        meta = BatchMeta(st.slot_ids[:b], st.q_start[:b + 1], st.base_len[:b], st.tokens[:b], st.want_rows[:b],
                         n_seqs=b, n_tokens=b, n_want=b, max_q_len=1, max_kv_len=bucket, want_is_identity=True)
        self.meta = meta
        # One eager pass loads every kernel before the capture.  It writes the same
        # keys and values the first replay writes again and advances nothing.
        self._body(advance=False)
        torch.cuda.current_stream().synchronize()
        before = ops.launch_count
        self.graph = torch.cuda.CUDAGraph()
        # An engine and its graphs refer to each other, so a dropped engine waits for the cycle
        # collector; destroying its graphs while this stream captures would make the capture invalid.
        # The collector stays off until the capture has ended (a full collection here instead would
        # add some 60 ms to the first decode step of every batch size and length bucket).
        collector_on = gc.isenabled()
        gc.disable()
        if engine._graph_pool is None:
            engine._graph_pool = torch.cuda.graph_pool_handle()
        try:
            with torch.cuda.graph(self.graph, pool=engine._graph_pool):
                self._body(advance=True)
        finally:
            if collector_on:
                gc.enable()
        self.kernels = ops.launch_count - before
        ops.launch_count = before

    def _body(self, advance: bool) -> None:
        eng, st, b = self.engine, self.st, self.b
        logits = eng.model.forward(self.meta, eng.cache, eng.options)
        if advance:
            self.logits = logits
        ops.sample(logits, st.temperature[:b], st.top_k[:b], st.top_p[:b], st.seeds[:b], st.draw_index[:b],
                   advance_index=advance, out=st.tokens[:b] if advance else None)
        if advance:
            ops.advance_lengths(st.base_len[:b], st.q_start[:b + 1], b)

    def replay(self) -> None:
        self.graph.replay()
        ops.launch_count += self.kernels
