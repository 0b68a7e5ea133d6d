"""The generation loop: requests -> batches -> prefill step -> decode steps.

For one request it behaves as the reference's loop (generate.py:122-238): a
capacity check on the prompt, one prefill step whose last position gives the
first token, then one token per step until ``max_new_tokens`` tokens exist, a
stop token is drawn (it is not emitted, generate.py:208-209) or the cache is
full (generate.py:194-195).  Unlike the reference's streaming variant, which
never yields the token sampled from the prefill (generate.py:95-119), every
token is emitted.

What the reference does not have is decided here: requests are cut into batches
that start together; a batch's prompts have unequal lengths and go through ONE
prefill step without padding; a sequence that ends leaves the batch and gives
its slot back at once; when a batch is done the next one starts, reusing the
slots.  The loop only decides; running a step and drawing tokens is the
backend's business (``Engine`` on the GPU, a scripted fake in the CPU tests).
"""

from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, Iterable, Iterator, List, Optional, Protocol, Sequence, Tuple

from ..sampling.params import SamplingParams


@dataclass
class Request:
    prompt: Sequence[int]
    max_new_tokens: int
    params: SamplingParams
    index: int = 0
    request_id: Optional[int] = None      # keys the request's random stream with its seed; None: the index
    # filled by the loop
    output: List[int] = field(default_factory=list)
    finish_reason: Optional[str] = None   # "stop" | "length" | "capacity"
    slot: Optional[int] = None


class Backend(Protocol):
    max_batch: int
    max_seq_len: int

    def fits(self, token_counts: Sequence[int]) -> bool: ...
    def open(self) -> int: ...
    def close(self, slot: int) -> None: ...
    def run(self, requests: Sequence[Request], new_tokens: Sequence[Sequence[int]]) -> List[int]: ...


def plan_batches(requests: Sequence[Request], backend: Backend) -> List[List[Request]]:
    """Cuts the requests, in order, into batches that start together: at most
    ``max_batch`` sequences, and together no more cache than the backend has when
    every member grows to its prompt plus ``max_new_tokens``."""
    batches: List[List[Request]] = []
    cur: List[Request] = []
    for r in requests:
        if len(r.prompt) == 0:
            raise ValueError(f"request {r.index} has an empty prompt")
        if len(r.prompt) >= backend.max_seq_len:
            raise ValueError(f"Prompt length {len(r.prompt)} exceeds cache capacity {backend.max_seq_len} "
                             f"(request {r.index})")
        need = lambda rs: [min(len(x.prompt) + x.max_new_tokens, backend.max_seq_len) for x in rs]  # noqa: E731
        if cur and (len(cur) >= backend.max_batch or not backend.fits(need(cur + [r]))):
            batches.append(cur)
            cur = []
        if not backend.fits(need([r])):
            raise ValueError(f"request {r.index} alone needs more cache than there is")
        cur.append(r)
    if cur:
        batches.append(cur)
    return batches


def run_batch(batch: List[Request], backend: Backend, stop_ids: frozenset,
              on_token: Optional[Callable[[int, int], None]] = None, timings: Optional[dict] = None) -> None:
    for index, tok in iter_batch(batch, backend, stop_ids, timings):
        if on_token is not None:
            on_token(index, tok)


def iter_batch(batch: List[Request], backend: Backend, stop_ids: frozenset,
               timings: Optional[dict] = None) -> Iterator[Tuple[int, int]]:
    """Runs one batch and yields ``(request index, token)`` as each token is drawn.  When the
    consumer stops early (the generator is closed), the slots still held are given back."""
    live = list(batch)
    for r in live:
        r.slot = backend.open()
    try:
        feed = [list(r.prompt) for r in live]
        first = True
        while live:
            t0 = time.perf_counter()
            drawn = backend.run(live, feed)
            if timings is not None:
                timings.setdefault("prefill_s" if first else "decode_s", []).append(time.perf_counter() - t0)
                timings.setdefault("prefill_seqs" if first else "decode_seqs", []).append(len(live))
            first = False
            nxt_live, nxt_feed = [], []
            for r, tok in zip(live, drawn):
                tok = int(tok)
                if tok in stop_ids:
                    r.finish_reason = "stop"
                else:
                    r.output.append(tok)
                    yield r.index, tok
                    if len(r.output) >= r.max_new_tokens:
                        r.finish_reason = "length"
                    elif len(r.prompt) + len(r.output) >= backend.max_seq_len:
                        r.finish_reason = "capacity"
                if r.finish_reason is None:
                    nxt_live.append(r)
                    nxt_feed.append([tok])
                else:
                    backend.close(r.slot)
                    r.slot = None
            live, feed = nxt_live, nxt_feed
    finally:
        for r in batch:
            if r.slot is not None:
                backend.close(r.slot)
                r.slot = None


def generate(backend: Backend, prompts: Sequence[Sequence[int]], params, max_new_tokens, stop_token_ids: Iterable[int] = (),
             on_token: Optional[Callable[[int, int], None]] = None, timings: Optional[dict] = None,
             request_ids: Optional[Sequence[int]] = None) -> List[Request]:
    """Runs all requests, batch after batch; returns them with ``output`` and
    ``finish_reason`` filled.  ``params`` and ``max_new_tokens`` are one value for
    all requests or one per request."""
    requests = make_requests(prompts, params, max_new_tokens, request_ids)
    stop = frozenset(int(t) for t in stop_token_ids)
    for batch in plan_batches([r for r in requests if r.finish_reason is None], backend):
        run_batch(batch, backend, stop, on_token, timings)
    return requests


def stream(backend: Backend, prompts: Sequence[Sequence[int]], params, max_new_tokens,
           stop_token_ids: Iterable[int] = (), timings: Optional[dict] = None,
           request_ids: Optional[Sequence[int]] = None) -> Iterator[Tuple[int, int]]:
    """The same loop as a generator: yields ``(request index, token)`` the moment a token exists
    (the reference streams its single request the same way, generate.py:50-119)."""
    requests = make_requests(prompts, params, max_new_tokens, request_ids)
    stop = frozenset(int(t) for t in stop_token_ids)
    for batch in plan_batches([r for r in requests if r.finish_reason is None], backend):
        yield from iter_batch(batch, backend, stop, timings)


def make_requests(prompts: Sequence[Sequence[int]], params, max_new_tokens,
                  request_ids: Optional[Sequence[int]] = None) -> List[Request]:
    n = len(prompts)
    if request_ids is not None and len(request_ids) != n:
        raise ValueError("request_ids must hold one id per prompt")
    plist = list(params) if isinstance(params, (list, tuple)) else [params] * n
    mlist = list(max_new_tokens) if isinstance(max_new_tokens, (list, tuple)) else [max_new_tokens] * n
    if len(plist) != n or len(mlist) != n:
        raise ValueError("params / max_new_tokens must be one value or one per prompt")
    requests = [Request(list(p), int(m), sp, index=i, request_id=None if request_ids is None else int(request_ids[i]))
                for i, (p, m, sp) in enumerate(zip(prompts, mlist, plist))]
    for r in requests:
        if r.max_new_tokens <= 0:
            r.finish_reason = "length"
    return requests
