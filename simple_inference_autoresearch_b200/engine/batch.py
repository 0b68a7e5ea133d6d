"""Description of one step's batch, on the host and on the device.

A step carries, for each of B sequences, its slot, the number of tokens it
already holds (``base_len``) and its new tokens, packed without padding:
sequence b owns rows ``q_start[b] .. q_start[b+1]-1``; row t sits at position
``base_len[b] + t - q_start[b]``.  ``want_rows`` lists the packed rows whose
logits are asked for.  The reference can only express a rectangular ``(B, T)``
batch with one start position (model/llama.py:137-141).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence

import numpy as np
import torch


@dataclass
class StepEntry:
    """One sequence's share of a step: its slot, its next tokens, and the places
    among these tokens whose logits are wanted."""

    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


class BatchMeta:
    """Device arrays of a step plus the host numbers that size the launches."""

    def __init__(self, slot_ids, q_start, base_len, tokens, want_rows, n_seqs, n_tokens, n_want, max_q_len,
                 max_kv_len, want_is_identity, q_lens=None, base_lens=None, slots=None):
        self.slot_ids, self.q_start, self.base_len = slot_ids, q_start, base_len
        self.tokens, self.want_rows = tokens, want_rows
        self.n_seqs, self.n_tokens, self.n_want = n_seqs, n_tokens, n_want
        self.max_q_len, self.max_kv_len = max_q_len, max_kv_len
        self.is_decode = max_q_len == 1
        self.want_is_identity = want_is_identity
        # host copies, for parts written in plain Python (tests' toy mixers)
        self.q_lens, self.base_lens, self.slots = q_lens, base_lens, slots

    @classmethod
    def build(cls, entries: Sequence[StepEntry], base_lens: Sequence[int], device) -> "BatchMeta":
        b = len(entries)
        q_lens = [len(e.tokens) for e in entries]
        if b == 0 or min(q_lens) <= 0:
            raise ValueError("a step needs at least one sequence and every sequence at least one token")
        q_start = np.zeros(b + 1, dtype=np.int32)
        np.cumsum(q_lens, out=q_start[1:])
        n = int(q_start[-1])
        want: List[int] = []
        for i, e in enumerate(entries):
            for w in e.want:
                if not (0 <= w < q_lens[i]):
                    raise ValueError(f"want index {w} outside the {q_lens[i]} tokens of the entry")
                want.append(int(q_start[i]) + int(w))
        packed = np.concatenate([
            np.asarray([e.slot for e in entries], dtype=np.int32),
            q_start,
            np.asarray(base_lens, dtype=np.int32),
            np.asarray(want, dtype=np.int32),
            np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries]).astype(np.int32),
        ])
        host = torch.from_numpy(packed)
        dev = torch.device(device)
        if dev.type == "cuda":
            host = host.pin_memory()
        buf = host.to(dev, non_blocking=True)
        o = 0
        slot_ids = buf[o:o + b]; o += b
        q_start_d = buf[o:o + b + 1]; o += b + 1
        base_len = buf[o:o + b]; o += b
        want_rows = buf[o:o + len(want)]; o += len(want)
        tokens = buf[o:o + n]
        return cls(slot_ids, q_start_d, base_len, tokens, want_rows, b, n, len(want), max(q_lens),
                   max(bl + ql for bl, ql in zip(base_lens, q_lens)), want == list(range(n)),
                   q_lens=q_lens, base_lens=list(base_lens), slots=[e.slot for e in entries])
