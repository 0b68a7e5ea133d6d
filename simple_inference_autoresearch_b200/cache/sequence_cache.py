"""The cache: one slot per live sequence, keys and values per cache entry in pages,
and per-sequence state of fixed size.

The reference keeps two dense pools ``(layers, max_batch, kv_heads, max_seq_len,
head_dim)`` in which batch row b *is* the slot, one shared position for the whole
batch and a ``reset()`` that does nothing (model/kv_cache.py:126-128,178-198).
Here a sequence holds a *slot* (a small integer) with its own length; its keys
and values live in pages of ``page_tokens`` positions that the slot's row of a
block table names, so that memory is bounded by the tokens live requests hold
(each rounded up to a page), not by slots x longest sequence.  Slots and pages go
back to their free lists when a sequence ends and are handed out again.

Storage is organised in *groups*: every cache entry (one per position of the
model's run order that writes a cache) declares a need (``KVNeed`` or
``StateNeed``); entries with equal needs share a group, and each group owns its
pools, its block table and its page allocator, because groups differ in what they
must keep (all keys, or a window of them) and therefore in which pages they can
give back early.

All bookkeeping here is host-side Python and runs without a GPU; the device
tensors (pools, block tables) are only allocated and indexed.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..parts.base import KVNeed, StateNeed


#: positions per page of keys and values: the key tile of the tensor-core attention kernels
DEFAULT_PAGE_TOKENS = 64


class CacheError(RuntimeError):
    """Misuse or exhaustion of the cache (raised before anything is launched)."""


class FreeList:
    """Hands out integers ``0..n-1``; refuses a double free or a foreign id."""

    def __init__(self, n: int, what: str):
        self.n = n
        self.what = what
        self._free = list(range(n - 1, -1, -1))  # pop() yields the lowest id first
        self._held = [False] * n

    def __len__(self) -> int:
        return len(self._free)

    @property
    def held(self) -> int:
        return self.n - len(self._free)

    def take(self) -> int:
        if not self._free:
            raise CacheError(f"out of {self.what}s: all {self.n} are held")
        i = self._free.pop()
        self._held[i] = True
        return i

    def give(self, i: int) -> None:
        if not (0 <= i < self.n):
            raise CacheError(f"{self.what} {i} does not exist (0..{self.n - 1})")
        if not self._held[i]:
            raise CacheError(f"{self.what} {i} is not held (freed twice?)")
        self._held[i] = False
        self._free.append(i)

    def is_held(self, i: int) -> bool:
        return 0 <= i < self.n and self._held[i]


@dataclass
class KVEntry:
    """What a mixer sees of its cache entry: pools ``[n_pages, kv_heads,
    page_tokens, head_dim]`` and the group's block table ``[n_slots, max_pages]``."""

    k: torch.Tensor
    v: torch.Tensor
    block_table: torch.Tensor
    page_tokens: int


@dataclass
class StateEntry:
    """Fixed-size per-sequence state of one cache entry: ``[n_slots, *shape]``,
    zeroed when a slot is handed out."""

    state: torch.Tensor


class KVGroup:
    def __init__(self, need: KVNeed, n_entries: int, n_slots: int, n_pages: int, max_pages_per_seq: int,
                 page_tokens: int, dtype: torch.dtype, device):
        if need.window is not None and need.window <= 0:
            raise CacheError(f"a window of keys must be positive, got {need.window}")
        self.need = need
        self.n_entries = n_entries
        self.page_tokens = page_tokens
        self.max_pages_per_seq = max_pages_per_seq
        self.pages = FreeList(n_pages, "cache page")
        shape = (n_entries, n_pages, need.n_kv_heads, page_tokens)
        self.k = torch.zeros(shape + (need.head_dim,), dtype=dtype, device=device)
        self.v = torch.zeros(shape + (need.v_head_dim or need.head_dim,), dtype=dtype, device=device)
        # -1 marks "no page"; the cache-write kernel flags a write through it.
        self.block_table = torch.full((n_slots, max_pages_per_seq), -1, dtype=torch.int32, device=device)
        # per slot: the page of every page index so far; None once a windowed group gave it back
        self.slot_pages: Dict[int, List[Optional[int]]] = {}

    def entry(self, i: int) -> KVEntry:
        return KVEntry(self.k[i], self.v[i], self.block_table, self.page_tokens)

    def open_slot(self, slot: int) -> None:
        self.slot_pages[slot] = []

    def pages_needed(self, slot: int, new_len: int) -> int:
        have = len(self.slot_pages[slot])
        return max(0, -(-new_len // self.page_tokens) - have)

    def grow(self, slot: int, new_len: int) -> List[Tuple[int, int, int]]:
        """Makes room for ``new_len`` positions; returns (slot, page index, page) rows to upload."""
        pages = self.slot_pages[slot]
        need = -(-new_len // self.page_tokens)
        if need > self.max_pages_per_seq:
            raise CacheError(f"sequence of {new_len} tokens exceeds the longest sequence the cache was "
                             f"built for ({self.max_pages_per_seq * self.page_tokens} tokens)")
        added = []
        while len(pages) < need:
            p = self.pages.take()
            added.append((slot, len(pages), p))
            pages.append(p)
        return added

    def release_before(self, slot: int, length: int) -> List[Tuple[int, int, int]]:
        """A group with a window: after the sequence has reached ``length`` tokens, the next query
        (position ``length``) sees keys from ``length - window + 1`` on, so pages that lie wholly in
        front of that are given back.  Returns (slot, page index, -1) rows for the block table."""
        if self.need.window is None:
            return []
        first_needed = max(0, length - self.need.window + 1)
        pages = self.slot_pages[slot]
        cells = []
        for idx in range(min(first_needed // self.page_tokens, len(pages))):
            if pages[idx] is not None:
                self.pages.give(pages[idx])
                pages[idx] = None
                cells.append((slot, idx, -1))
        return cells

    def held_pages(self, slot: int) -> int:
        return sum(p is not None for p in self.slot_pages[slot])

    def close_slot(self, slot: int) -> List[Tuple[int, int, int]]:
        """Gives the slot's pages back; returns (slot, page index, -1) rows for the block table, so
        that the next sequence in this slot finds no page number of this one beyond its own length
        (a read past the reserved pages then meets -1 and is reported)."""
        pages = self.slot_pages.pop(slot)
        for p in pages:
            if p is not None:
                self.pages.give(p)
        return [(slot, idx, -1) for idx, p in enumerate(pages) if p is not None]

    def bytes(self) -> int:
        return (self.k.numel() + self.v.numel()) * self.k.element_size()


class StateGroup:
    def __init__(self, need: StateNeed, n_entries: int, n_slots: int, device):
        self.need = need
        self.n_entries = n_entries
        dtype = getattr(torch, need.dtype)
        self.state = torch.zeros((n_entries, n_slots) + tuple(need.shape), dtype=dtype, device=device)

    def entry(self, i: int) -> StateEntry:
        return StateEntry(self.state[i])

    def open_slot(self, slot: int) -> None:
        self.state[:, slot].zero_()

    def bytes(self) -> int:
        return self.state.numel() * self.state.element_size()


def round_up(n: int, m: int) -> int:
    return -(-n // m) * m


class SequenceCache:
    """All groups of one model plus the slot allocator and each slot's length.

    ``needs``: one need (or None) per cache entry, in the model's entry order.
    ``max_tokens``: the most positions live sequences hold at any time, each
    sequence's count rounded up to ``page_tokens``.
    """

    def __init__(self, needs: Sequence[object], max_tokens: int, max_slots: int, max_seq_len: int,
                 dtype: torch.dtype, device, page_tokens: int = DEFAULT_PAGE_TOKENS):
        if max_tokens <= 0 or max_slots <= 0 or max_seq_len <= 0:
            raise CacheError("max_tokens, max_slots and max_seq_len must be positive")
        self.page_tokens = page_tokens
        self.n_pages = -(-max_tokens // page_tokens)
        self.n_slots = min(max_slots, self.n_pages)
        # the caller's limit stands as given (only the page count is rounded up)
        self.max_seq_len = min(int(max_seq_len), self.n_pages * page_tokens)
        self.dtype, self.device = dtype, device
        self.slots = FreeList(self.n_slots, "cache slot")
        self.lengths: Dict[int, int] = {}
        self.groups: List[object] = []
        self._entry_ref: List[Optional[Tuple[int, int]]] = []  # entry -> (group, index in group)
        by_need: Dict[object, List[int]] = {}
        for e, need in enumerate(needs):
            if need is not None:
                by_need.setdefault(need, []).append(e)
        self._entry_ref = [None] * len(needs)
        for need, entries in by_need.items():
            if isinstance(need, KVNeed):
                g = KVGroup(need, len(entries), self.n_slots, self.n_pages,
                            -(-self.max_seq_len // page_tokens), page_tokens, dtype, device)
            elif isinstance(need, StateNeed):
                g = StateGroup(need, len(entries), self.n_slots, device)
            else:
                raise TypeError(f"unknown cache need {need!r}")
            for i, e in enumerate(entries):
                self._entry_ref[e] = (len(self.groups), i)
            self.groups.append(g)

    # ---- what mixers see
    def entry(self, e: int):
        ref = self._entry_ref[e]
        if ref is None:
            return None
        g, i = ref
        return self.groups[g].entry(i)

    # ---- slots
    def alloc(self) -> int:
        slot = self.slots.take()
        self.lengths[slot] = 0
        for g in self.groups:
            g.open_slot(slot)
        return slot

    def free(self, slot: int) -> None:
        if not self.slots.is_held(slot):
            raise CacheError(f"cache slot {slot} is not held (freed twice?)")
        for g in self.groups:
            if isinstance(g, KVGroup):
                self._upload_cells(g, g.close_slot(slot))
        del self.lengths[slot]
        self.slots.give(slot)

    def length(self, slot: int) -> int:
        return self.lengths[slot]

    def live_slots(self) -> List[int]:
        return sorted(self.lengths)

    # ---- growth, before a step is launched
    def reserve(self, slots: Sequence[int], new_tokens: Sequence[int]) -> None:
        """Gives every sequence of the step the pages its new tokens need and
        uploads the changed block-table cells.  Raises before changing anything
        if the pages do not suffice."""
        if len(set(slots)) != len(slots):
            raise CacheError("a slot appears twice in one step")
        for s in slots:
            if s not in self.lengths:
                raise CacheError(f"cache slot {s} is not held")
        for g in self.groups:
            if not isinstance(g, KVGroup):
                continue
            want = 0
            for s, n in zip(slots, new_tokens):
                new_len = self.lengths[s] + n
                if new_len > self.max_seq_len:
                    raise CacheError(f"sequence in slot {s} would reach {new_len} tokens; the cache holds "
                                     f"sequences of up to {self.max_seq_len}")
                want += g.pages_needed(s, new_len)
            if want > len(g.pages):
                raise CacheError(f"the step needs {want} more cache pages of {self.page_tokens} tokens but only "
                                 f"{len(g.pages)} of {g.pages.n} are free")
        for g in self.groups:
            if not isinstance(g, KVGroup):
                continue
            cells = []
            for s, n in zip(slots, new_tokens):
                cells += g.grow(s, self.lengths[s] + n)
            self._upload_cells(g, cells)

    def _upload_cells(self, g: "KVGroup", cells) -> None:
        if not cells:
            return
        if torch.device(self.device).type == "cuda":
            from ..kernels import ops
            triples = torch.tensor([[c[0], c[1], c[2]] for c in cells], dtype=torch.int32)
            ops.set_table_cells(g.block_table, triples.pin_memory().to(self.device, non_blocking=True))
            return
        idx = torch.tensor([[c[0], c[1]] for c in cells], dtype=torch.int64)
        g.block_table[idx[:, 0], idx[:, 1]] = torch.tensor([c[2] for c in cells], dtype=torch.int32)

    def commit(self, slots: Sequence[int], new_tokens: Sequence[int]) -> None:
        """The step ran: lengths advance, and groups that keep a window of keys give back the
        pages that no later query can see."""
        for s, n in zip(slots, new_tokens):
            self.lengths[s] += n
        for g in self.groups:
            if isinstance(g, KVGroup) and g.need.window is not None:
                cells = []
                for s in slots:
                    cells += g.release_before(s, self.lengths[s])
                self._upload_cells(g, cells)

    # ---- accounting
    def held_tokens(self) -> int:
        return sum(round_up(n, self.page_tokens) for n in self.lengths.values())

    def bytes(self) -> int:
        return sum(g.bytes() for g in self.groups)
