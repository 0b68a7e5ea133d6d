"""Slots and pages: none lost, none held twice, none freed twice; lengths per
sequence; groups with storage of their own; fixed-size state (no GPU)."""

import random

import pytest
import torch

from simple_inference_autoresearch_b200.cache import CacheError, FreeList, SequenceCache
from simple_inference_autoresearch_b200.parts.base import KVNeed, StateNeed


def make(needs=None, max_tokens=640, max_slots=4, max_seq_len=256):
    needs = needs if needs is not None else [KVNeed(2, 16), KVNeed(2, 16)]
    return SequenceCache(needs, max_tokens, max_slots, max_seq_len, torch.float32, "cpu")


def test_free_list_refuses_double_free_and_foreign_ids():
    fl = FreeList(3, "thing")
    a, b, c = fl.take(), fl.take(), fl.take()
    assert sorted([a, b, c]) == [0, 1, 2]
    with pytest.raises(CacheError, match="out of things"):
        fl.take()
    fl.give(b)
    with pytest.raises(CacheError, match="not held"):
        fl.give(b)
    with pytest.raises(CacheError, match="does not exist"):
        fl.give(7)
    assert fl.take() == b and fl.held == 3


def test_slots_and_pages_survive_random_traffic():
    c = make(max_tokens=64 * 12, max_slots=5, max_seq_len=64 * 6)
    kv = c.groups[0]
    rng = random.Random(0)
    live = {}
    for _ in range(2000):
        op = rng.random()
        if op < 0.3 and len(live) < c.n_slots:
            s = c.alloc()
            assert s not in live
            live[s] = 0
        elif op < 0.8 and live:
            s = rng.choice(list(live))
            n = rng.randint(1, 70)
            try:
                c.reserve([s], [n])
            except CacheError:
                continue
            c.commit([s], [n])
            live[s] += n
        elif live:
            s = rng.choice(list(live))
            c.free(s)
            del live[s]
        # invariants: every page is either free or in exactly one slot's list
        held = [p for pages in kv.slot_pages.values() for p in pages]
        assert len(held) == len(set(held)) == kv.pages.held
        assert kv.pages.held + len(kv.pages) == kv.pages.n
        assert c.slots.held == len(live) and set(c.lengths) == set(live)
        for s, n in live.items():
            assert c.length(s) == n and len(kv.slot_pages[s]) == -(-n // 64)
            assert kv.block_table[s, :len(kv.slot_pages[s])].tolist() == kv.slot_pages[s]
    for s in list(live):
        c.free(s)
    assert kv.pages.held == 0 and c.slots.held == 0


def test_double_free_and_unknown_slot():
    c = make()
    s = c.alloc()
    c.free(s)
    with pytest.raises(CacheError, match="not held"):
        c.free(s)
    with pytest.raises(CacheError, match="not held"):
        c.reserve([s], [1])
    a = c.alloc()
    with pytest.raises(CacheError, match="twice"):
        c.reserve([a, a], [1, 1])


def test_reserve_is_all_or_nothing():
    c = make(max_tokens=64 * 3, max_slots=3, max_seq_len=192)
    a, b = c.alloc(), c.alloc()
    c.reserve([a], [100]); c.commit([a], [100])          # two of three pages
    with pytest.raises(CacheError, match="more cache pages"):
        c.reserve([a, b], [30, 10])                       # needs 1 (a: 130 > 128) + 1 (b)
    assert c.groups[0].pages.held == 2 and c.groups[0].slot_pages[b] == []
    c.reserve([b], [10])
    with pytest.raises(CacheError, match="holds sequences of up to"):
        c.reserve([a], [200])


def test_max_tokens_counts_each_sequence_rounded_up_to_a_page():
    c = make(max_tokens=256, max_slots=8, max_seq_len=256)
    slots = [c.alloc() for _ in range(4)]
    c.reserve(slots, [1, 64, 33, 5]); c.commit(slots, [1, 64, 33, 5])
    assert c.held_tokens() == 256
    with pytest.raises(CacheError):
        c.reserve([slots[1]], [1])
    c.free(slots[0])
    c.reserve([slots[1]], [1])


def test_groups_by_need_and_state_is_zeroed_on_alloc():
    needs = [KVNeed(2, 16), StateNeed((3, 5)), KVNeed(1, 32), KVNeed(2, 16), None, StateNeed((3, 5))]
    c = make(needs)
    kinds = [(type(g).__name__, g.n_entries) for g in c.groups]
    assert sorted(kinds) == [("KVGroup", 1), ("KVGroup", 2), ("StateGroup", 2)]
    assert c.entry(4) is None
    assert c.entry(0).k.shape == (c.n_pages, 2, 64, 16) and c.entry(2).k.shape == (c.n_pages, 1, 64, 32)
    assert c.entry(0).k.data_ptr() != c.entry(3).k.data_ptr()
    assert c.entry(0).block_table.data_ptr() == c.entry(3).block_table.data_ptr()   # same group
    assert c.entry(0).block_table.data_ptr() != c.entry(2).block_table.data_ptr()   # own storage
    s = c.alloc()
    st = c.entry(1).state
    assert st.shape == (c.n_slots, 3, 5)
    st[s] += 7.0
    c.entry(5).state[s] += 1.0
    c.free(s)
    s2 = c.alloc()
    assert s2 == s and torch.all(c.entry(1).state[s2] == 0) and torch.all(c.entry(5).state[s2] == 0)


def test_a_window_group_keeps_its_own_pages_and_gives_back_what_no_query_can_see():
    """Two groups from two needs (all keys / the last 100): same slots, storage of their own.  The
    windowed one frees a page as soon as the next query's window starts behind it, marks the cell
    -1, never frees twice, and ends with every page free."""
    c = make([KVNeed(2, 16), KVNeed(2, 16, window=100), KVNeed(2, 16, window=100)], max_tokens=1280, max_seq_len=640)
    assert len(c.groups) == 2 and c.groups[1].n_entries == 2
    full, win = c.groups
    a, b = c.alloc(), c.alloc()
    c.reserve([a, b], [300, 70]); c.commit([a, b], [300, 70])
    # a: next query at 300 sees keys 201..300 -> pages 0..2 (keys 0..191) are gone, 3 and 4 stay
    assert [p is None for p in win.slot_pages[a]] == [True, True, True, False, False]
    assert [p is None for p in win.slot_pages[b]] == [False, False]
    assert win.block_table[a, :5].tolist()[:3] == [-1, -1, -1] and win.block_table[a, 3] >= 0
    assert full.held_pages(a) == 5 and win.held_pages(a) == 2
    for _ in range(200):                      # one token at a time: at most ceil(100/64) + 1 pages stay
        c.reserve([a, b], [1, 1]); c.commit([a, b], [1, 1])
        assert win.held_pages(a) <= 3 and win.held_pages(b) <= 3
    assert c.length(a) == 500 and full.held_pages(a) == 8
    free_before = len(win.pages)
    c.free(a)
    assert len(win.pages) > free_before
    c.free(b)
    assert len(win.pages) == win.pages.n and len(full.pages) == full.pages.n
    with pytest.raises(CacheError, match="positive"):
        make([KVNeed(2, 16, window=0)])


# ----------------------------------------------------------------------------- the argument checks of the debugging mode
def _fake_launch(slot_ids, q_start, base_len, table, n_pages=6, page=4, max_q_len=None, max_kv_len=None):
    from types import SimpleNamespace
    i32 = lambda v: torch.tensor(v, dtype=torch.int32)  # noqa: E731
    kv = SimpleNamespace(k=torch.zeros(n_pages, 2, page, 8), v=torch.zeros(n_pages, 2, page, 8),
                         block_table=i32(table), page_tokens=page)
    q_lens = [b - a for a, b in zip(q_start, q_start[1:])]
    meta = SimpleNamespace(n_seqs=len(slot_ids), slot_ids=i32(slot_ids), q_start=i32(q_start), base_len=i32(base_len),
                           max_q_len=max_q_len or max(q_lens + [1]),
                           max_kv_len=max_kv_len or max([b + q for b, q in zip(base_len, q_lens)] + [1]))
    return kv, meta


def test_argument_checks_name_the_first_index_that_leaves_its_tensor():
    from simple_inference_autoresearch_b200.kernels.ops import check_batch
    table = [[0, 1, -1], [2, 3, 4], [-1, 5, -1]]
    good = dict(slot_ids=[1, 0], q_start=[0, 3, 4], base_len=[6, 4], table=table)
    check_batch(*_fake_launch(**good), n_rows=4, writes=True)                    # nothing to say
    cases = [
        (dict(good, slot_ids=[3, 0]), "slot_ids[0] = 3"),
        (dict(good, q_start=[0, 3, 3]), "non-empty runs"),
        (dict(good, q_start=[0, 3, 5]), "non-empty runs"),                        # more rows than the tensor has
        (dict(good, base_len=[10, 4]), "do not fit the block table"),
        (dict(good, base_len=[6, 8]), "holds no page for keys 8..11"),            # slot 0 has two pages
        (dict(good, table=[[0, 1, -1], [2, 9, 4], [-1, 5, -1]]), "block_table[1, 1] = 9 is no page"),
        (dict(good, max_kv_len=8), "sized for max_kv_len = 8"),
        (dict(good, max_q_len=2), "sized for max_q_len = 2"),
    ]
    for args, message in cases:
        with pytest.raises(ValueError, match=message.replace("[", r"\[").replace("]", r"\]")):
            check_batch(*_fake_launch(**args), n_rows=4, writes=True)
    # a window of keys: older pages may have been given back, the ones in sight may not
    windowed = dict(slot_ids=[2], q_start=[0, 1], base_len=[6], table=table)
    check_batch(*_fake_launch(**windowed), n_rows=1, writes=True, window=3)
    with pytest.raises(ValueError, match="holds no page for keys 0..3"):
        check_batch(*_fake_launch(**windowed), n_rows=1, writes=True, window=4)
    with pytest.raises(ValueError, match="holds no page for keys 0..3"):
        check_batch(*_fake_launch(**windowed), n_rows=1, writes=True)
