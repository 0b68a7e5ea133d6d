"""The generation loop's decisions with a scripted backend (no GPU): how requests
are cut into batches, what a step is fed, when a sequence ends, that slots are
given back at once and used again, and that the stop token is not emitted."""

import pytest

from simple_inference_autoresearch_b200.engine import generation
from simple_inference_autoresearch_b200.sampling import GREEDY, SamplingParams


class ScriptedBackend:
    """Draws token ``script[request][n]`` as the n-th token of a request and logs every call."""

    def __init__(self, script, max_batch=2, max_seq_len=64, page=8, pages=16):
        self.script, self.max_batch, self.max_seq_len = script, max_batch, max_seq_len
        self.page, self.pages = page, pages
        self.free = list(range(max_batch))[::-1]
        self.held, self.log, self.lengths = set(), [], {}

    def fits(self, counts):
        return len(counts) <= len(self.free) and sum(-(-c // self.page) for c in counts) <= self.pages

    def open(self):
        s = self.free.pop()
        assert s not in self.held
        self.held.add(s)
        self.lengths[s] = 0
        self.log.append(("open", s))
        return s

    def close(self, slot):
        assert slot in self.held, "slot freed twice"
        self.held.remove(slot)
        self.free.append(slot)
        self.log.append(("close", slot))

    def run(self, requests, new_tokens):
        assert len({r.slot for r in requests}) == len(requests)
        self.log.append(("run", [r.index for r in requests], [list(t) for t in new_tokens]))
        out = []
        for r, t in zip(requests, new_tokens):
            assert r.slot in self.held
            self.lengths[r.slot] += len(t)
            out.append(self.script[r.index][len(r.output)])
        return out


def runs(backend):
    return [e for e in backend.log if e[0] == "run"]


def test_prompts_go_in_one_step_then_one_token_each():
    be = ScriptedBackend({0: [10, 11, 12], 1: [20, 21, 22]})
    reqs = generation.generate(be, [[1, 2, 3], [4]], GREEDY, 3)
    assert [r.output for r in reqs] == [[10, 11, 12], [20, 21, 22]]
    assert [r.finish_reason for r in reqs] == ["length", "length"]
    assert runs(be) == [("run", [0, 1], [[1, 2, 3], [4]]), ("run", [0, 1], [[10], [20]]),
                        ("run", [0, 1], [[11], [21]])]
    assert not be.held


def test_stop_token_ends_a_sequence_is_not_emitted_and_frees_the_slot_at_once():
    be = ScriptedBackend({0: [10, 99, 12, 13], 1: [20, 21, 22, 23]})
    reqs = generation.generate(be, [[1, 2], [3]], GREEDY, 4, stop_token_ids=[99])
    assert reqs[0].output == [10] and reqs[0].finish_reason == "stop"
    assert reqs[1].output == [20, 21, 22, 23]
    r = runs(be)
    assert r[1] == ("run", [0, 1], [[10], [20]]) and r[2] == ("run", [1], [[21]]) and len(r) == 4
    i_close = be.log.index(("close", 0))
    assert be.log.index(r[1]) < i_close < be.log.index(r[2])   # freed before the next step


def test_stop_at_the_first_token():
    be = ScriptedBackend({0: [99], 1: [5, 99]})
    reqs = generation.generate(be, [[1], [2]], GREEDY, 5, stop_token_ids={99})
    assert [r.output for r in reqs] == [[], [5]] and len(runs(be)) == 2


def test_batches_follow_one_another_and_reuse_slots():
    script = {i: [100 + i] * 5 for i in range(5)}
    be = ScriptedBackend(script, max_batch=2)
    lens = [2, 1, 3, 1, 2]
    reqs = generation.generate(be, [[1]] * 5, GREEDY, lens)
    assert [len(r.output) for r in reqs] == lens
    firsts = [e for e in runs(be) if any(len(t) == 1 and t[0] == 1 for t in e[2])]
    assert [e[1] for e in firsts] == [[0, 1], [2, 3], [4]]
    opens = [e[1] for e in be.log if e[0] == "open"]
    assert set(opens) == {0, 1} and len(opens) == 5
    # no batch starts before the one before it has ended
    for a, b in zip(firsts, firsts[1:]):
        between = be.log[be.log.index(a):be.log.index(b)]
        assert sum(e[0] == "close" for e in between) >= len(a[1])


def test_batches_respect_the_cache_budget():
    be = ScriptedBackend({i: [7] * 4 for i in range(3)}, max_batch=3, page=8, pages=4)
    generation.generate(be, [[1] * 12, [1] * 10, [1] * 3], GREEDY, 4)     # 2 + 2 + 1 pages
    firsts = [e[1] for e in runs(be) if len(e[2][0]) > 1]
    assert firsts == [[0, 1], [2]]
    with pytest.raises(ValueError, match="alone needs more cache"):
        generation.generate(ScriptedBackend({0: [1]}, pages=1), [[1] * 20], GREEDY, 4)


def test_capacity_and_prompt_checks():
    be = ScriptedBackend({0: [7] * 100}, max_seq_len=8, pages=100)
    with pytest.raises(ValueError, match="exceeds cache capacity"):
        generation.generate(be, [[1] * 8], GREEDY, 4)
    with pytest.raises(ValueError, match="empty prompt"):
        generation.generate(be, [[]], GREEDY, 4)
    reqs = generation.generate(be, [[1] * 5], GREEDY, 50)
    assert reqs[0].finish_reason == "capacity" and len(reqs[0].output) == 3   # 5 + 3 == 8
    assert generation.generate(be, [[1]], GREEDY, 0)[0].output == []


def test_per_request_params_and_callbacks():
    be = ScriptedBackend({0: [1, 2], 1: [3, 4]})
    seen = []
    ps = [SamplingParams(temperature=0.0), SamplingParams(temperature=0.8, seed=3)]
    reqs = generation.generate(be, [[9], [9]], ps, [2, 1], on_token=lambda i, t: seen.append((i, t)))
    assert reqs[1].params.seed == 3 and seen == [(0, 1), (1, 3), (0, 2)]
    with pytest.raises(ValueError):
        generation.generate(be, [[9], [9]], ps[:1] * 3, 2)
    with pytest.raises(ValueError, match="temperature"):
        SamplingParams(temperature=-1.0)


def test_slots_are_freed_when_a_step_raises():
    class Boom(ScriptedBackend):
        def run(self, requests, new_tokens):
            if len(runs(self)) == 1:
                raise RuntimeError("boom")
            return super().run(requests, new_tokens)
    be = Boom({0: [1, 2], 1: [3, 4]})
    with pytest.raises(RuntimeError, match="boom"):
        generation.generate(be, [[9], [9]], GREEDY, 2)
    assert not be.held


def test_stream_yields_each_token_when_it_is_drawn_and_gives_slots_back_when_abandoned():
    script = {0: [10, 11, 12], 1: [20, 99, 22], 2: [30, 31, 32]}
    be = ScriptedBackend(script)
    seen = []
    for index, tok in generation.stream(be, [[1, 2, 3], [4], [5, 6]], GREEDY, 3, stop_token_ids=[99]):
        seen.append((index, tok, len(runs(be))))          # how many steps had run when the token came out
    assert seen == [(0, 10, 1), (1, 20, 1), (0, 11, 2), (0, 12, 3), (2, 30, 4), (2, 31, 5), (2, 32, 6)]
    assert not be.held
    # the same tokens as the loop that returns everything at the end
    be2 = ScriptedBackend(script)
    reqs = generation.generate(be2, [[1, 2, 3], [4], [5, 6]], GREEDY, 3, stop_token_ids=[99])
    assert [r.output for r in reqs] == [[10, 11, 12], [20], [30, 31, 32]] and be2.log == be.log
    # a consumer that stops after the first token: the batch's slots are closed with the generator
    be3 = ScriptedBackend(script)
    it = generation.stream(be3, [[1, 2, 3], [4]], GREEDY, 3)
    assert next(it) == (0, 10) and be3.held
    it.close()
    assert not be3.held


def test_random_traffic_keeps_the_loops_promises():
    """Random prompts, budgets and stop tokens: every request gets its script's tokens up to the first stop
    token, its budget or the cache's capacity; a prompt is fed once and whole; every later step feeds each live
    request the token it drew last; no step holds more requests than the backend allows; every slot comes back."""
    from hypothesis import given, settings, strategies as st

    @settings(max_examples=80, deadline=None)
    @given(st.lists(st.tuples(st.integers(1, 20), st.integers(0, 9)), min_size=1, max_size=9),
           st.integers(1, 4), st.randoms(use_true_random=False))
    def check(shape, max_batch, rnd):
        n = len(shape)
        prompts = [[rnd.randrange(3, 50) for _ in range(p)] for p, _ in shape]
        budgets = [m for _, m in shape]
        script = {i: [rnd.choice([1, 2, 60, 61, 62, 63]) for _ in range(12)] for i in range(n)}
        stop = {1, 2}
        max_seq_len = 24
        be = ScriptedBackend(script, max_batch=max_batch, max_seq_len=max_seq_len, page=8, pages=3 * max_batch)
        reqs = generation.generate(be, prompts, GREEDY, budgets, stop_token_ids=stop)
        assert not be.held and sorted(be.free) == list(range(max_batch))
        drawn = {i: 0 for i in range(n)}              # tokens request i has drawn so far
        for _, indices, feeds in runs(be):
            assert 1 <= len(indices) <= max_batch and len(set(indices)) == len(indices)
            for i, f in zip(indices, feeds):
                assert f == (prompts[i] if drawn[i] == 0 else [script[i][drawn[i] - 1]])
                drawn[i] += 1
        for i, r in enumerate(reqs):
            want, reason = [], "length"
            for tok in script[i]:
                if len(want) >= budgets[i]:
                    break
                if tok in stop:
                    reason = "stop"
                    break
                want.append(tok)
                if len(want) < budgets[i] and len(prompts[i]) + len(want) >= max_seq_len:
                    reason = "capacity"
                    break
            assert (r.output, r.finish_reason) == (want, reason), (i, prompts[i], budgets[i], script[i])
            assert drawn[i] == (0 if budgets[i] == 0 else len(want) + (reason == "stop"))
    check()
