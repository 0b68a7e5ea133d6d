"""The step function's Python side without a GPU: the CUDA kernels are swapped
for their plain restatements (tests/emulated_kernels.py), so what is checked is
batching, positions, cache pages and slots, and the wanted rows, against the plain
implementation.  The kernels themselves are checked in the ``-m gpu`` tests."""

import pytest
import torch

import simple_inference_autoresearch_b200 as siar
from simple_inference_autoresearch_b200 import SamplingParams, StepEntry
from tests import emulated_kernels, plain_llama, tiny_configs


@pytest.fixture(autouse=True)
def emulated(monkeypatch):
    emulated_kernels.install(monkeypatch)


def build(tmp_path, name, **kw):
    folder = tiny_configs.make_folder(tmp_path, name, seed=3)
    raw, w = tiny_configs.read_folder(folder)
    loaded = siar.load_model(folder, device="cpu", dtype=torch.float32)
    kw.setdefault("max_batch", 4)
    kw.setdefault("max_seq_len", 128)
    return siar.Engine(loaded.model, use_cuda_graph=False, **kw), raw, w


def toks(vocab, n, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


@pytest.mark.parametrize("name", "ABC")
def test_whole_cut_and_batched_agree_with_plain(tmp_path, name):
    eng, raw, w = build(tmp_path, name, max_tokens=5 * 64)
    reqs = [toks(raw["vocab_size"], n, i) for i, n in enumerate((70, 9, 33))]
    refs = [plain_llama.forward(w, raw, r) for r in reqs]
    # whole
    s = eng.open()
    torch.testing.assert_close(eng.step([StepEntry(s, reqs[0], range(70))]), refs[0], rtol=1e-5, atol=2e-6)
    eng.close(s)
    # unequal batch, then one token each; only some rows wanted; the shortest ends first
    slots = [eng.open() for _ in reqs]
    heads = [len(r) - 3 for r in reqs]
    out = eng.step([StepEntry(s, r[:h], [0, h - 1]) for s, r, h in zip(slots, reqs, heads)])
    for i, h in enumerate(heads):
        torch.testing.assert_close(out[2 * i], refs[i][0], rtol=1e-5, atol=2e-6)
        torch.testing.assert_close(out[2 * i + 1], refs[i][h - 1], rtol=1e-5, atol=2e-6)
    for k in range(3):
        live = [i for i in range(3) if not (i == 1 and k == 2)]
        if k == 2:
            eng.close(slots[1])
        out = eng.step([StepEntry(slots[i], [reqs[i][heads[i] + k]], [0]) for i in live])
        for j, i in enumerate(live):
            torch.testing.assert_close(out[j], refs[i][heads[i] + k], rtol=1e-5, atol=2e-6)
    assert eng.cache.held_tokens() == 128 + 64


def test_generate_greedy_and_sampled(tmp_path):
    eng, raw, w = build(tmp_path, "A", max_batch=2)
    reqs = [toks(raw["vocab_size"], n, 10 + i) for i, n in enumerate((5, 11, 17))]
    outs = eng.generate(reqs, SamplingParams(temperature=0.0), max_new_tokens=4, ignore_eos=True)
    for r, o in zip(reqs, outs):
        cur, want = list(r), []
        for _ in range(4):
            want.append(int(torch.argmax(plain_llama.forward(w, raw, cur)[-1])))
            cur.append(want[-1])
        assert o == want
    p = SamplingParams(temperature=0.8, top_k=20, top_p=0.9, seed=5)
    a = eng.generate(reqs, p, max_new_tokens=4, ignore_eos=True)
    assert a == eng.generate(reqs, p, max_new_tokens=4, ignore_eos=True)
    assert a != eng.generate(reqs, SamplingParams(temperature=0.8, top_k=20, top_p=0.9, seed=6), 4, ignore_eos=True)
    assert eng.cache.slots.held == 0


def test_stream_and_the_one_prompt_generator_give_generates_tokens(tmp_path):
    eng, raw, _ = build(tmp_path, "B", max_batch=2)
    reqs = [toks(raw["vocab_size"], n, 20 + i) for i, n in enumerate((4, 13, 7))]
    p = SamplingParams(temperature=0.8, top_k=0, top_p=1.0, seed=9)
    new = [5, 2, 6]
    outs = eng.generate(reqs, p, max_new_tokens=new, ignore_eos=True)
    assert [len(o) for o in outs] == new
    got = [[] for _ in reqs]
    for index, tok in eng.stream(reqs, p, max_new_tokens=new, ignore_eos=True):
        got[index].append(tok)
    assert got == outs
    # the first request alone draws the same tokens (request index 0, the same seed stream)
    assert list(siar.generate(reqs[0], eng, max_new_tokens=5, temperature=0.8, top_k=0, top_p=1.0, seed=9,
                              ignore_eos=True)) == outs[0]
    it = eng.stream(reqs, p, max_new_tokens=new, ignore_eos=True)
    next(it)
    assert eng.cache.slots.held == 2
    it.close()                                   # an abandoned stream gives its slots and pages back
    assert eng.cache.slots.held == 0 and eng.cache.held_tokens() == 0


def test_step_errors_come_before_any_launch(tmp_path):
    eng, raw, _ = build(tmp_path, "A", max_batch=2, max_tokens=128)
    s = eng.open()
    with pytest.raises(ValueError, match="want index"):
        eng.step([StepEntry(s, [1, 2], [2])])
    with pytest.raises(siar.cache.CacheError):
        eng.step([StepEntry(s, [1] * 129, [])])
    assert eng.cache.length(s) == 0
    with pytest.raises(RuntimeError, match="token id outside"):
        eng.step([StepEntry(s, [raw["vocab_size"]], [0])])


def test_kernels_refuse_cpu_tensors(monkeypatch):
    monkeypatch.undo()
    from simple_inference_autoresearch_b200.kernels import ops
    with pytest.raises(RuntimeError, match="CUDA device only"):
        ops.swiglu(torch.zeros(2, 4))
