"""The engine against the plain implementation, in 32-bit and in bfloat16: each
request alone and whole; with the last 32 tokens one by one; in batches of
unequal lengths whose shorter requests end earlier, one batch after another so
that slots and pages are used again; long decoding; the first tokens of a
sequence; greedy generation through the entry point."""

import pytest
import torch

import simple_inference_autoresearch_b200 as siar
from simple_inference_autoresearch_b200 import SamplingParams, StepEntry
from tests import plain_llama, tiny_configs

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]

# Largest |logit difference| allowed against the plain float32 implementation
# (run on the same stored weights), relative to the largest |logit| of the
# request.  float32: reduction order only.  bfloat16: activations are rounded to
# bfloat16 between kernels (8 bits of mantissa) through 2-3 layers.
REL_TOL = {torch.float32: 2e-5, torch.bfloat16: 3e-2}


def close(out, ref, dtype, what=""):
    scale = ref.abs().max().item()
    err = (out.float().cpu() - ref).abs().max().item()
    assert err <= REL_TOL[dtype] * scale, f"{what}: max |diff| {err:.3e} vs scale {scale:.3e}"


def prompts(vocab, lengths, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lengths]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("models")
    return {n: tiny_configs.make_folder(tmp, n, seed=11 + i) for i, n in enumerate("ABC")}


@pytest.fixture(scope="module")
def oracle(folders):
    cache = {}

    def get(name, tokens):
        key = (name, tuple(tokens))
        if key not in cache:
            raw, w = tiny_configs.read_folder(folders[name])
            cache[key] = plain_llama.forward(w, raw, tokens)
        return cache[key]
    return get


def engine_for(folders, name, dtype, **kw):
    loaded = siar.load_model(folders[name], device="cuda", dtype=dtype)
    kw.setdefault("max_batch", 4)
    kw.setdefault("max_seq_len", tiny_configs.CONFIGS[name]["max_position_embeddings"])
    return siar.Engine(loaded.model, **kw)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", "ABC")
def test_whole_requests(folders, oracle, name, dtype):
    eng = engine_for(folders, name, dtype)
    vocab = tiny_configs.CONFIGS[name]["vocab_size"]
    for toks in prompts(vocab, [1, 5, 40, 97]):
        s = eng.open()
        out = eng.step([StepEntry(s, toks, range(len(toks)))])
        close(out, oracle(name, toks), dtype, f"whole {len(toks)}")
        eng.close(s)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", "ABC")
def test_last_32_tokens_one_by_one(folders, oracle, name, dtype):
    eng = engine_for(folders, name, dtype)
    vocab = tiny_configs.CONFIGS[name]["vocab_size"]
    for toks in prompts(vocab, [33, 70, 100], seed=1):
        s = eng.open()
        head = len(toks) - 32
        outs = [eng.step([StepEntry(s, toks[:head], range(head))])]
        for t in toks[head:]:
            outs.append(eng.step([StepEntry(s, [t], [0])]))
        close(torch.cat(outs), oracle(name, toks), dtype, f"cut {len(toks)}")
        eng.close(s)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", "ABC")
def test_unequal_batches_one_after_another(folders, oracle, name, dtype):
    """Three batches on a cache that only holds one of them at a time: prompts of
    unequal lengths start together, then one token each; shorter requests end
    earlier and free their slot, which the next batch takes."""
    vocab = tiny_configs.CONFIGS[name]["vocab_size"]
    eng = engine_for(folders, name, dtype, max_batch=4, max_tokens=4 * 128)
    seen_slots = []
    for bi, lens in enumerate([[5, 11, 17, 60], [1, 7, 23, 40], [90, 2, 64]]):
        reqs = prompts(vocab, lens, seed=20 + bi)
        tails = [min(len(r) - 1, 3 + 2 * i) for i, r in enumerate(reqs)]   # tokens fed one by one
        slots = [eng.open() for _ in reqs]
        seen_slots.append(tuple(slots))
        got = [[] for _ in reqs]
        heads = [len(r) - t for r, t in zip(reqs, tails)]
        out = eng.step([StepEntry(s, r[:h], range(h)) for s, r, h in zip(slots, reqs, heads)])
        o = 0
        for i, h in enumerate(heads):
            got[i].append(out[o:o + h]); o += h
        live = list(range(len(reqs)))
        k = 0
        while live:
            live = [i for i in live if k < tails[i]]
            for i in range(len(reqs)):
                if i not in live and slots[i] is not None and k >= tails[i]:
                    eng.close(slots[i]); slots[i] = None
            if not live:
                break
            out = eng.step([StepEntry(slots[i], [reqs[i][heads[i] + k]], [0]) for i in live])
            for j, i in enumerate(live):
                got[i].append(out[j:j + 1])
            k += 1
        for i, r in enumerate(reqs):
            close(torch.cat(got[i]), oracle(name, r), dtype, f"batch {bi} request {i}")
        assert eng.cache.slots.held == 0 and all(g.pages.held == 0 for g in eng.cache.groups)
    assert set(seen_slots[1]) == set(seen_slots[0]) and set(seen_slots[2]) <= set(seen_slots[0]), \
        "slots were not used again"


@pytest.mark.parametrize("dtype", DTYPES)
def test_padding_changes_nothing(folders, oracle, dtype):
    """The same request alone and beside longer and shorter neighbours: identical logits."""
    name = "B"
    vocab = tiny_configs.CONFIGS[name]["vocab_size"]
    reqs = prompts(vocab, [9, 50, 3], seed=5)
    eng = engine_for(folders, name, dtype)
    s = eng.open()
    alone = eng.step([StepEntry(s, reqs[0], range(9))])
    eng.close(s)
    slots = [eng.open() for _ in reqs]
    both = eng.step([StepEntry(s, r, range(len(r)) if i == 0 else []) for i, (s, r) in enumerate(zip(slots, reqs))])
    if dtype == torch.float32:
        assert torch.equal(alone, both)
    else:
        close(both, alone.float().cpu(), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(folders, oracle, dtype):
    """300 single-token steps after a short prompt: crosses pages (64), attention
    tiles (32) and the decode chunk (256)."""
    name = "C"
    vocab = tiny_configs.CONFIGS[name]["vocab_size"]
    toks = prompts(vocab, [310], seed=9)[0]
    eng = engine_for(folders, name, dtype, max_batch=2)
    s = eng.open()
    outs = [eng.step([StepEntry(s, toks[:10], range(10))])]
    for t in toks[10:]:
        outs.append(eng.step([StepEntry(s, [t], [0])]))
    close(torch.cat(outs), oracle(name, toks), dtype, "long decode")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", "AB")
def test_first_tokens_of_a_sequence(folders, oracle, name, dtype):
    vocab = tiny_configs.CONFIGS[name]["vocab_size"]
    toks = prompts(vocab, [4], seed=3)[0]
    eng = engine_for(folders, name, dtype)
    s = eng.open()
    outs = [eng.step([StepEntry(s, [t], [0])]) for t in toks]
    close(torch.cat(outs), oracle(name, toks), dtype, "first tokens")


def plain_greedy(folder, prompt, n, stop=()):
    raw, w = tiny_configs.read_folder(folder)
    toks, out = list(prompt), []
    for _ in range(n):
        t = int(torch.argmax(plain_llama.forward(w, raw, toks)[-1]))
        if t in stop:
            break
        out.append(t)
        toks.append(t)
    return out


@pytest.mark.parametrize("graph", [False, True])
@pytest.mark.parametrize("name", "AB")
def test_greedy_generation_through_the_entry_point(folders, name, graph):
    vocab = tiny_configs.CONFIGS[name]["vocab_size"]
    reqs = prompts(vocab, [5, 11, 17, 3, 30], seed=4)
    loaded = siar.load_model(folders[name], device="cuda", dtype=torch.float32)
    eng = siar.build_engine(loaded, max_batch=3, max_seq_len=128, use_cuda_graph=graph)
    outs, stats = eng.generate(reqs, SamplingParams(temperature=0.0), max_new_tokens=8, ignore_eos=True,
                               return_stats=True)
    for r, o in zip(reqs, outs):
        assert o == plain_greedy(folders[name], r, 8), "greedy tokens differ from the plain implementation"
    assert stats["new_tokens"] == 8 * len(reqs) and stats["finish_reasons"] == ["length"] * len(reqs)
    one, st = siar.generate_with_stats(reqs[0], eng, max_new_tokens=8, temperature=0.0, ignore_eos=True)
    assert one == outs[0] and st["prompt_tokens"] == len(reqs[0])
    # the streaming forms: one prompt's tokens one by one, and (prompt index, token) pairs of a batch
    assert list(siar.generate(reqs[0], eng, max_new_tokens=8, temperature=0.0, ignore_eos=True)) == outs[0]
    streamed = [[] for _ in reqs]
    for index, tok in eng.stream(reqs, SamplingParams(temperature=0.0), max_new_tokens=8, ignore_eos=True):
        streamed[index].append(tok)
    assert streamed == outs


def test_captured_steps_share_one_pool_and_the_oldest_are_dropped(folders, monkeypatch):
    """Requests that end at different times give a captured step per batch size; with room for two
    of them the engine drops the one used longest ago and captures it again when it is needed, all
    in one memory pool.  The tokens are those of the engine without graphs."""
    from simple_inference_autoresearch_b200.engine import engine as engine_module
    monkeypatch.setattr(engine_module, "MAX_CAPTURED_STEPS", 2)
    name = "A"
    vocab = tiny_configs.CONFIGS[name]["vocab_size"]
    reqs = prompts(vocab, [9, 4, 21, 2], seed=12)
    new = [3, 14, 7, 10]                                 # batch sizes 4, 3, 2, 1 in turn
    loaded = siar.load_model(folders[name], device="cuda", dtype=torch.bfloat16)
    outs = {}
    for graph in (True, False):
        eng = siar.build_engine(loaded, max_batch=4, max_seq_len=128, use_cuda_graph=graph)
        for _ in range(2):                               # the second round captures the dropped steps again
            outs.setdefault(graph, []).append(eng.generate(reqs, SamplingParams(temperature=0.0),
                                                           max_new_tokens=new, ignore_eos=True))
        if graph:
            assert len(eng._graphs) == 2 and eng._graph_pool is not None
    assert outs[True] == outs[False]
    assert [len(o) for o in outs[True][0]] == new


def test_generation_stops_at_stop_tokens_and_samples_reproducibly(folders):
    name = "B"
    vocab = tiny_configs.CONFIGS[name]["vocab_size"]
    reqs = prompts(vocab, [1, 7, 23, 40], seed=6)
    loaded = siar.load_model(folders[name], device="cuda", dtype=torch.float32)
    eng = siar.build_engine(loaded, max_batch=4, max_seq_len=128)
    greedy = eng.generate(reqs, SamplingParams(temperature=0.0), max_new_tokens=12, ignore_eos=True)
    stop = greedy[1][4]
    cut = eng.generate(reqs, SamplingParams(temperature=0.0), max_new_tokens=12, ignore_eos=True,
                       stop_token_ids=[stop])
    for g, c in zip(greedy, cut):
        want = g[:g.index(stop)] if stop in g else g
        assert c == want
    p = SamplingParams(temperature=0.8, seed=123)
    a = eng.generate(reqs, p, max_new_tokens=12, ignore_eos=True)
    b = eng.generate(reqs, p, max_new_tokens=12, ignore_eos=True)
    assert a == b
    # a request draws the same tokens alone as in the batch (per-request counter RNG);
    # request index 2 alone is index 0, so give it the seed stream of index 2 explicitly
    eng1 = siar.build_engine(loaded, max_batch=1, max_seq_len=128, use_cuda_graph=False)
    alone = eng1.generate([reqs[0]], p, max_new_tokens=12, ignore_eos=True)
    assert alone[0] == a[0]


def test_programmatic_launch_on_and_off_give_the_same_tokens_and_logits(folders):
    """Kernels launched with and without programmatic dependent launch: identical results
    (a kernel that read its input before its predecessor had finished would show here)."""
    from simple_inference_autoresearch_b200.kernels import ops
    name = "C"
    vocab = tiny_configs.CONFIGS[name]["vocab_size"]
    reqs = prompts(vocab, [40, 9, 77], seed=8)
    results = []
    for on in (True, False, True):
        ops.set_programmatic_launch(on)
        try:
            eng = engine_for(folders, name, torch.bfloat16, max_batch=3)
            toks = eng.generate(reqs, SamplingParams(temperature=0.0), max_new_tokens=20, ignore_eos=True)
            s = eng.open()
            logits = eng.step([StepEntry(s, reqs[2], range(len(reqs[2])))]).cpu()
            results.append((toks, logits))
        finally:
            ops.set_programmatic_launch(True)
    assert results[0][0] == results[1][0] == results[2][0]
    assert torch.equal(results[0][1], results[1][1]) and torch.equal(results[0][1], results[2][1])


@pytest.mark.parametrize("name", "ABC")
def test_products_inside_the_residual_stream_change_rounding_only(folders, oracle, name):
    """Decode steps with the residual add and the norm inside the products, and with the separate
    norm kernel: both within the bfloat16 tolerance of the plain implementation, and close to each
    other (same arithmetic, another order of the sums of squares)."""
    from simple_inference_autoresearch_b200.kernels import ops
    vocab = tiny_configs.CONFIGS[name]["vocab_size"]
    req = prompts(vocab, [50], seed=11)[0]
    ref = oracle(name, req)
    outs = []
    for fuse in (True, False):
        ops.fuse_residual_stream = fuse
        try:
            eng = engine_for(folders, name, torch.bfloat16, max_batch=1)
            s = eng.open()
            o = [eng.step([StepEntry(s, req[:10], range(10))])]
            o += [eng.step([StepEntry(s, [t], [0])]) for t in req[10:]]
            outs.append(torch.cat(o).float().cpu())
        finally:
            ops.fuse_residual_stream = True
    scale = ref.abs().max().item()
    for o in outs:
        assert (o - ref).abs().max().item() <= REL_TOL[torch.bfloat16] * scale
    assert (outs[0] - outs[1]).abs().max().item() <= REL_TOL[torch.bfloat16] * scale


def test_command_line(folders, capsys):
    from simple_inference_autoresearch_b200 import inference
    rc = inference.main(["--model", str(folders["A"]), "--prompt-ids", "5,17,3", "--max-new-tokens", "6",
                         "--temperature", "0", "--dtype", "float32", "--ignore-eos"])
    out = capsys.readouterr().out
    assert rc == 0
    first = [int(t) for t in out.splitlines()[0].split()]
    assert first == plain_greedy(folders["A"], [5, 17, 3], 6)
    assert "decode_tok_s" in out and "ttft_ms" in out and "prompt_tokens" in out


def test_command_line_with_random_weights_a_batch_and_stop_ids(capsys):
    """A shipped configuration with seeded random weights, several random prompts of unequal lengths
    at once, and a further stop token: the same seed gives the same lines, and no line holds the stop token."""
    from simple_inference_autoresearch_b200 import inference
    base = ["--model", "tiny-b", "--random-weights", "--seed", "3", "--prompt-len", "12", "--batch", "3",
            "--max-new-tokens", "10", "--temperature", "0", "--dtype", "float32", "--ignore-eos"]
    assert inference.main(base) == 0
    first = capsys.readouterr().out
    lines = [ln for ln in first.splitlines() if ln.startswith("[")]
    assert [ln.split()[1] for ln in lines] == ["12", "9", "6"]                 # prompt lengths from N down to N/2
    tokens = [[int(t) for t in ln.split("->")[1].split()] for ln in lines]
    assert all(len(t) == 10 for t in tokens)
    assert inference.main(base) == 0
    assert [ln for ln in capsys.readouterr().out.splitlines() if ln.startswith("[")] == lines
    stop = tokens[1][4]
    assert inference.main(base + ["--stop-id", str(stop)]) == 0
    cut = [[int(t) for t in ln.split("->")[1].split()] for ln in capsys.readouterr().out.splitlines() if ln.startswith("[")]
    for full, c in zip(tokens, cut):
        assert c == (full[:full.index(stop)] if stop in full else full)
    assert inference.main(["--model", "tiny-a", "--random-weights", "--prompt-len", "5", "--max-new-tokens", "4",
                           "--temperature", "0.8", "--top-k", "0", "--top-p", "1.0"]) == 0
    assert "decode_tok_s" in capsys.readouterr().out
