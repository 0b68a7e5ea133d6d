"""The engine against the plain implementation, in 32-bit and in bfloat16: each
request alone and whole; with the last 32 tokens one by one; in batches of
unequal lengths whose shorter requests end earlier, one batch after another so
that slots and pages are used again; long decoding; the first tokens of a
sequence; greedy generation through the entry point."""

import pytest
import torch

import simple_inference_autoresearch_b200 as siar
from simple_inference_autoresearch_b200 import SamplingParams, StepEntry
from simple_inference_autoresearch_b200.engine import generation
from simple_inference_autoresearch_b200.sampling.params import GREEDY, request_seed
from tests import plain_llama, tiny_configs

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
NAMES = "ABCDE"
#: the configurations whose heads have real sizes (64 and 128): in bfloat16 their attention runs on
#: the tensor-core kernels and their products on the tcgen05 kernel, as the 8B shape's do
WIDE = "DE"

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
    return {n: tiny_configs.make_folder(tmp, n, seed=11 + i) for i, n in enumerate(NAMES)}


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
@pytest.mark.parametrize("name", NAMES)
def test_whole_requests(folders, oracle, name, dtype):
    eng = engine_for(folders, name, dtype)
    vocab = tiny_configs.CONFIGS[name]["vocab_size"]
    # the longer prompts span several query tiles of the tensor-core prompt attention
    for toks in prompts(vocab, [1, 5, 40, 97] + ([129, 300] if name in WIDE else [])):
        s = eng.open()
        out = eng.step([StepEntry(s, toks, range(len(toks)))])
        close(out, oracle(name, toks), dtype, f"whole {len(toks)}")
        eng.close(s)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_last_32_tokens_one_by_one(folders, oracle, name, dtype):
    eng = engine_for(folders, name, dtype)
    vocab = tiny_configs.CONFIGS[name]["vocab_size"]
    # 600 tokens: the single tokens read more than one chunk of keys
    for toks in prompts(vocab, [33, 70, 100] + ([200, 600] if name in WIDE else []), seed=1):
        s = eng.open()
        head = len(toks) - 32
        outs = [eng.step([StepEntry(s, toks[:head], range(head))])]
        for t in toks[head:]:
            outs.append(eng.step([StepEntry(s, [t], [0])]))
        close(torch.cat(outs), oracle(name, toks), dtype, f"cut {len(toks)}")
        eng.close(s)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_one_after_another(folders, oracle, name, dtype):
    """Three batches (five with the longer prompts of the wide configurations) on a cache that
    only holds one of them at a time: prompts of unequal lengths start together, then one token
    each; shorter requests end earlier and free their slot, which the next batch takes."""
    vocab = tiny_configs.CONFIGS[name]["vocab_size"]
    batches = [[5, 11, 17, 60], [1, 7, 23, 40], [90, 2, 64]]
    max_tokens = 4 * 128
    if name in WIDE:
        batches += [[300, 129, 64, 513], [100, 700, 33]]
        max_tokens = 18 * 64                # the pages of the largest batch, no more
    eng = engine_for(folders, name, dtype, max_batch=4, max_tokens=max_tokens)
    seen_slots = []
    for bi, lens in enumerate(batches):
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
@pytest.mark.parametrize("name", "CDE")
def test_long_decoding(folders, oracle, name, dtype):
    """300 single-token steps after a short prompt (690 for the wide configurations): crosses pages
    (64), attention tiles (32, 16), decode chunks (128, 256) and 512 keys."""
    vocab = tiny_configs.CONFIGS[name]["vocab_size"]
    toks = prompts(vocab, [700 if name in WIDE else 310], seed=9)[0]
    eng = engine_for(folders, name, dtype, max_batch=2)
    s = eng.open()
    outs = [eng.step([StepEntry(s, toks[:10], range(10))])]
    for t in toks[10:]:
        outs.append(eng.step([StepEntry(s, [t], [0])]))
    close(torch.cat(outs), oracle(name, toks), dtype, "long decode")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", "ABDE")
def test_first_tokens_of_a_sequence(folders, oracle, name, dtype):
    vocab = tiny_configs.CONFIGS[name]["vocab_size"]
    toks = prompts(vocab, [4], seed=3)[0]
    eng = engine_for(folders, name, dtype)
    s = eng.open()
    outs = [eng.step([StepEntry(s, [t], [0])]) for t in toks]
    close(torch.cat(outs), oracle(name, toks), dtype, "first tokens")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,n_seqs", [("B", 5), ("D", 24), ("E", 40), ("D", 70), ("E", 9)])
def test_captured_decode_steps_give_the_plain_logits(folders, oracle, name, n_seqs, dtype):
    """Decode steps through ``Engine.run`` with CUDA graphs on, fed the requests' own tokens: the
    logits of every captured step (its static output buffer) against the plain implementation.
    Prompts of unequal lengths start together; the sequences end at different times, so the batch
    shrinks through many sizes (9 .. 70 live sequences: every tile width of the few-rows products);
    the longest sequence crosses 512 keys while it decodes (a second length bucket); a second batch
    then takes the slots and pages of the first."""
    vocab = tiny_configs.CONFIGS[name]["vocab_size"]
    wide = name in WIDE
    g = torch.Generator().manual_seed(100 + n_seqs)
    lens = torch.randint(2, 150 if wide else 60, (n_seqs,), generator=g).tolist()
    tails = [min(n - 1, 1 + (5 * i) % 11) for i, n in enumerate(lens)]
    if wide:
        lens[0], tails[0] = 517, 12                      # 505 keys after the prompt step, 517 at the end
    pages = sum(-(-n // 64) for n in lens)
    eng = engine_for(folders, name, dtype, max_batch=n_seqs, max_tokens=64 * pages, use_cuda_graph=True)
    for rnd_i in range(2):
        toks = prompts(vocab, lens, seed=40 + rnd_i)
        reqs = [generation.Request(t, 0, GREEDY, index=i) for i, t in enumerate(toks)]
        for r in reqs:
            r.slot = eng.open()
        heads = [len(t) - tl for t, tl in zip(toks, tails)]
        got = [[] for _ in reqs]
        out = eng.step([StepEntry(r.slot, t[:h], range(h)) for r, t, h in zip(reqs, toks, heads)])
        o = 0
        for i, h in enumerate(heads):
            got[i].append(out[o:o + h].cpu()); o += h
        sizes = set()
        for k in range(max(tails)):
            for r, tl in zip(reqs, tails):
                if r.slot is not None and k >= tl:
                    eng.close(r.slot); r.slot = None
            live = [i for i, tl in enumerate(tails) if k < tl]
            eng.run([reqs[i] for i in live], [[toks[i][heads[i] + k]] for i in live])
            step_logits = eng.last_logits()
            assert step_logits.shape == (len(live), vocab)
            step_logits = step_logits.cpu()
            for j, i in enumerate(live):
                got[i].append(step_logits[j:j + 1])
            sizes.add(len(live))
        for r in reqs:
            if r.slot is not None:
                eng.close(r.slot); r.slot = None
        assert len(eng._graphs) >= 2                         # captured steps did run
        for i, t in enumerate(toks):
            close(torch.cat(got[i]), oracle(name, t), dtype, f"round {rnd_i} request {i} of {n_seqs}")
        assert eng.cache.slots.held == 0 and all(gr.pages.held == 0 for gr in eng.cache.groups)
    if wide:
        assert len({b for (_, b) in eng._graphs}) == 2, "the 512-key bucket edge was not crossed"


def test_more_sequences_than_the_captured_buffers_hold(folders):
    """``run`` with more sequences than ``max_batch``: the buffers of the captured steps are made
    again, and the steps captured against the old ones go with them (a later step with an earlier
    batch size would otherwise replay a graph that reads the old buffers)."""
    name = "A"
    vocab = tiny_configs.CONFIGS[name]["vocab_size"]
    toks = prompts(vocab, [6, 9, 4, 12, 7], seed=31)
    loaded = siar.load_model(folders[name], device="cuda", dtype=torch.float32)
    drawn = {}
    for graph in (True, False):
        eng = siar.Engine(loaded.model, max_batch=2, max_slots=8, max_tokens=8 * 64, max_seq_len=64, use_cuda_graph=graph)
        reqs = [generation.Request(t, 0, GREEDY, index=i) for i, t in enumerate(toks)]
        for r in reqs:
            r.slot = eng.open()
        eng.step([StepEntry(r.slot, t[:-1]) for r, t in zip(reqs, toks)])
        feed = {i: t[-1] for i, t in enumerate(toks)}
        out = []
        for group in ([0], [1, 2, 3, 4], [0], [1, 2], [0, 3, 4, 1]):     # 1, then 4 (> max_batch), then 1 again
            res = eng.run([reqs[i] for i in group], [[feed[i]] for i in group])
            for i, t in zip(group, res):
                feed[i] = t
            out.append(res)
        drawn[graph] = out
    assert drawn[True] == drawn[False]


@pytest.mark.parametrize("name,dtype", [("B", torch.float32), ("D", torch.bfloat16)])
def test_argument_checks_pass_what_the_engine_launches_and_stop_a_spoilt_block_table(folders, name, dtype):
    """``KernelOptions(check_arguments=True)``: the host redoes the kernels' index arithmetic before
    every launch that follows the block table.  What the engine itself launches passes (prompts of
    unequal lengths, single tokens, slots used again) and draws the same tokens; a block-table cell
    that points outside the pool, or a slot whose page is missing, raises before anything runs."""
    vocab = tiny_configs.CONFIGS[name]["vocab_size"]
    toks = prompts(vocab, [70, 9, 33], seed=12)
    loaded = siar.load_model(folders[name], device="cuda", dtype=dtype)
    checked = siar.Engine(loaded.model, max_batch=3, max_seq_len=256, use_cuda_graph=False,
                          options=siar.KernelOptions(check_arguments=True))
    plain = siar.Engine(loaded.model, max_batch=3, max_seq_len=256, use_cuda_graph=False)
    for _ in range(2):
        assert checked.generate(toks, GREEDY, max_new_tokens=6, ignore_eos=True) == \
            plain.generate(toks, GREEDY, max_new_tokens=6, ignore_eos=True)
    s = checked.open()
    checked.step([StepEntry(s, toks[0])])
    table = checked.cache.groups[0].block_table
    keep = table[s, 0].item()
    table[s, 0] = 10 ** 6
    with pytest.raises(ValueError, match="is no page of the pool"):
        checked.step([StepEntry(s, [1], [0])])
    table[s, 0] = -1
    with pytest.raises(ValueError, match="holds no page for keys 0..63"):
        checked.step([StepEntry(s, [1], [0])])
    table[s, 0] = keep


def plain_check_draw(logits_row, params, u, tok, what=""):
    """The token the engine drew from ``logits_row`` must be the plain sampler's choice for the
    same uniform, or (the uniform within rounding of an edge of the cumulative distribution)
    a kept token whose interval reaches ``u`` within 1e-5."""
    x = logits_row.double().cpu()
    if params.temperature > 0 and 0 < params.top_k < x.numel():
        # tokens outside the k largest have probability zero: the plain sampler on the candidates
        # alone (kept in token order; ten more than k, so that tokens tied with the k-th are all
        # there) is the plain sampler on the whole row
        cand = sorted(torch.topk(x, min(x.numel(), params.top_k + 10)).indices.tolist())
    else:
        cand = list(range(x.numel()))
    sub = x[cand]
    want = cand[plain_llama.sample(sub, params.temperature, params.top_k, params.top_p, u)]
    if tok == want:
        return
    assert tok in cand, f"{what}: drew token {tok}, outside the candidates"
    probs = plain_llama.kept_probabilities(sub, params.temperature, params.top_k, params.top_p)
    cdf = torch.cumsum(probs, 0)
    j = cand.index(tok)
    assert probs[j] > 0, f"{what}: drew token {tok}, which the plain sampler does not keep"
    lo = cdf[j] - probs[j]
    assert lo - 1e-5 <= u <= cdf[j] + 1e-5, (what, tok, want, u, float(lo), float(cdf[j]))


@pytest.mark.parametrize("graph", [False, True])
def test_sampled_generation_draws_what_the_plain_sampler_draws(folders, graph):
    """Configuration B, float32, 4 prompts of 1, 7, 23 and 40 tokens, 12 tokens each at
    temperature 0.8 (and once with top-k and top-p): every drawn token against the plain
    implementation's logits for the tokens so far and the plain sampler fed the same counter
    uniform; and a request repeated alone under its request id draws the same tokens."""
    name = "B"
    raw, w = tiny_configs.read_folder(folders[name])
    reqs = prompts(raw["vocab_size"], [1, 7, 23, 40], seed=6)
    loaded = siar.load_model(folders[name], device="cuda", dtype=torch.float32)
    eng = siar.build_engine(loaded, max_batch=4, max_seq_len=128, use_cuda_graph=graph)
    for params in (SamplingParams(temperature=0.8, seed=123), SamplingParams(0.8, 20, 0.9, seed=7)):
        ids = [11, 3, 8, 5]
        outs = eng.generate(reqs, params, max_new_tokens=12, ignore_eos=True, request_ids=ids)
        for r, o, rid in zip(reqs, outs, ids):
            assert len(o) == 12
            seed64 = request_seed(params.seed, rid)
            for n, tok in enumerate(o):
                logits = plain_llama.forward(w, raw, list(r) + o[:n])[-1]
                plain_check_draw(logits, params, plain_llama.counter_uniform(seed64, n), tok, f"request {rid} token {n}")
        # the third request alone, at index 0 of its own call, under its id
        eng1 = siar.build_engine(loaded, max_batch=1, max_seq_len=128, use_cuda_graph=graph)
        assert eng1.generate([reqs[2]], params, max_new_tokens=12, ignore_eos=True, request_ids=[ids[2]])[0] == outs[2]
        assert eng.generate(reqs, params, max_new_tokens=12, ignore_eos=True, request_ids=ids) == outs


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
    # a request draws the same tokens alone as in the batch (per-request counter RNG): the request
    # at index 2, alone at index 0 of another call, under request id 2
    eng1 = siar.build_engine(loaded, max_batch=1, max_seq_len=128, use_cuda_graph=False)
    alone = eng1.generate([reqs[2]], p, max_new_tokens=12, ignore_eos=True, request_ids=[2])
    assert alone[0] == a[2]


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


@pytest.mark.parametrize("name", NAMES)
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
        eng = engine_for(folders, name, torch.bfloat16, max_batch=1,
                         options=siar.KernelOptions(fuse_residual_stream=fuse))
        s = eng.open()
        o = [eng.step([StepEntry(s, req[:10], range(10))])]
        o += [eng.step([StepEntry(s, [t], [0])]) for t in req[10:]]
        outs.append(torch.cat(o).float().cpu())
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
