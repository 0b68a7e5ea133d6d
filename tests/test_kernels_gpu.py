"""Each CUDA kernel alone against its plain restatement (tests/emulated_kernels.py),
at sizes other than the engine's: widths and vocabularies that are no power of
two, head sizes in steps of 16, any number of heads and groups, lengths that
cross page, tile and chunk boundaries."""

import math

import pytest
import torch

from simple_inference_autoresearch_b200.cache import SequenceCache
from simple_inference_autoresearch_b200.engine.batch import BatchMeta, StepEntry
from simple_inference_autoresearch_b200.kernels import ops
from simple_inference_autoresearch_b200.kernels.options import DEFAULT as OPTS
from simple_inference_autoresearch_b200.parts.base import KVNeed
from tests import emulated_kernels as emu
from tests import plain_llama

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rnd(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def tol(dtype):
    return dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,h,v", [(1, 64, 256), (7, 80, 331), (33, 4096, 1000), (3, 44, 50), (2, 5000, 300)])
def test_embed(dtype, n, h, v):
    table = rnd(v, h, dtype=dtype)
    tokens = torch.randint(0, v, (n,), dtype=torch.int32)
    out = ops.embed(tokens.to(DEV), table.to(DEV))
    assert out.dtype == torch.float32
    torch.testing.assert_close(out.cpu(), emu.embed(tokens, table), rtol=0, atol=0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed_flags_bad_token(dtype):
    table = rnd(16, 32, dtype=dtype).to(DEV)
    out = ops.embed(torch.tensor([3, 16, -1], dtype=torch.int32, device=DEV), table)
    with pytest.raises(RuntimeError, match="token id outside"):
        ops.check_status(DEV)
    ops.check_status(DEV)  # cleared
    assert torch.equal(out[0].cpu(), table[3].float().cpu()) and not out[1:].any()


def test_set_table_cells():
    table = torch.full((7, 40), -1, dtype=torch.int32, device=DEV)
    cells = torch.tensor([[0, 0, 5], [6, 39, 17], [3, 12, 0], [3, 13, -1]], dtype=torch.int32)
    ops.set_table_cells(table, cells.to(DEV))
    want = torch.full((7, 40), -1, dtype=torch.int32)
    for r, c, v in cells.tolist():
        want[r, c] = v
    assert torch.equal(table.cpu(), want)
    n = torch.arange(280)                        # every cell once, more than one block of threads
    big = torch.stack([n % 7, n // 7, n + 100], 1).to(torch.int32)
    ops.set_table_cells(table, big.to(DEV))
    for r, c, v in big.tolist():
        want[r, c] = v
    assert torch.equal(table.cpu(), want)


def test_gather_rows():
    src = rnd(9, 331)
    rows = torch.tensor([8, 0, 3, 3], dtype=torch.int32)
    out = ops.gather_rows(src.to(DEV), rows.to(DEV))
    torch.testing.assert_close(out.cpu(), emu.gather_rows(src, rows), rtol=0, atol=0)


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("w_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,h,eps", [(1, 64, 1e-5), (5, 80, 1e-6), (3, 331, 1e-5), (2, 4096, 1e-5), (2, 5000, 1e-3)])
@pytest.mark.parametrize("with_delta", [False, True])
def test_add_rmsnorm(out_dtype, w_dtype, n, h, eps, with_delta):
    res = rnd(n, h, seed=1)
    delta = rnd(n, h, seed=2) if with_delta else None
    w = (1 + rnd(h, seed=3, scale=0.1)).to(w_dtype)
    res_ref = res.clone()
    ref = emu.add_rmsnorm(res_ref, None if delta is None else delta.clone(), w, eps, out_dtype)
    res_d = res.to(DEV)
    out = ops.add_rmsnorm(res_d, None if delta is None else delta.to(DEV), w.to(DEV), eps, out_dtype)
    torch.testing.assert_close(res_d.cpu(), res_ref, rtol=0, atol=0)
    if out_dtype == torch.float32:
        torch.testing.assert_close(out.cpu(), ref, rtol=1e-5, atol=1e-6)
    else:
        torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=1e-2, atol=1e-3)


def test_rmsnorm_rows_do_not_depend_on_batch():
    h = 331
    res = rnd(6, h, seed=4)
    w = (1 + rnd(h, seed=5, scale=0.1))
    whole = ops.add_rmsnorm(res.to(DEV), None, w.to(DEV), 1e-5, torch.float32).cpu()
    for i in range(6):
        one = ops.add_rmsnorm(res[i:i + 1].contiguous().to(DEV), None, w.to(DEV), 1e-5, torch.float32).cpu()
        assert torch.equal(one[0], whole[i])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("m,n,k", [(1, 37, 80), (70, 331, 96), (5, 256, 64), (16, 130, 264), (3, 64, 20),
                                   (130, 65, 176), (8, 512, 1024), (17, 40, 8)])
def test_linear(dtype, m, n, k):
    x = rnd(m, k, dtype=dtype, seed=1)
    w = rnd(n, k, dtype=dtype, seed=2, scale=0.1)
    for out_dtype in {torch.float32, dtype}:
        out = ops.linear(x.to(DEV), w.to(DEV), out_dtype)
        ref = emu.linear(x, w, torch.float32)
        if dtype == torch.float32:
            torch.testing.assert_close(out.cpu(), ref, rtol=1e-5, atol=1e-5)
        elif out_dtype == torch.float32:
            torch.testing.assert_close(out.cpu(), ref, rtol=1e-4, atol=1e-4)
        else:
            torch.testing.assert_close(out.cpu().float(), ref, rtol=1e-2, atol=1e-2)


def test_linear_fp32_rows_do_not_depend_on_batch():
    x = rnd(70, 96, seed=1)
    w = rnd(331, 96, seed=2, scale=0.1).to(DEV)
    whole = ops.linear(x.to(DEV), w, torch.float32).cpu()
    for i in (0, 13, 69):
        one = ops.linear(x[i:i + 1].contiguous().to(DEV), w, torch.float32).cpu()
        assert torch.equal(one[0], whole[i])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("interleaved", [False, True])
@pytest.mark.parametrize("i", [176, 331, 14336])
def test_swiglu(dtype, interleaved, i):
    gu = rnd(5, 2 * i, dtype=dtype, scale=2.0)
    out = ops.swiglu(gu.to(DEV), interleaved)
    ref = emu.swiglu(gu, interleaved)
    torch.testing.assert_close(out.cpu().float(), ref.float(), **(dict(rtol=1e-5, atol=1e-6)
                               if dtype == torch.float32 else dict(rtol=1e-2, atol=1e-2)))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("m,i,k", [(1, 176, 64), (8, 14336, 512), (70, 136, 80), (64, 256, 96), (130, 331, 96),
                                   (300, 1024, 264), (2048, 512, 128), (5, 44, 20), (33, 331, 96), (64, 14336, 512),
                                   (20, 178, 72), (128, 130, 264)])
def test_linear_with_swiglu_epilogue(dtype, m, i, k):
    """The fused product + activation (tensor cores, both orientations) and its unfused fallback."""
    x = rnd(m, k, dtype=dtype, seed=1)
    w = rnd(2 * i, k, dtype=dtype, seed=2, scale=0.2)
    out = ops.linear_swiglu(x.to(DEV), w.to(DEV))
    ops.check_status(DEV)
    assert out.shape == (m, i) and out.dtype == dtype
    ref = emu.swiglu(emu.linear(x, w, torch.float32), interleaved=True)
    # float32: gate * up multiplies two sums of k terms, so rounding of the sums shows scaled by the other factor
    torch.testing.assert_close(out.cpu().float(), ref, **(dict(rtol=1e-4, atol=1e-4) if dtype == torch.float32
                                                          else dict(rtol=2e-2, atol=2e-2)))


# ----------------------------------------------------------------------------- attention over the cache
def make_cache(n_kv, d, dtype, device, max_tokens=8192, max_slots=12, max_seq_len=2048, window=None):
    return SequenceCache([KVNeed(n_kv, d, window)], max_tokens, max_slots, max_seq_len, dtype, device)


def run_attention_case(dtype, hq, hkv, d, lens_before, q_lens, seed=0, theta=10000.0, boost=None, qk_scale=1.0,
                       window=None, cache_size=None, options=OPTS):
    """Fills two caches (GPU kernel / CPU restatement) with the same history through
    rope_kv_write, then compares rope + attention of a last step."""
    torch.manual_seed(seed)
    caches = {dev: make_cache(hkv, d, dtype, dev, window=window, **(cache_size or {})) for dev in ("cpu", DEV)}
    kw = {"options": options} if window is None else {"window": window, "options": options}
    backends = {"cpu": emu, DEV: ops}
    inv_freq = plain_llama.rope_inv_freq(d, theta, None)
    b = len(q_lens)
    width = (hq + 2 * hkv) * d
    # Decoy sequences are opened, grown and partly closed first, so that the slots of the batch
    # are not 0..b-1 in order and their pages are neither contiguous nor ascending: a kernel that
    # took the batch index for the slot, or the page index for the page, would read the wrong keys.
    slots = {}
    for dev, c in caches.items():
        decoys = [c.alloc() for _ in range(3)]
        c.reserve(decoys, [70, 130, 5]); c.commit(decoys, [70, 130, 5])
        real = [c.alloc() for _ in range(b)]
        c.free(decoys[1])
        if b >= 2:
            real[0], real[-1] = real[-1], real[0]
        slots[dev] = real
    hist = [rnd(max(n, 1), width, dtype=dtype, seed=10 + i) for i, n in enumerate(lens_before)]
    new = [rnd(n, width, dtype=dtype, seed=50 + i) for i, n in enumerate(q_lens)]
    if qk_scale != 1.0:
        for x in hist + new:
            x[:, :(hq + hkv) * d] *= qk_scale
    if boost is not None:
        # one far key whose score stands out for the last query of `seq` (no rotation,
        # so that the key can simply be a multiple of the query of head 0)
        seq, key_pos, scale = boost
        inv_freq = None
        hist[seq][key_pos, hq * d:(hq + 1) * d] = (new[seq][-1, :d].float() * scale).to(dtype)
    outs = {}
    for dev in ("cpu", DEV):
        c, be = caches[dev], backends[dev]
        live = [(i, s) for i, s in enumerate(slots[dev]) if lens_before[i] > 0]
        if live:
            ent = [StepEntry(s, [0] * lens_before[i]) for i, s in live]
            c.reserve([s for _, s in live], [lens_before[i] for i, _ in live])
            meta = BatchMeta.build(ent, [0] * len(live), dev)
            qkv = torch.cat([hist[i] for i, _ in live]).to(dev)
            be.rope_kv_write(qkv, None if inv_freq is None else inv_freq.to(dev), c.entry(0), meta, hq, hkv, d, True)
            c.commit([s for _, s in live], [lens_before[i] for i, _ in live])
        ent = [StepEntry(s, [0] * q_lens[i]) for i, s in enumerate(slots[dev])]
        c.reserve(slots[dev], q_lens)
        meta = BatchMeta.build(ent, list(lens_before), dev)
        qkv = torch.cat(new).to(dev)
        be.rope_kv_write(qkv, None if inv_freq is None else inv_freq.to(dev), c.entry(0), meta, hq, hkv, d, True)
        out = be.attention(qkv, c.entry(0), meta, hq, hkv, d, 1.0 / math.sqrt(d), **kw)
        outs[dev] = (out.cpu().float(), qkv.cpu().float(), c.entry(0).k.cpu().float(), c.entry(0).v.cpu().float())
    t = tol(dtype)
    torch.testing.assert_close(outs[DEV][1], outs["cpu"][1], **t)   # rotated q (and untouched k, v columns)
    torch.testing.assert_close(outs[DEV][2], outs["cpu"][2], **t)   # cached k
    torch.testing.assert_close(outs[DEV][3], outs["cpu"][3], **t)   # cached v
    torch.testing.assert_close(outs[DEV][0], outs["cpu"][0], **t)
    return outs


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hq,hkv,d", [(4, 2, 16), (3, 1, 32), (6, 2, 48), (8, 8, 64), (8, 2, 128), (2, 1, 80)])
def test_attention_prefill_sizes(dtype, hq, hkv, d):
    run_attention_case(dtype, hq, hkv, d, lens_before=[0, 0, 0], q_lens=[5, 70, 33])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_prefill_continues_from_cache(dtype):
    run_attention_case(dtype, 6, 2, 48, lens_before=[63, 0, 130], q_lens=[3, 65, 1])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hq,hkv,d", [(4, 2, 16), (3, 1, 32), (6, 2, 48), (8, 8, 64), (8, 2, 128), (12, 1, 32)])
def test_attention_decode_sizes(dtype, hq, hkv, d):
    # lengths around the page (64), tile (32) and chunk (256) edges, and position 0
    run_attention_case(dtype, hq, hkv, d, lens_before=[0, 63, 255, 256, 600], q_lens=[1, 1, 1, 1, 1])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("key_pos", [0, 31, 255, 256, 511])
def test_attention_decode_finds_a_far_key(dtype, key_pos):
    hq, hkv, d = 4, 2, 32
    outs = run_attention_case(dtype, hq, hkv, d, lens_before=[700], q_lens=[1], boost=(0, key_pos, 8.0))
    # head 0's softmax is all but one-hot on that key: its output is that key's value row
    v_row = rnd(700, (hq + 2 * hkv) * d, dtype=dtype, seed=10)[key_pos, (hq + hkv) * d:(hq + hkv + 1) * d].float()
    torch.testing.assert_close(outs[DEV][0][0, :d], v_row, rtol=5e-2, atol=5e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_prefill_finds_a_far_key(dtype):
    run_attention_case(dtype, 4, 2, 32, lens_before=[300], q_lens=[40], boost=(0, 7, 8.0))


def test_decode_and_prefill_kernels_agree():
    """One new token through the prefill kernel and through the split decode
    kernel: same keys, different reduction order, so equal beyond rounding."""
    hq, hkv, d, n = 6, 2, 48, 517
    c = make_cache(hkv, d, torch.float32, DEV)
    inv_freq = plain_llama.rope_inv_freq(d, 10000.0, None).to(DEV)
    s = c.alloc()
    width = (hq + 2 * hkv) * d
    hist = rnd(n, width, seed=1).to(DEV)
    c.reserve([s], [n])
    ops.rope_kv_write(hist, inv_freq, c.entry(0), BatchMeta.build([StepEntry(s, [0] * n)], [0], DEV), hq, hkv, d)
    c.commit([s], [n])
    c.reserve([s], [1])
    new = rnd(1, width, seed=2).to(DEV)
    meta = BatchMeta.build([StepEntry(s, [0])], [n], DEV)
    ops.rope_kv_write(new, inv_freq, c.entry(0), meta, hq, hkv, d)
    dec = ops.attention(new, c.entry(0), meta, hq, hkv, d, 0.2)
    meta.is_decode = False
    pre = ops.attention(new, c.entry(0), meta, hq, hkv, d, 0.2)
    torch.testing.assert_close(dec, pre, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("hq,hkv,d", [(32, 8, 128), (6, 2, 48), (40, 8, 256), (5, 5, 80), (16, 2, 64)])
@pytest.mark.parametrize("write_kv", [True, False])
def test_rotate_and_write_of_many_bfloat16_tokens(hq, hkv, d, write_kv):
    """256 tokens and more take the 16-byte kernel: two prompts, one of them continuing a cache,
    against the restatement (rotated q in place, k rotated into the pages, v copied)."""
    lens_before, q_lens = [0, 70], [190, 130]
    width = (hq + 2 * hkv) * d
    inv_freq = plain_llama.rope_inv_freq(d, 10000.0, None)
    res = {}
    for dev, be in (("cpu", emu), (DEV, ops)):
        c = make_cache(hkv, d, torch.bfloat16, dev)
        decoy = c.alloc()
        c.reserve([decoy], [100]); c.commit([decoy], [100])
        slots = [c.alloc(), c.alloc()][::-1]
        hist = rnd(70, width, dtype=torch.bfloat16, seed=3).to(dev)
        c.reserve([slots[1]], [70])
        be.rope_kv_write(hist, inv_freq.to(dev), c.entry(0), BatchMeta.build([StepEntry(slots[1], [0] * 70)], [0], dev), hq, hkv, d)
        c.commit([slots[1]], [70])
        c.reserve(slots, q_lens)
        qkv = rnd(sum(q_lens), width, dtype=torch.bfloat16, seed=4).to(dev)
        meta = BatchMeta.build([StepEntry(s, [0] * n) for s, n in zip(slots, q_lens)], lens_before, dev)
        be.rope_kv_write(qkv, inv_freq.to(dev), c.entry(0), meta, hq, hkv, d, write_kv)
        res[dev] = (qkv.float().cpu(), c.entry(0).k.float().cpu(), c.entry(0).v.float().cpu())
    ops.check_status(DEV)
    for got, want in zip(res[DEV], res["cpu"]):
        torch.testing.assert_close(got, want, rtol=2e-2, atol=2e-2)
    if not write_kv:      # the pages hold the 70 earlier tokens only
        assert torch.equal(res[DEV][1], res["cpu"][1]) or (res[DEV][1] - res["cpu"][1]).abs().max() <= 2e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [1, 33, 100, 700])
def test_attention_over_a_window_of_keys(dtype, window):
    """Keys in front of the window are not seen, and their pages have been given back (the
    block table says -1 there): prompts that continue a cache, and single tokens."""
    hq, hkv, d = 6, 2, 48
    run_attention_case(dtype, hq, hkv, d, lens_before=[0, 300, 63], q_lens=[200, 150, 66], window=window)
    run_attention_case(dtype, hq, hkv, d, lens_before=[0, 31, 127, 128, 129, 1000], q_lens=[1] * 6, window=window)
    # a far key that would dominate is out of sight (or, with the widest window, still in)
    outs = run_attention_case(dtype, 8, 2, 128, lens_before=[700], q_lens=[1], boost=(0, 200, 8.0), window=window)
    v_row = rnd(700, 12 * 128, dtype=dtype, seed=10)[200, 10 * 128:11 * 128].float()
    if window < 500:
        assert (outs[DEV][0][0, :128] - v_row).abs().max() > 0.1
    else:                 # position 700 sees keys 1..700: the far key is in sight and wins
        torch.testing.assert_close(outs[DEV][0][0, :128], v_row, rtol=5e-2, atol=5e-2)


def test_attention_refuses_sizes_it_cannot_take():
    with pytest.raises(ValueError, match="head_dim"):
        ops.check_attention_sizes(4, 2, 24)
    with pytest.raises(ValueError, match="head_dim"):
        ops.check_attention_sizes(4, 2, 512)
    with pytest.raises(ValueError, match="multiple"):
        ops.check_attention_sizes(5, 2, 32)


def test_rope_without_rotation_only_copies():
    hq, hkv, d = 2, 1, 16
    c = make_cache(hkv, d, torch.float32, DEV)
    s = c.alloc()
    c.reserve([s], [3])
    qkv = rnd(3, (hq + 2 * hkv) * d).to(DEV)
    before = qkv.clone()
    ops.rope_kv_write(qkv, None, c.entry(0), BatchMeta.build([StepEntry(s, [0, 0, 0])], [0], DEV), hq, hkv, d)
    assert torch.equal(qkv, before)
    page = int(c.entry(0).block_table[s, 0])
    assert torch.equal(c.entry(0).k[page, 0, :3], before[:, hq * d:(hq + 1) * d])
    assert torch.equal(c.entry(0).v[page, 0, :3], before[:, (hq + 1) * d:])


# ----------------------------------------------------------------------------- sampling
def sample_case(logits, temperature, top_k, top_p, seed, index):
    r, v = logits.shape
    dev = lambda x, dt: torch.tensor(x, dtype=dt, device=DEV)  # noqa: E731
    out = ops.sample(logits.to(DEV), dev(temperature, torch.float32), dev(top_k, torch.int32),
                     dev(top_p, torch.float32), dev(seed, torch.int64), dev(index, torch.int32))
    return out.cpu().tolist()


@pytest.mark.parametrize("v", [256, 331, 5000])
def test_sample_greedy_is_argmax_with_lowest_index_on_ties(v):
    logits = rnd(4, v, seed=3)
    logits[1, 7] = logits[1, 200] = 9.0
    got = sample_case(logits, [0.0] * 4, [0] * 4, [1.0] * 4, [1, 2, 3, 4], [0] * 4)
    assert got == [int(torch.argmax(logits[i])) for i in range(4)]
    assert got[1] == 7


@pytest.mark.parametrize("v", [256, 331, 3000])
@pytest.mark.parametrize("temperature,top_k,top_p", [(0.8, 0, 1.0), (1.0, 5, 1.0), (0.7, 50, 0.9), (1.3, 0, 0.6),
                                                     (1.0, 1, 1.0), (0.5, 40, 0.0), (1.0, 100000, 0.95)])
def test_sample_matches_plain_sampler(v, temperature, top_k, top_p):
    rows = 6
    logits = rnd(rows, v, seed=11, scale=2.0)
    seeds = [1234567 + 17 * i for i in range(rows)]
    idx = [0, 1, 2, 3, 40, 41]
    got = sample_case(logits, [temperature] * rows, [top_k] * rows, [top_p] * rows, seeds, idx)
    for i in range(rows):
        u = plain_llama.counter_uniform(seeds[i], idx[i])
        want = plain_llama.sample(logits[i], temperature, top_k, top_p, u)
        if got[i] != want:
            # u may sit within rounding of a boundary of the cumulative distribution
            probs = plain_llama.kept_probabilities(logits[i], temperature, top_k, top_p)
            cdf = torch.cumsum(probs, 0)
            assert probs[got[i]] > 0, "drew a token outside the kept set"
            lo = cdf[got[i]] - probs[got[i]]
            assert lo - 1e-5 <= u <= cdf[got[i]] + 1e-5, (got[i], want, u, float(lo), float(cdf[got[i]]))


@pytest.mark.parametrize("v,scale,temperature,top_k,top_p", [
    (5000, 6.0, 1.0, 0, 0.9),       # a peaked row: the nucleus lies within the gathered candidates
    (5000, 0.1, 1.0, 0, 0.5),       # a flat row: the nucleus is far larger than the candidates (whole-row bisection)
    (3000, 2.0, 1.0, 600, 1.0),     # top-k beyond what the candidate way takes
    (3000, 2.0, 0.9, 600, 0.8),
    (5000, 3.0, 0.7, 512, 0.95),    # the largest top-k of the candidate way
    (1500, 2.0, 1.0, 1499, 1.0),
])
def test_sample_both_ways_to_the_thresholds_match_the_plain_sampler(v, scale, temperature, top_k, top_p):
    rows = 4
    logits = rnd(rows, v, seed=21, scale=scale)
    seeds = [99 + 5 * i for i in range(rows)]
    idx = [0, 7, 8, 300]
    got = sample_case(logits, [temperature] * rows, [top_k] * rows, [top_p] * rows, seeds, idx)
    for i in range(rows):
        u = plain_llama.counter_uniform(seeds[i], idx[i])
        probs = plain_llama.kept_probabilities(logits[i], temperature, top_k, top_p)
        cdf = torch.cumsum(probs, 0)
        assert probs[got[i]] > 0, "drew a token outside the kept set"
        lo = cdf[got[i]] - probs[got[i]]
        assert lo - 1e-5 <= u <= cdf[got[i]] + 1e-5, (got[i], u, float(lo), float(cdf[got[i]]))


@pytest.mark.parametrize("v", [300, 6000])
def test_sample_tokens_of_equal_logit_enter_or_leave_the_nucleus_together(v):
    logits = torch.full((1, v), -10.0)
    logits[0, 10] = 5.0
    logits[0, [20, 30, 40]] = 4.0           # weights 1 and 3 x e^-1: the group's mass before it is 1 of 2.10
    inside, outside = set(), set()
    for i in range(150):
        inside.add(sample_case(logits, [1.0], [0], [0.6], [5], [i])[0])     # limit 1.26 >= 1: the group stays
        outside.add(sample_case(logits, [1.0], [0], [0.4], [5], [i])[0])    # limit 0.84 < 1: the group leaves
    assert inside == {10, 20, 30, 40}
    assert outside == {10}


def test_sample_top_k_keeps_exactly_k_and_ties_go_to_lower_ids():
    v = 300
    logits = torch.zeros(1, v)
    logits[0, [5, 9, 100]] = 3.0
    logits[0, [50, 60, 70, 80]] = 2.0        # four tied at the 4th..7th rank, k = 5 keeps 50 and 60
    seen = set()
    for i in range(200):
        seen.add(sample_case(logits, [1.0], [5], [1.0], [99], [i])[0])
    assert seen <= {5, 9, 100, 50, 60} and {5, 9, 100} <= seen and seen & {50, 60}


def test_sample_frequencies_follow_the_distribution():
    v = 331
    logits = rnd(1, v, seed=5, scale=1.5)
    n = 4000
    big = logits.repeat(n, 1)
    got = sample_case(big, [0.9] * n, [0] * n, [1.0] * n, [7] * n, list(range(n)))
    probs = plain_llama.kept_probabilities(logits[0], 0.9, 0, 1.0)
    freq = torch.bincount(torch.tensor(got), minlength=v).double() / n
    assert (freq - probs).abs().max() < 0.02


def test_sample_same_request_same_draw_in_any_batch():
    logits = rnd(5, 500, seed=8)
    alone = sample_case(logits[2:3], [0.8], [0], [1.0], [42], [3])[0]
    batch = sample_case(logits, [0.8] * 5, [0] * 5, [1.0] * 5, [1, 2, 42, 4, 5], [0, 0, 3, 0, 0])
    assert batch[2] == alone


# ----------------------------------------------------------------------------- tensor-core products
@pytest.mark.parametrize("m,n,k", [
    (1, 128, 64), (1, 4096, 4096), (8, 6144, 4096), (8, 512, 14336), (16, 130, 264), (17, 256, 128),
    (33, 1000, 72), (64, 4096, 1024), (65, 384, 512), (128, 256, 256), (129, 256, 256), (200, 331, 96),
    (300, 520, 4096), (1024, 768, 512), (5, 40, 8), (2048, 256, 128),
    (20, 130, 264), (40, 331, 96), (64, 6144, 4096), (48, 4096, 14336), (100, 4096, 4096), (128, 1002, 520),
    (256, 6144, 4096), (192, 4096, 8192), (500, 1000, 2048), (200, 330, 2048), (130, 257, 1024),
])
def test_tensor_core_linear(m, n, k):
    from simple_inference_autoresearch_b200.kernels import gemm_tc
    x = rnd(m, k, dtype=torch.bfloat16, seed=1)
    w = rnd(n, k, dtype=torch.bfloat16, seed=2, scale=0.1)
    ref = x.double() @ w.double().T
    for out_dtype in (torch.float32, torch.bfloat16):
        out = torch.full((m, n), float("nan"), dtype=out_dtype, device=DEV)
        assert gemm_tc.try_linear(x.to(DEV), w.to(DEV), out), "shape refused"
        ops.check_status(DEV)
        got = out.cpu().double()
        assert not torch.isnan(got).any()
        bound = 1e-5 * k ** 0.5 + (0 if out_dtype == torch.float32 else 8e-3 * ref.abs().max().item())
        assert (got - ref).abs().max().item() <= bound + 1e-4, (m, n, k, out_dtype)
    # the CUDA-core kernel gives the same numbers beyond rounding
    simt = ops.linear(x.to(DEV), w.to(DEV), torch.float32, options=OPTS.but(use_tc_gemm=False)).cpu()
    tc = ops.linear(x.to(DEV), w.to(DEV), torch.float32).cpu()
    torch.testing.assert_close(tc, simt, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("m,n,k", [(2048, 4096, 4096), (256, 512, 128), (129, 256, 72), (1500, 1000, 2048), (384, 28672 // 8, 512)])
def test_two_sms_on_one_tile_give_the_one_sm_kernels_numbers(m, n, k):
    """Products of many rows with cta_group::2 (a pair of blocks per 256 x 256 tile) and with one
    block per 128 x 256 tile: the same k order, so the same numbers; plain, SwiGLU and adding epilogues,
    whole and ragged tiles, an odd number of 128-row blocks."""
    from simple_inference_autoresearch_b200.kernels import gemm_tc
    x = rnd(m, k, dtype=torch.bfloat16, seed=1).to(DEV)
    w = rnd(n, k, dtype=torch.bfloat16, seed=2, scale=0.05).to(DEV)
    outs = []
    for pairs in (2, 0):
        o = OPTS.but(pair_mode=pairs)
        a = ops.linear(x, w, torch.float32, options=o)
        b = ops.linear(x, w, torch.bfloat16, options=o)
        c = ops.linear_swiglu(x, w, options=o)
        res = torch.ones(m, n, device=DEV)
        assert isinstance(ops.linear(x, w, torch.float32, add_to=res, options=o), ops.Added)
        ops.check_status(DEV)
        outs.append((a.cpu(), b.float().cpu(), c.float().cpu(), res.cpu()))
    ref = x.cpu().double() @ w.cpu().double().T
    assert (outs[0][0].double() - ref).abs().max().item() <= 1e-5 * k ** 0.5 + 1e-4
    for u, v in zip(*outs):
        assert torch.equal(u, v)


@pytest.mark.parametrize("tile_n", [128, 160, 192, 224])
@pytest.mark.parametrize("m,n,k", [(300, 1000, 264), (2048, 6144, 512), (1024, 28672 // 4, 256), (640, 736, 1024)])
def test_every_tile_width_of_the_many_row_kernel_gives_the_same_numbers(m, n, k, tile_n):
    """The persistent kernel with narrower tiles (chosen when they make the waves of tiles come out more
    even): the same k order per output, so the same numbers as the 256-column tile; plain, SwiGLU and adding
    epilogues with the next norm's inputs, whole and ragged tiles."""
    x = rnd(m, k, dtype=torch.bfloat16, seed=1).to(DEV)
    w = rnd(n, k, dtype=torch.bfloat16, seed=2, scale=0.05).to(DEV)
    norm_w = (1.0 + rnd(n, seed=5, scale=0.1)).to(torch.bfloat16).to(DEV)
    outs = []
    for tn in (tile_n, 256):
        o = OPTS.but(tile_n=tn, pair_mode=0, max_splits=1)        # max_splits 1: no clusters for few tiles either
        a = ops.linear(x, w, torch.float32, options=o)
        b = ops.linear_swiglu(x, w, options=o)
        res = torch.ones(m, n, device=DEV)
        added = ops.linear(x, w, torch.float32, add_to=res, next_norm=ops.NormHint(norm_w, 1e-5), options=o)
        assert isinstance(added, ops.Added) and added.ss_parts.shape[1] == -(-n // tn)
        ops.check_status(DEV)
        outs.append((a.cpu(), b.float().cpu(), res.cpu(), added.scaled.float().cpu(), added.ss_parts.sum(1).cpu()))
    ref = x.cpu().double() @ w.cpu().double().T
    assert (outs[0][0].double() - ref).abs().max().item() <= 1e-5 * k ** 0.5 + 1e-4
    for u, v in list(zip(*outs))[:4]:
        assert torch.equal(u, v)
    torch.testing.assert_close(outs[0][4], outs[1][4], rtol=1e-5, atol=1e-5)      # the parts differ, their sums agree


def test_tensor_core_linear_refuses_unaligned_k():
    from simple_inference_autoresearch_b200.kernels import gemm_tc
    x, w = rnd(4, 20, dtype=torch.bfloat16).to(DEV), rnd(8, 20, dtype=torch.bfloat16).to(DEV)
    out = torch.empty(4, 8, dtype=torch.float32, device=DEV)
    assert gemm_tc.try_linear(x, w, out) is False
    torch.testing.assert_close(ops.linear(x, w, torch.float32).cpu(), emu.linear(x.cpu(), w.cpu(), torch.float32),
                               rtol=1e-4, atol=1e-4)


def test_tensor_core_rows_do_not_depend_on_batch_within_an_orientation():
    from simple_inference_autoresearch_b200.kernels import gemm_tc
    w = rnd(512, 1024, dtype=torch.bfloat16, seed=2, scale=0.1).to(DEV)
    x = rnd(64, 1024, dtype=torch.bfloat16, seed=1).to(DEV)
    whole = ops.linear(x, w, torch.float32)
    for rows in (1, 8, 17):
        part = ops.linear(x[:rows].contiguous(), w, torch.float32)
        assert torch.equal(part, whole[:rows])


# ----------------------------------------------------------------------------- products inside the residual stream
# rows x outputs x inner size: every kernel that can add (16-column tiles with and without a split along K,
# wider tiles as clusters, clusters in the plain orientation, the persistent kernel and pairs of SMs)
ADDING_SHAPES = [(1, 4096, 4096), (8, 4096, 14336), (8, 256, 128), (16, 384, 512), (5, 200, 72), (3, 128, 4096),
                 (16, 2048, 8192), (17, 4096, 4096), (24, 320, 520), (40, 256, 344), (64, 4096, 14336), (70, 256, 1024),
                 (100, 4096, 4096), (128, 2048, 8192), (129, 256, 256), (300, 520, 136), (2048, 4096, 512),
                 (1000, 331 * 4, 264), (300, 520, 4096), (256, 4096, 4096), (192, 1000, 14336), (500, 331 * 4, 1024),
                 (200, 336, 2048), (4100, 512, 256)]


@pytest.mark.parametrize("m,n,k", ADDING_SHAPES)
@pytest.mark.parametrize("w_dtype", [torch.bfloat16, torch.float32])
def test_product_adds_into_the_residual_and_leaves_the_next_norms_inputs(m, n, k, w_dtype):
    """epilogue 2 with a hint of the norm that follows: residual += x @ w^T in float32, the parts of
    every row's sum of squares add up to the row's sum of squares, and the scaled copy is
    bf16(residual * norm weight); through ``ops.linear`` the same, as an ``Added``."""
    from simple_inference_autoresearch_b200.kernels import gemm_tc
    x = rnd(m, k, dtype=torch.bfloat16, seed=1).to(DEV)
    w = rnd(n, k, dtype=torch.bfloat16, seed=2, scale=0.05).to(DEV)
    norm_w = (1.0 + rnd(n, seed=5, scale=0.1)).to(w_dtype).to(DEV)
    res0 = rnd(m, n, seed=3)
    want = res0.double() + x.cpu().double() @ w.cpu().double().T
    parts = gemm_tc.ss_parts(m, n, k, DEV)
    res = res0.to(DEV)
    out = ops.linear(x, w, torch.float32, add_to=res, next_norm=ops.NormHint(norm_w, 1e-5))
    ops.check_status(DEV)
    if parts == 0:        # a shape whose kernel cannot add: the product comes back and the caller adds
        assert isinstance(out, torch.Tensor) or out.ss_parts is None
        return
    assert isinstance(out, ops.Added) and out.ss_parts.shape == (m, parts) and out.weight is norm_w
    bound = 1e-5 * k ** 0.5 + 1e-4
    got = res.cpu().double()
    assert (got - want).abs().max().item() <= bound
    ss = out.ss_parts.cpu().double()
    assert torch.isfinite(ss).all()
    torch.testing.assert_close(ss.sum(1), got.pow(2).sum(1), rtol=1e-5, atol=1e-6)
    scaled = (res.cpu() * norm_w.cpu().float()).to(torch.bfloat16)
    assert out.scaled.dtype == torch.bfloat16 and out.scaled.shape == (m, n)
    # the kernel multiplies in float32 and rounds once, as the line above does: equal but for products on a rounding edge
    assert (out.scaled.cpu().float() - scaled.float()).abs().max().item() <= 2e-2 * scaled.float().abs().max().item() / 4
    assert (out.scaled.cpu() != scaled).float().mean().item() < 1e-3
    # the same residual as the product alone followed by the add, and as an add without a hint
    res2 = res0.to(DEV)
    plain = ops.linear(x, w, torch.float32, add_to=res2)
    assert isinstance(plain, ops.Added) and plain.ss_parts is None and plain.scaled is None
    assert torch.equal(res2, res)
    if m > 16:            # one kernel, one order of addition: the product alone gives the same numbers
        assert torch.equal(res, res0.to(DEV) + ops.linear(x, w, torch.float32))


@pytest.mark.parametrize("m,n,k,pieces", [(1, 6144, 4096, 32), (8, 28672, 4096, 32), (8, 256, 128, 1), (16, 384, 520, 5),
                                          (5, 200, 72, 1), (3, 1024, 14336, 112), (24, 640, 320, 3), (64, 28672, 4096, 32),
                                          (100, 6144, 4096, 7), (128, 500, 256, 2), (129, 512, 256, 2), (300, 1040, 320, 6),
                                          (2048, 6144, 1024, 4), (640, 28672, 512, 16), (4200, 512, 256, 1)])
@pytest.mark.parametrize("swiglu", [False, True])
def test_product_applies_the_norm_in_front_to_its_rows(m, n, k, pieces, swiglu):
    """A ``NormedResidual`` as the input: the product of bf16(residual * norm weight) with the rows
    multiplied by rsqrt(mean square + eps) on the accumulators, the sums of squares given in parts,
    against add_rmsnorm followed by the plain product, at every number of rows."""
    eps = 1e-5
    resid = rnd(m, k, seed=4, scale=2.0).to(DEV)
    norm_w = (1.0 + rnd(k, seed=5, scale=0.1)).to(torch.bfloat16).to(DEV)
    w = rnd(n, k, dtype=torch.bfloat16, seed=6, scale=0.05).to(DEV)
    # any split of the rows' sums of squares into parts will do
    cols = [resid[:, (k * i) // pieces:(k * (i + 1)) // pieces].double().pow(2).sum(1) for i in range(pieces)]
    ss = torch.stack(cols, 1).float().contiguous()
    scaled = (resid * norm_w.float()).to(torch.bfloat16)
    lazy = ops.NormedResidual(resid, ss, scaled, norm_w, eps, torch.bfloat16)
    x = ops.add_rmsnorm(resid.clone(), None, norm_w, eps, torch.bfloat16)
    if swiglu:
        got = ops.linear_swiglu(lazy, w)
        ref = ops.linear_swiglu(x, w)
    else:
        got = ops.linear(lazy, w, torch.float32)
        ref = ops.linear(x, w, torch.float32)
    ops.check_status(DEV)
    # both round the activations to bfloat16 once (before or after the row factor); against the exact product
    exact = (resid.double() * torch.rsqrt(resid.double().pow(2).mean(1, keepdim=True) + eps) * norm_w.double()) @ w.double().T
    if swiglu:
        exact = exact[:, 0::2] * torch.sigmoid(exact[:, 0::2]) * exact[:, 1::2]
    scale = exact.abs().max().item()
    err_fused = (got.double() - exact).abs().max().item()
    err_plain = (ref.double() - exact).abs().max().item()
    assert err_fused <= 2 * err_plain + 4e-3 * scale, (m, n, k, err_fused, err_plain, scale)
    assert (got.float() - ref.float()).abs().max().item() <= 1.2e-2 * scale + 1e-4, (m, n, k)
    # without the fused stream the same call computes the norm first
    off = ops.linear_swiglu(lazy, w, options=OPTS.but(fuse_residual_stream=False)) if swiglu else \
        ops.linear(lazy, w, torch.float32, options=OPTS.but(fuse_residual_stream=False))
    assert torch.equal(off, ref)


def test_fused_residual_stream_can_be_switched_off_and_wide_tiles_without_a_split_do_not_add():
    x = rnd(8, 256, dtype=torch.bfloat16, seed=1).to(DEV)
    w = rnd(128, 256, dtype=torch.bfloat16, seed=2, scale=0.05).to(DEV)
    res = rnd(8, 128, seed=3).to(DEV)
    before = res.clone()
    out8 = ops.linear(x, w, torch.float32, add_to=res, options=OPTS.but(fuse_residual_stream=False))
    assert isinstance(out8, torch.Tensor) and torch.equal(res, before)       # the caller adds later
    # 40 rows on 64-column tiles with so many outputs that nothing is split along K: that kernel does not add
    x = rnd(40, 64, dtype=torch.bfloat16, seed=1).to(DEV)
    w = rnd(148 * 128, 64, dtype=torch.bfloat16, seed=2, scale=0.05).to(DEV)
    res = rnd(40, 148 * 128, seed=3).to(DEV)
    before = res.clone()
    out = ops.linear(x, w, torch.float32, add_to=res, next_norm=ops.NormHint(torch.ones(148 * 128, device=DEV), 1e-5))
    assert isinstance(out, torch.Tensor) and torch.equal(res, before)
    torch.testing.assert_close(out.cpu(), emu.linear(x.cpu(), w.cpu(), torch.float32), rtol=1e-4, atol=1e-4)


# ----------------------------------------------------------------------------- tensor-core attention
@pytest.mark.parametrize("hq,hkv,d", [(6, 2, 128), (16, 1, 64), (4, 4, 128), (32, 8, 128), (8, 4, 64)])
def test_mma_attention_decode_groups_and_lengths(hq, hkv, d):
    assert ops.mma_attention_takes(torch.bfloat16, hq, hkv, d, 64)
    run_attention_case(torch.bfloat16, hq, hkv, d, lens_before=[0, 31, 127, 128, 129, 1000], q_lens=[1] * 6)


@pytest.mark.parametrize("hq,hkv,d", [(32, 8, 128), (6, 2, 128), (16, 4, 64)])
@pytest.mark.parametrize("lens", [[0], [0, 0, 0], [5000], [63, 64, 65, 1, 0, 2047, 2048, 300, 129, 4000],
                                  [700] * 37, [31, 2200] * 9])
def test_mma_attention_decode_over_many_sequences_of_unequal_lengths(hq, hkv, d, lens):
    """One new token for each of up to 37 sequences whose histories run from nothing to thousands of
    keys: one chunk and many chunks per (sequence, kv head), chunks past a short sequence's end, more
    blocks than the GPU holds at once, and a grid sized by the longest sequence."""
    run_attention_case(torch.bfloat16, hq, hkv, d, lens_before=lens, q_lens=[1] * len(lens),
                       cache_size={"max_tokens": sum(lens) + 128 * len(lens) + 1024, "max_slots": len(lens) + 4,
                                   "max_seq_len": max(max(lens) + 128, 256)})


@pytest.mark.parametrize("hq,hkv,d", [(6, 2, 128), (16, 1, 64), (4, 4, 128), (32, 8, 128), (8, 4, 64)])
def test_mma_attention_prefill_groups_and_lengths(hq, hkv, d):
    run_attention_case(torch.bfloat16, hq, hkv, d, lens_before=[0, 0, 300, 63], q_lens=[1, 200, 150, 66])


def test_mma_and_cuda_core_attention_agree():
    for lens_before, q_lens in (([500, 64], [1, 1]), ([100, 0], [90, 130])):
        a = run_attention_case(torch.bfloat16, 8, 2, 128, lens_before, q_lens)[DEV][0]
        b = run_attention_case(torch.bfloat16, 8, 2, 128, lens_before, q_lens,
                               options=OPTS.but(use_mma_attention=False))[DEV][0]
        torch.testing.assert_close(a, b, rtol=2e-2, atol=2e-2)


def test_mma_attention_is_refused_where_it_does_not_apply():
    assert not ops.mma_attention_takes(torch.float32, 8, 2, 128, 64)
    assert not ops.mma_attention_takes(torch.bfloat16, 8, 2, 48, 64)
    assert not ops.mma_attention_takes(torch.bfloat16, 32, 1, 128, 64)     # 32 heads on one kv head
    assert not ops.mma_attention_takes(torch.bfloat16, 8, 2, 128, 32)      # pages smaller than a key tile


def test_mma_attention_far_key_and_rows_do_not_depend_on_batch():
    hq, hkv, d = 8, 2, 128
    outs = run_attention_case(torch.bfloat16, hq, hkv, d, lens_before=[700], q_lens=[1], boost=(0, 200, 8.0))
    v_row = rnd(700, (hq + 2 * hkv) * d, dtype=torch.bfloat16, seed=10)[200, (hq + hkv) * d:(hq + hkv + 1) * d].float()
    torch.testing.assert_close(outs[DEV][0][0, :d], v_row, rtol=5e-2, atol=5e-2)
    # the same sequence alone and beside others: identical rows
    alone = run_attention_case(torch.bfloat16, hq, hkv, d, lens_before=[0], q_lens=[150])[DEV][0]
    both = run_attention_case(torch.bfloat16, hq, hkv, d, lens_before=[0, 0], q_lens=[150, 77])[DEV][0]
    assert torch.equal(alone, both[:150])


# ----------------------------------------------------------------------------- tcgen05 attention for prompts
@pytest.mark.parametrize("d", [128, 64])
@pytest.mark.parametrize("hq,hkv", [(8, 2), (4, 4), (32, 8), (16, 1), (2, 1), (64, 2), (6, 2), (24, 8), (5, 1), (7, 7)])
def test_tc_attention_prefill_groups_and_lengths(hq, hkv, d):
    """Query tiles that are full, half empty and absent; prompts that start at 0 and that continue a
    cache whose length is no multiple of the key tile; one token among prompts.  Groups of 3 and 5
    heads leave the last rows of a 128-row tile unused (42 tokens x 3, 25 x 5)."""
    assert ops.tc_attention_takes(torch.bfloat16, hq, hkv, d, 64)
    run_attention_case(torch.bfloat16, hq, hkv, d, lens_before=[0, 0, 300, 63, 64], q_lens=[1, 200, 150, 66, 129])


@pytest.mark.parametrize("hq,hkv,d", [(24, 8, 128), (32, 8, 64)])
def test_tc_attention_far_key_at_the_sizes_of_the_smaller_models(hq, hkv, d):
    outs = run_attention_case(torch.bfloat16, hq, hkv, d, lens_before=[900, 0], q_lens=[300, 1100], boost=(0, 200, 8.0))
    v_row = rnd(900, (hq + 2 * hkv) * d, dtype=torch.bfloat16, seed=10)[200, (hq + hkv) * d:(hq + hkv + 1) * d].float()
    torch.testing.assert_close(outs[DEV][0][299, :d], v_row, rtol=5e-2, atol=5e-2)


def test_tc_attention_long_prompt_and_far_key():
    hq, hkv, d = 8, 2, 128
    outs = run_attention_case(torch.bfloat16, hq, hkv, d, lens_before=[900, 0], q_lens=[300, 1100], boost=(0, 200, 8.0))
    v_row = rnd(900, (hq + 2 * hkv) * d, dtype=torch.bfloat16, seed=10)[200, (hq + hkv) * d:(hq + hkv + 1) * d].float()
    torch.testing.assert_close(outs[DEV][0][299, :d], v_row, rtol=5e-2, atol=5e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_decode_over_tens_of_thousands_of_keys(dtype):
    """Many chunks per sequence in the decode kernels (the cap on chunks, the join over dozens of
    partials), beside short sequences in the same batch; the key that matters is the fourth of 20,000."""
    hq, hkv, d = 8, 2, 128
    outs = run_attention_case(dtype, hq, hkv, d, lens_before=[20000, 9000, 70], q_lens=[1, 1, 1], boost=(0, 3, 8.0),
                              cache_size=dict(max_tokens=32768, max_seq_len=20480))
    v_row = rnd(20000, (hq + 2 * hkv) * d, dtype=dtype, seed=10)[3, (hq + hkv) * d:(hq + hkv + 1) * d].float()
    torch.testing.assert_close(outs[DEV][0][0, :d], v_row, rtol=5e-2, atol=5e-2)


def test_tc_attention_prompt_of_thousands_of_tokens():
    """Ninety-odd key tiles for the last rows (the barriers' phases turn over dozens of times)."""
    hq, hkv, d = 2, 1, 128
    outs = run_attention_case(torch.bfloat16, hq, hkv, d, lens_before=[100], q_lens=[6000], boost=(0, 10, 8.0),
                              cache_size=dict(max_tokens=8192, max_seq_len=6144))
    v_row = rnd(100, (hq + 2 * hkv) * d, dtype=torch.bfloat16, seed=10)[10, (hq + hkv) * d:(hq + hkv + 1) * d].float()
    torch.testing.assert_close(outs[DEV][0][5999, :d], v_row, rtol=5e-2, atol=5e-2)


def test_tc_attention_large_scores_rescale():
    """Scores that grow along the keys by far more than the lazy-rescale gap: every row has to
    rescale its accumulator several times."""
    hq, hkv, d = 4, 1, 128
    torch.manual_seed(3)
    outs = run_attention_case(torch.bfloat16, hq, hkv, d, lens_before=[0], q_lens=[400], qk_scale=6.0)
    assert torch.isfinite(outs[DEV][0]).all()


def test_tc_and_mma_attention_agree_and_rows_do_not_depend_on_batch():
    hq, hkv, d = 8, 2, 128
    a = run_attention_case(torch.bfloat16, hq, hkv, d, [100, 0], [90, 330])[DEV][0]
    no_tc = OPTS.but(use_tc_attention=False)
    assert ops.tc_attention_takes(torch.bfloat16, hq, hkv, d, 64) and not ops.tc_attention_takes(torch.bfloat16, hq, hkv, d, 64, no_tc)
    b = run_attention_case(torch.bfloat16, hq, hkv, d, [100, 0], [90, 330], options=no_tc)[DEV][0]
    torch.testing.assert_close(a, b, rtol=2e-2, atol=2e-2)
    alone = run_attention_case(torch.bfloat16, hq, hkv, d, lens_before=[0], q_lens=[150])[DEV][0]
    both = run_attention_case(torch.bfloat16, hq, hkv, d, lens_before=[0, 0], q_lens=[150, 77])[DEV][0]
    assert torch.equal(alone, both[:150])


def test_tc_attention_is_refused_where_it_does_not_apply():
    assert not ops.tc_attention_takes(torch.float32, 8, 2, 128, 64)
    assert not ops.tc_attention_takes(torch.bfloat16, 8, 2, 32, 64)        # head_dim other than 64 and 128
    assert not ops.tc_attention_takes(torch.bfloat16, 8, 2, 96, 64)
    assert not ops.tc_attention_takes(torch.bfloat16, 7, 2, 128, 64)       # heads that do not fall into equal groups
    assert not ops.tc_attention_takes(torch.bfloat16, 8, 2, 128, 32)       # pages smaller than a key tile


@pytest.mark.parametrize("hq,hkv,d", [(8, 2, 128), (6, 2, 128), (16, 4, 64), (4, 4, 64)])
@pytest.mark.parametrize("write_kv", [True, False])
def test_fused_rope_decode_attention_equals_the_two_kernels(hq, hkv, d, write_kv):
    """One token per sequence: rotary + cache write + attention in one kernel against the separate
    rotate-and-write kernel followed by attention (same cache contents afterwards, same output)."""
    lens = [0, 15, 16, 63, 64, 700, 1029]
    width = (hq + 2 * hkv) * d
    inv_freq = plain_llama.rope_inv_freq(d, 10000.0, None).to(DEV)
    results = []
    for fused in (True, False):
        c = make_cache(hkv, d, torch.bfloat16, DEV, max_tokens=8192, max_slots=8)
        slots = [c.alloc() for _ in lens]
        live = [(i, s) for i, s in enumerate(slots) if lens[i] > 0]
        hist = torch.cat([rnd(lens[i], width, dtype=torch.bfloat16, seed=10 + i) for i, _ in live]).to(DEV)
        c.reserve([s for _, s in live], [lens[i] for i, _ in live])
        ops.rope_kv_write(hist, inv_freq, c.entry(0), BatchMeta.build([StepEntry(s, [0] * lens[i]) for i, s in live],
                                                                      [0] * len(live), DEV), hq, hkv, d)
        c.commit([s for _, s in live], [lens[i] for i, _ in live])
        c.reserve(slots, [1] * len(lens))
        if not write_kv:      # a layer that reads a cache another layer wrote: the new token is already there
            other = rnd(len(lens), width, dtype=torch.bfloat16, seed=77).to(DEV)
            ops.rope_kv_write(other, inv_freq, c.entry(0), BatchMeta.build([StepEntry(s, [0]) for s in slots], lens, DEV),
                              hq, hkv, d)
        new = rnd(len(lens), width, dtype=torch.bfloat16, seed=50).to(DEV)
        meta = BatchMeta.build([StepEntry(s, [0]) for s in slots], lens, DEV)
        o = OPTS.but(fuse_decode_rope=fused)
        assert ops.decode_fuses_rope(meta, torch.bfloat16, hq, hkv, d, 64, o) == fused
        out = ops.rope_and_attention(new, inv_freq, c.entry(0), meta, hq, hkv, d, 1.0 / math.sqrt(d), write_kv=write_kv,
                                     options=o)
        results.append((out.float().cpu(), c.entry(0).k.float().cpu(), c.entry(0).v.float().cpu()))
    ops.check_status(DEV)
    torch.testing.assert_close(results[0][1], results[1][1], rtol=0, atol=0)     # cached keys: same rounding, same bits
    torch.testing.assert_close(results[0][2], results[1][2], rtol=0, atol=0)
    torch.testing.assert_close(results[0][0], results[1][0], rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("dtype,path", [(torch.bfloat16, "fused"), (torch.bfloat16, "mma"), (torch.bfloat16, "mma_prefill"),
                                        (torch.bfloat16, "tc_prefill"), (torch.bfloat16, "cuda_core"),
                                        (torch.bfloat16, "cuda_core_prefill"), (torch.float32, "cuda_core"),
                                        (torch.float32, "cuda_core_prefill")])
@pytest.mark.parametrize("history_only", [False, True])
def test_a_page_the_sequence_does_not_hold_is_reported_and_no_other_memory_is_touched(dtype, path, history_only):
    """A block-table cell of -1 inside the keys a step reads and writes (a replay of a captured step
    without the pages reserved first would meet one): the kernels read page 0 instead of an address
    in front of the pool, store nothing for the token without a page, and the status word says so.
    ``history_only``: only a page of earlier keys is absent, so the report has to come from the
    attention kernel itself (the rotate-and-write kernel meets no absent page)."""
    hq, hkv, d = 8, 2, 128
    width = (hq + 2 * hkv) * d
    n_before, q_len = 300, (70 if path.endswith("prefill") else 1)
    c = make_cache(hkv, d, dtype, DEV, max_tokens=4096, max_slots=4)
    decoy, slot = c.alloc(), c.alloc()
    c.reserve([decoy], [64]); c.commit([decoy], [64])           # page 0 belongs to another sequence
    hist = rnd(n_before, width, dtype=dtype, seed=3).to(DEV)
    c.reserve([slot], [n_before])
    ops.rope_kv_write(hist, None, c.entry(0), BatchMeta.build([StepEntry(slot, [0] * n_before)], [0], DEV), hq, hkv, d)
    c.commit([slot], [n_before])
    c.reserve([slot], [q_len])
    ops.check_status(DEV)
    table = c.entry(0).block_table
    table[slot, 2] = -1                                          # keys 128..191 of the history
    if not history_only:
        table[slot, (n_before + q_len - 1) // 64] = -1           # and the page of the newest token
    k_before, v_before = c.entry(0).k.clone(), c.entry(0).v.clone()
    new = rnd(q_len, width, dtype=dtype, seed=4).to(DEV)
    meta = BatchMeta.build([StepEntry(slot, [0] * q_len)], [n_before], DEV)
    o = OPTS.but(fuse_decode_rope=path == "fused", use_mma_attention=not path.startswith("cuda_core"),
                 use_tc_attention=path == "tc_prefill")
    out = ops.rope_and_attention(new, None, c.entry(0), meta, hq, hkv, d, 1.0 / math.sqrt(d), options=o)
    torch.cuda.synchronize()
    assert out.shape == (q_len, hq * d)
    with pytest.raises(RuntimeError, match="without a page"):
        ops.check_status(DEV)
    ops.check_status(DEV)                                        # the word is cleared once it has been read
    # tokens whose page exists were stored (a prompt's first tokens), the one without a page nowhere
    new_pages = {table[slot, i].item() for i in range(n_before // 64, (n_before + q_len - 1) // 64 + 1)}
    changed_k = (c.entry(0).k != k_before).flatten(1).any(1).nonzero().flatten().tolist()
    assert set(changed_k) <= new_pages - {-1}
    assert torch.equal(c.entry(0).v[0], v_before[0]) and torch.equal(c.entry(0).k[0], k_before[0])
