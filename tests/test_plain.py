"""The plain implementation itself: against outputs of the reference's own model
code (stored under tests/golden/, made by tests/golden/make_golden.py), and each
of its parts against an independent restatement (no GPU)."""

import json
import math
from pathlib import Path

import pytest
import torch
from safetensors import safe_open

from tests import plain_llama

GOLDEN = Path(__file__).resolve().parent / "golden"


def load_golden(name):
    with safe_open(str(GOLDEN / f"{name}.safetensors"), framework="pt") as f:
        raw = json.loads(f.metadata()["config"])
        t = {k: f.get_tensor(k) for k in f.keys()}
    weights = {k[2:]: v for k, v in t.items() if k.startswith("w:")}
    return raw, weights, t["ids"].long(), t["whole_last"], t["stepwise"]


@pytest.mark.parametrize("name", ["g1", "g2"])
def test_plain_matches_the_reference_model_code(name):
    raw, weights, ids, whole_last, stepwise = load_golden(name)
    for b in range(ids.shape[0]):
        logits = plain_llama.forward(weights, raw, ids[b].tolist())
        # the reference's whole-prompt forward returns the last position only
        torch.testing.assert_close(logits[-1], whole_last[b], rtol=1e-5, atol=2e-6)
        # token by token through its cache: every position
        torch.testing.assert_close(logits, stepwise[b], rtol=1e-5, atol=2e-6)


def test_rope_frequencies_cover_all_three_llama3_branches():
    scaling = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
               "original_max_position_embeddings": 32}
    base = plain_llama.rope_inv_freq(32, 500000.0, None)
    scaled = plain_llama.rope_inv_freq(32, 500000.0, scaling)
    ratio = (scaled / base).tolist()
    kept = [r for r in ratio if abs(r - 1) < 1e-6]
    full = [r for r in ratio if abs(r - 1 / 8) < 1e-6]
    assert kept and full and len(kept) + len(full) < len(ratio)      # some interpolated ones in between
    assert base[0] == 1.0 and abs(base[1].item() - 500000.0 ** (-2 / 32)) < 1e-7


def test_rope_apply_is_a_rotation_of_split_half_pairs():
    d = 8
    x = torch.arange(1.0, d + 1).view(1, 1, d)
    inv = torch.tensor([0.5, 0.25, 0.125, 1.0])
    cos, sin = plain_llama.rope_tables(torch.tensor([3]), inv)
    y = plain_llama.rope_apply(x, cos, sin)[0, 0]
    for i in range(d // 2):
        a, b, ang = x[0, 0, i].item(), x[0, 0, i + d // 2].item(), 3 * inv[i].item()
        assert abs(y[i].item() - (a * math.cos(ang) - b * math.sin(ang))) < 1e-5
        assert abs(y[i + d // 2].item() - (b * math.cos(ang) + a * math.sin(ang))) < 1e-5


def test_rmsnorm_formula():
    x = torch.tensor([[3.0, 4.0]])
    w = torch.tensor([2.0, 0.5])
    y = plain_llama.rmsnorm(x, w, 1e-5)
    r = 1 / math.sqrt((9 + 16) / 2 + 1e-5)
    torch.testing.assert_close(y, torch.tensor([[3 * r * 2, 4 * r * 0.5]]))


def test_attention_is_causal_and_groups_heads():
    t, hq, hkv, d = 5, 4, 2, 8
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(t, h, d, generator=g) for h in (hq, hkv, hkv))
    out = plain_llama.attention_causal(q, k, v).view(t, hq, d)
    # position 0 sees only key 0: its output is v[0] of its kv head
    for h in range(hq):
        torch.testing.assert_close(out[0, h], v[0, h // 2])
    # changing a later key leaves earlier rows alone
    k2 = k.clone(); k2[4] += 1.0
    out2 = plain_llama.attention_causal(q, k2, v).view(t, hq, d)
    assert torch.equal(out[:4], out2[:4]) and not torch.equal(out[4], out2[4])


def test_swiglu_formula():
    w = {"gate_proj.weight": torch.tensor([[1.0], [0.0]]), "up_proj.weight": torch.tensor([[2.0], [1.0]]),
         "down_proj.weight": torch.tensor([[1.0, 1.0]])}
    y = plain_llama.swiglu_mlp(torch.tensor([[1.5]]), w, "")
    g = 1.5
    assert abs(y.item() - (g / (1 + math.exp(-g)) * 3.0)) < 1e-6


def test_plain_sampler_options():
    logits = torch.tensor([1.0, 3.0, 2.0, 3.0, -1.0])
    assert plain_llama.sample(logits, 0.0, 0, 1.0, 0.5) == 1              # greedy: lowest id among ties
    p = plain_llama.kept_probabilities(logits, 1.0, 2, 1.0)
    assert (p > 0).tolist() == [False, True, False, True, False]           # exactly k
    p = plain_llama.kept_probabilities(logits, 1.0, 0, 0.0)
    assert (p > 0).tolist() == [False, True, False, True, False]           # top_p <= 0: top token(s) only
    p = plain_llama.kept_probabilities(logits, 1.0, 0, 1.0)
    torch.testing.assert_close(p, torch.softmax(logits.double(), 0))       # both off: plain softmax
    p = plain_llama.kept_probabilities(logits, 0.5, 0, 1.0)
    torch.testing.assert_close(p, torch.softmax(logits.double() / 0.5, 0))
    # nucleus: mass before token 2 (0.7869..) exceeds 0.75 -> dropped; before the 3.0s it is 0
    p = plain_llama.kept_probabilities(logits, 1.0, 0, 0.75)
    assert (p > 0).tolist() == [False, True, False, True, False]
    assert plain_llama.sample(logits, 1.0, 0, 1.0, 0.0) == 0
    assert 0 <= plain_llama.counter_uniform(123, 0) < 1
    assert plain_llama.counter_uniform(123, 0) != plain_llama.counter_uniform(123, 1)


def test_plain_sampler_keeps_what_the_reference_sampler_keeps():
    """The probabilities the reference's own ``sample`` draws from (recorded on the CPU by
    tests/golden/make_sampler_golden.py: temperature, top-k taken before the temperature, nucleus
    with the crossing token kept, every combination) against ``kept_probabilities``, on rows without
    equal logits (where logits tie the plain sampler keeps the tied tokens together; the reference
    leaves it to its sort)."""
    with safe_open(str(GOLDEN / "sampler.safetensors"), framework="pt") as f:
        cases = json.loads(f.metadata()["cases"])
        t = {k: f.get_tensor(k) for k in f.keys()}
    for ci, (temperature, top_k, top_p) in enumerate(cases):
        for ri in range(t["logits"].shape[0]):
            mine = plain_llama.kept_probabilities(t["logits"][ri], temperature, top_k, top_p).float()
            ref = t[f"probs{ci}"][ri]
            assert torch.equal(mine > 0, ref > 0), (temperature, top_k, top_p, ri)
            torch.testing.assert_close(mine, ref, rtol=1e-5, atol=1e-7)
