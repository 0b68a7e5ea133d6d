"""Seeded random tiny configurations (widths and vocabularies that are no multiple of anything useful,
head sizes in steps of 16 up to 128, one to seven query heads per kv head, one to three layers, rotary
scaling on and off, tied and untied heads) through the engine against the plain implementation, in
32-bit and in bfloat16, eager and with captured decode steps: requests whole, an unequal batch whose
last tokens go one by one, and generation through the entry point."""

import random

import pytest
import torch

import simple_inference_autoresearch_b200 as siar
from simple_inference_autoresearch_b200 import StepEntry
from simple_inference_autoresearch_b200.config import LlamaConfig
from simple_inference_autoresearch_b200.weights import write_model_folder
from tests import plain_llama, tiny_configs

pytestmark = pytest.mark.gpu

REL_TOL = {torch.float32: 2e-5, torch.bfloat16: 4e-2}     # of the request's largest |logit|


def random_config(case: int) -> dict:
    rng = random.Random(1000 + case)
    d = rng.choice([16, 32, 48, 64, 80, 96, 112, 128])
    hkv = rng.choice([1, 2, 3, 5])
    hq = hkv * rng.choice([1, 2, 3, 4, 7])
    scaling = rng.choice([None, {"rope_type": "llama3", "factor": rng.choice([2.0, 8.0]), "low_freq_factor": 1.0,
                                 "high_freq_factor": 4.0, "original_max_position_embeddings": rng.choice([32, 64])}])
    return {"architectures": ["LlamaForCausalLM"], "model_type": "llama",
            "hidden_size": rng.choice([36, 50, 72, 100, 132, 200, 264]),
            "intermediate_size": rng.choice([70, 99, 136, 250, 344, 513]),
            "num_hidden_layers": rng.choice([1, 2, 3]), "vocab_size": rng.choice([101, 257, 331, 500, 1003]),
            "num_attention_heads": hq, "num_key_value_heads": hkv, "head_dim": d,
            "rms_norm_eps": rng.choice([1e-5, 1e-6, 3e-4]), "rope_theta": rng.choice([10000.0, 500000.0]),
            "max_position_embeddings": 512, "rope_scaling": scaling,
            "tie_word_embeddings": rng.choice([True, False]), "bos_token_id": 0, "eos_token_id": 1,
            "torch_dtype": "bfloat16"}


@pytest.mark.parametrize("case", range(10))
def test_random_configuration_against_the_plain_implementation(case, tmp_path):
    raw = random_config(case)
    folder = write_model_folder(tmp_path / "m", LlamaConfig.from_dict(raw), seed=case, norm_weight_init="ones_plus_normal")
    raw, w = tiny_configs.read_folder(folder)
    gen = torch.Generator().manual_seed(case)
    toks = [torch.randint(0, raw["vocab_size"], (n,), generator=gen).tolist() for n in (150, 9, 41, 70)]
    refs = [plain_llama.forward(w, raw, t) for t in toks]

    def close(out, ref, what):
        err = (out.float().cpu() - ref).abs().max().item()
        assert err <= REL_TOL[dtype] * ref.abs().max().item(), f"{what}: {err:.3e} of {ref.abs().max().item():.3e}; {raw}"

    for dtype in (torch.float32, torch.bfloat16):
        loaded = siar.load_model(folder, device="cuda", dtype=dtype)
        for graph in (False, True):
            eng = siar.Engine(loaded.model, max_batch=4, max_seq_len=512, use_cuda_graph=graph)
            for t, r in zip(toks[:2], refs[:2]):
                s = eng.open()
                close(eng.step([StepEntry(s, t, range(len(t)))]), r, f"whole {len(t)}")
                eng.close(s)
            slots = [eng.open() for _ in toks]
            heads = [len(t) - 6 for t in toks]
            got = [[] for _ in toks]
            out = eng.step([StepEntry(s, t[:h], range(h)) for s, t, h in zip(slots, toks, heads)])
            o = 0
            for i, h in enumerate(heads):
                got[i].append(out[o:o + h])
                o += h
            for k in range(6):
                out = eng.step([StepEntry(s, [t[h + k]], [0]) for s, t, h in zip(slots, toks, heads)])
                for i in range(len(toks)):
                    got[i].append(out[i:i + 1])
            for i, r in enumerate(refs):
                close(torch.cat(got[i]), r, f"batch, sequence {i}")
            for s in slots:
                eng.close(s)
            # greedy generation (captured decode steps when graph is on): the first new token of every
            # prompt is the plain implementation's, unless its two best logits are within the tolerance
            prompts = [t[:20] for t in toks]
            outs = eng.generate(prompts, siar.SamplingParams(temperature=0.0), max_new_tokens=5, ignore_eos=True)
            assert all(len(o) == 5 for o in outs)
            for p, o in zip(prompts, outs):
                last = plain_llama.forward(w, raw, p)[-1]
                top2 = last.topk(2).values
                if (top2[0] - top2[1]).item() > 2 * REL_TOL[dtype] * last.abs().max().item():
                    assert o[0] == int(last.argmax()), raw


@pytest.mark.parametrize("case", range(4))
def test_random_batch_schedule_against_the_plain_implementation(case, tmp_path):
    """17 to 70 requests of unequal lengths start together, go on by one token and end at different
    times (some with their prompt); a second batch takes their slots and pages.  Eight requests of
    each batch are compared with the plain implementation, in both dtypes."""
    rng = random.Random(2000 + case)
    d = rng.choice([32, 64, 128])
    hkv = rng.choice([1, 2, 4])
    raw = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": rng.choice([64, 100, 256]),
           "intermediate_size": rng.choice([136, 250]), "num_hidden_layers": rng.choice([1, 2]),
           "vocab_size": rng.choice([257, 500]), "num_attention_heads": hkv * rng.choice([1, 2, 3, 4]),
           "num_key_value_heads": hkv, "head_dim": d, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
           "max_position_embeddings": 2048, "rope_scaling": None, "tie_word_embeddings": rng.choice([True, False]),
           "bos_token_id": 0, "eos_token_id": 1, "torch_dtype": "bfloat16"}
    folder = write_model_folder(tmp_path / "m", LlamaConfig.from_dict(raw), seed=case)
    raw, w = tiny_configs.read_folder(folder)
    gen = torch.Generator().manual_seed(case)
    for dtype in (torch.float32, torch.bfloat16):
        loaded = siar.load_model(folder, device="cuda", dtype=dtype)
        nb = rng.choice([17, 40, 70])
        eng = siar.Engine(loaded.model, max_batch=nb, max_seq_len=1024, max_tokens=nb * 320, use_cuda_graph=False)
        for batch in range(2):
            lens = [rng.choice([1, 2, 5, 33, 64, 65, 130, 200]) for _ in range(nb)]
            tails = [rng.randint(0, min(n - 1, 12)) for n in lens]           # tokens fed one by one
            toks = [torch.randint(0, raw["vocab_size"], (n,), generator=gen).tolist() for n in lens]
            slots = [eng.open() for _ in toks]
            heads = [n - t for n, t in zip(lens, tails)]
            got = [[] for _ in toks]
            out = eng.step([StepEntry(s, t[:h], range(h)) for s, t, h in zip(slots, toks, heads)])
            o = 0
            for i, h in enumerate(heads):
                got[i].append(out[o:o + h])
                o += h
            for i in range(nb):
                if tails[i] == 0:
                    eng.close(slots[i])
            live = [i for i in range(nb) if tails[i] > 0]
            k = 0
            while live:
                out = eng.step([StepEntry(slots[i], [toks[i][heads[i] + k]], [0]) for i in live])
                for j, i in enumerate(live):
                    got[i].append(out[j:j + 1])
                k += 1
                for i in live:
                    if tails[i] == k:
                        eng.close(slots[i])
                live = [i for i in live if tails[i] > k]
            for i in rng.sample(range(nb), 8):
                ref = plain_llama.forward(w, raw, toks[i])
                err = (torch.cat(got[i]).float().cpu() - ref).abs().max().item()
                assert err <= REL_TOL[dtype] * ref.abs().max().item(), (dtype, batch, i, lens[i], tails[i], err, raw)
