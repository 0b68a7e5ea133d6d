"""The three shipped presets' layer shapes (Llama-3.2-1B: head_dim 64, tied embeddings;
Llama-3.2-3B: three query heads per kv head; Llama-3.1-8B) with two layers and random weights:
the bfloat16 path (tensor-core products and attention at their real tile sizes) against the
library's own float32 path, which the other tests tie to the plain implementation.  Unequal
prompts in one step, then single tokens."""

import dataclasses

import pytest
import torch

import simple_inference_autoresearch_b200 as siar
from simple_inference_autoresearch_b200 import StepEntry
from simple_inference_autoresearch_b200.config import LlamaConfig, preset_path
from tests.test_engine_gpu import REL_TOL

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("preset", ["llama-3.2-1b", "llama-3.2-3b", "llama-3.1-8b"])
def test_bfloat16_path_at_real_layer_shapes(preset):
    cfg = dataclasses.replace(LlamaConfig.from_json(preset_path(preset)), num_hidden_layers=2)
    g = torch.Generator().manual_seed(0)
    reqs = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (300, 77, 513)]
    outs = {}
    for dtype in (torch.float32, torch.bfloat16):
        loaded = siar.init_random(siar.build_model(cfg, dtype, "cuda"), seed=1)
        eng = siar.Engine(loaded.model, max_batch=3, max_seq_len=1024, use_cuda_graph=False)
        slots = [eng.open() for _ in reqs]
        o = [eng.step([StepEntry(s, r[:-3], [0, len(r) - 4]) for s, r in zip(slots, reqs)])]
        for k in range(3):
            o.append(eng.step([StepEntry(s, [r[len(r) - 3 + k]], [0]) for s, r in zip(slots, reqs)]))
        outs[dtype] = torch.cat(o).float().cpu()
        del eng, loaded
        torch.cuda.empty_cache()
    ref, got = outs[torch.float32], outs[torch.bfloat16]
    assert torch.isfinite(got).all()
    err = (got - ref).abs().max().item()
    assert err <= REL_TOL[torch.bfloat16] * ref.abs().max().item(), err


def test_captured_decode_steps_across_a_length_bucket_equal_eager_steps():
    """Greedy decoding at the 8B layer shapes from a 2,040-token prompt: the captured step (graphs per
    512-key bucket, products inside the residual stream, attention with the rotary fused) crosses
    the 2,048-key bucket and draws the same tokens as eager steps."""
    cfg = dataclasses.replace(LlamaConfig.from_json(preset_path("llama-3.1-8b")), num_hidden_layers=2)
    loaded = siar.init_random(siar.build_model(cfg, torch.bfloat16, "cuda"), seed=3)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (2040, 1500)]
    outs = []
    for graph in (True, False):
        eng = siar.Engine(loaded.model, max_batch=2, max_seq_len=4096, use_cuda_graph=graph)
        outs.append(eng.generate(prompts, siar.SamplingParams(temperature=0.0), max_new_tokens=24, ignore_eos=True))
        if graph:
            assert len(eng._graphs) >= 2          # one per bucket crossed
        del eng
    assert outs[0] == outs[1]
    assert all(len(o) == 24 for o in outs[0])


@pytest.mark.parametrize("preset,batch,lo,hi,new,temperature", [
    ("llama-3.2-1b", 16, 64, 2048, 24, 0.0),      # head_dim 64, tied embeddings, greedy
    ("llama-3.2-3b", 32, 128, 4096, 12, 0.7),     # three query heads per kv head, seeded sampling
])
def test_unequal_batches_of_long_prompts_at_real_layer_shapes(preset, batch, lo, hi, new, temperature):
    """The two workloads the smaller presets are meant for (an unequal batch of long prompts in one
    step, then decoding; two layers here): every request gets its tokens, the same seed draws the
    same tokens again, captured and eager steps agree, and a request alone draws what it drew in
    the batch."""
    cfg = dataclasses.replace(LlamaConfig.from_json(preset_path(preset)), num_hidden_layers=2)
    loaded = siar.init_random(siar.build_model(cfg, torch.bfloat16, "cuda"), seed=5)
    g = torch.Generator().manual_seed(7)
    lens = torch.randint(lo, hi + 1, (batch,), generator=g).tolist()
    lens[0], lens[-1] = hi, lo
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]
    params = siar.SamplingParams(temperature=temperature, top_k=50 if temperature else 0, top_p=0.9 if temperature else 1.0,
                                 seed=11)
    runs = []
    for graph in (True, False, True):
        eng = siar.Engine(loaded.model, max_batch=batch, max_seq_len=hi + 64, use_cuda_graph=graph)
        runs.append(eng.generate(prompts, params, max_new_tokens=new, ignore_eos=True))
        if graph and len(runs) == 1:
            alone = eng.generate(prompts[3:4], params, max_new_tokens=new, ignore_eos=True)
        del eng
    assert all(len(o) == new for o in runs[0])
    assert runs[0] == runs[2]                       # same seed, same tokens
    if temperature == 0.0:
        assert runs[0] == runs[1]                   # captured steps == eager steps
        assert alone[0] == runs[0][3]               # a request alone == the same request in the batch


def test_float32_path_at_the_8b_layer_shapes_equals_the_plain_implementation():
    """One layer of the Llama-3.1-8B shape (all its sizes, its vocabulary, its scaled rotary) with
    random weights: the true 32-bit path, a prompt whole and its last tokens one by one, against
    the plain implementation on the CPU."""
    from simple_inference_autoresearch_b200.weights import random_tensors
    from tests import plain_llama

    cfg = dataclasses.replace(LlamaConfig.from_json(preset_path("llama-3.1-8b")), num_hidden_layers=1)
    built = siar.build_model(cfg, torch.float32, "cuda")
    w = random_tensors(built.model.tensor_specs(), 9, torch.float32)
    built.model.load({k: v.to("cuda") for k, v in w.items()})
    toks = torch.randint(0, cfg.vocab_size, (40,), generator=torch.Generator().manual_seed(3)).tolist()
    eng = siar.Engine(built.model, max_batch=1, max_seq_len=128, use_cuda_graph=False)
    s = eng.open()
    outs = [eng.step([StepEntry(s, toks[:32], range(32))])]
    outs += [eng.step([StepEntry(s, [t], [0])]) for t in toks[32:]]
    got = torch.cat(outs).cpu()
    ref = plain_llama.forward(w, cfg.to_dict(), toks)
    err = (got - ref).abs().max().item()
    assert err <= REL_TOL[torch.float32] * ref.abs().max().item(), err
