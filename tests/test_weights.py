"""Weights by name: what is held in which dtype, and ONE error that lists all
missing and unexpected tensors and wrong shapes (no GPU)."""

import json

import pytest
import torch
from safetensors.torch import load_file, save_file

import simple_inference_autoresearch_b200 as siar
from simple_inference_autoresearch_b200.weights import WeightError, write_model_folder
from simple_inference_autoresearch_b200.weights.loader import INDEX_FILE, SINGLE_FILE
from tests import tiny_configs


def test_random_folder_has_the_checkpoint_names_and_is_reproducible(tmp_path):
    a = tiny_configs.make_folder(tmp_path / "1", "A", seed=7)
    b = tiny_configs.make_folder(tmp_path / "2", "A", seed=7)
    c = tiny_configs.make_folder(tmp_path / "3", "A", seed=8)
    wa, wb, wc = (load_file(str(f / SINGLE_FILE)) for f in (a, b, c))
    names = set(wa)
    assert "model.embed_tokens.weight" in names and "model.norm.weight" in names
    assert "model.layers.1.self_attn.k_proj.weight" in names and "model.layers.0.mlp.down_proj.weight" in names
    assert "lm_head.weight" not in names          # tied
    assert len(names) == 1 + 2 * 9 + 1
    assert all(torch.equal(wa[n], wb[n]) for n in names)
    assert not torch.equal(wa["model.embed_tokens.weight"], wc["model.embed_tokens.weight"])
    assert wa["model.layers.0.self_attn.q_proj.weight"].dtype == torch.bfloat16
    assert abs(wa["model.embed_tokens.weight"].float().std().item() - 0.02) < 0.002
    assert torch.all(wa["model.norm.weight"] == 1)
    wB = load_file(str(tiny_configs.make_folder(tmp_path, "B") / SINGLE_FILE))
    assert "lm_head.weight" in wB and not torch.all(wB["model.norm.weight"] == 1)
    assert wB["model.layers.2.self_attn.k_proj.weight"].shape == (32, 96)
    raw = json.loads((a / "config.json").read_text())
    assert raw["architectures"] == ["LlamaForCausalLM"] and raw["num_hidden_layers"] == 2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_held_dtypes(tmp_path, dtype):
    # norm weights stored in float32 stay float32; matrices take the compute dtype
    folder = tiny_configs.make_folder(tmp_path, "B", vector_dtype=torch.float32)
    m = siar.load_model(folder, device="cpu", dtype=dtype).model
    assert m.embedding.dtype == dtype and m.head.dtype == dtype
    assert m.layers[0].mixer.w_qkv.dtype == dtype and m.layers[0].mixer.w_qkv.shape == (5 * 32, 96)
    assert m.layers[0].ffn.w_gate_up.shape == (512, 96)
    assert m.layers[0].mixer_norm.weight.dtype == torch.float32
    assert m.final_norm.weight.dtype == torch.float32
    folder = tiny_configs.make_folder(tmp_path / "x", "B")
    m = siar.load_model(folder, device="cpu", dtype=dtype).model
    assert m.final_norm.weight.dtype == dtype
    # merged weights are the checkpoint's rows in q, k, v / gate, up order
    w = load_file(str(folder / SINGLE_FILE))
    p = "model.layers.1.self_attn."
    want = torch.cat([w[p + "q_proj.weight"], w[p + "k_proj.weight"], w[p + "v_proj.weight"]]).to(dtype)
    assert torch.equal(m.layers[1].mixer.w_qkv, want)
    # gate and up rows alternate in the merged feed-forward weight
    q = "model.layers.1.mlp."
    gu = m.layers[1].ffn.w_gate_up
    assert torch.equal(gu[0::2], w[q + "gate_proj.weight"].to(dtype)) and torch.equal(gu[1::2], w[q + "up_proj.weight"].to(dtype))


def test_tied_head_is_the_embedding(tmp_path):
    m = siar.load_model(tiny_configs.make_folder(tmp_path, "A"), device="cpu", dtype=torch.float32).model
    assert m.head.data_ptr() == m.embedding.data_ptr()
    m = siar.load_model(tiny_configs.make_folder(tmp_path, "B"), device="cpu", dtype=torch.float32).model
    assert m.head.data_ptr() != m.embedding.data_ptr()


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = tiny_configs.make_folder(tmp_path, "B")
    w = load_file(str(folder / SINGLE_FILE))
    del w["model.layers.1.mlp.up_proj.weight"]
    del w["lm_head.weight"]
    w["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)
    w["model.layers.2.self_attn.q_proj.weight"] = torch.zeros(96, 95, dtype=torch.bfloat16)
    w["model.norm.weight"] = torch.zeros(97, dtype=torch.bfloat16)
    save_file(w, str(folder / SINGLE_FILE))
    with pytest.raises(WeightError) as e:
        siar.load_model(folder, device="cpu", dtype=torch.float32)
    err = e.value
    assert err.missing == ["lm_head.weight", "model.layers.1.mlp.up_proj.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert sorted(n for n, _, _ in err.wrong_shape) == ["model.layers.2.self_attn.q_proj.weight", "model.norm.weight"]
    text = str(err)
    for piece in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (2)", "expected (96, 96)",
                  "file has (96, 95)"):
        assert piece in text


def test_tied_model_may_carry_a_stored_head(tmp_path):
    folder = tiny_configs.make_folder(tmp_path, "A")
    w = load_file(str(folder / SINGLE_FILE))
    w["lm_head.weight"] = w["model.embed_tokens.weight"].clone()
    save_file(w, str(folder / SINGLE_FILE))
    siar.load_model(folder, device="cpu", dtype=torch.float32)


def test_what_a_checkpoint_may_hold_beside_the_models_tensors_is_the_architectures_to_say(tmp_path):
    """The model's spec names the tensors a checkpoint may hold beside the ones the model reads, by
    name or by ``*suffix``; the loader takes the list as it is."""
    from simple_inference_autoresearch_b200.weights.loader import load_checkpoint
    folder = tiny_configs.make_folder(tmp_path, "B")
    model = siar.load_model(folder, device="cpu", dtype=torch.float32).model
    assert model.spec.ignorable_tensors == ()          # untied: nothing may be left over
    w = load_file(str(folder / SINGLE_FILE))
    for i in range(3):
        w[f"model.layers.{i}.self_attn.rotary_emb.inv_freq"] = torch.ones(16)
    w["extra.table"] = torch.ones(4)
    save_file(w, str(folder / SINGLE_FILE))
    with pytest.raises(WeightError) as e:
        load_checkpoint(folder, model.tensor_specs(), torch.float32, "cpu", ("extra.table",))
    assert e.value.unexpected == [f"model.layers.{i}.self_attn.rotary_emb.inv_freq" for i in range(3)]
    got = load_checkpoint(folder, model.tensor_specs(), torch.float32, "cpu", ("extra.table", "*.rotary_emb.inv_freq"))
    assert set(got) == {s.name for s in model.tensor_specs()}


def test_sharded_checkpoint_with_index(tmp_path):
    folder = tiny_configs.make_folder(tmp_path, "A")
    w = load_file(str(folder / SINGLE_FILE))
    names = sorted(w)
    half = len(names) // 2
    shards = {"model-00001-of-00002.safetensors": names[:half], "model-00002-of-00002.safetensors": names[half:]}
    for fname, ns in shards.items():
        save_file({n: w[n] for n in ns}, str(folder / fname))
    (folder / INDEX_FILE).write_text(json.dumps({"weight_map": {n: f for f, ns in shards.items() for n in ns}}))
    (folder / SINGLE_FILE).unlink()
    m = siar.load_model(folder, device="cpu", dtype=torch.float32).model
    assert torch.equal(m.embedding, w["model.embed_tokens.weight"].float())
    (folder / "model-00002-of-00002.safetensors").unlink()
    with pytest.raises(FileNotFoundError, match="shard"):
        siar.load_model(folder, device="cpu", dtype=torch.float32)


def test_folder_without_weights(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(tiny_configs.TINY_A))
    with pytest.raises(FileNotFoundError, match="neither"):
        siar.load_model(tmp_path, device="cpu", dtype=torch.float32)


# ----------------------------------------------------------------------------- the seeded generator
def test_random_values_are_normal_and_do_not_depend_on_how_they_are_drawn(monkeypatch):
    from simple_inference_autoresearch_b200.parts.base import TensorSpec
    from simple_inference_autoresearch_b200.weights import random_init

    z = random_init.standard_normal(400_000, key=random_init._tensor_seed(3, "some.tensor"))
    assert abs(z.mean().item()) < 0.01 and abs(z.std().item() - 1) < 0.01
    assert abs((z ** 3).mean().item()) < 0.03 and abs((z ** 4).mean().item() - 3) < 0.06
    assert 4.0 < z.abs().max().item() < 6.0 and torch.isfinite(z).all()
    # a tensor drawn whole and in pieces (the writer draws 2^24 elements at a time): the same bits
    spec = TensorSpec("model.layers.0.mlp.up_proj.weight", (37, 53), std=0.02)
    whole = random_init.random_tensor(spec, 5, torch.float32)
    monkeypatch.setattr(random_init, "_CHUNK", 100)
    assert torch.equal(random_init.random_tensor(spec, 5, torch.float32), whole)
    # another name or another seed: another stream
    other = random_init.random_tensor(TensorSpec("model.layers.1.mlp.up_proj.weight", (37, 53)), 5, torch.float32)
    assert not torch.equal(other, whole) and not torch.equal(random_init.random_tensor(spec, 6, torch.float32), whole)


def test_the_shipped_tiny_b_configuration_carries_its_rule_for_norm_weights(tmp_path):
    """``--model tiny-b --random-weights`` is the second tiny configuration as specified: norm
    weights 1 + N(0, 0.02), everything else N(0, 0.02); the rule travels in the configuration
    (``norm_weight_init``) and survives a round trip through config.json."""
    from simple_inference_autoresearch_b200 import registry
    from simple_inference_autoresearch_b200.config import preset_path

    _arch, cfg = registry.resolve_path(preset_path("tiny-b"))
    assert cfg.norm_weight_init == "ones_plus_normal" and cfg.initializer_range == 0.02
    folder = write_model_folder(tmp_path / "b", cfg, seed=1)
    w = load_file(str(folder / SINGLE_FILE))
    norm = w["model.layers.1.post_attention_layernorm.weight"].float()
    assert not torch.all(norm == 1) and abs(norm.mean().item() - 1) < 0.02 and 0.005 < norm.std().item() < 0.04
    _arch, again = registry.resolve_path(folder)
    assert again.norm_weight_init == "ones_plus_normal"
    _arch, a = registry.resolve_path(preset_path("tiny-a"))
    assert a.norm_weight_init == "ones" and "norm_weight_init" not in a.to_dict()


@pytest.mark.gpu
def test_random_weights_hold_the_same_bits_on_the_cpu_and_on_the_gpu(tmp_path):
    """``init_random`` (drawn on the GPU) and ``write_model_folder`` (drawn on the CPU) give identical
    tensors for one seed: every tensor of the second tiny configuration, and a tensor longer than
    one piece of the generator."""
    from simple_inference_autoresearch_b200 import registry
    from simple_inference_autoresearch_b200.config import preset_path
    from simple_inference_autoresearch_b200.parts.base import TensorSpec
    from simple_inference_autoresearch_b200.weights import random_init, random_tensors

    _arch, cfg = registry.resolve_path(preset_path("tiny-b"))
    loaded = siar.build_model(cfg, torch.bfloat16, "cuda")
    specs = loaded.model.tensor_specs()
    on_gpu = random_tensors(specs, 21, torch.bfloat16, "cuda")
    on_cpu = random_tensors(specs, 21, torch.bfloat16, "cpu")
    assert all(torch.equal(on_gpu[s.name].cpu(), on_cpu[s.name]) for s in specs)
    folder = write_model_folder(tmp_path / "b", cfg, seed=21)
    stored = load_file(str(folder / SINGLE_FILE))
    assert all(torch.equal(on_gpu[s.name].cpu(), stored[s.name]) for s in specs)
    big = TensorSpec("big", (random_init._CHUNK + 4097,), std=1.0)
    a = random_init.random_tensor(big, 2, torch.float32, "cuda").cpu()
    b = random_init.random_tensor(big, 2, torch.float32, "cpu")
    assert torch.equal(a, b)
