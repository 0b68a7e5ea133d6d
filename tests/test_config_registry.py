"""Typed configuration and the architecture registry (no GPU)."""

import json

import pytest

from simple_inference_autoresearch_b200 import registry
from simple_inference_autoresearch_b200.config import ConfigError, LlamaConfig, RopeScaling, preset_path
from tests import tiny_configs


def test_reads_every_key_of_both_tiny_configs():
    a = LlamaConfig.from_dict(tiny_configs.TINY_A)
    assert (a.hidden_size, a.intermediate_size, a.num_hidden_layers, a.vocab_size) == (64, 176, 2, 256)
    assert (a.num_attention_heads, a.num_key_value_heads, a.head_dim, a.num_kv_groups) == (4, 2, 16, 2)
    assert a.rms_norm_eps == 1e-5 and a.rope_theta == 10000.0 and a.rope_scaling is None
    assert a.tie_word_embeddings and a.stop_token_ids == (2,)
    b = LlamaConfig.from_dict(tiny_configs.TINY_B)
    assert b.head_dim == 32 and b.num_kv_groups == 3 and not b.tie_word_embeddings
    assert b.rope_scaling == RopeScaling("llama3", 8.0, 1.0, 4.0, 32)
    assert b.stop_token_ids == (6, 7) and b.rms_norm_eps == 1e-6


def test_head_dim_is_honoured_or_derived():
    c = LlamaConfig.from_dict(tiny_configs.TINY_C)
    assert c.head_dim == 48 and c.hidden_size != c.head_dim * c.num_attention_heads
    raw = dict(tiny_configs.TINY_A)
    assert LlamaConfig.from_dict(raw).head_dim == 16


def test_defaults_of_optional_keys_follow_the_reference():
    raw = {k: v for k, v in tiny_configs.TINY_A.items()
           if k not in ("tie_word_embeddings", "bos_token_id", "eos_token_id", "torch_dtype", "rope_scaling")}
    c = LlamaConfig.from_dict(raw)
    assert c.tie_word_embeddings is True and c.bos_token_id == 128000 and c.eos_token_id == (128001,)
    assert c.torch_dtype == "bfloat16" and c.rope_scaling is None
    rs = RopeScaling.from_dict({})
    assert (rs.rope_type, rs.factor, rs.low_freq_factor, rs.high_freq_factor,
            rs.original_max_position_embeddings) == ("default", 1.0, 1.0, 4.0, 8192)


def test_round_trip_through_json(tmp_path):
    for raw in tiny_configs.CONFIGS.values():
        c = LlamaConfig.from_dict(raw)
        p = tmp_path / "config.json"
        p.write_text(json.dumps(c.to_dict()))
        assert LlamaConfig.from_json(p) == c
        assert LlamaConfig.from_json(tmp_path) == c


@pytest.mark.parametrize("change,match", [
    ({"hidden_size": None}, "required"),
    ({"num_attention_heads": 5}, "divisible"),
    ({"num_key_value_heads": 3}, "divisible"),
    ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
    ({"attention_bias": True}, "attention_bias"),
    ({"mlp_bias": True}, "mlp_bias"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "rope_type"),
    ({"head_dim": 15}, "head_dim"),
    ({"torch_dtype": "int8"}, "torch_dtype"),
    ({"vocab_size": -1}, "vocab_size"),
])
def test_refuses_what_it_cannot_run(change, match):
    raw = dict(tiny_configs.TINY_A)
    for k, v in change.items():
        if v is None:
            raw.pop(k)
        else:
            raw[k] = v
    with pytest.raises(ConfigError, match=match):
        LlamaConfig.from_dict(raw)


def test_preset_is_a_config_file_with_the_8b_sizes():
    c = LlamaConfig.from_json(preset_path("llama-3.1-8b"))
    assert c.num_parameters() == 8_030_261_248
    assert LlamaConfig.from_json(preset_path("llama-3.2-1b")).num_parameters() == 1_235_814_400
    assert LlamaConfig.from_json(preset_path("llama-3.2-3b")).num_parameters() == 3_212_749_824
    with pytest.raises(FileNotFoundError):
        preset_path("nope")


# ---- registry (mirrors the reference's benchmarks/test_model_registry.py:29-47)
def test_registry_resolves_llama_by_architecture_and_by_model_type():
    assert "LlamaForCausalLM" in registry.registered()
    assert registry.resolve({"architectures": ["LlamaForCausalLM"]}).config_cls is LlamaConfig
    assert registry.resolve({"model_type": "llama"}).name == "LlamaForCausalLM"


def test_registry_prefers_nested_text_config_model_type():
    arch = registry.resolve({"model_type": "some_wrapper", "text_config": {"model_type": "llama"}})
    assert arch.name == "LlamaForCausalLM"


def test_registry_rejects_unknown_and_duplicate():
    with pytest.raises(ValueError, match="unsupported architecture"):
        registry.resolve({"architectures": ["MambaForCausalLM"], "model_type": "mamba"})
    with pytest.raises(ValueError, match="neither"):
        registry.resolve({})
    with pytest.raises(ValueError, match="already registered"):
        registry.register_architecture("LlamaForCausalLM", ("llama",), config_cls=dict, spec_builder=len)
    with pytest.raises(ValueError, match="already registered"):
        registry.register_architecture("Other", ("llama",), config_cls=dict, spec_builder=len)


def test_registry_takes_a_new_architecture_and_lets_it_go():
    registry.register_architecture("ToyForCausalLM", ("toy",), config_cls=LlamaConfig, spec_builder=len)
    try:
        assert registry.resolve({"model_type": "toy"}).name == "ToyForCausalLM"
    finally:
        registry.unregister_architecture("ToyForCausalLM")
    with pytest.raises(ValueError):
        registry.resolve({"model_type": "toy"})


def test_resolve_path(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(tiny_configs.TINY_B))
    arch, cfg = registry.resolve_path(tmp_path)
    assert arch.name == "LlamaForCausalLM" and cfg.num_hidden_layers == 3
    with pytest.raises(FileNotFoundError):
        registry.resolve_path(tmp_path / "missing")


def test_shipped_configurations_include_the_two_tiny_ones():
    a = LlamaConfig.from_json(preset_path("tiny-a"))
    b = LlamaConfig.from_json(preset_path("tiny-b"))
    assert (a.num_hidden_layers, a.hidden_size, a.num_attention_heads, a.num_key_value_heads, a.head_dim,
            a.intermediate_size, a.vocab_size, a.tie_word_embeddings, a.rope_scaling) == (2, 64, 4, 2, 16, 176, 256, True, None)
    assert (b.num_hidden_layers, b.hidden_size, b.num_attention_heads, b.num_key_value_heads, b.head_dim,
            b.intermediate_size, b.vocab_size, b.tie_word_embeddings) == (3, 96, 3, 1, 32, 256, 384, False)
    assert b.rope_scaling.rope_type == "llama3" and b.rope_scaling.original_max_position_embeddings == 32
    assert b.rms_norm_eps == 1e-6 and a.rms_norm_eps == 1e-5


def test_command_line_refusals(capsys):
    from simple_inference_autoresearch_b200 import inference
    for argv, words in (
        (["--model", "no-such-model", "--prompt-len", "4"], "no such folder"),
        (["--model", "no-such-model", "--random-weights", "--prompt-len", "4"], "no preset"),
        (["--model", "tiny-a", "--random-weights", "--prompt-len", "4", "--batch", "0"], "--batch must be at least 1"),
    ):
        with pytest.raises(SystemExit) as e:
            inference.main(argv)
        assert e.value.code == 2 and words in capsys.readouterr().err
