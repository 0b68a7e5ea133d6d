"""Two tiny Llama configurations that differ in every size and option, as plain
config.json dictionaries, plus helpers that make model folders in a temp dir."""

from __future__ import annotations

import json
from pathlib import Path

import torch

# 2 layers, GQA 4:2, head_dim 16, tied, unscaled rotary, eps 1e-5, norm weights 1
TINY_A = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 64, "intermediate_size": 176, "num_hidden_layers": 2, "vocab_size": 256,
    "num_attention_heads": 4, "num_key_value_heads": 2, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
    "max_position_embeddings": 128, "rope_scaling": None, "tie_word_embeddings": True,
    "bos_token_id": 1, "eos_token_id": 2, "torch_dtype": "bfloat16",
}

# 3 layers, MQA 3:1, head_dim 32 (given explicitly), untied, llama3 scaling, eps 1e-6, norm weights 1 + noise
TINY_B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 96, "intermediate_size": 256, "num_hidden_layers": 3, "vocab_size": 384,
    "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 32, "rms_norm_eps": 1e-6,
    "rope_theta": 500000.0, "max_position_embeddings": 256,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 32},
    "tie_word_embeddings": False, "bos_token_id": 5, "eos_token_id": [6, 7], "torch_dtype": "bfloat16",
}

# a third shape for the sizes the first two do not reach: hidden != heads * head_dim,
# GQA group 3, head_dim 48 (a step of 16 that is no power of two), odd vocabulary
TINY_C = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 80, "intermediate_size": 136, "num_hidden_layers": 2, "vocab_size": 331,
    "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 48, "rms_norm_eps": 1e-5,
    "rope_theta": 10000.0, "max_position_embeddings": 512, "rope_scaling": None,
    "tie_word_embeddings": False, "bos_token_id": 0, "eos_token_id": 330, "torch_dtype": "bfloat16",
}

# Tiny widths with heads of real size, so that the bfloat16 path runs on the tensor-core attention
# kernels (head_dim 64 and 128) and the tensor-core products while the plain implementation stays cheap.
# D: head_dim 64, pairs of query heads, tied, llama3 scaling whose bands all occur below position 1024
TINY_D = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 256, "intermediate_size": 344, "num_hidden_layers": 2, "vocab_size": 500,
    "num_attention_heads": 4, "num_key_value_heads": 2, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "max_position_embeddings": 1024,
    "rope_scaling": {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 64},
    "tie_word_embeddings": True, "bos_token_id": 1, "eos_token_id": 2, "torch_dtype": "bfloat16",
}

# E: head_dim 128 given explicitly (hidden / heads would be 53.3), groups of 3 query heads, untied,
# norm weights 1 + noise, an odd vocabulary
TINY_E = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 320, "intermediate_size": 520, "num_hidden_layers": 2, "vocab_size": 777,
    "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 128, "rms_norm_eps": 1e-6,
    "rope_theta": 10000.0, "max_position_embeddings": 1024, "rope_scaling": None,
    "tie_word_embeddings": False, "bos_token_id": 0, "eos_token_id": [775, 776], "torch_dtype": "bfloat16",
}

NORM_INIT = {"A": "ones", "B": "ones_plus_normal", "C": "ones_plus_normal", "D": "ones", "E": "ones_plus_normal"}
CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E}


def make_folder(tmp_path, name: str, seed: int = 0, store_dtype=torch.bfloat16, vector_dtype=None) -> Path:
    from simple_inference_autoresearch_b200.config import LlamaConfig
    from simple_inference_autoresearch_b200.weights import write_model_folder

    cfg = LlamaConfig.from_dict(CONFIGS[name])
    return write_model_folder(Path(tmp_path) / f"tiny_{name}", cfg, seed, store_dtype=store_dtype,
                              vector_dtype=vector_dtype, norm_weight_init=NORM_INIT[name])


def read_folder(folder):
    """(raw config dict, {name: tensor}) read with the safetensors library directly."""
    from safetensors.torch import load_file

    with open(Path(folder) / "config.json") as f:
        raw = json.load(f)
    return raw, load_file(str(Path(folder) / "model.safetensors"))
