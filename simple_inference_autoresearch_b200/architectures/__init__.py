"""Architectures the library can build; importing this package registers them."""
from ..registry import register_architecture
from ..config.llama import LlamaConfig
from .llama import llama_model_spec

register_architecture("LlamaForCausalLM", model_types=("llama",), config_cls=LlamaConfig,
                      spec_builder=llama_model_spec)
