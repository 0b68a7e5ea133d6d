"""The Llama dense decoder described with the library's parts.

Tensor names are the checkpoint's own (the reference's rename table,
loader.py:64-123, lists the same twelve patterns): ``model.embed_tokens.weight``,
``model.layers.{i}.input_layernorm.weight``, ``...self_attn.{q,k,v,o}_proj.weight``,
``...post_attention_layernorm.weight``, ``...mlp.{gate,up,down}_proj.weight``,
``model.norm.weight`` and, when the embeddings are not tied, ``lm_head.weight``
(model/llama.py:107-135).
"""

from __future__ import annotations

from ..config.llama import LlamaConfig
from ..engine.model import ModelSpec
from ..parts.base import PartSpec


def llama_model_spec(cfg: LlamaConfig, norm_weight_init: str = None) -> ModelSpec:
    """``norm_weight_init`` (default: the configuration's) and the configuration's
    ``initializer_range`` only matter to the random-weights writer."""
    scaling = cfg.rope_scaling.to_dict() if cfg.rope_scaling is not None else None
    std = cfg.initializer_range
    norm_weight_init = norm_weight_init or cfg.norm_weight_init
    norm = lambda prefix: PartSpec("rmsnorm", {"prefix": prefix, "hidden_size": cfg.hidden_size,  # noqa: E731
                                               "eps": cfg.rms_norm_eps, "weight_init": norm_weight_init,
                                               "weight_std": std})
    layers = []
    for i in range(cfg.num_hidden_layers):
        layers.append(PartSpec("prenorm", {
            "prefix": f"model.layers.{i}.",
            "mixer_norm": norm("input_layernorm."),
            "mixer": PartSpec("gqa_attention", {
                "prefix": "self_attn.", "hidden_size": cfg.hidden_size, "n_heads": cfg.num_attention_heads,
                "n_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim, "init_std": std}),
            "ffn_norm": norm("post_attention_layernorm."),
            "feed_forward": PartSpec("swiglu", {
                "prefix": "mlp.", "hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size,
                "init_std": std}),
        }))
    return ModelSpec(
        architecture=cfg.architecture,
        vocab_size=cfg.vocab_size,
        hidden_size=cfg.hidden_size,
        max_position=cfg.max_position_embeddings,
        embedding_name="model.embed_tokens.weight",
        head_name=None if cfg.tie_word_embeddings else "lm_head.weight",
        position=PartSpec("rotary", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta, "scaling": scaling}),
        layers=tuple(layers),
        final_norm=norm("model.norm."),
        stop_token_ids=cfg.stop_token_ids,
        embedding_std=std,
        # a tied model's checkpoint may still carry the head; every other extra tensor is an error
        ignorable_tensors=("lm_head.weight",) if cfg.tie_word_embeddings else (),
    )
