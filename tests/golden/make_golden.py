"""Runs the reference project's own model code on the CPU for two tiny random
models and stores its logits, so that the plain implementation in
``tests/plain_llama.py`` can be compared with it without the reference present.

    USE_TRITON=false USE_CUDA_GRAPH=false USE_FUSED_SAMPLE=false \
        python tests/golden/make_golden.py /path/to/reference

The reference quantises every linear weight to int8 at load, also on its CPU
path (ops/attention.py:127-137, ops/mlp.py:127-135, ops/embedding.py:113-121), so
what is stored beside the logits are its *effective* weights (int8 value times
per-row scale, read back from its buffers); the plain implementation is run on
those.  Stored per model: the config.json dictionary, the effective weights
under checkpoint names (float32), the token ids, the reference's logits at the
last position of two whole prompts of equal length (its forward returns the last
position only, model/llama.py:189-191) and its logits at every position of a
sequence fed token by token through its KVCache (float32, 64 positions at most,
below the length where it switches to int8 keys, model/kv_cache.py:74,115).
"""

import json
import os
import sys
from pathlib import Path

os.environ.setdefault("USE_TRITON", "false")
os.environ.setdefault("USE_CUDA_GRAPH", "false")
os.environ.setdefault("USE_FUSED_SAMPLE", "false")

import torch  # noqa: E402

HERE = Path(__file__).resolve().parent

MODELS = {
    # smaller than the test suite's tiny configurations so that the stored files stay small
    "g1": {"hidden_size": 32, "intermediate_size": 48, "num_hidden_layers": 2, "vocab_size": 64,
           "num_attention_heads": 4, "num_key_value_heads": 2, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
           "max_position_embeddings": 64, "rope_scaling": None, "tie_word_embeddings": True},
    "g2": {"hidden_size": 48, "intermediate_size": 80, "num_hidden_layers": 3, "vocab_size": 96,
           "num_attention_heads": 3, "num_key_value_heads": 1, "rms_norm_eps": 1e-6, "rope_theta": 500000.0,
           "max_position_embeddings": 64,
           "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                            "original_max_position_embeddings": 16},
           "tie_word_embeddings": False},
}


def main(ref_path: str) -> None:
    sys.path.insert(0, ref_path)
    from config import ModelConfig, RopeScalingConfig
    from model.kv_cache import KVCache
    from model.llama import LlamaModel

    for name, raw in MODELS.items():
        g = torch.Generator().manual_seed({"g1": 101, "g2": 202}[name])
        rs = raw["rope_scaling"]
        scaling = (RopeScalingConfig.from_dict(rs) if rs else RopeScalingConfig("default", 1.0, 1.0, 4.0, 8192))
        cfg = ModelConfig(**{k: v for k, v in raw.items() if k != "rope_scaling"}, rope_scaling=scaling,
                          torch_dtype="float32")
        H, I, V, D = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size, cfg.head_dim
        n = lambda *s: torch.randn(*s, generator=g) * 0.05  # noqa: E731
        short = {"embed_tokens": n(V, H), "norm": 1 + n(H)}
        if not cfg.tie_word_embeddings:
            short["lm_head"] = n(V, H)
        for i in range(cfg.num_hidden_layers):
            p = f"layers.{i}."
            short.update({p + "attn_norm": 1 + n(H), p + "mlp_norm": 1 + n(H),
                          p + "attn.wq": n(cfg.num_attention_heads * D, H),
                          p + "attn.wk": n(cfg.num_key_value_heads * D, H),
                          p + "attn.wv": n(cfg.num_key_value_heads * D, H),
                          p + "attn.wo": n(H, cfg.num_attention_heads * D),
                          p + "mlp.w_gate": n(I, H), p + "mlp.w_up": n(I, H), p + "mlp.w_down": n(H, I)})

        class Fake:
            def get(self, key, device="cpu"):
                return short[key].clone()

        model = LlamaModel(cfg, torch.device("cpu"))
        model.load_weights(Fake())
        model.eval()

        # effective weights under checkpoint names
        eff = {"model.embed_tokens.weight": model.embed.weight.detach().float(),
               "model.norm.weight": model.norm.weight.detach().float()}
        if not cfg.tie_word_embeddings:
            eff["lm_head.weight"] = model.head.w_int8.float() * model.head.w_scale[:, None].float()
        nq, nkv = cfg.num_attention_heads * D, cfg.num_key_value_heads * D
        for i, layer in enumerate(model.layers):
            p = f"model.layers.{i}."
            qkv = layer.attn.w_qkv_int8.float() * layer.attn.w_qkv_scale[:, None].float()
            gu = layer.mlp.w_gate_up_int8.float() * layer.mlp.w_gate_up_scale[:, None].float()
            eff.update({
                p + "input_layernorm.weight": layer.attn_norm.weight.detach().float(),
                p + "post_attention_layernorm.weight": layer.mlp_norm.weight.detach().float(),
                p + "self_attn.q_proj.weight": qkv[:nq], p + "self_attn.k_proj.weight": qkv[nq:nq + nkv],
                p + "self_attn.v_proj.weight": qkv[nq + nkv:], p + "self_attn.o_proj.weight": layer.attn.wo.detach().float(),
                p + "mlp.gate_proj.weight": gu[:I], p + "mlp.up_proj.weight": gu[I:],
                p + "mlp.down_proj.weight": layer.mlp.w_down_int8.float() * layer.mlp.w_down_scale[:, None].float(),
            })

        ids = torch.randint(0, V, (2, 40), generator=g)
        with torch.no_grad():
            whole_last = model(ids, start_pos=0)[:, -1, :].float()
            cache = KVCache(cfg.num_hidden_layers, 2, 64, cfg.num_key_value_heads, D, dtype=torch.float32,
                            device=torch.device("cpu"))
            steps = [model(ids[:, t:t + 1], start_pos=t, kv_cache=cache)[:, -1, :].float() for t in range(40)]
        stepwise = torch.stack(steps, dim=1)   # [2, 40, V]
        from safetensors.torch import save_file
        out = {"ids": ids.to(torch.int32), "whole_last": whole_last.contiguous(), "stepwise": stepwise.contiguous()}
        out.update({"w:" + k: v.contiguous() for k, v in eff.items()})
        save_file(out, str(HERE / f"{name}.safetensors"), metadata={"config": json.dumps(raw)})
        print(name, "saved", sum(v.numel() for v in out.values()) * 4 // 1024, "KiB")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/reference")
    main(sys.argv[1])
