"""Typed configuration of the Llama dense decoder, read from its config.json keys.

Key names, required/optional status and defaults follow the reference's
``ModelConfig.from_hf_config`` (config.py:84-109) and ``RopeScalingConfig.from_dict``
(config.py:29-36).  Differences, all deliberate:

* ``head_dim`` is honoured when config.json carries it (the reference always
  derives ``hidden_size // num_attention_heads``, config.py:81).
* ``rope_scaling: null`` (or ``rope_type == "default"``) means unscaled rotary
  frequencies; the reference's model constructor cannot take ``null``
  (model/llama.py:65-70).
* ``eos_token_id`` may be an int or a list; it becomes the model's stop set.
* Options the kernels do not implement (biases, an activation other than SiLU,
  an unknown rope_type) are refused here with a clear error instead of being
  silently ignored.
* Two keys only the random-weights mode reads (the reference has no such mode):
  ``initializer_range`` (the checkpoint format's own key: the standard deviation of
  matrices and embeddings, default 0.02) and ``norm_weight_init`` (this library's:
  ``"ones"`` or ``"ones_plus_normal"``, norm weights 1 or 1 + N(0, initializer_range)).
"""

from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Mapping, Optional, Tuple


class ConfigError(ValueError):
    """A config.json that this library cannot run, with the offending key named."""


@dataclass(frozen=True)
class RopeScaling:
    """``rope_scaling`` block of config.json (reference: config.py:19-36)."""

    rope_type: str = "default"
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position_embeddings: int = 8192

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "RopeScaling":
        # HF configs written before the rename use "type" for the same key.
        rope_type = d.get("rope_type", d.get("type", "default"))
        return cls(
            rope_type=str(rope_type),
            factor=float(d.get("factor", 1.0)),
            low_freq_factor=float(d.get("low_freq_factor", 1.0)),
            high_freq_factor=float(d.get("high_freq_factor", 4.0)),
            original_max_position_embeddings=int(d.get("original_max_position_embeddings", 8192)),
        )

    def to_dict(self) -> dict:
        return {
            "rope_type": self.rope_type,
            "factor": self.factor,
            "low_freq_factor": self.low_freq_factor,
            "high_freq_factor": self.high_freq_factor,
            "original_max_position_embeddings": self.original_max_position_embeddings,
        }


_REQUIRED = (
    "hidden_size",
    "intermediate_size",
    "num_hidden_layers",
    "vocab_size",
    "num_attention_heads",
    "num_key_value_heads",
    "rms_norm_eps",
    "rope_theta",
    "max_position_embeddings",
)

_DTYPES = ("bfloat16", "float16", "float32")


@dataclass(frozen=True)
class LlamaConfig:
    """Every size and constant of a Llama checkpoint; nothing else in the library
    carries a model size (reference: config.py:39-82)."""

    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    vocab_size: int
    num_attention_heads: int
    num_key_value_heads: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    rope_scaling: Optional[RopeScaling] = None
    head_dim: int = 0  # 0 = derive from hidden_size // num_attention_heads
    bos_token_id: int = 128000
    eos_token_id: Tuple[int, ...] = (128001,)
    tie_word_embeddings: bool = True
    torch_dtype: str = "bfloat16"
    architecture: str = field(default="LlamaForCausalLM")
    initializer_range: float = 0.02
    norm_weight_init: str = "ones"

    def __post_init__(self):
        def bad(msg):
            raise ConfigError(msg)

        for key in ("hidden_size", "intermediate_size", "num_hidden_layers", "vocab_size",
                    "num_attention_heads", "num_key_value_heads", "max_position_embeddings"):
            v = getattr(self, key)
            if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
                bad(f"{key} must be a positive integer, got {v!r}")
        if self.head_dim == 0:
            if self.hidden_size % self.num_attention_heads:
                bad(f"hidden_size {self.hidden_size} is not divisible by num_attention_heads "
                    f"{self.num_attention_heads} and no head_dim is given")
            object.__setattr__(self, "head_dim", self.hidden_size // self.num_attention_heads)
        if self.head_dim <= 0 or self.head_dim % 2:
            bad(f"head_dim must be positive and even (rotary pairs), got {self.head_dim}")
        if self.num_attention_heads % self.num_key_value_heads:
            bad(f"num_attention_heads {self.num_attention_heads} is not divisible by "
                f"num_key_value_heads {self.num_key_value_heads}")
        if not (self.rms_norm_eps > 0):
            bad(f"rms_norm_eps must be > 0, got {self.rms_norm_eps!r}")
        if not (self.rope_theta > 0):
            bad(f"rope_theta must be > 0, got {self.rope_theta!r}")
        if self.torch_dtype not in _DTYPES:
            bad(f"torch_dtype must be one of {_DTYPES}, got {self.torch_dtype!r}")
        if not (self.initializer_range > 0):
            bad(f"initializer_range must be > 0, got {self.initializer_range!r}")
        if self.norm_weight_init not in ("ones", "ones_plus_normal"):
            bad(f"norm_weight_init must be 'ones' or 'ones_plus_normal', got {self.norm_weight_init!r}")
        if isinstance(self.eos_token_id, int):
            object.__setattr__(self, "eos_token_id", (int(self.eos_token_id),))
        else:
            object.__setattr__(self, "eos_token_id", tuple(int(t) for t in self.eos_token_id))
        rs = self.rope_scaling
        if rs is not None:
            if rs.rope_type not in ("default", "llama3"):
                bad(f"rope_scaling.rope_type {rs.rope_type!r} is not supported "
                    f"(supported: 'default', 'llama3')")
            if rs.rope_type == "llama3":
                if rs.factor <= 0:
                    bad(f"rope_scaling.factor must be > 0, got {rs.factor}")
                if rs.high_freq_factor == rs.low_freq_factor:
                    bad("rope_scaling.high_freq_factor must differ from low_freq_factor")
                if rs.original_max_position_embeddings <= 0:
                    bad("rope_scaling.original_max_position_embeddings must be > 0")

    # ---- derived -----------------------------------------------------------
    @property
    def num_kv_groups(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    @property
    def stop_token_ids(self) -> Tuple[int, ...]:
        return self.eos_token_id

    # ---- json --------------------------------------------------------------
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "LlamaConfig":
        missing = [k for k in _REQUIRED if k not in d]
        if missing:
            raise ConfigError(f"config.json lacks required key(s): {', '.join(missing)}")
        for flag in ("attention_bias", "mlp_bias"):
            if d.get(flag):
                raise ConfigError(f"{flag}=true is not supported (no bias tensors are read)")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"hidden_act {act!r} is not supported (the feed-forward is SwiGLU)")
        rs = d.get("rope_scaling")
        rope_scaling = RopeScaling.from_dict(rs) if rs is not None else None
        archs = d.get("architectures") or ["LlamaForCausalLM"]
        return cls(
            hidden_size=d["hidden_size"],
            intermediate_size=d["intermediate_size"],
            num_hidden_layers=d["num_hidden_layers"],
            vocab_size=d["vocab_size"],
            num_attention_heads=d["num_attention_heads"],
            num_key_value_heads=d["num_key_value_heads"],
            rms_norm_eps=float(d["rms_norm_eps"]),
            rope_theta=float(d["rope_theta"]),
            max_position_embeddings=d["max_position_embeddings"],
            rope_scaling=rope_scaling,
            head_dim=int(d.get("head_dim") or 0),
            bos_token_id=d.get("bos_token_id", 128000),
            eos_token_id=d.get("eos_token_id", 128001),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", True)),
            torch_dtype=d.get("torch_dtype", d.get("dtype", "bfloat16")),
            architecture=str(archs[0]),
            initializer_range=float(d.get("initializer_range", 0.02)),
            norm_weight_init=str(d.get("norm_weight_init", "ones")),
        )

    @classmethod
    def from_json(cls, path) -> "LlamaConfig":
        path = Path(path)
        if path.is_dir():
            path = path / "config.json"
        with open(path) as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> dict:
        eos = list(self.eos_token_id)
        extra = {} if self.norm_weight_init == "ones" else {"norm_weight_init": self.norm_weight_init}
        return {
            **extra,
            "initializer_range": self.initializer_range,
            "architectures": [self.architecture],
            "model_type": "llama",
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "vocab_size": self.vocab_size,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings,
            "rope_scaling": self.rope_scaling.to_dict() if self.rope_scaling else None,
            "bos_token_id": self.bos_token_id,
            "eos_token_id": eos[0] if len(eos) == 1 else eos,
            "tie_word_embeddings": self.tie_word_embeddings,
            "torch_dtype": self.torch_dtype,
            "hidden_act": "silu",
            "attention_bias": False,
            "mlp_bias": False,
        }

    def num_parameters(self) -> int:
        h, i, v = self.hidden_size, self.intermediate_size, self.vocab_size
        qkv = (self.num_attention_heads + 2 * self.num_key_value_heads) * self.head_dim * h
        o = h * self.num_attention_heads * self.head_dim
        per_layer = qkv + o + 3 * h * i + 2 * h
        head = 0 if self.tie_word_embeddings else v * h
        return v * h + self.num_hidden_layers * per_layer + h + head
