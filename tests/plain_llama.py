"""A plain, slow Llama decoder: whole sequences, no cache, float32 on the CPU.

This file is the oracle the engine is compared with.  It is written from the
reference project's formulas (each function cites the file and lines it restates)
and shares no code with the library: it parses ``config.json`` dictionaries
itself, takes weights as a plain ``{checkpoint name: tensor}`` dict, and has one
function per part.  Agreement with the reference's own model code is checked
once in ``tests/golden/`` (see ``make_golden.py`` there).
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch


# ----------------------------------------------------------------------------- configuration
def parse_config(raw: dict) -> dict:
    """Sizes and constants from config.json keys (config.py:84-109); ``head_dim``
    is honoured when present, else hidden_size // num_attention_heads (config.py:81)."""
    c = {
        "H": raw["hidden_size"],
        "I": raw["intermediate_size"],
        "L": raw["num_hidden_layers"],
        "V": raw["vocab_size"],
        "Hq": raw["num_attention_heads"],
        "Hkv": raw["num_key_value_heads"],
        "eps": float(raw["rms_norm_eps"]),
        "theta": float(raw["rope_theta"]),
        "max_pos": raw["max_position_embeddings"],
        "scaling": raw.get("rope_scaling"),
        "tied": bool(raw.get("tie_word_embeddings", True)),  # default True: config.py:107
    }
    c["D"] = raw.get("head_dim") or c["H"] // c["Hq"]
    return c


# ----------------------------------------------------------------------------- parts
def rope_inv_freq(D: int, theta: float, scaling: Optional[dict]) -> torch.Tensor:
    """ops/rope.py:97-98 (base frequencies, float32) and ops/rope.py:128-163
    (llama3 scaling: per frequency in Python floats, stored as float32)."""
    idx = torch.arange(0, D, 2, dtype=torch.float32)
    freqs = 1.0 / (theta ** (idx / D))
    rope_type = (scaling or {}).get("rope_type", (scaling or {}).get("type", "default"))
    if rope_type == "llama3":
        factor = float(scaling.get("factor", 1.0))
        low = float(scaling.get("low_freq_factor", 1.0))
        high = float(scaling.get("high_freq_factor", 4.0))
        orig = int(scaling.get("original_max_position_embeddings", 8192))
        low_wl, high_wl = orig / low, orig / high
        new = []
        for f in freqs.tolist():
            wl = 2 * math.pi / f
            if wl < high_wl:
                new.append(f)
            elif wl > low_wl:
                new.append(f / factor)
            else:
                smooth = (orig / wl - low) / (high - low)
                new.append((1 - smooth) * f / factor + smooth * f)
        freqs = torch.tensor(new, dtype=torch.float32)
    return freqs


def rope_tables(positions: torch.Tensor, inv_freq: torch.Tensor):
    """ops/rope.py:108-118: angles = outer(position, freq) in float32, duplicated
    over both halves, then cos and sin."""
    ang = torch.outer(positions.to(torch.float32), inv_freq)
    ang = torch.cat([ang, ang], dim=-1)
    return ang.cos(), ang.sin()


def rope_apply(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x: [T, heads, D].  Split-half pairing (ops/rope.py:188-203,230-234):
    out = x * cos + rotate_half(x) * sin with rotate_half = cat(-x2, x1)."""
    half = x.shape[-1] // 2
    rot = torch.cat([-x[..., half:], x[..., :half]], dim=-1)
    return x * cos[:, None, :] + rot * sin[:, None, :]


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """kernels/rmsnorm_kernel.py:99-107: x * w * rsqrt(mean(x^2) + eps), all float32."""
    x = x.to(torch.float32)
    var = x.pow(2).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(var + eps) * w.to(torch.float32)


def attention_causal(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: Optional[int] = None) -> torch.Tensor:
    """q: [T, Hq, D], k, v: [T, Hkv, D] -> [T, Hq*D].
    Query head hq reads kv head hq // G (kernels/attention_kernel.py:169); scores
    (q.k) * 1/sqrt(D), the scale after the dot (kernels/attention_kernel.py:204,275-276);
    key j visible to row i iff j <= i (kernels/attention_kernel.py:184,206-209 with
    Tq == Tk); softmax over the visible keys (kernels/attention_kernel.py:212-226).
    ``window`` is not the reference's (it has no sliding window, ops/attention.py:337-342): the
    test of a windowed cache group uses it; row i then sees keys i - window + 1 .. i."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    G = Hq // Hkv
    scale = 1.0 / math.sqrt(D)
    out = torch.empty(T, Hq, D, dtype=torch.float32)
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    if window is not None:
        mask &= torch.ones(T, T, dtype=torch.bool).triu(-(window - 1))
    for hq in range(Hq):
        hkv = hq // G
        s = (q[:, hq, :] @ k[:, hkv, :].T) * scale
        s = s.masked_fill(~mask, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, hq, :] = p @ v[:, hkv, :]
    return out.reshape(T, Hq * D)


def attention_block(h: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str, c: dict,
                    inv_freq: torch.Tensor, kv_override=None, return_kv: bool = False, window: Optional[int] = None):
    """ops/attention.py:139-178 (q, k, v projections, head index the slow axis),
    :291-292 (rotate q and k), :315-332 (attention), :348 (output projection)."""
    T = h.shape[0]
    q = (h @ w[prefix + "q_proj.weight"].T).view(T, c["Hq"], c["D"])
    k = (h @ w[prefix + "k_proj.weight"].T).view(T, c["Hkv"], c["D"])
    v = (h @ w[prefix + "v_proj.weight"].T).view(T, c["Hkv"], c["D"])
    cos, sin = rope_tables(torch.arange(T), inv_freq)
    q = rope_apply(q, cos, sin)
    k = rope_apply(k, cos, sin)
    if kv_override is not None:       # a run that reads the cache another run wrote
        k, v = kv_override
    a = attention_causal(q, k, v, window)
    out = a @ w[prefix + "o_proj.weight"].T
    return (out, (k, v)) if return_kv else out


def swiglu_mlp(h: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str) -> torch.Tensor:
    """ops/mlp.py:208-214: gate and up projections, silu(gate) * up
    (kernels/swiglu_kernel.py:139-140: gate * sigmoid(gate) * up), down projection."""
    g = h @ w[prefix + "gate_proj.weight"].T
    u = h @ w[prefix + "up_proj.weight"].T
    f = g * torch.sigmoid(g) * u
    return f @ w[prefix + "down_proj.weight"].T


def block(x: torch.Tensor, w: Dict[str, torch.Tensor], i: int, c: dict, inv_freq: torch.Tensor,
          kv_override=None, return_kv: bool = False, window: Optional[int] = None):
    """model/block.py:8-9: x += Attn(norm(x)); x += MLP(norm(x))."""
    p = f"model.layers.{i}."
    h = rmsnorm(x, w[p + "input_layernorm.weight"], c["eps"])
    a = attention_block(h, w, p + "self_attn.", c, inv_freq, kv_override, return_kv, window)
    kv = None
    if return_kv:
        a, kv = a
    x = x + a
    h = rmsnorm(x, w[p + "post_attention_layernorm.weight"], c["eps"])
    x = x + swiglu_mlp(h, w, p + "mlp.")
    return (x, kv) if return_kv else x


# ----------------------------------------------------------------------------- whole model
def forward(weights: Dict[str, torch.Tensor], raw_config: dict, tokens: Sequence[int],
            schedule: Optional[List[tuple]] = None, windows: Optional[dict] = None,
            rows: Optional[Sequence[int]] = None) -> torch.Tensor:
    """Logits [T, V] at every position of one whole sequence (model/llama.py:170-199,
    without its last-position slice).  ``schedule``: optional run order as
    (layer, cache_entry, writes_cache) tuples; default layer 0..L-1.  ``windows``: layer -> key
    window, for tests of windowed layers only (see ``attention_causal``).  ``rows``: the positions
    whose logits are returned ([len(rows), V]; the reference keeps the last one, model/llama.py:189-191)."""
    windows = windows or {}
    c = parse_config(raw_config)
    w = {k: v.to(torch.float32) for k, v in weights.items()}
    inv_freq = rope_inv_freq(c["D"], c["theta"], c["scaling"])
    ids = torch.as_tensor(list(tokens), dtype=torch.long)
    x = w["model.embed_tokens.weight"][ids]                      # ops/embedding.py:62-65
    if schedule is None:
        for i in range(c["L"]):
            x = block(x, w, i, c, inv_freq, window=windows.get(i))
    else:
        stored = {}
        for layer, entry, writes in schedule:
            if writes:
                x, kv = block(x, w, layer, c, inv_freq, return_kv=True)
                stored[entry] = kv
            else:
                x = block(x, w, layer, c, inv_freq, kv_override=stored[entry])
    if rows is not None:
        x = x[torch.as_tensor(list(rows), dtype=torch.long)]
    x = rmsnorm(x, w["model.norm.weight"], c["eps"])             # model/llama.py:194
    head = w["model.embed_tokens.weight"] if c["tied"] else w["lm_head.weight"]   # ops/embedding.py:109-126
    return x @ head.T


# ----------------------------------------------------------------------------- sampling
_M64 = (1 << 64) - 1


def counter_uniform(seed64: int, index: int) -> float:
    """splitmix64 of (seed, index) -> 24-bit uniform in [0, 1); the library's
    counter-based generator restated (the reference uses torch's global generator)."""
    z = ((seed64 & _M64) + 0x9E3779B97F4A7C15 * (index + 1)) & _M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    z ^= z >> 31
    return (z >> 40) / 16777216.0


def kept_probabilities(logits: torch.Tensor, temperature: float, top_k: int, top_p: float) -> torch.Tensor:
    """Probabilities [V] after temperature -> top-k -> top-p, in the reference's
    order and meaning (sampling.py:151-236): exactly k candidates (ties at the
    k-th value: lower ids first); nucleus keeps a token iff the mass strictly
    before it in descending order is <= top_p (sampling.py:216-221), tokens of
    equal logit together."""
    x = logits.to(torch.float64)
    V = x.numel()
    keep = torch.ones(V, dtype=torch.bool)
    if 0 < top_k < V:
        order = sorted(range(V), key=lambda i: (-x[i].item(), i))
        keep[:] = False
        keep[order[:top_k]] = True
    z = x / temperature
    probs = torch.where(keep, torch.exp(z - z[keep].max()), torch.zeros_like(z))
    probs = probs / probs.sum()
    if top_p < 1.0:
        mass_gt = torch.tensor([probs[(x > x[i]) & keep].sum().item() for i in range(V)], dtype=torch.float64)
        keep = keep & (mass_gt <= top_p)
        probs = torch.where(keep, probs, torch.zeros_like(probs))
        probs = probs / probs.sum()
    return probs


def sample(logits: torch.Tensor, temperature: float, top_k: int, top_p: float, u: float) -> int:
    """temperature == 0: argmax, lowest id on ties (sampling.py:170-171).  Else the
    first token, in token-id order, whose cumulative kept probability reaches u."""
    if temperature == 0:
        return int(torch.argmax(logits.to(torch.float64)).item())
    probs = kept_probabilities(logits, temperature, top_k, top_p)
    cdf = torch.cumsum(probs, 0)
    idx = torch.nonzero((cdf >= u) & (probs > 0))
    if idx.numel() == 0:
        return int(torch.nonzero(probs > 0)[-1].item())
    return int(idx[0].item())
