"""Plain torch restatements of every CUDA kernel, one function per kernel, with
the kernels' own signatures (see ``simple_inference_autoresearch_b200/kernels/ops.py``).

Two uses, both in tests only:
 * the ``-m gpu`` kernel tests compare each CUDA kernel with its function here,
   at sizes other than the engine's;
 * the CPU tests of the engine's logic (batching, cache, slots, schedule) swap
   these in for ``ops`` so that the step function can run without a GPU.  The
   library itself never does that: it has no CPU path.

Arithmetic is float32 throughout (float64 where noted); inputs in bfloat16 are
upcast first and outputs are rounded once, as the kernels do.
"""

from __future__ import annotations

import math
from typing import Optional

import torch

from tests import plain_llama

DECODE_CHUNK = 256


def embed(tokens, table):
    v = table.shape[0]
    ids = tokens.long()
    if ((ids < 0) | (ids >= v)).any():
        raise RuntimeError("a kernel reported: a token id outside [0, vocab_size) was fed")
    return table[ids].to(torch.float32)


def gather_rows(src, rows):
    return src[rows.long()].clone()


def add_rmsnorm(residual, delta, weight, eps, out_dtype):
    if delta is not None:
        residual += delta
    var = residual.pow(2).mean(dim=-1, keepdim=True)
    return (residual * torch.rsqrt(var + eps) * weight.to(torch.float32)).to(out_dtype)


def linear(x, w, out_dtype, add_to=None, next_norm=None, options=None):
    return (x.to(torch.float32) @ w.to(torch.float32).T).to(out_dtype)


def _positions(meta):
    qs = meta.q_start.tolist()
    base = meta.base_len.tolist()
    pos, seq = [], []
    for b in range(meta.n_seqs):
        for t in range(qs[b], qs[b + 1]):
            pos.append(base[b] + t - qs[b])
            seq.append(b)
    return pos, seq


def rotate(x, positions, inv_freq, rotary_dim, interleaved):
    """x: [T, heads, D]; the first ``rotary_dim`` dims of every head rotated by position *
    inv_freq, in pairs (i, i + rotary_dim/2) or, ``interleaved``, (2i, 2i+1); the rest untouched."""
    ang = torch.outer(torch.as_tensor(positions, dtype=torch.float32), inv_freq.cpu().float())
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    out = x.clone()
    half = rotary_dim // 2
    if interleaved:
        a, c = x[..., 0:rotary_dim:2], x[..., 1:rotary_dim:2]
        out[..., 0:rotary_dim:2] = a * cos - c * sin
        out[..., 1:rotary_dim:2] = c * cos + a * sin
    else:
        a, c = x[..., :half], x[..., half:rotary_dim]
        out[..., :half] = a * cos - c * sin
        out[..., half:rotary_dim] = c * cos + a * sin
    return out


def rope_kv_write(qkv, rotary, kv, meta, n_heads, n_kv_heads, head_dim, write_kv=True):
    n = qkv.shape[0]
    pos, seq = _positions(meta)
    x = qkv.view(n, n_heads + 2 * n_kv_heads, head_dim).to(torch.float32)
    q, k, v = x[:, :n_heads], x[:, n_heads:n_heads + n_kv_heads], x[:, n_heads + n_kv_heads:]
    if rotary is not None:
        inv_freq = getattr(rotary, "inv_freq", rotary)
        rotary_dim = int(getattr(rotary, "rotary_dim", None) or 2 * inv_freq.numel())
        interleaved = bool(getattr(rotary, "interleaved", False))
        q = rotate(q, pos, inv_freq, rotary_dim, interleaved)
        k = rotate(k, pos, inv_freq, rotary_dim, interleaved)
    qkv.view(n, n_heads + 2 * n_kv_heads, head_dim)[:, :n_heads] = q.to(qkv.dtype)
    if not write_kv:
        return
    slots = meta.slot_ids.tolist()
    P = kv.page_tokens
    for t in range(n):
        slot = slots[seq[t]]
        page = int(kv.block_table[slot, pos[t] // P])
        if page < 0:
            raise RuntimeError("a kernel reported: a cache write met a position without a page")
        kv.k[page, :, pos[t] % P, :] = k[t].to(kv.k.dtype)
        kv.v[page, :, pos[t] % P, :] = v[t].to(kv.v.dtype)


def _gather_kv(kv, slot, length):
    P = kv.page_tokens
    pages = kv.block_table[slot, : -(-length // P)].long()
    k = kv.k[pages].permute(1, 0, 2, 3).reshape(kv.k.shape[1], -1, kv.k.shape[3])[:, :length]
    v = kv.v[pages].permute(1, 0, 2, 3).reshape(kv.v.shape[1], -1, kv.v.shape[3])[:, :length]
    return k.to(torch.float32), v.to(torch.float32)


def attention(qkv, kv, meta, n_heads, n_kv_heads, head_dim, scale, window=None, options=None):
    n = qkv.shape[0]
    out = torch.zeros(n, n_heads * head_dim, dtype=torch.float32)
    q_all = qkv.view(n, n_heads + 2 * n_kv_heads, head_dim)[:, :n_heads].to(torch.float32)
    qs, base, slots = meta.q_start.tolist(), meta.base_len.tolist(), meta.slot_ids.tolist()
    g = n_heads // n_kv_heads
    for b in range(meta.n_seqs):
        ql = qs[b + 1] - qs[b]
        k, v = _gather_kv(kv, slots[b], base[b] + ql)
        for i in range(ql):
            t = qs[b] + i
            visible = base[b] + i + 1
            first = 0 if window is None else max(0, visible - window)
            for hq in range(n_heads):
                s = (k[hq // g, first:visible] @ q_all[t, hq]) * scale
                p = torch.softmax(s, dim=0)
                out[t, hq * head_dim:(hq + 1) * head_dim] = p @ v[hq // g, first:visible]
    return out.to(qkv.dtype)


def rope_and_attention(qkv, rotary, kv, meta, n_heads, n_kv_heads, head_dim, scale, write_kv=True, window=None,
                       options=None):
    rope_kv_write(qkv, rotary, kv, meta, n_heads, n_kv_heads, head_dim, write_kv=write_kv)
    return attention(qkv, kv, meta, n_heads, n_kv_heads, head_dim, scale, window=window)


def swiglu(gate_up, interleaved=False):
    i = gate_up.shape[1] // 2
    x = gate_up.to(torch.float32)
    g, u = (x[:, 0::2], x[:, 1::2]) if interleaved else (x[:, :i], x[:, i:])
    return (g * torch.sigmoid(g) * u).to(gate_up.dtype)


def linear_swiglu(x, w_interleaved, options=None):
    return swiglu(linear(x, w_interleaved, torch.float32), interleaved=True).to(x.dtype)


def advance_lengths(base_len, q_start, n_seqs):
    base_len[:n_seqs] += q_start[1:n_seqs + 1] - q_start[:n_seqs]


def sample(logits, temperature, top_k, top_p, seeds, draw_index, advance_index=False, out=None):
    r = logits.shape[0]
    res = torch.empty(r, dtype=torch.int32) if out is None else out
    for i in range(r):
        u = plain_llama.counter_uniform(int(seeds[i]), int(draw_index[i]))
        res[i] = plain_llama.sample(logits[i].cpu(), float(temperature[i]), int(top_k[i]), float(top_p[i]), u)
        if advance_index:
            draw_index[i] += 1
    return res


def check_status(device):
    return None


def install(monkeypatch) -> None:
    """Swaps the functions above in for the CUDA ones (CPU tests of engine logic)."""
    from simple_inference_autoresearch_b200.kernels import ops

    for name in ("embed", "gather_rows", "add_rmsnorm", "linear", "linear_swiglu", "rope_kv_write", "attention", "rope_and_attention",
                 "swiglu",
                 "advance_lengths", "sample", "check_status"):
        monkeypatch.setattr(ops, name, globals()[name])
