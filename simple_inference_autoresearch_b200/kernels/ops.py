"""Python face of the CUDA kernels: one function per kernel (or fused pair).

Each function checks shapes and dtypes on the host, allocates the output with
torch (torch is only the allocator here) and launches the kernel on torch's
current stream through the unit's C entry point.  Nothing here computes with
torch, and nothing falls back to the CPU: a tensor that is not on a CUDA device,
or an extension that cannot be built, raises.

The parts call these functions through the module (``ops.linear(...)``).
"""

from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import build
from .options import DEFAULT, KernelOptions

c_int, c_float, c_void_p, c_longlong = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_longlong

# ------------------------------------------------------------------ plumbing
#: kernels launched through this module since import (graph replays add what the graph holds)
launch_count = 0

_signatures = {
    "elementwise": {
        "siar_embed_gather": [c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p],
        "siar_gather_rows": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
        "siar_add_rmsnorm": [c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p],
        "siar_rope_kv_write": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                               c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                               c_void_p, c_void_p, c_int, c_int],
        "siar_swiglu": [c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
        "siar_advance_lengths": [c_void_p, c_void_p, c_int, c_void_p],
        "siar_set_table_cells": [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    },
    "gemm_simt": {
        "siar_gemm_nt_simt": [c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    },
    "attention": {
        "siar_attn_prefill": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                              c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p,
                              c_void_p],
        "siar_attn_decode": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                             c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                             c_void_p, c_void_p],
        "siar_attn_decode_chunk": [],
        "siar_attn_max_head_dim": [],
    },
    "attention_mma": {
        "siar_attn_mma_prefill": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                  c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p],
        "siar_attn_mma_decode": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                 c_float, c_void_p, c_void_p],
        "siar_attn_mma_decode_rope": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                      c_int, c_int, c_int, c_float, c_void_p, c_void_p, c_int, c_int],
        "siar_attn_mma_supported": [c_int, c_int, c_int, c_int],
        "siar_attn_mma_decode_scratch_floats": [c_int, c_int, c_int, c_int, c_int, c_int],
    },
    "attention_tc": {
        # qkv, k_pool, v_pool, block_table, slot_ids, q_start, base_len, out, N, B, Hq, Hkv, D, page_tokens,
        # max_pages, n_pages, max_q_len, scale, status, stream
        "siar_attn_tc_prefill": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p,
                                 c_void_p],
        "siar_attn_tc_supported": [c_int, c_int, c_int, c_int],
    },
    "sampling": {
        "siar_sample": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                        c_void_p, c_void_p],
    },
}
_bound = {}


def _fn(unit: str, name: str):
    key = (unit, name)
    f = _bound.get(key)
    if f is None:
        lib = build.load_unit(unit)
        f = getattr(lib, name)
        f.argtypes = _signatures[unit][name]
        f.restype = c_int
        _bound[key] = f
    return f


def _launch(unit: str, name: str, *args, kernels: int = 1) -> None:
    global launch_count
    err = _fn(unit, name)(*args)
    if err != 0:
        raise RuntimeError(f"{name} failed to launch: CUDA error {err} (see cudaError_t); "
                           "sizes the kernel refuses are reported as cudaErrorInvalidValue (1)")
    launch_count += kernels


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("this library runs on a CUDA device only (no CPU path); got a "
                               f"{t.device} tensor of shape {tuple(t.shape)}")


def _is_bf16(dtype: torch.dtype) -> int:
    if dtype == torch.bfloat16:
        return 1
    if dtype == torch.float32:
        return 0
    raise TypeError(f"compute dtype must be bfloat16 or float32, got {dtype}")


# ------------------------------------------------------------------ status word
_status = {}

STATUS_MESSAGES = {
    1: "a token id outside [0, vocab_size) was fed",
    2: "a bounded device-side wait expired",
    4: "a key or a cache write met a position without a page",
    8: "a sequence is longer than the decode step was sized for (a captured step replayed past its length bucket)",
}


def status_word(device) -> torch.Tensor:
    dev = torch.device(device)
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    t = _status.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=dev)
        _status[key] = t
    return t


def check_status(device) -> None:
    """Reads the device status word (synchronises) and raises if a kernel flagged an error."""
    t = status_word(device)
    v = int(t.item())
    if v:
        t.zero_()
        what = [m for bit, m in STATUS_MESSAGES.items() if v & bit] or [f"status {v}"]
        raise RuntimeError("a kernel reported: " + "; ".join(what))


# ------------------------------------------------------------------ kernels
def embed(tokens: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """float32 [N, H] rows of ``table`` picked by int32 ``tokens``."""
    _need_cuda(tokens, table)
    assert tokens.dtype == torch.int32 and tokens.dim() == 1 and table.dim() == 2 and table.is_contiguous()
    n, (v, h) = tokens.numel(), table.shape
    out = torch.empty((n, h), dtype=torch.float32, device=table.device)
    _launch("elementwise", "siar_embed_gather", _is_bf16(table.dtype), _ptr(tokens), _ptr(table), _ptr(out),
            n, h, v, _ptr(status_word(table.device)), _stream())
    return out


def gather_rows(src: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    _need_cuda(src, rows)
    assert src.dtype == torch.float32 and src.dim() == 2 and src.is_contiguous() and rows.dtype == torch.int32
    out = torch.empty((rows.numel(), src.shape[1]), dtype=torch.float32, device=src.device)
    _launch("elementwise", "siar_gather_rows", _ptr(src), _ptr(rows), _ptr(out), rows.numel(), src.shape[1],
            _stream())
    return out


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype) -> torch.Tensor:
    """residual += delta (if given), returns rmsnorm(residual) * weight in ``out_dtype``."""
    _need_cuda(residual, delta, weight)
    assert residual.dtype == torch.float32 and residual.dim() == 2 and residual.is_contiguous()
    n, h = residual.shape
    assert weight.shape == (h,) and weight.is_contiguous()
    if delta is not None:
        assert delta.dtype == torch.float32 and delta.shape == residual.shape and delta.is_contiguous()
    out = torch.empty((n, h), dtype=out_dtype, device=residual.device)
    _launch("elementwise", "siar_add_rmsnorm", _is_bf16(out_dtype), _is_bf16(weight.dtype), _ptr(residual),
            _ptr(delta), _ptr(weight), _ptr(out), n, h, float(eps), _stream())
    return out


class NormHint:
    """What a sublayer's last product is told of the RMSNorm that follows it, so that it can leave
    that norm's inputs behind: the norm's weight (and eps, for the record)."""

    __slots__ = ("weight", "eps")

    def __init__(self, weight: torch.Tensor, eps: float):
        self.weight, self.eps = weight, eps


class Added:
    """Stands for a sublayer output that the product kernel has already added into the residual
    stream.  When the product knew the norm that follows (``NormHint``) it also left
    ``ss_parts`` [rows, parts] float32, partial sums of squares of every row of the updated residual,
    and ``scaled`` [rows, H] bfloat16 = residual * ``weight`` (that norm's weight): with
    rmsnorm(r) W^T = rsqrt(mean(r^2) + eps) * ((r * w) W^T) the next product takes ``scaled`` as its
    operand and applies the row factors to its accumulators, and no norm kernel runs.  All three are
    None when the kernel only added (the norm then runs as a kernel, without an add)."""

    __slots__ = ("ss_parts", "scaled", "weight")

    def __init__(self, ss_parts: Optional[torch.Tensor] = None, scaled: Optional[torch.Tensor] = None,
                 weight: Optional[torch.Tensor] = None):
        self.ss_parts, self.scaled, self.weight = ss_parts, scaled, weight


class NormedResidual:
    """``rmsnorm(residual) * weight`` that has not been computed: ``linear`` and ``linear_swiglu``
    take it in place of their input and, where their kernel can, multiply ``scaled`` (see ``Added``)
    with their weight and the result's rows with the norm's factors.  Anything else calls
    ``materialize``."""

    __slots__ = ("residual", "ss_parts", "scaled", "weight", "eps", "dtype")

    def __init__(self, residual: torch.Tensor, ss_parts: torch.Tensor, scaled: torch.Tensor, weight: torch.Tensor,
                 eps: float, dtype: torch.dtype):
        self.residual, self.ss_parts, self.scaled = residual, ss_parts, scaled
        self.weight, self.eps, self.dtype = weight, eps, dtype

    @property
    def shape(self):
        return self.residual.shape

    def materialize(self) -> torch.Tensor:
        return add_rmsnorm(self.residual, None, self.weight, self.eps, self.dtype)


def _fused_input(x: "NormedResidual", w: torch.Tensor, out: torch.Tensor, epilogue: int,
                 options: KernelOptions) -> bool:
    if not (options.fuse_residual_stream and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and x.scaled is not None):
        return False
    from . import gemm_tc
    return gemm_tc.try_linear(None, w, out, epilogue=epilogue, normed=x, options=options)


def linear(x, w: torch.Tensor, out_dtype: torch.dtype, add_to: Optional[torch.Tensor] = None,
           next_norm: Optional[NormHint] = None, options: KernelOptions = DEFAULT):
    """y[M, N] = x[M, K] @ w[N, K]^T with 32-bit accumulation.

    ``x`` may be a ``NormedResidual``.  With ``add_to`` (the float32 residual [M, N]) the kernel may
    add y into it instead of returning it; the result is then an ``Added``, otherwise y as always
    (the caller adds it later).  ``next_norm`` names the RMSNorm that follows the add: the kernel then
    also leaves that norm's inputs for the next product (see ``Added``)."""
    if isinstance(x, NormedResidual):
        if add_to is None and out_dtype in (torch.float32, x.dtype):
            out = torch.empty((x.shape[0], w.shape[0]), dtype=out_dtype, device=w.device)
            if _fused_input(x, w, out, 0, options):
                return out
        x = x.materialize()
    _need_cuda(x, w)
    assert x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1], (x.shape, w.shape)
    assert x.dtype == w.dtype and x.is_contiguous() and w.is_contiguous()
    m, k = x.shape
    n = w.shape[0]
    if out_dtype not in (torch.float32, x.dtype):
        raise TypeError(f"linear: output dtype {out_dtype} with input dtype {x.dtype}")
    if x.dtype == torch.bfloat16:
        from . import gemm_tc
        if (add_to is not None and options.fuse_residual_stream and out_dtype == torch.float32
                and add_to.dtype == torch.float32 and add_to.shape == (m, n) and add_to.is_contiguous()):
            parts = gemm_tc.ss_parts(m, n, k, x.device, options) if next_norm is not None else 0
            if parts > 0:
                ss = torch.empty((m, parts), dtype=torch.float32, device=x.device)
                rb = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
                if gemm_tc.try_linear(x, w, add_to, epilogue=2, ss_out=ss, rb_out=rb, next_w=next_norm.weight,
                                      options=options):
                    return Added(ss, rb, next_norm.weight)
            if gemm_tc.try_linear(x, w, add_to, epilogue=2, options=options):
                return Added()
    out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    if x.dtype == torch.bfloat16:
        if gemm_tc.try_linear(x, w, out, options=options):
            return out
    _launch("gemm_simt", "siar_gemm_nt_simt", _is_bf16(x.dtype), int(out_dtype == torch.float32), _ptr(x),
            _ptr(w), _ptr(out), m, n, k, 1, _stream())
    return out


def tc_attention_takes(dtype: torch.dtype, n_heads: int, n_kv_heads: int, head_dim: int, page_tokens: int,
                       options: KernelOptions = DEFAULT) -> bool:
    """True when the tcgen05 kernel for prompts takes these sizes (bfloat16, head_dim 64 or 128, at
    most 128 query heads per kv head, pages of 64 tokens or a multiple)."""
    if dtype != torch.bfloat16 or not (options.use_tc_attention and options.use_mma_attention):
        return False
    if head_dim not in (64, 128) or n_kv_heads <= 0 or n_heads % n_kv_heads:      # the unit is not even compiled for these
        return False
    return bool(_fn("attention_tc", "siar_attn_tc_supported")(n_heads, n_kv_heads, head_dim, page_tokens))


def rotary_layout(rotary, head_dim: int):
    """(inv_freq, rotary_dim, interleaved) of what a position encoding's ``rotary()`` returned:
    None (no rotation), a bare float32 tensor of head_dim/2 frequencies (the whole head, pairs
    (i, i + head_dim/2)), or an object with ``inv_freq`` and optionally ``rotary_dim`` (only the
    first that many dims of a head are rotated) and ``interleaved`` (pairs (2i, 2i+1))."""
    if rotary is None:
        return None, head_dim, False
    inv_freq = getattr(rotary, "inv_freq", rotary)
    rotary_dim = int(getattr(rotary, "rotary_dim", None) or 2 * inv_freq.numel())
    interleaved = bool(getattr(rotary, "interleaved", False))
    if rotary_dim % 2 or not 0 < rotary_dim <= head_dim:
        raise ValueError(f"rotary_dim must be even and within head_dim {head_dim}, got {rotary_dim}")
    if inv_freq.dtype != torch.float32 or inv_freq.numel() != rotary_dim // 2:
        raise ValueError(f"inv_freq must hold rotary_dim / 2 = {rotary_dim // 2} float32 frequencies, "
                         f"got {inv_freq.numel()} of {inv_freq.dtype}")
    return inv_freq, rotary_dim, interleaved


def check_batch(kv, meta, n_rows: int, writes: bool, window: Optional[int] = None) -> None:
    """The index arithmetic of the attention and cache-write kernels, done on the host for one launch:
    raises ``ValueError`` naming the first value with which a kernel would leave its tensors.
    ``kv``: the cache entry (``k``, ``v`` pools [pages, kv heads, page_tokens, head_dim], ``block_table``
    [slots, pages per sequence]); ``meta``: the batch description; ``n_rows``: rows of the qkv tensor;
    ``writes``: the launch stores the new tokens' keys and values (they are read in any case);
    ``window``: keys older than that may have given their pages back (cell -1).  Plain torch on whatever device the tensors live on."""
    b = int(meta.n_seqs)
    table = kv.block_table
    n_slots, max_pages = table.shape
    n_pages, page = int(kv.k.shape[0]), int(kv.page_tokens)
    slot = meta.slot_ids[:b].to(torch.int64).cpu()
    start = meta.q_start[:b + 1].to(torch.int64).cpu()
    base = meta.base_len[:b].to(torch.int64).cpu()
    for name, t in (("slot_ids", meta.slot_ids), ("q_start", meta.q_start), ("base_len", meta.base_len),
                    ("block_table", table)):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise ValueError(f"{name} must be a contiguous int32 tensor, got {t.dtype}")
    bad = ((slot < 0) | (slot >= n_slots)).nonzero()
    if len(bad):
        i = int(bad[0])
        raise ValueError(f"slot_ids[{i}] = {int(slot[i])} is no row of the block table ({n_slots} slots)")
    q_len = start[1:] - start[:-1]
    if int(start[0]) < 0 or bool((q_len <= 0).any()) or int(start[-1]) > n_rows:
        raise ValueError(f"q_start {start.tolist()} does not cut the {n_rows} rows into non-empty runs")
    if int(q_len.max()) > meta.max_q_len:
        raise ValueError(f"a sequence brings {int(q_len.max())} tokens, the launch is sized for max_q_len = {meta.max_q_len}")
    end = base + q_len
    if bool((base < 0).any()) or int(end.max()) > max_pages * page:
        i = int(((base < 0) | (end > max_pages * page)).nonzero()[0])
        raise ValueError(f"sequence {i}: keys {int(base[i])} + {int(q_len[i])} do not fit the block table's "
                         f"{max_pages} pages of {page} tokens")
    if int(end.max()) > meta.max_kv_len:
        raise ValueError(f"a sequence holds {int(end.max())} keys, the launch is sized for max_kv_len = {meta.max_kv_len}")
    rows = table.to(torch.int64).cpu()
    for i in range(b):
        used = rows[int(slot[i]), :-(-int(end[i]) // page)]
        first_seen = 0 if window is None else max(0, int(base[i]) - window + 1) // page
        if bool((used >= n_pages).any()) or bool((used < -1).any()):
            j = int(((used >= n_pages) | (used < -1)).nonzero()[0])
            raise ValueError(f"block_table[{int(slot[i])}, {j}] = {int(used[j])} is no page of the pool ({n_pages} pages)")
        held = used[first_seen:]              # every page a query of this launch reads, or a new token is stored in
        if bool((held < 0).any()):
            j = first_seen + int((held < 0).nonzero()[0])
            raise ValueError(f"sequence {i} (slot {int(slot[i])}) holds no page for keys {j * page}..{(j + 1) * page - 1} "
                             f"(block_table[{int(slot[i])}, {j}] = {int(used[j])})")


def _check_if_asked(options: KernelOptions, kv, meta, n_rows: int, writes: bool, window: Optional[int] = None) -> None:
    if options.check_arguments and not (kv.k.is_cuda and torch.cuda.is_current_stream_capturing()):
        check_batch(kv, meta, n_rows, writes, window)


def rope_kv_write(qkv: torch.Tensor, rotary, kv, meta, n_heads: int, n_kv_heads: int,
                  head_dim: int, write_kv: bool = True, options: KernelOptions = DEFAULT) -> None:
    """Rotates the q (in place) and k heads of the fused ``qkv`` rows by their
    positions and writes k and v into the pages of ``kv`` (a cache entry).  ``rotary``: see
    ``rotary_layout``; every layout it describes is taken."""
    inv_freq, rotary_dim, interleaved = rotary_layout(rotary, head_dim)
    _need_cuda(qkv, inv_freq, kv.k)
    n = qkv.shape[0]
    assert qkv.is_contiguous() and qkv.shape[1] == (n_heads + 2 * n_kv_heads) * head_dim
    assert qkv.dtype == kv.k.dtype and n == meta.n_tokens
    assert kv.k.shape[1:] == (n_kv_heads, kv.page_tokens, head_dim) and kv.v.shape == kv.k.shape, \
        "the attention kernels take keys and values of one width"
    _check_if_asked(options, kv, meta, n, write_kv)
    _launch("elementwise", "siar_rope_kv_write", _is_bf16(qkv.dtype), _ptr(qkv), _ptr(inv_freq), _ptr(kv.k),
            _ptr(kv.v), _ptr(kv.block_table), _ptr(meta.slot_ids), _ptr(meta.q_start), _ptr(meta.base_len), n,
            meta.n_seqs, n_heads, n_kv_heads, head_dim, kv.page_tokens, kv.block_table.shape[1],
            kv.k.shape[0], int(write_kv), _ptr(status_word(qkv.device)), _stream(), rotary_dim, int(interleaved))


_attn_consts = {}


def attention_limits() -> dict:
    if not _attn_consts:
        lib = build.load_unit("attention")
        _attn_consts["decode_chunk"] = lib.siar_attn_decode_chunk()
        _attn_consts["max_head_dim"] = lib.siar_attn_max_head_dim()
    return _attn_consts


def check_attention_sizes(n_heads: int, n_kv_heads: int, head_dim: int) -> None:
    """Raises for sizes the attention kernels refuse (never a wrong result)."""
    if head_dim % 16 or head_dim <= 0 or head_dim > 256:
        raise ValueError(f"attention kernels take head_dim in steps of 16 up to 256, got {head_dim}")
    if n_heads % n_kv_heads:
        raise ValueError(f"num heads {n_heads} is not a multiple of kv heads {n_kv_heads}")


_counters = {}
_sms = {}


def _sm_count(device) -> int:
    dev = torch.device(device)
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    if key not in _sms:
        _sms[key] = torch.cuda.get_device_properties(dev).multi_processor_count
    return _sms[key]


def _decode_counters(device, need: int) -> torch.Tensor:
    """Zeroed int32 counters the split decode attention uses to find the block that
    finishes last; the kernel leaves them zero.  Allocated once per device."""
    dev = torch.device(device)
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    t = _counters.get(key)
    if t is None or t.numel() < need:
        t = torch.zeros(max(need, 1 << 16), dtype=torch.int32, device=dev)
        _counters[key] = t
    return t


def set_programmatic_launch(on: bool) -> None:
    """Turns programmatic dependent launch on or off for every loaded and future unit
    (off = plain stream order between kernels; results are the same either way)."""
    global _pdl
    _pdl = bool(on)
    for unit in build.available_units():
        lib = build.load_unit(unit)
        if hasattr(lib, "siar_set_pdl"):
            lib.siar_set_pdl(int(_pdl))


_pdl = True


def mma_attention_takes(dtype: torch.dtype, n_heads: int, n_kv_heads: int, head_dim: int, page_tokens: int,
                        options: KernelOptions = DEFAULT) -> bool:
    if dtype != torch.bfloat16 or not options.use_mma_attention:
        return False
    return bool(_fn("attention_mma", "siar_attn_mma_supported")(n_heads, n_kv_heads, head_dim, page_tokens))


def decode_scratch_floats(n_seqs: int, n_heads: int, head_dim: int, max_kv_len: int, chunk: int) -> int:
    chunks = (max_kv_len + chunk - 1) // chunk
    return n_seqs * n_heads * chunks * (head_dim + 2)


def decode_fuses_rope(meta, dtype: torch.dtype, n_heads: int, n_kv_heads: int, head_dim: int, page_tokens: int,
                      options: KernelOptions = DEFAULT) -> bool:
    """True when ``rope_and_attention`` runs one kernel for this step (one token per sequence
    on the tensor-core path); otherwise it is ``rope_kv_write`` followed by ``attention``."""
    return bool(meta.is_decode) and options.fuse_decode_rope and mma_attention_takes(
        dtype, n_heads, n_kv_heads, head_dim, page_tokens, options)


def rope_and_attention(qkv: torch.Tensor, rotary, kv, meta, n_heads: int, n_kv_heads: int,
                       head_dim: int, scale: float, write_kv: bool = True, window: Optional[int] = None,
                       options: KernelOptions = DEFAULT) -> torch.Tensor:
    """Rotates q and k by the tokens' positions, writes k and v to the cache entry and attends:
    what a rotary attention mixer does between its two products.  For steps of one token per
    sequence on the tensor-core path this is ONE kernel (q is rotated in registers, the new k and
    v go to the cache and are used from shared memory); otherwise two.  The one kernel rotates whole
    heads in pairs (i, i + head_dim/2) only: any other rotary layout (see ``rotary_layout``) takes the
    two-kernel way.  ``window``: see ``attention``."""
    inv_freq, rotary_dim, interleaved = rotary_layout(rotary, head_dim)
    plain_layout = inv_freq is None or (rotary_dim == head_dim and not interleaved)
    if window is not None or not plain_layout or not decode_fuses_rope(meta, qkv.dtype, n_heads, n_kv_heads, head_dim,
                                                                       kv.page_tokens, options):
        rope_kv_write(qkv, rotary, kv, meta, n_heads, n_kv_heads, head_dim, write_kv=write_kv, options=options)
        return attention(qkv, kv, meta, n_heads, n_kv_heads, head_dim, scale, window=window, options=options)
    _need_cuda(qkv, kv.k, inv_freq)
    check_attention_sizes(n_heads, n_kv_heads, head_dim)
    assert qkv.is_contiguous() and qkv.shape == (meta.n_seqs, (n_heads + 2 * n_kv_heads) * head_dim)
    _check_if_asked(options, kv, meta, qkv.shape[0], write_kv)
    out = torch.empty((meta.n_seqs, n_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    sms = _sm_count(qkv.device)
    f = _fn("attention_mma", "siar_attn_mma_decode_scratch_floats")
    f.restype = c_longlong
    scratch = torch.empty(f(meta.n_seqs, n_heads, n_kv_heads, head_dim, meta.max_kv_len, sms), dtype=torch.float32,
                          device=qkv.device)
    _launch("attention_mma", "siar_attn_mma_decode_rope", _ptr(qkv), _ptr(kv.k), _ptr(kv.v), _ptr(kv.block_table),
            _ptr(meta.slot_ids), _ptr(meta.q_start), _ptr(meta.base_len), _ptr(out), _ptr(scratch),
            _ptr(_decode_counters(qkv.device, meta.n_seqs * n_kv_heads)), _ptr(inv_freq), int(write_kv), meta.n_seqs,
            n_heads, n_kv_heads, head_dim, kv.page_tokens, kv.block_table.shape[1], meta.max_kv_len, sms, float(scale),
            _stream(), _ptr(status_word(qkv.device)), rotary_dim, int(interleaved))
    return out


def attention(qkv: torch.Tensor, kv, meta, n_heads: int, n_kv_heads: int, head_dim: int, scale: float,
              window: Optional[int] = None, options: KernelOptions = DEFAULT) -> torch.Tensor:
    """Causal attention of the new tokens' (already rotated) queries over the
    cache entry ``kv``; returns [N, n_heads * head_dim] in qkv's dtype.  bfloat16
    with head_dim 64 or 128 runs on the tensor cores, everything else on the CUDA cores.
    ``window`` = w: a query at position p sees keys p - w + 1 .. p only (CUDA-core kernels)."""
    if window is not None and window <= 0:
        raise ValueError(f"an attention window must be positive, got {window}")
    _need_cuda(qkv, kv.k)
    check_attention_sizes(n_heads, n_kv_heads, head_dim)
    n = qkv.shape[0]
    _check_if_asked(options, kv, meta, n, False, window)
    out = torch.empty((n, n_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    common = (_ptr(kv.block_table), _ptr(meta.slot_ids), _ptr(meta.q_start), _ptr(meta.base_len))
    sizes = (meta.n_seqs, n_heads, n_kv_heads, head_dim, kv.page_tokens, kv.block_table.shape[1])
    mma = window is None and mma_attention_takes(qkv.dtype, n_heads, n_kv_heads, head_dim, kv.page_tokens, options)
    win = int(window or 0)
    if meta.is_decode:
        if mma:
            sms = _sm_count(qkv.device)
            f = _fn("attention_mma", "siar_attn_mma_decode_scratch_floats")
            f.restype = c_longlong
            scratch = torch.empty(f(meta.n_seqs, n_heads, n_kv_heads, head_dim, meta.max_kv_len, sms),
                                  dtype=torch.float32, device=qkv.device)
            _launch("attention_mma", "siar_attn_mma_decode", _ptr(qkv), _ptr(kv.k), _ptr(kv.v), *common, _ptr(out),
                    _ptr(scratch), _ptr(_decode_counters(qkv.device, meta.n_seqs * n_kv_heads)), *sizes,
                    meta.max_kv_len, sms, float(scale), _stream(), _ptr(status_word(qkv.device)))
        else:
            chunk = attention_limits()["decode_chunk"]
            scratch = torch.empty(decode_scratch_floats(meta.n_seqs, n_heads, head_dim, meta.max_kv_len, chunk),
                                  dtype=torch.float32, device=qkv.device)
            _launch("attention", "siar_attn_decode", _is_bf16(qkv.dtype), _ptr(qkv), _ptr(kv.k), _ptr(kv.v), *common,
                    _ptr(out), _ptr(scratch), *sizes, meta.max_kv_len, win, float(scale), _stream(),
                    _ptr(status_word(qkv.device)), kernels=2)
    elif window is None and tc_attention_takes(qkv.dtype, n_heads, n_kv_heads, head_dim, kv.page_tokens, options):
        _launch("attention_tc", "siar_attn_tc_prefill", _ptr(qkv), _ptr(kv.k), _ptr(kv.v), *common, _ptr(out), n,
                *sizes, kv.k.shape[0], meta.max_q_len, float(scale), _ptr(status_word(qkv.device)), _stream())
    elif mma:
        _launch("attention_mma", "siar_attn_mma_prefill", _ptr(qkv), _ptr(kv.k), _ptr(kv.v), *common, _ptr(out),
                *sizes, meta.max_q_len, float(scale), _stream(), _ptr(status_word(qkv.device)))
    else:
        _launch("attention", "siar_attn_prefill", _is_bf16(qkv.dtype), _ptr(qkv), _ptr(kv.k), _ptr(kv.v), *common,
                _ptr(out), *sizes, meta.max_q_len, win, float(scale), _stream(), _ptr(status_word(qkv.device)))
    return out


def swiglu(gate_up: torch.Tensor, interleaved: bool = False) -> torch.Tensor:
    """silu(gate) * up.  Rows are laid out as [gate (I) | up (I)], or with ``interleaved`` as
    (gate_0, up_0, gate_1, up_1, ...)."""
    _need_cuda(gate_up)
    assert gate_up.dim() == 2 and gate_up.shape[1] % 2 == 0 and gate_up.is_contiguous()
    n, two_i = gate_up.shape
    out = torch.empty((n, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    _launch("elementwise", "siar_swiglu", _is_bf16(gate_up.dtype), _ptr(gate_up), _ptr(out), n, two_i // 2,
            int(interleaved), _stream())
    return out


def linear_swiglu(x: torch.Tensor, w_interleaved: torch.Tensor, options: KernelOptions = DEFAULT) -> torch.Tensor:
    """silu(x @ Wg^T) * (x @ Wu^T) for a weight whose rows alternate (gate_0, up_0, gate_1, ...);
    returns [M, N/2] in x's dtype.  On the bfloat16 path the activation runs in the product's
    epilogue on the float32 accumulators; otherwise it is a product followed by ``swiglu``.
    ``x`` may be a ``NormedResidual``."""
    if isinstance(x, NormedResidual):
        out = torch.empty((x.shape[0], w_interleaved.shape[0] // 2), dtype=x.dtype, device=w_interleaved.device)
        if w_interleaved.shape[0] % 2 == 0 and _fused_input(x, w_interleaved, out, 1, options):
            return out
        x = x.materialize()
    _need_cuda(x, w_interleaved)
    assert x.dim() == 2 and w_interleaved.dim() == 2 and x.shape[1] == w_interleaved.shape[1]
    assert w_interleaved.shape[0] % 2 == 0 and x.dtype == w_interleaved.dtype
    if x.dtype == torch.bfloat16:
        from . import gemm_tc
        out = torch.empty((x.shape[0], w_interleaved.shape[0] // 2), dtype=x.dtype, device=x.device)
        if gemm_tc.try_linear(x, w_interleaved, out, epilogue=1, options=options):
            return out
    return swiglu(linear(x, w_interleaved, x.dtype, options=options), interleaved=True)


def advance_lengths(base_len: torch.Tensor, q_start: torch.Tensor, n_seqs: int) -> None:
    _need_cuda(base_len, q_start)
    _launch("elementwise", "siar_advance_lengths", _ptr(base_len), _ptr(q_start), n_seqs, _stream())


def set_table_cells(table: torch.Tensor, cells: torch.Tensor) -> None:
    """``table[r, c] = v`` for every (r, c, v) row of the int32 tensor ``cells`` [n, 3] (both on the GPU)."""
    _need_cuda(table, cells)
    assert table.dtype == torch.int32 and table.dim() == 2 and table.is_contiguous()
    assert cells.dtype == torch.int32 and cells.dim() == 2 and cells.shape[1] == 3 and cells.is_contiguous()
    _launch("elementwise", "siar_set_table_cells", _ptr(table), _ptr(cells), cells.shape[0], table.shape[0],
            table.shape[1], _stream())


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           seeds: torch.Tensor, draw_index: torch.Tensor, advance_index: bool = False,
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token id per row of float32 ``logits`` [R, V]; per-row options are
    device arrays (temperature f32, top_k i32, top_p f32, seeds i64, draw_index i32)."""
    _need_cuda(logits, temperature, top_k, top_p, seeds, draw_index)
    assert logits.dtype == torch.float32 and logits.dim() == 2 and logits.is_contiguous()
    r, v = logits.shape
    assert temperature.dtype == torch.float32 and top_p.dtype == torch.float32
    assert top_k.dtype == torch.int32 and draw_index.dtype == torch.int32 and seeds.dtype == torch.int64
    for t in (temperature, top_k, top_p, seeds, draw_index):
        assert t.numel() >= r
    if out is None:
        out = torch.empty(r, dtype=torch.int32, device=logits.device)
    _launch("sampling", "siar_sample", _ptr(logits), r, v, _ptr(temperature), _ptr(top_k), _ptr(top_p),
            _ptr(seeds), _ptr(draw_index), int(advance_index), _ptr(out), _stream())
    return out
