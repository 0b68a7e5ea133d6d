"""The decode-attention entry point that allocates nothing (csrc/no_alloc.h), called
through its exported C symbol the way a caller without an allocator would: this test
allocates inputs and the output, the entry point brings its own scratch.

Some users of these kernels cannot call cudaMalloc where they call the kernels (a host
application that owns all device memory, a loop in which allocation is forbidden).  For
them the entry point keeps the scratch of the split decode attention in an array inside
the shared object.  Checked here: its output equals the ordinary entry point's (which
gets scratch from torch) on two calls in a row, with different batches, so that the
second call meets what the first one left in the shared array; and sizes beyond the
array are refused with a message.

The file sorts last on purpose: it runs after every other test (and also passes alone).
"""

import ctypes
import math

import pytest
import torch

from simple_inference_autoresearch_b200.cache import SequenceCache
from simple_inference_autoresearch_b200.engine.batch import BatchMeta, StepEntry
from simple_inference_autoresearch_b200.kernels import build, ops
from simple_inference_autoresearch_b200.parts.base import KVNeed

pytestmark = pytest.mark.gpu
DEV = "cuda"


def entry_point():
    lib = build.load_unit("attention_mma")
    f = lib.siar_attn_mma_decode_noalloc
    c = ctypes
    f.argtypes = [c.c_void_p] * 8 + [c.c_int] * 8 + [c.c_float, c.c_void_p, c.c_char_p, c.c_int]
    f.restype = c.c_int
    lib.siar_attn_mma_noalloc_max_floats.restype = c.c_longlong
    return lib, f


def make_case(lens, hq, hkv, d, seed):
    """A cache with sequences of the given lengths plus one new token each, filled through the
    library's own rotary/cache-write kernel; returns (qkv of the new tokens, cache entry, meta)."""
    g = torch.Generator().manual_seed(seed)
    b = len(lens)
    cache = SequenceCache([KVNeed(hkv, d)], sum(-(-(n + 1) // 64) * 64 for n in lens), b, max(lens) + 64,
                          torch.bfloat16, DEV)
    slots = [cache.alloc() for _ in lens]
    width = (hq + 2 * hkv) * d
    hist = torch.randn(sum(lens), width, generator=g).to(torch.bfloat16).to(DEV)
    cache.reserve(slots, lens)
    ops.rope_kv_write(hist, None, cache.entry(0), BatchMeta.build([StepEntry(s, [0] * n) for s, n in zip(slots, lens)],
                                                                  [0] * b, DEV), hq, hkv, d)
    cache.commit(slots, lens)
    cache.reserve(slots, [1] * b)
    new = torch.randn(b, width, generator=g).to(torch.bfloat16).to(DEV)
    meta = BatchMeta.build([StepEntry(s, [0]) for s in slots], lens, DEV)
    ops.rope_kv_write(new, None, cache.entry(0), meta, hq, hkv, d)
    return new, cache, meta


def call_noalloc(f, qkv, kv, meta, hq, hkv, d, out):
    msg = ctypes.create_string_buffer(256)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    rc = f(qkv.data_ptr(), kv.k.data_ptr(), kv.v.data_ptr(), kv.block_table.data_ptr(), meta.slot_ids.data_ptr(),
           meta.q_start.data_ptr(), meta.base_len.data_ptr(), out.data_ptr(), meta.n_seqs, hq, hkv, d,
           kv.page_tokens, kv.block_table.shape[1], meta.max_kv_len, sms, 1.0 / math.sqrt(d),
           torch.cuda.current_stream().cuda_stream, msg, len(msg))
    return rc, msg.value.decode()


def test_no_alloc_entry_matches_the_ordinary_one_on_two_calls_in_a_row():
    _, f = entry_point()
    hq, hkv, d = 8, 2, 128
    for seed, lens in ((1, [700, 130, 5, 1000]), (2, [257, 900])):       # second call: other shapes, same array
        qkv, cache, meta = make_case(lens, hq, hkv, d, seed)
        want = ops.attention(qkv, cache.entry(0), meta, hq, hkv, d, 1.0 / math.sqrt(d))
        got = torch.full_like(want, float("nan"))
        before = torch.cuda.memory_allocated()
        rc, msg = call_noalloc(f, qkv, cache.entry(0), meta, hq, hkv, d, got)
        assert rc == 0, msg
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert not torch.isnan(got.float()).any()
        torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=2e-2)   # the kernel tests' bf16 tolerance
        assert torch.equal(got, want)           # same kernel, same chunking: the same numbers
    ops.check_status(DEV)


def test_no_alloc_entry_refuses_what_does_not_fit():
    """Refusals happen on the host before anything is launched, so the (small) buffers passed
    here are never touched."""
    lib, f = entry_point()
    hq, hkv, d = 32, 8, 128
    qkv, cache, meta = make_case([300], hq, hkv, d, 3)
    out = torch.zeros(1, hq * d, dtype=torch.bfloat16, device=DEV)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    need = lib.siar_attn_mma_decode_scratch_floats
    need.restype = ctypes.c_longlong
    limit = lib.siar_attn_mma_noalloc_max_floats()
    meta.n_seqs, meta.max_kv_len = 256, 4096          # 256 sequences: more partials than the array holds
    assert need(256, hq, hkv, d, 4096, sms) > limit
    rc, msg = call_noalloc(f, qkv, cache.entry(0), meta, hq, hkv, d, out)
    assert rc == -3 and "floats of scratch" in msg and str(limit) in msg, (rc, msg)
    # more (sequence, kv head) pairs than counters, with partials that would fit: 1,024 sequences of
    # 8 kv heads, one chunk each
    meta.n_seqs, meta.max_kv_len = 1024, 128
    assert need(1024, 8, 8, 64, 128, sms) <= limit
    rc, msg = call_noalloc(f, qkv, cache.entry(0), meta, 8, 8, 64, out)
    assert rc == -3 and "pairs" in msg and "8192" in msg, (rc, msg)
    meta.n_seqs, meta.max_kv_len = 1, 301
    rc, msg = call_noalloc(f, qkv, cache.entry(0), meta, hq, hkv, 48, out)     # a head size the kernel does not take
    assert rc == -2 and "head_dim 48" in msg, (rc, msg)
