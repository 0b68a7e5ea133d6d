/* Decode attention for callers that must not allocate device memory.
 *
 * This entry point has no counterpart in the reference project.  It exists for
 * programs that drive the kernels from a context in which cudaMalloc is not
 * available to them: code that runs inside a region where allocation is forbidden
 * (a real-time loop, a host that pre-sizes all of its memory and forbids growth, a
 * plugin whose host application owns the allocator), or a runtime that hands the
 * library nothing but finished input and output buffers.  The library's ordinary
 * decode attention, siar_attn_mma_decode, needs two pieces of scratch from its
 * caller (float partial results per chunk of keys, and a few zeroed counters); this
 * variant keeps that scratch in one array that is part of the shared object itself.
 *
 *   int siar_attn_mma_decode_noalloc(qkv, k_pool, v_pool, block_table, slot_ids,
 *                                    q_start, base_len, out,
 *                                    B, Hq, Hkv, D, page_tokens, max_pages,
 *                                    max_kv_len, sm_count, scale, stream,
 *                                    message, message_len)
 *
 * The arguments are those of siar_attn_mma_decode without `scratch` and `counters`
 * (bfloat16 fused qkv rows of one new token per sequence, the paged key and value
 * pools, the batch description, the bfloat16 output [B, Hq * D]); inputs and the
 * output are still the caller's.  Returns 0 after launching on `stream`, otherwise a
 * non-zero code with a sentence in `message` (when message_len > 0):
 *   -2  sizes the kernel does not take (see siar_attn_mma_supported)
 *   -3  the sizes need more scratch than the built-in array holds
 *   >0  a cudaError_t from set-up or launch
 *
 * Limits.  The array is SIAR_NOALLOC_SCRATCH_BYTES (4 MiB) per GPU: every device
 * on which this library is loaded holds it from load until the process exits,
 * whether the entry point is used or not.  A call fits when
 *   B * Hkv <= SIAR_NOALLOC_MAX_PAIRS  and
 *   siar_attn_mma_decode_scratch_floats(B, Hq, Hkv, D, max_kv_len, sm_count)
 *       <= siar_attn_mma_noalloc_max_floats().
 * (Llama-3.1-8B heads: batch 8 up to 16k keys, batch 64 up to 4k keys.)
 *
 * Set-up.  The first call on a device, made with that device current, looks up the
 * array's device address once (cudaGetSymbolAddress) and remembers it; make that
 * first call outside any stream capture.  Nothing is ever allocated or freed: no
 * cudaMalloc, no cudaFree, no library routine that allocates.
 *
 * Sharing.  All calls on a device use the same array, and it keeps what the last
 * call left in it.  The counters it holds are cleared on `stream` before every
 * launch; the partial results need no clearing (every value read was written by the
 * same call).  Two calls whose work overlaps on the GPU (different streams, or one
 * stream with programmatic overlap and no dependency) would race on the array: run
 * calls that share a device one after the other.
 *
 * Pages.  Every key position up to base_len[b] must have a page in the block table.
 * A cell below zero (a page the sequence does not hold) is read as page 0, so the
 * call touches no address outside the pools, but its result is then meaningless and,
 * unlike the ordinary entry point, this one has no status word to say so.
 */
#ifndef SIAR_NO_ALLOC_H
#define SIAR_NO_ALLOC_H

#define SIAR_NOALLOC_SCRATCH_BYTES (4 * 1024 * 1024)
#define SIAR_NOALLOC_MAX_PAIRS 4096 /* (sequence, kv head) pairs, one counter each */

#ifdef __cplusplus
extern "C" {
#endif

int siar_attn_mma_decode_noalloc(const void* qkv, const void* k_pool, const void* v_pool, const int* block_table,
                                 const int* slot_ids, const int* q_start, const int* base_len, void* out, int B,
                                 int Hq, int Hkv, int D, int page_tokens, int max_pages, int max_kv_len,
                                 int sm_count, float scale, void* stream, char* message, int message_len);

/* Float elements of the array that are available for partial results. */
long long siar_attn_mma_noalloc_max_floats(void);

#ifdef __cplusplus
}
#endif

#endif
