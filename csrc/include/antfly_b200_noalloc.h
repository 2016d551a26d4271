/* Allocation-free entry point of libafb_cuda.so.
 *
 * This entry point has no counterpart in the reference project; it exists for callers of this library that are
 * not allowed to allocate device memory at the moment they need a kernel: code running inside a memory pool that
 * is already sized to the byte (a serving process that gave all of HBM to weights and KV cache), a host thread
 * that must not take the allocator's locks or trigger an implicit synchronisation (cudaMalloc / cudaFree can
 * synchronise the device), or an embedding host (C, Rust, Go through cgo) that links the shared object directly
 * and has no tensor allocator to hand scratch buffers from.
 *
 * It runs the same split-KV paged decode attention as afb_attention(..., paged = 1, split_keys = 1,
 * num_splits > 1, ...): every (sequence, KV head) pair is processed by `num_splits` CTAs that each cover a slice of
 * the keys and write an un-normalised partial output plus its log-sum-exp, and a second kernel merges the slices.
 * The partial outputs live in a scratch array that is part of the library image instead of a buffer supplied by
 * the caller:
 *
 *   - The scratch is a file-scope `static __device__` array of AFB_NOALLOC_SCRATCH_BYTES (4 MiB + 32 KiB).  Every
 *     GPU that loads the library holds that much memory for it until the process exits.
 *   - A call with num_splits > 1 is rejected (return value -1, message through afb_last_error()) when
 *     num_splits * T * Hq * (D + 1) * 4 bytes exceed the array, i.e. when num_splits * T * Hq > 8192 for D = 128.
 *     A call with num_splits = 1 writes `out` directly, uses no scratch and has no such limit.
 *   - The first call on each device looks up the device address of the array (cudaGetSymbolAddress, with that
 *     device current) and remembers it.  Make that first call outside of any stream capture.  Two host threads
 *     that make the first call on a device at the same moment both do the lookup and store the same value; the
 *     table is filled without a lock and that is harmless.
 *   - The entry point itself calls no cudaMalloc / cudaFree and no allocating library routine.  The array is part
 *     of the library's device image, though, and with lazy module loading (the CUDA default) the driver places
 *     that image on a device when the library's first kernel or symbol is used there: the array's 4 MiB + 32 KiB
 *     are taken from the device at THAT moment.  A process that sizes its own pool to the last byte should make
 *     one warm-up call per device (any small valid call) before it commits the pool.
 *   - All calls on a device share the one array, and it keeps the previous call's contents.  Nothing in it has to
 *     start at zero: the split kernels write the partial rows of every token that belongs to a sequence before
 *     the merge reads them.  Rows of `out` for token slots that belong to NO sequence (a padded batch, T larger
 *     than the sum of q_lens) are unspecified: the merge fills them from whatever earlier calls left in the
 *     array (a caller that indexes `out` through q_starts / q_lens never reads them).  Two calls
 *     whose kernels overlap on the GPU (different streams, no dependency between them) race on the array;
 *     serialise them.
 *
 * Inputs and outputs are the caller's, exactly as for afb_attention: q [T, Hq, D] bf16 with token pitch q_stride
 * elements, k_cache / v_cache [num_blocks, page, Hkv, D] bf16, block_tables [B, max_blocks] int32, q_starts /
 * q_lens / kv_lens [B] int32, out [T, Hq, D] bf16 with token pitch out_stride.  q_len * (Hq / Hkv) must be <= 16
 * for every sequence (decode, or a short speculative verify).  Returns 0 on success.
 */
#ifndef ANTFLY_B200_NOALLOC_H
#define ANTFLY_B200_NOALLOC_H

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AFB_NOALLOC_SCRATCH_BYTES (4 * 1024 * 1024 + 32 * 1024)

int afb_paged_decode_attention_noalloc(const void* q, long q_stride, const void* k_cache, const void* v_cache,
                                       const int* block_tables, int max_blocks, int page, const int* q_starts,
                                       const int* q_lens, const int* kv_lens, void* out, long out_stride, int B,
                                       int T, int Hq, int Hkv, int D, int max_q_len, int window, float scale,
                                       int num_splits, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif
