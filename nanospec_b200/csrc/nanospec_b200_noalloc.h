/* nanospec_b200_noalloc.h - decode attention for callers that must not allocate.
 *
 * This entry point has no counterpart in the reference (ved1beta/nanospec ships no native
 * code); it is an addition of this library.
 *
 * Who it is for.  ns_attention_decode() needs scratch memory in which the blocks that share
 * one request's keys leave their partial results, and it expects the caller to pass that
 * memory in.  Some callers have nowhere to get it from: a host that handed the whole device
 * to another allocator before this library was loaded, a plug-in called from inside a
 * framework's execution callback where allocation is forbidden, or a latency-bound loop that
 * cannot afford the device-wide synchronisation that cudaMalloc and cudaFree imply.  For them
 * ns_attention_decode_noalloc() does the same work with its scratch in a fixed array that is
 * part of the library image.  It calls no cudaMalloc, cudaFree or any allocating library routine.
 *
 * What to know before using it.
 *  - The array is NS_NOALLOC_SCRATCH_BYTES (8 MiB) of device memory on EVERY GPU on which the
 *    library is loaded, held until the process exits, whether or not this function is called.
 *  - Problem sizes whose scratch does not fit are refused with NS_ERR_UNSUPPORTED and a message
 *    (ns_last_error()) that states the bytes needed and the limit.  The need is
 *        4 * n_tokens * nq * n_splits * (head_dim + 2)  bytes for the partial results
 *      + 4 * n_tokens * nkv * ceil((nq / nkv) / 16)     bytes for the arrival counters,
 *    each part rounded up to 256 bytes.  With n_splits == 1 nothing is shared between blocks, the array is
 *    not touched and no size is refused.  Arguments that ns_attention_decode() would refuse are refused here
 *    before anything is put on the stream.
 *  - The first call on a device looks up the array's device address (cudaGetSymbolAddress) with
 *    that device current.  Make that first call at start-up, before any stream capture begins.
 *  - All calls on a device share the one array and it keeps the previous call's contents.  The
 *    function clears the counters it depends on at the start of every call (an asynchronous memset
 *    on `stream`); the partial results need no clearing.  Two calls whose kernels can overlap on
 *    the GPU (different streams without an ordering between them) race on the array and give
 *    wrong results: order such calls yourself.
 *  - Inputs, outputs, meaning of the arguments and numerical results are those of
 *    ns_attention_decode(); only part_o, part_ml and counters are gone from the argument list.
 */
#ifndef NANOSPEC_B200_NOALLOC_H
#define NANOSPEC_B200_NOALLOC_H

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NS_NOALLOC_SCRATCH_BYTES (8u * 1024u * 1024u)

/* Returns 0 on success, a non-zero NsStatus otherwise (text from ns_last_error()).
 * q, k_cache, v_cache, out: bfloat16 device memory; block_table, token_req, positions, qo_indptr,
 * rows: int32 device memory (`rows` may be NULL: then the tokens are 0 .. n_tokens-1). */
int ns_attention_decode_noalloc(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                                const int* block_table, int table_stride, const int* token_req, const int* positions,
                                const int* qo_indptr, void* out, int o_stride, const int* rows, int n_tokens, int nq,
                                int nkv, int head_dim, int page_size, float scale, int window, int n_splits,
                                cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif
