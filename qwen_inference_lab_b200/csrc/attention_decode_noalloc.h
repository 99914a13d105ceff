/* Single-token paged attention for callers that cannot allocate device memory.
 *
 * This entry point has no counterpart in the reference (provoke210/qwen-inference-lab):
 * it exists for users of this library, not for parity.
 *
 * Who it is for.  The regular entry point, qil_attn_decode, takes two scratch
 * buffers that its caller allocates.  Some callers have nowhere to get them:
 * a host program that gave all device memory to its own pool at start-up and
 * forbids cudaMalloc afterwards, or a loop that may not stall (cudaMalloc and
 * cudaFree can synchronise the whole device).  Those callers use this function:
 * it keeps its scratch in a fixed array inside the library.
 *
 * What it does.  The same computation as qil_attn_decode, with the same kernels
 * and the same arguments minus the two scratch pointers: attention of n_decode
 * single tokens over their requests' paged keys and values (bfloat16, head size
 * fixed when the library was compiled).  q, kv, out and the int arrays are the
 * caller's; decode_info holds four ints per token (its row in q and out, its
 * absolute position, its row of the block table, 0); span_len is the number of
 * key positions one block covers (a multiple of 64) and n_spans * span_len must
 * reach the longest context; a token whose position lies beyond n_spans * span_len
 * gets a row of NaN, not a softmax over a shortened context.
 *
 * Limits and rules.
 *  - The scratch array holds qil_attn_decode_noalloc_max_floats() floats (16 MiB;
 *    every GPU that loads the library holds that much until the process exits).
 *    A call needs  n_decode * n_q_heads * n_spans * (head_dim + 2)  floats, rounded up
 *    to a multiple of 64; a call that needs more returns -1 and qil_last_error()
 *    says by how much.  Nothing is launched in that case.
 *    A call also uses one counter per (token, kv head, 16 query heads of that kv head) from
 *    a second fixed array of 65536 counters; more than that is refused the same way.
 *  - It calls no cudaMalloc, cudaFree or any routine that allocates.
 *  - The first call on each device looks up the array's device address and sets
 *    a kernel attribute; make that first call outside any stream capture, with
 *    the device it is meant for current.  That attribute (the kernel's shared-memory
 *    limit) is shared with qil_attn_decode of the same library and only ever raised,
 *    so the two may be called in any order.
 *  - Host threads: the per-device set-up and the error text are plain statics.  Call
 *    this function (and the other entry points of the library) from one host thread
 *    at a time per device, or put your own lock around them.
 *  - All calls share the one array, and it keeps what the last call left in it.
 *    Nothing in it has to start at zero: every slot a call reads, that call wrote
 *    first.  The counters must start at zero: each call clears the ones it uses on the
 *    stream before its kernel runs.  Two calls whose kernels overlap on the GPU (different streams, no
 *    ordering between them) race on the array; order them.
 *
 * Returns 0 when the kernels were queued on `stream`, a positive cudaError_t if a
 * CUDA call failed, -1 if the arguments were refused.
 */
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

int qil_attn_decode_noalloc(const void* q, const void* kv, void* out, const int* decode_info, int n_decode,
                            int n_spans, int span_len, const int* block_table, int table_stride,
                            int n_q_heads, int n_kv_heads, int page_size, int num_pages, int window,
                            float scale, cudaStream_t stream);

/* Capacity of the built-in scratch array, in floats. */
long long qil_attn_decode_noalloc_max_floats(void);

#ifdef __cplusplus
}
#endif
