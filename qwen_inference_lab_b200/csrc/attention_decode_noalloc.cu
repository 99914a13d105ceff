// qil_attn_decode_noalloc: the single-token attention of attention_mma.cu with its
// scratch in a file-scope device array instead of caller-allocated buffers.
// See attention_decode_noalloc.h for who needs this and for the rules of use.
//
// The kernels are the ones of attention_mma.cu, compiled into this library too.
#include "attention_mma.cu"
#include "attention_decode_noalloc.h"

#define QIL_NOALLOC_MAX_FLOATS (4ll * 1024 * 1024)     // 16 MiB
#define QIL_NOALLOC_MAX_TICKETS (64 * 1024)            // (token, kv head, chunk of 16 query heads) triples per call
#define QIL_NOALLOC_MAX_DEVICES 64

// Partial sums of the span kernel, then their (max, sum) pairs.  In host code this name is
// only a handle for cudaGetSymbolAddress; kernels get the address that call returns.
static __device__ __align__(256) float qil_noalloc_scratch[QIL_NOALLOC_MAX_FLOATS];

// One counter per (token, kv head, chunk of query heads): the span kernel's blocks count themselves in, the
// last one merges.  They must be zero when a call starts; the kernel puts them back, and every call clears
// the ones it uses first (a memset on the stream), so a call that was cut short leaves nothing behind.
static __device__ __align__(256) unsigned qil_noalloc_tickets[QIL_NOALLOC_MAX_TICKETS];

static float* noalloc_scratch_address[QIL_NOALLOC_MAX_DEVICES];   // per device, filled by the first call
static unsigned* noalloc_tickets_address[QIL_NOALLOC_MAX_DEVICES];

extern "C" long long qil_attn_decode_noalloc_max_floats(void) { return QIL_NOALLOC_MAX_FLOATS; }

// Once per device, with that device current: the array's address.  The span kernel's shared-memory
// limit is kept by ensure_decode_smem, which the regular entry points use too, so whichever of them
// runs first or last the limit only grows.  Neither call allocates.
static int noalloc_setup(int smem, float** scratch, unsigned** tickets) {
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) { snprintf(qil_error_text, sizeof(qil_error_text), "cudaGetDevice: %s", cudaGetErrorString(e)); return (int)e; }
    if (device < 0 || device >= QIL_NOALLOC_MAX_DEVICES) QIL_REFUSE("attention (no allocation): device %d is out of range", device);
    if (noalloc_scratch_address[device] == nullptr) {
        float* address = nullptr;
        e = cudaGetSymbolAddress((void**)&address, qil_noalloc_scratch);
        if (e != cudaSuccess || address == nullptr) {
            snprintf(qil_error_text, sizeof(qil_error_text), "cudaGetSymbolAddress: %s", cudaGetErrorString(e));
            return e != cudaSuccess ? (int)e : -1;
        }
        unsigned* counters = nullptr;
        e = cudaGetSymbolAddress((void**)&counters, qil_noalloc_tickets);
        if (e != cudaSuccess || counters == nullptr) {
            snprintf(qil_error_text, sizeof(qil_error_text), "cudaGetSymbolAddress: %s", cudaGetErrorString(e));
            return e != cudaSuccess ? (int)e : -1;
        }
        noalloc_scratch_address[device] = address;
        noalloc_tickets_address[device] = counters;
    }
    if (ensure_decode_smem(attn_decode_span_kernel, smem)) return -1;
    *scratch = noalloc_scratch_address[device];
    *tickets = noalloc_tickets_address[device];
    return 0;
}

extern "C" int qil_attn_decode_noalloc(const void* q, const void* kv, void* out, const int* decode_info, int n_decode,
                                       int n_spans, int span_len, const int* block_table, int table_stride,
                                       int n_q_heads, int n_kv_heads, int page_size, int num_pages, int window,
                                       float scale, cudaStream_t stream) {
    if (n_decode <= 0) return 0;
    AttnParams p;
    if (fill_params(p, q, kv, out, block_table, table_stride, n_q_heads, n_kv_heads, page_size, num_pages,
                    window, scale)) return -1;
    if (check_decode_span(span_len, n_spans)) return -1;
    if (span_len <= 0) QIL_REFUSE("attention (no allocation): the span length must be positive (a multiple of %d)", KV_TILE);
    if ((uintptr_t)decode_info & 15) QIL_REFUSE("attention (no allocation): decode_info must be 16-byte aligned");
    const int chunks = (n_q_heads / n_kv_heads + 15) / 16;
    const long long slots = (long long)n_decode * n_q_heads * n_spans;
    const long long o_floats = (slots * D + 63) / 64 * 64;          // part_ml starts on a 256-byte boundary
    const long long needed = o_floats + (slots * 2 + 63) / 64 * 64;
    if (needed > QIL_NOALLOC_MAX_FLOATS)
        QIL_REFUSE("attention (no allocation): %d tokens x %d heads x %d spans need %lld floats of scratch, "
                   "the built-in array holds %lld; use qil_attn_decode with your own buffers",
                   n_decode, n_q_heads, n_spans, needed, (long long)QIL_NOALLOC_MAX_FLOATS);
    if (n_decode > 65535 || n_spans > 65535) QIL_REFUSE("attention (no allocation): grid too large");
    const long long n_tickets = (long long)n_decode * n_kv_heads * chunks;
    if (n_tickets > QIL_NOALLOC_MAX_TICKETS)
        QIL_REFUSE("attention (no allocation): %d tokens x %d kv heads need %lld ticket counters, the library holds %d",
                   n_decode, n_kv_heads, n_tickets, QIL_NOALLOC_MAX_TICKETS);
    // the largest shared memory any legal span can ask for, so that one set-up serves every later call
    const int smem_limit = decode_smem_bytes(MAX_DECODE_SPAN, 1);
    const int smem = decode_smem_bytes(span_len, page_size);
    float* scratch = nullptr;
    unsigned* tickets = nullptr;
    const int status = noalloc_setup(smem_limit, &scratch, &tickets);
    if (status != 0) return status;
    float* part_o = scratch;
    float* part_ml = scratch + o_floats;
    cudaError_t cleared = cudaMemsetAsync(tickets, 0, (size_t)n_tickets * sizeof(unsigned), stream);
    if (cleared != cudaSuccess) { snprintf(qil_error_text, sizeof(qil_error_text), "%s", cudaGetErrorString(cleared)); return (int)cleared; }
    attn_decode_span_kernel<<<dim3(n_kv_heads * chunks, n_decode, n_spans), 128, smem, stream>>>(
        p, (const int4*)decode_info, part_o, part_ml, tickets, n_spans, span_len, DecodeTail{});
    QIL_CHECK_LAUNCH();
}
