// Per-head Q/K RMSNorm, rotary position encoding and the write of K and V into
// the paged cache, in one pass over the projection output.
//
// Order as in the reference (qil/model.py:52-57): norm over head_dim of every q
// and k head with one weight vector shared by the heads, then rotation of q and
// k by the position's angles (half-split: element j pairs with j + rotary_dim/2;
// cos and sin come from a float32 table built on the host and already rounded
// to the activation dtype), then k and v go into the request's pages.  v is
// neither normed nor rotated.  Elements at or beyond rotary_dim pass unrotated.
//
// Cache layout of one layer: [page][2 (K,V)][kv_head][slot in page][head_dim].
#include "common.cuh"

#define QIL_MAX_HEAD_DIM 512

template <typename T, typename W>
__global__ void qk_norm_rope_store_kernel(
    const T* __restrict__ qkv, T* __restrict__ q_out, T* __restrict__ kv_cache,
    const W* __restrict__ q_norm_w, const W* __restrict__ k_norm_w, float eps,
    const float* __restrict__ rope_table, int rotary_dim, int table_rows,
    const int* __restrict__ positions, const int* __restrict__ token_row,
    const int* __restrict__ block_table, int table_stride,
    int n_q_heads, int n_kv_heads, int head_dim, int page_size, int num_pages) {
    extern __shared__ float stage[];  // [warps][head_dim]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int token = blockIdx.x;
    const int head = blockIdx.y * (blockDim.x >> 5) + warp;
    const int total_heads = n_q_heads + 2 * n_kv_heads;
    if (head >= total_heads) return;
    float* s = stage + warp * head_dim;
    const T* src = qkv + ((size_t)token * total_heads + head) * head_dim;

    const bool is_q = head < n_q_heads;
    const bool is_k = !is_q && head < n_q_heads + n_kv_heads;
    const W* norm_w = is_q ? q_norm_w : (is_k ? k_norm_w : nullptr);

    float sq = 0.f;
    for (int j = lane; j < head_dim; j += 32) {
        const float v = to_f32<T>(src[j]);
        s[j] = v;
        sq += v * v;
    }
    if (norm_w != nullptr) {
        sq = warp_sum(sq);
        const float scale = 1.0f / sqrtf(sq / (float)head_dim + eps);
        for (int j = lane; j < head_dim; j += 32) {
            const float normed = round_to<T>(s[j] * scale);
            s[j] = round_to<T>(normed * to_f32<W>(norm_w[j]));
        }
    }
    __syncwarp();

    int pos = positions[token];
    T* dst;
    if (is_q) {
        dst = q_out + ((size_t)token * n_q_heads + head) * head_dim;
    } else {
        const int kv_head = is_k ? head - n_q_heads : head - n_q_heads - n_kv_heads;
        const int page = block_table[(size_t)token_row[token] * table_stride + pos / page_size];
        if (page < 0 || page >= num_pages) return;  // host validation failed; never write outside the pool
        dst = kv_cache + ((((size_t)page * 2 + (is_k ? 0 : 1)) * n_kv_heads + kv_head) * page_size
                          + (pos % page_size)) * head_dim;
    }
    const bool rotate = (is_q || is_k) && rope_table != nullptr && rotary_dim > 0;
    if (rotate) {
        if (pos >= table_rows) pos = table_rows - 1;
        const int half = rotary_dim / 2;
        const float* cs = rope_table + (size_t)pos * rotary_dim;
        for (int j = lane; j < half; j += 32) {
            const float a = s[j], b = s[j + half];
            const float c = cs[j], sn = cs[half + j];
            // Each product and the sum round separately, as elementwise tensor code does.
            const float lo = __fsub_rn(round_to<T>(__fmul_rn(a, c)), round_to<T>(__fmul_rn(b, sn)));
            const float hi = __fadd_rn(round_to<T>(__fmul_rn(a, sn)), round_to<T>(__fmul_rn(b, c)));
            dst[j] = from_f32<T>(lo);
            dst[j + half] = from_f32<T>(hi);
        }
        for (int j = rotary_dim + lane; j < head_dim; j += 32) dst[j] = from_f32<T>(s[j]);
    } else {
        for (int j = lane; j < head_dim; j += 32) dst[j] = from_f32<T>(s[j]);
    }
}

extern "C" int qil_qk_norm_rope_store(
    const void* qkv, void* q_out, void* kv_cache, const void* q_norm_w, const void* k_norm_w,
    int norm_w_dtype, float eps, const float* rope_table, int rotary_dim, int table_rows,
    const int* positions, const int* token_row, const int* block_table, int table_stride,
    int n_tokens, int n_q_heads, int n_kv_heads, int head_dim, int page_size, int num_pages,
    int act_dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (head_dim <= 0 || head_dim > QIL_MAX_HEAD_DIM)
        QIL_REFUSE("qk_norm_rope_store: head_dim %d is outside 1..%d", head_dim, QIL_MAX_HEAD_DIM);
    if (rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 1))
        QIL_REFUSE("qk_norm_rope_store: rotary_dim %d must be even and at most head_dim %d", rotary_dim, head_dim);
    if (n_q_heads < 0 || n_kv_heads < 0 || n_q_heads + n_kv_heads == 0)
        QIL_REFUSE("qk_norm_rope_store: head counts %d/%d", n_q_heads, n_kv_heads);
    if (n_kv_heads > 0 && (kv_cache == nullptr || block_table == nullptr || page_size <= 0))
        QIL_REFUSE("qk_norm_rope_store: a cache and a block table are needed to store keys and values");
    if ((q_norm_w == nullptr) != (k_norm_w == nullptr) && n_kv_heads > 0)
        QIL_REFUSE("qk_norm_rope_store: give both norm weights or neither");
    const int warps = 4;
    const int total_heads = n_q_heads + 2 * n_kv_heads;
    dim3 grid(n_tokens, (total_heads + warps - 1) / warps);
    const size_t smem = (size_t)warps * head_dim * sizeof(float);
    QIL_DISPATCH_2(act_dtype, norm_w_dtype,
        (qk_norm_rope_store_kernel<T, W><<<grid, warps * 32, smem, stream>>>(
            (const T*)qkv, (T*)q_out, (T*)kv_cache, (const W*)q_norm_w, (const W*)k_norm_w, eps,
            rope_table, rotary_dim, table_rows, positions, token_row, block_table, table_stride,
            n_q_heads, n_kv_heads, head_dim, page_size, num_pages)));
    QIL_CHECK_LAUNCH();
}
