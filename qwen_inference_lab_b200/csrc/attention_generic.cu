// Causal grouped-query attention over the paged cache for any head size, page
// size and dtype, on the CUDA cores with float32 arithmetic throughout.
//
// This is the attention of the true 32-bit path, and the one that serves head
// sizes or dtypes the tensor-core kernels do not take.  One block computes one
// (token, query head): scores against the keys of its request from the window's
// start to the token's own position (absolute positions, so a chunk that
// continues a cached prefix is masked correctly; qil/model.py:62-64), softmax
// and the weighted sum of values (qil/model.py:65-68, scale head_dim^-1/2;
// query head h reads kv head h / (Hq/Hkv), qil/paged_attention.py:21).
//
// Keys are walked in tiles of 128 aligned to absolute positions and summed in
// ascending order, so a token's result depends only on its own query and the
// cache contents: not on how the batch was cut or what else is in it.
#include "common.cuh"

#define GEN_TILE 128
#define GEN_MAX_D 512
#define GEN_DPT (GEN_MAX_D / GEN_TILE)

template <typename T>
__global__ void __launch_bounds__(GEN_TILE)
attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ kv_cache, T* __restrict__ out,
                         const int* __restrict__ positions, const int* __restrict__ token_row,
                         const int* __restrict__ block_table, int table_stride,
                         int n_q_heads, int n_kv_heads, int head_dim, int page_size, int num_pages,
                         int window, float scale) {
    extern __shared__ long long smem_ll[];
    long long* row_off = smem_ll;                      // [GEN_TILE] element offset of each key row, -1 if none
    float* ks = reinterpret_cast<float*>(row_off + GEN_TILE);  // [GEN_TILE][33]
    float* ps = ks + GEN_TILE * 33;                    // [GEN_TILE]
    float* red = ps + GEN_TILE;                        // [32]
    float* qs = red + 32;                              // [head_dim]

    const int tid = threadIdx.x;
    const int token = blockIdx.x, head = blockIdx.y;
    const int kv_head = head / (n_q_heads / n_kv_heads);
    const int pos = positions[token];
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int* table = block_table + (size_t)token_row[token] * table_stride;

    const T* qrow = q + ((size_t)token * n_q_heads + head) * head_dim;
    for (int d = tid; d < head_dim; d += GEN_TILE) qs[d] = to_f32<T>(qrow[d]);

    float m_run = -INFINITY, l_run = 0.f;
    float acc[GEN_DPT];
#pragma unroll
    for (int i = 0; i < GEN_DPT; ++i) acc[i] = 0.f;

    const size_t v_plane = (size_t)n_kv_heads * page_size * head_dim;  // K plane -> V plane of a page
    for (int tile = lo / GEN_TILE; tile * GEN_TILE <= pos; ++tile) {
        const int key = tile * GEN_TILE + tid;
        const bool valid = key >= lo && key <= pos;
        long long off = -1;
        if (valid) {
            const int page = key / page_size < table_stride ? table[key / page_size] : -1;
            if (page >= 0 && page < num_pages)
                off = ((((long long)page * 2) * n_kv_heads + kv_head) * page_size + (key % page_size)) * head_dim;
        }
        __syncthreads();  // previous tile's readers of row_off / ps are done
        row_off[tid] = off;
        __syncthreads();

        float dot = 0.f;
        for (int d0 = 0; d0 < head_dim; d0 += 32) {
            const int chunk = head_dim - d0 < 32 ? head_dim - d0 : 32;
            for (int idx = tid; idx < GEN_TILE * 32; idx += GEN_TILE) {
                const int kk = idx >> 5, dd = idx & 31;
                const long long ro = row_off[kk];
                ks[kk * 33 + dd] = (ro >= 0 && dd < chunk) ? to_f32<T>(kv_cache[ro + d0 + dd]) : 0.f;
            }
            __syncthreads();
            for (int dd = 0; dd < chunk; ++dd) dot = fmaf(qs[d0 + dd], ks[tid * 33 + dd], dot);
            __syncthreads();
        }
        const float score = (valid && off >= 0) ? dot * scale : -INFINITY;
        const float tile_max = block_max(score, red);
        const float m_new = fmaxf(m_run, tile_max);
        const float p = (score == -INFINITY) ? 0.f : expf(score - m_new);
        const float corr = (m_run == -INFINITY) ? 0.f : expf(m_run - m_new);
        ps[tid] = p;
        const float tile_sum = block_sum(p, red);   // has __syncthreads inside: ps is visible after it
        l_run = l_run * corr + tile_sum;
        m_run = m_new;
#pragma unroll
        for (int i = 0; i < GEN_DPT; ++i) {
            const int d = tid + i * GEN_TILE;
            if (d < head_dim) {
                float a = acc[i] * corr;
                for (int kk = 0; kk < GEN_TILE; ++kk) {
                    const long long ro = row_off[kk];
                    if (ro >= 0) a = fmaf(ps[kk], to_f32<T>(kv_cache[ro + v_plane + d]), a);
                }
                acc[i] = a;
            }
        }
    }
    T* orow = out + ((size_t)token * n_q_heads + head) * head_dim;
#pragma unroll
    for (int i = 0; i < GEN_DPT; ++i) {
        const int d = tid + i * GEN_TILE;
        if (d < head_dim) orow[d] = from_f32<T>(l_run > 0.f ? acc[i] / l_run : 0.f);
    }
}

extern "C" int qil_attention_generic(
    const void* q, const void* kv_cache, void* out, const int* positions, const int* token_row,
    const int* block_table, int table_stride, int n_tokens, int n_q_heads, int n_kv_heads,
    int head_dim, int page_size, int num_pages, int window, float scale, int act_dtype,
    cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (head_dim <= 0 || head_dim > GEN_MAX_D)
        QIL_REFUSE("attention_generic: head_dim %d is outside 1..%d", head_dim, GEN_MAX_D);
    if (n_kv_heads <= 0 || n_q_heads <= 0 || n_q_heads % n_kv_heads)
        QIL_REFUSE("attention_generic: %d query heads do not divide into %d kv heads", n_q_heads, n_kv_heads);
    if (n_q_heads > 65535) QIL_REFUSE("attention_generic: too many heads (%d)", n_q_heads);
    if (page_size <= 0 || window < 0) QIL_REFUSE("attention_generic: page_size %d window %d", page_size, window);
    dim3 grid(n_tokens, n_q_heads);
    const size_t smem = (size_t)(head_dim + GEN_TILE * 33 + GEN_TILE + 32) * sizeof(float)
                        + GEN_TILE * sizeof(long long);
    QIL_DISPATCH_1(act_dtype,
        (attention_generic_kernel<T><<<grid, GEN_TILE, smem, stream>>>(
            (const T*)q, (const T*)kv_cache, (T*)out, positions, token_row, block_table, table_stride,
            n_q_heads, n_kv_heads, head_dim, page_size, num_pages, window, scale)));
    QIL_CHECK_LAUNCH();
}
