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
        const int index = pos / page_size;       // a position the table has no entry for writes nothing
        const int page = (pos >= 0 && index < table_stride) ? block_table[(size_t)token_row[token] * table_stride + index] : -1;
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

// bfloat16 fast path (bfloat16 norm weights, head sizes up to 256, rotary_dim a multiple of 4): a block
// per token, each warp walks heads warp, warp+8, ...  A lane keeps 2-element vectors (elements 2l, 2l+1
// of every run of 64 in the rotated half and their partners rotary_dim/2 further on), so every access
// is a coalesced 128-byte row of 4-byte words.  The arithmetic is packed bfloat16: a product of two
// bfloat16 values rounded once is what elementwise tensor code computes, and two of them cost one
// instruction instead of the six that emulating the rounding in float32 takes (the kernel was bound by
// instruction issue, not by memory, before).
// HD > 0 fixes the head size at compile time and means that the whole head rotates (rotary_dim == HD):
// the loops then have no dead iterations and no predicates, which matters because the kernel is bound
// by instruction issue.  HD == 0 takes any head size up to 256 and any rotary_dim.
#define ROPE_FAST_MAX_D 256
template <int HD>
__global__ void __launch_bounds__(256)
qk_norm_rope_store_bf16_kernel(
    const bf16* __restrict__ qkv, bf16* __restrict__ q_out, bf16* __restrict__ kv_cache,
    const bf16* __restrict__ q_norm_w, const bf16* __restrict__ k_norm_w, float eps,
    const float* __restrict__ rope_table, int rotary_dim_arg, int table_rows,
    const int* __restrict__ positions, const int* __restrict__ token_row,
    const int* __restrict__ block_table, int table_stride,
    int n_q_heads, int n_kv_heads, int head_dim_arg, int page_size, int num_pages) {
    typedef __nv_bfloat162 bf2;
    const int head_dim = HD ? HD : head_dim_arg;
    const int rotary_dim = HD ? HD : rotary_dim_arg;
    qil_wait_for_producer();
    qil_release_consumer();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int token = blockIdx.x;
    const int total_heads = n_q_heads + 2 * n_kv_heads;
    // the token's position and page first: their latency hides behind the first head's loads
    int pos = positions[token];
    const int page = (n_kv_heads > 0) ? ((pos >= 0 && pos / page_size < table_stride)
        ? block_table[(size_t)token_row[token] * table_stride + pos / page_size] : -1) : 0;
    const int slot = page_size > 0 ? pos % page_size : 0;
    if (pos >= table_rows && table_rows > 0) pos = table_rows - 1;
    constexpr int RUNS = HD ? (HD / 2 + 63) / 64 : ROPE_FAST_MAX_D / 2 / 64;   // runs of 64 elements in a rotated half
    constexpr int REST = ROPE_FAST_MAX_D / 64;              // runs of 64 elements outside the rotated part (value heads)

    // Three heads at a time: all their loads are issued before any is used, so a warp has several
    // hundred bytes in flight instead of one head's worth (the kernel is bound by latency otherwise).
    constexpr int U = 3;
    for (int head0 = warp; head0 < total_heads; head0 += 8 * U) {
        bf2 lo[U][RUNS], hi[U][RUNS], rest[U][REST];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int head = head0 + 8 * u;
            if (head >= total_heads) continue;
            const bool rotate = head < n_q_heads + n_kv_heads && rope_table != nullptr && rotary_dim > 0;
            const int rot = rotate ? rotary_dim : 0, half = rot / 2;
            const bf2* src = reinterpret_cast<const bf2*>(qkv + ((size_t)token * total_heads + head) * head_dim);
#pragma unroll
            for (int i = 0; i < RUNS; ++i) {
                const int j = 2 * lane + 64 * i;
                if (j < half) { lo[u][i] = src[j / 2]; hi[u][i] = src[(j + half) / 2]; }
            }
#pragma unroll
            for (int i = 0; i < REST; ++i) {
                const int j = rot + 2 * lane + 64 * i;
                if (j < head_dim) rest[u][i] = src[j / 2];
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int head = head0 + 8 * u;
            if (head >= total_heads) continue;
            const bool is_q = head < n_q_heads;
            const bool is_k = !is_q && head < n_q_heads + n_kv_heads;
            const bf16* norm_w = is_q ? q_norm_w : (is_k ? k_norm_w : nullptr);
            const bool rotate = (is_q || is_k) && rope_table != nullptr && rotary_dim > 0;
            const int rot = rotate ? rotary_dim : 0, half = rot / 2;
            if (norm_w != nullptr) {
                float sq = 0.f;
#pragma unroll
                for (int i = 0; i < RUNS; ++i) {
                    if (2 * lane + 64 * i < half) {
                        const float2 a = __bfloat1622float2(lo[u][i]), b = __bfloat1622float2(hi[u][i]);
                        sq += a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y;
                    }
                }
#pragma unroll
                for (int i = 0; i < REST; ++i) {
                    if (rot + 2 * lane + 64 * i < head_dim) {
                        const float2 a = __bfloat1622float2(rest[u][i]);
                        sq += a.x * a.x + a.y * a.y;
                    }
                }
                sq = warp_sum(sq);
                const float scale = rsqrtf(sq / (float)head_dim + eps);   // 2 ulp; the result is rounded to bfloat16
                const bf2* w2 = reinterpret_cast<const bf2*>(norm_w);
                auto normed = [&](bf2 v, int j) {     // round(x * scale) in float32, then times the weight in bfloat16
                    const float2 f = __bfloat1622float2(v);
                    return __hmul2_rn(__floats2bfloat162_rn(f.x * scale, f.y * scale), w2[j / 2]);
                };
#pragma unroll
                for (int i = 0; i < RUNS; ++i) {
                    const int j = 2 * lane + 64 * i;
                    if (j < half) { lo[u][i] = normed(lo[u][i], j); hi[u][i] = normed(hi[u][i], j + half); }
                }
#pragma unroll
                for (int i = 0; i < REST; ++i) {
                    const int j = rot + 2 * lane + 64 * i;
                    if (j < head_dim) rest[u][i] = normed(rest[u][i], j);
                }
            }
            bf16* dst;
            if (is_q) {
                dst = q_out + ((size_t)token * n_q_heads + head) * head_dim;
            } else {
                const int kv_head = is_k ? head - n_q_heads : head - n_q_heads - n_kv_heads;
                if (page < 0 || page >= num_pages) continue;  // host validation failed; never write outside the pool
                dst = kv_cache + ((((size_t)page * 2 + (is_k ? 0 : 1)) * n_kv_heads + kv_head) * page_size + slot) * head_dim;
            }
            bf2* out2 = reinterpret_cast<bf2*>(dst);
            if (rotate) {
                const float* cs = rope_table + (size_t)pos * rotary_dim;
#pragma unroll
                for (int i = 0; i < RUNS; ++i) {
                    const int j = 2 * lane + 64 * i;
                    if (j < half) {
                        // the table holds values already rounded to bfloat16: the conversion is exact
                        const float2 cf = *reinterpret_cast<const float2*>(cs + j);
                        const float2 sf = *reinterpret_cast<const float2*>(cs + half + j);
                        const bf2 c = __floats2bfloat162_rn(cf.x, cf.y), sn = __floats2bfloat162_rn(sf.x, sf.y);
                        // each product and the sum round separately, as elementwise tensor code does: the _rn
                        // forms, because the plain ones may be contracted into fused multiply-adds, which round
                        // once where the reference rounds twice (one value in five then differs in its last bit)
                        out2[j / 2] = __hsub2_rn(__hmul2_rn(lo[u][i], c), __hmul2_rn(hi[u][i], sn));
                        out2[(j + half) / 2] = __hadd2_rn(__hmul2_rn(lo[u][i], sn), __hmul2_rn(hi[u][i], c));
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < REST; ++i) {
                const int j = rot + 2 * lane + 64 * i;
                if (j < head_dim) out2[j / 2] = rest[u][i];
            }
        }
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
    const int total_heads = n_q_heads + 2 * n_kv_heads;
    if (act_dtype == QIL_BF16 && (q_norm_w == nullptr || norm_w_dtype == QIL_BF16) &&
        head_dim <= ROPE_FAST_MAX_D && head_dim % 2 == 0 && rotary_dim % 4 == 0 &&
        (rope_table == nullptr || rotary_dim == 0 || ((uintptr_t)rope_table & 7) == 0) &&
        (((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)kv_cache | (uintptr_t)q_norm_w | (uintptr_t)k_norm_w) & 3) == 0) {
        dim3 fast_grid(n_tokens);
#define QIL_ROPE_FAST(HD)                                                                                   \
        qil_launch_chained(qk_norm_rope_store_bf16_kernel<HD>, fast_grid, dim3(256), 0, stream,                \
            (const bf16*)qkv, (bf16*)q_out, (bf16*)kv_cache, (const bf16*)q_norm_w, (const bf16*)k_norm_w, eps, \
            rope_table, rotary_dim, table_rows, positions, token_row, block_table, table_stride,               \
            n_q_heads, n_kv_heads, head_dim, page_size, num_pages)
        const bool whole = rope_table != nullptr && rotary_dim == head_dim;
        if (whole && head_dim == 128) QIL_ROPE_FAST(128);
        else if (whole && head_dim == 64) QIL_ROPE_FAST(64);
        else QIL_ROPE_FAST(0);
#undef QIL_ROPE_FAST
        QIL_CHECK_LAUNCH();
    }
    const int warps = 4;
    dim3 grid(n_tokens, (total_heads + warps - 1) / warps);
    const size_t smem = (size_t)warps * head_dim * sizeof(float);
    QIL_DISPATCH_2(act_dtype, norm_w_dtype,
        (qk_norm_rope_store_kernel<T, W><<<grid, warps * 32, smem, stream>>>(
            (const T*)qkv, (T*)q_out, (T*)kv_cache, (const W*)q_norm_w, (const W*)k_norm_w, eps,
            rope_table, rotary_dim, table_rows, positions, token_row, block_table, table_stride,
            n_q_heads, n_kv_heads, head_dim, page_size, num_pages)));
    QIL_CHECK_LAUNCH();
}
