// bfloat16 causal grouped-query attention over the paged cache on the tensor
// cores (mma.sync m16n8k16, float32 accumulation, float32 softmax), compiled for
// one head size: -DQIL_HEAD_DIM=<multiple of 16, at most 256>.
//
// Two forms, one arithmetic (scores = q k^T * head_dim^-1/2 over keys j <= the
// token's absolute position and inside the window; softmax; times v;
// qil/model.py:59-68, qil/paged_attention.py:25-41):
//
//  * portions of prompts: one block per (tile of 64 query tokens of a segment,
//    query head).  Keys and values of the segment's request stream through
//    shared memory in tiles of 64 positions, found through the block table, with
//    an online softmax; history written by earlier steps and the portion's own
//    keys are treated alike.
//  * single tokens: one block per (span of positions, kv head, token) serves
//    all query heads of that kv head at once, so every key byte is read once;
//    blocks write unnormalised partial sums and (max, sum) to scratch memory and
//    a second kernel merges the spans in ascending order
//    (the reference's partition + merge kernels, qil/paged_attention.py:13-58).
//    The span length is the caller's choice (a multiple of 64): short spans fill
//    the GPU when few tokens decode, long spans amortise a block's start-up when
//    many do.
//
// Key tiles and spans are aligned to absolute positions.
// Cache layout of one layer: [page][2 (K,V)][kv_head][slot in page][head_dim].
#include "common.cuh"

#ifndef QIL_HEAD_DIM
#error "compile with -DQIL_HEAD_DIM=<head size>"
#endif
static_assert(QIL_HEAD_DIM % 16 == 0 && QIL_HEAD_DIM >= 16 && QIL_HEAD_DIM <= 256,
              "the tensor-core attention takes head sizes 16, 32, ..., 256");

QIL_ERROR_STORAGE

#define KV_TILE 64          // key positions per shared-memory tile
#define Q_TILE 64           // query tokens per block (prompt portions)
#define MAX_DECODE_SPAN 8192 // most key positions per block (single tokens)

constexpr int D = QIL_HEAD_DIM;
constexpr int LDS = D + 8;           // shared-memory row stride in elements: rows start 16 bytes apart mod 128
constexpr int KSTEPS = D / 16;
constexpr bool Q_IN_REGS = (D <= 128);

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem);
    const int bytes = valid ? 16 : 0;   // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gmem), "r"(bytes));
}
// The same for bytes that are read once a step (a single token's keys and values): they are the first to leave L2,
// so that what is read again (activations, partial sums, tables) stays.
__device__ __forceinline__ void cp_async16_stream(void* smem, const void* gmem, bool valid) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem);
    const int bytes = valid ? 16 : 0;
    unsigned long long policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;\n" : "=l"(policy));
    asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2, %3;\n" ::"r"(dst), "l"(gmem), "r"(bytes), "l"(policy));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x on the special-function unit (about 2 ulp; -inf gives 0): the softmax stays in float32, only the
// library routine's range handling is skipped.
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

struct AttnParams {
    const bf16* q;            // [N, Hq, D]
    const bf16* kv;           // one layer's pages
    bf16* out;                // [N, Hq, D]
    const int* block_table;
    int table_stride;
    int n_q_heads, n_kv_heads, page_size, num_pages, window;
    float scale_log2;         // head_dim^-1/2 * log2(e)
};

// Where the key row of position ``pos`` of one kv head starts, in units of 16 bytes from the layer's
// base (the value row lies one (kv_heads * page_size * D) plane further); -1 when the position is outside
// [lo, hi] or holds no page.  ``pages`` holds the request's page ids from logical page ``first_page`` on.
__device__ __forceinline__ int kv_row_offset(const AttnParams& p, const int* pages, int first_page, int kv_head,
                                             int pos, int lo, int hi) {
    if (pos < lo || pos > hi || pos / p.page_size >= p.table_stride) return -1;
    const int page = pages[pos / p.page_size - first_page];
    if (page < 0 || page >= p.num_pages) return -1;
    return (int)((((size_t)page * 2 * p.n_kv_heads + kv_head) * p.page_size + (pos % p.page_size)) * (D / 8));
}

// Queue the copies of 64 key rows and 64 value rows into shared memory; rows without an offset are
// zero-filled.  Consecutive threads take consecutive 16-byte pieces of a row, so one warp request
// covers whole 128-byte lines (a request that touches 32 different lines costs 32 tag look-ups).
__device__ __forceinline__ void issue_kv_tile(const AttnParams& p, const int* row_off, bf16* sK, bf16* sV, int tid) {
    constexpr int CPR = D / 8;                  // 16-byte pieces per row
    constexpr int PASSES = KV_TILE * CPR / 128; // D is a multiple of 16, so this is exact
    const size_t v_plane = (size_t)p.n_kv_heads * p.page_size * D;
#pragma unroll
    for (int i = 0; i < PASSES; ++i) {
        const int idx = i * 128 + tid;
        const int row = idx / CPR, piece = idx % CPR;
        const int off = row_off[row];
        const bool valid = off >= 0;
        const bf16* src = p.kv + (size_t)(valid ? off : 0) * 8 + piece * 8;
        cp_async16(sK + row * LDS + piece * 8, src, valid);
        cp_async16(sV + row * LDS + piece * 8, src + v_plane, valid);
    }
}

// ------------------------------------------------------------------ prompt portions
__global__ void __launch_bounds__(128, (QIL_HEAD_DIM <= 128) ? 3 : 1)
attn_prefill_kernel(AttnParams p, const int4* __restrict__ tile_info) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    // [K stage 0][K stage 1][V stage 0][V stage 1]; when the queries live in registers (head sizes up to
    // 128) their tile borrows K stage 1 until the fragments are loaded, else it has a region of its own
    bf16* sK = reinterpret_cast<bf16*>(smem_raw);      // [2][64][LDS]
    bf16* sV = sK + 2 * KV_TILE * LDS;                  // [2][64][LDS]
    bf16* sQ = Q_IN_REGS ? sK + KV_TILE * LDS : sV + 2 * KV_TILE * LDS;   // [64][LDS]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // heads vary fastest, so all heads of the longest tile start first (tiles come sorted, longest first)
    const int head = blockIdx.x;
    const int kv_head = head / (p.n_q_heads / p.n_kv_heads);
    // tile_info: (first token in the flat batch, its absolute position, rows in the tile, block-table row)
    const int4 info = tile_info[blockIdx.y];
    const int n0 = info.x, pos0 = info.y, rows = min(Q_TILE, info.z);
    const int hi = pos0 + rows - 1;
    const int lo = (p.window > 0 && pos0 - p.window + 1 > 0) ? pos0 - p.window + 1 : 0;
    const int* table = p.block_table + (size_t)info.w * p.table_stride;

    {   // queries of this tile: two threads per row
        const int row = tid >> 1, half = tid & 1;
        const bool valid = row < rows;
        const bf16* src = p.q + ((size_t)(n0 + (valid ? row : 0)) * p.n_q_heads + head) * D;
        constexpr int CHUNKS = D / 16;
#pragma unroll
        for (int c = 0; c < CHUNKS; ++c) {
            const int col = (half * CHUNKS + c) * 8;
            cp_async16(sQ + row * LDS + col, src + col, valid);
        }
    }
    __shared__ int row_off[2][KV_TILE];
    const int first_tile = lo / KV_TILE, last_tile = hi / KV_TILE;
    if (tid < KV_TILE) {
        row_off[0][tid] = kv_row_offset(p, table, 0, kv_head, first_tile * KV_TILE + tid, lo, hi);
        row_off[1][tid] = kv_row_offset(p, table, 0, kv_head, (first_tile + 1) * KV_TILE + tid, lo, hi);
    }
    cp_async_commit();                 // group: the queries
    __syncthreads();
    issue_kv_tile(p, row_off[0], sK, sV, tid);
    cp_async_commit();                 // group: the first tile

    unsigned qf[Q_IN_REGS ? KSTEPS : 1][4];
    if (Q_IN_REGS) {
        cp_async_wait<1>();            // the queries have landed (the first tile may still be under way)
        __syncthreads();
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks)
            ldmatrix_x4(qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3],
                        sQ + (warp * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * LDS + ks * 16 + (lane >> 4) * 8);
        __syncthreads();               // K stage 1 is free for the second tile
    }
    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
    const int row_a = warp * 16 + (lane >> 2), row_b = row_a + 8;
    const int pos_a = pos0 + row_a, pos_b = pos0 + row_b;

    for (int tile = first_tile; tile <= last_tile; ++tile) {
        const int buf = (tile - first_tile) & 1;
        if (tile + 1 <= last_tile)
            issue_kv_tile(p, row_off[buf ^ 1], sK + (buf ^ 1) * KV_TILE * LDS, sV + (buf ^ 1) * KV_TILE * LDS, tid);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        // the row offsets of the tile after next go where this tile's were (everyone has used those)
        if (tile + 2 <= last_tile && tid < KV_TILE)
            row_off[buf][tid] = kv_row_offset(p, table, 0, kv_head, (tile + 2) * KV_TILE + tid, lo, hi);
        const bf16* tK = sK + buf * KV_TILE * LDS;
        const bf16* tV = sV + buf * KV_TILE * LDS;

        float s[KV_TILE / 8][4];
#pragma unroll
        for (int i = 0; i < KV_TILE / 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            unsigned a[4];
            if (Q_IN_REGS) {
                a[0] = qf[ks][0]; a[1] = qf[ks][1]; a[2] = qf[ks][2]; a[3] = qf[ks][3];
            } else {
                ldmatrix_x4(a[0], a[1], a[2], a[3],
                            sQ + (warp * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * LDS + ks * 16 + (lane >> 4) * 8);
            }
#pragma unroll
            for (int np = 0; np < KV_TILE / 16; ++np) {
                unsigned b0, b1, b2, b3;
                ldmatrix_x4(b0, b1, b2, b3,
                            tK + (np * 16 + (lane >> 4) * 8 + (lane & 7)) * LDS + ks * 16 + ((lane >> 3) & 1) * 8);
                mma_bf16(s[2 * np], a, b0, b1);
                mma_bf16(s[2 * np + 1], a, b2, b3);
            }
        }
        // scale, mask by absolute position, online softmax (float32).  A tile that lies wholly at or before
        // the first row's position and inside the last row's window needs no mask.
        float tmax_a = -INFINITY, tmax_b = -INFINITY;
        const bool full = (tile + 1) * KV_TILE - 1 <= pos0 && (p.window == 0 || tile * KV_TILE > hi - p.window);
        if (full) {
#pragma unroll
            for (int nt = 0; nt < KV_TILE / 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) s[nt][e] *= p.scale_log2;
                tmax_a = fmaxf(tmax_a, fmaxf(s[nt][0], s[nt][1]));
                tmax_b = fmaxf(tmax_b, fmaxf(s[nt][2], s[nt][3]));
            }
        } else {
#pragma unroll
            for (int nt = 0; nt < KV_TILE / 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = tile * KV_TILE + nt * 8 + (lane & 3) * 2 + (e & 1);
                    const int pos = (e < 2) ? pos_a : pos_b;
                    const bool ok = key <= pos && (p.window == 0 || key > pos - p.window);
                    const float v = ok ? s[nt][e] * p.scale_log2 : -INFINITY;
                    s[nt][e] = v;
                    if (e < 2) tmax_a = fmaxf(tmax_a, v); else tmax_b = fmaxf(tmax_b, v);
                }
            }
        }
        tmax_a = fmaxf(tmax_a, __shfl_xor_sync(0xffffffffu, tmax_a, 1));
        tmax_a = fmaxf(tmax_a, __shfl_xor_sync(0xffffffffu, tmax_a, 2));
        tmax_b = fmaxf(tmax_b, __shfl_xor_sync(0xffffffffu, tmax_b, 1));
        tmax_b = fmaxf(tmax_b, __shfl_xor_sync(0xffffffffu, tmax_b, 2));
        const float mn_a = fmaxf(m_a, tmax_a), mn_b = fmaxf(m_b, tmax_b);
        const float ms_a = (mn_a == -INFINITY) ? 0.f : mn_a, ms_b = (mn_b == -INFINITY) ? 0.f : mn_b;
        const float corr_a = fast_exp2(m_a - ms_a), corr_b = fast_exp2(m_b - ms_b);
        m_a = mn_a; m_b = mn_b;
        float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
        for (int nt = 0; nt < KV_TILE / 8; ++nt) {
            s[nt][0] = fast_exp2(s[nt][0] - ms_a); s[nt][1] = fast_exp2(s[nt][1] - ms_a);
            s[nt][2] = fast_exp2(s[nt][2] - ms_b); s[nt][3] = fast_exp2(s[nt][3] - ms_b);
            sum_a += s[nt][0] + s[nt][1];
            sum_b += s[nt][2] + s[nt][3];
        }
        l_a = l_a * corr_a + sum_a;
        l_b = l_b * corr_b + sum_b;
#pragma unroll
        for (int i = 0; i < D / 8; ++i) { o[i][0] *= corr_a; o[i][1] *= corr_a; o[i][2] *= corr_b; o[i][3] *= corr_b; }
#pragma unroll
        for (int kt = 0; kt < KV_TILE / 16; ++kt) {
            unsigned a[4];
            a[0] = pack_bf16(s[2 * kt][0], s[2 * kt][1]);
            a[1] = pack_bf16(s[2 * kt][2], s[2 * kt][3]);
            a[2] = pack_bf16(s[2 * kt + 1][0], s[2 * kt + 1][1]);
            a[3] = pack_bf16(s[2 * kt + 1][2], s[2 * kt + 1][3]);
#pragma unroll
            for (int dp = 0; dp < D / 16; ++dp) {
                unsigned b0, b1, b2, b3;
                ldmatrix_x4_trans(b0, b1, b2, b3,
                                  tV + (kt * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * LDS + dp * 16 + (lane >> 4) * 8);
                mma_bf16(o[2 * dp], a, b0, b1);
                mma_bf16(o[2 * dp + 1], a, b2, b3);
            }
        }
        __syncthreads();   // everyone is done with this buffer before the next prefetch overwrites it
    }
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1); l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1); l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
    const float inv_a = l_a > 0.f ? 1.f / l_a : 0.f, inv_b = l_b > 0.f ? 1.f / l_b : 0.f;
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) {
        const int col = dt * 8 + (lane & 3) * 2;
        if (row_a < rows)
            *reinterpret_cast<unsigned*>(p.out + ((size_t)(n0 + row_a) * p.n_q_heads + head) * D + col) =
                pack_bf16(o[dt][0] * inv_a, o[dt][1] * inv_a);
        if (row_b < rows)
            *reinterpret_cast<unsigned*>(p.out + ((size_t)(n0 + row_b) * p.n_q_heads + head) * D + col) =
                pack_bf16(o[dt][2] * inv_b, o[dt][3] * inv_b);
    }
}

// ------------------------------------------------------------------ single tokens: how long a span
// With a negative span length the caller fixes the number of spans (the grid's) and leaves their length to
// the kernels: both kernels of the pair cut the step's longest context (the fourth int of every decode_info
// entry) into n_spans equal runs of whole tiles.  A recorded graph can so be replayed while contexts grow:
// every block of the grid keeps a share of the work, whatever the context (a span that nobody needs would
// still take a slot away from the others when it starts).  Blocks are numbered span by span (the span index
// is the grid's slowest dimension), so the short last spans start last.
__device__ __forceinline__ int span_len_of(int longest_context, int n_spans, int at_most) {
    const int tiles = max(1, (longest_context + KV_TILE - 1) / KV_TILE);
    const int span_len = (tiles + n_spans - 1) / n_spans * KV_TILE;
    return min(span_len, at_most);        // the caller sized shared memory for `at_most`
}

// ------------------------------------------------------------------ single tokens: the projection's tail
// A step of single tokens may hand this kernel the raw output of the query/key/value projection instead
// of finished queries: every block then norms and rotates the query heads it serves itself, and the
// block whose span holds the token's own position does the same for that token's key and copies its
// value, both into the token's cache page, before it reads that tile.  That is the work of the
// stand-alone kernel in rope_kv.cu, with the same arithmetic and rounding points (per-head RMSNorm with
// float32 statistics, qil/model.py:52-55; every product and sum of the rotation rounded by itself),
// without a launch of its own between the projection and the attention.
struct DecodeTail {
    const bf16* qkv;          // [N, (Hq + 2 * own_kv_heads) * D]; null: p.q holds finished queries
    const bf16* q_norm;       // [D] or null
    const bf16* k_norm;
    const float* rope;        // [rope_rows][rotary_dim]: cosines then sines; null: no rotation
    bf16* kv_out;             // the layer's pages, writable
    float eps;
    int rotary_dim, rope_rows;
    int own_kv_heads;         // 0: the layer reads another layer's cache and writes nothing
};

// One warp: a head of D values from ``src`` through RMSNorm (when ``norm_w``) and the rotation of its
// first ``rot`` values by the row ``cs`` of the table (when ``cs``), into ``dst`` (shared or global).
// A lane holds pairs (2 lane + 64 i, +1) of the rotated half, their partners rot / 2 further on, and
// pairs of the values behind the rotated part.  rot is a multiple of 4.
__device__ __forceinline__ void warp_norm_rotate_head(const bf16* __restrict__ src, const bf16* __restrict__ norm_w,
                                                      float eps, const float* __restrict__ cs, int rot,
                                                      bf16* dst, int lane) {
    typedef __nv_bfloat162 bf2;
    constexpr int RUNS = (D / 2 + 63) / 64, REST = (D + 63) / 64;
    if (cs == nullptr) rot = 0;
    const int half = rot / 2;
    const bf2* src2 = reinterpret_cast<const bf2*>(src);
    bf2 lo[RUNS], hi[RUNS], rest[REST];
#pragma unroll
    for (int i = 0; i < RUNS; ++i) {
        const int j = 2 * lane + 64 * i;
        if (j < half) { lo[i] = src2[j / 2]; hi[i] = src2[(j + half) / 2]; }
    }
#pragma unroll
    for (int i = 0; i < REST; ++i) {
        const int j = rot + 2 * lane + 64 * i;
        if (j < D) rest[i] = src2[j / 2];
    }
    if (norm_w != nullptr) {
        float sq = 0.f;
#pragma unroll
        for (int i = 0; i < RUNS; ++i)
            if (2 * lane + 64 * i < half) {
                const float2 a = __bfloat1622float2(lo[i]), b = __bfloat1622float2(hi[i]);
                sq += a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y;
            }
#pragma unroll
        for (int i = 0; i < REST; ++i)
            if (rot + 2 * lane + 64 * i < D) {
                const float2 a = __bfloat1622float2(rest[i]);
                sq += a.x * a.x + a.y * a.y;
            }
        sq = warp_sum(sq);
        const float scale = rsqrtf(sq / (float)D + eps);
        const bf2* w2 = reinterpret_cast<const bf2*>(norm_w);
        auto normed = [&](bf2 v, int j) {
            const float2 f = __bfloat1622float2(v);
            return __hmul2_rn(__floats2bfloat162_rn(f.x * scale, f.y * scale), w2[j / 2]);
        };
#pragma unroll
        for (int i = 0; i < RUNS; ++i) {
            const int j = 2 * lane + 64 * i;
            if (j < half) { lo[i] = normed(lo[i], j); hi[i] = normed(hi[i], j + half); }
        }
#pragma unroll
        for (int i = 0; i < REST; ++i) {
            const int j = rot + 2 * lane + 64 * i;
            if (j < D) rest[i] = normed(rest[i], j);
        }
    }
    bf2* out2 = reinterpret_cast<bf2*>(dst);
#pragma unroll
    for (int i = 0; i < RUNS; ++i) {
        const int j = 2 * lane + 64 * i;
        if (j < half) {
            const float2 cf = *reinterpret_cast<const float2*>(cs + j);
            const float2 sf = *reinterpret_cast<const float2*>(cs + half + j);
            const bf2 c = __floats2bfloat162_rn(cf.x, cf.y), sn = __floats2bfloat162_rn(sf.x, sf.y);   // exact: the table is rounded
            out2[j / 2] = __hsub2_rn(__hmul2_rn(lo[i], c), __hmul2_rn(hi[i], sn));
            out2[(j + half) / 2] = __hadd2_rn(__hmul2_rn(lo[i], sn), __hmul2_rn(hi[i], c));
        }
    }
#pragma unroll
    for (int i = 0; i < REST; ++i) {
        const int j = rot + 2 * lane + 64 * i;
        if (j < D) out2[j / 2] = rest[i];
    }
}

// The spans of one (token, query head) folded into its output row, by one warp.  Spans are taken sixteen at a
// time: their (max, sum) pairs and this lane's columns of their partial outputs are all asked for before any is
// used, so a batch costs one trip to L2; batches are folded into the running result as in the loops of the
// kernels (rescale by exp2(old max - new max)).  The order of the sums is fixed by the span numbers.
__device__ __forceinline__ void merge_spans_of_head(const AttnParams& p, const float* __restrict__ part_o,
                                                    const float* __restrict__ part_ml, int d_idx, int n, int head,
                                                    int n_spans, int s_lo, int s_hi, bool uncovered, int lane) {
    constexpr int COLS = (D + 31) / 32, BATCH = 16;
    const size_t base = ((size_t)d_idx * p.n_q_heads + head) * n_spans;
    float mx = -INFINITY, sum = 0.f;
    float acc[COLS];
#pragma unroll
    for (int i = 0; i < COLS; ++i) acc[i] = 0.f;
    for (int s0 = s_lo; s0 <= s_hi; s0 += BATCH) {
        float m[BATCH], l[BATCH], o_part[BATCH][COLS];
#pragma unroll
        for (int j = 0; j < BATCH; ++j) {
            const bool live = s0 + j <= s_hi;
            const size_t slot = base + (live ? s0 + j : s_lo);
            const float2 ml = __ldcg(reinterpret_cast<const float2*>(part_ml + slot * 2));
            m[j] = live ? ml.x : -INFINITY;
            l[j] = ml.y;
#pragma unroll
            for (int i = 0; i < COLS; ++i) {
                const int col = lane + i * 32;
                o_part[j][i] = col < D ? __ldcg(part_o + slot * D + col) : 0.f;
            }
        }
        float batch_max = m[0];
#pragma unroll
        for (int j = 1; j < BATCH; ++j) batch_max = fmaxf(batch_max, m[j]);
        const float new_max = fmaxf(mx, batch_max);
        const float ms = (new_max == -INFINITY) ? 0.f : new_max;
        const float keep = exp2f(mx - ms);               // 0 for the first batch (mx = -inf)
        sum *= keep;
#pragma unroll
        for (int i = 0; i < COLS; ++i) acc[i] *= keep;
#pragma unroll
        for (int j = 0; j < BATCH; ++j) {
            const float f = exp2f(m[j] - ms);            // 0 for a slot past the last span
            sum += f * l[j];
#pragma unroll
            for (int i = 0; i < COLS; ++i) acc[i] += f * o_part[j][i];
        }
        mx = new_max;
    }
    const float inv = sum > 0.f ? 1.f / sum : 0.f;
#pragma unroll
    for (int i = 0; i < COLS; ++i) {
        const int col = lane + i * 32;
        if (col < D)
            p.out[((size_t)n * p.n_q_heads + head) * D + col] =
                __float2bfloat16_rn(uncovered ? __int_as_float(0x7fc00000) : acc[i] * inv);
    }
}

// ------------------------------------------------------------------ single tokens: spans
// decode_info: (token in the flat batch, its absolute position, block-table row, unused) per token.
// part_o  [n_decode, Hq, n_spans, D] float32, unnormalised; part_ml [n_decode, Hq, n_spans, 2] (max, sum).
//
// The work of one block, as a function of its place in the grid (``block_x`` of ``grid_x``, ``d_idx``, ``span``)
// so that a kernel that walks several such places in a loop can call it too.  ``wait_for_inputs`` is called once,
// after the first key and value tiles have been asked for: up to there only memory that nothing of this step
// writes is read.
template <typename Wait>
__device__ __forceinline__ void attn_decode_span_block(
        const AttnParams& p, const int4* __restrict__ decode_info, float* __restrict__ part_o,
        float* __restrict__ part_ml, unsigned* __restrict__ tickets, int n_spans, int span_len_arg,
        const DecodeTail& tail, unsigned char* smem_raw, int block_x, int grid_x, int d_idx, int span,
        Wait wait_for_inputs) {
    bf16* sQ = reinterpret_cast<bf16*>(smem_raw);      // [16][LDS]
    bf16* sK = sQ + 16 * LDS;                           // [2][64][LDS]
    bf16* sV = sK + 2 * KV_TILE * LDS;                  // [2][64][LDS]
    int* s_pages = reinterpret_cast<int*>(sV + 2 * KV_TILE * LDS);   // [span_len / page_size + 2]
    // Up to qil_wait_for_producer() below only memory that no kernel of this step writes is read:
    // the step's description, the block table, and keys and values of earlier positions.
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int group = p.n_q_heads / p.n_kv_heads;
    const int chunks = (group + 15) / 16;
    const int kv_head = block_x / chunks, g0 = (block_x % chunks) * 16;
    const int gcount = min(16, group - g0);
    const int4 info = decode_info[d_idx];
    const int n = info.x, pos = info.y;
    const int hi = pos;
    const int lo = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
    const int span_len = span_len_arg > 0 ? span_len_arg : span_len_of(info.w, n_spans, -span_len_arg);
    const int k_begin = span * span_len;
    if (k_begin > hi || k_begin + span_len <= lo) return;    // takes no ticket: the merge counts the same spans
    const int* table = p.block_table + (size_t)info.z * p.table_stride;
    const int first_tile = max(k_begin, lo) / KV_TILE;
    const int last_tile = min(k_begin + span_len - 1, hi) / KV_TILE;

    // the page ids of the whole span, once: a tile's loads then wait for no table read
    const int first_page = (first_tile * KV_TILE) / p.page_size;
    const int last_page = min((last_tile + 1) * KV_TILE - 1, hi) / p.page_size;
    for (int i = tid; i <= last_page - first_page; i += 128)
        s_pages[i] = first_page + i < p.table_stride ? table[first_page + i] : -1;
    __syncthreads();
    // From here to the merge at the end the four warps run on their own.  A warp owns 16 keys of every
    // 64-key tile: it copies exactly those rows of K and V into its part of the two tile buffers, needs
    // only warp-level barriers around them, and asks for the rows of tile t + 2 as soon as it is done
    // with the rows of tile t (K after the scores, V after the output), so two tiles are in flight per
    // warp instead of one per block.  cp.async groups of a thread, in order: K0, V0, K1, V1, K2, ...
    constexpr int CPR = D / 8;                   // 16-byte pieces per row
    const size_t v_plane = (size_t)p.n_kv_heads * p.page_size * D;
    auto row_offset = [&](int tile) {            // lanes 0..15: where this warp's row `lane` of the tile starts
        return (lane < 16 && tile <= last_tile)
            ? kv_row_offset(p, s_pages, first_page, kv_head, tile * KV_TILE + warp * 16 + lane, lo, hi) : -1;
    };
    auto issue_rows = [&](int offset_of_lane, bf16* dst, size_t plane) {
#pragma unroll
        for (int i = 0; i < 16 * CPR / 32; ++i) {
            const int idx = i * 32 + lane;
            const int row = idx / CPR, piece = idx % CPR;
            const int off = __shfl_sync(0xffffffffu, offset_of_lane, row);
            const bool valid = off >= 0;
            cp_async16_stream(dst + row * LDS + piece * 8, p.kv + (size_t)(valid ? off : 0) * 8 + piece * 8 + (valid ? plane : 0), valid);
        }
    };
    bf16* const my_k = sK + warp * 16 * LDS;    // this warp's rows of buffer 0; buffer 1 lies KV_TILE rows further
    bf16* const my_v = sV + warp * 16 * LDS;
    constexpr int BUFFER = KV_TILE * LDS;
    const int off0 = row_offset(first_tile), off1 = row_offset(first_tile + 1);
    // The first tile starts before the wait unless it holds this step's own position, whose key and
    // value are written below (or by the kernel before this one).
    const bool early = first_tile != hi / KV_TILE;
    if (early) issue_rows(off0, my_k, 0);
    cp_async_commit();
    if (early) issue_rows(off0, my_v, v_plane);
    cp_async_commit();
    wait_for_inputs();
    if (tail.qkv == nullptr) {   // finished queries: the heads of this kv head, 8 threads per row
        const int row = tid >> 3;
        const bool valid = row < gcount;
        const bf16* src = p.q + ((size_t)n * p.n_q_heads + kv_head * group + g0 + (valid ? row : 0)) * D;
        for (int c = tid & 7; c < D / 8; c += 8) cp_async16(sQ + row * LDS + c * 8, src + c * 8, valid);
    } else {
        // raw projection: a warp per query head; rows past the group are zero as the copy above leaves them
        const int total_heads = p.n_q_heads + 2 * tail.own_kv_heads;
        const bf16* token = tail.qkv + (size_t)n * total_heads * D;
        const int rope_row = (tail.rope_rows > 0 && pos >= tail.rope_rows) ? tail.rope_rows - 1 : pos;
        const float* cs = (tail.rope != nullptr && tail.rotary_dim > 0) ? tail.rope + (size_t)rope_row * tail.rotary_dim : nullptr;
        for (int row = warp; row < 16; row += 4) {
            if (row < gcount) {
                warp_norm_rotate_head(token + (size_t)(kv_head * group + g0 + row) * D, tail.q_norm, tail.eps, cs,
                                      tail.rotary_dim, sQ + row * LDS, lane);
            } else {
                for (int c = lane; c < D / 2; c += 32) reinterpret_cast<unsigned*>(sQ + row * LDS)[c] = 0u;
            }
        }
        // The token's own key and value: by the block whose span holds its position, into its page, before
        // that block (the only one that reads the position) asks for the tile.  The host sends groups of
        // more than 16 query heads, where several blocks share a kv head's spans, to the stand-alone kernel.
        if (tail.own_kv_heads > 0 && k_begin <= hi && hi < k_begin + span_len && warp < 2) {
            const int page = s_pages[hi / p.page_size - first_page];
            if (page >= 0 && page < p.num_pages) {
                const size_t slot = (((size_t)page * 2 + warp) * p.n_kv_heads + kv_head) * p.page_size + hi % p.page_size;
                if (warp == 0)
                    warp_norm_rotate_head(token + (size_t)(p.n_q_heads + kv_head) * D, tail.k_norm, tail.eps, cs,
                                          tail.rotary_dim, tail.kv_out + slot * D, lane);
                else
                    warp_norm_rotate_head(token + (size_t)(p.n_q_heads + tail.own_kv_heads + kv_head) * D, nullptr, 0.f,
                                          nullptr, 0, tail.kv_out + slot * D, lane);
            }
            __threadfence();      // in L2 before this block's copies of the tile read it
        }
        __syncthreads();
    }
    if (!early) { issue_rows(off0, my_k, 0); issue_rows(off0, my_v, v_plane); }
    if (first_tile + 1 <= last_tile) issue_rows(off1, my_k + BUFFER, 0);
    cp_async_commit();
    if (first_tile + 1 <= last_tile) issue_rows(off1, my_v + BUFFER, v_plane);
    cp_async_commit();
    cp_async_wait<1>();          // the queries and the first tiles' keys; only the second tile's values may be under way
    __syncthreads();             // the query rows are every warp's

    unsigned qf[Q_IN_REGS ? KSTEPS : 1][4];
    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;

    for (int tile = first_tile; tile <= last_tile; ++tile) {
        const int buf = (tile - first_tile) & 1;
        const int off2 = row_offset(tile + 2);
        cp_async_wait<3>();          // this tile's keys: at most V(t), K(t+1), V(t+1) may still be under way
        __syncwarp();
        if (Q_IN_REGS && tile == first_tile) {
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks)
                ldmatrix_x4(qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3],
                            sQ + (((lane >> 3) & 1) * 8 + (lane & 7)) * LDS + ks * 16 + (lane >> 4) * 8);
        }
        const bf16* tK = my_k + buf * BUFFER;   // this warp's 16 keys of the tile
        const bf16* tV = my_v + buf * BUFFER;
        float s[2][4];
        s[0][0] = s[0][1] = s[0][2] = s[0][3] = 0.f;
        s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            unsigned a[4];
            if (Q_IN_REGS) {
                a[0] = qf[ks][0]; a[1] = qf[ks][1]; a[2] = qf[ks][2]; a[3] = qf[ks][3];
            } else {
                ldmatrix_x4(a[0], a[1], a[2], a[3],
                            sQ + (((lane >> 3) & 1) * 8 + (lane & 7)) * LDS + ks * 16 + (lane >> 4) * 8);
            }
            unsigned b0, b1, b2, b3;
            ldmatrix_x4(b0, b1, b2, b3, tK + ((lane >> 4) * 8 + (lane & 7)) * LDS + ks * 16 + ((lane >> 3) & 1) * 8);
            mma_bf16(s[0], a, b0, b1);
            mma_bf16(s[1], a, b2, b3);
        }
        __syncwarp();                // every lane has read the keys: their rows take tile t + 2
        if (tile + 2 <= last_tile) issue_rows(off2, my_k + buf * BUFFER, 0);
        cp_async_commit();
        // every row is the same position: one mask for all
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int key = tile * KV_TILE + warp * 16 + nt * 8 + (lane & 3) * 2 + (e & 1);
                const bool ok = key <= hi && key >= lo;
                s[nt][e] = ok ? s[nt][e] * p.scale_log2 : -INFINITY;
            }
        }
        float tmax_a = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
        float tmax_b = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
        tmax_a = fmaxf(tmax_a, __shfl_xor_sync(0xffffffffu, tmax_a, 1));
        tmax_a = fmaxf(tmax_a, __shfl_xor_sync(0xffffffffu, tmax_a, 2));
        tmax_b = fmaxf(tmax_b, __shfl_xor_sync(0xffffffffu, tmax_b, 1));
        tmax_b = fmaxf(tmax_b, __shfl_xor_sync(0xffffffffu, tmax_b, 2));
        const float mn_a = fmaxf(m_a, tmax_a), mn_b = fmaxf(m_b, tmax_b);
        const float ms_a = (mn_a == -INFINITY) ? 0.f : mn_a, ms_b = (mn_b == -INFINITY) ? 0.f : mn_b;
        const float corr_a = fast_exp2(m_a - ms_a), corr_b = fast_exp2(m_b - ms_b);
        m_a = mn_a; m_b = mn_b;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            s[nt][0] = fast_exp2(s[nt][0] - ms_a); s[nt][1] = fast_exp2(s[nt][1] - ms_a);
            s[nt][2] = fast_exp2(s[nt][2] - ms_b); s[nt][3] = fast_exp2(s[nt][3] - ms_b);
        }
        l_a = l_a * corr_a + (s[0][0] + s[0][1] + s[1][0] + s[1][1]);
        l_b = l_b * corr_b + (s[0][2] + s[0][3] + s[1][2] + s[1][3]);
#pragma unroll
        for (int i = 0; i < D / 8; ++i) { o[i][0] *= corr_a; o[i][1] *= corr_a; o[i][2] *= corr_b; o[i][3] *= corr_b; }
        unsigned a[4];
        a[0] = pack_bf16(s[0][0], s[0][1]);
        a[1] = pack_bf16(s[0][2], s[0][3]);
        a[2] = pack_bf16(s[1][0], s[1][1]);
        a[3] = pack_bf16(s[1][2], s[1][3]);
        cp_async_wait<3>();          // this tile's values: K(t+1), V(t+1), K(t+2) may still be under way
        __syncwarp();
#pragma unroll
        for (int dp = 0; dp < D / 16; ++dp) {
            unsigned b0, b1, b2, b3;
            ldmatrix_x4_trans(b0, b1, b2, b3, tV + (((lane >> 3) & 1) * 8 + (lane & 7)) * LDS + dp * 16 + (lane >> 4) * 8);
            mma_bf16(o[2 * dp], a, b0, b1);
            mma_bf16(o[2 * dp + 1], a, b2, b3);
        }
        __syncwarp();
        if (tile + 2 <= last_tile) issue_rows(off2, my_v + buf * BUFFER, v_plane);
        cp_async_commit();
    }
    cp_async_wait<0>();
    __syncthreads();             // every warp is done with its rows: the buffers become the merge's scratch
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1); l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1); l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);

    // merge the four warps' (max, sum, acc) through shared memory (the tile buffers are free now)
    float* wm = reinterpret_cast<float*>(sK);          // [4][16]
    float* wl = wm + 4 * 16;                            // [4][16]
    float* wo = wl + 4 * 16;                            // [4][16][D]
    const int ra = lane >> 2, rb = ra + 8;
    if ((lane & 3) == 0) {
        wm[warp * 16 + ra] = m_a; wm[warp * 16 + rb] = m_b;
        wl[warp * 16 + ra] = l_a; wl[warp * 16 + rb] = l_b;
    }
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) {
        const int col = dt * 8 + (lane & 3) * 2;
        wo[(warp * 16 + ra) * D + col] = o[dt][0]; wo[(warp * 16 + ra) * D + col + 1] = o[dt][1];
        wo[(warp * 16 + rb) * D + col] = o[dt][2]; wo[(warp * 16 + rb) * D + col + 1] = o[dt][3];
    }
    __syncthreads();
    // The spans that hold keys of this token (the others returned at the top).  n_spans * span_len short of the
    // token's position: no block saw its last keys, and a softmax over a shortened context would look like a
    // result; the rows are filled with NaN instead.
    const int s_lo = lo / span_len;
    int s_hi = pos / span_len;
    const bool uncovered = s_hi >= n_spans;
    if (uncovered) s_hi = n_spans - 1;
    const bool alone = s_lo == s_hi;             // this block holds the whole context: its sums are the result
    for (int idx = tid; idx < gcount * D; idx += 128) {
        const int r = idx / D, col = idx - r * D;
        float mx = fmaxf(fmaxf(wm[r], wm[16 + r]), fmaxf(wm[32 + r], wm[48 + r]));
        const float ms = (mx == -INFINITY) ? 0.f : mx;
        float acc = 0.f, sum = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float f = fast_exp2(wm[w * 16 + r] - ms);
            acc += f * wo[(w * 16 + r) * D + col];
            sum += f * wl[w * 16 + r];
        }
        const int head = kv_head * group + g0 + r;
        if (alone) {
            const float inv = sum > 0.f ? 1.f / sum : 0.f;
            p.out[((size_t)n * p.n_q_heads + head) * D + col] =
                __float2bfloat16_rn(uncovered ? __int_as_float(0x7fc00000) : acc * inv);
            continue;
        }
        const size_t slot = ((size_t)d_idx * p.n_q_heads + head) * n_spans + span;
        part_o[slot * D + col] = acc;
        if (col == 0) { part_ml[slot * 2] = mx; part_ml[slot * 2 + 1] = sum; }
    }
    if (alone || tickets == nullptr) return;        // no counters: a merge kernel follows

    // ---- the merge of the spans, by whichever block of this (token, kv head, head chunk) finishes last.
    // Every block that got this far takes a ticket after its partial results are in L2; the one that draws
    // the last ticket reads all of them back and writes the output rows, and puts the ticket counter back to
    // zero for the next launch.  The order of the sums is fixed by the span numbers, not by who merges.
    __shared__ int merges;
    __syncthreads();             // every thread's partial results are written ...
    if (tid == 0) {
        __threadfence();         // ... and in L2 before the ticket is (one fence after the barrier covers them all)
        unsigned* ticket = tickets + (size_t)d_idx * grid_x + block_x;
        const unsigned drawn = atomicAdd(ticket, 1u);
        merges = drawn == (unsigned)(s_hi - s_lo);
        if (merges) { *ticket = 0u; __threadfence(); }      // the other blocks' results, read below from L2
    }
    __syncthreads();
    if (!merges) return;
    for (int r = warp; r < gcount; r += 4)
        merge_spans_of_head(p, part_o, part_ml, d_idx, n, kv_head * group + g0 + r, n_spans, s_lo, s_hi, uncovered, lane);
}

// The merge as a kernel of its own, for launches without ticket counters: a warp per (token, query head).
__global__ void __launch_bounds__(128)
attn_decode_merge_kernel(AttnParams p, const int4* __restrict__ decode_info, const float* __restrict__ part_o,
                         const float* __restrict__ part_ml, int n_spans, int span_len_arg) {
    // the step's description is older than the kernel before this one: read it while that one finishes
    const int d_idx = blockIdx.y, head = blockIdx.x * 4 + (threadIdx.x >> 5);
    const int4 info = decode_info[d_idx];
    const int pos = info.y;
    const int lo = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
    const int span_len = span_len_arg > 0 ? span_len_arg : span_len_of(info.w, n_spans, -span_len_arg);
    const int s_lo = lo / span_len;
    int s_hi = pos / span_len;
    const bool uncovered = s_hi >= n_spans;
    if (uncovered) s_hi = n_spans - 1;
    qil_wait_for_producer();
    qil_release_consumer();
    if (s_lo == s_hi) return;       // one span held the whole context: its block wrote the rows itself
    if (head < p.n_q_heads)
        merge_spans_of_head(p, part_o, part_ml, d_idx, info.x, head, n_spans, s_lo, s_hi, uncovered, threadIdx.x & 31);
}

__global__ void __launch_bounds__(128)
attn_decode_span_kernel(AttnParams p, const int4* __restrict__ decode_info, float* __restrict__ part_o,
                        float* __restrict__ part_ml, unsigned* __restrict__ tickets, int n_spans, int span_len_arg,
                        DecodeTail tail) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    // the span index varies slowest: see span_len_of
    attn_decode_span_block(p, decode_info, part_o, part_ml, tickets, n_spans, span_len_arg, tail, smem_raw,
                           (int)blockIdx.x, (int)gridDim.x, (int)blockIdx.y, (int)blockIdx.z,
                           [] { qil_wait_for_producer(); qil_release_consumer(); });
}

// ------------------------------------------------------------------ entry points
static int fill_params(AttnParams& p, const void* q, const void* kv, void* out, const int* block_table,
                       int table_stride, int n_q_heads, int n_kv_heads, int page_size, int num_pages,
                       int window, float scale) {
    if (n_kv_heads <= 0 || n_q_heads <= 0 || n_q_heads % n_kv_heads)
        QIL_REFUSE("attention: %d query heads do not divide into %d kv heads", n_q_heads, n_kv_heads);
    if (page_size <= 0 || num_pages <= 0 || window < 0 || table_stride <= 0)
        QIL_REFUSE("attention: page_size %d pages %d window %d table width %d", page_size, num_pages, window, table_stride);
    if (((uintptr_t)q | (uintptr_t)kv | (uintptr_t)out) & 15)
        QIL_REFUSE("attention: q, cache and out must be 16-byte aligned");
    p.q = (const bf16*)q; p.kv = (const bf16*)kv; p.out = (bf16*)out;
    p.block_table = block_table; p.table_stride = table_stride;
    p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads; p.page_size = page_size; p.num_pages = num_pages;
    p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f;
    return 0;
}

// Shared memory of the span kernel: query rows, two stages of key and value tiles (reused for the
// merge of the four warps), and the span's page ids.
static int decode_smem_bytes(int span_len, int page_size) {
    const int tile_bytes = (16 + 4 * KV_TILE) * LDS * (int)sizeof(bf16);
    return tile_bytes + (span_len / page_size + 3) * (int)sizeof(int);
}

// The span kernel's dynamic shared-memory limit is a setting of the function on a device: every entry point
// that launches the kernel goes through here, so the limit is only ever raised.  One slot per device
// ordinal; not safe for host threads that call these entry points at the same time.
#define QIL_ATTN_MAX_DEVICES 64
static int decode_smem_configured[QIL_ATTN_MAX_DEVICES];
template <typename Kernel>
static int ensure_decode_smem(Kernel kernel, int smem) {
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) QIL_REFUSE("attention: cudaGetDevice: %s", cudaGetErrorString(e));
    if (device < 0 || device >= QIL_ATTN_MAX_DEVICES) QIL_REFUSE("attention: device %d is out of range", device);
    if (smem > decode_smem_configured[device]) {
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) QIL_REFUSE("attention: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
        decode_smem_configured[device] = smem;
    }
    return 0;
}

static int check_decode_span(int span_len, int n_spans) {
    const int length = span_len < 0 ? -span_len : span_len;      // negative: the longest the kernels may choose
    if (length < KV_TILE || length > MAX_DECODE_SPAN || length % KV_TILE)
        QIL_REFUSE("attention: a span of %d positions; spans are multiples of %d up to %d", span_len, KV_TILE, MAX_DECODE_SPAN);
    if (n_spans <= 0) QIL_REFUSE("attention: n_spans %d", n_spans);
    return 0;
}

extern "C" int qil_attn_head_dim() { return D; }
extern "C" int qil_attn_max_decode_span() { return MAX_DECODE_SPAN; }

// tile_info: int32 [n_tiles, 4] = (first token, its absolute position, rows <= 64, block-table row).
extern "C" int qil_attn_prefill(const void* q, const void* kv, void* out, const int* tile_info, int n_tiles,
                                const int* block_table, int table_stride, int n_q_heads, int n_kv_heads,
                                int page_size, int num_pages, int window, float scale, cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    AttnParams p;
    if (fill_params(p, q, kv, out, block_table, table_stride, n_q_heads, n_kv_heads, page_size, num_pages,
                    window, scale)) return -1;
    if (n_tiles > 65535) QIL_REFUSE("attention: %d query tiles in one launch; at most 65535", n_tiles);
    if ((uintptr_t)tile_info & 15) QIL_REFUSE("attention: tile_info must be 16-byte aligned");
    const int smem = ((Q_IN_REGS ? 0 : Q_TILE) + 4 * KV_TILE) * LDS * (int)sizeof(bf16);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) QIL_REFUSE("attention: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    attn_prefill_kernel<<<dim3(n_q_heads, n_tiles), 128, smem, stream>>>(p, (const int4*)tile_info);
    QIL_CHECK_LAUNCH();
}

// decode_info: int32 [n_decode, 4] = (token, its absolute position, block-table row, 0).
// Scratch: part_o needs n_decode * Hq * n_spans * D floats, part_ml n_decode * Hq * n_spans * 2 floats, tickets
// n_decode * n_kv_heads * ceil(Hq / n_kv_heads / 16) unsigned ints that are zero before the first launch (every
// launch leaves them zero again), or null: then a second kernel merges the spans (what many tokens want: a
// ticket costs every block a fence and an atomic at its end, a merge kernel costs one launch).
// n_spans * span_len must cover the longest context of the batch (max position + 1).
// A negative span_len leaves the length to the kernels (see span_len_of): the fourth int of every decode_info
// entry must then hold the step's longest context, and -span_len is the longest span that may come of it
// (n_spans * -span_len covers the longest context the launch, or a graph recorded from it, will ever see).
static int launch_decode(const void* q, const void* kv, void* out, const int* decode_info, int n_decode,
                         float* part_o, float* part_ml, unsigned* tickets, int n_spans, int span_len,
                         const int* block_table, int table_stride, int n_q_heads, int n_kv_heads,
                         int page_size, int num_pages, int window, float scale, const DecodeTail& tail,
                         cudaStream_t stream) {
    if (n_decode <= 0) return 0;
    AttnParams p;
    if (fill_params(p, q, kv, out, block_table, table_stride, n_q_heads, n_kv_heads, page_size, num_pages,
                    window, scale)) return -1;
    if (check_decode_span(span_len, n_spans)) return -1;
    if (part_o == nullptr || part_ml == nullptr) QIL_REFUSE("attention: decode needs scratch for %d spans", n_spans);
    if ((uintptr_t)decode_info & 15) QIL_REFUSE("attention: decode_info must be 16-byte aligned");
    const int chunks = (n_q_heads / n_kv_heads + 15) / 16;
    if (n_decode > 65535 || n_spans > 65535) QIL_REFUSE("attention: grid too large");
    const int smem = decode_smem_bytes(span_len > 0 ? span_len : -span_len, page_size);
    if (ensure_decode_smem(attn_decode_span_kernel, smem)) return -1;
    qil_launch_chained(attn_decode_span_kernel, dim3(n_kv_heads * chunks, n_decode, n_spans), dim3(128), smem, stream,
                       p, (const int4*)decode_info, part_o, part_ml, tickets, n_spans, span_len, tail);
    if (tickets == nullptr) {
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) { snprintf(qil_error_text, sizeof(qil_error_text), "%s", cudaGetErrorString(e)); return (int)e; }
        qil_launch_chained(attn_decode_merge_kernel, dim3((n_q_heads + 3) / 4, n_decode), dim3(128), 0, stream,
                           p, (const int4*)decode_info, (const float*)part_o, (const float*)part_ml, n_spans, span_len);
    }
    QIL_CHECK_LAUNCH();
}

extern "C" int qil_attn_decode(const void* q, const void* kv, void* out, const int* decode_info, int n_decode,
                               float* part_o, float* part_ml, unsigned* tickets, int n_spans, int span_len,
                               const int* block_table, int table_stride, int n_q_heads, int n_kv_heads,
                               int page_size, int num_pages, int window, float scale, cudaStream_t stream) {
    DecodeTail none = {};
    return launch_decode(q, kv, out, decode_info, n_decode, part_o, part_ml, tickets, n_spans, span_len, block_table,
                         table_stride, n_q_heads, n_kv_heads, page_size, num_pages, window, scale, none, stream);
}

// The same over the raw output of the query/key/value projection, for steps in which every token is a single
// token of its request: qkv [N, (n_q_heads + 2 * own_kv_heads) * D] (queries, keys, values), own_kv_heads
// either n_kv_heads or 0 (a layer that reads another layer's cache).  The kernel norms and rotates the
// queries, and norms, rotates and stores each token's key and value into its page of ``kv`` (see DecodeTail).
// q_norm, k_norm bfloat16 [D] or null; rope float32 [rope_rows, rotary_dim] or null, rotary_dim a multiple
// of 4.  At most 16 query heads per kv head.
extern "C" int qil_attn_decode_qkv(const void* qkv, void* kv, void* out, const int* decode_info, int n_decode,
                                   float* part_o, float* part_ml, unsigned* tickets, int n_spans, int span_len,
                                   const int* block_table, int table_stride, int n_q_heads, int n_kv_heads,
                                   int own_kv_heads, int page_size, int num_pages, int window, float scale,
                                   const void* q_norm, const void* k_norm, float eps, const float* rope,
                                   int rotary_dim, int rope_rows, cudaStream_t stream) {
    if (qkv == nullptr) QIL_REFUSE("attention: the projection's output is missing");
    if (n_kv_heads <= 0 || n_q_heads / n_kv_heads > 16)
        QIL_REFUSE("attention: the fused tail takes at most 16 query heads per kv head");
    if (own_kv_heads != 0 && own_kv_heads != n_kv_heads) QIL_REFUSE("attention: own_kv_heads is %d or 0", n_kv_heads);
    if (rope != nullptr && (rotary_dim < 0 || rotary_dim > D || rotary_dim % 4 || rope_rows <= 0))
        QIL_REFUSE("attention: rotary_dim %d of head size %d, %d table rows", rotary_dim, D, rope_rows);
    if (((uintptr_t)qkv | (uintptr_t)q_norm | (uintptr_t)k_norm) & 3 || ((uintptr_t)rope & 7))
        QIL_REFUSE("attention: the projection, norm weights and rotary table must be aligned to 4 and 8 bytes");
    DecodeTail tail = {};
    tail.qkv = (const bf16*)qkv; tail.q_norm = (const bf16*)q_norm; tail.k_norm = (const bf16*)k_norm;
    tail.rope = rope; tail.kv_out = (bf16*)kv; tail.eps = eps; tail.rotary_dim = rope ? rotary_dim : 0;
    tail.rope_rows = rope_rows; tail.own_kv_heads = own_kv_heads;
    return launch_decode(qkv, kv, out, decode_info, n_decode, part_o, part_ml, tickets, n_spans, span_len, block_table,
                         table_stride, n_q_heads, n_kv_heads, page_size, num_pages, window, scale, tail, stream);
}
