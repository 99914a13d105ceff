// out[M,N] = x[M,K] * W[N,K]^T (+ bias) (+ residual), bfloat16 in, float32
// accumulation, for the few rows of a decode step (M <= 16): a weight-streaming
// kernel whose time is the time to read W once from HBM.
//
// A block owns 16 output features and streams their weight rows through a ring
// of shared-memory stages with cp.async (16 rows x 512 k-values a stage, each row
// segment 1 KB contiguous in memory), so that several stages per block and a few
// blocks per SM keep well over 100 KB in flight per SM.  Output features sit on
// the 16-row axis of mma.sync m16n8k16 and tokens on its 8-column axis, so
// nothing is wasted on padding the token count.  Within a run of 32 k-values,
// quad-thread t takes elements 8t..8t+7 of its weight rows (one 16-byte read
// from shared memory) and of its token's activations (which ride through the
// same ring) and feeds them to two MMAs; the same
// permutation of k on both operands leaves the dot product unchanged.  The four
// warps of a block split every stage's k-range; their partial sums are added in
// shared memory in warp order, so the result is deterministic.
//
// With a norm weight the kernel also does the RMSNorm that precedes the product
// (qil/model.py:21-23,30-31): x arrives un-normed, each element is multiplied by the
// norm weight on its way into the MMA (one bfloat16 rounding), the squares of x are
// summed in float32 alongside (as the diagonal of X X^T, two more MMAs per 32 k-values),
// and the accumulators are scaled by rsqrt(mean(x^2) + eps) in the epilogue.  The norm weight rides through the ring as
// one more stage row.
//
// Epilogues: bias, residual (may alias out), float32 output for the LM head,
// and `silu_pairs`: weight rows stored as groups of [8 gate rows, 8 up rows], for
// which the block writes silu(gate) * up, 8 values per token
// (qil/model.py:71; silu(gate) is rounded to bfloat16 before the multiply).
#include "common.cuh"

#define GSM_ROWS 16
#ifndef GSM_WARPS
#define GSM_WARPS 4
#endif
#define GSM_THREADS (GSM_WARPS * 32)
#define GSM_PASS_ROWS (GSM_THREADS / 64)     // stage rows one pass of all threads copies
#define GSM_RUNS (GSM_STAGE_K / GSM_WARPS / 32)   // runs of 32 k-values per warp and stage
#define GSM_STAGE_K 512                    // k-values per stage
#define GSM_STAGES 4
#define GSM_L2_AHEAD 2048                  // bytes of each weight row that a waiting block asks L2 for beyond its ring
#define GSM_ROW_BYTES (GSM_STAGE_K * 2 + 64)   // row stride = 64 mod 128 bytes: 16-byte reads of 8 rows x 4 pieces hit every bank once
#define GSM_STAGE_BYTES (GSM_ROWS * GSM_ROW_BYTES)

__device__ __forceinline__ void gsm_mma(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                        unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Queueing a stage.  64 pieces of 16 bytes a row, GSM_PASS_ROWS rows per pass of all threads: thread
// `tid` always copies piece `tid & 63` of rows `GSM_PASS_ROWS * i + (tid >> 6)`, so a warp request covers 512 contiguous bytes of
// one row, and everything but the k-offset is the same for every stage.
struct GsmCopy {
    const bf16* W; const bf16* x;
    const bf16* w;      // W + (n0 + (tid >> 6)) * K + (tid & 63) * 8   (short path)
    const bf16* xs;     // x + (tid >> 6) * K + (tid & 63) * 8
    unsigned ring;      // shared address of the ring
    unsigned dst;       // ring + (tid >> 6) * ROW_BYTES + (tid & 63) * 16
    int n0, N, M, K, tid;
    bool short_path;    // all 16 weight rows of the block exist
};

// Weights are read once a step and there are far more of them than L2 holds: their copies carry the policy
// "first to leave L2", so that what is read again (activations, partial sums, tables) stays.  Measured on the
// Qwen3-8B decode step, together with the same hint on the single-token attention's keys and values: 4.65 -> 4.61 ms
// at batch 8, 3.24 -> 3.21 at batch 1.
__device__ __forceinline__ unsigned long long gsm_stream_policy() {
    unsigned long long policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;\n" : "=l"(policy));
    return policy;
}
__device__ __forceinline__ void gsm_cp16_stream(unsigned dst, const void* src, unsigned long long policy) {
    asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "l"(policy));
}
__device__ __forceinline__ void gsm_cp16_zfill_stream(unsigned dst, const void* src, bool valid, unsigned long long policy) {
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2, %3;\n" ::"r"(dst), "l"(src), "r"(bytes), "l"(policy));
}
__device__ __forceinline__ void gsm_cp16(unsigned dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src));
}

__device__ __forceinline__ void gsm_cp16_zfill(unsigned dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;       // 0: zero-fill
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes));
}

// Rows FIRST..LAST-1 of a stage (0..15 weights, 16.. activations of tokens 0..), k-values k0..k0+511.
// A stage wholly inside K of a block with all its weight rows takes the short path: straight-line
// copies from one base pointer plus multiples of the row stride.  Everything else (the last, partial
// stage, whose tail must be zero because it enters the sums; the last block of an N that is no
// multiple of 16) takes the general path, which zero-fills what does not exist.
template <int FIRST_ROW, int LAST_ROW>
__device__ __forceinline__ void gsm_issue_rows(const GsmCopy& c, unsigned stage_offset, int k0) {
    if (c.short_path && k0 + GSM_STAGE_K <= c.K) {
        const bf16* w = c.w + k0;
        const bf16* xs = c.xs + k0;
        const unsigned dst = c.dst + stage_offset;
        const int half = c.tid >> 6;
#pragma unroll
        for (int row2 = FIRST_ROW; row2 < LAST_ROW; row2 += GSM_PASS_ROWS) {
            if (row2 < GSM_ROWS) {
                gsm_cp16_stream(dst + row2 * GSM_ROW_BYTES, w + (size_t)row2 * c.K, gsm_stream_policy());
            } else if (row2 - GSM_ROWS + half < c.M) {    // a token past M feeds only its own, unwritten column
                gsm_cp16(dst + row2 * GSM_ROW_BYTES, xs + (size_t)(row2 - GSM_ROWS) * c.K);
            }
        }
        return;
    }
#pragma unroll
    for (int i = FIRST_ROW * 64 / GSM_THREADS; i < LAST_ROW * 64 / GSM_THREADS; ++i) {
        const int idx = i * GSM_THREADS + c.tid;
        const int row = idx >> 6, piece = idx & 63;
        const int k = k0 + piece * 8;
        const bool is_w = row < GSM_ROWS;
        const int src_row = is_w ? c.n0 + row : row - GSM_ROWS;
        const bool valid = (k < c.K) && (is_w ? src_row < c.N : src_row < c.M);   // K is a multiple of 8
        const bf16* src = (is_w ? c.W : c.x) + (size_t)(valid ? src_row : 0) * c.K + (valid ? k : 0);
        if (is_w) gsm_cp16_zfill_stream(c.ring + stage_offset + row * GSM_ROW_BYTES + piece * 16, src, valid, gsm_stream_policy());
        else gsm_cp16_zfill(c.ring + stage_offset + row * GSM_ROW_BYTES + piece * 16, src, valid);
    }
}

// The norm weight's k-values k0..k0+511 into a stage row of their own (64 pieces of 16 bytes).
__device__ __forceinline__ void gsm_issue_norm_row(const bf16* __restrict__ norm_w, unsigned row_dst, int K, int k0,
                                                   int tid) {
    if (tid < 64) {
        const int k = k0 + tid * 8;
        const bool valid = k < K;
        gsm_cp16_zfill(row_dst + tid * 16, norm_w + (valid ? k : 0), valid);
    }
}

__device__ __forceinline__ unsigned gsm_mul2(unsigned a, unsigned b) {
    const __nv_bfloat162 r = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
    return *reinterpret_cast<const unsigned*>(&r);
}

// NT: token tiles of 8.  NORM = 1: fused RMSNorm (see the top of the file).  The activations travel through the
// ring with the weights: reading them from global memory in the threads that need them was slower at every
// token count, because those reads miss the small L1 left beside the ring and stall the warp.
template <int NT, int NORM>
__global__ void __launch_bounds__(GSM_WARPS * 32)
gemm_small_m_kernel(const bf16* __restrict__ x, const bf16* __restrict__ W, const bf16* __restrict__ bias,
                    const bf16* residual, void* out, const bf16* __restrict__ norm_w, float norm_eps,
                    int M, int N, int K, int out_f32, int silu_pairs, int first_wave) {
    extern __shared__ __align__(128) unsigned char ring[];          // [STAGES][STAGE_BYTES]
    constexpr int XROWS = 8 * NT;
    constexpr int NORM_ROW = GSM_ROWS + XROWS;                      // the stage row of the norm weight
    constexpr int STAGE_BYTES = (GSM_ROWS + XROWS + NORM) * GSM_ROW_BYTES;
    constexpr int STAGES = NT == 2 ? 3 : GSM_STAGES;
    __shared__ float red[GSM_WARPS][GSM_ROWS][8 * NT + 1];
    __shared__ float squares[GSM_WARPS][8 * NT];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * GSM_ROWS;
    const int stages_total = (K + GSM_STAGE_K - 1) / GSM_STAGE_K;
    GsmCopy copy;
    copy.W = W; copy.x = x; copy.n0 = n0; copy.N = N; copy.M = M; copy.K = K; copy.tid = tid;
    copy.short_path = n0 + GSM_ROWS <= N;
    copy.w = W + (size_t)(copy.short_path ? n0 + (tid >> 6) : 0) * K + (tid & 63) * 8;
    copy.xs = x + (size_t)((tid >> 6) < M ? (tid >> 6) : 0) * K + (tid & 63) * 8;
    copy.ring = (unsigned)__cvta_generic_to_shared(ring);
    copy.dst = copy.ring + (tid >> 6) * GSM_ROW_BYTES + (tid & 63) * 16;
    const unsigned ring_address = copy.ring;

    // Weights do not depend on the kernel before this one: their first stages are requested before the
    // wait for that kernel, the activations (its output) right after.  Groups: W0..W(S-2), X0..X(S-2),
    // then one group per later stage; "at most S-2 groups pending" still means "stage s has landed".
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < stages_total) {
            gsm_issue_rows<0, GSM_ROWS>(copy, s * STAGE_BYTES, s * GSM_STAGE_K);
            if (NORM) gsm_issue_norm_row(norm_w, ring_address + s * STAGE_BYTES + NORM_ROW * GSM_ROW_BYTES, K,
                                         s * GSM_STAGE_K, tid);
        }
        asm volatile("cp.async.commit_group;\n" ::);
    }
    // While a block of the first wave waits for the kernel before it, L2 can fetch a little more of its
    // weight rows than the ring holds (lane r of warp 0 asks for the next GSM_L2_AHEAD bytes of row r), so the
    // memory system has work while that kernel drains.  Measured on the Qwen3-8B decode step: 1 % of the step
    // with 1 to 2 KB a row, nothing with 3 KB, a loss from 5 KB on and when later waves do it too.
    if (warp == 0 && lane < GSM_ROWS && (int)blockIdx.x < first_wave && copy.short_path) {
        const long long begin = (long long)(STAGES - 1) * GSM_STAGE_K * 2;
        long long bytes = (long long)K * 2 - begin;
        if (bytes > GSM_L2_AHEAD) bytes = GSM_L2_AHEAD;
        bytes &= ~15ll;
        if (bytes > 0) {
            const char* row = reinterpret_cast<const char*>(W + (size_t)(n0 + lane) * K) + begin;
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" ::"l"(row), "r"((unsigned)bytes) : "memory");
        }
    }
    qil_wait_for_producer();
    qil_release_consumer();
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < stages_total)
            gsm_issue_rows<GSM_ROWS, GSM_ROWS + XROWS>(copy, s * STAGE_BYTES, s * GSM_STAGE_K);
        asm volatile("cp.async.commit_group;\n" ::);
    }

    float acc[NT][4];
    // With the norm: X X^T of the token tile on the tensor cores, of which the diagonal is each token's
    // sum of squares (products of bfloat16 values are exact in float32, the sums are float32).
    float gram[NORM ? NT : 1][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
        if (NORM) gram[j][0] = gram[j][1] = gram[j][2] = gram[j][3] = 0.f;
    }

    for (int s = 0; s < stages_total; ++s) {
        // stage s has landed once at most STAGES-2 newer groups are still in flight
        asm volatile("cp.async.wait_group %0;\n" ::"n"(STAGES - 2));
        __syncthreads();            // visible to all; everyone is also done with stage s-1's buffer
        {
            const int next = s + STAGES - 1;
            if (next < stages_total) {
                const unsigned offset = (next % STAGES) * STAGE_BYTES;
                gsm_issue_rows<0, GSM_ROWS + XROWS>(copy, offset, next * GSM_STAGE_K);
                if (NORM) gsm_issue_norm_row(norm_w, ring_address + offset + NORM_ROW * GSM_ROW_BYTES, K,
                                             next * GSM_STAGE_K, tid);
            }
            asm volatile("cp.async.commit_group;\n" ::);
        }
        const unsigned char* stage = ring + (s % STAGES) * STAGE_BYTES;
        // this warp's share of the stage: GSM_RUNS runs of 32 k-values
        const int kw = warp * (GSM_STAGE_K / GSM_WARPS);
        uint4 vx[GSM_RUNS][NT];
#pragma unroll
        for (int r = 0; r < GSM_RUNS; ++r) {
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                vx[r][j] = *reinterpret_cast<const uint4*>(stage + (GSM_ROWS + 8 * j + g) * GSM_ROW_BYTES
                                                           + (kw + r * 32 + 8 * t) * 2);
            }
            if (NORM) {
                const uint4 vn = *reinterpret_cast<const uint4*>(stage + NORM_ROW * GSM_ROW_BYTES + (kw + r * 32 + 8 * t) * 2);
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    // the activations as both operands: rows = tokens 8j..8j+7 (rows 8..15 of the tile are zero)
                    gsm_mma(gram[j], vx[r][j].x, 0u, vx[r][j].y, 0u, vx[r][j].x, vx[r][j].y);
                    gsm_mma(gram[j], vx[r][j].z, 0u, vx[r][j].w, 0u, vx[r][j].z, vx[r][j].w);
                    vx[r][j] = make_uint4(gsm_mul2(vx[r][j].x, vn.x), gsm_mul2(vx[r][j].y, vn.y),
                                          gsm_mul2(vx[r][j].z, vn.z), gsm_mul2(vx[r][j].w, vn.w));
                }
            }
        }
#pragma unroll
        for (int r = 0; r < GSM_RUNS; ++r) {
            const int byte = (kw + r * 32 + 8 * t) * 2;
            const uint4 va = *reinterpret_cast<const uint4*>(stage + g * GSM_ROW_BYTES + byte);
            const uint4 vb = *reinterpret_cast<const uint4*>(stage + (g + 8) * GSM_ROW_BYTES + byte);
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                gsm_mma(acc[j], va.x, vb.x, va.y, vb.y, vx[r][j].x, vx[r][j].y);
                gsm_mma(acc[j], va.z, vb.z, va.w, vb.w, vx[r][j].z, vx[r][j].w);
            }
        }
    }
    asm volatile("cp.async.wait_group 0;\n" ::);
    // c0,c1: (feature g, tokens 2t, 2t+1); c2,c3: (feature g+8, same tokens)
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        red[warp][g][8 * j + 2 * t] = acc[j][0];
        red[warp][g][8 * j + 2 * t + 1] = acc[j][1];
        red[warp][g + 8][8 * j + 2 * t] = acc[j][2];
        red[warp][g + 8][8 * j + 2 * t + 1] = acc[j][3];
        // gram[j][0..1] are entries (g, 2t) and (g, 2t + 1): the diagonal one belongs to thread t == g / 2
        if (NORM && t == (g >> 1)) squares[warp][8 * j + g] = (g & 1) ? gram[j][1] : gram[j][0];
    }
    __syncthreads();
    // 1 / rms of a token's activations, the warps' partial sums added in warp order
    auto inverse_rms = [&](int token) {
        if (!NORM) return 1.f;
        float total = 0.f;
#pragma unroll
        for (int w = 0; w < GSM_WARPS; ++w) total += squares[w][token];
        return rsqrtf(total / (float)K + norm_eps);
    };
    if (silu_pairs) {
        // rows 0..7 of the block are gate features, rows 8..15 the matching up features
        const int out_width = N / 2;
        for (int idx = tid; idx < 8 * 8 * NT; idx += GSM_WARPS * 32) {
            const int token = idx >> 3, r = idx & 7;
            const int col = blockIdx.x * 8 + r;
            if (token >= M || col >= out_width) continue;
            float gate = 0.f, up = 0.f;
#pragma unroll
            for (int w = 0; w < GSM_WARPS; ++w) { gate += red[w][r][token]; up += red[w][r + 8][token]; }
            const float scale = inverse_rms(token);
            gate = round_to<bf16>(gate * scale);
            up = round_to<bf16>(up * scale);
            const float act = round_to<bf16>(__fdividef(gate, 1.0f + __expf(-gate)));   // as the stand-alone bfloat16 kernel
            reinterpret_cast<bf16*>(out)[(size_t)token * out_width + col] = __float2bfloat16_rn(act * up);
        }
        return;
    }
    for (int idx = tid; idx < GSM_ROWS * 8 * NT; idx += GSM_WARPS * 32) {
        const int token = idx / GSM_ROWS, r = idx % GSM_ROWS;
        const int n = n0 + r;
        if (token >= M || n >= N) continue;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < GSM_WARPS; ++w) v += red[w][r][token];
        v *= inverse_rms(token);
        if (bias != nullptr) v += __bfloat162float(bias[n]);
        if (residual != nullptr) v = __bfloat162float(residual[(size_t)token * N + n]) + v;
        if (out_f32) reinterpret_cast<float*>(out)[(size_t)token * N + n] = v;
        else reinterpret_cast<bf16*>(out)[(size_t)token * N + n] = __float2bfloat16_rn(v);
    }
}

// ------------------------------------------------------------------ 32 output features a block
// The same product with two 16-row weight tiles per block and stages of 256 k-values (row segments of 512 bytes).
// A run's activation fragments, the norm weight's multiply and the two MMAs for the rows' sums of squares then serve
// 32 output features instead of 16, so the instructions per weight byte drop by about a third (the kernel above
// is bound by its instruction stream once the norm is inside), and weights are 78 % of what goes through the ring
// instead of 64 %.  Whole blocks only (N a multiple of 32); the last, partial stage is zero-filled as above.
#define GW_ROWS 32
#define GW_STAGE_K 256
#define GW_STAGES 4
#define GW_PIECES (GW_STAGE_K / 8)                 // 16-byte pieces a row segment
#define GW_PASS_ROWS (GSM_THREADS / GW_PIECES)     // rows one pass of all threads copies
#define GW_RUNS (GW_STAGE_K / GSM_WARPS / 32)      // runs of 32 k-values per warp and stage
#define GW_ROW_BYTES (GW_STAGE_K * 2 + 64)         // 576: again 64 mod 128

// Rows [FIRST, LAST) of a stage: thread tid copies piece tid % 32 of rows FIRST + i * 4 + tid / 32.
template <int FIRST_ROW, int LAST_ROW>
__device__ __forceinline__ void gw_issue_rows(const bf16* __restrict__ W, const bf16* __restrict__ x, unsigned ring,
                                              unsigned stage_offset, int n0, int M, int K, int k0, int tid) {
    const int piece = tid % GW_PIECES, sub = tid / GW_PIECES;
    const int k = k0 + piece * 8;
    const bool in_k = k < K;                      // K is a multiple of 8
#pragma unroll
    for (int row = FIRST_ROW + sub; row < LAST_ROW; row += GW_PASS_ROWS) {
        const bool is_w = row < GW_ROWS;
        const int src_row = is_w ? n0 + row : row - GW_ROWS;
        if (!is_w && src_row >= M) continue;     // a token past M feeds only its own, unwritten column
        const bf16* src = (is_w ? W : x) + (size_t)src_row * K + (in_k ? k : 0);
        if (is_w) gsm_cp16_zfill_stream(ring + stage_offset + row * GW_ROW_BYTES + piece * 16, src, in_k, gsm_stream_policy());
        else gsm_cp16_zfill(ring + stage_offset + row * GW_ROW_BYTES + piece * 16, src, in_k);
    }
}

template <int NT, int NORM>
__global__ void __launch_bounds__(GSM_THREADS)
gemm_small_m_wide_kernel(const bf16* __restrict__ x, const bf16* __restrict__ W, const bf16* __restrict__ bias,
                         const bf16* residual, void* out, const bf16* __restrict__ norm_w, float norm_eps,
                         int M, int N, int K, int out_f32, int silu_pairs, int first_wave) {
    extern __shared__ __align__(128) unsigned char ring[];
    constexpr int XROWS = 8 * NT;
    constexpr int NORM_ROW = GW_ROWS + XROWS;
    constexpr int STAGE_BYTES = (GW_ROWS + XROWS + NORM) * GW_ROW_BYTES;
    constexpr int STAGES = NT == 2 ? GW_STAGES - 1 : GW_STAGES;     // two blocks an SM either way
    __shared__ float red[GSM_WARPS][GW_ROWS][8 * NT + 1];
    __shared__ float squares[GSM_WARPS][8 * NT];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * GW_ROWS;
    const int stages_total = (K + GW_STAGE_K - 1) / GW_STAGE_K;
    const unsigned ring_address = (unsigned)__cvta_generic_to_shared(ring);
    auto issue_norm = [&](unsigned offset, int k0) {
        if (NORM && tid < GW_PIECES) {
            const int k = k0 + tid * 8;
            const bool valid = k < K;
            gsm_cp16_zfill(ring_address + offset + NORM_ROW * GW_ROW_BYTES + tid * 16, norm_w + (valid ? k : 0), valid);
        }
    };
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < stages_total) {
            gw_issue_rows<0, GW_ROWS>(W, x, ring_address, s * STAGE_BYTES, n0, M, K, s * GW_STAGE_K, tid);
            issue_norm(s * STAGE_BYTES, s * GW_STAGE_K);
        }
        asm volatile("cp.async.commit_group;\n" ::);
    }
    if (warp == 0 && (int)blockIdx.x < first_wave) {     // see the kernel above: a little more of each row into L2
        const long long begin = (long long)(STAGES - 1) * GW_STAGE_K * 2;
        long long bytes = (long long)K * 2 - begin;
        if (bytes > GSM_L2_AHEAD / 2) bytes = GSM_L2_AHEAD / 2;
        bytes &= ~15ll;
        if (bytes > 0) {
            const char* row = reinterpret_cast<const char*>(W + (size_t)(n0 + lane) * K) + begin;
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" ::"l"(row), "r"((unsigned)bytes) : "memory");
        }
    }
    qil_wait_for_producer();
    qil_release_consumer();
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < stages_total)
            gw_issue_rows<GW_ROWS, GW_ROWS + XROWS>(W, x, ring_address, s * STAGE_BYTES, n0, M, K, s * GW_STAGE_K, tid);
        asm volatile("cp.async.commit_group;\n" ::);
    }
    float acc[2][NT][4];
    float gram[NORM ? NT : 1][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
#pragma unroll
        for (int rt = 0; rt < 2; ++rt) acc[rt][j][0] = acc[rt][j][1] = acc[rt][j][2] = acc[rt][j][3] = 0.f;
        if (NORM) gram[j][0] = gram[j][1] = gram[j][2] = gram[j][3] = 0.f;
    }
    for (int s = 0; s < stages_total; ++s) {
        asm volatile("cp.async.wait_group %0;\n" ::"n"(STAGES - 2));
        __syncthreads();
        {
            const int next = s + STAGES - 1;
            if (next < stages_total) {
                const unsigned offset = (next % STAGES) * STAGE_BYTES;
                gw_issue_rows<0, GW_ROWS + XROWS>(W, x, ring_address, offset, n0, M, K, next * GW_STAGE_K, tid);
                issue_norm(offset, next * GW_STAGE_K);
            }
            asm volatile("cp.async.commit_group;\n" ::);
        }
        const unsigned char* stage = ring + (s % STAGES) * STAGE_BYTES;
        const int kw = warp * (GW_STAGE_K / GSM_WARPS);
#pragma unroll
        for (int r = 0; r < GW_RUNS; ++r) {
            const int byte = (kw + r * 32 + 8 * t) * 2;
            uint4 vx[NT];
#pragma unroll
            for (int j = 0; j < NT; ++j)
                vx[j] = *reinterpret_cast<const uint4*>(stage + (GW_ROWS + 8 * j + g) * GW_ROW_BYTES + byte);
            if (NORM) {
                const uint4 vn = *reinterpret_cast<const uint4*>(stage + NORM_ROW * GW_ROW_BYTES + byte);
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    gsm_mma(gram[j], vx[j].x, 0u, vx[j].y, 0u, vx[j].x, vx[j].y);
                    gsm_mma(gram[j], vx[j].z, 0u, vx[j].w, 0u, vx[j].z, vx[j].w);
                    vx[j] = make_uint4(gsm_mul2(vx[j].x, vn.x), gsm_mul2(vx[j].y, vn.y),
                                       gsm_mul2(vx[j].z, vn.z), gsm_mul2(vx[j].w, vn.w));
                }
            }
#pragma unroll
            for (int rt = 0; rt < 2; ++rt) {
                const uint4 va = *reinterpret_cast<const uint4*>(stage + (16 * rt + g) * GW_ROW_BYTES + byte);
                const uint4 vb = *reinterpret_cast<const uint4*>(stage + (16 * rt + g + 8) * GW_ROW_BYTES + byte);
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    gsm_mma(acc[rt][j], va.x, vb.x, va.y, vb.y, vx[j].x, vx[j].y);
                    gsm_mma(acc[rt][j], va.z, vb.z, va.w, vb.w, vx[j].z, vx[j].w);
                }
            }
        }
    }
    asm volatile("cp.async.wait_group 0;\n" ::);
#pragma unroll
    for (int j = 0; j < NT; ++j) {
#pragma unroll
        for (int rt = 0; rt < 2; ++rt) {
            red[warp][16 * rt + g][8 * j + 2 * t] = acc[rt][j][0];
            red[warp][16 * rt + g][8 * j + 2 * t + 1] = acc[rt][j][1];
            red[warp][16 * rt + g + 8][8 * j + 2 * t] = acc[rt][j][2];
            red[warp][16 * rt + g + 8][8 * j + 2 * t + 1] = acc[rt][j][3];
        }
        if (NORM && t == (g >> 1)) squares[warp][8 * j + g] = (g & 1) ? gram[j][1] : gram[j][0];
    }
    __syncthreads();
    auto inverse_rms = [&](int token) {
        if (!NORM) return 1.f;
        float total = 0.f;
#pragma unroll
        for (int w = 0; w < GSM_WARPS; ++w) total += squares[w][token];
        return rsqrtf(total / (float)K + norm_eps);
    };
    if (silu_pairs) {
        // each 16-row tile holds 8 gate features (rows 0..7) and the matching 8 up features (rows 8..15)
        const int out_width = N / 2;
        for (int idx = tid; idx < 2 * 8 * 8 * NT; idx += GSM_THREADS) {
            const int r = idx & 7, rt = (idx >> 3) & 1, token = idx >> 4;
            const int col = (blockIdx.x * 2 + rt) * 8 + r;
            if (token >= M || col >= out_width) continue;
            float gate = 0.f, up = 0.f;
#pragma unroll
            for (int w = 0; w < GSM_WARPS; ++w) { gate += red[w][16 * rt + r][token]; up += red[w][16 * rt + r + 8][token]; }
            const float scale = inverse_rms(token);
            gate = round_to<bf16>(gate * scale);
            up = round_to<bf16>(up * scale);
            const float act = round_to<bf16>(__fdividef(gate, 1.0f + __expf(-gate)));
            reinterpret_cast<bf16*>(out)[(size_t)token * out_width + col] = __float2bfloat16_rn(act * up);
        }
        return;
    }
    for (int idx = tid; idx < GW_ROWS * 8 * NT; idx += GSM_THREADS) {
        const int token = idx / GW_ROWS, r = idx % GW_ROWS;
        const int n = n0 + r;
        if (token >= M || n >= N) continue;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < GSM_WARPS; ++w) v += red[w][r][token];
        v *= inverse_rms(token);
        if (bias != nullptr) v += __bfloat162float(bias[n]);
        if (residual != nullptr) v = __bfloat162float(residual[(size_t)token * N + n]) + v;
        if (out_f32) reinterpret_cast<float*>(out)[(size_t)token * N + n] = v;
        else reinterpret_cast<bf16*>(out)[(size_t)token * N + n] = __float2bfloat16_rn(v);
    }
}

extern "C" int qil_gemm_small_m_max_rows() { return 16; }

// norm_w: null, or the K weights of the RMSNorm to apply to x first (with norm_eps).
extern "C" int qil_gemm_small_m(const void* x, const void* W, const void* bias, const void* residual, void* out,
                                const void* norm_w, float norm_eps, int M, int N, int K, int out_f32, int silu_pairs,
                                int rows_per_block, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (rows_per_block != 16 && rows_per_block != 32) QIL_REFUSE("gemm_small_m: %d output features a block; 16 or 32", rows_per_block);
    if (rows_per_block == 32 && N % 32) QIL_REFUSE("gemm_small_m: 32 output features a block need N %% 32 == 0, got %d", N);
    if (M > 16) QIL_REFUSE("gemm_small_m: %d rows; this kernel takes at most 16", M);
    if (K <= 0 || K % 8) QIL_REFUSE("gemm_small_m: K %d must be a positive multiple of 8", K);
    if (((uintptr_t)x | (uintptr_t)W | (uintptr_t)norm_w) & 15)
        QIL_REFUSE("gemm_small_m: x, W and the norm weight must be 16-byte aligned");
    if (silu_pairs && (N % 16 || bias != nullptr || residual != nullptr || out_f32))
        QIL_REFUSE("gemm_small_m: silu_pairs needs N %% 16 == 0 and no bias, residual or float32 output");
    const int blocks = (N + GSM_ROWS - 1) / GSM_ROWS;
    const int smem1 = GSM_STAGES * (GSM_ROWS + 8) * GSM_ROW_BYTES, smem1n = GSM_STAGES * (GSM_ROWS + 8 + 1) * GSM_ROW_BYTES;
    const int smem2 = 3 * (GSM_ROWS + 16) * GSM_ROW_BYTES, smem2n = 3 * (GSM_ROWS + 16 + 1) * GSM_ROW_BYTES;
    static bool configured = false;
    static int first_wave = 0;          // blocks that run at once: two a multiprocessor
    if (!configured) {
        int device = 0, sms = 0;
        if (cudaGetDevice(&device) == cudaSuccess &&
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) == cudaSuccess) first_wave = 2 * sms;
        cudaError_t e[4] = {
            cudaFuncSetAttribute(gemm_small_m_kernel<1, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem1),
            cudaFuncSetAttribute(gemm_small_m_kernel<2, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem2),
            cudaFuncSetAttribute(gemm_small_m_kernel<1, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem1n),
            cudaFuncSetAttribute(gemm_small_m_kernel<2, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem2n)};
        for (int i = 0; i < 4; ++i)
            if (e[i] != cudaSuccess) QIL_REFUSE("gemm_small_m: cannot reserve %d bytes of shared memory", smem1n);
        configured = true;
    }
    if (rows_per_block == 32) {
        const int w1 = GW_STAGES * (GW_ROWS + 8) * GW_ROW_BYTES, w1n = GW_STAGES * (GW_ROWS + 8 + 1) * GW_ROW_BYTES;
        const int w2 = (GW_STAGES - 1) * (GW_ROWS + 16) * GW_ROW_BYTES, w2n = (GW_STAGES - 1) * (GW_ROWS + 16 + 1) * GW_ROW_BYTES;
        static bool wide_configured = false;
        if (!wide_configured) {
            cudaError_t e[4] = {
                cudaFuncSetAttribute(gemm_small_m_wide_kernel<1, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, w1),
                cudaFuncSetAttribute(gemm_small_m_wide_kernel<2, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, w2),
                cudaFuncSetAttribute(gemm_small_m_wide_kernel<1, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, w1n),
                cudaFuncSetAttribute(gemm_small_m_wide_kernel<2, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, w2n)};
            for (int i = 0; i < 4; ++i)
                if (e[i] != cudaSuccess) QIL_REFUSE("gemm_small_m: cannot reserve %d bytes of shared memory", w2n);
            wide_configured = true;
        }
#define GW_LAUNCH(NT, NORM, SMEM)                                                                                   \
        qil_launch_chained(gemm_small_m_wide_kernel<NT, NORM>, dim3(N / GW_ROWS), dim3(GSM_THREADS), SMEM, stream,  \
                           (const bf16*)x, (const bf16*)W, (const bf16*)bias, (const bf16*)residual, out,            \
                           (const bf16*)norm_w, norm_eps, M, N, K, out_f32, silu_pairs, first_wave)
        if (norm_w == nullptr) {
            if (M <= 8) GW_LAUNCH(1, 0, w1); else GW_LAUNCH(2, 0, w2);
        } else {
            if (M <= 8) GW_LAUNCH(1, 1, w1n); else GW_LAUNCH(2, 1, w2n);
        }
#undef GW_LAUNCH
        QIL_CHECK_LAUNCH();
    }
#define GSM_LAUNCH(NT, NORM, SMEM)                                                                                  \
    qil_launch_chained(gemm_small_m_kernel<NT, NORM>, dim3(blocks), dim3(GSM_WARPS * 32), SMEM, stream,           \
                       (const bf16*)x, (const bf16*)W, (const bf16*)bias, (const bf16*)residual, out,                \
                       (const bf16*)norm_w, norm_eps, M, N, K, out_f32, silu_pairs, first_wave)
    if (norm_w == nullptr) {
        if (M <= 8) GSM_LAUNCH(1, 0, smem1); else GSM_LAUNCH(2, 0, smem2);
    } else {
        if (M <= 8) GSM_LAUNCH(1, 1, smem1n); else GSM_LAUNCH(2, 1, smem2n);
    }
#undef GSM_LAUNCH
    QIL_CHECK_LAUNCH();
}
