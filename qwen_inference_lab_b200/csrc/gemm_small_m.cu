// out[M,N] = x[M,K] * W[N,K]^T (+ bias) (+ residual), bfloat16 in, float32
// accumulation, for the few rows of a decode step (M <= 16): a weight-streaming
// kernel whose time is the time to read W once from HBM.
//
// Output features sit on the 16-row axis of mma.sync m16n8k16 and tokens on its
// 8-column axis, so nothing is wasted on padding the token count.  Operands go
// from global memory straight to registers as 16-byte vectors: within a run of
// 32 k-values, quad-thread t reads elements 8t..8t+7 of its weight rows and of
// its token's activations and feeds them to two MMAs; the same permutation of k
// on both operands leaves the dot product unchanged.  A block owns 16 output
// features; its warps take interleaved 64-wide slices of K (neighbouring warps
// read neighbouring 128-byte segments of a row) and their partial sums are added
// in shared memory in warp order, so the result is deterministic.
//
// Epilogues: bias, residual (may alias out), float32 output for the LM head,
// and `silu_pairs`: weight rows stored as groups of [8 gate rows, 8 up rows], for
// which the block writes silu(gate) * up, 8 values per token
// (qil/model.py:71; silu(gate) is rounded to bfloat16 before the multiply).
#include "common.cuh"

#define GSM_ROWS 16

__device__ __forceinline__ void gsm_mma(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                        unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 gsm_load(const bf16* p, bool ok) {
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (ok) {
        // weights are read once: do not let them displace the activations in L1
        asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    }
    return v;
}

// One block owns 16 output features; its WARPS warps take interleaved 64-wide slices of K, so that
// the block reads 16 rows x (WARPS x 128) contiguous bytes per sweep.  With 32 warps and K = 4096
// every warp issues all its loads at once: the whole matrix is in flight across the GPU.
template <int NT, int UNROLL, int WARPS>
__global__ void __launch_bounds__(WARPS * 32)
gemm_small_m_kernel(const bf16* __restrict__ x, const bf16* __restrict__ W, const bf16* __restrict__ bias,
                    const bf16* residual, void* out, int M, int N, int K, int out_f32, int silu_pairs) {
    __shared__ float red[WARPS][GSM_ROWS][8 * NT + 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * GSM_ROWS;
    const int row_a = n0 + g, row_b = n0 + g + 8;
    const bool ok_a = row_a < N, ok_b = row_b < N;
    const bf16* wa = W + (size_t)(ok_a ? row_a : 0) * K + 8 * t;
    const bf16* wb = W + (size_t)(ok_b ? row_b : 0) * K + 8 * t;
    const bf16* xp[NT];
    bool ok_x[NT];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        const int token = 8 * j + g;
        ok_x[j] = token < M;
        xp[j] = x + (size_t)(ok_x[j] ? token : 0) * K + 8 * t;
    }
    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

    // 64 k-values per chunk: quad-thread t reads elements 8t..8t+7 and 32+8t..32+8t+7 of each row,
    // so a warp request covers 128 contiguous bytes of every row it touches.
    const int chunks = (K + 63) / 64;
    for (int c0 = warp; c0 < chunks; c0 += WARPS * UNROLL) {
        uint4 va[UNROLL][2], vb[UNROLL][2], vx[UNROLL][NT][2];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int k = (c0 + u * WARPS) * 64;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int kk = k + 32 * h;
                const bool in_k = kk + 8 * t < K;   // K is a multiple of 8: a vector is wholly inside or outside
                va[u][h] = gsm_load(wa + kk, ok_a && in_k);
                vb[u][h] = gsm_load(wb + kk, ok_b && in_k);
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    vx[u][j][h] = make_uint4(0u, 0u, 0u, 0u);
                    if (ok_x[j] && in_k) vx[u][j][h] = *reinterpret_cast<const uint4*>(xp[j] + kk);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    gsm_mma(acc[j], va[u][h].x, vb[u][h].x, va[u][h].y, vb[u][h].y, vx[u][j][h].x, vx[u][j][h].y);
                    gsm_mma(acc[j], va[u][h].z, vb[u][h].z, va[u][h].w, vb[u][h].w, vx[u][j][h].z, vx[u][j][h].w);
                }
            }
        }
    }
    // c0,c1: (feature g, tokens 2t, 2t+1); c2,c3: (feature g+8, same tokens)
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        red[warp][g][8 * j + 2 * t] = acc[j][0];
        red[warp][g][8 * j + 2 * t + 1] = acc[j][1];
        red[warp][g + 8][8 * j + 2 * t] = acc[j][2];
        red[warp][g + 8][8 * j + 2 * t + 1] = acc[j][3];
    }
    __syncthreads();
    if (silu_pairs) {
        // rows 0..7 of the block are gate features, rows 8..15 the matching up features
        const int out_width = N / 2;
        for (int idx = threadIdx.x; idx < 8 * 8 * NT; idx += WARPS * 32) {
            const int token = idx >> 3, r = idx & 7;
            const int col = blockIdx.x * 8 + r;
            if (token >= M || col >= out_width) continue;
            float gate = 0.f, up = 0.f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) { gate += red[w][r][token]; up += red[w][r + 8][token]; }
            gate = round_to<bf16>(gate);
            up = round_to<bf16>(up);
            const float act = round_to<bf16>(gate / (1.0f + expf(-gate)));
            reinterpret_cast<bf16*>(out)[(size_t)token * out_width + col] = __float2bfloat16_rn(act * up);
        }
        return;
    }
    for (int idx = threadIdx.x; idx < GSM_ROWS * 8 * NT; idx += WARPS * 32) {
        const int token = idx / GSM_ROWS, r = idx % GSM_ROWS;
        const int n = n0 + r;
        if (token >= M || n >= N) continue;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) v += red[w][r][token];
        if (bias != nullptr) v += __bfloat162float(bias[n]);
        if (residual != nullptr) v = __bfloat162float(residual[(size_t)token * N + n]) + v;
        if (out_f32) reinterpret_cast<float*>(out)[(size_t)token * N + n] = v;
        else reinterpret_cast<bf16*>(out)[(size_t)token * N + n] = __float2bfloat16_rn(v);
    }
}

template <int NT, int WARPS>
static void gsm_launch(const void* x, const void* W, const void* bias, const void* residual, void* out,
                       int M, int N, int K, int out_f32, int silu_pairs, cudaStream_t stream) {
    const int blocks = (N + GSM_ROWS - 1) / GSM_ROWS;
    gemm_small_m_kernel<NT, 2, WARPS><<<blocks, WARPS * 32, 0, stream>>>(
        (const bf16*)x, (const bf16*)W, (const bf16*)bias, (const bf16*)residual, out, M, N, K, out_f32, silu_pairs);
}

extern "C" int qil_gemm_small_m_max_rows() { return 16; }

extern "C" int qil_gemm_small_m(const void* x, const void* W, const void* bias, const void* residual, void* out,
                                int M, int N, int K, int out_f32, int silu_pairs, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 16) QIL_REFUSE("gemm_small_m: %d rows; this kernel takes at most 16", M);
    if (K <= 0 || K % 8) QIL_REFUSE("gemm_small_m: K %d must be a positive multiple of 8", K);
    if (((uintptr_t)x | (uintptr_t)W) & 15) QIL_REFUSE("gemm_small_m: x and W must be 16-byte aligned");
    if (silu_pairs && (N % 16 || bias != nullptr || residual != nullptr || out_f32))
        QIL_REFUSE("gemm_small_m: silu_pairs needs N %% 16 == 0 and no bias, residual or float32 output");
    // Few output features (o and down projections): 16 warps a block, so that enough loads are in
    // flight although there are few blocks.  Many features: 8 warps a block and several sweeps per
    // warp, which streams best (measured on B200 at K = 4096 and 12288).
    const bool wide = N > 4096 || K < 2048;
    if (M <= 8) {
        if (wide) gsm_launch<1, 8>(x, W, bias, residual, out, M, N, K, out_f32, silu_pairs, stream);
        else gsm_launch<1, 16>(x, W, bias, residual, out, M, N, K, out_f32, silu_pairs, stream);
    } else {
        if (wide) gsm_launch<2, 8>(x, W, bias, residual, out, M, N, K, out_f32, silu_pairs, stream);
        else gsm_launch<2, 16>(x, W, bias, residual, out, M, N, K, out_f32, silu_pairs, stream);
    }
    QIL_CHECK_LAUNCH();
}
