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
// Epilogues: bias, residual (may alias out), float32 output for the LM head,
// and `silu_pairs`: weight rows stored as groups of [8 gate rows, 8 up rows], for
// which the block writes silu(gate) * up, 8 values per token
// (qil/model.py:71; silu(gate) is rounded to bfloat16 before the multiply).
#include "common.cuh"

#define GSM_ROWS 16
#define GSM_WARPS 4
#define GSM_STAGE_K 512                    // k-values per stage
#define GSM_STAGES 4
#define GSM_ROW_BYTES (GSM_STAGE_K * 2 + 64)   // row stride = 64 mod 128 bytes: 16-byte reads of 8 rows x 4 pieces hit every bank once
#define GSM_STAGE_BYTES (GSM_ROWS * GSM_ROW_BYTES)

__device__ __forceinline__ void gsm_mma(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                        unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void gsm_cp_async16(void* smem, const void* gmem, bool valid) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem);
    const int bytes = valid ? 16 : 0;       // 0: zero-fill
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gmem), "r"(bytes));
}

// Queue one stage: weight rows n0..n0+15 and, when XROWS > 0, the activations of tokens 0..XROWS-1
// (stage rows 16..), k-values k0..k0+511.  128 threads, 64 pieces of 16 bytes a row: a warp request
// covers 512 contiguous bytes of one row.
// FIRST_ROW..LAST_ROW select weight rows (0..15), activation rows (16..) or both.
template <int FIRST_ROW, int LAST_ROW>
__device__ __forceinline__ void gsm_issue_stage(const bf16* __restrict__ W, const bf16* __restrict__ x,
                                                unsigned char* stage, int n0, int N, int M, int K, int k0, int tid) {
#pragma unroll
    for (int i = FIRST_ROW * 64 / 128; i < LAST_ROW * 64 / 128; ++i) {
        const int idx = i * 128 + tid;
        const int row = idx >> 6, piece = idx & 63;
        const int k = k0 + piece * 8;
        const bool is_w = row < GSM_ROWS;
        const int src_row = is_w ? n0 + row : row - GSM_ROWS;
        const bool valid = (k < K) && (is_w ? src_row < N : src_row < M);   // K is a multiple of 8
        const bf16* src = (is_w ? W : x) + (size_t)(valid ? src_row : 0) * K + (valid ? k : 0);
        gsm_cp_async16(stage + row * GSM_ROW_BYTES + piece * 16, src, valid);
    }
}

// NT: token tiles of 8.  XS = 1: activations travel through the ring with the weights.  (XS = 0 reads
// them from global memory in the threads that need them; measured slower at every token count, because
// those reads miss the small L1 left beside the ring and stall the warp.  Kept for comparison.)
template <int NT, int XS>
__global__ void __launch_bounds__(GSM_WARPS * 32)
gemm_small_m_kernel(const bf16* __restrict__ x, const bf16* __restrict__ W, const bf16* __restrict__ bias,
                    const bf16* residual, void* out, int M, int N, int K, int out_f32, int silu_pairs) {
    extern __shared__ __align__(128) unsigned char ring[];          // [STAGES][STAGE_BYTES]
    constexpr int XROWS = XS ? 8 * NT : 0;
    constexpr int STAGE_BYTES = (GSM_ROWS + XROWS) * GSM_ROW_BYTES;
    constexpr int STAGES = (XS && NT == 2) ? 3 : GSM_STAGES;
    __shared__ float red[GSM_WARPS][GSM_ROWS][8 * NT + 1];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * GSM_ROWS;
    const int stages_total = (K + GSM_STAGE_K - 1) / GSM_STAGE_K;

    // Weights do not depend on the kernel before this one: their first stages are requested before the
    // wait for that kernel, the activations (its output) right after.  Groups: W0..W(S-2), X0..X(S-2),
    // then one group per later stage; "at most S-2 groups pending" still means "stage s has landed".
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < stages_total)
            gsm_issue_stage<0, GSM_ROWS>(W, x, ring + s * STAGE_BYTES, n0, N, M, K, s * GSM_STAGE_K, tid);
        asm volatile("cp.async.commit_group;\n" ::);
    }
    qil_wait_for_producer();
    qil_release_consumer();
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (XS && s < stages_total)
            gsm_issue_stage<GSM_ROWS, GSM_ROWS + XROWS>(W, x, ring + s * STAGE_BYTES, n0, N, M, K, s * GSM_STAGE_K, tid);
        asm volatile("cp.async.commit_group;\n" ::);
    }

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

    for (int s = 0; s < stages_total; ++s) {
        // stage s has landed once at most STAGES-2 newer groups are still in flight
        asm volatile("cp.async.wait_group %0;\n" ::"n"(STAGES - 2));
        __syncthreads();            // visible to all; everyone is also done with stage s-1's buffer
        {
            const int next = s + STAGES - 1;
            if (next < stages_total)
                gsm_issue_stage<0, GSM_ROWS + XROWS>(W, x, ring + (next % STAGES) * STAGE_BYTES, n0, N, M, K,
                                                     next * GSM_STAGE_K, tid);
            asm volatile("cp.async.commit_group;\n" ::);
        }
        const unsigned char* stage = ring + (s % STAGES) * STAGE_BYTES;
        // this warp's quarter of the stage: 128 k-values = 4 runs of 32
        const int kw = warp * (GSM_STAGE_K / GSM_WARPS);
        uint4 vx[4][NT];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int k = s * GSM_STAGE_K + kw + r * 32;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                if (XS) {
                    vx[r][j] = *reinterpret_cast<const uint4*>(stage + (GSM_ROWS + 8 * j + g) * GSM_ROW_BYTES
                                                               + (kw + r * 32 + 8 * t) * 2);
                } else {
                    vx[r][j] = make_uint4(0u, 0u, 0u, 0u);
                    if (ok_x[j] && k + 8 * t < K) vx[r][j] = *reinterpret_cast<const uint4*>(xp[j] + k);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) {
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
    }
    __syncthreads();
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
            gate = round_to<bf16>(gate);
            up = round_to<bf16>(up);
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
        if (bias != nullptr) v += __bfloat162float(bias[n]);
        if (residual != nullptr) v = __bfloat162float(residual[(size_t)token * N + n]) + v;
        if (out_f32) reinterpret_cast<float*>(out)[(size_t)token * N + n] = v;
        else reinterpret_cast<bf16*>(out)[(size_t)token * N + n] = __float2bfloat16_rn(v);
    }
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
    const int blocks = (N + GSM_ROWS - 1) / GSM_ROWS;
    const int smem_staged1 = GSM_STAGES * (GSM_ROWS + 8) * GSM_ROW_BYTES;
    const int smem_staged2 = 3 * (GSM_ROWS + 16) * GSM_ROW_BYTES;
    static bool configured = false;
    if (!configured) {
        cudaError_t e1 = cudaSuccess;
        cudaError_t e2 = cudaFuncSetAttribute(gemm_small_m_kernel<1, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_staged1);
        cudaError_t e3 = cudaFuncSetAttribute(gemm_small_m_kernel<2, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_staged2);
        if (e1 != cudaSuccess || e2 != cudaSuccess || e3 != cudaSuccess)
            QIL_REFUSE("gemm_small_m: cannot reserve %d bytes of shared memory", smem_staged1);
        configured = true;
    }
    if (M <= 8)
        qil_launch_chained(gemm_small_m_kernel<1, 1>, dim3(blocks), dim3(GSM_WARPS * 32), smem_staged1, stream,
            (const bf16*)x, (const bf16*)W, (const bf16*)bias, (const bf16*)residual, out, M, N, K, out_f32, silu_pairs);
    else
        qil_launch_chained(gemm_small_m_kernel<2, 1>, dim3(blocks), dim3(GSM_WARPS * 32), smem_staged2, stream,
            (const bf16*)x, (const bf16*)W, (const bf16*)bias, (const bf16*)residual, out, M, N, K, out_f32, silu_pairs);
    QIL_CHECK_LAUNCH();
}
