// C[M,N] = A[M,K] * W[N,K]^T (+ bias[N]) (+ residual[M,N]) with float32 FMA on the
// CUDA cores: the matrix product of the true 32-bit path (no TF32, no tensor
// cores), also used when a weight is stored in float32 inside a bfloat16 model.
//
// Every output element sums its K products in ascending k with one accumulator,
// whatever M is and wherever the element lies in a tile, so a row's result does
// not depend on which other rows share the launch.
// Weights are row-major [out_features, in_features] as in the checkpoint
// (qil/model.py:32-40: nn.Linear).
#include "common.cuh"

#define BM 64
#define BN 64
#define BK 16

template <typename TA, typename TW>
__global__ void __launch_bounds__(256)
gemm_f32_kernel(const TA* __restrict__ A, const TW* __restrict__ Wt, const TW* __restrict__ bias,
                const TA* residual, TA* C, int M, int N, int K, int lda) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;      // 16 x 16 threads, 4 x 4 outputs each
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // 64 rows x 16 k = 1024 elements per operand, 4 per thread
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int idx = tid + e * 256;
            const int r = idx >> 4, kk = idx & 15;
            const int k = k0 + kk;
            float a = 0.f, w = 0.f;
            if (k < K) {
                if (m0 + r < M) a = to_f32<TA>(A[(size_t)(m0 + r) * lda + k]);
                if (n0 + r < N) w = to_f32<TW>(Wt[(size_t)(n0 + r) * K + k]);
            }
            As[kk][r] = a;
            Ws[kk][r] = w;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias != nullptr) v += to_f32<TW>(bias[n]);
            if (residual != nullptr) v = to_f32<TA>(residual[(size_t)m * N + n]) + v;
            C[(size_t)m * N + n] = from_f32<TA>(v);
        }
    }
}

// residual may alias C (each element is read and written by the same thread).
extern "C" int qil_gemm_f32(const void* A, int lda, const void* Wt, const void* bias, const void* residual,
                            void* C, int M, int N, int K, int act_dtype, int weight_dtype,
                            cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || lda < K) QIL_REFUSE("gemm_f32: K %d lda %d", K, lda);
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (grid.y > 65535) QIL_REFUSE("gemm_f32: M %d is too large for one launch", M);
    QIL_DISPATCH_2(act_dtype, weight_dtype,
        (gemm_f32_kernel<T, W><<<grid, 256, 0, stream>>>((const T*)A, (const W*)Wt, (const W*)bias,
                                                        (const T*)residual, (T*)C, M, N, K, lda)));
    QIL_CHECK_LAUNCH();
}
