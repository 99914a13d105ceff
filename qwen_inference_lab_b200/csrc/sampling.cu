// Next-token choice from float32 logits, one block per row.
//
// Greedy rows take the largest logit, the lowest index among equals, and report
// non-finite logits instead of choosing silently (qil/engine.py:96-100).
// Temperature rows add Gumbel noise to logit / temperature and take the largest
// sum, which draws from softmax(logit / temperature).  The noise of vocabulary
// entry i is a pure function of (seed, draw counter, i), so a request's tokens do
// not depend on which other requests share the batch.
#include "common.cuh"

__device__ __forceinline__ float qil_uniform(unsigned long long seed, unsigned long long counter,
                                             unsigned long long index) {
    unsigned long long z = seed ^ (0x9E3779B97F4A7C15ull * (counter + 1ull));
    z += index * 0xBF58476D1CE4E5B9ull;
    z ^= z >> 30; z *= 0xBF58476D1CE4E5B9ull;
    z ^= z >> 27; z *= 0x94D049BB133111EBull;
    z ^= z >> 31;
    return ((float)(z >> 40) + 0.5f) * (1.0f / 16777216.0f);   // in (0, 1)
}

__global__ void __launch_bounds__(512)
sample_rows_kernel(const float* __restrict__ logits, int vocab, long long row_stride,
                   const float* __restrict__ temperature, const long long* __restrict__ seed,
                   const long long* __restrict__ counter, int* __restrict__ token_out,
                   int* __restrict__ nonfinite_out) {
    __shared__ float best_v[16];
    __shared__ int best_i[16];
    __shared__ int bad_s[16];
    const int row = blockIdx.x;
    const float* x = logits + (size_t)row * row_stride;
    const float temp = temperature ? temperature[row] : 0.f;
    const unsigned long long sd = seed ? (unsigned long long)seed[row] : 0ull;
    const unsigned long long ct = counter ? (unsigned long long)counter[row] : 0ull;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    int bad = 0;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = x[i];
        if (!isfinite(v)) bad = 1;
        float key = v;
        if (temp > 0.f) {
            const float u = qil_uniform(sd, ct, (unsigned long long)i);
            key = v / temp - logf(-logf(u));
        }
        if (key > bv) { bv = key; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        bad |= __shfl_xor_sync(0xffffffffu, bad, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; bad_s[warp] = bad; }
    __syncthreads();
    if (warp == 0) {
        const int warps = blockDim.x >> 5;
        bv = lane < warps ? best_v[lane] : -INFINITY;
        bi = lane < warps ? best_i[lane] : 0x7fffffff;
        bad = lane < warps ? bad_s[lane] : 0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            bad |= __shfl_xor_sync(0xffffffffu, bad, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) {
            token_out[row] = bi == 0x7fffffff ? 0 : bi;
            nonfinite_out[row] = bad;
        }
    }
}

extern "C" int qil_sample_rows(const float* logits, int n_rows, int vocab, long long row_stride,
                               const float* temperature, const long long* seed, const long long* counter,
                               int* token_out, int* nonfinite_out, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (vocab <= 0 || row_stride < vocab) QIL_REFUSE("sample_rows: vocab %d row stride %lld", vocab, row_stride);
    sample_rows_kernel<<<n_rows, 512, 0, stream>>>(logits, vocab, row_stride, temperature, seed, counter,
                                                  token_out, nonfinite_out);
    QIL_CHECK_LAUNCH();
}
