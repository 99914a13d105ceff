// Next-token choice from float32 logits.
//
// Greedy rows take the largest logit, the lowest index among equals, and report
// non-finite logits instead of choosing silently (qil/engine.py:96-100).
// Temperature rows add Gumbel noise to logit / temperature and take the largest
// sum, which draws from softmax(logit / temperature).  The noise of vocabulary
// entry i is a pure function of (seed, draw counter, i), so a request's tokens do
// not depend on which other requests share the batch.
//
// The settings of a row come either from three arrays the caller uploads (temperature, seed, draw
// counter per row) or from the requests' state slots: ``state`` int64 [slots, 4] holds, per request,
// (the temperature's float bits, the seed, the number of draws so far, unused) and ``owner`` names each
// row's slot.  With slots the kernel counts the draws itself, so a step uploads nothing for sampling.
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

// A row is cut into up to SAMPLE_SPLITS slices, one block each, so that a handful of rows over a large
// vocabulary keeps more than a handful of SMs busy; the block that finishes a row's last slice (a
// ticket per row, which it also resets) combines the slices' candidates.  The candidates and tickets
// live in arrays inside the library: calls on different streams must not overlap.
#define SAMPLE_SPLITS 32
#define SAMPLE_MAX_ROWS 4096
static __device__ float sample_part_v[SAMPLE_MAX_ROWS * SAMPLE_SPLITS];
static __device__ int sample_part_i[SAMPLE_MAX_ROWS * SAMPLE_SPLITS];
static __device__ int sample_part_bad[SAMPLE_MAX_ROWS * SAMPLE_SPLITS];
static __device__ unsigned sample_tickets[SAMPLE_MAX_ROWS];

__device__ __forceinline__ void sample_better(float& bv, int& bi, float ov, int oi) {
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }      // the lowest index among equals
}

__global__ void __launch_bounds__(256)
sample_rows_kernel(const float* __restrict__ logits, int vocab, long long row_stride, int splits, int slice,
                   const float* __restrict__ temperature, const long long* __restrict__ seed,
                   const long long* __restrict__ counter, long long* __restrict__ state,
                   const int* __restrict__ owner, int* __restrict__ token_out, int* __restrict__ nonfinite_out) {
    __shared__ float best_v[8];
    __shared__ int best_i[8];
    __shared__ int bad_s[8];
    __shared__ int is_last;
    const int row = blockIdx.y, split = blockIdx.x;
    const float* x = logits + (size_t)row * row_stride;
    long long* const slot_state = state ? state + (size_t)owner[row] * 4 : nullptr;
    // every block of the row reads the draw count before it takes its ticket; the block that takes the last
    // ticket moves the count on
    const float temp = slot_state ? __int_as_float((int)slot_state[0]) : (temperature ? temperature[row] : 0.f);
    const unsigned long long sd = slot_state ? (unsigned long long)slot_state[1] : (seed ? (unsigned long long)seed[row] : 0ull);
    const unsigned long long ct = slot_state ? (unsigned long long)slot_state[2] : (counter ? (unsigned long long)counter[row] : 0ull);
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    int bad = 0;
    const int end = min(vocab, (split + 1) * slice);
    for (int i = split * slice + threadIdx.x; i < end; i += blockDim.x) {
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
        sample_better(bv, bi, ov, oi);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; bad_s[warp] = bad; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w) { sample_better(bv, bi, best_v[w], best_i[w]); bad |= bad_s[w]; }
        const int slot = row * SAMPLE_SPLITS + split;
        sample_part_v[slot] = bv; sample_part_i[slot] = bi; sample_part_bad[slot] = bad;
        __threadfence();
        const unsigned drawn = atomicAdd(&sample_tickets[row], 1u);
        is_last = drawn == (unsigned)splits - 1u;
        if (is_last) {
            sample_tickets[row] = 0u;
            if (slot_state) slot_state[2] = (long long)(ct + 1ull);
        }
    }
    __syncthreads();
    if (!is_last || threadIdx.x >= 32) return;
    __threadfence();
    bv = -INFINITY; bi = 0x7fffffff; bad = 0;
    if (lane < splits) {
        const int slot = row * SAMPLE_SPLITS + lane;
        bv = __ldcg(&sample_part_v[slot]); bi = __ldcg(&sample_part_i[slot]); bad = __ldcg(&sample_part_bad[slot]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        bad |= __shfl_xor_sync(0xffffffffu, bad, o);
        sample_better(bv, bi, ov, oi);
    }
    if (lane == 0) {
        token_out[row] = bi == 0x7fffffff ? 0 : bi;
        nonfinite_out[row] = bad;
    }
}

extern "C" int qil_sample_rows(const float* logits, int n_rows, int vocab, long long row_stride,
                               const float* temperature, const long long* seed, const long long* counter,
                               long long* state, const int* owner, int* token_out, int* nonfinite_out,
                               cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (vocab <= 0 || row_stride < vocab) QIL_REFUSE("sample_rows: vocab %d row stride %lld", vocab, row_stride);
    if ((state == nullptr) != (owner == nullptr)) QIL_REFUSE("sample_rows: state slots need the rows' owners, and the reverse");
    if (state != nullptr && (temperature || seed || counter))
        QIL_REFUSE("sample_rows: settings come from state slots or from arrays, not both");
    int splits = (vocab + 2047) / 2048;
    if (splits > SAMPLE_SPLITS) splits = SAMPLE_SPLITS;
    const int slice = (vocab + splits - 1) / splits;
    for (int first = 0; first < n_rows; first += SAMPLE_MAX_ROWS) {
        const int rows = n_rows - first < SAMPLE_MAX_ROWS ? n_rows - first : SAMPLE_MAX_ROWS;
        sample_rows_kernel<<<dim3(splits, rows), 256, 0, stream>>>(
            logits + (size_t)first * row_stride, vocab, row_stride, splits, slice,
            temperature ? temperature + first : nullptr, seed ? seed + first : nullptr,
            counter ? counter + first : nullptr, state, owner ? owner + first : nullptr, token_out + first,
            nonfinite_out + first);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) { snprintf(qil_error_text, sizeof(qil_error_text), "%s", cudaGetErrorString(e)); return (int)e; }
    }
    return 0;
}
