// Memory-bound row kernels: embedding gather, RMSNorm (optionally through a row
// index), SiLU-gate multiply, in-place add and dtype casts.
//
// Formulas follow the reference: the norm squares, averages, adds eps, takes the
// reciprocal square root and scales in float32, rounds to the activation dtype and
// only then multiplies by the weight (qil/model.py:21-23); the gate is
// silu(gate) rounded to the activation dtype, times up (qil/model.py:71).
#include "common.cuh"

QIL_ERROR_STORAGE

// ---------------------------------------------------------------- embedding
template <typename T, typename W>
__global__ void embed_gather_kernel(const W* __restrict__ table, const int* __restrict__ ids,
                                    T* __restrict__ out, int width, int vocab) {
    const int row = blockIdx.x;
    int id = ids[row];
    // Host code validates ids; clamp so that a bad id can never read out of bounds.
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    const W* src = table + (size_t)id * width;
    T* dst = out + (size_t)row * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = from_f32<T>(to_f32<W>(src[i]));
}

// bfloat16 table and output with a width that allows 16-byte copies
__global__ void embed_gather_bf16x8_kernel(const bf16* __restrict__ table, const int* __restrict__ ids,
                                           bf16* __restrict__ out, int width, int vocab) {
    qil_wait_for_producer();
    qil_release_consumer();
    const int row = blockIdx.x;
    int id = ids[row];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)id * width);
    uint4* dst = reinterpret_cast<uint4*>(out + (size_t)row * width);
    for (int i = threadIdx.x; i < width / 8; i += blockDim.x) dst[i] = src[i];
}

extern "C" int qil_embed_gather(const void* table, int table_dtype, const int* ids, void* out,
                                int out_dtype, int n_rows, int width, int vocab, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (width <= 0 || vocab <= 0) QIL_REFUSE("embed_gather: width %d vocab %d", width, vocab);
    if (out_dtype == QIL_BF16 && table_dtype == QIL_BF16 && width % 8 == 0 &&
        (((uintptr_t)table | (uintptr_t)out) & 15) == 0) {
        qil_launch_chained(embed_gather_bf16x8_kernel, dim3(n_rows), dim3(128), 0, stream,
                           (const bf16*)table, ids, (bf16*)out, width, vocab);
        QIL_CHECK_LAUNCH();
    }
    QIL_DISPATCH_2(out_dtype, table_dtype,
        embed_gather_kernel<T, W><<<n_rows, 256, 0, stream>>>((const W*)table, ids, (T*)out, width, vocab));
    QIL_CHECK_LAUNCH();
}

// ---------------------------------------------------------------- RMSNorm
// One block per output row.  rows == nullptr: row r reads x[r]; else x[rows[r]].
template <typename T, typename W>
__global__ void rmsnorm_kernel(const T* __restrict__ x, const W* __restrict__ weight,
                               const int* __restrict__ rows, T* __restrict__ out,
                               int width, float eps) {
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const int src_row = rows ? rows[r] : r;
    const T* src = x + (size_t)src_row * width;
    T* dst = out + (size_t)r * width;
    float sq = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = to_f32<T>(src[i]);
        sq += v * v;
    }
    sq = block_sum(sq, scratch);
    const float scale = 1.0f / sqrtf(sq / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float normed = round_to<T>(to_f32<T>(src[i]) * scale);
        dst[i] = from_f32<T>(normed * to_f32<W>(weight[i]));
    }
}

// bfloat16 rows of up to 256 * 8 * RMS_VPT elements: the whole row sits in registers, every load is
// 16 bytes wide and issued before the first use, so a row costs one memory round trip, not one per element.
#define RMS_VPT 4
template <typename W>
__global__ void __launch_bounds__(256)
rmsnorm_bf16x8_kernel(const bf16* __restrict__ x, const W* __restrict__ weight, const int* __restrict__ rows,
                      bf16* __restrict__ out, int width, float eps) {
    __shared__ float scratch[32];
    qil_wait_for_producer();
    qil_release_consumer();
    const int r = blockIdx.x;
    const int src_row = rows ? rows[r] : r;
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)src_row * width);
    uint4* dst = reinterpret_cast<uint4*>(out + (size_t)r * width);
    const int vectors = width / 8;
    uint4 v[RMS_VPT];
#pragma unroll
    for (int i = 0; i < RMS_VPT; ++i) {
        const int idx = threadIdx.x + i * 256;
        v[i] = idx < vectors ? src[idx] : make_uint4(0u, 0u, 0u, 0u);
    }
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < RMS_VPT; ++i) {
        const bf16* e = reinterpret_cast<const bf16*>(&v[i]);
#pragma unroll
        for (int k = 0; k < 8; ++k) { const float f = __bfloat162float(e[k]); sq += f * f; }
    }
    sq = block_sum(sq, scratch);
    const float scale = 1.0f / sqrtf(sq / (float)width + eps);
#pragma unroll
    for (int i = 0; i < RMS_VPT; ++i) {
        const int idx = threadIdx.x + i * 256;
        if (idx >= vectors) continue;
        uint4 o4;
        if (sizeof(W) == 2) {
            // bfloat16 weights: one 16-byte read, and the product of the rounded value and the weight as a
            // packed bfloat16 multiply (one rounding, never contracted with anything)
            const uint4 w4 = *reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(weight) + idx * 8);
            const __nv_bfloat162* e2 = reinterpret_cast<const __nv_bfloat162*>(&v[i]);
            const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&w4);
            __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 f = __bfloat1622float2(e2[k]);
                o2[k] = __hmul2_rn(__floats2bfloat162_rn(f.x * scale, f.y * scale), w2[k]);
            }
        } else {
            const bf16* e = reinterpret_cast<const bf16*>(&v[i]);
            bf16* o = reinterpret_cast<bf16*>(&o4);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const float normed = round_to<bf16>(__bfloat162float(e[k]) * scale);
                o[k] = __float2bfloat16_rn(normed * to_f32<W>(weight[idx * 8 + k]));
            }
        }
        dst[idx] = o4;
    }
}

extern "C" int qil_rmsnorm(const void* x, const void* weight, const int* rows, void* out,
                           int n_rows, int width, float eps, int act_dtype, int weight_dtype,
                           cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (width <= 0) QIL_REFUSE("rmsnorm: width %d", width);
    if (act_dtype == QIL_BF16 && width % 8 == 0 && width <= 256 * 8 * RMS_VPT &&
        (((uintptr_t)x | (uintptr_t)out | (uintptr_t)weight) & 15) == 0) {
        if (weight_dtype == QIL_BF16)
            qil_launch_chained(rmsnorm_bf16x8_kernel<bf16>, dim3(n_rows), dim3(256), 0, stream,
                               (const bf16*)x, (const bf16*)weight, rows, (bf16*)out, width, eps);
        else if (weight_dtype == QIL_F32)
            qil_launch_chained(rmsnorm_bf16x8_kernel<float>, dim3(n_rows), dim3(256), 0, stream,
                               (const bf16*)x, (const float*)weight, rows, (bf16*)out, width, eps);
        else QIL_REFUSE("unknown dtype code %d", weight_dtype);
        QIL_CHECK_LAUNCH();
    }
    QIL_DISPATCH_2(act_dtype, weight_dtype,
        rmsnorm_kernel<T, W><<<n_rows, 256, 0, stream>>>((const T*)x, (const W*)weight, rows, (T*)out, width, eps));
    QIL_CHECK_LAUNCH();
}

// ---------------------------------------------------------------- SiLU(gate) * up
// gate_up: [n_rows, 2 * width]; out: [n_rows, width].  pairs8 == 0: gate columns first, then up
// columns.  pairs8 == 1: groups of 16 columns, 8 gate columns then the 8 matching up columns
// (the layout the decode GEMM's fused epilogue wants its weight rows in).
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int width,
                                size_t total, int pairs8) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < total; i += stride) {
        const size_t row = i / width;
        const int col = (int)(i - row * width);
        const int gcol = pairs8 ? (col >> 3) * 16 + (col & 7) : col;
        const int ucol = pairs8 ? gcol + 8 : width + col;
        const float g = to_f32<T>(gate_up[row * 2 * width + gcol]);
        const float u = to_f32<T>(gate_up[row * 2 * width + ucol]);
        const float act = round_to<T>(g / (1.0f + expf(-g)));
        out[i] = from_f32<T>(act * u);
    }
}

// 8 bf16 values per thread when the width allows 16-byte accesses.
__global__ void silu_mul_bf16x8_kernel(const bf16* __restrict__ gate_up, bf16* __restrict__ out,
                                       int width, size_t total_vec, int pairs8) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const int vec_per_row = width / 8;
    for (; i < total_vec; i += stride) {
        const size_t row = i / vec_per_row;
        const int col = (int)(i - row * vec_per_row) * 8;
        const int gcol = pairs8 ? 2 * col : col;
        const int ucol = pairs8 ? 2 * col + 8 : width + col;
        const uint4 g4 = *reinterpret_cast<const uint4*>(gate_up + row * 2 * width + gcol);
        const uint4 u4 = *reinterpret_cast<const uint4*>(gate_up + row * 2 * width + ucol);
        const bf16* g = reinterpret_cast<const bf16*>(&g4);
        const bf16* u = reinterpret_cast<const bf16*>(&u4);
        uint4 o4;
        bf16* o = reinterpret_cast<bf16*>(&o4);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float gv = __bfloat162float(g[k]);
            // fast exp and divide (a few ulp in float32): the value is rounded to bfloat16 next
            const float act = round_to<bf16>(__fdividef(gv, 1.0f + __expf(-gv)));
            o[k] = __float2bfloat16_rn(act * __bfloat162float(u[k]));
        }
        *reinterpret_cast<uint4*>(out + row * width + col) = o4;
    }
}

extern "C" int qil_silu_mul(const void* gate_up, void* out, int n_rows, int width, int act_dtype,
                            int pairs8, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (width <= 0) QIL_REFUSE("silu_mul: width %d", width);
    if (pairs8 && width % 8) QIL_REFUSE("silu_mul: the paired layout needs a width that is a multiple of 8, got %d", width);
    const size_t total = (size_t)n_rows * width;
    if (act_dtype == QIL_BF16 && width % 8 == 0 && ((uintptr_t)gate_up % 16) == 0 && ((uintptr_t)out % 16) == 0) {
        const size_t total_vec = total / 8;
        const int blocks = (int)((total_vec + 255) / 256 < 148 * 16 ? (total_vec + 255) / 256 : 148 * 16);
        silu_mul_bf16x8_kernel<<<blocks, 256, 0, stream>>>((const bf16*)gate_up, (bf16*)out, width, total_vec, pairs8);
        QIL_CHECK_LAUNCH();
    }
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    QIL_DISPATCH_1(act_dtype,
        silu_mul_kernel<T><<<blocks, 256, 0, stream>>>((const T*)gate_up, (T*)out, width, total, pairs8));
    QIL_CHECK_LAUNCH();
}

// ---------------------------------------------------------------- x += y (float32 sum, one rounding)
template <typename T>
__global__ void add_inplace_kernel(T* __restrict__ x, const T* __restrict__ y, size_t total) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < total; i += stride) x[i] = from_f32<T>(to_f32<T>(x[i]) + to_f32<T>(y[i]));
}

extern "C" int qil_add_inplace(void* x, const void* y, long long total, int act_dtype, cudaStream_t stream) {
    if (total <= 0) return 0;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    QIL_DISPATCH_1(act_dtype,
        add_inplace_kernel<T><<<blocks, 256, 0, stream>>>((T*)x, (const T*)y, (size_t)total));
    QIL_CHECK_LAUNCH();
}

// ---------------------------------------------------------------- token ids that are still on the device
// token_ids[pairs[2i]] = source[pairs[2i + 1]]: a step may be queued before the host has read the tokens
// that the step before it sampled; their places in the step's token list are filled in here, on the
// stream, from the sampler's device buffer.  A source index outside [0, n_source) leaves the place as it is.
__global__ void feed_tokens_kernel(int* __restrict__ token_ids, const int* __restrict__ pairs, int count,
                                   const int* __restrict__ source, int n_source, int n_tokens) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const int dst = pairs[2 * i], src = pairs[2 * i + 1];
    if (dst >= 0 && dst < n_tokens && src >= 0 && src < n_source) token_ids[dst] = source[src];
}

extern "C" int qil_feed_tokens(int* token_ids, const int* pairs, int count, const int* source, int n_source,
                               int n_tokens, cudaStream_t stream) {
    if (count <= 0) return 0;
    feed_tokens_kernel<<<(count + 127) / 128, 128, 0, stream>>>(token_ids, pairs, count, source, n_source, n_tokens);
    QIL_CHECK_LAUNCH();
}

// ---------------------------------------------------------------- dtype cast (src dtype -> dst dtype)
template <typename T, typename W>
__global__ void cast_kernel(const W* __restrict__ src, T* __restrict__ dst, size_t total) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (; i < total; i += stride) dst[i] = from_f32<T>(to_f32<W>(src[i]));
}

extern "C" int qil_cast(const void* src, int src_dtype, void* dst, int dst_dtype, long long total,
                        cudaStream_t stream) {
    if (total <= 0) return 0;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    QIL_DISPATCH_2(dst_dtype, src_dtype,
        cast_kernel<T, W><<<blocks, 256, 0, stream>>>((const W*)src, (T*)dst, (size_t)total));
    QIL_CHECK_LAUNCH();
}

// ---------------------------------------------------------------- random weights
// out[i] = mean + std * z(seed, i) with z close to N(0, 1): the sum of twelve 16-bit uniforms drawn from
// three rounds of a 64-bit counter hash, centred and divided by 65536.  Integer arithmetic and three
// correctly rounded float operations only, so the host twin (weights/random_init.py) gives the same bits.
__device__ __forceinline__ unsigned long long fill_hash(unsigned long long seed, unsigned long long counter) {
    unsigned long long z = seed + (counter + 1ull) * 0x9E3779B97F4A7C15ull;
    z ^= z >> 30; z *= 0xBF58476D1CE4E5B9ull;
    z ^= z >> 27; z *= 0x94D049BB133111EBull;
    z ^= z >> 31;
    return z;
}

template <typename T>
__global__ void fill_normal_kernel(T* __restrict__ out, long long total, unsigned long long seed, float std,
                                   float mean) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        int sum = 0;
#pragma unroll
        for (int round = 0; round < 3; ++round) {
            const unsigned long long h = fill_hash(seed, 3ull * (unsigned long long)i + round);
            sum += (int)(h & 0xFFFFull) + (int)((h >> 16) & 0xFFFFull) + (int)((h >> 32) & 0xFFFFull) + (int)(h >> 48);
        }
        const float z = __fmul_rn((float)(sum - 393210), 1.0f / 65536.0f);
        out[i] = from_f32<T>(__fadd_rn(__fmul_rn(z, std), mean));
    }
}

extern "C" int qil_fill_normal(void* out, int out_dtype, long long total, unsigned long long seed, float std,
                               float mean, cudaStream_t stream) {
    if (total <= 0) return 0;
    const long long blocks = (total + 255) / 256;
    const int grid = (int)(blocks < 148 * 16 ? blocks : 148 * 16);
    QIL_DISPATCH_1(out_dtype, fill_normal_kernel<T><<<grid, 256, 0, stream>>>((T*)out, total, seed, std, mean));
    QIL_CHECK_LAUNCH();
}
