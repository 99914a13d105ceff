// C[M,N] = A[M,K] * W[N,K]^T (+ bias) (+ residual) in bfloat16 with float32
// accumulation on the fifth-generation tensor cores: the projections of prompt
// portions (M from a few dozen to thousands of tokens).
//
// Blackwell-native structure, one persistent block per SM, 192 threads:
//   warp 0      one thread issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle) of a
//               128 x 64 tile of A and a 256 x 64 tile of W per stage into a 4-stage ring and
//               arms the stage's mbarrier with the byte count;
//   warp 1      one thread issues tcgen05.mma (128 x 256 x 16, operands from shared memory
//               through matrix descriptors, accumulator in tensor memory) four times per stage,
//               then tcgen05.commit, which frees the stage when the MMAs have read it; the warp
//               also allocates and frees the 512 columns of tensor memory;
//   warps 2-5   read the finished accumulator with tcgen05.ld (each warp its quarter of the 128
//               lanes), apply the epilogue and store bfloat16; meanwhile warp 1 already fills
//               the other half of tensor memory with the next tile.
// Tiles go round-robin over the blocks: tile = blockIdx.x + i * gridDim.x, tokens fastest, so
// blocks that run together share the same weight columns in L2.
//
// Epilogues: bias, residual (may alias out), or `silu_pairs`: W's rows are stored as groups of
// [8 gate rows, 8 up rows] and the kernel writes silu(gate) * up, N/2 values per token
// (qil/model.py:71), so the [M, 2I] intermediate never exists in memory.
//
// Every wait on an mbarrier is bounded.  A wait that runs out records its place in the error
// word, the role stops issuing, every role runs out in turn, the producer drains its copies in
// flight (again bounded), the tensor memory is freed and the kernel returns; the host reads the
// error word.  No multicast loads are used.
#include "common.cuh"
#include <cuda.h>
#include <stdlib.h>

QIL_ERROR_STORAGE

#define TC_BM 128
#define TC_BN 256
#define TC_BK 64
#define TC_STAGES 4
#define TC_A_BYTES (TC_BM * TC_BK * 2)
#define TC_B_BYTES (TC_BN * TC_BK * 2)
#define TC_STAGE_BYTES (TC_A_BYTES + TC_B_BYTES)
#define TC_WAIT_CYCLES 2000000000ll      // about a second

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, unsigned parity) {
    unsigned done;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}\n"
                 : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return done != 0;
}
// Bounded wait: false when the barrier did not complete in about a second.
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long start = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (clock64() - start > TC_WAIT_CYCLES) return false;
    }
    return true;
}

__device__ __forceinline__ void tma_load_2d(void* smem, const CUtensorMap* map, unsigned long long* bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
                 ::"r"(smem_u32(smem)), "l"((unsigned long long)map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}

// The same with the hint that these bytes are the first to leave L2: a weight tile that only one tile of tokens reads
// (a product of at most 128 rows) is read once a step.
__device__ __forceinline__ void tma_load_2d_stream(void* smem, const CUtensorMap* map, unsigned long long* bar, int x, int y) {
    unsigned long long policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;\n" : "=l"(policy));
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;\n"
                 ::"r"(smem_u32(smem)), "l"((unsigned long long)map), "r"(smem_u32(bar)), "r"(x), "r"(y), "l"(policy) : "memory");
}

// Shared-memory matrix descriptor: K-major operand, rows of 128 bytes, 128-byte swizzle, groups of 8
// rows 1024 bytes apart (the layout a TMA load with CU_TENSOR_MAP_SWIZZLE_128B writes).
__device__ __forceinline__ unsigned long long umma_desc(unsigned smem_addr) {
    unsigned long long d = 0;
    d |= (unsigned long long)((smem_addr & 0x3FFFF) >> 4);          // start address, 16-byte units
    d |= (unsigned long long)1 << 16;                                // leading byte offset (unused with swizzle)
    d |= (unsigned long long)(1024 >> 4) << 32;                      // stride byte offset: 8 rows
    d |= (unsigned long long)1 << 46;                                // descriptor version of sm_100
    d |= (unsigned long long)2 << 61;                                // 128-byte swizzle
    return d;
}
// Instruction descriptor: bfloat16 x bfloat16 -> float32, both operands K-major, M = 128, N = 256.
__device__ __forceinline__ unsigned umma_idesc() {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(TC_BN >> 3) << 17) | ((unsigned)(TC_BM >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(unsigned tmem_d, unsigned long long desc_a, unsigned long long desc_b,
                                          unsigned idesc, unsigned accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
                 ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }

__device__ __forceinline__ void tmem_load_32(unsigned taddr, float (&v)[32]) {
    unsigned r[32];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// The query/key/value projection can end in what otherwise is a kernel of its own: per-head RMSNorm of
// queries and keys, the rotation of both by the token's position, queries to their buffer and keys and
// values into the token's page of the cache (qil/model.py:52-57, qil/cache.py:93-94).  Heads are 128 wide,
// so every 128-column half of an output tile is one whole head and one thread holds a token's head in
// registers.  The arithmetic and its rounding points are those of rope_kv.cu's bfloat16 kernel: the
// product rounded to bfloat16 first, sums of squares and the normalising factor in float32, the normed
// value rounded before the weight multiplies it, every product and sum of the rotation rounded by itself.
struct TcQkvTail {
    bf16* q_out;                 // [tokens, n_q_heads, 128]; null: the ordinary epilogue
    bf16* pages;                 // one layer's cache: [page][2][n_kv_heads][page_size][128]
    const float* rope;           // [rope_rows][128]: 64 cosines then 64 sines per position; null: no rotation
    const bf16* q_norm;          // [128] or null
    const bf16* k_norm;
    const int* positions;        // [tokens]
    const int* token_row;        // [tokens] block-table row
    const int* block_table;
    float eps;
    int table_stride, rope_rows, n_q_heads, n_kv_heads, page_size, num_pages;
};

__device__ __forceinline__ void tc_store_qkv_head(unsigned taddr, int m, int M, int head, const TcQkvTail& t,
                                                  const bf16* __restrict__ bias) {
    typedef __nv_bfloat162 bf2;
    // The head as 64 packed pairs (elements 2i, 2i + 1), rounded to bfloat16 as the product's output is.
    // Packed arithmetic from here on: one instruction per two values, and half the registers; the single
    // epilogue warp of a scheduler runs one dependent instruction after the other, so their number is
    // what the epilogue costs.
    bf2 pk[64];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        float part[32];
        __syncwarp();                              // the load is a warp-wide instruction: every lane takes part
        tmem_load_32(taddr + c * 32, part);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            float x = part[2 * i], y = part[2 * i + 1];
            if (bias != nullptr) {
                const float2 b = __bfloat1622float2(*reinterpret_cast<const bf2*>(bias + head * 128 + c * 32 + 2 * i));
                x += b.x; y += b.y;
            }
            pk[c * 16 + i] = __floats2bfloat162_rn(x, y);
        }
    }
    if (m >= M) return;
    const bool is_q = head < t.n_q_heads;
    const bool is_k = !is_q && head < t.n_q_heads + t.n_kv_heads;
    const bf16* norm_w = is_q ? t.q_norm : (is_k ? t.k_norm : nullptr);
    if (norm_w != nullptr) {
        float sq = 0.f;
#pragma unroll
        for (int i = 0; i < 64; ++i) {
            const float2 f = __bfloat1622float2(pk[i]);
            sq = fmaf(f.x, f.x, sq);
            sq = fmaf(f.y, f.y, sq);
        }
        const float scale = rsqrtf(sq / 128.0f + t.eps);
        const bf2* w2 = reinterpret_cast<const bf2*>(norm_w);
#pragma unroll
        for (int i = 0; i < 64; ++i) {
            const float2 f = __bfloat1622float2(pk[i]);
            pk[i] = __hmul2_rn(__floats2bfloat162_rn(f.x * scale, f.y * scale), w2[i]);
        }
    }
    const int pos = t.positions[m];
    if ((is_q || is_k) && t.rope != nullptr) {
        const int row = (pos >= t.rope_rows && t.rope_rows > 0) ? t.rope_rows - 1 : pos;
        const float4* cs = reinterpret_cast<const float4*>(t.rope + (size_t)row * 128);
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
            // the table holds values already rounded to bfloat16: the conversion is exact
            const float4 cf = cs[i / 2], sf = cs[16 + i / 2];
            const bf2 c0 = __floats2bfloat162_rn(cf.x, cf.y), c1 = __floats2bfloat162_rn(cf.z, cf.w);
            const bf2 s0 = __floats2bfloat162_rn(sf.x, sf.y), s1 = __floats2bfloat162_rn(sf.z, sf.w);
            const bf2 lo0 = pk[i], lo1 = pk[i + 1], hi0 = pk[32 + i], hi1 = pk[32 + i + 1];
            // every product and sum rounds by itself (the _rn forms are never contracted into fused multiply-adds)
            pk[i] = __hsub2_rn(__hmul2_rn(lo0, c0), __hmul2_rn(hi0, s0));
            pk[i + 1] = __hsub2_rn(__hmul2_rn(lo1, c1), __hmul2_rn(hi1, s1));
            pk[32 + i] = __hadd2_rn(__hmul2_rn(lo0, s0), __hmul2_rn(hi0, c0));
            pk[32 + i + 1] = __hadd2_rn(__hmul2_rn(lo1, s1), __hmul2_rn(hi1, c1));
        }
    }
    bf16* dst;
    if (is_q) {
        dst = t.q_out + ((size_t)m * t.n_q_heads + head) * 128;
    } else {
        const int kv_head = is_k ? head - t.n_q_heads : head - t.n_q_heads - t.n_kv_heads;
        const int index = pos / t.page_size;                 // a position the table has no entry for writes nothing
        const int page = (pos >= 0 && index < t.table_stride) ? t.block_table[(size_t)t.token_row[m] * t.table_stride + index] : -1;
        if (page < 0 || page >= t.num_pages) return;        // never write outside the pool
        dst = t.pages + ((((size_t)page * 2 + (is_k ? 0 : 1)) * t.n_kv_heads + kv_head) * t.page_size + pos % t.page_size) * 128;
    }
#pragma unroll
    for (int q = 0; q < 16; ++q) {
        uint4 packed;
        packed.x = *reinterpret_cast<const unsigned*>(&pk[4 * q]);
        packed.y = *reinterpret_cast<const unsigned*>(&pk[4 * q + 1]);
        packed.z = *reinterpret_cast<const unsigned*>(&pk[4 * q + 2]);
        packed.w = *reinterpret_cast<const unsigned*>(&pk[4 * q + 3]);
        *reinterpret_cast<uint4*>(dst + q * 8) = packed;
    }
}

// One warp's quarter (32 rows) of a finished 128 x 256 accumulator: tcgen05.ld 32 columns at a time,
// epilogue, bfloat16 stores.  m is this lane's output row, n0 the tile's first output column.
__device__ __forceinline__ void tc_store_accumulator(unsigned taddr, int m, int n0, int M, int N, int silu_pairs,
                                                     const bf16* __restrict__ bias, const bf16* residual, bf16* out) {
#pragma unroll 1
    for (int c = 0; c < TC_BN / 32; ++c) {
        float v[32];
        __syncwarp();                              // the load below is a warp-wide instruction
        tmem_load_32(taddr + c * 32, v);
        const int n = n0 + c * 32;
        if (m >= M || n >= N) {
            // nothing to store for this lane
        } else if (silu_pairs) {
            // columns come as [8 gate, 8 up] groups: 32 columns give 16 outputs
            const int out_width = N / 2;
            bf16* dst = out + (size_t)m * out_width + n / 2;
#pragma unroll
            for (int grp = 0; grp < 2; ++grp) {
                uint4 packed;
                bf16* o = reinterpret_cast<bf16*>(&packed);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float gate = round_to<bf16>(v[grp * 16 + i]);
                    const float up = round_to<bf16>(v[grp * 16 + 8 + i]);
                    const float act = round_to<bf16>(__fdividef(gate, 1.0f + __expf(-gate)));
                    o[i] = __float2bfloat16_rn(act * up);
                }
                if (n + grp * 16 < N) *reinterpret_cast<uint4*>(dst + grp * 8) = packed;
            }
        } else {
            bf16* dst = out + (size_t)m * N + n;
            const bf16* res = residual ? residual + (size_t)m * N + n : nullptr;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                if (n + q * 8 >= N) break;
                uint4 packed, rv = make_uint4(0u, 0u, 0u, 0u);
                if (res) rv = *reinterpret_cast<const uint4*>(res + q * 8);
                const bf16* r8 = reinterpret_cast<const bf16*>(&rv);
                bf16* o = reinterpret_cast<bf16*>(&packed);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    float x = v[q * 8 + i];
                    if (bias) x += __bfloat162float(bias[n + q * 8 + i]);
                    if (res) x = __bfloat162float(r8[i]) + x;
                    o[i] = __float2bfloat16_rn(x);
                }
                *reinterpret_cast<uint4*>(dst + q * 8) = packed;
            }
        }
    }
}

struct TcShared {
    unsigned long long full[TC_STAGES];
    unsigned long long empty[TC_STAGES];
    unsigned long long acc_full[2];
    unsigned long long acc_empty[2];
    unsigned tmem_base;
    unsigned pad;
};

__global__ void __launch_bounds__(192, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
               const bf16* __restrict__ bias, const bf16* residual, bf16* out,
               int M, int N, int K, int silu_pairs, int* error_word, const TcQkvTail tail) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    TcShared* sh = reinterpret_cast<TcShared*>(tiles + TC_STAGES * TC_STAGE_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (M + TC_BM - 1) / TC_BM, tiles_n = (N + TC_BN - 1) / TC_BN;
    const int n_tiles = tiles_m * tiles_n;
    const int k_blocks = (K + TC_BK - 1) / TC_BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TC_STAGES; ++s) { mbar_init(&sh->full[s], 1); mbar_init(&sh->empty[s], 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(&sh->acc_full[a], 1); mbar_init(&sh->acc_empty[a], 4); }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(&sh->tmem_base)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_base = sh->tmem_base;

    if (warp == 0) {
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];\n" ::"l"((unsigned long long)&map_a) : "memory");
            asm volatile("prefetch.tensormap [%0];\n" ::"l"((unsigned long long)&map_w) : "memory");
            int stage = 0;
            unsigned phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                const int m0 = (tile % tiles_m) * TC_BM, n0 = (tile / tiles_m) * TC_BN;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(&sh->empty[stage], phase ^ 1)) { atomicExch(error_word, 1); ok = false; break; }
                    mbar_arrive_expect_tx(&sh->full[stage], TC_STAGE_BYTES);
                    unsigned char* a_dst = tiles + stage * TC_STAGE_BYTES;
                    tma_load_2d(a_dst, &map_a, &sh->full[stage], kb * TC_BK, m0);
                    if (tiles_m == 1) tma_load_2d_stream(a_dst + TC_A_BYTES, &map_w, &sh->full[stage], kb * TC_BK, n0);
                    else tma_load_2d(a_dst + TC_A_BYTES, &map_w, &sh->full[stage], kb * TC_BK, n0);
                    if (++stage == TC_STAGES) { stage = 0; phase ^= 1; }
                }
            }
            // copies still in flight land in this block's shared memory: wait for them (bounded)
            // before the block may leave, whether or not anyone consumes them
            for (int i = 0; i < TC_STAGES; ++i) {
                if (!mbar_wait(&sh->empty[stage], phase ^ 1)) { atomicExch(error_word, 2); break; }
                if (++stage == TC_STAGES) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const unsigned idesc = umma_idesc();
            int stage = 0, acc = 0;
            unsigned phase = 0, acc_phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                if (!mbar_wait(&sh->acc_empty[acc], acc_phase ^ 1)) { atomicExch(error_word, 3); ok = false; break; }
                tc_fence_after();
                const unsigned tmem_d = tmem_base + (unsigned)acc * TC_BN;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(&sh->full[stage], phase)) { atomicExch(error_word, 4); ok = false; break; }
                    tc_fence_after();
                    const unsigned a_addr = smem_u32(tiles + stage * TC_STAGE_BYTES);
                    const unsigned b_addr = a_addr + TC_A_BYTES;
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k) {
                        // 16 k-values are 32 bytes: advance the start address inside the swizzled row
                        umma_bf16(tmem_d, umma_desc(a_addr + k * 32), umma_desc(b_addr + k * 32), idesc,
                                  (kb | k) ? 1u : 0u);
                    }
                    umma_commit(&sh->empty[stage]);      // the stage is free once these MMAs have read it
                    if (++stage == TC_STAGES) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                umma_commit(&sh->acc_full[acc]);          // the accumulator is complete once all MMAs are done
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1;
            }
        }
    } else {
        const int quarter = warp & 3;                      // the TMEM lanes this warp may read
        int acc = 0;
        unsigned acc_phase = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
            const int m0 = (tile % tiles_m) * TC_BM, n0 = (tile / tiles_m) * TC_BN;
            if (!mbar_wait(&sh->acc_full[acc], acc_phase)) { if (lane == 0) atomicExch(error_word, 5); ok = false; break; }
            tc_fence_after();
            const int m = m0 + quarter * 32 + lane;
            const unsigned taddr = tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)acc * TC_BN;
            if (tail.q_out != nullptr) {
#pragma unroll 1
                for (int h = 0; h < TC_BN / 128; ++h)
                    if (n0 + h * 128 < N) tc_store_qkv_head(taddr + h * 128, m, M, (n0 + h * 128) / 128, tail, bias);
            } else {
                tc_store_accumulator(taddr, m, n0, M, N, silu_pairs, bias, residual, out);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh->acc_empty[acc]);
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

// ------------------------------------------------------------------ two SMs on one tile
// The same product with pairs of blocks (a cluster of two, on neighbouring SMs) working on one
// 256 x 256 output tile with tcgen05.mma.cta_group::2.  Each block of a pair loads its own 128 rows of A
// and its own half (128 output features) of the W tile; one thread of the pair's first block issues the
// MMAs, which read A and W from both blocks' shared memory and write each block's 128 x 256 half of the
// accumulator into that block's tensor memory.  Against the one-block kernel every MMA reads half as
// many bytes of shared memory per block (8 KB instead of 12 KB per 128 x 256 x 16 step), which is what
// keeps the tensor pipe fed, and a stage is 32 KB instead of 48 KB, so six stages fit instead of four.
//
// Barriers.  full[s] lives in the first block: its producer arms it with the bytes of both blocks and
// the second block's copies complete on it too (the barrier operand of a cta_group::2 copy may be the
// peer's).  empty[s] and acc_full[a] exist in both blocks and are signalled by one tcgen05.commit with a
// multicast mask of both.  acc_empty[a] lives in the first block and collects the arrivals of the eight
// epilogue warps of the pair, the second block's through shared::cluster addresses.  Every wait is
// local to the waiting block and bounded as in the kernel above; the pair meets at a cluster barrier
// before either block frees its tensor memory and leaves.  None of the loads is a multicast load.
#define T2_STAGES 6
#define T2_A_BYTES (128 * TC_BK * 2)
#define T2_B_BYTES (128 * TC_BK * 2)
#define T2_STAGE_BYTES (T2_A_BYTES + T2_B_BYTES)

struct Tc2Shared {
    unsigned long long full[T2_STAGES];
    unsigned long long empty[T2_STAGES];
    unsigned long long acc_full[2];
    unsigned long long acc_empty[2];
    unsigned tmem_base;
    unsigned pad;
};

__device__ __forceinline__ unsigned cluster_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
// The shared::cluster address of the same shared-memory offset in block `rank` of the cluster.
__device__ __forceinline__ unsigned map_to_rank(unsigned shared_addr, unsigned rank) {
    unsigned r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(shared_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(unsigned cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(cluster_addr) : "memory");
}
// A tile copy of a block of a pair; `bar_cluster` may be a barrier of the pair's other block.
__device__ __forceinline__ void tma_load_2d_pair(void* smem, const CUtensorMap* map, unsigned bar_cluster, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
                 ::"r"(smem_u32(smem)), "l"((unsigned long long)map), "r"(bar_cluster), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(unsigned tmem_d, unsigned long long desc_a, unsigned long long desc_b,
                                               unsigned idesc, unsigned accumulate) {
    const unsigned zero = 0u;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}\n"
                 ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(zero) : "memory");
}
// Arrives, once the pair's MMAs so far are done, on the barrier at this offset in both blocks.
__device__ __forceinline__ void umma_commit_pair(unsigned long long* bar) {
    const unsigned short both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n"
                 ::"r"(smem_u32(bar)), "h"(both) : "memory");
}
// bfloat16 x bfloat16 -> float32, both operands K-major, M = 256 over the pair, N = 256.
__device__ __forceinline__ unsigned umma_idesc_pair() {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(256 >> 3) << 17) | ((unsigned)(256 >> 4) << 24);
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    const bf16* __restrict__ bias, const bf16* residual, bf16* out,
                    int M, int N, int K, int silu_pairs, int* error_word, const TcQkvTail tail) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    Tc2Shared* sh = reinterpret_cast<Tc2Shared*>(tiles + T2_STAGES * T2_STAGE_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned rank = cluster_rank();
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int tiles_m = (M + 255) / 256, tiles_n = (N + TC_BN - 1) / TC_BN;
    const int n_tiles = tiles_m * tiles_n;
    const int k_blocks = (K + TC_BK - 1) / TC_BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < T2_STAGES; ++s) { mbar_init(&sh->full[s], 1); mbar_init(&sh->empty[s], 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(&sh->acc_full[a], 1); mbar_init(&sh->acc_empty[a], 8); }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {     // the same warp of both blocks, the same address: the pair's allocation
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(&sh->tmem_base)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();          // the other block's barriers are initialised before anything arrives on them
    tc_fence_after();
    const unsigned tmem_base = sh->tmem_base;

    if (warp == 0) {
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];\n" ::"l"((unsigned long long)&map_a) : "memory");
            asm volatile("prefetch.tensormap [%0];\n" ::"l"((unsigned long long)&map_w) : "memory");
            int stage = 0;
            unsigned phase = 0;
            bool ok = true;
            for (int tile = pair; tile < n_tiles && ok; tile += n_pairs) {
                const int m0 = (tile % tiles_m) * 256 + (int)rank * 128, n0 = (tile / tiles_m) * TC_BN + (int)rank * 128;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(&sh->empty[stage], phase ^ 1)) { atomicExch(error_word, 1); ok = false; break; }
                    if (rank == 0) mbar_arrive_expect_tx(&sh->full[stage], 2 * T2_STAGE_BYTES);
                    const unsigned full_of_first = map_to_rank(smem_u32(&sh->full[stage]), 0);
                    unsigned char* a_dst = tiles + stage * T2_STAGE_BYTES;
                    tma_load_2d_pair(a_dst, &map_a, full_of_first, kb * TC_BK, m0);
                    tma_load_2d_pair(a_dst + T2_A_BYTES, &map_w, full_of_first, kb * TC_BK, n0);
                    if (++stage == T2_STAGES) { stage = 0; phase ^= 1; }
                }
            }
            for (int i = 0; i < T2_STAGES; ++i) {      // this block's copies in flight land before it leaves
                if (!mbar_wait(&sh->empty[stage], phase ^ 1)) { atomicExch(error_word, 2); break; }
                if (++stage == T2_STAGES) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            const unsigned idesc = umma_idesc_pair();
            int stage = 0, acc = 0;
            unsigned phase = 0, acc_phase = 0;
            bool ok = true;
            for (int tile = pair; tile < n_tiles && ok; tile += n_pairs) {
                if (!mbar_wait(&sh->acc_empty[acc], acc_phase ^ 1)) { atomicExch(error_word, 3); ok = false; break; }
                tc_fence_after();
                const unsigned tmem_d = tmem_base + (unsigned)acc * TC_BN;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(&sh->full[stage], phase)) { atomicExch(error_word, 4); ok = false; break; }
                    tc_fence_after();
                    const unsigned a_addr = smem_u32(tiles + stage * T2_STAGE_BYTES);
                    const unsigned b_addr = a_addr + T2_A_BYTES;
#pragma unroll
                    for (int k = 0; k < TC_BK / 16; ++k)
                        umma_bf16_pair(tmem_d, umma_desc(a_addr + k * 32), umma_desc(b_addr + k * 32), idesc,
                                       (kb | k) ? 1u : 0u);
                    umma_commit_pair(&sh->empty[stage]);
                    if (++stage == T2_STAGES) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                umma_commit_pair(&sh->acc_full[acc]);
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1;
            }
        }
    } else {
        const int quarter = warp & 3;
        int acc = 0;
        unsigned acc_phase = 0;
        bool ok = true;
        for (int tile = pair; tile < n_tiles && ok; tile += n_pairs) {
            const int m0 = (tile % tiles_m) * 256 + (int)rank * 128, n0 = (tile / tiles_m) * TC_BN;
            if (!mbar_wait(&sh->acc_full[acc], acc_phase)) { if (lane == 0) atomicExch(error_word, 5); ok = false; break; }
            tc_fence_after();
            const int m = m0 + quarter * 32 + lane;
            const unsigned taddr = tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)acc * TC_BN;
            if (tail.q_out != nullptr) {
#pragma unroll 1
                for (int h = 0; h < TC_BN / 128; ++h)
                    if (n0 + h * 128 < N) tc_store_qkv_head(taddr + h * 128, m, M, (n0 + h * 128) / 128, tail, bias);
            } else {
                tc_store_accumulator(taddr, m, n0, M, N, silu_pairs, bias, residual, out);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_rank(smem_u32(&sh->acc_empty[acc]), 0));
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1;
        }
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();          // neither block leaves while the other may still read its tiles or signal it
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult status;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &status) == cudaSuccess &&
            status == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)ptr;
    }
    return fn;
}

// A row-major bfloat16 matrix [rows, cols] seen through boxes of [box_rows, 64] with 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* base, int rows, int cols, int box_rows) {
    EncodeTiledFn encode = encode_tiled();
    if (encode == nullptr) QIL_REFUSE("gemm_tc: the driver does not offer cuTensorMapEncodeTiled");
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    const cuuint32_t box[2] = {TC_BK, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) QIL_REFUSE("gemm_tc: cuTensorMapEncodeTiled failed with %d for a [%d, %d] matrix", (int)r, rows, cols);
    return 0;
}

extern "C" int qil_gemm_tc_min_rows() { return 17; }

static int launch_gemm_tc(const void* a, const void* w, const void* bias, const void* residual, void* out,
                          int M, int N, int K, int silu_pairs, int sm_count, int* error_word, const TcQkvTail& tail,
                          cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8) QIL_REFUSE("gemm_tc: K %d must be a positive multiple of 8 (16-byte rows for TMA)", K);
    if (N % 8) QIL_REFUSE("gemm_tc: N %d must be a multiple of 8", N);
    if (((uintptr_t)a | (uintptr_t)w | (uintptr_t)out | (uintptr_t)residual) & 15)
        QIL_REFUSE("gemm_tc: operands must be 16-byte aligned");
    if (silu_pairs && (N % 16 || bias != nullptr || residual != nullptr))
        QIL_REFUSE("gemm_tc: silu_pairs needs N %% 16 == 0 and neither bias nor residual");
    if (error_word == nullptr || sm_count <= 0) QIL_REFUSE("gemm_tc: needs an error word and the SM count");
    CUtensorMap map_a, map_w;
    if (make_map(&map_a, a, M, K, TC_BM)) return -1;
    if (make_map(&map_w, w, N, K, TC_BN)) return -1;
    const int smem = TC_STAGES * TC_STAGE_BYTES + (int)sizeof(TcShared) + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) QIL_REFUSE("gemm_tc: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    static int pair_env = -1;
    if (pair_env < 0) {
        const char* e = getenv("QIL_GEMM_TC_PAIRS");
        pair_env = (e != nullptr && e[0] == '0') ? 0 : 1;
    }
    if (M >= 256 && pair_env == 1) {
        // two SMs per 256 x 256 tile; the W map's box is the 128 output features one block loads
        if (make_map(&map_w, w, N, K, 128)) return -1;
        const int smem_pair = T2_STAGES * T2_STAGE_BYTES + (int)sizeof(Tc2Shared) + 1024;
        static int pairs_resident = 0;
        if (pairs_resident == 0) {
            cudaError_t e = cudaFuncSetAttribute(gemm_tc_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_pair);
            if (e != cudaSuccess) QIL_REFUSE("gemm_tc: cannot reserve %d bytes of shared memory: %s", smem_pair, cudaGetErrorString(e));
            cudaLaunchConfig_t config = {};
            config.gridDim = dim3(sm_count & ~1);
            config.blockDim = dim3(192);
            config.dynamicSmemBytes = smem_pair;
            int clusters = 0;
            e = cudaOccupancyMaxActiveClusters(&clusters, gemm_tc_pair_kernel, &config);
            if (e != cudaSuccess || clusters <= 0) { (void)cudaGetLastError(); clusters = sm_count / 2; }
            pairs_resident = clusters < sm_count / 2 ? clusters : sm_count / 2;
        }
        const int pair_tiles = ((M + 255) / 256) * ((N + TC_BN - 1) / TC_BN);
        const int pairs = pair_tiles < pairs_resident ? pair_tiles : pairs_resident;
        gemm_tc_pair_kernel<<<2 * pairs, 192, smem_pair, stream>>>(map_a, map_w, (const bf16*)bias, (const bf16*)residual,
                                                                   (bf16*)out, M, N, K, silu_pairs, error_word, tail);
        QIL_CHECK_LAUNCH();
    }
    const int n_tiles = ((M + TC_BM - 1) / TC_BM) * ((N + TC_BN - 1) / TC_BN);
    const int blocks = n_tiles < sm_count ? n_tiles : sm_count;
    gemm_tc_kernel<<<blocks, 192, smem, stream>>>(map_a, map_w, (const bf16*)bias, (const bf16*)residual, (bf16*)out,
                                                  M, N, K, silu_pairs, error_word, tail);
    QIL_CHECK_LAUNCH();
}

// error_word: a device int the caller zeroes once and reads after synchronising; non-zero means a
// bounded wait inside the kernel ran out (1-2 producer, 3-4 MMA issuer, 5 epilogue).
extern "C" int qil_gemm_tc(const void* a, const void* w, const void* bias, const void* residual, void* out,
                           int M, int N, int K, int silu_pairs, int sm_count, int* error_word, cudaStream_t stream) {
    TcQkvTail none = {};
    return launch_gemm_tc(a, w, bias, residual, out, M, N, K, silu_pairs, sm_count, error_word, none, stream);
}

// The stacked query/key/value projection of heads of 128 with its tail fused (see TcQkvTail): w is
// [(n_q_heads + 2 n_kv_heads) * 128, K] (queries, then keys, then values; n_kv_heads may be 0 for a layer
// that reads another layer's cache), q_out [M, n_q_heads * 128], pages one layer of the cache.  rope
// float32 [rope_rows, 128] (cosines then sines, values representable in bfloat16) or null; q_norm, k_norm
// bfloat16 [128] or null; positions, token_row int32 [M]; block_table int32 rows of table_stride.
extern "C" int qil_gemm_tc_qkv(const void* a, const void* w, const void* bias, void* q_out, void* pages,
                               const float* rope, int rope_rows, const void* q_norm, const void* k_norm, float eps,
                               const int* positions, const int* token_row, const int* block_table, int table_stride,
                               int n_q_heads, int n_kv_heads, int page_size, int num_pages,
                               int M, int K, int sm_count, int* error_word, cudaStream_t stream) {
    if (n_q_heads <= 0 || n_kv_heads < 0) QIL_REFUSE("gemm_tc_qkv: %d query heads, %d kv heads", n_q_heads, n_kv_heads);
    if (q_out == nullptr || positions == nullptr) QIL_REFUSE("gemm_tc_qkv: needs the query buffer and the positions");
    if (n_kv_heads > 0 && (pages == nullptr || token_row == nullptr || block_table == nullptr || page_size <= 0 || num_pages <= 0))
        QIL_REFUSE("gemm_tc_qkv: keys and values need the cache, the block table and the tokens' rows");
    if (((uintptr_t)q_out | (uintptr_t)pages | (uintptr_t)rope | (uintptr_t)q_norm | (uintptr_t)k_norm) & 15)
        QIL_REFUSE("gemm_tc_qkv: buffers must be 16-byte aligned");
    TcQkvTail tail = {};
    tail.q_out = (bf16*)q_out; tail.pages = (bf16*)pages; tail.rope = rope; tail.rope_rows = rope_rows;
    tail.q_norm = (const bf16*)q_norm; tail.k_norm = (const bf16*)k_norm; tail.eps = eps;
    tail.positions = positions; tail.token_row = token_row; tail.block_table = block_table;
    tail.table_stride = table_stride; tail.n_q_heads = n_q_heads; tail.n_kv_heads = n_kv_heads;
    tail.page_size = page_size > 0 ? page_size : 1; tail.num_pages = num_pages;
    const int N = (n_q_heads + 2 * n_kv_heads) * 128;
    return launch_gemm_tc(a, w, bias, nullptr, q_out, M, N, K, 0, sm_count, error_word, tail, stream);
}
