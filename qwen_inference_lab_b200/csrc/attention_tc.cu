// Causal grouped-query attention of whole 128-token query tiles over the paged cache on the
// fifth-generation tensor cores (tcgen05.mma, accumulators in tensor memory, operands brought by
// TMA), for head size 128 and bfloat16.  Same arithmetic as attention_mma.cu (scores = q k^T *
// head_dim^-1/2 over keys j <= the token's absolute position, float32 softmax, times v;
// qil/model.py:59-68); this kernel takes the bulk of long prompt portions, the mma.sync kernel what
// is left over.
//
// One block per (tile of 128 query tokens, query head), 224 threads:
//   warp 0, 6   issue TMA loads: warp 0 the query tile once and then per 64 keys the pages of K, warp 6 the
//               pages of V (one box per page and 64-wide half of the head, 128-byte swizzle);
//   warp 1      one thread issues tcgen05.mma: S = Q K^T (128 x 128 x 128) into one of two score
//               buffers in tensor memory, and O += P V once the softmax warps have published P;
//               it runs one score tile ahead of the softmax;
//   warps 2-5   one thread per query row: tcgen05.ld of its 128 scores, mask, running maximum, exp2,
//               row sum, P as bfloat16 back into tensor memory over the scores it came from (the
//               second MMA takes its first operand from there: no shared memory, no proxy fence),
//               and the rescale of O in tensor memory when the running maximum moved by more than
//               2^8 (until then P is computed against the older maximum, which is exact algebra and
//               safe in float32); finally O / l -> global memory.
// K tiles are K-major operands and V tiles MN-major operands of the same shared-memory image
// ([key][64 elements = 128 bytes] x two halves of the head).
//
// Every mbarrier wait is bounded (about a second), records its place in the error word when it runs
// out and makes its role stop; the block then frees its tensor memory and returns.
#include "common.cuh"
#include <cuda.h>

QIL_ERROR_STORAGE

#define AT_D 128
#define AT_M 128                 // query tokens per block
#ifndef AT_N
#define AT_N 64                  // keys per tile (64: two blocks fit an SM and overlap each other's softmax and MMAs)
#endif
#define AT_QSLAB (AT_M * 128)    // bytes of a [128 query rows][64 elements] slab (also of a P slab: 64 keys)
#define AT_QTILE (2 * AT_QSLAB)  // the query tile: two halves of the head
#define AT_SLAB (AT_N * 128)     // bytes of a [keys][64 elements] slab of K or V
#define AT_TILE (2 * AT_SLAB)    // a K or V tile: two halves of the head
#define AT_TMEM_COLS (AT_N == 64 ? 256 : 512)
#define AT_STAGES 2
#define AT_WAIT_CYCLES 2000000000ll

__device__ __forceinline__ unsigned at_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void at_mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(at_smem(bar)), "r"(count));
}
__device__ __forceinline__ void at_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(at_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void at_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(at_smem(bar)) : "memory");
}
__device__ __forceinline__ bool at_try_wait(unsigned long long* bar, unsigned parity) {
    unsigned done;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}\n"
                 : "=r"(done) : "r"(at_smem(bar)), "r"(parity) : "memory");
    return done != 0;
}
__device__ __forceinline__ bool at_wait(unsigned long long* bar, unsigned parity) {
    if (at_try_wait(bar, parity)) return true;
    const long long start = clock64();
    while (!at_try_wait(bar, parity)) {
        if (clock64() - start > AT_WAIT_CYCLES) return false;
    }
    return true;
}
__device__ __forceinline__ void at_tma_2d(void* smem, const CUtensorMap* map, unsigned long long* bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
                 ::"r"(at_smem(smem)), "l"((unsigned long long)map), "r"(at_smem(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void at_tma_3d(void* smem, const CUtensorMap* map, unsigned long long* bar, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];\n"
                 ::"r"(at_smem(smem)), "l"((unsigned long long)map), "r"(at_smem(bar)), "r"(x), "r"(y), "r"(z) : "memory");
}
// K-major operand: rows of 128 bytes (64 elements of k), 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ unsigned long long at_desc_kmajor(unsigned addr) {
    unsigned long long d = 0;
    d |= (unsigned long long)((addr & 0x3FFFF) >> 4);
    d |= (unsigned long long)1 << 16;
    d |= (unsigned long long)(1024 >> 4) << 32;
    d |= (unsigned long long)1 << 46;
    d |= (unsigned long long)2 << 61;
    return d;
}
// MN-major operand from the same image: 64 elements of n contiguous (one 128-byte row), rows are k;
// the next 64 n lie one slab further (leading offset), the next 8 k lie 1024 bytes further (stride offset).
__device__ __forceinline__ unsigned long long at_desc_mnmajor(unsigned addr) {
    unsigned long long d = 0;
    d |= (unsigned long long)((addr & 0x3FFFF) >> 4);
    d |= (unsigned long long)(AT_SLAB >> 4) << 16;
    d |= (unsigned long long)(1024 >> 4) << 32;
    d |= (unsigned long long)1 << 46;
    d |= (unsigned long long)2 << 61;
    return d;
}
__device__ __forceinline__ void at_mma(unsigned tmem_d, unsigned long long da, unsigned long long db, unsigned idesc, unsigned acc) {
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
                 ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(acc) : "memory");
}
// The same with the first operand in tensor memory (lane = row, two 16-bit elements per 32-bit column,
// the reduction dimension along the columns).
__device__ __forceinline__ void at_mma_ts(unsigned tmem_d, unsigned tmem_a, unsigned long long db, unsigned idesc, unsigned acc) {
    const unsigned zero = 0u;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}\n"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(acc), "r"(zero) : "memory");
}
__device__ __forceinline__ void at_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(at_smem(bar)) : "memory");
}
__device__ __forceinline__ void at_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void at_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }

__device__ __forceinline__ void at_tmem_ld32(unsigned taddr, unsigned (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
}
__device__ __forceinline__ void at_tmem_st32(unsigned taddr, const unsigned (&r)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
                 "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n"
                 ::"r"(taddr),
                   "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                   "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                   "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
                 : "memory");
}
__device__ __forceinline__ void at_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void at_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ float at_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

// Optional time stamps of one block's roles (compile with -DAT_TRACE=1): trace[role * 1024 + event].
#ifdef AT_TRACE
#define AT_STAMP(role, idx) do { if (p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && (idx) < 1024) \
    p.trace[(role) * 1024 + (idx)] = clock64(); } while (0)
#else
#define AT_STAMP(role, idx) do { } while (0)
#endif

struct AtShared {
    unsigned long long q_full;
    unsigned long long k_full[AT_STAGES], k_empty[AT_STAGES];
    unsigned long long v_full[AT_STAGES], v_empty[AT_STAGES];
    unsigned long long s_full[2];
    unsigned long long p_full[2], pv_done;
    unsigned tmem_base;
    unsigned pad;
};

struct AtParams {
    bf16* out;                  // [N, Hq, 128]
    const int* block_table;
    int table_stride;
    int n_q_heads, n_kv_heads, page_size;
    float scale_log2;
    int* error_word;
    long long* trace;           // only read when compiled with AT_TRACE
};

#define AT_VALUE_WARP 6                  // warps: 0 keys, 1 MMA issue, 2-5 softmax, 6 values
#define AT_THREADS 224
__global__ void __launch_bounds__(AT_THREADS, (AT_N == 64) ? 2 : 1)
attn_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
               AtParams p, const int4* __restrict__ tile_info) {
    // swizzled operand tiles need 1024-byte alignment; the declaration asks for it and a misaligned
    // window is refused below rather than padded, so that two blocks fit the SM's shared memory
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* base = smem_raw;
    if ((at_smem(base) & 1023u) != 0) {
        if (threadIdx.x == 0) atomicExch(p.error_word, 31);
        return;
    }
    unsigned char* sQ = base;                               // [2 slabs]
    unsigned char* sK = sQ + AT_QTILE;                      // [stages][2 slabs]
    unsigned char* sV = sK + AT_STAGES * AT_TILE;           // [stages][2 slabs]
    AtShared* sh = reinterpret_cast<AtShared*>(sV + AT_STAGES * AT_TILE);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // heads vary fastest, so all heads of the longest tile start first (tiles come sorted, longest first)
    const int head = blockIdx.x;
    const int kv_head = head / (p.n_q_heads / p.n_kv_heads);
    // tile_info: (first token in the flat batch, its absolute position, 128, block-table row)
    const int4 info = tile_info[blockIdx.y];
    const int n0 = info.x, pos0 = info.y;
    const int hi = pos0 + AT_M - 1;                          // last key any row of the tile may see
    const int n_tiles = hi / AT_N + 1;
    const int* table = p.block_table + (size_t)info.w * p.table_stride;

    if (threadIdx.x == 0) {
        at_mbar_init(&sh->q_full, 1);
        for (int s = 0; s < AT_STAGES; ++s) {
            at_mbar_init(&sh->k_full[s], 1); at_mbar_init(&sh->k_empty[s], 1);
            at_mbar_init(&sh->v_full[s], 1); at_mbar_init(&sh->v_empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) at_mbar_init(&sh->s_full[b], 1);
        at_mbar_init(&sh->p_full[0], 4);
        at_mbar_init(&sh->p_full[1], 4);
        at_mbar_init(&sh->pv_done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(at_smem(&sh->tmem_base)), "r"((unsigned)AT_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    at_fence_before();
    __syncthreads();
    at_fence_after();
    const unsigned tmem = sh->tmem_base;
    auto tmem_s = [tmem](int buffer) { return tmem + (unsigned)(buffer * AT_N); };    // the two score buffers
    const unsigned tmem_o = tmem + 2u * AT_N;

    if (warp == 0 || warp == AT_VALUE_WARP) {
        // Two producer warps, one for the keys (and the queries) and one for the values: a stage of keys is
        // free as soon as the scores of two tiles ago are computed, a stage of values only when that tile's
        // output is, and the next scores must not wait behind a copy of values.  The whole warp walks the
        // tiles: every lane fetches one block-table entry of a batch of 32 in one coalesced read, lane 0
        // waits and arms the barrier, and the copies go out one per lane (lane = half of the head, page of
        // the tile) with page ids handed over by shuffles; issuing a tile's copies from one thread one after
        // the other would cost that thread more than the tile's MMAs take.
        const int kv = warp == 0 ? 0 : 1;
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];\n" ::"l"((unsigned long long)&map_kv) : "memory");
            if (kv == 0) {
                asm volatile("prefetch.tensormap [%0];\n" ::"l"((unsigned long long)&map_q) : "memory");
                // queries: box (64 elements, 1 head, 128 tokens) per half of the head
                at_expect_tx(&sh->q_full, AT_QTILE);
                at_tma_3d(sQ, &map_q, &sh->q_full, 0, head, n0);
                at_tma_3d(sQ + AT_QSLAB, &map_q, &sh->q_full, 64, head, n0);
            }
        }
        unsigned long long* const full = kv == 0 ? sh->k_full : sh->v_full;
        unsigned long long* const empty = kv == 0 ? sh->k_empty : sh->v_empty;
        unsigned char* const tiles = kv == 0 ? sK : sV;
        const int pages_per_tile = AT_N / p.page_size;
        const int tiles_per_batch = 32 / pages_per_tile;       // pages_per_tile is 1, 2, 4 or 8
        const int page_bytes = p.page_size * 128;               // one page of one half: page_size rows of 128 bytes
        const int last_page = hi / p.page_size;
        int ok = 1;
        int my_page = -1;
        for (int j = 0; j < n_tiles; ++j) {
            if (j % tiles_per_batch == 0) {
                const int index = j * pages_per_tile + lane;
                my_page = (index <= last_page && index < p.table_stride) ? table[index] : -1;
            }
            const int stage = j % AT_STAGES;
            const unsigned parity = ((j / AT_STAGES) & 1) ^ 1;
            const int first_key = j * AT_N;
            int pages = pages_per_tile;
            if (first_key + AT_N - 1 > hi) pages = (hi - first_key) / p.page_size + 1;
            const int pg = lane % pages_per_tile, half = (lane / pages_per_tile) & 1;
            const int page = __shfl_sync(0xffffffffu, my_page, (j % tiles_per_batch) * pages_per_tile + pg);
            if (lane == 0) {
                if (!at_wait(&empty[stage], parity)) {
                    atomicExch(p.error_word, 11);
                    ok = 0;
                } else {
                    at_expect_tx(&full[stage], (unsigned)(pages * 2 * page_bytes));
                }
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            if (lane < 2 * pages_per_tile && pg < pages) {
                // cache rows of one layer: ((page * 2 + kv) * kv_heads + kv_head) * page_size + slot
                const int row = ((page * 2 + kv) * p.n_kv_heads + kv_head) * p.page_size;
                at_tma_2d(tiles + stage * AT_TILE + half * AT_SLAB + pg * page_bytes, &map_kv, &full[stage], half * 64, row);
            }
            if (lane == 0) AT_STAMP(0, 2 * j + kv);
        }
        // leave only after the copies have been consumed or have had a second to land
        if (lane == 0 && ok) {
            for (int j = n_tiles; j < n_tiles + AT_STAGES; ++j) {
                if (!at_wait(&empty[j % AT_STAGES], ((j / AT_STAGES) & 1) ^ 1)) {
                    atomicExch(p.error_word, 12);
                    break;
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // bfloat16 -> float32, M = 128; scores: N = keys; output: N = head size, B (V) read MN-major
            const unsigned idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(AT_N >> 3) << 17) | ((unsigned)(AT_M >> 4) << 24);
            const unsigned idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((unsigned)(AT_D >> 3) << 17) | ((unsigned)(AT_M >> 4) << 24);
            bool ok = at_wait(&sh->q_full, 0);
            if (!ok) atomicExch(p.error_word, 13);
            auto issue_scores = [&](int j) -> bool {
                const int stage = j % AT_STAGES, buf = j & 1;
                if (!at_wait(&sh->k_full[stage], (j / AT_STAGES) & 1)) { atomicExch(p.error_word, 14); return false; }
                // The score buffer of tile j held P of tile j - 2: the MMA that read it was issued before this one
                // and MMAs run in the order of their issue, so the buffer needs no barrier of its own.
                at_fence_after();
                const unsigned q_addr = at_smem(sQ), k_addr = at_smem(sK + stage * AT_TILE);
#pragma unroll
                for (int kk = 0; kk < AT_D / 16; ++kk) {
                    // half of the head, then 16 elements = 32 bytes inside the 128-byte row
                    at_mma(tmem_s(buf), at_desc_kmajor(q_addr + (kk >> 2) * AT_QSLAB + (kk & 3) * 32),
                           at_desc_kmajor(k_addr + (kk >> 2) * AT_SLAB + (kk & 3) * 32), idesc_s, kk ? 1u : 0u);
                }
                at_commit(&sh->s_full[buf]);
                at_commit(&sh->k_empty[stage]);
                AT_STAMP(1, 4 * j);
                return true;
            };
            if (ok) ok = issue_scores(0);
            for (int j = 0; j < n_tiles && ok; ++j) {
                if (j + 1 < n_tiles) { ok = issue_scores(j + 1); if (!ok) break; }
                const int stage = j % AT_STAGES;
                if (!at_wait(&sh->v_full[stage], (j / AT_STAGES) & 1)) { atomicExch(p.error_word, 16); ok = false; break; }
                AT_STAMP(1, 4 * j + 1);
                // one barrier per score buffer: the softmax may publish P of the next tile before this thread has
                // looked at this tile's barrier (nothing holds it back but the scores, which are issued above),
                // and a single barrier would then be two phases on, which a parity cannot tell from none
                if (!at_wait(&sh->p_full[j & 1], (j >> 1) & 1)) { atomicExch(p.error_word, 17); ok = false; break; }
                AT_STAMP(1, 4 * j + 2);
                at_fence_after();
                const unsigned v_addr = at_smem(sV + stage * AT_TILE);
#pragma unroll
                for (int kk = 0; kk < AT_N / 16; ++kk) {
                    // P: 16 keys = 8 columns of tensor memory; V: 16 keys = 16 rows of 128 bytes
                    at_mma_ts(tmem_o, tmem_s(j & 1) + kk * 8, at_desc_mnmajor(v_addr + kk * 2048), idesc_pv,
                              (j | kk) ? 1u : 0u);
                }
                at_commit(&sh->pv_done);
                at_commit(&sh->v_empty[stage]);
                AT_STAMP(1, 4 * j + 3);
            }
        }
    } else if (warp < AT_VALUE_WARP) {
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;                 // query row of this thread = its TMEM lane
        const int pos = pos0 + row;
        const unsigned lane_base = (unsigned)(quarter * 32) << 16;
        float m_used = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < n_tiles && ok; ++j) {
            const int buf = j & 1, stage = j % AT_STAGES;
            if (warp == 2 && lane == 0) AT_STAMP(2, 6 * j);
            if (!at_wait(&sh->s_full[buf], (j >> 1) & 1)) { if (lane == 0) atomicExch(p.error_word, 21); ok = false; break; }
            if (warp == 2 && lane == 0) AT_STAMP(2, 6 * j + 1);
            at_fence_after();
            float s[AT_N];
            {
                unsigned r[AT_N / 32][32];
#pragma unroll
                for (int c = 0; c < AT_N / 32; ++c) at_tmem_ld32(tmem_s(buf) + lane_base + c * 32, r[c]);
                at_wait_ld();                                  // one wait for all the loads
#pragma unroll
                for (int c = 0; c < AT_N / 32; ++c)
#pragma unroll
                    for (int i = 0; i < 32; ++i) s[c * 32 + i] = __uint_as_float(r[c][i]);
            }
            if (warp == 2 && lane == 0) AT_STAMP(2, 6 * j + 2);
            // Mask by absolute position (only tiles that reach past the first row's position need it) and take
            // the row's maximum of the raw scores; the scale (positive) is applied to the maximum and, fused
            // with the subtraction, inside the exponent.  Four running maxima and four running sums: one
            // chain of 64 dependent operations would cost this warp, alone on its scheduler, their latency.
            const int key0 = j * AT_N;
            if (key0 + AT_N - 1 > pos0) {
#pragma unroll
                for (int i = 0; i < AT_N; ++i) s[i] = (key0 + i <= pos) ? s[i] : -INFINITY;
            }
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < AT_N; i += 4) {
                mx[0] = fmaxf(mx[0], s[i]); mx[1] = fmaxf(mx[1], s[i + 1]);
                mx[2] = fmaxf(mx[2], s[i + 2]); mx[3] = fmaxf(mx[3], s[i + 3]);
            }
            const float tmax = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * p.scale_log2;
            // Move the maximum only when it grew by more than 2^8: until then exp2(s - m_used) <= 256,
            // harmless in float32 and bfloat16, and O needs no rescale (which costs a TMEM round trip).
            const bool grow = tmax > m_used + 8.0f;            // also true at the first tile (m_used = -inf)
            const float factor = (grow && j > 0) ? at_exp2(m_used - tmax) : 1.0f;
            if (grow) m_used = tmax;
            const float minus_m = (m_used == -INFINITY) ? 0.f : -m_used;
            // P = exp2(s * scale - m) as bfloat16, kept in registers until it is stored
            float sums[4] = {0.f, 0.f, 0.f, 0.f};
            uint4 packed[AT_N / 8];
#pragma unroll
            for (int c = 0; c < AT_N / 8; ++c) {
                float e[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    e[i] = at_exp2(fmaf(s[c * 8 + i], p.scale_log2, minus_m));
                    sums[i & 3] += e[i];
                }
                __nv_bfloat162 b0 = __floats2bfloat162_rn(e[0], e[1]), b1 = __floats2bfloat162_rn(e[2], e[3]);
                __nv_bfloat162 b2 = __floats2bfloat162_rn(e[4], e[5]), b3 = __floats2bfloat162_rn(e[6], e[7]);
                packed[c].x = *reinterpret_cast<unsigned*>(&b0); packed[c].y = *reinterpret_cast<unsigned*>(&b1);
                packed[c].z = *reinterpret_cast<unsigned*>(&b2); packed[c].w = *reinterpret_cast<unsigned*>(&b3);
            }
            const float sum = (sums[0] + sums[1]) + (sums[2] + sums[3]);
            if (warp == 2 && lane == 0) AT_STAMP(2, 6 * j + 3);
            if (__any_sync(0xffffffffu, factor != 1.0f)) {
                // O may be touched once the previous tile's second MMA is done.  (P needs no such wait: it goes
                // over this tile's own scores.  The barrier is at most one phase ahead of the awaited one, as
                // the next second MMA cannot be issued before this warp has published P.)
                if (!at_wait(&sh->pv_done, (j - 1) & 1)) { if (lane == 0) atomicExch(p.error_word, 22); ok = false; break; }
                at_fence_after();
#pragma unroll 1
                for (int c = 0; c < AT_D / 32; ++c) {
                    unsigned r[32];
                    at_tmem_ld32(tmem_o + lane_base + c * 32, r);
                    at_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * factor);
                    at_tmem_st32(tmem_o + lane_base + c * 32, r);
                }
                at_wait_st();
            }
            l = l * factor + sum;
            // on the last tile, value rows past the last visible key may hold anything (unwritten slots):
            // zero them so that 0 * garbage cannot become NaN; they are this thread's key row
            if (j == n_tiles - 1) {
                if (!at_wait(&sh->v_full[stage], (j / AT_STAGES) & 1)) { if (lane == 0) atomicExch(p.error_word, 23); ok = false; break; }
                if (row < AT_N && key0 + row > hi) {
                    unsigned char* v_row = sV + stage * AT_TILE + row * 128;
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        *reinterpret_cast<uint4*>(v_row + c * 16) = make_uint4(0u, 0u, 0u, 0u);
                        *reinterpret_cast<uint4*>(v_row + AT_SLAB + c * 16) = make_uint4(0u, 0u, 0u, 0u);
                    }
                }
            }
            // P over the scores it came from: this thread's row, two keys per 32-bit column
            {
                unsigned words[AT_N / 2];
#pragma unroll
                for (int c = 0; c < AT_N / 8; ++c) {
                    words[4 * c] = packed[c].x; words[4 * c + 1] = packed[c].y;
                    words[4 * c + 2] = packed[c].z; words[4 * c + 3] = packed[c].w;
                }
                static_assert(AT_N == 64, "one 32-column store per row");
                at_tmem_st32(tmem_s(buf) + lane_base, words);
                at_wait_st();
            }
            if (j == n_tiles - 1) asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // the zeroed value rows
            at_fence_before();
            __syncwarp();
            if (lane == 0) at_arrive(&sh->p_full[j & 1]);
            if (warp == 2 && lane == 0) AT_STAMP(2, 6 * j + 5);
        }
        if (ok) {
            if (!at_wait(&sh->pv_done, (n_tiles - 1) & 1)) { if (lane == 0) atomicExch(p.error_word, 24); ok = false; }
        }
        if (ok) {
            at_fence_after();
            const float inv = l > 0.f ? 1.f / l : 0.f;
            bf16* dst = p.out + ((size_t)(n0 + row) * p.n_q_heads + head) * AT_D;
#pragma unroll 1
            for (int c = 0; c < AT_D / 32; ++c) {
                unsigned r[32];
                __syncwarp();
                at_tmem_ld32(tmem_o + lane_base + c * 32, r);
                at_wait_ld();
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    uint4 packed;
                    bf16* o = reinterpret_cast<bf16*>(&packed);
#pragma unroll
                    for (int i = 0; i < 8; ++i) o[i] = __float2bfloat16_rn(__uint_as_float(r[q * 8 + i]) * inv);
                    *reinterpret_cast<uint4*>(dst + c * 32 + q * 8) = packed;
                }
            }
        }
    }
    at_fence_before();
    __syncthreads();
    if (warp == 1) {
        at_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"((unsigned)AT_TMEM_COLS) : "memory");
    }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*AtEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static AtEncodeFn at_encode() {
    static AtEncodeFn fn = nullptr;
    if (fn == nullptr) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult status;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &status) == cudaSuccess &&
            status == cudaDriverEntryPointSuccess)
            fn = (AtEncodeFn)ptr;
    }
    return fn;
}

extern "C" int qil_attn_tc_head_dim() { return AT_D; }
extern "C" int qil_attn_tc_keys_per_tile() { return AT_N; }

// q [N, Hq, 128], kv one layer's pages [pages, 2, Hkv, page_size, 128], out [N, Hq, 128], all bfloat16.
// tile_info int32 [n_tiles, 4] = (first token, its absolute position, 128, block-table row): whole tiles only.
// page_size must divide the keys per tile and be a multiple of 8.  error_word: a device int, zeroed by the
// caller once.  trace: null, or 3 * 1024 int64 for the time stamps of block (0, 0) in a build with AT_TRACE.
extern "C" int qil_attn_tc_prefill(const void* q, const void* kv, void* out, const int* tile_info, int n_tiles,
                                   int n_tokens, const int* block_table, int table_stride, int n_q_heads,
                                   int n_kv_heads, int page_size, int num_pages, float scale, int* error_word,
                                   long long* trace, cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    if (n_kv_heads <= 0 || n_q_heads % n_kv_heads) QIL_REFUSE("attn_tc: %d query heads, %d kv heads", n_q_heads, n_kv_heads);
    if (page_size < 8 || page_size > AT_N || AT_N % page_size || page_size % 8)
        QIL_REFUSE("attn_tc: pages of %d positions; this kernel takes multiples of 8 that divide %d", page_size, AT_N);
    if (n_tiles > 65535) QIL_REFUSE("attn_tc: %d tiles in one launch; at most 65535", n_tiles);
    if (((uintptr_t)q | (uintptr_t)kv | (uintptr_t)out | (uintptr_t)tile_info) & 15) QIL_REFUSE("attn_tc: operands must be 16-byte aligned");
    if (error_word == nullptr) QIL_REFUSE("attn_tc: needs an error word");
    AtEncodeFn encode = at_encode();
    if (encode == nullptr) QIL_REFUSE("attn_tc: the driver does not offer cuTensorMapEncodeTiled");
    CUtensorMap map_q, map_kv;
    {
        const cuuint64_t dims[3] = {AT_D, (cuuint64_t)n_q_heads, (cuuint64_t)n_tokens};
        const cuuint64_t strides[2] = {AT_D * 2, (cuuint64_t)n_q_heads * AT_D * 2};
        const cuuint32_t box[3] = {64, 1, AT_M};
        const cuuint32_t elem[3] = {1, 1, 1};
        const CUresult r = encode(&map_q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, elem,
                                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) QIL_REFUSE("attn_tc: cuTensorMapEncodeTiled failed for the queries (%d)", (int)r);
    }
    {
        const cuuint64_t rows = (cuuint64_t)num_pages * 2 * n_kv_heads * page_size;
        const cuuint64_t dims[2] = {AT_D, rows};
        const cuuint64_t strides[1] = {AT_D * 2};
        const cuuint32_t box[2] = {64, (cuuint32_t)page_size};
        const cuuint32_t elem[2] = {1, 1};
        const CUresult r = encode(&map_kv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(kv), dims, strides, box, elem,
                                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) QIL_REFUSE("attn_tc: cuTensorMapEncodeTiled failed for the cache (%d)", (int)r);
    }
    AtParams p;
    p.out = (bf16*)out; p.block_table = block_table; p.table_stride = table_stride;
    p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads; p.page_size = page_size;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.error_word = error_word;
    p.trace = trace;
    const int smem = AT_QTILE + 2 * AT_STAGES * AT_TILE + (int)sizeof(AtShared);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) QIL_REFUSE("attn_tc: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    attn_tc_kernel<<<dim3(n_q_heads, n_tiles), AT_THREADS, smem, stream>>>(map_q, map_kv, p, (const int4*)tile_info);
    QIL_CHECK_LAUNCH();
}
