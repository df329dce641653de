// Flash-style causal attention for prompt portions on the 5th-generation tensor cores
// (head size 128, bf16 pages).  Formula as in attention.cu
// (src/backend/cpu/cpu_backend.cpp:174-198); softmax statistics and the output are fp32.
//
// One block handles 128 query rows -- (token, head-of-group) pairs, so the heads of a group share
// every key tile -- of one key/value head and walks the key tiles of 64 keys up to the causal
// diagonal:
//   warp 0      fetches key and value pages by TMA (one box per page and 64-wide half, 128-byte
//               swizzle) into two rings: a key tile is free once S = Q K^T has read it, its values
//               only after O += P V, so keys (two stages) run as far ahead as values (three);
//   warp 1      issues tcgen05.mma: S_j = Q K_j^T (128 x 64, accumulator in tensor memory, two
//               buffers) and O_j = P_j V_j (128 x 128, V read MN-major straight from the page layout);
//   warps 2-5   own one query row per thread: they read S_j from tensor memory (tcgen05.ld), keep
//               the reference maximum and the denominator, and write P_j = exp2(S_j - max) as packed
//               bf16 back into the tensor-memory columns S_j came from; the second product takes P
//               straight from tensor memory (A operand) and accumulates O in tensor memory.
//               The reference maximum of a row is only raised when the true maximum has grown by
//               more than 8 (a factor 256, harmless in bf16 and fp32); then the row of O is rescaled
//               in tensor memory (tcgen05.ld / tcgen05.st).  After the first tiles this is rare, so O
//               stays in tensor memory and the output registers are only filled at the end.
// S_{j+1} is multiplied while the rows of S_j are being exponentiated.  What bounds a tile is the
// issuing thread (a tcgen05.mma costs it about 60 cycles, a wait that passes at once 100, twelve
// instructions and four commits a tile) and the chain S visible -> exponentials -> P ready -> O += P V;
// measured per 64-key tile: 2,200 cycles, of which the softmax warps work 960.  Every wait is bounded
// (EMBER_ERR_WAIT_LIMIT) and the tensor memory is freed on every path.
//
// The reference's prefill attention (src/backend/cuda/k_attention.cu:214-370) is a Turing
// mma.sync kernel; only the mathematics is shared.
#include <cuda.h>

#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"

EMBER_DEFINE_LAST_ERROR

namespace ember {

constexpr int FA_ROWS = 128;          // query rows per block = TMEM lanes
constexpr int FA_KT = 64;             // keys per tile
constexpr int FA_D = 128;             // head size
constexpr int FA_K_STAGES = 2;        // key tiles in flight or in use (a key tile is free once S = Q K^T has read it,
                                      // two tiles before its values are: two stages look as far ahead as three of values)
constexpr int FA_V_STAGES = 3;        // value tiles (free once O += P V has read them)
constexpr int FA_THREADS = 192;
constexpr float FA_LOG2E = 1.4426950408889634f;

struct FaParams {
    const __nv_bfloat16* q;   // [T, n_heads, 128]
    __nv_bfloat16* out;       // [T, n_heads, 128]
    const int* tiles;         // [n_tiles, 4] = (sequence, first token row, queries, position of the first query)
    const int* block_table;
    int max_blocks, page, num_pages;
    int n_heads, n_kv;
    int window;
    float scale_log2;
    int n_tiles;
    int* err;
};

__device__ __forceinline__ uint32_t fa_s32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void fa_mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(fa_s32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fa_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(fa_s32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void fa_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(fa_s32(bar)) : "memory");
}
__device__ __forceinline__ bool fa_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    return mbarrier_wait_bounded(fa_s32(bar), parity, abort_flag);      // bounded by time (common.cuh)
}
__device__ __forceinline__ void fa_tma_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(fa_s32(dst)), "l"((uint64_t)map), "r"(fa_s32(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void fa_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(fa_s32(bar)) : "memory");
}
__device__ __forceinline__ void fa_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// Second product: the A operand (P, packed bf16 pairs, one row per lane) is read from tensor memory.
__device__ __forceinline__ void fa_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void fa_tmem_st32(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
          "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
          "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void fa_tmem_ld16(uint32_t taddr, float* v) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; i++) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ void fa_tmem_ld32_nowait(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void fa_tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void fa_tmem_st16(uint32_t taddr, const float* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
          "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])),
          "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])),
          "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
          "r"(__float_as_uint(v[15]))
        : "memory");
}
__device__ __forceinline__ void fa_tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// K-major operand tile: rows of 128 bytes (64 bf16), 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t fa_desc_k(const void* tile) {
    const uint64_t addr = (uint64_t)(fa_s32(tile) >> 4) & 0x3FFFull;
    return addr | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// MN-major operand (the value tile: keys are the K dimension, head elements the N dimension): each key is a
// 128-byte row of 64 head elements; 8-key groups are 1024 bytes apart (stride byte offset) and the second
// 64-element half of the head lies `half_bytes` further (leading byte offset).
__device__ __forceinline__ uint64_t fa_desc_mn(const void* tile, uint32_t half_bytes) {
    const uint64_t addr = (uint64_t)(fa_s32(tile) >> 4) & 0x3FFFull;
    return addr | ((uint64_t)((half_bytes >> 4) & 0x3FFF) << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: fp32 accumulate, bf16 operands, A K-major, M = 128.
__device__ __forceinline__ uint32_t fa_idesc(int n, int b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(FA_ROWS >> 4) << 24);
}

__device__ __forceinline__ float fa_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t fa_swz(int row, int chunk) { return (uint32_t)(row * 128 + ((chunk ^ (row & 7)) << 4)); }

__global__ void __launch_bounds__(FA_THREADS, 2)
attention_fa_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const FaParams p) {
    constexpr int Q_HALF = FA_ROWS * 128;                // 16 KiB: [128 rows][64 bf16]
    constexpr int KV_HALF = FA_KT * 128;                 // 8 KiB:  [64 keys][64 bf16]
    constexpr int KV_TILE = 2 * KV_HALF;                 // 16 KiB
    // 1024-byte alignment (needed by the 128-byte swizzle) is asked of the declaration instead of padded for:
    // two blocks have to fit into one SM's shared memory
    extern __shared__ __align__(1024) uint8_t fa_smem_raw[];
    uint8_t* smem = fa_smem_raw;
    if ((fa_s32(smem) & 1023u) != 0) {
        if (threadIdx.x == 0 && p.err) atomicOr(p.err, EMBER_ERR_WAIT_LIMIT);
        return;
    }
    uint8_t* q_s = smem;                                  // 32 KiB, two halves
    uint8_t* k_s = q_s + 2 * Q_HALF;                      // FA_K_STAGES x 16 KiB
    uint8_t* v_s = k_s + FA_K_STAGES * KV_TILE;           // FA_V_STAGES x 16 KiB
    uint64_t* k_full = (uint64_t*)(v_s + FA_V_STAGES * KV_TILE);
    uint64_t* k_empty = k_full + FA_K_STAGES;
    uint64_t* v_full = k_empty + FA_K_STAGES;
    uint64_t* v_empty = v_full + FA_V_STAGES;
    uint64_t* s_full = v_empty + FA_V_STAGES;             // [2]
    uint64_t* q_ready = s_full + 2;
    uint64_t* p_full = q_ready + 1;                       // [2]: the softmax warps may be a tile ahead of the MMA thread
    uint64_t* pv_full = p_full + 2;
    uint64_t* o_done = pv_full + 1;                       // the last O += P V has finished
    uint32_t* tmem_slot = (uint32_t*)(o_done + 1);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = p.n_tiles - 1 - (int)blockIdx.x;     // later tiles have more keys: start them first
    const int kvh = blockIdx.y;
    const int seq = p.tiles[tile * 4 + 0], row0 = p.tiles[tile * 4 + 1], nq = p.tiles[tile * 4 + 2],
              pos0 = p.tiles[tile * 4 + 3];
    const int G = p.n_heads / p.n_kv;
    const int rows = nq * G;
    const int lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
    const int hi = pos0 + nq;
    const int k_begin = lo - (lo % FA_KT);
    const int n_kt = hi > k_begin ? (hi - k_begin + FA_KT - 1) / FA_KT : 0;

    if (threadIdx.x == 0) {
        for (int i = 0; i < FA_K_STAGES; i++) {
            fa_mbar_init(&k_full[i], 1);
            fa_mbar_init(&k_empty[i], 1);
        }
        for (int i = 0; i < FA_V_STAGES; i++) {
            fa_mbar_init(&v_full[i], 1);
            fa_mbar_init(&v_empty[i], 1);
        }
        for (int i = 0; i < 2; i++) {
            fa_mbar_init(&s_full[i], 1);
        }
        fa_mbar_init(q_ready, 4);
        fa_mbar_init(&p_full[0], 4);
        fa_mbar_init(&p_full[1], 4);
        fa_mbar_init(pv_full, 1);
        fa_mbar_init(o_done, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(fa_s32(tmem_slot)), "r"(256) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    const uint32_t tmem_s0 = tmem, tmem_o = tmem + 128;   // S buffers at columns 0 and 64, O tile at 128

    pdl_launch_dependents();
    pdl_wait();

    if (warp == 0) {
        // ---------------------------------------------------------------- page fetcher
        const int* bt = p.block_table + (size_t)seq * p.max_blocks;
        const int boxes = FA_KT / p.page;
        auto page_row = [&](int it) {
            int blk = 0;
            if (lane < boxes && it < n_kt) {
                blk = bt[min((k_begin + it * FA_KT + lane * p.page) / p.page, p.max_blocks - 1)];
                if (blk < 0 || blk >= p.num_pages) blk = 0;
            }
            return (blk * p.n_kv + kvh) * p.page;
        };
        // Keys and values travel in rings of their own: a key tile is free as soon as S = Q K^T has read it,
        // long before the value tile of the same keys, so key tiles are requested three tiles ahead and the
        // latency of a fetch (16 small boxes a tile with 16-token pages) stays off the critical path.
        // (the tensor maps are named directly: the copy instruction wants the address of the kernel parameter)
        auto fetch_k = [&](uint8_t* dst, uint64_t* bar, int y) {
            if (lane == 0) fa_expect_tx(bar, (uint32_t)KV_TILE);
            __syncwarp();
            if (lane < boxes) {
#pragma unroll
                for (int h = 0; h < 2; h++) fa_tma_2d(dst + h * KV_HALF + lane * p.page * 128, &map_k, bar, h * 64, y);
            }
        };
        auto fetch_v = [&](uint8_t* dst, uint64_t* bar, int y) {
            if (lane == 0) fa_expect_tx(bar, (uint32_t)KV_TILE);
            __syncwarp();
            if (lane < boxes) {
#pragma unroll
                for (int h = 0; h < 2; h++) fa_tma_2d(dst + h * KV_HALF + lane * p.page * 128, &map_v, bar, h * 64, y);
            }
        };
        bool ok = true;
        // order of need: K_0 .. K_{ks-1}, then V_i before K_{i + ks}
        int yk = page_row(0);
        for (int it = 0; it < min(n_kt, FA_K_STAGES); it++) {
            const int y_next = page_row(it + 1);
            fetch_k(k_s + it * KV_TILE, &k_full[it], yk);
            yk = y_next;
        }
        int yv = page_row(0);
        for (int it = 0; it < n_kt && ok; it++) {
            const int bv = it % FA_V_STAGES;
            const int yv_next = page_row(it + 1);
            if (it >= FA_V_STAGES) ok = fa_wait(&v_empty[bv], (uint32_t)(it / FA_V_STAGES - 1) & 1u, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            fetch_v(v_s + bv * KV_TILE, &v_full[bv], yv);
            yv = yv_next;
            const int ik = it + FA_K_STAGES;
            if (ik < n_kt) {
                const int bk = ik % FA_K_STAGES;
                const int yk_next = page_row(ik + 1);
                ok = fa_wait(&k_empty[bk], (uint32_t)(ik / FA_K_STAGES - 1) & 1u, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                fetch_k(k_s + bk * KV_TILE, &k_full[bk], yk);
                yk = yk_next;
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0 && n_kt > 0) {
            const uint32_t idesc_s = fa_idesc(FA_KT, 0), idesc_o = fa_idesc(FA_D, 1);
            bool ok = fa_wait(q_ready, 0, abort_flag);
            // operand descriptors are made once: the issuing thread is the critical path of a tile (every
            // instruction it spends between two waits is time the softmax warps wait for S)
            uint64_t dq[FA_D / 16];
#pragma unroll
            for (int kk = 0; kk < FA_D / 16; kk++) dq[kk] = fa_desc_k(q_s + (kk >> 2) * Q_HALF) + (uint64_t)(2 * (kk & 3));
            const uint64_t dk0 = fa_desc_k(k_s), dv0 = fa_desc_mn(v_s, KV_HALF);      // stage b: + b * KV_TILE / 16
            auto issue_s = [&](int j) {
                const int b = j % FA_K_STAGES;
                const uint32_t d = tmem_s0 + (uint32_t)((j & 1) * FA_KT);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int kk = 0; kk < FA_D / 16; kk++) {
                    // second half of the head: KV_HALF bytes further; 16 elements: 32 bytes inside the swizzled row
                    const uint64_t db = dk0 + (uint64_t)((b * KV_TILE + (kk >> 2) * KV_HALF) >> 4) + (uint64_t)(2 * (kk & 3));
                    fa_mma(d, dq[kk], db, idesc_s, kk > 0 ? 1u : 0u);
                }
                fa_commit(&s_full[j & 1]);
                fa_commit(&k_empty[b]);          // the keys of tile j are no longer read
            };
            if (ok) ok = fa_wait(&k_full[0], 0, abort_flag);
            if (ok) issue_s(0);
            for (int j = 0; j < n_kt && ok; j++) {
                if (j + 1 < n_kt) {
                    ok = fa_wait(&k_full[(j + 1) % FA_K_STAGES], (uint32_t)((j + 1) / FA_K_STAGES) & 1u, abort_flag);
                    // S_{j+1} reuses the columns of S_{j-1} / P_{j-1}: the second product of tile j - 1 was
                    // issued before and the tensor core runs in order, and p_full(j - 1) said S_{j-1} was read
                    if (!ok) break;
                    issue_s(j + 1);
                }
                const int b = j % FA_V_STAGES;
                // (one barrier per S buffer: the softmax warps finish tile j + 1 without this thread, so a single
                // barrier could complete twice before it is looked at here)
                ok = fa_wait(&p_full[j & 1], (uint32_t)(j >> 1) & 1u, abort_flag);
                if (ok) ok = fa_wait(&v_full[b], (uint32_t)(j / FA_V_STAGES) & 1u, abort_flag);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int kk = 0; kk < FA_KT / 16; kk++) {
                    // P_j: 64 keys = 32 packed columns in the S buffer of tile j; 16 keys = 8 columns per step
                    const uint32_t pa = tmem_s0 + (uint32_t)((j & 1) * FA_KT + kk * 8);
                    const uint64_t db = dv0 + (uint64_t)((b * KV_TILE + kk * 16 * 128) >> 4);
                    fa_mma_ts(tmem_o, pa, db, idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
                }
                fa_commit(&v_empty[b]);         // the values of tile j are no longer read
                fa_commit(pv_full);             // O_j is complete, P may be overwritten
                if (j == n_kt - 1) fa_commit(o_done);
            }
        }
    } else {
        // ------------------------------------------------- softmax / accumulation: one row per thread
        const int quad = warp & 3;
        const int r = quad * 32 + lane;
        const int qi = min(r, rows - 1) / G;
        const int qpos = pos0 + qi;
        // query rows -> shared memory (zero beyond `rows`)
        {
            const int rq = r / G, rg = r - rq * G;
            const __nv_bfloat16* src = p.q + ((size_t)(row0 + rq) * p.n_heads + kvh * G + rg) * FA_D;
#pragma unroll
            for (int c = 0; c < 16; c++) {
                uint4 val = make_uint4(0, 0, 0, 0);
                if (r < rows) val = *reinterpret_cast<const uint4*>(src + c * 8);
                *reinterpret_cast<uint4*>(q_s + (c >> 3) * Q_HALF + fa_swz(r, c & 7)) = val;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) fa_arrive(q_ready);
        }
        float m_ref = -INFINITY, l_run = 0.0f;      // reference maximum (exponent base) and denominator
        const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
        bool ok = true;
        for (int j = 0; j < n_kt; j++) {
            const int k0 = k_begin + j * FA_KT;
            if (ok) ok = fa_wait(&s_full[j & 1], (uint32_t)(j >> 1) & 1u, abort_flag);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t su[FA_KT];
            fa_tmem_ld32_nowait(tmem_s0 + lane_base + (uint32_t)((j & 1) * FA_KT), su);
            fa_tmem_ld32_nowait(tmem_s0 + lane_base + (uint32_t)((j & 1) * FA_KT + 32), su + 32);
            fa_tmem_wait_ld();
            float* s = reinterpret_cast<float*>(su);

            const bool interior = k0 >= lo && k0 + FA_KT <= hi && k0 + FA_KT - 1 <= pos0 &&
                                  (p.window <= 0 || k0 > pos0 + (rows - 1) / G - p.window);
            // the maximum is taken over the raw scores; the scale (> 0) is folded into the exponent below
            float tmax;
            if (!interior) {
#pragma unroll
                for (int i = 0; i < FA_KT; i++) {
                    const int key = k0 + i;
                    const bool vis = key >= lo && key < hi && key <= qpos && (p.window <= 0 || key > qpos - p.window);
                    s[i] = vis ? s[i] : -INFINITY;
                }
            }
            {   // four independent chains instead of one of 64 dependent maxima
                float t0 = s[0], t1 = s[1], t2 = s[2], t3 = s[3];
#pragma unroll
                for (int i = 4; i < FA_KT; i += 4) {
                    t0 = fmaxf(t0, s[i]);
                    t1 = fmaxf(t1, s[i + 1]);
                    t2 = fmaxf(t2, s[i + 2]);
                    t3 = fmaxf(t3, s[i + 3]);
                }
                tmax = fmaxf(fmaxf(t0, t1), fmaxf(t2, t3));
            }
            tmax *= p.scale_log2;
            // raise the reference maximum only when the true one has outgrown it by more than 2^8
            const bool raise = tmax > m_ref + 8.0f || (m_ref == -INFINITY && tmax > -INFINITY);
            const bool warp_raise = __any_sync(0xffffffffu, raise);
            if (warp_raise && j > 0) {
                // O is complete up to tile j - 1 once the previous second product has finished
                if (ok) ok = fa_wait(pv_full, (uint32_t)(j - 1) & 1u, abort_flag);
                const float factor = raise ? (m_ref == -INFINITY ? 0.0f : exp2f(m_ref - tmax)) : 1.0f;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int c = 0; c < FA_D / 16; c++) {
                    float t[16];
                    fa_tmem_ld16(tmem_o + lane_base + (uint32_t)(c * 16), t);
#pragma unroll
                    for (int i = 0; i < 16; i++) t[i] *= factor;
                    fa_tmem_st16(tmem_o + lane_base + (uint32_t)(c * 16), t);
                }
                fa_tmem_wait_st();
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            }
            if (raise) {
                l_run *= m_ref == -INFINITY ? 0.0f : exp2f(m_ref - tmax);
                m_ref = tmax;
            }
            const float neg_base = m_ref == -INFINITY ? 0.0f : -m_ref;
            float sum0 = 0.0f, sum1 = 0.0f, sum2 = 0.0f, sum3 = 0.0f;
            uint32_t packed[FA_KT / 2];
#pragma unroll
            for (int i = 0; i < FA_KT / 2; i += 2) {
                const float p0 = fa_ex2(fmaf(s[2 * i], p.scale_log2, neg_base)), p1 = fa_ex2(fmaf(s[2 * i + 1], p.scale_log2, neg_base));
                const float p2 = fa_ex2(fmaf(s[2 * i + 2], p.scale_log2, neg_base)), p3 = fa_ex2(fmaf(s[2 * i + 3], p.scale_log2, neg_base));
                sum0 += p0; sum1 += p1; sum2 += p2; sum3 += p3;
                __nv_bfloat162 h2 = __floats2bfloat162_rn(p0, p1), h3 = __floats2bfloat162_rn(p2, p3);
                packed[i] = *reinterpret_cast<uint32_t*>(&h2);
                packed[i + 1] = *reinterpret_cast<uint32_t*>(&h3);
            }
            const float sum = (sum0 + sum1) + (sum2 + sum3);
            // P_j replaces S_j in tensor memory (its first 32 columns)
            fa_tmem_st32(tmem_s0 + lane_base + (uint32_t)((j & 1) * FA_KT), packed);
            fa_tmem_wait_st();
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            l_run += sum;
            __syncwarp();
            if (lane == 0) fa_arrive(&p_full[j & 1]);
        }
        // (a barrier of its own: the rows of the last tile can be done while O += P V of the tile before the last
        // still waits for its values, two phases of pv_full behind, and a parity cannot tell two phases apart;
        // the wait in the loop above is safe, S_j being complete only after O += P V of tile j - 2)
        if (n_kt > 0 && ok) ok = fa_wait(o_done, 0, abort_flag);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (n_kt > 0) {
            const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
            const int rq = r / G, rg = r - rq * G;
            __nv_bfloat16* dst = p.out + ((size_t)(row0 + rq) * p.n_heads + kvh * G + rg) * FA_D;
#pragma unroll
            for (int c = 0; c < FA_D / 32; c++) {
                uint32_t tu[32];
                fa_tmem_ld32_nowait(tmem_o + lane_base + (uint32_t)(c * 32), tu);
                fa_tmem_wait_ld();
                if (ok && r < rows) {
#pragma unroll
                    for (int q4 = 0; q4 < 4; q4++) {
                        uint4 packed;
                        __nv_bfloat162* h2 = (__nv_bfloat162*)&packed;
#pragma unroll
                        for (int e = 0; e < 4; e++)
                            h2[e] = __floats2bfloat162_rn(__uint_as_float(tu[q4 * 8 + 2 * e]) * inv, __uint_as_float(tu[q4 * 8 + 2 * e + 1]) * inv);
                        *reinterpret_cast<uint4*>(dst + c * 32 + q4 * 8) = packed;
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag && p.err) atomicOr(p.err, EMBER_ERR_WAIT_LIMIT);
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256) : "memory");
    }
}

typedef CUresult (*FaEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static FaEncodeFn fa_encode_fn() {
    static FaEncodeFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (FaEncodeFn)ptr;
    });
    return fn;
}

static bool fa_pool_map(const void* pool, long long total_rows, int page, CUtensorMap* out) {
    static std::map<std::tuple<const void*, long long, int>, CUtensorMap> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    auto key = std::make_tuple(pool, total_rows, page);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return true;
    }
    FaEncodeFn fn = fa_encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)FA_D, (cuuint64_t)total_rows};
    cuuint64_t strides[1] = {(cuuint64_t)FA_D * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)page};
    cuuint32_t elem[2] = {1, 1};
    CUtensorMap m;
    if (fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pool), dims, strides, box, elem,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    if (cache.size() > 4096) cache.clear();
    cache[key] = m;
    *out = m;
    return true;
}

}  // namespace ember

using namespace ember;

// 1 if this kernel takes the geometry: head size 128, a group size that divides 128, pages of 16/32/64.
EMBER_API int ember_attention_fa_supported(int D, int group, int page) {
    if (D != FA_D) return 0;
    if (page != 16 && page != 32 && page != 64) return 0;
    return group >= 1 && group <= FA_ROWS && FA_ROWS % group == 0;
}

// Query tokens per tile.
EMBER_API int ember_attention_fa_tile_queries(int group) { return group >= 1 && FA_ROWS % group == 0 ? FA_ROWS / group : 0; }

EMBER_API int ember_attention_fa(const void* q, const void* k_pool, const void* v_pool, void* out, int n_heads, int n_kv,
                                 int D, const int* tiles, int n_tiles, const int* block_table, int max_blocks, int page,
                                 int num_pages, int window, float scale, int* err, void* stream) {
    if (n_tiles <= 0) return 0;
    if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv) return fail("attention_fa: bad head counts %d/%d", n_heads, n_kv);
    if (!ember_attention_fa_supported(D, n_heads / n_kv, page))
        return fail("attention_fa: head size %d, group %d, page %d are not taken", D, n_heads / n_kv, page);
    if (n_kv > 65535) return fail("attention_fa: grid too large");
    CUtensorMap mk, mv;
    const long long total_rows = (long long)num_pages * n_kv * page;
    if (!fa_pool_map(k_pool, total_rows, page, &mk) || !fa_pool_map(v_pool, total_rows, page, &mv))
        return fail("attention_fa: cuTensorMapEncodeTiled failed or is unavailable");
    FaParams p;
    p.q = (const __nv_bfloat16*)q; p.out = (__nv_bfloat16*)out; p.tiles = tiles; p.block_table = block_table;
    p.max_blocks = max_blocks; p.page = page; p.num_pages = num_pages; p.n_heads = n_heads; p.n_kv = n_kv;
    p.window = window; p.scale_log2 = scale * FA_LOG2E; p.n_tiles = n_tiles; p.err = err;
    const size_t smem = (size_t)2 * FA_ROWS * 128 + (size_t)(FA_K_STAGES + FA_V_STAGES) * 2 * FA_KT * 128 + 256;
    static bool attr = false;
    if (!attr) {
        cudaError_t e = cudaFuncSetAttribute(attention_fa_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail("attention_fa: shared memory %zu: %s", smem, cudaGetErrorString(e));
        cudaFuncSetAttribute(attention_fa_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
        attr = true;
    }
    launch_kernel(attention_fa_kernel, dim3(n_tiles, n_kv), dim3(FA_THREADS), smem, (cudaStream_t)stream, mk, mv, p);
    return check_launch("attention_fa");
}
