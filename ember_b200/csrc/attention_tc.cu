// bf16 attention over the paged cache on tensor cores, for head sizes 64 and 128.
//
// Formula as in attention.cu (src/backend/cpu/cpu_backend.cpp:174-198); softmax statistics, the
// running maximum, the denominators and the output accumulators are fp32.
//
// Key and value pages are fetched by TMA (cp.async.bulk.tensor with the 128-byte swizzle, one
// box per page and 64-element half of the head) into a double-buffered shared-memory tile of 64
// keys; completion is signalled on mbarriers; fragments are read with ldmatrix and multiplied
// with mma.sync m16n8k16 (bf16 in, fp32 accumulate).  Scores never leave registers (flash-style
// online softmax).  A work unit is one tile of query rows x one key/value head; the rows are
// (query token, query head of the group) pairs, so all heads of a group share each key tile.
//
// Two modes share the code:
//   PREFILL: up to 64 rows (64 / group consecutive query tokens); each of the 4 warps owns 16 rows
//            and walks all keys up to the causal diagonal.
//   DECODE:  one query token (group <= 16 rows); the 4 warps split every 64-key tile between them
//            and are merged in shared memory; long contexts are also split over gridDim.z into
//            fixed key ranges whose partial results attention_combine merges in ascending order.
//
// Every mbarrier wait is bounded (EMBER_ERR_WAIT_LIMIT is recorded and the block falls through).
// The reference's attention kernels (src/backend/cuda/k_attention.cu:29-370) are Turing
// mma.sync/SIMT kernels with manual gathers; this file shares only the mathematics.
#include <cuda.h>

#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"

EMBER_DEFINE_LAST_ERROR

namespace ember {

constexpr int KT = 64;                 // keys per shared-memory tile
constexpr int ATC_CONSUMERS = 128;     // four warps multiply
constexpr int ATC_THREADS = 160;       // + one warp that only fetches pages
constexpr float LOG2E = 1.4426950408889634f;

struct AttnTcParams {
    const __nv_bfloat16* q;   // [T, n_heads, D]
    __nv_bfloat16* out;       // [T, n_heads, D]
    float* part_o;            // [T, n_heads, n_splits, D]
    float* part_ml;           // [T, n_heads, n_splits, 2] (max in natural-log units, denominator)
    const int* tiles;         // [n_tiles, 4] = (sequence, first token row, queries, position of the first query)
    const int* block_table;
    int max_blocks, page, num_pages;
    int n_heads, n_kv;
    int window;
    float scale_log2;         // softmax scale * log2(e)
    int n_splits, split_keys;
    int n_tiles;
    int cluster_merge;        // the splits of a tile are a thread-block cluster and are merged in its first block's shared memory
    int* err;
};

__device__ __forceinline__ uint32_t s32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ void atc_mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void atc_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void atc_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s32(bar)) : "memory");
}
__device__ __forceinline__ bool atc_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    return mbarrier_wait_bounded(s32(bar), parity, abort_flag);      // bounded by time (common.cuh)
}
__device__ __forceinline__ void atc_tma_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(s32(dst)), "l"((uint64_t)map), "r"(s32(bar)), "r"(x), "r"(y) : "memory");
}

__device__ __forceinline__ uint32_t atc_map_to_rank(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void atc_st_cluster(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void atc_cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void atc_cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

// Byte offset of (row, 16-byte chunk) inside a [rows][64 bf16] half-tile with the 128-byte swizzle.
__device__ __forceinline__ uint32_t swz(int row, int chunk) { return (uint32_t)(row * 128 + ((chunk ^ (row & 7)) << 4)); }

// HALVES = head_dim / 64.  DECODE: warps split the keys of a tile; else warps split the rows.
template <int HALVES, bool DECODE>
__global__ void __launch_bounds__(ATC_THREADS)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                    const AttnTcParams p) {
    constexpr int D = HALVES * 64;
    constexpr int HALF_BYTES = KT * 128;            // one 64-wide half of a 64-row tile: 8 KiB
    constexpr int TILE_BYTES = HALVES * HALF_BYTES; // Q, K or V tile
    constexpr int NKG = DECODE ? 2 : 8;             // groups of 8 keys a warp scores per tile
    constexpr int ND = D / 8;                       // output column groups of 8
    constexpr int NSTAGE = DECODE ? 3 : 2;          // key/value tiles in flight or in use
    constexpr int QROWS = DECODE ? 16 : 64;         // query rows kept in shared memory
    constexpr int Q_HALF_BYTES = QROWS * 128;

    extern __shared__ uint8_t atc_smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)atc_smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* q_s = smem;                            // HALVES x [QROWS][64]
    uint8_t* k_s = q_s + ((HALVES * Q_HALF_BYTES + 1023) & ~1023);   // NSTAGE buffers
    uint8_t* v_s = k_s + NSTAGE * TILE_BYTES;       // NSTAGE buffers
    uint64_t* full_bar = (uint64_t*)(v_s + NSTAGE * TILE_BYTES);
    uint64_t* empty_bar = full_bar + NSTAGE;
    volatile int* abort_flag = (volatile int*)(empty_bar + NSTAGE);
    // cluster merge (decode): what every split of the tile hands to the first one: [splits][rows][D] sums, then
    // [splits][rows][2] maxima (log2 units) and denominators.  A region of its own: it is written by the other
    // blocks while this one may still be multiplying.
    float* recv = reinterpret_cast<float*>((reinterpret_cast<uintptr_t>(abort_flag + 1) + 15) & ~(uintptr_t)15);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g8 = lane >> 2, t4 = lane & 3;
    const int tile = p.n_tiles - 1 - (int)blockIdx.x;      // later tiles have more keys: start them first
    const int kvh = blockIdx.y, split = blockIdx.z;
    const int seq = p.tiles[tile * 4 + 0], row0 = p.tiles[tile * 4 + 1], nq = p.tiles[tile * 4 + 2],
              pos0 = p.tiles[tile * 4 + 3];
    const int G = p.n_heads / p.n_kv;
    const int rows = nq * G;

    int lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
    int hi = pos0 + nq;
    if (p.n_splits > 1) {
        lo = max(lo, split * p.split_keys);
        hi = min(hi, (split + 1) * p.split_keys);
    }
    const int k_begin = lo - (lo % KT);
    const int n_kt = hi > k_begin ? (hi - k_begin + KT - 1) / KT : 0;

    if (threadIdx.x == 0) {
        for (int i = 0; i < NSTAGE; i++) {
            atc_mbar_init(&full_bar[i], 1);
            atc_mbar_init(&empty_bar[i], 4);        // one arrival per multiplying warp
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }

    const bool merge_in_cluster = DECODE && p.cluster_merge && p.n_splits > 1;
    if (merge_in_cluster) atc_cluster_arrive();     // phase 1: every block of the cluster runs before anyone writes to it
    pdl_launch_dependents();
    pdl_wait();       // queries and the newest keys are written by the kernel before this one

    // ---- query rows -> shared memory (row r = token r / G, head kvh * G + r % G), zero beyond `rows`
    for (int idx = threadIdx.x; idx < QROWS * (D / 8); idx += ATC_THREADS) {
        const int r = idx / (D / 8), c = idx % (D / 8);
        uint4 val = make_uint4(0, 0, 0, 0);
        if (r < rows) {
            const int qi = r / G, g = r - qi * G;
            val = *reinterpret_cast<const uint4*>(p.q + ((size_t)(row0 + qi) * p.n_heads + kvh * G + g) * D + c * 8);
        }
        *reinterpret_cast<uint4*>(q_s + (c >> 3) * Q_HALF_BYTES + swz(r, c & 7)) = val;
    }
    __syncthreads();

    const int* bt = p.block_table + (size_t)seq * p.max_blocks;
    const int boxes = KT / p.page;

    if (warp == 4) {
        // ---------------------------------------------------------------- page fetcher
        // Lane i fetches box i of every tile (its page id is looked up one tile ahead); the warp
        // runs up to NSTAGE tiles ahead of the multiplying warps and never waits for them otherwise.
        auto page_row = [&](int it) {
            int blk = 0;
            if (lane < boxes && it < n_kt) {
                blk = bt[min((k_begin + it * KT + lane * p.page) / p.page, p.max_blocks - 1)];
                if (blk < 0 || blk >= p.num_pages) blk = 0;     // beyond the context or given back: masked below
            }
            return (blk * p.n_kv + kvh) * p.page;
        };
        int y = page_row(0);
        bool ok = true;
        for (int it = 0; it < n_kt && ok; it++) {
            const int b = it % NSTAGE;
            const int y_next = page_row(it + 1);
            if (it >= NSTAGE) ok = atc_wait(&empty_bar[b], (uint32_t)(it / NSTAGE - 1) & 1u, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            if (lane == 0) atc_expect_tx(&full_bar[b], (uint32_t)(2 * TILE_BYTES));
            __syncwarp();
            if (lane < boxes) {
#pragma unroll
                for (int h = 0; h < HALVES; h++) {
                    const int off = h * HALF_BYTES + lane * p.page * 128;
                    atc_tma_2d(k_s + b * TILE_BYTES + off, &map_k, &full_bar[b], h * 64, y);
                    atc_tma_2d(v_s + b * TILE_BYTES + off, &map_v, &full_bar[b], h * 64, y);
                }
            }
            y = y_next;
        }
    }

    // ---- this warp's query fragments (16 rows x D)
    const int wrow = DECODE ? 0 : (warp & 3) * 16;
    uint32_t qf[D / 16][4];
    {
        const int mat = lane >> 3, rin = lane & 7;
        const int r = wrow + (mat & 1) * 8 + rin;
#pragma unroll
        for (int kc = 0; kc < D / 16; kc++) {
            const int chunk = kc * 2 + (mat >> 1);
            ldsm_x4(s32(q_s + (chunk >> 3) * Q_HALF_BYTES + swz(r, chunk & 7)), qf[kc][0], qf[kc][1], qf[kc][2], qf[kc][3]);
        }
    }
    const int r_a = wrow + g8, r_b = wrow + g8 + 8;          // the two rows this thread holds
    const int qpos_a = pos0 + min(r_a, rows - 1) / G, qpos_b = pos0 + min(r_b, rows - 1) / G;

    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.0f, l_b = 0.0f;
    float o[ND][4];
#pragma unroll
    for (int j = 0; j < ND; j++) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;

    bool alive = true;
    for (int it = 0; it < n_kt && warp < 4; it++) {
        const int b = it % NSTAGE;
        if (alive) alive = atc_wait(&full_bar[b], (uint32_t)(it / NSTAGE) & 1u, abort_flag);
        if (alive) {
            const uint8_t* kb = k_s + b * TILE_BYTES;
            const uint8_t* vb = v_s + b * TILE_BYTES;
            const int k0 = k_begin + it * KT;
            const int koff = DECODE ? warp * 16 : 0;                // this warp's keys inside the tile
            // in prefill mode a warp whose rows all lie before this key tile has nothing to do
            const int warp_last_q = pos0 + min(wrow + 15, rows - 1) / G;
            if (DECODE || (wrow < rows && k0 <= warp_last_q)) {
                float s[NKG][4];
#pragma unroll
                for (int j = 0; j < NKG; j++) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
                {
                    const int mat = lane >> 3, rin = lane & 7;
#pragma unroll
                    for (int kc = 0; kc < D / 16; kc++) {
#pragma unroll
                        for (int jp = 0; jp < NKG / 2; jp++) {
                            const int key = koff + jp * 16 + (mat >> 1) * 8 + rin;
                            const int chunk = kc * 2 + (mat & 1);
                            uint32_t b0, b1, b2, b3;
                            ldsm_x4(s32(kb + (chunk >> 3) * HALF_BYTES + swz(key, chunk & 7)), b0, b1, b2, b3);
                            mma_bf16(s[2 * jp], qf[kc], b0, b1);
                            mma_bf16(s[2 * jp + 1], qf[kc], b2, b3);
                        }
                    }
                }
                // scale, mask, running maximum.  A tile that every row of this warp sees completely
                // (all keys at or before the warp's first query, inside the window and the split) needs
                // no mask: only tiles at the causal diagonal and at range edges pay for the compares.
                float tmax_a = -INFINITY, tmax_b = -INFINITY;
                const int first_q = pos0 + min(wrow, rows - 1) / G;          // earliest query position of this warp
                const bool interior = k0 + koff >= lo && k0 + koff + NKG * 8 <= hi && k0 + koff + NKG * 8 - 1 <= first_q &&
                                      (p.window <= 0 || k0 + koff > warp_last_q - p.window);
                if (interior) {
#pragma unroll
                    for (int j = 0; j < NKG; j++) {
#pragma unroll
                        for (int e = 0; e < 4; e++) s[j][e] *= p.scale_log2;
                        tmax_a = fmaxf(tmax_a, fmaxf(s[j][0], s[j][1]));
                        tmax_b = fmaxf(tmax_b, fmaxf(s[j][2], s[j][3]));
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < NKG; j++) {
#pragma unroll
                        for (int e = 0; e < 2; e++) {
                            const int key = k0 + koff + j * 8 + 2 * t4 + e;
                            const bool in = key >= lo && key < hi;
                            const bool va = in && key <= qpos_a && (p.window <= 0 || key > qpos_a - p.window);
                            const bool vb2 = in && key <= qpos_b && (p.window <= 0 || key > qpos_b - p.window);
                            s[j][e] = va ? s[j][e] * p.scale_log2 : -INFINITY;
                            s[j][2 + e] = vb2 ? s[j][2 + e] * p.scale_log2 : -INFINITY;
                            tmax_a = fmaxf(tmax_a, s[j][e]);
                            tmax_b = fmaxf(tmax_b, s[j][2 + e]);
                        }
                    }
                }
                tmax_a = fmaxf(tmax_a, __shfl_xor_sync(0xffffffffu, tmax_a, 1));
                tmax_a = fmaxf(tmax_a, __shfl_xor_sync(0xffffffffu, tmax_a, 2));
                tmax_b = fmaxf(tmax_b, __shfl_xor_sync(0xffffffffu, tmax_b, 1));
                tmax_b = fmaxf(tmax_b, __shfl_xor_sync(0xffffffffu, tmax_b, 2));
                const float mn_a = fmaxf(m_a, tmax_a), mn_b = fmaxf(m_b, tmax_b);
                // a row that has seen no key yet keeps exp2(-inf - -inf) out of the arithmetic
                const float base_a = mn_a == -INFINITY ? 0.0f : mn_a, base_b = mn_b == -INFINITY ? 0.0f : mn_b;
                const float corr_a = exp2f(m_a - base_a), corr_b = exp2f(m_b - base_b);
                m_a = mn_a;
                m_b = mn_b;
                float sum_a = 0.0f, sum_b = 0.0f;
                uint32_t pf[NKG / 2][4];
#pragma unroll
                for (int j = 0; j < NKG; j++) {
                    const float p0 = exp2f(s[j][0] - base_a), p1 = exp2f(s[j][1] - base_a);
                    const float p2 = exp2f(s[j][2] - base_b), p3 = exp2f(s[j][3] - base_b);
                    sum_a += p0 + p1;
                    sum_b += p2 + p3;
                    pf[j >> 1][(j & 1) * 2 + 0] = pack_bf16(p0, p1);
                    pf[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
                }
                sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 1);
                sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 2);
                sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 1);
                sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 2);
                l_a = l_a * corr_a + sum_a;
                l_b = l_b * corr_b + sum_b;
#pragma unroll
                for (int j = 0; j < ND; j++) {
                    o[j][0] *= corr_a; o[j][1] *= corr_a;
                    o[j][2] *= corr_b; o[j][3] *= corr_b;
                }
                // O += P . V
                {
                    const int mat = lane >> 3, rin = lane & 7;
#pragma unroll
                    for (int kk = 0; kk < NKG / 2; kk++) {
                        const int key = koff + kk * 16 + (mat & 1) * 8 + rin;
#pragma unroll
                        for (int jd = 0; jd < ND / 2; jd++) {
                            const int chunk = jd * 2 + (mat >> 1);
                            uint32_t b0, b1, b2, b3;
                            ldsm_x4_t(s32(vb + (chunk >> 3) * HALF_BYTES + swz(key, chunk & 7)), b0, b1, b2, b3);
                            mma_bf16(o[2 * jd], pf[kk], b0, b1);
                            mma_bf16(o[2 * jd + 1], pf[kk], b2, b3);
                        }
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0) atc_arrive(&empty_bar[b]);   // this warp is done with buffer b
    }
    __syncthreads();       // every tile has landed and has been read: the buffers are free
    if (threadIdx.x == 0 && *abort_flag && p.err) atomicOr(p.err, EMBER_ERR_WAIT_LIMIT);
    if (warp == 4 && !DECODE) return;

    if (!DECODE) {
        // ---- rows are private to a warp: normalise and store
        const float inv_a = l_a > 0.0f ? 1.0f / l_a : 0.0f, inv_b = l_b > 0.0f ? 1.0f / l_b : 0.0f;
        if (r_a < rows) {
            const int qi = r_a / G, g = r_a - qi * G;
            __nv_bfloat16* dst = p.out + ((size_t)(row0 + qi) * p.n_heads + kvh * G + g) * D;
#pragma unroll
            for (int j = 0; j < ND; j++)
                *reinterpret_cast<uint32_t*>(dst + j * 8 + 2 * t4) = pack_bf16(o[j][0] * inv_a, o[j][1] * inv_a);
        }
        if (r_b < rows) {
            const int qi = r_b / G, g = r_b - qi * G;
            __nv_bfloat16* dst = p.out + ((size_t)(row0 + qi) * p.n_heads + kvh * G + g) * D;
#pragma unroll
            for (int j = 0; j < ND; j++)
                *reinterpret_cast<uint32_t*>(dst + j * 8 + 2 * t4) = pack_bf16(o[j][2] * inv_b, o[j][3] * inv_b);
        }
        return;
    }

    // ---- decode: merge the four warps (each saw a quarter of the keys) through shared memory
    float* mo = reinterpret_cast<float*>(k_s);                 // [4 warps][16 rows][D]   (K/V buffers are free now)
    float* mm = reinterpret_cast<float*>(v_s);                 // [4][16] maxima, then [4][16] denominators
    if (warp < 4 && t4 == 0) {
        mm[warp * 16 + g8] = m_a;
        mm[warp * 16 + g8 + 8] = m_b;
        mm[64 + warp * 16 + g8] = l_a;
        mm[64 + warp * 16 + g8 + 8] = l_b;
    }
#pragma unroll
    for (int j = 0; j < ND && warp < 4; j++) {
        float* ra = mo + ((size_t)warp * 16 + g8) * D + j * 8 + 2 * t4;
        float* rb = mo + ((size_t)warp * 16 + g8 + 8) * D + j * 8 + 2 * t4;
        ra[0] = o[j][0]; ra[1] = o[j][1];
        rb[0] = o[j][2]; rb[1] = o[j][3];
    }
    __syncthreads();
    if (merge_in_cluster) atc_cluster_wait();
    const uint32_t recv_o0 = atc_map_to_rank(s32(recv), 0);
    const uint32_t recv_ml0 = recv_o0 + (uint32_t)(p.n_splits * rows * D) * 4u;
    for (int idx = threadIdx.x; idx < rows * D; idx += ATC_THREADS) {
        const int r = idx / D, d = idx - r * D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; w++) M = fmaxf(M, mm[w * 16 + r]);
        float L = 0.0f, acc = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; w++) {
            const float mw = mm[w * 16 + r];
            if (mw == -INFINITY) continue;
            const float f = exp2f(mw - M);
            L += mm[64 + w * 16 + r] * f;
            acc += mo[((size_t)w * 16 + r) * D + d] * f;
        }
        // nq == 1: row r is head r of the group
        if (p.n_splits <= 1) {
            p.out[((size_t)row0 * p.n_heads + kvh * G + r) * D + d] = __float2bfloat16_rn(L > 0.0f ? acc / L : 0.0f);
        } else if (merge_in_cluster) {
            atc_st_cluster(recv_o0 + (uint32_t)((split * rows + r) * D + d) * 4u, acc);
            if (d == 0) {
                atc_st_cluster(recv_ml0 + (uint32_t)((split * rows + r) * 2) * 4u, M);
                atc_st_cluster(recv_ml0 + (uint32_t)((split * rows + r) * 2 + 1) * 4u, L);
            }
        } else {
            const size_t ph = (size_t)tile * p.n_heads + kvh * G + r;      // partials are indexed by tile
            p.part_o[(ph * p.n_splits + split) * D + d] = acc;
            if (d == 0) {
                p.part_ml[(ph * p.n_splits + split) * 2 + 0] = M == -INFINITY ? -INFINITY : M * (1.0f / LOG2E);
                p.part_ml[(ph * p.n_splits + split) * 2 + 1] = L;
            }
        }
    }
    if (merge_in_cluster) {
        // ---- the tile's first block merges the splits in ascending order (the arithmetic of the merge kernel)
        atc_cluster_arrive();                       // phase 2: every split's results are written ...
        atc_cluster_wait();                         // ... and visible
        if (split != 0) return;
        const float* ro = recv;
        const float* rml = recv + (size_t)p.n_splits * rows * D;
        for (int idx = threadIdx.x; idx < rows * D; idx += ATC_THREADS) {
            const int r = idx / D, d = idx - r * D;
            float M = -INFINITY;
            for (int sp = 0; sp < p.n_splits; sp++) M = fmaxf(M, rml[(sp * rows + r) * 2]);
            float L = 0.0f, acc = 0.0f;
            for (int sp = 0; sp < p.n_splits; sp++) {
                const float ms = rml[(sp * rows + r) * 2];
                if (ms == -INFINITY) continue;
                const float f = exp2f(ms - M);
                L += rml[(sp * rows + r) * 2 + 1] * f;
                acc = fmaf(ro[((size_t)sp * rows + r) * D + d], f, acc);
            }
            p.out[((size_t)row0 * p.n_heads + kvh * G + r) * D + d] = __float2bfloat16_rn(L > 0.0f ? acc * (1.0f / L) : 0.0f);
        }
    }
}

// Merges split partials in ascending order (same arithmetic as attention.cu's combine).  The maxima and
// denominators of a head are read once into shared memory, and the weights exp(m_s - M) are formed once, so
// that a thread's loads of the partial sums are independent of one another (they were a chain of n_splits
// dependent loads before, which is what the kernel's time was at batch 1 with 13 splits).
__global__ void attention_tc_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                            __nv_bfloat16* __restrict__ out, const int* __restrict__ tiles,
                                            int n_heads, int n_splits, int D) {
    extern __shared__ float w_s[];                                         // [n_splits] weights, then 1 / L
    float& inv_s = w_s[n_splits];
    pdl_launch_dependents();
    pdl_wait();
    const size_t th = blockIdx.x;                                          // tile * n_heads + head
    const int tile = (int)(th / n_heads), head = (int)(th % n_heads);
    const size_t oh = (size_t)tiles[tile * 4 + 1] * n_heads + head;        // the tile's single token row
    const float* ml = part_ml + th * n_splits * 2;
    // Up to 16 splits (what the planner makes): a thread's partial sums are requested now, so that they travel
    // while the first warp forms the weights (one trip to memory behind the dependency instead of two).
    constexpr int EARLY = 16;
    const bool early = n_splits <= EARLY && (int)threadIdx.x < D;
    float a[EARLY];
    if (early) {
        const float* po = part_o + th * n_splits * D + threadIdx.x;
#pragma unroll
        for (int s = 0; s < EARLY; s++) a[s] = s < n_splits ? po[(size_t)s * D] : 0.0f;
    }
    if (threadIdx.x < 32) {
        // one warp: lanes take the splits (in rounds of 32), the sums run in ascending order of the split
        float M = -INFINITY;
        for (int s = threadIdx.x; s < n_splits; s += 32) M = fmaxf(M, ml[2 * s]);
        M = warp_max(M);
        float L = 0.0f;
        for (int s0 = 0; s0 < n_splits; s0 += 32) {
            const int s = s0 + (int)threadIdx.x;
            float w = 0.0f, l = 0.0f;
            if (s < n_splits) {
                const float ms = ml[2 * s];
                if (ms != -INFINITY) { w = expf(ms - M); l = ml[2 * s + 1] * w; }
                w_s[s] = w;
            }
            for (int i = 0; i < 32 && s0 + i < n_splits; i++) L += __shfl_sync(0xffffffffu, l, i);   // ascending
        }
        if (threadIdx.x == 0) inv_s = L > 0.0f ? 1.0f / L : 0.0f;
    }
    __syncthreads();
    const float inv = inv_s;
    if (early) {
        float o = 0.0f;
#pragma unroll
        for (int s = 0; s < EARLY; s++)
            if (s < n_splits) o = fmaf(a[s], w_s[s], o);                   // ascending, as below
        out[oh * D + threadIdx.x] = __float2bfloat16_rn(o * inv);
    }
    for (int d = (int)threadIdx.x + (early ? (int)blockDim.x : 0); d < D; d += blockDim.x) {
        const float* po = part_o + th * n_splits * D + d;
        float o = 0.0f;
        int s = 0;
        for (; s + 4 <= n_splits; s += 4) {
            const float a0 = po[(size_t)s * D], a1 = po[(size_t)(s + 1) * D], a2 = po[(size_t)(s + 2) * D], a3 = po[(size_t)(s + 3) * D];
            o = fmaf(a0, w_s[s], o);
            o = fmaf(a1, w_s[s + 1], o);
            o = fmaf(a2, w_s[s + 2], o);
            o = fmaf(a3, w_s[s + 3], o);
        }
        for (; s < n_splits; s++) o = fmaf(po[(size_t)s * D], w_s[s], o);
        out[oh * D + d] = __float2bfloat16_rn(o * inv);
    }
}

typedef CUresult (*AtcEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static AtcEncodeFn atc_encode_fn() {
    static AtcEncodeFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (AtcEncodeFn)ptr;
    });
    return fn;
}

// A pool [pages][kv_heads][page][D] seen as a matrix [pages * kv_heads * page rows][D]; one box is
// one page of one head, 64 elements wide.
static bool pool_map(const void* pool, long long total_rows, int D, int page, CUtensorMap* out) {
    static std::map<std::tuple<const void*, long long, int, int>, CUtensorMap> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    auto key = std::make_tuple(pool, total_rows, D, page);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return true;
    }
    AtcEncodeFn fn = atc_encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)total_rows};
    cuuint64_t strides[1] = {(cuuint64_t)D * 2};
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

// 1 if the tensor-core kernels take this geometry.  mode 0 = prompt portions, 1 = single tokens.
EMBER_API int ember_attention_tc_supported(int D, int group, int page, int mode) {
    if (D != 64 && D != 128) return 0;
    if (page != 16 && page != 32 && page != 64) return 0;
    if (group < 1) return 0;
    return mode == 1 ? (group <= 16) : (group <= 64);
}

// Query tokens per tile in mode 0.
EMBER_API int ember_attention_tc_tile_queries(int group) { return group >= 1 && group <= 64 ? 64 / group : 0; }

EMBER_API int ember_attention_tc(const void* q, const void* k_pool, const void* v_pool, void* out, int mode,
                                 int n_heads, int n_kv, int D, const int* tiles, int n_tiles,
                                 const int* block_table, int max_blocks, int page, int num_pages, int window,
                                 float scale, int n_splits, int split_keys, float* part_o, float* part_ml,
                                 int* err, void* stream) {
    if (n_tiles <= 0) return 0;
    if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv) return fail("attention_tc: bad head counts %d/%d", n_heads, n_kv);
    const int G = n_heads / n_kv;
    if (!ember_attention_tc_supported(D, G, page, mode))
        return fail("attention_tc: head size %d, group %d, page %d are not taken in mode %d", D, G, page, mode);
    if (mode == 0 && n_splits != 1) return fail("attention_tc: prompt portions are not split");
    // splits without buffers for their partial results: the splits of a tile form a thread-block cluster (at most 8
    // blocks) and are merged in shared memory
    const bool cluster_merge = n_splits > 1 && !part_o && !part_ml;
    if (n_splits < 1 || (n_splits > 1 && (split_keys <= 0 || split_keys % KT || (!cluster_merge && (!part_o || !part_ml)))))
        return fail("attention_tc: bad split configuration (%d splits of %d keys)", n_splits, split_keys);
    if (cluster_merge && n_splits > 8) return fail("attention_tc: %d splits are too many for a cluster (at most 8)", n_splits);
    if (n_splits > 8192 || n_kv > 65535) return fail("attention_tc: grid too large");
    CUtensorMap mk, mv;
    const long long total_rows = (long long)num_pages * n_kv * page;
    if (!pool_map(k_pool, total_rows, D, page, &mk) || !pool_map(v_pool, total_rows, D, page, &mv))
        return fail("attention_tc: cuTensorMapEncodeTiled failed or is unavailable");
    AttnTcParams p;
    p.q = (const __nv_bfloat16*)q; p.out = (__nv_bfloat16*)out; p.part_o = part_o; p.part_ml = part_ml;
    p.tiles = tiles; p.block_table = block_table; p.max_blocks = max_blocks; p.page = page; p.num_pages = num_pages;
    p.n_heads = n_heads; p.n_kv = n_kv; p.window = window; p.scale_log2 = scale * LOG2E;
    p.n_splits = n_splits; p.split_keys = split_keys; p.n_tiles = n_tiles; p.err = err;
    p.cluster_merge = cluster_merge ? 1 : 0;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t tile_bytes = (size_t)(D / 64) * KT * 128;
    const size_t q_bytes = ((size_t)(D / 64) * (mode == 1 ? 16 : 64) * 128 + 1023) & ~(size_t)1023;
    const size_t recv_bytes = cluster_merge ? (size_t)n_splits * G * (D + 2) * sizeof(float) + 16 : 0;
    const size_t smem = q_bytes + (size_t)(mode == 1 ? 3 : 2) * 2 * tile_bytes + 1024 + 128 + recv_bytes;
    dim3 grid(n_tiles, n_kv, n_splits);
    auto run = [&](auto kernel) -> int {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail("attention_tc: shared memory %zu: %s", smem, cudaGetErrorString(e));
        // ask for the largest shared-memory carve-out so that two blocks fit on an SM
        cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
        if (!cluster_merge) {
            launch_kernel(kernel, grid, ATC_THREADS, smem, st, mk, mv, p);
            return check_launch("attention_tc");
        }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(ATC_THREADS);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = st;
        cudaLaunchAttribute attrs[2];
        attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
        attrs[1].id = cudaLaunchAttributeClusterDimension;
        attrs[1].val.clusterDim.x = 1; attrs[1].val.clusterDim.y = 1; attrs[1].val.clusterDim.z = (unsigned)n_splits;
        cfg.attrs = attrs; cfg.numAttrs = 2;
        cudaLaunchKernelEx(&cfg, kernel, mk, mv, p);
        return check_launch("attention_tc (cluster)");
    };
    int rc;
    if (D == 128) rc = mode == 1 ? run(attention_tc_kernel<2, true>) : run(attention_tc_kernel<2, false>);
    else rc = mode == 1 ? run(attention_tc_kernel<1, true>) : run(attention_tc_kernel<1, false>);
    if (rc) return rc;
    if (n_splits > 1 && !cluster_merge) {
        launch_kernel(attention_tc_combine_kernel, (unsigned)((size_t)n_tiles * n_heads), D, (size_t)(n_splits + 1) * sizeof(float), st,
                      (const float*)part_o,
                      (const float*)part_ml, (__nv_bfloat16*)out, tiles, n_heads, n_splits, D);
        return check_launch("attention_tc_combine");
    }
    return 0;
}
