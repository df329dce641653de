// The prefill product on pairs of SMs: tcgen05.mma.cta_group::2, 256 tokens x 256 weight rows per tile.
//
// Two blocks of a cluster (ranks 0 and 1 of a pair) work on one output tile.  Each block brings its own 128
// token rows of A and its own half of the tile's weight rows (256 at most) by TMA into its own shared memory; the TMA
// loads of both blocks complete on the leader's (rank 0) mbarrier.  The leader's elected thread issues one
// 256 x 256 x 16 MMA per 16 elements of K for the pair: the tensor cores of each SM read that SM's A rows and
// its half of the weight rows (so an SM reads 8 KB of operands per MMA instead of the 12 KB of a single-SM
// 128 x 256 tile, and a stage is 32 KB instead of 48 KB, which lets the ring hold six stages).  Each SM's
// 128 x 256 accumulator lands in its own tensor memory.  tcgen05.commit with a multicast to both blocks hands
// stages back to both producers and signals both blocks' epilogue warps; the epilogue warps of both blocks
// release an accumulator by arriving on the leader's mbarrier through the cluster's shared-memory window.
// Persistent: 74 pairs walk the tiles; two accumulators per SM overlap the epilogue with the next tile.
//
// Every wait is bounded (EMBER_ERR_WAIT_LIMIT), and both blocks of a pair meet at a cluster barrier before
// tensor memory is freed, so neither leaves while the other may still signal it.
#pragma once

#include "gemm_tc_kernel.cuh"

namespace ember {

constexpr int PAIR_MAX_COLS = 256;      // weight rows per pair tile (a multiple of 16; each block holds half of them)

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// TMA load of a block of a pair: the bytes are counted on an mbarrier that may live in the peer's shared memory.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"((uint64_t)map), "r"(bar_cluster_addr), "r"(x), "r"(y)
        : "memory");
}
// Arrives, once the pair's earlier MMAs are done, on the mbarrier at this offset in both blocks of the pair.
__device__ __forceinline__ void tcgen05_commit_pair(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void tcgen05_mma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}
// fp32 accumulate, bf16 A and B, both K-major, M = 256 over the pair, N = n.
__host__ __device__ __forceinline__ uint32_t umma_idesc_pair(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)((2 * TILE_ROWS) >> 4) << 24);
}
__host__ __device__ __forceinline__ int pair_stage_bytes(int block_cols) {
    return TILE_ROWS * TILE_K * 2 + (((block_cols / 2) * TILE_K * 2 + 1023) & ~1023);
}

// p.block_cols: weight rows per pair tile; p.row_tiles / p.total_tiles count pair tiles (256 tokens x block_cols).
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_rows, const __grid_constant__ CUtensorMap map_cols,
                    const GemmTcParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int a_bytes = TILE_ROWS * TILE_K * 2;
    const int half_cols = p.block_cols / 2;
    const int b_bytes = half_cols * TILE_K * 2;
    const int stage_bytes = pair_stage_bytes(p.block_cols);
    uint64_t* full_bar = (uint64_t*)(smem + (size_t)p.stages * stage_bytes);   // used in the leader only
    uint64_t* empty_bar = full_bar + MAX_STAGES;
    uint64_t* tmem_full_bar = empty_bar + MAX_STAGES;      // [2]
    uint64_t* tmem_empty_bar = tmem_full_bar + 2;           // [2], used in the leader only
    uint32_t* tmem_base_slot = (uint32_t*)(tmem_empty_bar + 2);
    volatile int* abort_flag = (volatile int*)(tmem_base_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();                // 0: leader, 1: peer
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int n_kb = p.num_k_blocks;
    // units: a tile and a part of K (more than one part only for the adding epilogue of a product with few tiles)
    const int k_splits = (n_kb + p.k_blocks_per_split - 1) / p.k_blocks_per_split;
    const int units = p.total_tiles * k_splits;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; s++) {
            mbar_init(&full_bar[s], 1);                     // the leader's producer arrives; both blocks' bytes are counted
            mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(&tmem_full_bar[a], 1);
            mbar_init(&tmem_empty_bar[a], 8);               // four epilogue warps in each block of the pair
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_base_slot)), "r"(p.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_arrive();                                       // the peer's barriers exist before anything signals them
    cluster_wait();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = *tmem_base_slot;

    pdl_launch_dependents();
    pdl_wait();

    if (warp == 0) {
        if (lane == 0) {
            int s = 0;
            uint32_t phase = 0;
            bool ok = true, wrapped = false;
            uint8_t* st = smem;
            for (int u = pair; u < units && ok; u += n_pairs) {
                const int t = u / k_splits, kb0 = (u - t * k_splits) * p.k_blocks_per_split;
                const int kb1 = min(n_kb, kb0 + p.k_blocks_per_split);
                const int col_tile = t / p.row_tiles, row_tile = t - col_tile * p.row_tiles;
                const int row0 = row_tile * 2 * TILE_ROWS + (int)rank * TILE_ROWS;
                const int col0 = col_tile * p.block_cols + (int)rank * half_cols;
                for (int i = kb0; i < kb1; i++) {
                    if (wrapped) ok = mbar_wait(&empty_bar[s], phase ^ 1u, abort_flag);
                    if (!ok) break;
                    const uint32_t bar = map_to_rank(smem_u32(&full_bar[s]), 0);
                    if (rank == 0) mbar_expect_tx(&full_bar[s], (uint32_t)(2 * (a_bytes + b_bytes)));
                    tma_load_2d_pair(st, &map_rows, bar, i * TILE_K, row0);
                    tma_load_2d_pair(st + a_bytes, &map_cols, bar, i * TILE_K, col0);
                    st += stage_bytes;
                    if (++s == p.stages) { s = 0; st = smem; phase ^= 1u; wrapped = true; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = umma_idesc_pair(p.block_cols);
            int li = 0, s = 0;
            uint32_t phase = 0;
            bool ok = true;
            const uint64_t da0 = umma_desc_sw128(smem), db0 = umma_desc_sw128(smem + a_bytes);
            const uint64_t dstep = (uint64_t)(stage_bytes >> 4);
            uint64_t da = da0, db = db0;
            for (int u = pair; u < units && ok; u += n_pairs, li++) {
                const int kb0 = (u % k_splits) * p.k_blocks_per_split, kb1 = min(n_kb, kb0 + p.k_blocks_per_split);
                const int acc = li & 1;
                if (li >= 2) ok = mbar_wait(&tmem_empty_bar[acc], ((uint32_t)(li >> 1) & 1u) ^ 1u, abort_flag);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d = tmem_d + (uint32_t)(acc * p.block_cols);
                for (int i = kb0; i < kb1; i++) {
                    ok = mbar_wait(&full_bar[s], phase, abort_flag);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                    for (int k = 0; k < TILE_K / UMMA_K; k++)
                        tcgen05_mma_bf16_pair(d, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (i > kb0 || k > 0) ? 1u : 0u);
                    tcgen05_commit_pair(&empty_bar[s]);
                    da += dstep; db += dstep;
                    if (++s == p.stages) { s = 0; phase ^= 1u; da = da0; db = db0; }
                }
                if (ok) tcgen05_commit_pair(&tmem_full_bar[acc]);
            }
        }
    } else {
        const int quad = warp & 3;
        const int r = quad * 32 + lane;
        bool ok = true;
        int li = 0;
        for (int u = pair; u < units; u += n_pairs, li++) {
            const int t = u / k_splits;
            const int col_tile = t / p.row_tiles, row_tile = t - col_tile * p.row_tiles;
            const int acc = li & 1;
            const int m = row_tile * 2 * TILE_ROWS + (int)rank * TILE_ROWS + r;
            QkvRow row;
            if (p.epilogue == 4) qkv_row_prepare(p, m, ok && m < p.M, row);       // its loads travel during the wait
            if (ok) ok = mbar_wait(&tmem_full_bar[acc], (uint32_t)(li >> 1) & 1u, abort_flag);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t taddr_row = tmem_d + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * p.block_cols);
            if (p.epilogue == 4) {
                const int slot0 = col_tile * (p.block_cols >> 7);
                row.live = row.live && ok;
                store_heads_normal(p, row, slot0, min(p.block_cols >> 7, (p.N >> 7) - slot0), taddr_row);
            } else {
                // 64 columns a round trip to tensor memory (a load and its wait cost the same for 16 columns as for 64)
                int c0 = 0;
                for (; c0 + 64 <= p.block_cols; c0 += 64) {
                    uint32_t u[64];
                    tmem_ld64_nowait(taddr_row + (uint32_t)c0, u);
                    tmem_wait_ld();
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        const int n0 = col_tile * p.block_cols + c0 + q * 16;
                        if (!ok || m >= p.M || n0 >= p.N) continue;
                        store_chunk_normal(p, m, n0, min(16, p.N - n0), reinterpret_cast<const float*>(u + q * 16));
                    }
                }
                for (; c0 < p.block_cols; c0 += 16) {
                    float v[16];
                    tmem_ld16(taddr_row + (uint32_t)c0, v);
                    const int n0 = col_tile * p.block_cols + c0;
                    if (!ok || m >= p.M || n0 >= p.N) continue;
                    store_chunk_normal(p, m, n0, min(16, p.N - n0), v);
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_rank(smem_u32(&tmem_empty_bar[acc]), 0));
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag && p.err) atomicOr(p.err, EMBER_ERR_WAIT_LIMIT);
    cluster_arrive();                                       // nothing of the pair is in flight towards either block
    cluster_wait();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(p.tmem_cols) : "memory");
    }
}

}  // namespace ember
