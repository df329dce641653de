// Device code and host helpers of the tcgen05/TMA bf16 matrix product, shared by the files that
// export entry points for it (gemm_tc.cu, no_alloc.cu).  See gemm_tc.cu for the design.
#pragma once

#include <cuda.h>

#include <mutex>

#include "common.cuh"

namespace ember {

constexpr int TILE_ROWS = 128;     // UMMA M
constexpr int TILE_K = 64;         // bf16 elements per stage along K = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int GEMM_THREADS = 192;
constexpr int MAX_STAGES = 8;

// Epilogue 4: the output columns are head slots of 128 (query heads, then key heads, then value heads); instead of
// being stored as they are, a token's query and key heads get their RMSNorm and rotation and go to the query
// buffer and into the token's cache page, value heads go into the cache page.
struct QkvEpilogue {
    int n_heads, n_kv;
    const float* q_norm_w;          // [128] or null
    const float* k_norm_w;
    float eps;
    const float4* cos_sin;          // [32][cs_ld] (cos, cos, sin, sin) of position * inv_freq for frequencies 2j and 2j + 1 of
                                    // token t at [j][t]: the lanes of a warp (neighbouring tokens) read neighbouring 16 bytes; null: no rotation
    int cs_ld;
    const float* inv_freq;          // [64]: decode-sized steps (at most 16 tokens) compute their angles themselves; null: no rotation
    const int* positions;           // [tokens]
    const int* seq_of;              // [tokens] -> row of the block table
    const int* block_table;
    int max_blocks, page, num_pages;
    __nv_bfloat16* q_out;           // [tokens][n_heads][128]
    __nv_bfloat16* k_pool;          // [pages][n_kv][page][128]
    __nv_bfloat16* v_pool;
    int write_kv;
};

struct GemmTcParams {
    int M, N, K;
    int swapped;          // 0: accumulator rows are tokens; 1: accumulator rows are weight rows
    int block_cols;       // accumulator columns per tile (multiple of 16, <= 256)
    int stages;
    int num_k_blocks;     // ceil(K / TILE_K)
    int k_blocks_per_split;
    int epilogue;         // 0 store bf16, 1 store fp32, 2 add fp32, 3 silu(gate)*up -> bf16
    void* out;
    int ldc;
    float* accum;         // atomic split-K target: fp32 [M, accum_ld] (the residual itself for epilogue 2)
    int accum_ld;
    int cluster_splits;   // > 1: the K splits of a tile form a thread-block cluster and are summed in shared memory
    int rows_per;         // accumulator rows each block of the cluster finishes (even)
    int row_tiles;        // persistent kernel: tiles along M, and their total number
    int total_tiles;
    int tmem_cols;
    int* err;
    QkvEpilogue qkv;      // epilogue 4 only
};

// ------------------------------------------------------------------------------ PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait (common.cuh): returns false, with the abort flag raised, once the time limit is reached.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    return mbarrier_wait_bounded(smem_u32(bar), parity, abort_flag);
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tcgen05_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tcgen05_mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
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

// 64 consecutive columns of this thread's lane; the caller waits (tcgen05.wait::ld) before it uses them.
__device__ __forceinline__ void tmem_ld64_nowait(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x64.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ uint32_t map_to_rank(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void st_cluster_f32x4(uint32_t addr, float a, float b, float c, float d) {
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float a) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(a) : "memory");
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major bf16 tile whose rows are 128 bytes, written by TMA
// with the 128-byte swizzle: 8-row groups are 1024 bytes apart (stride byte offset), descriptor
// version 1, layout type 2 (128-byte swizzle).  The leading byte offset is not used by this layout.
__device__ __forceinline__ uint64_t umma_desc_sw128(const void* tile) {
    const uint64_t addr = (uint64_t)(smem_u32(tile) >> 4) & 0x3FFFull;
    return addr | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

// Instruction descriptor: fp32 accumulate, bf16 A and B, both K-major, M = 128, N = block_cols.
__host__ __device__ __forceinline__ uint32_t umma_idesc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(TILE_ROWS >> 4) << 24);
}

__device__ __forceinline__ float silu_mul(float g, float u) { return g / (1.0f + __expf(-g)) * u; }

// Fused epilogue of 16 consecutive output columns of one token row (normal orientation):
// store bf16 / store fp32 / add into the fp32 residual / silu(gate) * up.
__device__ __forceinline__ void store_chunk_normal(const GemmTcParams& p, int m, int n0, int nv, const float* v) {
    if (p.epilogue == 0) {
        __nv_bfloat16* dst = (__nv_bfloat16*)p.out + (size_t)m * p.ldc + n0;
        if (nv == 16 && (((uintptr_t)dst) & 15) == 0) {
            uint4 q[2];
            __nv_bfloat162* h = (__nv_bfloat162*)q;
#pragma unroll
            for (int j = 0; j < 8; j++) h[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
            ((uint4*)dst)[0] = q[0];
            ((uint4*)dst)[1] = q[1];
        } else {
            for (int j = 0; j < nv; j++) dst[j] = __float2bfloat16_rn(v[j]);
        }
    } else if (p.epilogue == 1 || p.epilogue == 2) {
        float* dst = (float*)p.out + (size_t)m * p.ldc + n0;
        if (nv == 16 && (((uintptr_t)dst) & 15) == 0) {
#pragma unroll
            for (int j = 0; j < 4; j++) {
                if (p.epilogue == 2) {
                    // the sum is formed at the L2 (one reduction per element, so the result is the same as a
                    // load, add and store); nothing comes back, so the epilogue never waits on memory
                    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + 4 * j), "f"(v[4 * j]),
                                 "f"(v[4 * j + 1]), "f"(v[4 * j + 2]), "f"(v[4 * j + 3]) : "memory");
                } else {
                    ((float4*)dst)[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                }
            }
        } else {
            for (int j = 0; j < nv; j++) {
                if (p.epilogue == 2) atomicAdd(dst + j, v[j]);          // (several units may add to one element)
                else dst[j] = v[j];
            }
        }
    } else {
        __nv_bfloat16* dst = (__nv_bfloat16*)p.out + (size_t)m * p.ldc + (n0 >> 1);
        if (nv == 16 && (((uintptr_t)dst) & 15) == 0) {
            uint4 q;
            __nv_bfloat162* h = (__nv_bfloat162*)&q;
#pragma unroll
            for (int j = 0; j < 4; j++)
                h[j] = __floats2bfloat162_rn(silu_mul(v[4 * j], v[4 * j + 1]), silu_mul(v[4 * j + 2], v[4 * j + 3]));
            *(uint4*)dst = q;
        } else {
            for (int j = 0; j + 1 < nv; j += 2) dst[j >> 1] = __float2bfloat16_rn(silu_mul(v[j], v[j + 1]));
        }
    }
}

// Packed fp32 pairs (one instruction for two lanes of arithmetic: the epilogue below shares its SM's issue slots
// with the thread that issues the MMAs, so its instruction count is what it costs).
__device__ __forceinline__ unsigned long long pk2(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(__float_as_uint(lo)), "r"(__float_as_uint(hi)));
    return r;
}
__device__ __forceinline__ void unpk2(unsigned long long v, float& lo, float& hi) {
    uint32_t a, b;
    asm("mov.b64 {%0, %1}, %2;" : "=r"(a), "=r"(b) : "l"(v));
    lo = __uint_as_float(a);
    hi = __uint_as_float(b);
}
__device__ __forceinline__ unsigned long long mul2(unsigned long long a, unsigned long long b) {
    unsigned long long d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

// Epilogue 4 for one token row (normal orientation), in two steps.
// Before the accumulator is waited for: where the row's keys and values go, and its 64 angles (32 registers of
// (cos, cos, sin, sin) pairs), so that these loads' latency hides behind the wait; the angles serve every head of
// the tile.
struct QkvRow {
    unsigned long long cs[64];      // [2j], [2j + 1] = (cos, cos), (sin, sin) of frequencies 2j, 2j + 1
    size_t kv_off;
    int m;
    bool live, kv_ok, turn;
};
__device__ __forceinline__ void qkv_row_prepare(const GemmTcParams& p, int m, bool live, QkvRow& row) {
    const QkvEpilogue& e = p.qkv;
    row.m = m;
    row.live = live;
    row.kv_ok = false;
    row.kv_off = 0;
    row.turn = e.cos_sin != nullptr;
    if (live && e.write_kv) {
        const int pos = e.positions[m];
        const int blk = e.block_table[(size_t)e.seq_of[m] * e.max_blocks + pos / e.page];
        if (blk < 0 || blk >= e.num_pages) {
            if (p.err) atomicOr(p.err, EMBER_ERR_PAGE_RANGE);
        } else {
            row.kv_ok = true;
            row.kv_off = ((size_t)blk * e.n_kv * e.page + (size_t)(pos % e.page)) * 128;
        }
    }
    if (row.turn) {
        const float4* src = e.cos_sin + (live ? m : 0);
#pragma unroll
        for (int j = 0; j < 32; j++) {
            const ulonglong2 t = __ldg(reinterpret_cast<const ulonglong2*>(src + (size_t)j * e.cs_ld));
            row.cs[2 * j] = t.x;
            row.cs[2 * j + 1] = t.y;
        }
    }
}
// Once the accumulator is complete: `heads` head slots of 128 columns starting at tensor-memory address `taddr`
// (this thread's lane) and at head slot `slot0`.  All of a head is in this thread's lane: the norm is a sum over
// the 128 columns (a first pass over tensor memory), the rotation pairs columns i and i + 64 of a second pass;
// sums, norm and rotation are fp32 on the fp32 accumulator, rounded to bf16 once.  Every lane runs the
// tensor-memory loads (they are warp-wide); only live rows are stored.
__device__ __forceinline__ void store_heads_normal(const GemmTcParams& p, const QkvRow& row, int slot0, int heads, uint32_t taddr) {
    const QkvEpilogue& e = p.qkv;
    for (int h = 0; h < heads; h++) {
        const int slot = slot0 + h;
        const int kind = slot < e.n_heads ? 0 : (slot < e.n_heads + e.n_kv ? 1 : 2);       // q, k, v
        const uint32_t th = taddr + (uint32_t)(h * 128);
        const float* nw = kind == 0 ? e.q_norm_w : (kind == 1 ? e.k_norm_w : nullptr);
        unsigned long long scale2 = 0;
        if (nw) {                                                   // uniform over the block
            unsigned long long s0 = 0, s1 = 0;                      // (+0, +0)
#pragma unroll
            for (int half = 0; half < 2; half++) {
                uint32_t u[64];
                tmem_ld64_nowait(th + (uint32_t)(half * 64), u);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 64; i += 4) {
                    const unsigned long long x0 = pk2(__uint_as_float(u[i]), __uint_as_float(u[i + 1]));
                    const unsigned long long x1 = pk2(__uint_as_float(u[i + 2]), __uint_as_float(u[i + 3]));
                    s0 = fma2(x0, x0, s0);
                    s1 = fma2(x1, x1, s1);
                }
            }
            float a0, a1, b0, b1;
            unpk2(s0, a0, a1);
            unpk2(s1, b0, b1);
            const float scale = 1.0f / sqrtf(((a0 + a1) + (b0 + b1)) / 128.0f + e.eps);
            scale2 = pk2(scale, scale);
        }
        __nv_bfloat16* dst = nullptr;
        if (row.live) {
            if (kind == 0) dst = e.q_out + ((size_t)row.m * e.n_heads + slot) * 128;
            else if (row.kv_ok) dst = (kind == 1 ? e.k_pool : e.v_pool) + row.kv_off + (size_t)(slot - e.n_heads - (kind == 2 ? e.n_kv : 0)) * e.page * 128;
        }
        const bool turn = kind != 2 && row.turn;
#pragma unroll
        for (int c = 0; c < 4; c++) {                               // columns 16c .. 16c + 15 and their partners 64 further
            uint32_t ua[16], ub[16];
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                : "=r"(ua[0]), "=r"(ua[1]), "=r"(ua[2]), "=r"(ua[3]), "=r"(ua[4]), "=r"(ua[5]), "=r"(ua[6]), "=r"(ua[7]), "=r"(ua[8]),
                  "=r"(ua[9]), "=r"(ua[10]), "=r"(ua[11]), "=r"(ua[12]), "=r"(ua[13]), "=r"(ua[14]), "=r"(ua[15])
                : "r"(th + (uint32_t)(c * 16)));
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                : "=r"(ub[0]), "=r"(ub[1]), "=r"(ub[2]), "=r"(ub[3]), "=r"(ub[4]), "=r"(ub[5]), "=r"(ub[6]), "=r"(ub[7]), "=r"(ub[8]),
                  "=r"(ub[9]), "=r"(ub[10]), "=r"(ub[11]), "=r"(ub[12]), "=r"(ub[13]), "=r"(ub[14]), "=r"(ub[15])
                : "r"(th + (uint32_t)(64 + c * 16)));
            tmem_wait_ld();
            if (!dst) continue;
            unsigned long long a[8], b[8];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                a[i] = pk2(__uint_as_float(ua[2 * i]), __uint_as_float(ua[2 * i + 1]));
                b[i] = pk2(__uint_as_float(ub[2 * i]), __uint_as_float(ub[2 * i + 1]));
            }
            if (nw) {
#pragma unroll
                for (int i = 0; i < 8; i += 2) {
                    const ulonglong2 ga = __ldg(reinterpret_cast<const ulonglong2*>(nw + c * 16 + 2 * i));
                    const ulonglong2 gb = __ldg(reinterpret_cast<const ulonglong2*>(nw + 64 + c * 16 + 2 * i));
                    a[i] = mul2(ga.x, mul2(a[i], scale2)); a[i + 1] = mul2(ga.y, mul2(a[i + 1], scale2));
                    b[i] = mul2(gb.x, mul2(b[i], scale2)); b[i + 1] = mul2(gb.y, mul2(b[i + 1], scale2));
                }
            }
            if (turn) {
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const unsigned long long cos2 = row.cs[2 * (c * 8 + i)], sin2 = row.cs[2 * (c * 8 + i) + 1];
                    const unsigned long long nsin = sin2 ^ 0x8000000080000000ull;
                    const unsigned long long an = fma2(a[i], cos2, mul2(b[i], nsin));      // a cos - b sin
                    const unsigned long long bn = fma2(b[i], cos2, mul2(a[i], sin2));      // b cos + a sin
                    a[i] = an;
                    b[i] = bn;
                }
            }
            uint4 qa[2], qb[2];
            __nv_bfloat162* ha = (__nv_bfloat162*)qa;
            __nv_bfloat162* hb = (__nv_bfloat162*)qb;
#pragma unroll
            for (int j2 = 0; j2 < 8; j2++) {
                float lo, hi;
                unpk2(a[j2], lo, hi);
                ha[j2] = __floats2bfloat162_rn(lo, hi);
                unpk2(b[j2], lo, hi);
                hb[j2] = __floats2bfloat162_rn(lo, hi);
            }
            ((uint4*)(dst + c * 16))[0] = qa[0];
            ((uint4*)(dst + c * 16))[1] = qa[1];
            ((uint4*)(dst + 64 + c * 16))[0] = qb[0];
            ((uint4*)(dst + 64 + c * 16))[1] = qb[1];
        }
    }
}

// Epilogue 4 of a decode-sized step (swapped orientation: the tile's 128 accumulator rows are one head slot, its
// columns the step's at most 16 tokens).  Block `split` of the cluster receives, from every block, the partial
// sums of the tokens split, split + S, ...: recv[s][token / S][row].  It sums them in block order, and thread r
// holds element r of the head: RMSNorm over the 128 elements, rotation with element r ^ 64 (the angle is
// float(position) * inv_freq[r & 63], its sine and cosine fp32), and the head goes to the query buffer or into
// the token's cache page.
// What does not depend on the product -- where the first two tokens' keys and values go, their angles, this
// thread's norm weight -- is fetched by heads_prepare before the cluster's barriers, so that the dependent loads
// (position -> block table) and the sine and cosine are not paid after them.
struct HeadsPrep {
    int kind;                   // 0 q, 1 k, 2 v
    bool norm, turn;
    float g, freq;
    int pos[2], blk[2];
    float cs[2], sn[2];
};
__device__ __forceinline__ void heads_token(const QkvEpilogue& e, int m, const HeadsPrep& h, int& pos, int& blk, float& cs, float& sn) {
    pos = e.positions[m];
    blk = -1;
    if (h.kind != 0 && e.write_kv) blk = e.block_table[(size_t)e.seq_of[m] * e.max_blocks + pos / e.page];
    cs = 1.0f; sn = 0.0f;
    if (h.turn) sincosf((float)pos * h.freq, &sn, &cs);
}
__device__ __forceinline__ void heads_prepare(const GemmTcParams& p, int slot, int split, HeadsPrep& h) {
    const QkvEpilogue& e = p.qkv;
    const int r = (int)threadIdx.x - 64;                   // the row this thread finishes (epilogue warps only)
    h.kind = slot < e.n_heads ? 0 : (slot < e.n_heads + e.n_kv ? 1 : 2);
    const float* nw = h.kind == 0 ? e.q_norm_w : (h.kind == 1 ? e.k_norm_w : nullptr);
    h.norm = nw != nullptr;
    h.turn = h.kind != 2 && e.inv_freq != nullptr;
    h.g = 1.0f; h.freq = 0.0f;
#pragma unroll
    for (int t = 0; t < 2; t++) { h.pos[t] = 0; h.blk[t] = -1; h.cs[t] = 1.0f; h.sn[t] = 0.0f; }
    if (r < 0) return;
    if (nw) h.g = nw[r];
    if (h.turn) h.freq = e.inv_freq[r & 63];
#pragma unroll
    for (int t = 0; t < 2; t++) {
        const int m = split + t * p.cluster_splits;
        if (m < p.M) heads_token(e, m, h, h.pos[t], h.blk[t], h.cs[t], h.sn[t]);
    }
}
// All threads of the block call this (it synchronises); the rows are held by the four epilogue warps (threads
// 64..191), the ones that called heads_prepare while the product ran.
__device__ __forceinline__ void finish_heads_swapped(const GemmTcParams& p, const float* recv, int slot, int split, bool failed,
                                                     const HeadsPrep& h) {
    const QkvEpilogue& e = p.qkv;
    const int S = p.cluster_splits, per = (p.block_cols + S - 1) / S;
    float* xs = const_cast<float*>(recv) + (size_t)S * per * TILE_ROWS;      // [128] the normed head, then 4 partial sums
    float* red = xs + TILE_ROWS;
    const int r = (int)threadIdx.x - 64;
    const bool row = r >= 0;
    auto finish_one = [&](int cl, int m, int pos, int blk, float cs, float sn) {
        float v = 0.0f;
        if (row)
            for (int s = 0; s < S; s++) v += recv[((size_t)s * per + cl) * TILE_ROWS + r];
        if (h.norm) {
            float ss = warp_sum(row ? v * v : 0.0f);
            if ((r & 31) == 0 && row) red[r >> 5] = ss;
            __syncthreads();
            ss = (red[0] + red[1]) + (red[2] + red[3]);
            v = h.g * (v * (1.0f / sqrtf(ss / 128.0f + e.eps)));
        }
        if (h.turn) {
            if (row) xs[r] = v;
            __syncthreads();
            if (row) {
                const float other = xs[r ^ 64];
                v = r < 64 ? v * cs - other * sn : v * cs + other * sn;
            }
        }
        __nv_bfloat16* dst = nullptr;
        if (h.kind == 0) {
            dst = e.q_out + ((size_t)m * e.n_heads + slot) * 128;
        } else if (e.write_kv) {
            if (blk < 0 || blk >= e.num_pages) {
                if (r == 0 && p.err) atomicOr(p.err, EMBER_ERR_PAGE_RANGE);
            } else {
                const int kvh = slot - e.n_heads - (h.kind == 2 ? e.n_kv : 0);
                dst = (h.kind == 1 ? e.k_pool : e.v_pool) + (((size_t)blk * e.n_kv + kvh) * e.page + (size_t)(pos % e.page)) * 128;
            }
        }
        if (dst && row && !failed) dst[r] = __float2bfloat16_rn(v);
    };
    if (split < p.M) finish_one(0, split, h.pos[0], h.blk[0], h.cs[0], h.sn[0]);
    if (per > 1 && split + S < p.M) {
        __syncthreads();                                            // xs and red are reused
        finish_one(1, split + S, h.pos[1], h.blk[1], h.cs[1], h.sn[1]);
    }
    for (int cl = 2; cl < per; cl++) {                              // more than two tokens a block: fetched here
        const int m = split + cl * S;                               // uniform over the block
        if (m >= p.M) break;
        int pos = 0, blk = -1;
        float cs = 1.0f, sn = 0.0f;
        if (row) heads_token(e, m, h, pos, blk, cs, sn);
        __syncthreads();
        finish_one(cl, m, pos, blk, cs, sn);
    }
}

// ------------------------------------------------------------------------------------ kernel
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_rows, const __grid_constant__ CUtensorMap map_cols,
               const GemmTcParams p) {
    extern __shared__ uint8_t smem_raw[];
    // tiles need 1024-byte alignment for the 128-byte swizzle
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int rows_bytes = TILE_ROWS * TILE_K * 2;               // 16 KiB
    const int cols_bytes = p.block_cols * TILE_K * 2;
    const int stage_bytes = rows_bytes + ((cols_bytes + 1023) & ~1023);
    uint64_t* full_bar = (uint64_t*)(smem + (size_t)p.stages * stage_bytes);
    uint64_t* empty_bar = full_bar + MAX_STAGES;
    uint64_t* tmem_full_bar = empty_bar + MAX_STAGES;
    uint32_t* tmem_base_slot = (uint32_t*)(tmem_full_bar + 1);
    volatile int* abort_flag = (volatile int*)(tmem_base_slot + 1);
    // cluster split-K: partial sums of the rows this block finishes, one slab per block of the cluster
    float* recv = (float*)((uint8_t*)full_bar + 256);            // [cluster_splits][rows_per][block_cols]
    const bool heads = p.swapped && p.epilogue == 4;           // the tile is one head slot; tokens are shared out (below)
    const bool clustered = p.cluster_splits > 1 || heads;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row_tile = blockIdx.x, col_tile = blockIdx.y, split = blockIdx.z;
    const int kb0 = split * p.k_blocks_per_split;
    const int kb1 = min(p.num_k_blocks, kb0 + p.k_blocks_per_split);
    const int n_kb = kb1 - kb0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; s++) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(tmem_full_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_base_slot)), "r"(p.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = *tmem_base_slot;
    if (clustered) cluster_arrive();        // phase 1: every block of the cluster is up before anyone writes to it

    pdl_launch_dependents();
    HeadsPrep prep;
    prep.kind = 0; prep.norm = false; prep.turn = false; prep.g = 1.0f; prep.freq = 0.0f;
    prep.pos[0] = prep.pos[1] = 0; prep.blk[0] = prep.blk[1] = -1; prep.cs[0] = prep.cs[1] = 1.0f; prep.sn[0] = prep.sn[1] = 0.0f;
    if (heads && warp < 2) heads_prepare(p, row_tile, split, prep);       // (the uniform fields; these warps hold no row)
    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        // The weight operand does not depend on earlier kernels: its first tiles are requested
        // before the grid dependency is awaited, so they stream in while the kernel before this
        // one is still finishing.  The activation operand is requested only after the wait.
        if (lane == 0 && n_kb > 0) {
            const CUtensorMap* map_w = p.swapped ? &map_rows : &map_cols;
            const CUtensorMap* map_x = p.swapped ? &map_cols : &map_rows;
            const int w_y = p.swapped ? row_tile * TILE_ROWS : col_tile * p.block_cols;
            const int x_y = p.swapped ? col_tile * p.block_cols : row_tile * TILE_ROWS;
            const int w_off = p.swapped ? 0 : rows_bytes, x_off = p.swapped ? rows_bytes : 0;
            const int ahead = min(n_kb, p.stages);
            for (int i = 0; i < ahead; i++) {
                uint8_t* st = smem + (size_t)i * stage_bytes;
                mbar_expect_tx(&full_bar[i], (uint32_t)(rows_bytes + cols_bytes));
                tma_load_2d(st + w_off, map_w, &full_bar[i], (kb0 + i) * TILE_K, w_y);
            }
            pdl_wait();
            for (int i = 0; i < ahead; i++)
                tma_load_2d(smem + (size_t)i * stage_bytes + x_off, map_x, &full_bar[i], (kb0 + i) * TILE_K, x_y);
            // the ring position advances by counting (a division per k-block would sit on the critical path)
            int s = 0;
            uint32_t phase = 1;                      // ahead == stages here, so the ring has wrapped once
            for (int i = ahead; i < n_kb; i++) {
                if (!mbar_wait(&empty_bar[s], phase ^ 1u, abort_flag)) break;
                uint8_t* st = smem + (size_t)s * stage_bytes;
                mbar_expect_tx(&full_bar[s], (uint32_t)(rows_bytes + cols_bytes));
                tma_load_2d(st + w_off, map_w, &full_bar[s], (kb0 + i) * TILE_K, w_y);
                tma_load_2d(st + x_off, map_x, &full_bar[s], (kb0 + i) * TILE_K, x_y);
                if (++s == p.stages) { s = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0 && n_kb > 0) {
            const uint32_t idesc = umma_idesc(p.block_cols);
            bool ok = true;
            int s = 0;
            uint32_t phase = 0;
            for (int i = 0; i < n_kb && ok; i++) {
                ok = mbar_wait(&full_bar[s], phase, abort_flag);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                uint8_t* a = smem + (size_t)s * stage_bytes;
                const uint64_t da = umma_desc_sw128(a), db = umma_desc_sw128(a + rows_bytes);
#pragma unroll
                for (int k = 0; k < TILE_K / UMMA_K; k++) {
                    // advancing 16 bf16 = 32 bytes inside the swizzled row: +2 in the 16-byte address field
                    tcgen05_mma_bf16(tmem_d, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (i > 0 || k > 0) ? 1u : 0u);
                }
                tcgen05_commit(&empty_bar[s]);      // the stage is free once these MMAs have read it
                if (++s == p.stages) { s = 0; phase ^= 1u; }
            }
            tcgen05_commit(tmem_full_bar);          // the accumulator is complete once all MMAs have finished
        }
    } else if (n_kb > 0) {
        // -------------------------------------------------------------------- epilogue
        const int quad = warp & 3;                  // TMEM lane quadrant this warp may read
        if (heads) heads_prepare(p, row_tile, split, prep);       // step inputs only: fetched while the product runs
        pdl_wait();                                 // the output may still be read by earlier kernels until here
        const bool ok = mbar_wait(tmem_full_bar, 0, abort_flag);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (clustered) {
            // hand this block's partial sums to the blocks that finish them: row r goes to block r / rows_per
            __syncwarp();
            cluster_wait();                         // phase 1 complete: all blocks of the cluster run
            const int r = quad * 32 + lane;
            const uint32_t taddr_row = tmem_d + ((uint32_t)(quad * 32) << 16);
            if (heads) {
                // token column c goes to block c % S, which then holds the whole head (all 128 rows) of its tokens:
                // recv[split][c / S][row]
                const int S = p.cluster_splits, per = (p.block_cols + S - 1) / S;
                for (int c0 = 0; c0 < p.block_cols; c0 += 16) {
                    float v[16];
                    tmem_ld16(taddr_row + (uint32_t)c0, v);
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        const int c = c0 + j;
                        if (!ok || c >= p.M) continue;
                        const int owner = c % S, cl = c / S;
                        st_cluster_f32(map_to_rank(smem_u32(recv + ((size_t)split * per + cl) * TILE_ROWS + r), (uint32_t)owner), v[j]);
                    }
                }
            } else {
                const int owner = r / p.rows_per, rl = r - owner * p.rows_per;
                const uint32_t dst_row = map_to_rank(smem_u32(recv + ((size_t)split * p.rows_per + rl) * p.block_cols), (uint32_t)owner);
                for (int c0 = 0; c0 < p.block_cols; c0 += 16) {
                    float v[16];
                    tmem_ld16(taddr_row + (uint32_t)c0, v);
                    if (ok) {
#pragma unroll
                        for (int j = 0; j < 4; j++)
                            st_cluster_f32x4(dst_row + (uint32_t)(c0 + 4 * j) * 4u, v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                    }
                }
            }
        } else {
            const int r = quad * 32 + lane;         // accumulator row of this thread
            const uint32_t taddr_row = tmem_d + ((uint32_t)(quad * 32) << 16);
            const bool splitk = gridDim.z > 1;
            // Swapped orientation, K not cut, more than 16 tokens: a thread holds one weight row, so a token's outputs
            // from this tile are spread over the block's threads and stored one by one they are 2-byte stores 32 bytes
            // a warp (at 128 tokens that was 14 of the 8B gate/up's 54 us).  The tile is turned in shared memory instead
            // (the stages are free: every MMA has finished) and goes out as whole 16-byte pieces of token rows.
            const int elt = p.epilogue == 1 ? 4 : 2;
            const int out_cols = p.epilogue == 3 ? TILE_ROWS / 2 : TILE_ROWS;       // outputs a token gets from this tile
            const int row_bytes = out_cols * elt;
            const bool turned = p.swapped && !splitk && p.epilogue != 2 && p.block_cols > 16 &&
                                (row_tile + 1) * TILE_ROWS <= p.N &&
                                (size_t)p.block_cols * row_bytes <= (size_t)p.stages * stage_bytes &&
                                (reinterpret_cast<uintptr_t>(p.out) & 15) == 0 && ((size_t)p.ldc * elt) % 16 == 0;
            // (the turned tile has a barrier of the four epilogue warps in it: they go through it together or not at
            // all, whatever each of them saw of a wait that ran out)
            bool go = ok;
            if (turned) {
                uint32_t all;
                asm volatile(
                    "{\n.reg .pred p, q;\n"
                    "setp.ne.u32 p, %1, 0;\n"
                    "bar.red.and.pred q, 1, 128, p;\n"
                    "selp.u32 %0, 1, 0, q;\n}"
                    : "=r"(all) : "r"((uint32_t)ok) : "memory");
                go = all != 0;
            }
            if (turned && go) {
                uint8_t* turn = smem;                // [token][outputs of this tile]
                auto put = [&](int c, float x) {     // this thread's weight row, token column c
                    uint8_t* row = turn + (size_t)c * row_bytes;
                    if (p.epilogue == 3) {
                        const float other = __shfl_xor_sync(0xffffffffu, x, 1);             // gate rows are even, up rows odd
                        if ((lane & 1) == 0) reinterpret_cast<__nv_bfloat16*>(row)[r >> 1] = __float2bfloat16_rn(silu_mul(x, other));
                    } else if (p.epilogue == 0) {
                        reinterpret_cast<__nv_bfloat16*>(row)[r] = __float2bfloat16_rn(x);
                    } else {
                        reinterpret_cast<float*>(row)[r] = x;
                    }
                };
                // (64 columns a round trip to tensor memory, as the prefill epilogues read, gained nothing here)
                for (int c0 = 0; c0 < p.block_cols; c0 += 16) {
                    float v[16];
                    tmem_ld16(taddr_row + (uint32_t)c0, v);
#pragma unroll
                    for (int j = 0; j < 16; j++) put(c0 + j, v[j]);
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");      // the four epilogue warps
                const int m0 = col_tile * p.block_cols;
                const int tokens = min(p.block_cols, p.M - m0);
                const int pieces = row_bytes >> 4;
                uint8_t* out0 = reinterpret_cast<uint8_t*>(p.out) + (size_t)(row_tile * out_cols) * elt;
                for (int idx = (int)threadIdx.x - 64; idx < tokens * pieces; idx += GEMM_THREADS - 64) {
                    const int c = idx / pieces, o = idx - c * pieces;
                    *reinterpret_cast<uint4*>(out0 + (size_t)(m0 + c) * p.ldc * elt + (size_t)o * 16) =
                        *reinterpret_cast<const uint4*>(turn + (size_t)c * row_bytes + (size_t)o * 16);
                }
            }
            for (int c0 = (turned || !go) ? p.block_cols : 0; c0 < p.block_cols; c0 += 16) {
                float v[16];
                tmem_ld16(taddr_row + (uint32_t)c0, v);
                if (!p.swapped) {
                    const int m = row_tile * TILE_ROWS + r;
                    const int n0 = col_tile * p.block_cols + c0;
                    if (m >= p.M || n0 >= p.N) continue;
                    const int nv = min(16, p.N - n0);
                    if (splitk) {
                        float* dst = p.accum + (size_t)m * p.accum_ld + n0;
                        for (int j = 0; j < nv; j++) atomicAdd(dst + j, v[j]);
                    } else {
                        store_chunk_normal(p, m, n0, nv, v);
                    }
                } else {
                    const int n = row_tile * TILE_ROWS + r;
                    const int m0 = col_tile * p.block_cols + c0;
                    if (p.epilogue == 3 && !splitk) {
                        // gate rows are even, up rows odd: neighbours in the warp
#pragma unroll
                        for (int j = 0; j < 16; j++) {
                            const float other = __shfl_xor_sync(0xffffffffu, v[j], 1);
                            const int m = m0 + j;
                            if ((lane & 1) == 0 && n + 1 < p.N && m < p.M)
                                ((__nv_bfloat16*)p.out)[(size_t)m * p.ldc + (n >> 1)] = __float2bfloat16_rn(silu_mul(v[j], other));
                        }
                        continue;
                    }
                    if (n >= p.N) continue;
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        const int m = m0 + j;
                        if (m >= p.M) break;
                        if (splitk) {
                            atomicAdd(p.accum + (size_t)m * p.accum_ld + n, v[j]);
                        } else if (p.epilogue == 0) {
                            ((__nv_bfloat16*)p.out)[(size_t)m * p.ldc + n] = __float2bfloat16_rn(v[j]);
                        } else if (p.epilogue == 1) {
                            ((float*)p.out)[(size_t)m * p.ldc + n] = v[j];
                        } else {
                            float* dst = (float*)p.out + (size_t)m * p.ldc + n;
                            *dst = *dst + v[j];
                        }
                    }
                }
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }

    if (clustered) {
        // ---- sum the cluster's partial results for the rows this block finishes, in block order
        __syncwarp();
        if (warp < 2 || n_kb <= 0) cluster_wait();          // the epilogue warps already passed phase 1
        cluster_arrive();                                   // phase 2: all partial sums are written ...
        cluster_wait();                                     // ... and visible
        pdl_wait();
        const int S = p.cluster_splits, RP = p.rows_per, C = p.block_cols;
        const int row_base = row_tile * TILE_ROWS + split * RP;       // first weight row this block finishes
        const int rows_here = max(0, min(RP, TILE_ROWS - split * RP));
        if (heads) {
            finish_heads_swapped(p, recv, row_tile, split, *abort_flag != 0, prep);
        } else if (p.epilogue == 3) {
            const int pairs = rows_here >> 1;
            for (int idx = threadIdx.x; idx < pairs * C; idx += GEMM_THREADS) {
                const int c = idx / pairs, pr = idx - c * pairs;
                const int n = row_base + 2 * pr, m = col_tile * C + c;
                if (n + 1 >= p.N || m >= p.M) continue;
                float g = 0.0f, u = 0.0f;
                for (int s = 0; s < S; s++) {
                    g += recv[((size_t)s * RP + 2 * pr) * C + c];
                    u += recv[((size_t)s * RP + 2 * pr + 1) * C + c];
                }
                ((__nv_bfloat16*)p.out)[(size_t)m * p.ldc + (n >> 1)] = __float2bfloat16_rn(silu_mul(g, u));
            }
        } else {
            for (int idx = threadIdx.x; idx < rows_here * C; idx += GEMM_THREADS) {
                const int c = idx / rows_here, rl = idx - c * rows_here;
                const int n = row_base + rl, m = col_tile * C + c;
                if (n >= p.N || m >= p.M) continue;
                float v = 0.0f;
                for (int s = 0; s < S; s++) v += recv[((size_t)s * RP + rl) * C + c];
                if (p.epilogue == 0) ((__nv_bfloat16*)p.out)[(size_t)m * p.ldc + n] = __float2bfloat16_rn(v);
                else if (p.epilogue == 1) ((float*)p.out)[(size_t)m * p.ldc + n] = v;
                else {
                    float* dst = (float*)p.out + (size_t)m * p.ldc + n;
                    *dst = *dst + v;
                }
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag && p.err) atomicOr(p.err, EMBER_ERR_WAIT_LIMIT);
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(p.tmem_cols) : "memory");
    }
}

// ------------------------------------------------------------------ persistent kernel (prefill)
// Normal orientation only (accumulator rows are tokens).  One block per SM walks over output tiles
// (tile t -> weight column tile t / row_tiles, token row tile t % row_tiles, so that blocks running at
// the same time share weight tiles in L2).  Two accumulators live in tensor memory: while the four
// epilogue warps drain and store tile i, the MMA warp already fills the other accumulator with tile
// i + 1, and the TMA warp runs ahead through the ring of stages across tile borders.
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_rows, const __grid_constant__ CUtensorMap map_cols,
                          const GemmTcParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int rows_bytes = TILE_ROWS * TILE_K * 2;
    const int cols_bytes = p.block_cols * TILE_K * 2;
    const int stage_bytes = rows_bytes + ((cols_bytes + 1023) & ~1023);
    uint64_t* full_bar = (uint64_t*)(smem + (size_t)p.stages * stage_bytes);
    uint64_t* empty_bar = full_bar + MAX_STAGES;
    uint64_t* tmem_full_bar = empty_bar + MAX_STAGES;      // [2]
    uint64_t* tmem_empty_bar = tmem_full_bar + 2;           // [2]
    uint32_t* tmem_base_slot = (uint32_t*)(tmem_empty_bar + 2);
    volatile int* abort_flag = (volatile int*)(tmem_base_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_kb = p.num_k_blocks;
    // With few tiles (a short prompt portion) the K range of the adding epilogue is cut: a unit is a tile and a part
    // of K, its sums are added at the L2 like any other, and every SM has work.
    const int k_splits = (n_kb + p.k_blocks_per_split - 1) / p.k_blocks_per_split;
    const int units = p.total_tiles * k_splits;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; s++) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(&tmem_full_bar[a], 1);
            mbar_init(&tmem_empty_bar[a], 4);               // one arrival per epilogue warp
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_base_slot)), "r"(p.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = *tmem_base_slot;

    pdl_launch_dependents();
    pdl_wait();

    if (warp == 0) {
        if (lane == 0) {
            int s = 0;
            uint32_t phase = 0;                      // parity of the ring's current lap
            bool ok = true, wrapped = false;
            uint8_t* st = smem;
            for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
                const int t = u / k_splits, kb0 = (u - t * k_splits) * p.k_blocks_per_split;
                const int kb1 = min(n_kb, kb0 + p.k_blocks_per_split);
                const int col_tile = t / p.row_tiles, row_tile = t - col_tile * p.row_tiles;
                for (int i = kb0; i < kb1; i++) {
                    if (wrapped) ok = mbar_wait(&empty_bar[s], phase ^ 1u, abort_flag);
                    if (!ok) break;
                    mbar_expect_tx(&full_bar[s], (uint32_t)(rows_bytes + cols_bytes));
                    tma_load_2d(st, &map_rows, &full_bar[s], i * TILE_K, row_tile * TILE_ROWS);
                    tma_load_2d(st + rows_bytes, &map_cols, &full_bar[s], i * TILE_K, col_tile * p.block_cols);
                    st += stage_bytes;
                    if (++s == p.stages) { s = 0; st = smem; phase ^= 1u; wrapped = true; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(p.block_cols);
            int li = 0, s = 0;
            uint32_t phase = 0;
            bool ok = true;
            // descriptors advance with the ring: one stage is stage_bytes / 16 in the 16-byte address field
            const uint64_t da0 = umma_desc_sw128(smem), db0 = umma_desc_sw128(smem + rows_bytes);
            const uint64_t dstep = (uint64_t)(stage_bytes >> 4);
            uint64_t da = da0, db = db0;
            for (int u = blockIdx.x; u < units && ok; u += gridDim.x, li++) {
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
                        tcgen05_mma_bf16(d, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (i > kb0 || k > 0) ? 1u : 0u);
                    tcgen05_commit(&empty_bar[s]);
                    da += dstep; db += dstep;
                    if (++s == p.stages) { s = 0; phase ^= 1u; da = da0; db = db0; }
                }
                if (ok) tcgen05_commit(&tmem_full_bar[acc]);
            }
        }
    } else {
        const int quad = warp & 3;
        const int r = quad * 32 + lane;
        bool ok = true;
        int li = 0;
        for (int u = blockIdx.x; u < units; u += gridDim.x, li++) {
            const int t = u / k_splits;
            const int col_tile = t / p.row_tiles, row_tile = t - col_tile * p.row_tiles;
            const int acc = li & 1;
            const int m = row_tile * TILE_ROWS + r;
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
            if (lane == 0) mbar_arrive(&tmem_empty_bar[acc]);      // this warp has drained the accumulator
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag && p.err) atomicOr(p.err, EMBER_ERR_WAIT_LIMIT);
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(p.tmem_cols) : "memory");
    }
}

// Split-K finalize for the store epilogues: out = epilogue(accum), accum = 0.
__global__ void gemm_tc_finalize_kernel(float* __restrict__ accum, int accum_ld, void* __restrict__ out, int ldc, int M,
                                        int N, int epilogue) {
    pdl_launch_dependents();
    pdl_wait();
    const int n_out = epilogue == 3 ? N / 2 : N;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)M * n_out) return;
    const int m = (int)(idx / n_out), j = (int)(idx % n_out);
    float* a = accum + (size_t)m * accum_ld;
    if (epilogue == 3) {
        const float g = a[2 * j], u = a[2 * j + 1];
        a[2 * j] = 0.0f;
        a[2 * j + 1] = 0.0f;
        ((__nv_bfloat16*)out)[(size_t)m * ldc + j] = __float2bfloat16_rn(silu_mul(g, u));
    } else {
        const float c = a[j];
        a[j] = 0.0f;
        if (epilogue == 0) ((__nv_bfloat16*)out)[(size_t)m * ldc + j] = __float2bfloat16_rn(c);
        else ((float*)out)[(size_t)m * ldc + j] = c;
    }
}

// The same, four outputs a thread (16-byte loads of the sums, one 8- or 16-byte store): the row widths are multiples
// of four and the rows 16-byte aligned.  At 64 tokens the one-element kernel took 11 us a call, a tenth of the step.
template <int EPI>
__global__ void gemm_tc_finalize4_kernel(float* __restrict__ accum, int accum_ld, void* __restrict__ out, int ldc, int M, int n_out) {
    pdl_launch_dependents();
    pdl_wait();
    const int groups = n_out >> 2;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)M * groups) return;
    const int m = (int)(idx / groups), j = 4 * (int)(idx % groups);
    const float4 zero = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    float r0, r1, r2, r3;
    if (EPI == 3) {
        float4* a = reinterpret_cast<float4*>(accum + (size_t)m * accum_ld + 2 * j);
        const float4 x0 = a[0], x1 = a[1];
        a[0] = zero;
        a[1] = zero;
        r0 = silu_mul(x0.x, x0.y); r1 = silu_mul(x0.z, x0.w); r2 = silu_mul(x1.x, x1.y); r3 = silu_mul(x1.z, x1.w);
    } else {
        float4* a = reinterpret_cast<float4*>(accum + (size_t)m * accum_ld + j);
        const float4 x = a[0];
        a[0] = zero;
        r0 = x.x; r1 = x.y; r2 = x.z; r3 = x.w;
    }
    if (EPI == 1) {
        *reinterpret_cast<float4*>((float*)out + (size_t)m * ldc + j) = make_float4(r0, r1, r2, r3);
    } else {
        __nv_bfloat162 lo = __floats2bfloat162_rn(r0, r1), hi = __floats2bfloat162_rn(r2, r3);
        uint2 u;
        u.x = *reinterpret_cast<uint32_t*>(&lo);
        u.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>((__nv_bfloat16*)out + (size_t)m * ldc + j) = u;
    }
}

// ------------------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

}  // namespace ember
