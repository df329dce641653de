// Causal grouped-query attention over a paged cache, general form (SIMT, fp32 math).
//
// Formula (src/backend/cpu/cpu_backend.cpp:174-198): for the token at position p and head h of
// key/value head kvh = h / group, s_j = dot(q_h, K[kvh][j]) * scale for the visible keys
// j <= p (and j > p - window when a window is set), softmax over j, o = sum_j w_j V[kvh][j].
// Causality is the key range, there is no mask tensor.
//
// This kernel serves the float32 path (fp32 pages) and is the bf16 path's fall-back for head
// sizes the tensor-core kernels do not take.  Work unit: a tile of up to `tile_q` consecutive
// query tokens of one sequence x one key/value head (all `group` query heads of it share the
// key tiles) x one split of the key range.  Splits have a fixed length anchored at key 0 and
// are merged in ascending order by attention_combine, so the result for a token does not
// depend on what else is in the step.
#include "common.cuh"

EMBER_DEFINE_LAST_ERROR

namespace ember {

constexpr int ATT_WARPS = 8;
constexpr int ATT_ROWS_PER_WARP = 4;
constexpr int ATT_MAX_ROWS = ATT_WARPS * ATT_ROWS_PER_WARP;  // tile_q * group <= 32
constexpr int ATT_KT = 32;                                     // keys per shared-memory tile

struct AttnParams {
    const void* q;        // [T, n_heads, D]
    const void* k_pool;   // [pages][n_kv][page][D]
    const void* v_pool;
    void* out;            // [T, n_heads, D]
    float* part_o;        // [T, n_heads, n_splits, D]   (n_splits > 1)
    float* part_ml;       // [T, n_heads, n_splits, 2]
    const int* tiles;     // [n_tiles, 4] = (sequence, first token row, queries, position of the first query)
    const int* block_table;
    int max_blocks, page, num_pages;
    int n_heads, n_kv, D;
    int window;           // 0 = all keys
    float scale;
    int n_splits, split_keys;
    int* err;
};

template <typename T, int NC>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attention_tile_kernel(AttnParams p) {
    extern __shared__ float smem[];
    pdl_launch_dependents();
    pdl_wait();
    const int D = p.D, DP = D + 1;
    float* Ks = smem;                       // [KT][D+1]
    float* Vs = Ks + ATT_KT * DP;           // [KT][D]
    float* Qs = Vs + ATT_KT * D;            // [rows][D]

    const int tile = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    const int seq = p.tiles[tile * 4 + 0], row0 = p.tiles[tile * 4 + 1], nq = p.tiles[tile * 4 + 2],
              pos0 = p.tiles[tile * 4 + 3];
    const int G = p.n_heads / p.n_kv;
    const int rows = nq * G;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T* q = (const T*)p.q;
    const T* kp = (const T*)p.k_pool;
    const T* vp = (const T*)p.v_pool;

    // queries of this tile -> shared memory (row r = query r / G, head kvh * G + r % G)
    for (int idx = threadIdx.x; idx < rows * D; idx += blockDim.x) {
        const int r = idx / D, d = idx - r * D;
        const int qi = r / G, g = r - qi * G;
        Qs[r * D + d] = to_float(q[((size_t)(row0 + qi) * p.n_heads + kvh * G + g) * D + d]);
    }

    int lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
    int hi = pos0 + nq;  // exclusive
    if (p.n_splits > 1) {
        lo = max(lo, split * p.split_keys);
        hi = min(hi, (split + 1) * p.split_keys);
    }

    float m[ATT_ROWS_PER_WARP], l[ATT_ROWS_PER_WARP], acc[ATT_ROWS_PER_WARP][NC];
#pragma unroll
    for (int i = 0; i < ATT_ROWS_PER_WARP; i++) {
        m[i] = -INFINITY;
        l[i] = 0.0f;
#pragma unroll
        for (int c = 0; c < NC; c++) acc[i][c] = 0.0f;
    }

    const int* bt = p.block_table + (size_t)seq * p.max_blocks;
    for (int k0 = lo - (lo % ATT_KT); k0 < hi; k0 += ATT_KT) {
        __syncthreads();  // previous tile fully consumed (also orders the Qs writes before the first use)
        for (int idx = threadIdx.x; idx < ATT_KT * D; idx += blockDim.x) {
            const int j = idx / D, d = idx - j * D;
            const int key = k0 + j;
            float kv = 0.0f, vv = 0.0f;
            if (key >= lo && key < hi) {
                const int blk = bt[key / p.page];
                if (blk >= 0 && blk < p.num_pages) {
                    const size_t off = (((size_t)blk * p.n_kv + kvh) * p.page + (key % p.page)) * D + d;
                    kv = to_float(kp[off]);
                    vv = to_float(vp[off]);
                } else if (d == 0 && p.err) {
                    atomicOr(p.err, EMBER_ERR_PAGE_RANGE);
                }
            }
            Ks[j * DP + d] = kv;
            Vs[j * D + d] = vv;
        }
        __syncthreads();

#pragma unroll
        for (int i = 0; i < ATT_ROWS_PER_WARP; i++) {
            const int r = warp + i * ATT_WARPS;
            if (r >= rows) continue;  // uniform per warp
            const int qpos = pos0 + r / G;
            const int key = k0 + lane;
            const bool visible = key >= lo && key < hi && key <= qpos && (p.window <= 0 || key > qpos - p.window);
            float s = 0.0f;
            const float* qr = Qs + r * D;
            const float* kr = Ks + lane * DP;
            for (int d = 0; d < D; d++) s = fmaf(qr[d], kr[d], s);
            s = visible ? s * p.scale : -INFINITY;
            const float tmax = warp_max(s);
            const float m_new = fmaxf(m[i], tmax);
            if (m_new == -INFINITY) continue;  // nothing visible so far (uniform per warp)
            const float corr = expf(m[i] - m_new);  // m = -inf -> 0
            const float pj = visible ? expf(s - m_new) : 0.0f;
            l[i] = l[i] * corr + warp_sum(pj);
            m[i] = m_new;
#pragma unroll
            for (int c = 0; c < NC; c++) acc[i][c] *= corr;
            for (int j = 0; j < ATT_KT; j++) {
                const float w = __shfl_sync(0xffffffffu, pj, j);
                const float* vr = Vs + j * D;
#pragma unroll
                for (int c = 0; c < NC; c++) {
                    const int d = lane + 32 * c;
                    if (d < D) acc[i][c] = fmaf(w, vr[d], acc[i][c]);
                }
            }
        }
    }

#pragma unroll
    for (int i = 0; i < ATT_ROWS_PER_WARP; i++) {
        const int r = warp + i * ATT_WARPS;
        if (r >= rows) continue;
        const int qi = r / G, g = r - qi * G;
        const size_t th = (size_t)(row0 + qi) * p.n_heads + kvh * G + g;
        if (p.n_splits <= 1) {
            const float inv = l[i] > 0.0f ? 1.0f / l[i] : 0.0f;
            T* o = (T*)p.out + th * D;
#pragma unroll
            for (int c = 0; c < NC; c++) {
                const int d = lane + 32 * c;
                if (d < D) o[d] = from_float<T>(acc[i][c] * inv);
            }
        } else {
            float* po = p.part_o + (th * p.n_splits + split) * D;
#pragma unroll
            for (int c = 0; c < NC; c++) {
                const int d = lane + 32 * c;
                if (d < D) po[d] = acc[i][c];
            }
            if (lane == 0) {
                float* ml = p.part_ml + (th * p.n_splits + split) * 2;
                ml[0] = m[i];
                ml[1] = l[i];
            }
        }
    }
}

// Merges the partial results of the splits of one (token, head) in ascending split order.
template <typename T>
__global__ void attention_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                         T* __restrict__ out, int n_splits, int D) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t th = blockIdx.x;
    const float* ml = part_ml + th * n_splits * 2;
    float M = -INFINITY;
    for (int s = 0; s < n_splits; s++) M = fmaxf(M, ml[2 * s]);
    float L = 0.0f;
    for (int s = 0; s < n_splits; s++) {
        const float ms = ml[2 * s];
        if (ms != -INFINITY) L += ml[2 * s + 1] * expf(ms - M);
    }
    const float inv = L > 0.0f ? 1.0f / L : 0.0f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float o = 0.0f;
        for (int s = 0; s < n_splits; s++) {
            const float ms = ml[2 * s];
            if (ms != -INFINITY) o = fmaf(part_o[(th * n_splits + s) * D + d], expf(ms - M), o);
        }
        out[th * D + d] = from_float<T>(o * inv);
    }
}

template <typename T>
int launch_attention(const AttnParams& p, int n_tiles, int T_tokens, cudaStream_t st) {
    const int D = p.D;
    const int G = p.n_heads / p.n_kv;
    const size_t smem = ((size_t)ATT_KT * (D + 1) + (size_t)ATT_KT * D + (size_t)ATT_MAX_ROWS * D) * sizeof(float);
    dim3 grid(n_tiles, p.n_kv, p.n_splits);
    const int nc = (D + 31) / 32;
    auto run = [&](auto kernel) -> int {
        if (smem > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return fail("attention: shared memory %zu: %s", smem, cudaGetErrorString(e));
        }
        launch_kernel(kernel, grid, ATT_WARPS * 32, smem, st, p);
        return check_launch("attention");
    };
    int rc;
    if (nc <= 1) rc = run(attention_tile_kernel<T, 1>);
    else if (nc <= 2) rc = run(attention_tile_kernel<T, 2>);
    else if (nc <= 4) rc = run(attention_tile_kernel<T, 4>);
    else rc = run(attention_tile_kernel<T, 8>);
    if (rc) return rc;
    (void)G;
    if (p.n_splits > 1) {
        launch_kernel(attention_combine_kernel<T>, (unsigned)((size_t)T_tokens * p.n_heads), D >= 128 ? 128 : 64, 0, st,
                      (const float*)p.part_o, (const float*)p.part_ml, (T*)p.out, p.n_splits, D);
        return check_launch("attention_combine");
    }
    return 0;
}

}  // namespace ember

using namespace ember;

// The largest number of query tokens a tile may hold for a given group size.
EMBER_API int ember_attention_tile_queries(int group) {
    if (group <= 0 || group > ATT_MAX_ROWS) return 0;
    return ATT_MAX_ROWS / group;
}

EMBER_API int ember_attention(const void* q, const void* k_pool, const void* v_pool, void* out, int dtype,
                              int T_tokens, int n_heads, int n_kv, int D, const int* tiles, int n_tiles, int tile_q,
                              const int* block_table, int max_blocks, int page, int num_pages, int window,
                              float scale, int n_splits, int split_keys, float* part_o, float* part_ml, int* err,
                              void* stream) {
    if (n_tiles <= 0 || T_tokens <= 0) return 0;
    if (D <= 0 || D > 256 || (D & 1)) return fail("attention: head size %d is not an even number up to 256", D);
    if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv) return fail("attention: %d heads do not divide into %d groups", n_heads, n_kv);
    const int G = n_heads / n_kv;
    if (G > ATT_MAX_ROWS) return fail("attention: %d query heads per key/value head; this kernel takes up to %d", G, ATT_MAX_ROWS);
    if (tile_q <= 0 || tile_q * G > ATT_MAX_ROWS) return fail("attention: tiles of %d queries x group %d exceed %d rows", tile_q, G, ATT_MAX_ROWS);
    if (n_splits < 1 || (n_splits > 1 && (split_keys <= 0 || !part_o || !part_ml)))
        return fail("attention: bad split configuration (%d splits of %d keys)", n_splits, split_keys);
    if (n_splits > 65535 || n_kv > 65535) return fail("attention: grid too large");
    if (page <= 0 || max_blocks <= 0 || num_pages <= 0) return fail("attention: bad cache geometry");
    AttnParams p;
    p.q = q; p.k_pool = k_pool; p.v_pool = v_pool; p.out = out; p.part_o = part_o; p.part_ml = part_ml;
    p.tiles = tiles; p.block_table = block_table; p.max_blocks = max_blocks; p.page = page; p.num_pages = num_pages;
    p.n_heads = n_heads; p.n_kv = n_kv; p.D = D; p.window = window; p.scale = scale;
    p.n_splits = n_splits; p.split_keys = split_keys; p.err = err;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == EMBER_F32) return launch_attention<float>(p, n_tiles, T_tokens, st);
    if (dtype == EMBER_BF16) return launch_attention<__nv_bfloat16>(p, n_tiles, T_tokens, st);
    return fail("attention: unsupported dtype %d", dtype);
}
