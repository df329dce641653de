// bf16 matrix product on the 5th-generation tensor cores: C[M,N] = A[M,K] . W[N,K]^T.
//
// Blackwell-native structure: operand tiles are brought to shared memory by TMA
// (cp.async.bulk.tensor, 128-byte swizzle) through a ring of mbarrier-guarded stages; one
// elected thread issues tcgen05.mma (128 x N x 16, bf16 in, fp32 accumulate) with the
// accumulator in tensor memory; tcgen05.commit hands stages back to the producer and signals
// the epilogue warps, which read the accumulator with tcgen05.ld and apply the fused epilogue.
// Warp roles: warp 0 TMA producer, warp 1 MMA issuer and TMEM owner, warps 2-5 epilogue.
//
// Two orientations share the kernel.  "normal": the 128 accumulator rows are 128 tokens, the
// columns a slice of weight rows (prefill).  "swapped": the 128 accumulator rows are 128 weight
// rows and the columns are the (few) tokens, so a decode step with 1..128 tokens wastes no
// tensor-core rows and streams every weight exactly once; the epilogue writes transposed.
// With few output tiles the K range is split over gridDim.z and partial sums are combined by
// fp32 atomic adds (into the residual for the add epilogue, else into a zeroed scratch matrix
// that a small finalize kernel converts and clears).
//
// Every wait on an mbarrier is bounded: when the limit is reached the kernel records
// EMBER_ERR_WAIT_LIMIT, every role falls through to the common exit, and the TMEM is freed.
//
// The reference's products (src/backend/cuda/k_gemm.cu:65-405) are mma.sync kernels for Turing;
// nothing of them is reused here.
#include <map>
#include <mutex>
#include <tuple>

#include "gemm_tc_kernel.cuh"
#include "gemm_tc_pair.cuh"

EMBER_DEFINE_LAST_ERROR

namespace ember {

// Tensor maps are cached by (pointer, rows, K, box rows): weights keep theirs for good, and the
// few activation buffers are reused step after step.
static bool tensor_map(const void* ptr, int rows, int K, int box_rows, CUtensorMap* out) {
    static std::map<std::tuple<const void*, int, int, int>, CUtensorMap> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    auto key = std::make_tuple(ptr, rows, K, box_rows);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return true;
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {(cuuint32_t)TILE_K, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUtensorMap m;
    CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return false;
    if (cache.size() > 4096) cache.clear();
    cache[key] = m;
    *out = m;
    return true;
}

// How many pairs of blocks of the pair kernel the device runs at once (0: it cannot).
static int pair_capacity(int num_sms) {
    static int max_pairs = -1;
    if (max_pairs < 0) {
        int n = 0;
        if (cudaFuncSetAttribute(gemm_tc_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) == cudaSuccess) {
            cudaLaunchConfig_t q = {};
            q.gridDim = dim3(2 * (num_sms / 2));
            q.blockDim = dim3(GEMM_THREADS);
            q.dynamicSmemBytes = 227 * 1024 - 2048;
            cudaLaunchAttribute a[1];
            a[0].id = cudaLaunchAttributeClusterDimension;
            a[0].val.clusterDim.x = 2; a[0].val.clusterDim.y = 1; a[0].val.clusterDim.z = 1;
            q.attrs = a; q.numAttrs = 1;
            if (cudaOccupancyMaxActiveClusters(&n, gemm_tc_pair_kernel, &q) != cudaSuccess) { cudaGetLastError(); n = 0; }
        } else {
            cudaGetLastError();
        }
        max_pairs = n < num_sms / 2 ? n : num_sms / 2;
    }
    return max_pairs;
}

// Tile width for a prefill-sized product.  The time is about (waves of tiles over the SMs) x (tile width + a
// fixed cost per tile), so a narrower tile wins when it fills the last wave or brings idle SMs in: N = 2048 on
// 148 SMs with 16 row tiles runs 144 tiles of 240 columns in one wave, faster than 128 tiles of 256.  Tiles
// narrower than 192 columns re-read the token rows too often to pay.
static int best_block_cols(int M, int N, int slots, int units, double* cost_out) {
    const int rows = TILE_ROWS * units, step = 16;
    const int row_tiles = (M + rows - 1) / rows;
    int best = 256;
    double best_cost = 1e30;
    for (int bc = 256; bc >= 192; bc -= step) {
        const long long tiles = (long long)row_tiles * ((N + bc - 1) / bc);
        const double cost = (double)((tiles + slots - 1) / slots) * (bc + 40);
        if (cost < best_cost * 0.999) { best_cost = cost; best = bc; }
    }
    if (N <= 128) { best = 128; best_cost = (double)((row_tiles + slots - 1) / slots) * (128 + 40); }
    if (const char* f = getenv("EMBER_GEMM_TILE_COLS")) {       // tuning aid: force the width (a multiple of 16)
        const int v = atoi(f);
        if (v >= 32 && v <= 256 && v % 16 == 0) best = v;
    }
    if (cost_out) *cost_out = best_cost;
    return best;
}

// The adding epilogue may cut K as well (its sums are added at the L2 whatever their number): tile width and number
// of K parts together, by a model of the time -- waves of units over the slots, a unit costing its k-blocks at the
// tile's MMA rate plus a fixed share for its fill and its epilogue.  (1,024 tokens, N = 2048, K = 6144: 88 tiles of
// 192 columns over all of K took 36 us; 64 tiles of 256 columns in two parts of K take half of that.)
static void best_tile_and_parts(int M, int N, int num_k_blocks, int slots, int units, int* block_cols, int* k_splits) {
    const int rows = TILE_ROWS * units;
    const int row_tiles = (M + rows - 1) / rows;
    double best = 1e30;
    for (int bc = 256; bc >= 192; bc -= 16) {
        const long long tiles = (long long)row_tiles * ((N + bc - 1) / bc);
        for (int ks = 1; ks <= 16; ks++) {
            if (ks > 1 && num_k_blocks / ks < 8) break;
            const int kbps = (num_k_blocks + ks - 1) / ks;
            const long long n_units = tiles * ((num_k_blocks + kbps - 1) / kbps);
            const double cost = (double)((n_units + slots - 1) / slots) * ((double)kbps * 2.0 * (bc + 40) + 6000.0);
            if (cost < best * 0.999) { best = cost; *block_cols = bc; *k_splits = ks; }
        }
    }
}

// The pair kernel: 256-token tiles on clusters of two blocks, as many pairs as the device co-schedules.
static int launch_pair(const void* A, const void* W, GemmTcParams p, int block_cols, int max_pairs, cudaStream_t st) {
    p.block_cols = block_cols;
    p.row_tiles = (p.M + 2 * TILE_ROWS - 1) / (2 * TILE_ROWS);
    p.total_tiles = p.row_tiles * ((p.N + block_cols - 1) / block_cols);
    p.tmem_cols = 512;
    p.cluster_splits = 1;
    int k_splits = 1;                                  // the adding epilogue: tile width and parts of K together
    if (p.epilogue == 2 && p.N > 128 && !getenv("EMBER_GEMM_TILE_COLS")) {
        best_tile_and_parts(p.M, p.N, p.num_k_blocks, max_pairs, 2, &block_cols, &k_splits);
        p.block_cols = block_cols;
        p.total_tiles = p.row_tiles * ((p.N + block_cols - 1) / block_cols);
    }
    p.k_blocks_per_split = (p.num_k_blocks + k_splits - 1) / k_splits;
    k_splits = (p.num_k_blocks + p.k_blocks_per_split - 1) / p.k_blocks_per_split;
    const int units = p.total_tiles * k_splits;
    const int stage_bytes = pair_stage_bytes(block_cols);
    int stages = (200 * 1024) / stage_bytes;
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    if (stages > p.num_k_blocks) stages = p.num_k_blocks < 2 ? 2 : p.num_k_blocks;
    p.stages = stages;
    const size_t smem = (size_t)stages * stage_bytes + 1024 + 256;
    CUtensorMap map_rows, map_cols;
    if (!tensor_map(A, p.M, p.K, TILE_ROWS, &map_rows) || !tensor_map(W, p.N, p.K, block_cols / 2, &map_cols))
        return fail("gemm_tc: cuTensorMapEncodeTiled failed or is unavailable");
    const int pairs = units < max_pairs ? units : max_pairs;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attrs[2];
    attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    attrs[1].id = cudaLaunchAttributeClusterDimension;
    attrs[1].val.clusterDim.x = 2; attrs[1].val.clusterDim.y = 1; attrs[1].val.clusterDim.z = 1;
    cfg.attrs = attrs; cfg.numAttrs = 2;
    cudaLaunchKernelEx(&cfg, gemm_tc_pair_kernel, map_rows, map_cols, p);
    return check_launch("gemm_tc_pair");
}

// The single-SM persistent kernel (normal orientation): one block per SM walks the tiles of 128 tokens x block_cols.
static int launch_persistent(const void* A, const void* W, GemmTcParams p, int block_cols, int num_sms, cudaStream_t st) {
    p.swapped = 0;
    p.block_cols = block_cols;
    p.row_tiles = (p.M + TILE_ROWS - 1) / TILE_ROWS;
    p.total_tiles = p.row_tiles * ((p.N + block_cols - 1) / block_cols);
    p.cluster_splits = 1;
    p.rows_per = TILE_ROWS;
    // a short prompt portion has fewer tiles than the device has SMs; the adding epilogue (its sums are added at the L2
    // anyway) then cuts K so that every SM gets a unit of at least 8 k-blocks (512 tokens, K = 6144: 34 -> 12 us)
    int k_splits = 1;
    if (p.epilogue == 2 && p.N > 128 && !getenv("EMBER_GEMM_TILE_COLS")) {
        best_tile_and_parts(p.M, p.N, p.num_k_blocks, num_sms, 1, &block_cols, &k_splits);
        p.block_cols = block_cols;
        p.total_tiles = p.row_tiles * ((p.N + block_cols - 1) / block_cols);
    }
    p.k_blocks_per_split = (p.num_k_blocks + k_splits - 1) / k_splits;
    k_splits = (p.num_k_blocks + p.k_blocks_per_split - 1) / p.k_blocks_per_split;
    const int units = p.total_tiles * k_splits;
    p.accum = nullptr; p.accum_ld = 0;
    int tc = 32;
    while (tc < 2 * block_cols) tc <<= 1;
    p.tmem_cols = tc;
    const int rows_bytes = TILE_ROWS * TILE_K * 2;
    const int stage_bytes = rows_bytes + ((block_cols * TILE_K * 2 + 1023) & ~1023);
    int stages = (200 * 1024) / stage_bytes;
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    if (stages < 2) stages = 2;
    if (stages > p.num_k_blocks) stages = p.num_k_blocks < 2 ? 2 : p.num_k_blocks;
    p.stages = stages;
    const size_t smem = (size_t)stages * stage_bytes + 1024 /* alignment slack */ + 256 /* barriers */;
    CUtensorMap map_rows, map_cols;
    if (!tensor_map(A, p.M, p.K, TILE_ROWS, &map_rows) || !tensor_map(W, p.N, p.K, block_cols, &map_cols))
        return fail("gemm_tc: cuTensorMapEncodeTiled failed or is unavailable");
    static bool pattr = false;
    if (!pattr) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return fail("gemm_tc: cannot raise the shared-memory limit: %s", cudaGetErrorString(e));
        pattr = true;
    }
    const int blocks = units < num_sms ? units : num_sms;
    launch_kernel(gemm_tc_persistent_kernel, dim3(blocks), dim3(GEMM_THREADS), smem, st, map_rows, map_cols, p);
    return check_launch("gemm_tc_persistent");
}

}  // namespace ember

using namespace ember;

// Whether the tensor-core product takes these sizes (bf16 operands are the caller's business).
EMBER_API int ember_gemm_tc_supported(int M, int N, int K, int epilogue) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if (K % 8) return 0;                       // TMA needs 16-byte row pitch
    if (epilogue == 3 && (N & 1)) return 0;
    if (epilogue == 5 && M > 128) return 0;    // the sums stay in the scratch of the small-M product
    return 1;
}

// How many floats of zeroed scratch a call may need (0 if none).
EMBER_API long long ember_gemm_tc_scratch_floats(int max_tokens_swapped, int N) {
    return (long long)max_tokens_swapped * N;
}

// C = A . W^T with the fused epilogue.  `scratch` is a zero-filled fp32 buffer of at least
// min(M, 128) * N floats (used only when the K range is split; it is left zeroed).
// Epilogue 5 (at most 128 tokens): the fp32 sums are left in `scratch` as [M, N] for a consumer that reads them and
// sets them back to zero (`out` is not used); it saves the pass that rounds, stores and clears.
EMBER_API int ember_gemm_tc(const void* A, const void* W, void* out, int ldc, int M, int N, int K, int epilogue,
                            float* scratch, long long scratch_floats, int num_sms, int split_mode, int* err, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    const bool sums = epilogue == 5;
    if (sums) {
        if (M > 128 || !scratch || scratch_floats < (long long)M * N)
            return fail("gemm_tc: sums in scratch need at most 128 tokens and %lld floats of scratch, got M=%d and %lld", (long long)M * N, M, scratch_floats);
        out = scratch; ldc = N; epilogue = 1;          // with K in one part the sums are stored like any fp32 result
    }
    if (!ember_gemm_tc_supported(M, N, K, epilogue))
        return fail("gemm_tc: sizes M=%d N=%d K=%d (epilogue %d) are not taken; K must be a multiple of 8", M, N, K, epilogue);
    if ((((uintptr_t)A) & 15) || (((uintptr_t)W) & 15)) return fail("gemm_tc: operands must be 16-byte aligned");
    if (num_sms <= 0) num_sms = 148;
    cudaStream_t st = (cudaStream_t)stream;

    GemmTcParams p;
    p.M = M; p.N = N; p.K = K;
    p.swapped = M <= 128 ? 1 : 0;
    p.num_k_blocks = (K + TILE_K - 1) / TILE_K;
    int row_tiles, col_tiles;
    if (p.swapped) {
        p.block_cols = ((M + 15) / 16) * 16;
        row_tiles = (N + TILE_ROWS - 1) / TILE_ROWS;
        col_tiles = 1;
    } else {
        // Prefill-sized products: the single-SM persistent kernel or pairs of SMs (tcgen05 cta_group::2),
        // each with the tile width that fills its waves best.  Under the power cap pairs are the more efficient
        // kernel (an SM reads half of the weight tile) and win from about 2,048 tokens on (a 2,048-token prefill
        // step: 7.55 ms with pairs, 7.9 ms without; at 1,024 tokens the single-SM kernel is 1 % ahead).
        // split_mode 4 asks for pairs whenever the device takes them, 5 forbids them, 3 runs one tile per block.
        double cost_single = 0, cost_pair = 0;
        const int bc_single = split_mode == 3 ? (N >= 1024 ? 256 : 128) : best_block_cols(M, N, num_sms, 1, &cost_single);
        if (split_mode != 3 && split_mode != 5 && N >= 32) {
            const int max_pairs = pair_capacity(num_sms);
            if (max_pairs > 0) {
                const int bc_pair = best_block_cols(M, N, max_pairs, 2, &cost_pair);
                if (split_mode == 4 || (M >= 2048 && cost_pair <= cost_single * 1.001)) {
                    p.epilogue = epilogue; p.out = out; p.ldc = ldc; p.err = err;
                    p.accum = nullptr; p.accum_ld = 0; p.rows_per = TILE_ROWS; p.stages = 0;
                    return launch_pair(A, W, p, bc_pair, max_pairs, st);
                }
            }
        }
        if (split_mode != 3) {
            p.epilogue = epilogue; p.out = out; p.ldc = ldc; p.err = err;
            return launch_persistent(A, W, p, bc_single, num_sms, st);
        }
        p.block_cols = bc_single;
        row_tiles = (M + TILE_ROWS - 1) / TILE_ROWS;
        col_tiles = (N + p.block_cols - 1) / p.block_cols;
    }
    // With few output tiles the K range is split so that every SM streams weights.  Two ways to
    // sum the partial results (split_mode 0 picks one):
    //   cluster: the splits of a tile form a thread-block cluster and are summed in shared memory,
    //            in block order (no scratch, no second kernel) -- best for up to 16 tokens;
    //   atomic:  fp32 atomic adds into the residual (add epilogue) or into zeroed scratch that a
    //            small kernel converts and clears -- best for wider token tiles.
    // The split count depends on N and K only.
    const int tiles = row_tiles * col_tiles;
    const bool store_epilogue = epilogue != 2;
    const bool use_cluster = split_mode == 2 || split_mode >= 32 || (split_mode == 0 && p.block_cols <= 16 && store_epilogue);
    int splits = 1;
    if (p.swapped && use_cluster && split_mode >= 32) {
        splits = split_mode - 32;                      // tuning and tests: a cluster of this many blocks
        if (splits > 8) splits = 8;
        if (splits < 1) splits = 1;
        while (splits > 1 && p.num_k_blocks / splits < 2) splits--;
    } else if (p.swapped && use_cluster) {
        // fill the SMs once: clusters of up to 8 blocks, at least 2 k-blocks each
        if (tiles < num_sms) {
            splits = (num_sms + tiles - 1) / tiles;
            if (splits > 8) splits = 8;
            while (splits > 1 && p.num_k_blocks / splits < 2) splits--;
        }
    } else if (p.swapped && split_mode >= 16 && split_mode < 32) {
        splits = split_mode - 16;                      // tuning and tests: this many parts of K, summed with atomics
        if (splits < 1) splits = 1;
        while (splits > 1 && p.num_k_blocks / splits < 2) splits--;
    } else if (p.swapped && p.block_cols > 16) {
        // Token tiles of 17 to 128: two such blocks fit on an SM, the stream reaches the memory's rate once about
        // that many blocks are in flight, and every further part of K costs atomics and a wider finalize pass.  So:
        // as many parts as keep tiles x parts within two blocks an SM, at least four k-blocks each.  Measured at 64
        // tokens (us; parts in brackets): 1.7B widths q/k/v 12.6 (8), O 7.7 (8), gate/up 18.1 (3), down 10.5 (16),
        // head 137 (1); 8B widths 18.6 (6), 11.9 (8), 43.0 (1), 22.3 (8), 232 (1).  (Counting waves over the SMs
        // alone gave the head 16 parts, 364 us, and the 8B gate/up 3 parts, 51 us.)
        splits = 2 * num_sms / (tiles > 0 ? tiles : 1);
        if (splits > 16) splits = 16;
        if (splits > p.num_k_blocks / 4) splits = p.num_k_blocks / 4;
        if (splits < 1) splits = 1;
    } else if (p.swapped) {
        // minimise the number of waves over the SMs; a larger split must pay for itself
        double best = 1e30;
        for (int sct = 1; sct <= 16; sct++) {
            if (sct > 1 && p.num_k_blocks / sct < 2) break;
            const double waves = (double)((tiles * sct + num_sms - 1) / num_sms) / sct;
            if (waves < best * 0.9) { best = waves; splits = sct; }
        }
    }
    p.k_blocks_per_split = (p.num_k_blocks + splits - 1) / splits;
    splits = (p.num_k_blocks + p.k_blocks_per_split - 1) / p.k_blocks_per_split;
    p.epilogue = epilogue; p.out = out; p.ldc = ldc; p.err = err;
    p.accum = nullptr; p.accum_ld = 0;
    p.cluster_splits = use_cluster ? splits : 1;
    p.rows_per = (use_cluster && splits > 1) ? 2 * ((TILE_ROWS / 2 + splits - 1) / splits) : TILE_ROWS;
    if (!use_cluster && splits > 1) {
        if (epilogue == 2) {
            p.accum = (float*)out;
            p.accum_ld = ldc;
        } else {
            if (!scratch || scratch_floats < (long long)M * N)
                return fail("gemm_tc: split-K needs %lld floats of zeroed scratch, got %lld", (long long)M * N, scratch_floats);
            p.accum = scratch;
            p.accum_ld = N;
        }
    }
    p.row_tiles = row_tiles;
    p.total_tiles = row_tiles * col_tiles;
    int tc = 32;
    while (tc < p.block_cols) tc <<= 1;
    p.tmem_cols = tc;
    const int rows_bytes = TILE_ROWS * TILE_K * 2;
    const int cols_bytes = p.block_cols * TILE_K * 2;
    const int stage_bytes = rows_bytes + ((cols_bytes + 1023) & ~1023);
    const size_t recv_bytes = p.cluster_splits > 1 ? (size_t)splits * p.rows_per * p.block_cols * sizeof(float) : 0;
    // Decode-sized tiles keep their blocks small (about 96 KiB of stages) so that two or three fit on
    // an SM: the next kernel's blocks become resident and prefetch their weights while this kernel
    // drains, and the memory system sees more independent streams.  Prefill tiles take all they can.
    const size_t budget = p.swapped ? (size_t)96 * 1024 : (size_t)200 * 1024 - recv_bytes;
    int stages = (int)(budget / stage_bytes);
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    if (stages < 2) stages = 2;
    if (stages > p.k_blocks_per_split) stages = p.k_blocks_per_split < 2 ? 2 : p.k_blocks_per_split;
    p.stages = stages;
    const size_t smem = (size_t)stages * stage_bytes + 1024 /* alignment slack */ + 256 /* barriers */ + recv_bytes;

    CUtensorMap map_rows, map_cols;
    const void* rows_ptr = p.swapped ? W : A;
    const void* cols_ptr = p.swapped ? A : W;
    const int rows_extent = p.swapped ? N : M, cols_extent = p.swapped ? M : N;
    if (!tensor_map(rows_ptr, rows_extent, K, TILE_ROWS, &map_rows) ||
        !tensor_map(cols_ptr, cols_extent, K, p.block_cols, &map_cols))
        return fail("gemm_tc: cuTensorMapEncodeTiled failed or is unavailable");

    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return fail("gemm_tc: cannot raise the shared-memory limit: %s", cudaGetErrorString(e));
        cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
        attr_set = true;
    }
    dim3 grid(row_tiles, col_tiles, splits);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attrs[2];
    attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cfg.numAttrs = 1;
    if (p.cluster_splits > 1) {
        attrs[1].id = cudaLaunchAttributeClusterDimension;
        attrs[1].val.clusterDim.x = 1;
        attrs[1].val.clusterDim.y = 1;
        attrs[1].val.clusterDim.z = (unsigned)splits;
        cfg.numAttrs = 2;
    }
    cfg.attrs = attrs;
    cudaLaunchKernelEx(&cfg, gemm_tc_kernel, map_rows, map_cols, p);
    int rc = check_launch("gemm_tc");
    if (rc) return rc;
    if (splits > 1 && p.cluster_splits <= 1 && epilogue != 2 && !sums) {
        const int n_out = epilogue == 3 ? N / 2 : N;
        const size_t total = (size_t)M * n_out;
        const bool by4 = n_out % 4 == 0 && ldc % 4 == 0 && p.accum_ld % 4 == 0 && ((((uintptr_t)p.accum) | ((uintptr_t)out)) & 15) == 0;
        if (by4) {
            const unsigned blocks = (unsigned)((total / 4 + 255) / 256);
            if (epilogue == 3) launch_kernel(gemm_tc_finalize4_kernel<3>, blocks, 256, 0, st, p.accum, p.accum_ld, out, ldc, M, n_out);
            else if (epilogue == 1) launch_kernel(gemm_tc_finalize4_kernel<1>, blocks, 256, 0, st, p.accum, p.accum_ld, out, ldc, M, n_out);
            else launch_kernel(gemm_tc_finalize4_kernel<0>, blocks, 256, 0, st, p.accum, p.accum_ld, out, ldc, M, n_out);
        } else {
            launch_kernel(gemm_tc_finalize_kernel, (unsigned)((total + 255) / 256), 256, 0, st, p.accum, p.accum_ld, out, ldc, M, N, epilogue);
        }
        return check_launch("gemm_tc_finalize");
    }
    return 0;
}

// The fused projection of a layer's attention: [q | k | v] = A . W^T for M > 128 tokens (rotation from the angle
// table cos_sin) or for at most 16 (rotation from the frequencies inv_freq; either may be null), and straight from the
// accumulator every query and key head gets its RMSNorm (weights may be null) and its rotation (cos_sin, the table
// of ember_rope_table with cs_ld tokens a row, may be null), queries go to q_out, keys and values into their cache pages.  Heads are 128 wide.  1 if these sizes are taken.
EMBER_API int ember_gemm_tc_qkv_supported(int M, int N, int K, int n_heads, int n_kv, int head_dim) {
    return M > 0 && (M <= 16 || M > 128) && K > 0 && K % 8 == 0 && head_dim == 128 && n_heads > 0 && n_kv > 0 &&
           N == (n_heads + 2 * n_kv) * 128;
}

// The fused projection of a decode-sized step (at most 16 tokens): 128 weight rows (one head slot) x the tokens per
// tile, the K range split over a thread-block cluster whose blocks share the tokens out and finish whole heads.
static int launch_heads_swapped(const void* A, const void* W, GemmTcParams p, int num_sms, cudaStream_t st) {
    p.swapped = 1;
    p.block_cols = 16;
    const int tiles = p.N / TILE_ROWS;
    int splits = 1;
    if (tiles < num_sms) {
        splits = (num_sms + tiles - 1) / tiles;
        if (splits > 8) splits = 8;
        while (splits > 1 && p.num_k_blocks / splits < 2) splits--;
    }
    p.k_blocks_per_split = (p.num_k_blocks + splits - 1) / splits;
    splits = (p.num_k_blocks + p.k_blocks_per_split - 1) / p.k_blocks_per_split;
    p.cluster_splits = splits;
    p.rows_per = TILE_ROWS;
    p.row_tiles = tiles;
    p.total_tiles = tiles;
    p.tmem_cols = 32;
    p.accum = nullptr; p.accum_ld = 0;
    const int per = (p.block_cols + splits - 1) / splits;
    const size_t recv_bytes = ((size_t)splits * per + 1) * TILE_ROWS * sizeof(float) + 64;     // partial sums, one head, 4 sums
    const int stage_bytes = TILE_ROWS * TILE_K * 2 + ((p.block_cols * TILE_K * 2 + 1023) & ~1023);
    int stages = (int)(((size_t)96 * 1024) / stage_bytes);
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    if (stages > p.k_blocks_per_split) stages = p.k_blocks_per_split < 2 ? 2 : p.k_blocks_per_split;
    p.stages = stages;
    const size_t smem = (size_t)stages * stage_bytes + 1024 + 256 + recv_bytes;
    CUtensorMap map_rows, map_cols;
    if (!tensor_map(W, p.N, p.K, TILE_ROWS, &map_rows) || !tensor_map(A, p.M, p.K, p.block_cols, &map_cols))
        return fail("gemm_tc: cuTensorMapEncodeTiled failed or is unavailable");
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return fail("gemm_tc: cannot raise the shared-memory limit: %s", cudaGetErrorString(e));
        cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
        attr_set = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tiles, 1, splits);
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attrs[2];
    attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    attrs[1].id = cudaLaunchAttributeClusterDimension;
    attrs[1].val.clusterDim.x = 1;
    attrs[1].val.clusterDim.y = 1;
    attrs[1].val.clusterDim.z = (unsigned)splits;
    cfg.attrs = attrs;
    cfg.numAttrs = 2;
    cudaLaunchKernelEx(&cfg, gemm_tc_kernel, map_rows, map_cols, p);
    return check_launch("gemm_tc_heads");
}

EMBER_API int ember_gemm_tc_qkv(const void* A, const void* W, int M, int N, int K, int n_heads, int n_kv,
                                const float* q_norm_w, const float* k_norm_w, float eps, const void* cos_sin, int cs_ld,
                                const float* inv_freq,
                                const int* positions, const int* seq_of, const int* block_table, int max_blocks, int page,
                                int num_pages, void* q_out, void* k_pool, void* v_pool, int write_kv, int num_sms,
                                int split_mode, int* err, void* stream) {
    if (!ember_gemm_tc_qkv_supported(M, N, K, n_heads, n_kv, 128))
        return fail("gemm_tc_qkv: M=%d N=%d K=%d with %d/%d heads of 128 is not taken", M, N, K, n_heads, n_kv);
    if ((((uintptr_t)A) | ((uintptr_t)W) | ((uintptr_t)q_out) | ((uintptr_t)k_pool) | ((uintptr_t)v_pool) | ((uintptr_t)cos_sin) |
         ((uintptr_t)q_norm_w) | ((uintptr_t)k_norm_w)) & 15)
        return fail("gemm_tc_qkv: operands must be 16-byte aligned");
    if (!positions || !seq_of || !block_table || page <= 0 || max_blocks <= 0 || num_pages <= 0)
        return fail("gemm_tc_qkv: bad cache geometry");
    if (num_sms <= 0) num_sms = 148;
    cudaStream_t st = (cudaStream_t)stream;
    GemmTcParams p = {};
    p.M = M; p.N = N; p.K = K;
    p.num_k_blocks = (K + TILE_K - 1) / TILE_K;
    p.epilogue = 4; p.out = nullptr; p.ldc = 0; p.err = err;
    p.rows_per = TILE_ROWS;
    p.qkv.n_heads = n_heads; p.qkv.n_kv = n_kv; p.qkv.q_norm_w = q_norm_w; p.qkv.k_norm_w = k_norm_w; p.qkv.eps = eps;
    if (cos_sin && cs_ld < M) return fail("gemm_tc_qkv: the rotation table has %d columns for %d tokens", cs_ld, M);
    if (M <= 16 ? (cos_sin && !inv_freq) : (inv_freq && !cos_sin))
        return fail("gemm_tc_qkv: %d tokens rotate with %s", M, M <= 16 ? "the frequencies" : "the angle table");
    p.qkv.inv_freq = inv_freq;
    p.qkv.cos_sin = (const float4*)cos_sin; p.qkv.cs_ld = cs_ld; p.qkv.positions = positions; p.qkv.seq_of = seq_of;
    p.qkv.block_table = block_table; p.qkv.max_blocks = max_blocks; p.qkv.page = page; p.qkv.num_pages = num_pages;
    p.qkv.q_out = (__nv_bfloat16*)q_out; p.qkv.k_pool = (__nv_bfloat16*)k_pool; p.qkv.v_pool = (__nv_bfloat16*)v_pool;
    p.qkv.write_kv = write_kv;
    if (M <= 16) return launch_heads_swapped(A, W, p, num_sms, st);
    const int block_cols = (N % 256 == 0) ? 256 : 128;          // whole heads in a tile
    if (split_mode != 5) {
        const int max_pairs = pair_capacity(num_sms);
        if (max_pairs > 0 && (split_mode == 4 || M >= 2048)) return launch_pair(A, W, p, block_cols, max_pairs, st);
    }
    return launch_persistent(A, W, p, block_cols, num_sms, st);
}
