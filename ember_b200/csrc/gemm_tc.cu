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

}  // namespace ember

using namespace ember;

// Whether the tensor-core product takes these sizes (bf16 operands are the caller's business).
EMBER_API int ember_gemm_tc_supported(int M, int N, int K, int epilogue) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if (K % 8) return 0;                       // TMA needs 16-byte row pitch
    if (epilogue == 3 && (N & 1)) return 0;
    return 1;
}

// How many floats of zeroed scratch a call may need (0 if none).
EMBER_API long long ember_gemm_tc_scratch_floats(int max_tokens_swapped, int N) {
    return (long long)max_tokens_swapped * N;
}

// C = A . W^T with the fused epilogue.  `scratch` is a zero-filled fp32 buffer of at least
// min(M, 128) * N floats (used only when the K range is split; it is left zeroed).
EMBER_API int ember_gemm_tc(const void* A, const void* W, void* out, int ldc, int M, int N, int K, int epilogue,
                            float* scratch, long long scratch_floats, int num_sms, int split_mode, int* err, void* stream) {
    if (M <= 0 || N <= 0) return 0;
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
        p.block_cols = N >= 1024 ? 256 : 128;
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
    const bool use_cluster = split_mode == 2 || (split_mode == 0 && p.block_cols <= 16 && store_epilogue);
    int splits = 1;
    if (p.swapped && use_cluster) {
        // fill the SMs once: clusters of up to 8 blocks, at least 2 k-blocks each
        if (tiles < num_sms) {
            splits = (num_sms + tiles - 1) / tiles;
            if (splits > 8) splits = 8;
            while (splits > 1 && p.num_k_blocks / splits < 2) splits--;
        }
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
    // Prefill-sized products run as persistent blocks with two accumulators in tensor memory.
    const bool persistent = !p.swapped && split_mode != 3;
    p.row_tiles = row_tiles;
    p.total_tiles = row_tiles * col_tiles;
    int tc = 32;
    while (tc < p.block_cols * (persistent ? 2 : 1)) tc <<= 1;
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
    if (persistent) {
        static bool pattr = false;
        if (!pattr) {
            cudaError_t e = cudaFuncSetAttribute(gemm_tc_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
            if (e != cudaSuccess) return fail("gemm_tc: cannot raise the shared-memory limit: %s", cudaGetErrorString(e));
            pattr = true;
        }
        const int blocks = p.total_tiles < num_sms ? p.total_tiles : num_sms;
        launch_kernel(gemm_tc_persistent_kernel, dim3(blocks), dim3(GEMM_THREADS), smem, st, map_rows, map_cols, p);
        return check_launch("gemm_tc_persistent");
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
    if (splits > 1 && p.cluster_splits <= 1 && epilogue != 2) {
        const size_t total = (size_t)M * (epilogue == 3 ? N / 2 : N);
        launch_kernel(gemm_tc_finalize_kernel, (unsigned)((total + 255) / 256), 256, 0, st, p.accum, p.accum_ld, out, ldc, M, N, epilogue);
        return check_launch("gemm_tc_finalize");
    }
    return 0;
}
