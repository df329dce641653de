// The allocation-free variant of the small-M tcgen05 matrix product (declared in no_alloc.h, which
// says who it is for).  It has no counterpart in the reference engine.
//
// Same device kernel as ember_gemm_tc (gemm_tc_kernel.cuh); the only difference is where the
// split-K scratch lives: in the file-scope device array below instead of a buffer the caller
// allocates.  Host code must not pass `noalloc_scratch` itself to a kernel: on the host that
// name is a stand-in, not a device address.  The address is looked up once per device with
// cudaGetSymbolAddress while that device is current, and that pointer is what the kernels get.
#include "gemm_tc_kernel.cuh"
#include "no_alloc.h"

EMBER_DEFINE_LAST_ERROR

static_assert(EMBER_NOALLOC_SCRATCH_FLOATS == (1 << 20), "the header and the array must agree");
static __device__ __align__(256) float noalloc_scratch[EMBER_NOALLOC_SCRATCH_FLOATS];

namespace {

constexpr int MAX_DEVICES = 64;
float* scratch_of_device[MAX_DEVICES] = {nullptr};
std::mutex setup_mutex;

// Device address of the scratch array on the current device (first call per device: set-up).
int scratch_pointer(float** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return ember::fail("gemm_tc_noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= MAX_DEVICES) return ember::fail("gemm_tc_noalloc: device index %d is out of range", dev);
    std::lock_guard<std::mutex> lock(setup_mutex);
    if (!scratch_of_device[dev]) {
        float* ptr = nullptr;
        e = cudaGetSymbolAddress((void**)&ptr, noalloc_scratch);
        if (e != cudaSuccess || !ptr)
            return ember::fail("gemm_tc_noalloc: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
        e = cudaFuncSetAttribute(ember::gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess)
            return ember::fail("gemm_tc_noalloc: cannot raise the shared-memory limit: %s", cudaGetErrorString(e));
        scratch_of_device[dev] = ptr;
    }
    *out = scratch_of_device[dev];
    return 0;
}

// One tensor map, encoded on the stack (no cache, no heap).
bool encode_map(const void* ptr, int rows, int K, int box_rows, CUtensorMap* out) {
    ember::EncodeTiledFn fn = ember::encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {(cuuint32_t)ember::TILE_K, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    return fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

using namespace ember;

EMBER_API int ember_gemm_tc_noalloc(const void* A, const void* W, void* out, int ldc, int M, int N, int K, int epilogue,
                                    int* err, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > TILE_ROWS) return fail("gemm_tc_noalloc: M=%d; this entry point takes up to %d rows", M, TILE_ROWS);
    if (K <= 0 || K % 8) return fail("gemm_tc_noalloc: K=%d must be a positive multiple of 8", K);
    if (epilogue < 0 || epilogue > 3) return fail("gemm_tc_noalloc: unknown epilogue %d", epilogue);
    if (epilogue == 3 && (N & 1)) return fail("gemm_tc_noalloc: the gated epilogue needs an even N, got %d", N);
    if ((long long)M * N > (long long)EMBER_NOALLOC_SCRATCH_FLOATS)
        return fail("gemm_tc_noalloc: M*N = %lld exceeds the built-in scratch of %d floats", (long long)M * N,
                    EMBER_NOALLOC_SCRATCH_FLOATS);
    if (A == nullptr || W == nullptr || out == nullptr) return fail("gemm_tc_noalloc: A, W and out must not be null");
    if ((((uintptr_t)A) & 15) || (((uintptr_t)W) & 15)) return fail("gemm_tc_noalloc: operands must be 16-byte aligned");
    const int out_width = epilogue == 3 ? N / 2 : N;
    if (ldc < out_width)
        return fail("gemm_tc_noalloc: ldc=%d is shorter than the %d values a row of the output holds", ldc, out_width);
    float* scratch = nullptr;
    if (int rc = scratch_pointer(&scratch)) return rc;
    cudaStream_t st = (cudaStream_t)stream;

    int num_sms = 148, dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);

    GemmTcParams p;
    p.M = M; p.N = N; p.K = K;
    p.swapped = 1;
    p.num_k_blocks = (K + TILE_K - 1) / TILE_K;
    p.block_cols = ((M + 15) / 16) * 16;
    const int row_tiles = (N + TILE_ROWS - 1) / TILE_ROWS;
    int splits = 1;
    if (row_tiles < num_sms) {
        const int by_sms = (num_sms + row_tiles - 1) / row_tiles;
        const int by_k = p.num_k_blocks / 4 > 0 ? p.num_k_blocks / 4 : 1;
        splits = by_sms < by_k ? by_sms : by_k;
        if (splits > 16) splits = 16;
        if (splits < 1) splits = 1;
    }
    p.k_blocks_per_split = (p.num_k_blocks + splits - 1) / splits;
    splits = (p.num_k_blocks + p.k_blocks_per_split - 1) / p.k_blocks_per_split;
    p.epilogue = epilogue; p.out = out; p.ldc = ldc; p.err = err;
    p.accum = nullptr; p.accum_ld = 0;
    p.row_tiles = 0; p.total_tiles = 0;
    p.cluster_splits = 1; p.rows_per = TILE_ROWS;      // this variant sums its K splits with atomics into the scratch
    if (splits > 1) {
        if (epilogue == 2) {
            p.accum = (float*)out;
            p.accum_ld = ldc;
        } else {
            // the array keeps the last call's contents: clear what this call adds into
            cudaError_t e = cudaMemsetAsync(scratch, 0, (size_t)M * N * sizeof(float), st);
            if (e != cudaSuccess) return fail("gemm_tc_noalloc: clearing the scratch: %s", cudaGetErrorString(e));
            p.accum = scratch;
            p.accum_ld = N;
        }
    }
    int tc = 32;
    while (tc < p.block_cols) tc <<= 1;
    p.tmem_cols = tc;
    const int rows_bytes = TILE_ROWS * TILE_K * 2;
    const int cols_bytes = p.block_cols * TILE_K * 2;
    const int stage_bytes = rows_bytes + ((cols_bytes + 1023) & ~1023);
    int stages = (200 * 1024) / stage_bytes;
    if (stages > MAX_STAGES) stages = MAX_STAGES;
    if (stages > p.k_blocks_per_split) stages = p.k_blocks_per_split < 2 ? 2 : p.k_blocks_per_split;
    p.stages = stages;
    const size_t smem = (size_t)stages * stage_bytes + 1024 + 256;

    CUtensorMap map_rows, map_cols;
    if (!encode_map(W, N, K, TILE_ROWS, &map_rows) || !encode_map(A, M, K, p.block_cols, &map_cols))
        return fail("gemm_tc_noalloc: cuTensorMapEncodeTiled failed or is unavailable");

    dim3 grid(row_tiles, 1, splits);
    gemm_tc_kernel<<<grid, GEMM_THREADS, smem, st>>>(map_rows, map_cols, p);
    if (int rc = check_launch("gemm_tc_noalloc")) return rc;
    if (splits > 1 && epilogue != 2) {
        const size_t total = (size_t)M * (epilogue == 3 ? N / 2 : N);
        gemm_tc_finalize_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(p.accum, p.accum_ld, out, ldc, M, N, epilogue);
        return check_launch("gemm_tc_noalloc_finalize");
    }
    return 0;
}
