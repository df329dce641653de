// Shared helpers of the sm_100a kernels: error reporting through a C ABI, dtype codes,
// loads that widen to float, warp/block reductions with a fixed order.
//
// Every exported function is `extern "C" int ember_<name>(..., void* stream)`: it
// validates its arguments on the host, launches on the given stream, and returns 0 or a
// non-zero code with a message readable through ember_last_error().  Kernels never trap:
// an index that is out of range is skipped and recorded in a device error word that the
// host can poll.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <utility>

#define EMBER_API extern "C" __attribute__((visibility("default")))

enum EmberDType : int { EMBER_F32 = 0, EMBER_BF16 = 1 };

// Device error word bits (set with atomicOr by kernels, read by the host after a sync).
enum EmberDeviceError : int {
    EMBER_ERR_TOKEN_RANGE = 1,   // a token id outside the vocabulary
    EMBER_ERR_PAGE_RANGE = 2,    // a page id outside the pool
    EMBER_ERR_WAIT_LIMIT = 4,    // a bounded wait on a barrier ran out
};

namespace ember {

inline char* error_buffer() {
    static thread_local char buf[512] = {0};
    return buf;
}

inline int fail(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(error_buffer(), 512, fmt, ap);
    va_end(ap);
    return 1;
}

inline int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail("%s: %s", what, cudaGetErrorString(e));
    return 0;
}

// Programmatic dependent launch.  Every kernel is launched with the stream-serialization attribute,
// so its blocks may start while the kernel before it is still draining; until pdl_wait() returns a
// kernel touches nothing that an earlier kernel writes (it may set up barriers and prefetch weights).
// pdl_wait() returns at once when the launch carried no such dependency.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

inline bool pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("EMBER_PDL");
        on = (e && e[0] == '0') ? 0 : 1;
    }
    return on != 0;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                 Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// ---- bounded waits on shared-memory barriers ------------------------------------------------------------------
// No kernel here waits without a limit.  A wait gives up after EMBER_WAIT_LIMIT_NS of the device's global timer
// (two seconds: far beyond any step, short enough that nobody takes the device for hung), raises the block's
// abort flag so that every role of the block falls through to the common exit (which frees tensor memory and
// records EMBER_ERR_WAIT_LIMIT in the device error word), and returns false.  The limit is time, not a number of
// polls: a suspended try_wait takes an implementation-defined while, so a poll count bounds nothing in seconds.
constexpr unsigned long long EMBER_WAIT_LIMIT_NS = 2000000000ull;

__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ bool mbarrier_try_wait_parity(uint32_t bar_shared, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok) : "r"(bar_shared), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbarrier_test_wait_parity(uint32_t bar_shared, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok) : "r"(bar_shared), "r"(parity) : "memory");
    return ok != 0;
}
// A phase that is already over is seen by one plain look (about 100 cycles; the suspending form costs about 240
// even then).  While waiting, the abort flag and the timer are looked at every 64 polls.
__device__ __forceinline__ bool mbarrier_wait_bounded(uint32_t bar_shared, uint32_t parity, volatile int* abort_flag,
                                                      unsigned long long limit_ns = EMBER_WAIT_LIMIT_NS) {
    if (mbarrier_test_wait_parity(bar_shared, parity)) return true;
    unsigned long long start = 0;
    for (unsigned i = 0;; i++) {
        if (mbarrier_try_wait_parity(bar_shared, parity)) return true;
        if ((i & 63u) == 63u) {
            if (*abort_flag) return false;
            const unsigned long long now = global_timer_ns();
            if (start == 0) start = now;
            else if (now - start > limit_ns) break;
        }
    }
    *abort_flag = 1;
    return false;
}

__device__ __forceinline__ float to_float(float x) { return x; }
__device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T>
__device__ __forceinline__ T from_float(float x);
template <>
__device__ __forceinline__ float from_float<float>(float x) { return x; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; the order of additions is fixed by the
// thread layout, so the result does not depend on anything but the inputs.
__device__ __forceinline__ float block_sum(float v, float* scratch /* >= 32 floats */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    const int nwarps = (blockDim.x + 31) >> 5;
    float r = (lane < nwarps) ? scratch[lane] : 0.0f;
    r = warp_sum(r);
    return r;
}

}  // namespace ember

// Each shared library exports its own copy of the message reader.
#define EMBER_DEFINE_LAST_ERROR \
    EMBER_API const char* ember_last_error() { return ember::error_buffer(); }
