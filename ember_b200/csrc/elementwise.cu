// Embedding gather, RMSNorm, and the fused per-head norm + rotation + cache write.
//
// Reference formulas: src/backend/cpu/cpu_backend.cpp:34-39 (RMSNorm), :131-135 (embedding),
// :156-172 (q/k norm, rotation, cache write), :263-272 (rotate-half).  The reference's own CUDA
// counterparts are src/backend/cuda/k_elementwise.cu:45-126; these kernels are written for
// sm_100a from the formulas and differ in layout: any head size up to 256 (even), partial
// rotation, bf16 or fp32 activations and cache, pages of any size.
#include "common.cuh"

EMBER_DEFINE_LAST_ERROR

namespace ember {

// ------------------------------------------------------------------------------ embedding
// h[t, :] = scale * float(table[tokens[t], :]) (scale 1 for the reference's model: no scaling).  A negative token -(r + 1) stands for the id that the
// sampler left in prev_ids[r]: a step can be launched before the host has read the step before it.
template <typename TW>
__global__ void embed_kernel(const int* __restrict__ tokens, const int* __restrict__ prev_ids, int n_prev,
                             const TW* __restrict__ table, float* __restrict__ out, int H, int V, float scale,
                             int* __restrict__ err) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    int tok = tokens[t];
    if (tok < 0 && prev_ids != nullptr && -tok <= n_prev) tok = prev_ids[-tok - 1];
    float* o = out + (size_t)t * H;
    if (tok < 0 || tok >= V) {
        if (threadIdx.x == 0 && err) atomicOr(err, EMBER_ERR_TOKEN_RANGE);
        for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = 0.0f;
        return;
    }
    const TW* row = table + (size_t)tok * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = scale * to_float(row[i]);
}

// -------------------------------------------------------------------------------- RMSNorm
// out[r, i] = w[i] * (x[row(r), i] * (1 / sqrt(mean(x^2) + eps))), statistics in fp32.
// `rows` (nullable) gathers input rows: the final norm runs only on the rows whose logits
// are wanted.
template <typename TO>
__device__ __forceinline__ void store4(TO* dst, float a, float b, float c, float d);
template <>
__device__ __forceinline__ void store4<float>(float* dst, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(dst) = make_float4(a, b, c, d);
}
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* dst, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&lo);
    u.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(dst) = u;
}

constexpr int NORM_THREADS = 256;
constexpr int NORM_MAX_VEC = 8;  // float4 per thread kept in registers: rows up to 256 * 8 * 4 = 8192 wide

// Rows whose width is a multiple of 4 and at most 8192 are read once, 16 bytes at a time, and kept in
// registers between the reduction and the scaling (NORM_VEC float4 per thread: the smallest of 1, 2, 4, 8 that
// covers the row, so that a narrow row does not pay for the registers of a wide one); other widths take the
// two-pass scalar path (NORM_VEC = 0).
template <typename TO, int NORM_VEC>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_kernel(const float* __restrict__ x, const int* __restrict__ rows,
               const float* __restrict__ w, float eps, TO* __restrict__ out, int H) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const float* in = x + (size_t)(rows ? rows[r] : r) * H;
    TO* o = out + (size_t)r * H;
    const int nvec = H >> 2;
    if constexpr (NORM_VEC > 0) {
        float4 v[NORM_VEC];
        float ss = 0.0f;
#pragma unroll
        for (int i = 0; i < NORM_VEC; i++) {
            const int idx = threadIdx.x + i * NORM_THREADS;
            if (idx < nvec) {
                v[i] = reinterpret_cast<const float4*>(in)[idx];
                ss = fmaf(v[i].x, v[i].x, fmaf(v[i].y, v[i].y, fmaf(v[i].z, v[i].z, fmaf(v[i].w, v[i].w, ss))));
            }
        }
        ss = block_sum(ss, scratch);
        const float scale = 1.0f / sqrtf(ss / (float)H + eps);
#pragma unroll
        for (int i = 0; i < NORM_VEC; i++) {
            const int idx = threadIdx.x + i * NORM_THREADS;
            if (idx < nvec) {
                const float4 g = reinterpret_cast<const float4*>(w)[idx];
                store4<TO>(o + 4 * idx, g.x * (v[i].x * scale), g.y * (v[i].y * scale), g.z * (v[i].z * scale), g.w * (v[i].w * scale));
            }
        }
        return;
    }
    float ss = 0.0f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = in[i];
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = from_float<TO>(w[i] * (in[i] * scale));
}

// ------------------------------------------------- per-head norm + rotation + cache write
// One warp per (token, head slot); slots are the query heads, then the key heads, then the
// value heads of the fused projection row [q | k | v].
//   q, k: optional RMSNorm over the head (weight shared by all heads), then rotate-half over
//         the first `rotary` elements with angle = float(pos) * inv_freq[i] in fp32.
//   q -> q_out[t, head, :];  k, v -> page bt[seq][pos / page], slot pos % page of the pools,
//   layout [page][kv_head][slot][D].
template <typename T>
__device__ __forceinline__ float2 load2(const T* p);
template <>
__device__ __forceinline__ float2 load2<float>(const float* p) { return *reinterpret_cast<const float2*>(p); }
template <>
__device__ __forceinline__ float2 load2<__nv_bfloat16>(const __nv_bfloat16* p) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}
template <typename T>
__device__ __forceinline__ void store2(T* p, float a, float b);
template <>
__device__ __forceinline__ void store2<float>(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
template <>
__device__ __forceinline__ void store2<__nv_bfloat16>(__nv_bfloat16* p, float a, float b) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}

// One block per token.  The sines and cosines of the token's position are computed once and shared
// by all heads; then each warp takes head slots in turn (element pairs are loaded and stored together).
template <typename T>
__global__ void qk_norm_rope_store_kernel(
    const T* __restrict__ qkv, int ld, int n_heads, int n_kv, int D,
    const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w, float eps,
    const float* __restrict__ inv_freq, int rotary,
    const int* __restrict__ positions, const int* __restrict__ seq_of,
    const int* __restrict__ block_table, int max_blocks, int page, int num_pages,
    T* __restrict__ q_out, T* __restrict__ k_pool, T* __restrict__ v_pool, int write_kv,
    int* __restrict__ err) {
    extern __shared__ float smem[];
    pdl_launch_dependents();
    pdl_wait();
    const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int slots = n_heads + 2 * n_kv;
    const int half = (inv_freq && rotary > 0) ? rotary >> 1 : 0;
    float* cs = smem;                 // [half]
    float* sn = cs + half;            // [half]
    float* bufs = sn + half;          // [warps][D]
    const int pos = positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf((float)pos * inv_freq[i], &sn[i], &cs[i]);
    __syncthreads();

    int blk = -1;
    if (write_kv) {
        blk = block_table[(size_t)seq_of[t] * max_blocks + pos / page];
        if (blk < 0 || blk >= num_pages) {
            if (threadIdx.x == 0 && err) atomicOr(err, EMBER_ERR_PAGE_RANGE);
            blk = -1;
        }
    }
    float* s = bufs + (size_t)warp * D;
    // blockIdx.y splits the head slots between blocks when a step has few tokens
    for (int slot = blockIdx.y * warps + warp; slot < slots; slot += warps * gridDim.y) {
        const int kind = slot < n_heads ? 0 : (slot < n_heads + n_kv ? 1 : 2);  // q, k, v
        if (kind != 0 && (!write_kv || blk < 0)) continue;
        const T* src = qkv + (size_t)t * ld + (size_t)slot * D;
        float ss = 0.0f;
        for (int i = 2 * lane; i < D; i += 64) {
            const float2 v = load2<T>(src + i);
            s[i] = v.x;
            s[i + 1] = v.y;
            ss = fmaf(v.x, v.x, fmaf(v.y, v.y, ss));
        }
        const float* nw = kind == 0 ? q_norm_w : (kind == 1 ? k_norm_w : nullptr);
        if (nw) {
            ss = warp_sum(ss);
            const float scale = 1.0f / sqrtf(ss / (float)D + eps);
            for (int i = 2 * lane; i < D; i += 64) {
                s[i] = nw[i] * (s[i] * scale);
                s[i + 1] = nw[i + 1] * (s[i + 1] * scale);
            }
        }
        __syncwarp();
        if (kind != 2 && half > 0) {
            for (int i = lane; i < half; i += 32) {
                const float a = s[i], b = s[i + half];
                s[i] = a * cs[i] - b * sn[i];
                s[i + half] = b * cs[i] + a * sn[i];
            }
            __syncwarp();
        }
        T* dst;
        if (kind == 0) {
            dst = q_out + ((size_t)t * n_heads + slot) * D;
        } else {
            const int kvh = kind == 1 ? slot - n_heads : slot - n_heads - n_kv;
            dst = (kind == 1 ? k_pool : v_pool) + (((size_t)blk * n_kv + kvh) * page + (pos % page)) * D;
        }
        for (int i = 2 * lane; i < D; i += 64) store2<T>(dst + i, s[i], s[i + 1]);
        __syncwarp();
    }
}

// Head size 128 with the whole head rotated (or no rotation): half a warp holds a head in registers, eight
// consecutive elements per lane, loaded and stored 16 (bf16) or 2 x 16 (fp32) bytes at a time; a warp works on
// two heads at once.  The rotation partner of element i is i +- 64, eight lanes away, and comes by shuffle.  The
// token's 64 sines and cosines are computed once per block.  Every lane runs every shuffle (heads that are not
// wanted are computed on zeros and not stored), so heads of different kinds may share a warp.
template <typename T>
__device__ __forceinline__ void load8(const T* p, float* x);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float* x) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float* x) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
        x[2 * i] = f.x;
        x[2 * i + 1] = f.y;
    }
}
template <typename T>
__device__ __forceinline__ void store8(T* p, const float* x);
template <>
__device__ __forceinline__ void store8<float>(float* p, const float* x) {
    reinterpret_cast<float4*>(p)[0] = make_float4(x[0], x[1], x[2], x[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(x[4], x[5], x[6], x[7]);
}
template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float* x) {
    uint4 u;
    __nv_bfloat162 h0 = __floats2bfloat162_rn(x[0], x[1]), h1 = __floats2bfloat162_rn(x[2], x[3]);
    __nv_bfloat162 h2 = __floats2bfloat162_rn(x[4], x[5]), h3 = __floats2bfloat162_rn(x[6], x[7]);
    u.x = *reinterpret_cast<uint32_t*>(&h0); u.y = *reinterpret_cast<uint32_t*>(&h1);
    u.z = *reinterpret_cast<uint32_t*>(&h2); u.w = *reinterpret_cast<uint32_t*>(&h3);
    *reinterpret_cast<uint4*>(p) = u;
}

constexpr int ROPE128_WARPS = 4;

// TI: what the projection is read as; T: queries and cache.  CLEAR (TI float only): the rows are the fp32 sums a
// product with a cut K range left in its zeroed scratch; every element is read once and set back to zero here,
// which stands in for that product's own pass that would round the sums, store them and clear the scratch.
template <typename TI, typename T, bool CLEAR>
__global__ void __launch_bounds__(ROPE128_WARPS * 32)
qk_norm_rope_store_d128_kernel(
    TI* __restrict__ qkv, int ld, int n_heads, int n_kv,
    const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w, float eps,
    const float* __restrict__ inv_freq, int rotate,
    const int* __restrict__ positions, const int* __restrict__ seq_of,
    const int* __restrict__ block_table, int max_blocks, int page, int num_pages,
    T* __restrict__ q_out, T* __restrict__ k_pool, T* __restrict__ v_pool, int write_kv,
    int* __restrict__ err) {
    constexpr int D = 128;
    __shared__ __align__(16) float cs_s[64];
    __shared__ __align__(16) float sn_s[64];
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int slots = n_heads + 2 * n_kv;
    const int pos = positions[t];
    if (rotate && threadIdx.x < 64) sincosf((float)pos * inv_freq[threadIdx.x], &sn_s[threadIdx.x], &cs_s[threadIdx.x]);
    int blk = -1;
    if (write_kv) {
        blk = block_table[(size_t)seq_of[t] * max_blocks + pos / page];
        if (blk < 0 || blk >= num_pages) {
            if (threadIdx.x == 0 && err) atomicOr(err, EMBER_ERR_PAGE_RANGE);
            blk = -1;
        }
    }
    __syncthreads();
    const int hl = lane & 15;                      // lane within the half-warp that holds one head
    const int e0 = 8 * hl;                         // this lane's elements e0 .. e0 + 7
    const bool upper = hl >= 8;                    // elements 64..127: rotated as b * cos + a * sin
    float cs[8], sn[8];
    if (rotate) {
        const int r0 = e0 & 63;
#pragma unroll
        for (int j = 0; j < 8; j += 4) {
            const float4 c = *reinterpret_cast<const float4*>(&cs_s[r0 + j]), sv = *reinterpret_cast<const float4*>(&sn_s[r0 + j]);
            cs[j] = c.x; cs[j + 1] = c.y; cs[j + 2] = c.z; cs[j + 3] = c.w;
            sn[j] = sv.x; sn[j + 1] = sv.y; sn[j + 2] = sv.z; sn[j + 3] = sv.w;
        }
    }
    // where this token's keys and values go: page blk, place pos % page (per key head: + kvh * page * D)
    const size_t kv_base = blk >= 0 ? ((size_t)blk * n_kv * page + (size_t)(pos % page)) * D + e0 : 0;
    const size_t kv_head = (size_t)page * D;
    TI* src_row = qkv + (size_t)t * ld + e0;
    T* q_row = q_out + (size_t)t * n_heads * D + e0;
    const bool kv_ok = write_kv && blk >= 0;
    // a warp takes two heads per turn; blockIdx.y splits the heads between blocks when a step has few tokens
    for (int slot = 2 * (blockIdx.y * ROPE128_WARPS + warp) + (lane >> 4); slot < slots + 1;
         slot += 2 * ROPE128_WARPS * gridDim.y) {
        const int kind = slot < n_heads ? 0 : (slot < n_heads + n_kv ? 1 : 2);  // q, k, v
        const bool act = slot < slots && (kind == 0 || kv_ok);
        float x[8];
        if (act || (CLEAR && slot < slots)) {
            load8<TI>(src_row + (size_t)slot * D, x);
            if constexpr (CLEAR) {              // (the only instance that writes to its input)
                const float zero[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
                store8<TI>(src_row + (size_t)slot * D, zero);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; j++) x[j] = 0.0f;
        }
        const int first = slot - (lane >> 4);       // the warp's lower head: values only from n_heads + n_kv on
        if (first < n_heads + n_kv) {               // uniform over the warp
            float ss = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; j++) ss = fmaf(x[j], x[j], ss);
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);     // within the half-warp
            const float* nw = kind == 0 ? q_norm_w : (kind == 1 ? k_norm_w : nullptr);
            if (nw && act) {
                const float scale = 1.0f / sqrtf(ss / (float)D + eps);
                const float4 g0 = *reinterpret_cast<const float4*>(nw + e0), g1 = *reinterpret_cast<const float4*>(nw + e0 + 4);
                x[0] = g0.x * (x[0] * scale); x[1] = g0.y * (x[1] * scale); x[2] = g0.z * (x[2] * scale); x[3] = g0.w * (x[3] * scale);
                x[4] = g1.x * (x[4] * scale); x[5] = g1.y * (x[5] * scale); x[6] = g1.z * (x[6] * scale); x[7] = g1.w * (x[7] * scale);
            }
            if (rotate) {
                const bool turn = kind != 2;
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const float other = __shfl_xor_sync(0xffffffffu, x[j], 8);
                    // lower half: a * cos - b * sin (a own, b partner); upper half: b * cos + a * sin (b own, a partner)
                    const float r = upper ? x[j] * cs[j] + other * sn[j] : x[j] * cs[j] - other * sn[j];
                    x[j] = turn ? r : x[j];
                }
            }
        }
        if (!act) continue;
        T* dst;
        if (kind == 0) {
            dst = q_row + (size_t)slot * D;
        } else {
            const int kvh = kind == 1 ? slot - n_heads : slot - n_heads - n_kv;
            dst = (kind == 1 ? k_pool : v_pool) + kv_base + (size_t)kvh * kv_head;
        }
        store8<T>(dst, x);
    }
}

// The angles of a step's tokens, made once per step for the products that rotate in their epilogue (the same fp32
// expression as the kernels above): out[i / 2][t] = (cos_i, cos_i+1, sin_i, sin_i+1) of float(position[t]) * inv_freq for
// frequencies i and i + 1, rows `ld` tokens long.  Token-minor, so that threads that hold neighbouring tokens read neighbouring
// 16 bytes.
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq, int T, int half,
                                  int ld, float4* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait();
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    const int pairs = half / 2;
    if (idx >= T * pairs) return;
    const int j = idx / T, t = idx - j * T;
    const float pos = (float)positions[t];
    float s0, c0, s1, c1;
    sincosf(pos * inv_freq[2 * j], &s0, &c0);
    sincosf(pos * inv_freq[2 * j + 1], &s1, &c1);
    out[(size_t)j * ld + t] = make_float4(c0, c1, s0, s1);
}

// out[m, j] = silu(x[m, 2j]) * x[m, 2j+1] for an unfused gate/up product (interleaved rows).
template <typename T>
__global__ void silu_mul_interleaved_kernel(const T* __restrict__ x, T* __restrict__ out, size_t n_out) {
    pdl_launch_dependents();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_out) return;
    const float g = to_float(x[2 * i]), u = to_float(x[2 * i + 1]);
    out[i] = from_float<T>(g / (1.0f + expf(-g)) * u);
}

// ------------------------------------------------------------------------- the bounded wait, run out on purpose
// One thread waits, with the helper every TMA/tcgen05 kernel here uses, on a barrier that nothing ever arrives
// at.  The wait has to give up after `limit_ns`, the kernel has to return, and the error word has to hold
// EMBER_ERR_WAIT_LIMIT: what a test checks without any kernel hanging or faulting.
__global__ void wait_limit_probe_kernel(unsigned long long limit_ns, int* __restrict__ err,
                                        unsigned long long* __restrict__ waited_ns) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"((uint32_t)__cvta_generic_to_shared(&bar)), "r"(1) : "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned long long t0 = global_timer_ns();
        const bool ok = mbarrier_wait_bounded((uint32_t)__cvta_generic_to_shared(&bar), 0, &abort_flag, limit_ns);
        if (waited_ns) *waited_ns = global_timer_ns() - t0;
        if (!ok && abort_flag && err) atomicOr(err, EMBER_ERR_WAIT_LIMIT);
    }
}

}  // namespace ember

using namespace ember;

EMBER_API int ember_wait_limit_probe(unsigned long long limit_ns, int* err, unsigned long long* waited_ns, void* stream) {
    if (limit_ns == 0 || limit_ns > 100000000ull) return fail("wait_limit_probe: the limit must be between 1 ns and 100 ms");
    wait_limit_probe_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(limit_ns, err, waited_ns);
    return check_launch("wait_limit_probe");
}

EMBER_API int ember_embed(const int* tokens, const int* prev_ids, int n_prev, const void* table, int table_dtype,
                          float* out, int T, int H, int V, float scale, int* err, void* stream) {
    if (T <= 0) return 0;
    if (H <= 0 || V <= 0) return fail("embed: bad sizes H=%d V=%d", H, V);
    cudaStream_t st = (cudaStream_t)stream;
    const int threads = H >= 1024 ? 256 : 128;
    if (table_dtype == EMBER_F32)
        launch_kernel(embed_kernel<float>, T, threads, 0, st, tokens, prev_ids, n_prev, (const float*)table, out, H, V, scale, err);
    else if (table_dtype == EMBER_BF16)
        launch_kernel(embed_kernel<__nv_bfloat16>, T, threads, 0, st, tokens, prev_ids, n_prev, (const __nv_bfloat16*)table, out, H, V,
                      scale, err);
    else
        return fail("embed: unsupported table dtype %d", table_dtype);
    return check_launch("embed");
}

EMBER_API int ember_rmsnorm(const float* x, const int* rows, const float* w, float eps, void* out, int out_dtype,
                            int n_rows, int H, void* stream) {
    if (n_rows <= 0) return 0;
    if (H <= 0) return fail("rmsnorm: bad width %d", H);
    cudaStream_t st = (cudaStream_t)stream;
    if ((((uintptr_t)x) | ((uintptr_t)w) | ((uintptr_t)out)) & 15) return fail("rmsnorm: buffers must be 16-byte aligned");
    const int threads = NORM_THREADS;
    const int nvec = H >> 2;
    int vec = 0;
    if ((H & 3) == 0 && nvec <= NORM_THREADS * NORM_MAX_VEC)
        vec = nvec <= NORM_THREADS ? 1 : (nvec <= 2 * NORM_THREADS ? 2 : (nvec <= 4 * NORM_THREADS ? 4 : 8));
    if (out_dtype != EMBER_F32 && out_dtype != EMBER_BF16) return fail("rmsnorm: unsupported output dtype %d", out_dtype);
#define EMBER_NORM_LAUNCH(TO, V) \
    launch_kernel(rmsnorm_kernel<TO, V>, n_rows, threads, 0, st, x, rows, w, eps, (TO*)out, H)
#define EMBER_NORM_DISPATCH(TO)                                             \
    switch (vec) {                                                          \
        case 1: EMBER_NORM_LAUNCH(TO, 1); break;                            \
        case 2: EMBER_NORM_LAUNCH(TO, 2); break;                            \
        case 4: EMBER_NORM_LAUNCH(TO, 4); break;                            \
        case 8: EMBER_NORM_LAUNCH(TO, 8); break;                            \
        default: EMBER_NORM_LAUNCH(TO, 0); break;                           \
    }
    if (out_dtype == EMBER_F32) { EMBER_NORM_DISPATCH(float) } else { EMBER_NORM_DISPATCH(__nv_bfloat16) }
#undef EMBER_NORM_DISPATCH
#undef EMBER_NORM_LAUNCH
    return check_launch("rmsnorm");
}

EMBER_API int ember_qk_norm_rope_store(const void* qkv, int dtype, int T, int ld, int n_heads, int n_kv, int D,
                                       const float* q_norm_w, const float* k_norm_w, float eps,
                                       const float* inv_freq, int rotary, const int* positions, const int* seq_of,
                                       const int* block_table, int max_blocks, int page, int num_pages,
                                       void* q_out, void* k_pool, void* v_pool, int write_kv, int* err,
                                       void* stream) {
    if (T <= 0) return 0;
    if (D <= 0 || D > 256 || (D & 1)) return fail("qk_norm_rope_store: head size %d is not an even number up to 256", D);
    if (rotary < 0 || rotary > D || (rotary & 1)) return fail("qk_norm_rope_store: rotary size %d does not fit head size %d", rotary, D);
    if (n_heads <= 0 || n_kv <= 0) return fail("qk_norm_rope_store: bad head counts %d/%d", n_heads, n_kv);
    if (ld < (n_heads + 2 * n_kv) * D) return fail("qk_norm_rope_store: row stride %d is too small", ld);
    if (page <= 0 || max_blocks <= 0 || num_pages <= 0) return fail("qk_norm_rope_store: bad cache geometry");
    cudaStream_t st = (cudaStream_t)stream;
    const int slots = n_heads + 2 * n_kv;
    const int warps = slots < 8 ? slots : 8;
    int ny = (296 + T - 1) / T;                       // enough blocks for a decode step of a few tokens
    const int ny_max = (slots + warps - 1) / warps;
    if (ny > ny_max) ny = ny_max;
    if (ny < 1) ny = 1;
    dim3 grid(T, ny);
    const size_t smem = ((size_t)warps * D + (size_t)(inv_freq ? rotary : 0)) * sizeof(float);
    if (ld & 1) return fail("qk_norm_rope_store: the row stride %d must be even", ld);
    const bool rotate = inv_freq != nullptr && rotary > 0;
    const bool aligned = (ld % 8) == 0 && (((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)k_pool | (uintptr_t)v_pool |
                                            (uintptr_t)q_norm_w | (uintptr_t)k_norm_w) & 15) == 0;
    if (D == 128 && (!rotate || rotary == 128) && aligned && (dtype == EMBER_F32 || dtype == EMBER_BF16)) {
        int gy = (592 + T - 1) / T;                       // a decode step of a few tokens still fills the SMs
        const int gy_max = (slots + 2 * ROPE128_WARPS - 1) / (2 * ROPE128_WARPS);
        if (gy > gy_max) gy = gy_max;
        if (gy < 1) gy = 1;
        dim3 g128(T, gy);
        if (dtype == EMBER_F32)
            launch_kernel(qk_norm_rope_store_d128_kernel<float, float, false>, g128, ROPE128_WARPS * 32, 0, st,
                (float*)const_cast<void*>(qkv), ld, n_heads, n_kv, q_norm_w, k_norm_w, eps, inv_freq, rotate ? 1 : 0, positions, seq_of,
                block_table, max_blocks, page, num_pages, (float*)q_out, (float*)k_pool, (float*)v_pool, write_kv, err);
        else
            launch_kernel(qk_norm_rope_store_d128_kernel<__nv_bfloat16, __nv_bfloat16, false>, g128, ROPE128_WARPS * 32, 0, st,
                (__nv_bfloat16*)const_cast<void*>(qkv), ld, n_heads, n_kv, q_norm_w, k_norm_w, eps, inv_freq, rotate ? 1 : 0, positions,
                seq_of, block_table, max_blocks, page, num_pages, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool,
                (__nv_bfloat16*)v_pool, write_kv, err);
        return check_launch("qk_norm_rope_store");
    }
    if (dtype == EMBER_F32)
        launch_kernel(qk_norm_rope_store_kernel<float>, grid, warps * 32, smem, st,
            (const float*)qkv, ld, n_heads, n_kv, D, q_norm_w, k_norm_w, eps, inv_freq, rotary, positions, seq_of,
            block_table, max_blocks, page, num_pages, (float*)q_out, (float*)k_pool, (float*)v_pool, write_kv, err);
    else if (dtype == EMBER_BF16)
        launch_kernel(qk_norm_rope_store_kernel<__nv_bfloat16>, grid, warps * 32, smem, st,
            (const __nv_bfloat16*)qkv, ld, n_heads, n_kv, D, q_norm_w, k_norm_w, eps, inv_freq, rotary, positions,
            seq_of, block_table, max_blocks, page, num_pages, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool,
            (__nv_bfloat16*)v_pool, write_kv, err);
    else
        return fail("qk_norm_rope_store: unsupported dtype %d", dtype);
    return check_launch("qk_norm_rope_store");
}

// The same on the fp32 sums of a q/k/v product (rows of `ld` floats, heads of 128, queries and cache bf16): the
// sums are read and set back to zero.  1 / 0 from the first function: whether this geometry is taken.
EMBER_API int ember_qk_norm_rope_store_sums_supported(int D, int rotary, int ld) {
    return D == 128 && (rotary == 0 || rotary == 128) && ld % 8 == 0;
}
EMBER_API int ember_qk_norm_rope_store_sums(float* sums, int T, int ld, int n_heads, int n_kv,
                                            const float* q_norm_w, const float* k_norm_w, float eps,
                                            const float* inv_freq, int rotary, const int* positions, const int* seq_of,
                                            const int* block_table, int max_blocks, int page, int num_pages,
                                            void* q_out, void* k_pool, void* v_pool, int write_kv, int* err, void* stream) {
    if (T <= 0) return 0;
    const bool rotate = inv_freq != nullptr && rotary > 0;
    if (!ember_qk_norm_rope_store_sums_supported(128, rotate ? rotary : 0, ld) || n_heads <= 0 || n_kv <= 0 ||
        ld < (n_heads + 2 * n_kv) * 128)
        return fail("qk_norm_rope_store_sums: %d/%d heads of 128 in rows of %d floats, rotation %d are not taken", n_heads, n_kv, ld, rotary);
    if (page <= 0 || max_blocks <= 0 || num_pages <= 0) return fail("qk_norm_rope_store_sums: bad cache geometry");
    if (((uintptr_t)sums | (uintptr_t)q_out | (uintptr_t)k_pool | (uintptr_t)v_pool | (uintptr_t)q_norm_w | (uintptr_t)k_norm_w) & 15)
        return fail("qk_norm_rope_store_sums: operands must be 16-byte aligned");
    const int slots = n_heads + 2 * n_kv;
    int gy = (592 + T - 1) / T;
    const int gy_max = (slots + 2 * ROPE128_WARPS - 1) / (2 * ROPE128_WARPS);
    if (gy > gy_max) gy = gy_max;
    if (gy < 1) gy = 1;
    launch_kernel(qk_norm_rope_store_d128_kernel<float, __nv_bfloat16, true>, dim3(T, gy), ROPE128_WARPS * 32, 0, (cudaStream_t)stream,
        sums, ld, n_heads, n_kv, q_norm_w, k_norm_w, eps, inv_freq, rotate ? 1 : 0, positions, seq_of,
        block_table, max_blocks, page, num_pages, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, write_kv, err);
    return check_launch("qk_norm_rope_store_sums");
}

EMBER_API int ember_rope_table(const int* positions, const float* inv_freq, int T, int half, int ld, void* out, void* stream) {
    if (T <= 0 || half <= 0) return 0;
    if ((half & 1) || ld < T) return fail("rope_table: %d frequencies (an even number is wanted), rows of %d for %d tokens", half, ld, T);
    if (((uintptr_t)out) & 15) return fail("rope_table: the output must be 16-byte aligned");
    launch_kernel(rope_table_kernel, (unsigned)(((long long)T * (half / 2) + 255) / 256), 256, 0, (cudaStream_t)stream, positions,
                  inv_freq, T, half, ld, (float4*)out);
    return check_launch("rope_table");
}

EMBER_API int ember_silu_mul_interleaved(const void* x, void* out, int dtype, long long n_out, void* stream) {
    if (n_out <= 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    const unsigned blocks = (unsigned)((n_out + 255) / 256);
    if (dtype == EMBER_F32)
        launch_kernel(silu_mul_interleaved_kernel<float>, blocks, 256, 0, st, (const float*)x, (float*)out, (size_t)n_out);
    else if (dtype == EMBER_BF16)
        launch_kernel(silu_mul_interleaved_kernel<__nv_bfloat16>, blocks, 256, 0, st, (const __nv_bfloat16*)x, (__nv_bfloat16*)out, (size_t)n_out);
    else
        return fail("silu_mul: unsupported dtype %d", dtype);
    return check_launch("silu_mul");
}
