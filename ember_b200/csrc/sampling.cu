// Sorting-free sampling, one block per logits row.
//
// Semantics (src/backend/sampling_host.cpp:20-85, src/backend/sampling_rng.hpp:21-33):
//   temperature <= 1e-5: argmax, lowest index on ties.
//   else x_i = logit_i / T; keep the top_k largest (value descending, index ascending); softmax
//   over the kept set; keep the smallest prefix (in that order) whose mass reaches top_p; drop
//   tokens with p < min_p * p(best); draw by Gumbel-max: argmax_i x_i + g(seed, counter, i),
//   g = -log(-log(u)), u = ((h >> 40) + 0.5) / 2^24, h = mix(seed ^ mix(counter * C + i)).
// The noise depends only on (seed, counter, token id), so a request draws the same tokens
// whatever shares its batch.
//
// Instead of sorting, the k-th largest value and the top-p cut are found by radix selection
// over an order-preserving integer image of the floats (4 passes of 8 bits; counts for top-k,
// probability mass in double for top-p).  Ties at a cut are resolved as the host does, by
// index: the cut keeps the lowest indices among equal values.  (The reference's device sampler,
// src/backend/cuda/k_sampling.cu:149-166, has the same outline; this one is written anew.)
#include "common.cuh"

EMBER_DEFINE_LAST_ERROR

namespace ember {

constexpr int SAMPLE_THREADS = 1024;

struct SampleParams {  // 32 bytes per row, mirrored by the Python side
    float temperature;
    int top_k;
    float top_p;
    float min_p;
    unsigned long long seed;
    unsigned long long counter;
};

__host__ __device__ __forceinline__ unsigned long long rng_mix(unsigned long long z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

__device__ __forceinline__ float gumbel_noise(unsigned long long seed, unsigned long long counter, unsigned id) {
    const unsigned long long h = rng_mix(seed ^ rng_mix(counter * 0x632BE59BD9B4E019ull + id));
    const float u = ((float)(h >> 40) + 0.5f) * (1.0f / 16777216.0f);
    return -logf(-logf(u));
}

// Monotone image of a float: larger float <=> larger key.
__device__ __forceinline__ unsigned float_key(float x) {
    const unsigned b = __float_as_uint(x);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

struct Shared {
    unsigned count[256];
    double mass[256];
    float red_f[32];
    int red_i[32];
    double red_d[32];
    unsigned prefix, select_mask;   // key bits fixed so far
    unsigned long long remaining_k;
    double remaining_mass;
    int warp_counts[32];
    int found;
};

__device__ float block_max_arg(float v, int idx, int* arg_out, Shared& sh) {
    // max value, lowest index among equals
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
    }
    __syncthreads();
    if (lane == 0) { sh.red_f[warp] = v; sh.red_i[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        v = sh.red_f[lane];
        idx = sh.red_i[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, v, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
        }
        if (lane == 0) { sh.red_f[0] = v; sh.red_i[0] = idx; }
    }
    __syncthreads();
    *arg_out = sh.red_i[0];
    return sh.red_f[0];
}

__device__ double block_sum_double(double v, Shared& sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) sh.red_d[warp] = v;
    __syncthreads();
    double r = sh.red_d[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
    return r;
}

// Index of the n-th (1-based) element, in index order, whose key equals `key` and passes `pred`.
// Returns V if there are fewer than n.
template <typename Pred>
__device__ int nth_equal_index(const float* __restrict__ logits, float inv_t_div, int V, unsigned key, int n, Pred pred,
                               Shared& sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int seen = 0;
    __syncthreads();
    if (threadIdx.x == 0) sh.found = V;
    __syncthreads();
    for (int base = 0; base < V; base += SAMPLE_THREADS) {
        const int i = base + threadIdx.x;
        bool hit = false;
        if (i < V) {
            const float x = logits[i] / inv_t_div;
            hit = float_key(x) == key && pred(i, x);
        }
        const unsigned ballot = __ballot_sync(0xffffffffu, hit);
        if (lane == 0) sh.warp_counts[warp] = __popc(ballot);
        __syncthreads();
        int before = 0, total = 0;
        for (int w = 0; w < SAMPLE_THREADS / 32; w++) {
            const int c = sh.warp_counts[w];
            if (w < warp) before += c;
            total += c;
        }
        const int rank = seen + before + __popc(ballot & ((1u << lane) - 1u)) + 1;  // 1-based if hit
        if (hit && rank == n) sh.found = i;
        seen += total;
        __syncthreads();
        if (seen >= n) break;
    }
    __syncthreads();
    return sh.found;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits_all, int V, const SampleParams* __restrict__ params,
              int* __restrict__ out) {
    __shared__ Shared sh;
    const int row = blockIdx.x;
    const float* logits = logits_all + (size_t)row * V;
    const SampleParams p = params[row];
    const int tid = threadIdx.x;

    // ---- greedy, and the maximum for everything else
    const bool greedy = p.temperature <= 1e-5f;
    const float tdiv = greedy ? 1.0f : p.temperature;
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int i = tid; i < V; i += SAMPLE_THREADS) {
        const float x = logits[i] / tdiv;
        if (x > best) { best = x; best_i = i; }   // ascending i: the first maximum stays
    }
    int arg;
    const float xmax = block_max_arg(best, best_i, &arg, sh);
    if (greedy) {
        if (tid == 0) out[row] = arg;
        return;
    }

    // ---- top-k: key of the k-th largest value, and the index cut among equal values
    unsigned k_key = 0;         // keep key > k_key, or key == k_key with index <= k_cut
    int k_cut = V;
    const bool use_k = p.top_k > 0 && p.top_k < V;
    if (use_k) {
        if (tid == 0) { sh.prefix = 0; sh.select_mask = 0; sh.remaining_k = (unsigned long long)p.top_k; }
        for (int pass = 0; pass < 4; pass++) {
            const int shift = 24 - 8 * pass;
            if (tid < 256) sh.count[tid] = 0;
            __syncthreads();
            const unsigned prefix = sh.prefix, mask = sh.select_mask;
            for (int i = tid; i < V; i += SAMPLE_THREADS) {
                const unsigned key = float_key(logits[i] / tdiv);
                if ((key & mask) == prefix) atomicAdd(&sh.count[(key >> shift) & 255u], 1u);
            }
            __syncthreads();
            if (tid == 0) {
                unsigned long long rem = sh.remaining_k;
                int b = 255;
                for (; b > 0; b--) {
                    if (sh.count[b] >= rem) break;
                    rem -= sh.count[b];
                }
                sh.remaining_k = rem;               // how many of bin b (with the prefix) are still wanted
                sh.prefix = prefix | ((unsigned)b << shift);
                sh.select_mask = mask | (255u << shift);
            }
            __syncthreads();
        }
        k_key = sh.prefix;
        const int need_eq = (int)sh.remaining_k;   // of the values equal to the k-th, the lowest need_eq indices
        k_cut = nth_equal_index(logits, tdiv, V, k_key, need_eq, [](int, float) { return true; }, sh);
    }
    auto kept_k = [&](int i, unsigned key) { return !use_k || key > k_key || (key == k_key && i <= k_cut); };

    // ---- mass of the kept set
    double z_local = 0.0;
    for (int i = tid; i < V; i += SAMPLE_THREADS) {
        const float x = logits[i] / tdiv;
        if (kept_k(i, float_key(x))) z_local += exp((double)x - (double)xmax);
    }
    const double Z = block_sum_double(z_local, sh);

    // ---- top-p: the smallest prefix (value descending, index ascending) whose mass reaches top_p * Z
    unsigned p_key = 0;
    int p_cut = V;
    const bool use_p = p.top_p < 1.0f;
    if (use_p) {
        if (tid == 0) { sh.prefix = 0; sh.select_mask = 0; sh.remaining_mass = (double)p.top_p * Z; }
        for (int pass = 0; pass < 4; pass++) {
            const int shift = 24 - 8 * pass;
            if (tid < 256) { sh.mass[tid] = 0.0; sh.count[tid] = 0; }
            __syncthreads();
            const unsigned prefix = sh.prefix, mask = sh.select_mask;
            for (int i = tid; i < V; i += SAMPLE_THREADS) {
                const float x = logits[i] / tdiv;
                const unsigned key = float_key(x);
                if ((key & mask) == prefix && kept_k(i, key)) {
                    atomicAdd(&sh.mass[(key >> shift) & 255u], exp((double)x - (double)xmax));
                    atomicAdd(&sh.count[(key >> shift) & 255u], 1u);
                }
            }
            __syncthreads();
            if (tid == 0) {
                double rem = sh.remaining_mass;
                int b = 255;
                for (; b > 0; b--) {
                    if (sh.count[b] == 0) continue;
                    if (sh.mass[b] >= rem) break;
                    rem -= sh.mass[b];
                }
                // if rounding left a sliver after the last populated bin, the cut is the lowest populated bin
                if (b == 0 && sh.count[0] == 0)
                    for (b = 0; b < 255 && sh.count[b] == 0; b++) {}
                sh.remaining_mass = rem;
                sh.prefix = prefix | ((unsigned)b << shift);
                sh.select_mask = mask | (255u << shift);
            }
            __syncthreads();
        }
        p_key = sh.prefix;
        // all values with key == p_key are equal floats: each carries the same mass e
        const float xv = __uint_as_float((p_key & 0x80000000u) ? (p_key & 0x7fffffffu) : ~p_key);
        const double e = exp((double)xv - (double)xmax);
        double need = ceil(sh.remaining_mass / e);
        if (!(need >= 1.0)) need = 1.0;
        const int need_eq = need > 2147483000.0 ? 2147483000 : (int)need;
        p_cut = nth_equal_index(logits, tdiv, V, p_key, need_eq,
                                [&](int i, float x) { return kept_k(i, float_key(x)); }, sh);
    }

    // ---- min-p and the draw
    const double floor_p = p.min_p > 0.0f ? (double)p.min_p : -1.0;
    float best_s = -INFINITY;
    int best_t = 0x7fffffff;
    for (int i = tid; i < V; i += SAMPLE_THREADS) {
        const float x = logits[i] / tdiv;
        const unsigned key = float_key(x);
        bool keep = kept_k(i, key);
        if (keep && use_p) keep = key > p_key || (key == p_key && i <= p_cut);
        if (keep && floor_p > 0.0 && i != arg) keep = exp((double)x - (double)xmax) >= floor_p;
        if (!keep) continue;
        const float s = x + gumbel_noise(p.seed, p.counter, (unsigned)i);
        if (s > best_s) { best_s = s; best_t = i; }
    }
    int tok;
    block_max_arg(best_s, best_t, &tok, sh);
    if (tid == 0) out[row] = tok == 0x7fffffff ? arg : tok;
}

// ---- greedy rows only: argmax in two steps so that many blocks share a row
constexpr int ARGMAX_CHUNKS = 32;

__global__ void __launch_bounds__(256)
argmax_partial_kernel(const float* __restrict__ logits_all, int V, float* __restrict__ part_v, int* __restrict__ part_i) {
    __shared__ float sv[8];
    __shared__ int si[8];
    const int row = blockIdx.x, chunk = blockIdx.y;
    const float* logits = logits_all + (size_t)row * V;
    const int per = (V + ARGMAX_CHUNKS - 1) / ARGMAX_CHUNKS;
    const int lo = chunk * per, hi = min(V, lo + per);
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int i = lo + threadIdx.x; i < hi; i += 256) {
        const float x = logits[i];
        if (x > best) { best = x; best_i = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { sv[warp] = best; si[warp] = best_i; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; w++)
            if (sv[w] > best || (sv[w] == best && si[w] < best_i)) { best = sv[w]; best_i = si[w]; }
        part_v[row * ARGMAX_CHUNKS + chunk] = best;
        part_i[row * ARGMAX_CHUNKS + chunk] = best_i;
    }
}

__global__ void argmax_final_kernel(const float* __restrict__ part_v, const int* __restrict__ part_i, int* __restrict__ out) {
    const int row = blockIdx.x, lane = threadIdx.x;      // 32 threads, one per chunk
    float best = part_v[row * ARGMAX_CHUNKS + lane];
    int best_i = part_i[row * ARGMAX_CHUNKS + lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if (lane == 0) out[row] = best_i == 0x7fffffff ? 0 : best_i;
}

}  // namespace ember

using namespace ember;

// Argmax of every row (lowest index on ties): the greedy case, spread over many blocks.
// part_v / part_i: scratch of rows * 32 floats / ints.
EMBER_API int ember_argmax(const float* logits, int rows, int V, float* part_v, int* part_i, int* out, void* stream) {
    if (rows <= 0) return 0;
    if (V <= 0) return fail("argmax: vocabulary %d", V);
    static_assert(ARGMAX_CHUNKS == 32, "the final step uses one warp");
    cudaStream_t st = (cudaStream_t)stream;
    argmax_partial_kernel<<<dim3(rows, ARGMAX_CHUNKS), 256, 0, st>>>(logits, V, part_v, part_i);
    argmax_final_kernel<<<rows, 32, 0, st>>>(part_v, part_i, out);
    return check_launch("argmax");
}

EMBER_API int ember_sample(const float* logits, int rows, int V, const void* params, int* out, void* stream) {
    if (rows <= 0) return 0;
    if (V <= 0) return fail("sample: vocabulary %d", V);
    static_assert(sizeof(SampleParams) == 32, "parameter rows are 32 bytes");
    sample_kernel<<<rows, SAMPLE_THREADS, 0, (cudaStream_t)stream>>>(logits, V, (const SampleParams*)params, out);
    return check_launch("sample");
}
