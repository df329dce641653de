// Sorting-free sampling: a logits row is shared by a cluster of eight blocks (one block for small vocabularies).
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
constexpr int SAMPLE_LIST = 1024;      // a top-k up to this size is finished on a list in shared memory

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

// A row is shared by a cluster of CL blocks (CL = 1: one block, no cluster).  Block r scans the r-th
// contiguous part of the row; whatever the single-block algorithm reduces over the block is reduced over the
// cluster through the first block's shared memory (distributed shared memory), in rank order, so that every
// block holds the same values and takes the same branches.
struct Shared {
    unsigned count[256];
    double mass[256];
    float red_f[32];
    int red_i[32];
    double red_d[32];
    int warp_counts[32];
    // written by the blocks of the cluster into the first block's copy, read back by all
    float x_f[16];
    int x_i[16];
    double x_d[16];
    unsigned prefix, select_mask;   // key bits fixed so far
    unsigned long long remaining_k;
    double remaining_mass;
    int found;
    // the kept set of a small top-k, gathered in the first block (any order), then sorted by (value descending,
    // index ascending)
    int n_list;
    float list_x[SAMPLE_LIST];
    int list_i[SAMPLE_LIST];
    float sort_x[SAMPLE_LIST];
    int sort_i[SAMPLE_LIST];
    double sort_e[SAMPLE_LIST];
};

__device__ __forceinline__ unsigned cl_rank() { unsigned r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
template <int CL>
__device__ __forceinline__ void cl_sync() {
    if constexpr (CL > 1) {
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    } else {
        __syncthreads();
    }
}
// The same object in block `rank` of the cluster.
template <int CL, typename T>
__device__ __forceinline__ T* cl_peer(T* local, unsigned rank) {
    if constexpr (CL > 1) {
        unsigned long long out;
        asm volatile("mapa.u64 %0, %1, %2;" : "=l"(out) : "l"((unsigned long long)local), "r"(rank));
        return (T*)out;
    } else {
        return local;
    }
}

// max value, lowest index among equals: over the block, then over the cluster
template <int CL>
__device__ float cluster_max_arg(float v, int idx, int* arg_out, Shared& sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
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
        v = lane < nwarps ? sh.red_f[lane] : -INFINITY;
        idx = lane < nwarps ? sh.red_i[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, v, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
        }
        if (lane == 0) {
            Shared* first = cl_peer<CL>(&sh, 0);
            const unsigned r = CL > 1 ? cl_rank() : 0;
            first->x_f[r] = v;
            first->x_i[r] = idx;
        }
    }
    cl_sync<CL>();
    Shared* first = cl_peer<CL>(&sh, 0);
    float bv = first->x_f[0];
    int bi = first->x_i[0];
#pragma unroll
    for (int r = 1; r < CL; r++) {
        const float ov = first->x_f[r];
        const int oi = first->x_i[r];
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    cl_sync<CL>();                      // everybody has read before the slots are written again
    *arg_out = bi;
    return bv;
}

template <int CL>
__device__ double cluster_sum_double(double v, Shared& sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) sh.red_d[warp] = v;
    __syncthreads();
    if (warp == 0) {
        double r = lane < nwarps ? sh.red_d[lane] : 0.0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
        if (lane == 0) cl_peer<CL>(&sh, 0)->x_d[CL > 1 ? cl_rank() : 0] = r;
    }
    cl_sync<CL>();
    Shared* first = cl_peer<CL>(&sh, 0);
    double total = 0.0;
#pragma unroll
    for (int r = 0; r < CL; r++) total += first->x_d[r];
    cl_sync<CL>();
    return total;
}

// After every block has filled its count[] (and mass[]): the first block's thread 0 gets the sums over the
// cluster in its own arrays.  Ends with a cluster barrier; the caller's decision step follows.
template <int CL, bool MASS>
__device__ void cluster_merge_bins(Shared& sh) {
    cl_sync<CL>();
    if constexpr (CL > 1) {
        if (cl_rank() == 0 && threadIdx.x < 256) {
            // the peers' bins are fetched together (independent loads), then added in rank order
            unsigned pc[CL];
            double pm[CL];
#pragma unroll
            for (unsigned r = 1; r < CL; r++) {
                Shared* peer = cl_peer<CL>(&sh, r);
                pc[r] = peer->count[threadIdx.x];
                pm[r] = MASS ? peer->mass[threadIdx.x] : 0.0;
            }
            unsigned c = sh.count[threadIdx.x];
            double m = MASS ? sh.mass[threadIdx.x] : 0.0;
#pragma unroll
            for (unsigned r = 1; r < CL; r++) {
                c += pc[r];
                if (MASS) m += pm[r];
            }
            sh.count[threadIdx.x] = c;
            if (MASS) sh.mass[threadIdx.x] = m;
        }
        __syncthreads();
    }
}
// The first block's decision (prefix, mask, remaining) copied into every block.
template <int CL>
__device__ void cluster_share_decision(Shared& sh) {
    cl_sync<CL>();
    if constexpr (CL > 1) {
        if (cl_rank() != 0 && threadIdx.x == 0) {
            Shared* first = cl_peer<CL>(&sh, 0);
            sh.prefix = first->prefix;
            sh.select_mask = first->select_mask;
            sh.remaining_k = first->remaining_k;
            sh.remaining_mass = first->remaining_mass;
        }
        cl_sync<CL>();                  // the first block may overwrite its bins and decision again
    }
}

// Index of the n-th (1-based) element, in index order, whose key equals `key` and passes `pred`.
// Returns V if there are fewer than n.  [lo, hi) is this block's part of the row.
template <int CL, typename Pred>
__device__ int nth_equal_index(const float* __restrict__ logits, float inv_t_div, int V, int lo, int hi, unsigned key, int n,
                               Pred pred, Shared& sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    // hits of this block, then of every block (in rank order)
    int mine = 0;
    for (int i = lo + (int)threadIdx.x; i < hi; i += blockDim.x) {
        const float x = logits[i] / inv_t_div;
        mine += (float_key(x) == key && pred(i, x)) ? 1 : 0;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, o);
    __syncthreads();
    if (lane == 0) sh.red_i[warp] = mine;
    __syncthreads();
    if (threadIdx.x == 0) {
        int total = 0;
        for (int w = 0; w < nwarps; w++) total += sh.red_i[w];
        Shared* first = cl_peer<CL>(&sh, 0);
        const unsigned r = CL > 1 ? cl_rank() : 0;
        first->x_i[r] = total;
        if (r == 0) first->found = V;
    }
    cl_sync<CL>();
    Shared* first = cl_peer<CL>(&sh, 0);
    const unsigned me = CL > 1 ? cl_rank() : 0;
    int before_me = 0, my_total = 0;
#pragma unroll
    for (unsigned r = 0; r < (unsigned)CL; r++) {
        const int c = first->x_i[r];
        if (r < me) before_me += c;
        if (r == me) my_total = c;
    }
    if (before_me < n && n <= before_me + my_total) {        // uniform over the block: the n-th lies in this part
        const int want = n - before_me;
        int seen = 0;
        for (int base = lo; base < hi; base += blockDim.x) {
            const int i = base + (int)threadIdx.x;
            bool hit = false;
            if (i < hi) {
                const float x = logits[i] / inv_t_div;
                hit = float_key(x) == key && pred(i, x);
            }
            const unsigned ballot = __ballot_sync(0xffffffffu, hit);
            if (lane == 0) sh.warp_counts[warp] = __popc(ballot);
            __syncthreads();
            int before = 0, total = 0;
            for (int w = 0; w < nwarps; w++) {
                const int c = sh.warp_counts[w];
                if (w < warp) before += c;
                total += c;
            }
            const int rank = seen + before + __popc(ballot & ((1u << lane) - 1u)) + 1;  // 1-based if hit
            if (hit && rank == want) first->found = i;
            seen += total;
            __syncthreads();
            if (seen >= want) break;
        }
    }
    cl_sync<CL>();
    const int found = first->found;
    cl_sync<CL>();
    return found;
}

template <int CL>
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits_all, int V, const SampleParams* __restrict__ params,
              int* __restrict__ out) {
    __shared__ Shared sh;
    const int row = blockIdx.x / CL;
    const unsigned rank = CL > 1 ? cl_rank() : 0;
    const float* logits = logits_all + (size_t)row * V;
    const SampleParams p = params[row];
    const int tid = threadIdx.x;
    // this block's part of the row: contiguous, so that "in index order" holds across the cluster in rank order
    const int per = (V + CL - 1) / CL;
    const int lo = min(V, (int)rank * per), hi = min(V, lo + per);

    // ---- greedy, and the maximum for everything else
    const bool greedy = p.temperature <= 1e-5f;
    const float tdiv = greedy ? 1.0f : p.temperature;
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int i = lo + tid; i < hi; i += SAMPLE_THREADS) {
        const float x = logits[i] / tdiv;
        if (x > best) { best = x; best_i = i; }   // ascending i: the first maximum stays
    }
    int arg;
    const float xmax = cluster_max_arg<CL>(best, best_i, &arg, sh);
    if (greedy) {
        if (tid == 0 && rank == 0) out[row] = arg;
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
            for (int i = lo + tid; i < hi; i += SAMPLE_THREADS) {
                const unsigned key = float_key(logits[i] / tdiv);
                if ((key & mask) == prefix) atomicAdd(&sh.count[(key >> shift) & 255u], 1u);
            }
            __syncthreads();
            cluster_merge_bins<CL, false>(sh);
            if (rank == 0 && tid < 256) {
                // the bin of the k-th largest: walking down from bin 255, the first bin (above 0) at which the
                // running count reaches what is still wanted, else bin 0.  Done by 256 threads: thread b holds
                // the count of bins b..255 (a suffix sum over eight warps).
                const int lane = tid & 31, warp = tid >> 5;
                const unsigned own = sh.count[tid];
                unsigned suf = own;                                 // within the warp: bins tid .. warp end
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const unsigned v = __shfl_down_sync(0xffffffffu, suf, o);
                    if (lane + o < 32) suf += v;
                }
                if (lane == 0) sh.warp_counts[warp] = (int)suf;     // total of this warp's 32 bins
                asm volatile("bar.sync 1, 256;" ::: "memory");
                unsigned above = 0;                                 // bins of the warps above this one
                for (int w = warp + 1; w < 8; w++) above += (unsigned)sh.warp_counts[w];
                const unsigned long long rem = sh.remaining_k;
                const unsigned long long s_b = (unsigned long long)suf + above;     // count of bins tid..255
                const unsigned long long s_next = s_b - own;                        // count of bins tid+1..255
                const bool here = tid > 0 && s_b >= rem && s_next < rem;
                const unsigned any = __ballot_sync(0xffffffffu, here);
                if (lane == 0) sh.red_i[warp] = (int)any;
                asm volatile("bar.sync 1, 256;" ::: "memory");
                bool found = false;
                for (int w = 0; w < 8; w++) found |= sh.red_i[w] != 0;
                if (here || (!found && tid == 0)) {
                    sh.remaining_k = rem - s_next;      // how many of this bin (with the prefix) are still wanted
                    sh.prefix = prefix | ((unsigned)tid << shift);
                    sh.select_mask = mask | (255u << shift);
                }
            }
            cluster_share_decision<CL>(sh);
            __syncthreads();
        }
        k_key = sh.prefix;
        const int need_eq = (int)sh.remaining_k;   // of the values equal to the k-th, the lowest need_eq indices
        k_cut = nth_equal_index<CL>(logits, tdiv, V, lo, hi, k_key, need_eq, [](int, float) { return true; }, sh);
    }
    auto kept_k = [&](int i, unsigned key) { return !use_k || key > k_key || (key == k_key && i <= k_cut); };

    if (use_k && p.top_k <= SAMPLE_LIST) {
        // ---- a small kept set: gather it in the first block and finish there as the host does, on a list
        // sorted by (value descending, index ascending): cumulative mass for top-p, min-p, the draw.  This
        // replaces seven more scans of the row (and their cluster barriers) by one.
        if (tid == 0 && rank == 0) sh.n_list = 0;
        cl_sync<CL>();
        Shared* first = cl_peer<CL>(&sh, 0);
        for (int i = lo + tid; i < hi; i += SAMPLE_THREADS) {
            const float x = logits[i] / tdiv;
            if (kept_k(i, float_key(x))) {
                const int slot = atomicAdd(&first->n_list, 1);
                if (slot < SAMPLE_LIST) { first->list_x[slot] = x; first->list_i[slot] = i; }
            }
        }
        cl_sync<CL>();
        if (rank != 0) return;                       // the first block goes on alone (block barriers only)
        const int n = min(sh.n_list, SAMPLE_LIST);
        // position of every element in the sorted order: how many come before it
        for (int j = tid; j < n; j += SAMPLE_THREADS) {
            const float xj = sh.list_x[j];
            const int ij = sh.list_i[j];
            int before = 0;
            for (int l = 0; l < n; l++) {
                const float xl = sh.list_x[l];
                before += (xl > xj || (xl == xj && sh.list_i[l] < ij)) ? 1 : 0;
            }
            sh.sort_x[before] = xj;
            sh.sort_i[before] = ij;
            sh.sort_e[before] = exp((double)xj - (double)xmax);
        }
        __syncthreads();
        // top-p: the shortest prefix whose mass reaches top_p * Z (one thread walks the list: it is short)
        if (tid == 0) {
            int keep_n = n;
            if (p.top_p < 1.0f) {
                double Z = 0.0;
                for (int j = 0; j < n; j++) Z += sh.sort_e[j];
                const double want = (double)p.top_p * Z;
                double cum = 0.0;
                keep_n = 0;
                while (keep_n < n) {
                    cum += sh.sort_e[keep_n++];
                    if (cum >= want) break;
                }
            }
            sh.found = keep_n;
        }
        __syncthreads();
        const int keep_n = sh.found;
        const double floor_p = p.min_p > 0.0f ? (double)p.min_p : -1.0;
        float best_s = -INFINITY;
        int best_t = 0x7fffffff;
        for (int j = tid; j < keep_n; j += SAMPLE_THREADS) {
            const int i = sh.sort_i[j];
            if (floor_p > 0.0 && i != arg && !(sh.sort_e[j] >= floor_p)) continue;
            const float s_ = sh.sort_x[j] + gumbel_noise(p.seed, p.counter, (unsigned)i);
            if (s_ > best_s || (s_ == best_s && i < best_t)) { best_s = s_; best_t = i; }
        }
        int tok;
        cluster_max_arg<1>(best_s, best_t, &tok, sh);
        if (tid == 0) out[row] = tok == 0x7fffffff ? arg : tok;
        return;
    }

    // ---- top-p: the smallest prefix (value descending, index ascending) whose mass reaches top_p * Z
    unsigned p_key = 0;
    int p_cut = V;
    const bool use_p = p.top_p < 1.0f;
    if (use_p) {
        // mass of the kept set (nothing else needs it)
        double z_local = 0.0;
        for (int i = lo + tid; i < hi; i += SAMPLE_THREADS) {
            const float x = logits[i] / tdiv;
            if (kept_k(i, float_key(x))) z_local += exp((double)x - (double)xmax);
        }
        const double Z = cluster_sum_double<CL>(z_local, sh);
        if (tid == 0) { sh.prefix = 0; sh.select_mask = 0; sh.remaining_mass = (double)p.top_p * Z; }
        for (int pass = 0; pass < 4; pass++) {
            const int shift = 24 - 8 * pass;
            if (tid < 256) { sh.mass[tid] = 0.0; sh.count[tid] = 0; }
            __syncthreads();
            const unsigned prefix = sh.prefix, mask = sh.select_mask;
            for (int i = lo + tid; i < hi; i += SAMPLE_THREADS) {
                const float x = logits[i] / tdiv;
                const unsigned key = float_key(x);
                if ((key & mask) == prefix && kept_k(i, key)) {
                    atomicAdd(&sh.mass[(key >> shift) & 255u], exp((double)x - (double)xmax));
                    atomicAdd(&sh.count[(key >> shift) & 255u], 1u);
                }
            }
            __syncthreads();
            cluster_merge_bins<CL, true>(sh);
            if (tid == 0 && rank == 0) {
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
            cluster_share_decision<CL>(sh);
            __syncthreads();
        }
        p_key = sh.prefix;
        // all values with key == p_key are equal floats: each carries the same mass e
        const float xv = __uint_as_float((p_key & 0x80000000u) ? (p_key & 0x7fffffffu) : ~p_key);
        const double e = exp((double)xv - (double)xmax);
        double need = ceil(sh.remaining_mass / e);
        if (!(need >= 1.0)) need = 1.0;
        const int need_eq = need > 2147483000.0 ? 2147483000 : (int)need;
        p_cut = nth_equal_index<CL>(logits, tdiv, V, lo, hi, p_key, need_eq,
                                    [&](int i, float x) { return kept_k(i, float_key(x)); }, sh);
    }

    // ---- min-p and the draw
    const double floor_p = p.min_p > 0.0f ? (double)p.min_p : -1.0;
    float best_s = -INFINITY;
    int best_t = 0x7fffffff;
    for (int i = lo + tid; i < hi; i += SAMPLE_THREADS) {
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
    cluster_max_arg<CL>(best_s, best_t, &tok, sh);
    if (tid == 0 && rank == 0) out[row] = tok == 0x7fffffff ? arg : tok;
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
    // A row is shared by a cluster of 8 blocks (one block alone spends 0.2-2 ms on a vocabulary of 150,000: its
    // passes are instruction-bound on one SM); small vocabularies stay with one block.
    constexpr int CL = 8;
    if (V >= 8192) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)rows * CL);
        cfg.blockDim = dim3(SAMPLE_THREADS);
        cfg.stream = (cudaStream_t)stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = CL; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr; cfg.numAttrs = 1;
        if (cudaLaunchKernelEx(&cfg, sample_kernel<CL>, logits, V, (const SampleParams*)params, out) == cudaSuccess)
            return check_launch("sample");
        cudaGetLastError();                     // clusters of 8 not available: one block per row
    }
    sample_kernel<1><<<rows, SAMPLE_THREADS, 0, (cudaStream_t)stream>>>(logits, V, (const SampleParams*)params, out);
    return check_launch("sample");
}
