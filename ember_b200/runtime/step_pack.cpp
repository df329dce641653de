// Host-side packing of one step's integer arrays into the staging buffer that is copied to the
// device: token ids, positions, run index of every token, run starts, cached lengths, state
// slots, wanted rows, one padded block table per cache group and the attention tile lists.
//
// This is the per-step inner loop of the engine's host side (the reference builds the same
// arrays in src/engine/engine.cpp:253-263, 339-354 and packs them in
// src/backend/cuda/cuda_backend.cu:153-202); it is C++ so that a decode step costs microseconds
// of host time.  Plain C ABI, no CUDA: it compiles with g++ and is tested on the CPU.
#include <cstdint>
#include <cstring>

extern "C" {

struct EmberStepLayout {     // element offsets into the packed buffer (each a multiple of 8)
    int32_t tokens, positions, seq_of, query_start, context_len, state_slots, logit_rows;
    int32_t tables[8];       // per cache group
    int32_t tiles[8];        // per requested tile list
    int32_t n_tiles[8];      // rows of every tile list
    int32_t total;           // ints used
    int32_t T, S, R;
    int32_t max_context;
};

static inline int32_t round8(int32_t n) { return (n + 7) / 8 * 8; }

// Runs are given as parallel arrays: counts[s] new tokens starting at position starts[s], state slot
// slots[s], want_counts[s] wanted rows; tokens and wanted rows are flat, in run order.
//
// Sizes the layout.  tile_q[i] / tile_kind[i] (0 all runs, 1 runs of two or more tokens, 2 single tokens)
// describe the tile lists wanted.  Returns 0, or a negative code: -1 empty step, -2 a run without tokens,
// -3 a wanted row outside its run, -4 a token id outside the vocabulary, -5 too many groups or lists.
// A token -(r + 1) with r < n_prev names the id sampled in row r of the step before (still on the device).
int ember_step_layout(int n_runs, const int32_t* counts, const int32_t* starts, const int32_t* want_counts,
                      const int32_t* tokens, const int32_t* want, int n_groups, const int32_t* table_widths,
                      int n_lists, const int32_t* tile_q, const int32_t* tile_kind, int vocab, int n_prev,
                      EmberStepLayout* out) {
    if (n_runs <= 0) return -1;
    if (n_groups > 8 || n_lists > 8) return -5;
    int32_t T = 0, R = 0, max_ctx = 0;
    for (int s = 0; s < n_runs; s++) {
        if (counts[s] <= 0) return -2;
        for (int i = 0; i < want_counts[s]; i++)
            if (want[R + i] < 0 || want[R + i] >= counts[s]) return -3;
        for (int i = 0; i < counts[s]; i++)
            if (tokens[T + i] < -n_prev || tokens[T + i] >= vocab) return -4;
        T += counts[s];
        R += want_counts[s];
        if (starts[s] + counts[s] > max_ctx) max_ctx = starts[s] + counts[s];
    }
    int32_t at = 0;
    out->tokens = at; at += round8(T);
    out->positions = at; at += round8(T);
    out->seq_of = at; at += round8(T);
    out->query_start = at; at += round8(n_runs + 1);
    out->context_len = at; at += round8(n_runs);
    out->state_slots = at; at += round8(n_runs);
    out->logit_rows = at; at += round8(R);
    for (int g = 0; g < n_groups; g++) { out->tables[g] = at; at += round8(n_runs * table_widths[g]); }
    for (int l = 0; l < n_lists; l++) {
        int32_t n = 0;
        for (int s = 0; s < n_runs; s++) {
            const int32_t len = counts[s];
            if ((tile_kind[l] == 1 && len < 2) || (tile_kind[l] == 2 && len != 1)) continue;
            n += (len + tile_q[l] - 1) / tile_q[l];
        }
        out->n_tiles[l] = n;
        out->tiles[l] = at;
        at += round8(n * 4);
    }
    out->total = at < 8 ? 8 : at;
    out->T = T; out->S = n_runs; out->R = R; out->max_context = max_ctx;
    return 0;
}

// Fills `dst` (at least layout->total ints) according to the layout.  tables[g * n_runs + s] is the address
// of run s's block table of group g with table_lens[g * n_runs + s] entries; shorter tables are padded with -1.
void ember_step_pack(int n_runs, const int32_t* counts, const int32_t* starts, const int32_t* slots,
                     const int32_t* want_counts, const int32_t* tokens, const int32_t* want, int n_groups,
                     const int32_t* table_widths, const uint64_t* tables, const int32_t* table_lens, int n_lists,
                     const int32_t* tile_q, const int32_t* tile_kind, const EmberStepLayout* lay, int32_t* dst) {
    int32_t t = 0, row = 0;
    int32_t* qs = dst + lay->query_start;
    qs[0] = 0;
    for (int s = 0; s < n_runs; s++) {
        const int32_t n = counts[s];
        std::memcpy(dst + lay->tokens + t, tokens + t, sizeof(int32_t) * (size_t)n);
        for (int i = 0; i < n; i++) {
            dst[lay->positions + t + i] = starts[s] + i;
            dst[lay->seq_of + t + i] = s;
        }
        for (int i = 0; i < want_counts[s]; i++) {
            dst[lay->logit_rows + row] = t + want[row];
            row++;
        }
        dst[lay->context_len + s] = starts[s] + n;
        dst[lay->state_slots + s] = slots[s];
        t += n;
        qs[s + 1] = t;
    }
    for (int g = 0; g < n_groups; g++) {
        const int32_t w = table_widths[g];
        int32_t* tb = dst + lay->tables[g];
        for (int s = 0; s < n_runs; s++) {
            int32_t n = table_lens[g * n_runs + s];
            if (n > w) n = w;
            if (n > 0) std::memcpy(tb + (size_t)s * w, reinterpret_cast<const int32_t*>(tables[g * n_runs + s]), sizeof(int32_t) * (size_t)n);
            for (int32_t i = n < 0 ? 0 : n; i < w; i++) tb[(size_t)s * w + i] = -1;
        }
    }
    for (int l = 0; l < n_lists; l++) {
        int32_t* tl = dst + lay->tiles[l];
        int32_t k = 0;
        for (int s = 0; s < n_runs; s++) {
            const int32_t len = counts[s];
            if ((tile_kind[l] == 1 && len < 2) || (tile_kind[l] == 2 && len != 1)) continue;
            for (int32_t a = 0; a < len; a += tile_q[l]) {
                tl[4 * k + 0] = s;
                tl[4 * k + 1] = qs[s] + a;
                tl[4 * k + 2] = len - a < tile_q[l] ? len - a : tile_q[l];
                tl[4 * k + 3] = starts[s] + a;
                k++;
            }
        }
    }
}

}  // extern "C"
