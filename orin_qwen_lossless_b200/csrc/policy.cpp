#include "policy.h"

namespace b16 {
namespace {

// Rows per unit of a dense HUFPAIR matrix. Candidates keep at least min_units units (512 in the reference: one per warp of a full machine in the
// decode GEMV's first wave). llama takes the largest such R; vLLM prefers a smaller R when its wave model says the
// last, partly empty wave of 512 units costs at least 5 % less (cost = waves * R rows per warp).
int dense_unit_rows(int64_t rows, Engine engine, int64_t min_units) noexcept {
    int pick = 1;
    int64_t pick_cost = 0;
    const int cand[4] = {16, 8, 4, 2};
    for (int r : cand) {
        const int64_t units = rows / r;
        if (rows % r != 0 || units < min_units) { continue; }
        const int64_t waves = (units + min_units - 1) / min_units;
        const int64_t cost = waves * r;
        if (pick == 1) {
            pick = r;
            pick_cost = cost;
            if (engine == Engine::llama) { return pick; }
        } else if ((double) cost <= 0.95 * (double) pick_cost) {
            pick = r;
            pick_cost = cost;
        }
    }
    return pick;
}

int64_t ceil_div(int64_t a, int64_t b) { return a / b + (a % b != 0); }

} // namespace

bool choose(int64_t rows, int64_t K, int64_t n_matrices, const PolicyOptions & o, PolicyChoice * out) noexcept {
    if (rows <= 0 || n_matrices <= 0 || K <= 0 || K % CHUNK != 0 || K > K_MAX) { return false; }
    const bool vllm = o.engine == Engine::vllm;
    const bool stack = n_matrices > 1;
    const bool expert = vllm ? stack : o.expert;
    // rows * K * n_matrices >= dense_min, evaluated without forming the product
    const bool large = o.dense_min <= 0 || rows >= ceil_div(ceil_div(o.dense_min, n_matrices), K);
    if (o.mode == Mode::nibble || (o.mode == Mode::hybrid && !expert && !large)) {
        *out = {FMT_NIBBLE, 0, false, false};
        return true;
    }
    const bool bands = rows % 16 == 0;
    const bool fo_dense = vllm && o.dense_frag_order && !stack && bands;     // opted-in linear layers
    const bool fo_gate_up = vllm && stack && K == 4 * CHUNK && bands;        // K = 2048 expert stacks
    int R;
    if (stack) {
        R = (fo_gate_up || (bands && rows >= 2048)) ? 16 : rows % 8 == 0 ? 8 : rows % 4 == 0 ? 4 : 1;
    } else {
        R = fo_dense ? 16 : dense_unit_rows(rows, o.engine, o.min_units > 0 ? o.min_units : 512);
    }
    const bool fo_down = vllm && stack && K == CHUNK && R == 16;             // K = 512 expert stacks
    const bool fo = fo_gate_up || fo_down || fo_dense;
    *out = {FMT_HUFPAIR, R, stack && K > CHUNK && !(fo_gate_up || fo_down), fo};
    return true;
}

} // namespace b16
