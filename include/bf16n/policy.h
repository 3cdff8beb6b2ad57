// bf16n::choose with the reference's types (core/include/bf16n/policy.h:12-38) over the C ABI.
#pragma once

#include "../bf16n_c.h"
#include "format.h"

#include <cstdint>
#include <optional>

namespace bf16n {

enum class policy_engine { llama, vllm };
enum class policy_mode { hybrid, huffman, nibble };

struct policy_options {
    policy_engine engine = policy_engine::vllm;
    policy_mode mode = policy_mode::hybrid;
    int64_t dense_min = 8ll << 20;
    bool expert = false;
    bool dense_frag_order = false;
};

struct policy_choice {
    int format;
    int R;
    bool chunk_major;
    bool frag_order = false;
};

inline std::optional<policy_choice> choose(int64_t rows, int64_t K, int64_t n_matrices = 1, policy_options o = {}) noexcept {
    int out[4];
    const int mode = o.mode == policy_mode::huffman ? 1 : o.mode == policy_mode::nibble ? 2 : 0;
    if (!bf16n_choose(rows, K, n_matrices, o.engine == policy_engine::vllm, mode, o.dense_min, o.expert, o.dense_frag_order, out)) {
        return std::nullopt;
    }
    return policy_choice{out[0], out[1], out[2] != 0, out[3] != 0};
}

} // namespace bf16n
