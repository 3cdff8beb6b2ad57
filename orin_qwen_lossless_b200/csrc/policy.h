// Shape policy: which BF16N format and unit layout a weight tensor gets. Mirrors the reference's bf16n::choose
// (core/include/bf16n/policy.h:12-38, core/src/policy.cpp:9-69) decision for decision; eligibility by dtype, name and
// device stays with the engine that calls it.
#pragma once

#include "format.h"

#include <cstdint>

namespace b16 {

enum class Engine { llama = 0, vllm = 1 };
enum class Mode { hybrid = 0, huffman = 1, nibble = 2 };

struct PolicyOptions {
    Engine engine = Engine::vllm;
    Mode mode = Mode::hybrid;
    int64_t dense_min = 8ll << 20;  // dense tensors with fewer weights take NIBBLE
    bool expert = false;            // llama: the loader says whether the tensor is a routed-expert stack
    bool dense_frag_order = false;  // vLLM linear layers opt in to fragment-order bands
    int64_t min_units = 512;        // a dense pair-Huffman matrix keeps at least this many units (one per warp of a full
                                    // machine in the decode GEMV's first wave). 512 is the reference's constant, sized
                                    // for the GPU it was written on; a B200 runs about 148 x 27 such warps, so a loader
                                    // that shards a matrix over several B200s passes its own machine size here.
};

struct PolicyChoice {
    int format;
    int R; // 0 for NIBBLE
    bool chunk_major;
    bool frag_order;
};

// false: the shape stays BF16. HUFPAIR is a request; the encoder may fall back to HUFFMAN.
bool choose(int64_t rows, int64_t K, int64_t n_matrices, const PolicyOptions & opts, PolicyChoice * out) noexcept;

} // namespace b16
