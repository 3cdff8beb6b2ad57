// Host encoder of the BF16N format (see encode.cpp). Mirrors the reference's bf16n::encode (core/include/bf16n/encode.h:12-26).
#pragma once

#include "format.h"

#include <cstdint>
#include <vector>

namespace b16 {

struct Encoded {
    std::vector<uint8_t> plane; // rows * K sign|mantissa bytes
    std::vector<uint8_t> aux;   // 256-byte header + exponent data
    int format = 0;             // format produced (a HUFPAIR request falls back to HUFFMAN above 4096 distinct pairs)
    int R = 0;                  // rows per unit, 0 for NIBBLE
};

// rows x K BF16 bit patterns, row-major. Argument rules and std::invalid_argument behaviour as the reference:
//   NIBBLE: R = 0, no layout flags; HUFFMAN/HUFPAIR: R in {1,2,4,8,16}, rows % R == 0;
//   chunk_major: HUFPAIR, K > 512, R in {4,8,16}; frag_order: HUFPAIR, R = 16, not chunk-major; 512 <= K <= 4096, K % 512 == 0.
Encoded encode(const uint16_t * w, int64_t rows, int64_t K, int format, int R, bool chunk_major, bool frag_order = false);

} // namespace b16
