// BF16N storage format constants with the reference's names (core/include/bf16n/format.h:12-51).
#pragma once

#include <cstdint>

namespace bf16n {

constexpr int FMT_NIBBLE = 1;
constexpr int FMT_HUFFMAN = 2;
constexpr int FMT_HUFPAIR = 3;

constexpr uint32_t MAGIC = 0x4e363142u; // "B16N"
constexpr int HUF_LMAX = 10;
constexpr int HP_LP = 12;
constexpr int HP_MAX_PAIRS = 1 << HP_LP;
constexpr int CHUNK = 512;
constexpr int K_MAX = 4096;
constexpr int HEADER_BYTES = 256;
constexpr uint32_t FLAG_CHUNK_MAJOR = 1;
constexpr uint32_t FLAG_FRAG_ORDER = 2;

struct aux_header {
    uint32_t magic, format, K, R;
    uint64_t rows;
    uint64_t off_a, off_b, off_c, off_d;
    uint64_t n_a, n_b;
    uint32_t flags, pad_;
};
static_assert(sizeof(aux_header) == 80, "aux header is 80 bytes");

inline constexpr int pos_of(int l, int s) { return 128 * (s >> 2) + 4 * l + (s & 3); }

} // namespace bf16n
