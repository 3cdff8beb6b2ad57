// BF16N storage format constants shared by the host encoder and the sm_100a kernels of this library.
// The byte layout is the reference project's (core/include/bf16n/format.h:12-51, docs/FORMAT.md): buffers produced by
// either encoder decode with either decoder.
#pragma once

#include <cstdint>

namespace b16 {

constexpr int FMT_NIBBLE = 1;  // 4-bit code per weight into a per-row 16-entry exponent table, escapes per row
constexpr int FMT_HUFFMAN = 2; // single-exponent canonical Huffman, codes <= 10 bits
constexpr int FMT_HUFPAIR = 3; // canonical Huffman over pairs of adjacent exponents, codes <= 12 bits

constexpr uint32_t MAGIC = 0x4e363142u; // "B16N"
constexpr int HUF_LMAX = 10;
constexpr int HP_LMAX = 12;
constexpr int HP_MAX_PAIRS = 1 << HP_LMAX;
constexpr int CHUNK = 512; // weights per lane-major chunk
constexpr int K_MAX = 4096;
constexpr int HEADER_BYTES = 256;
constexpr int HP_TAIL_WORDS = 32;  // zero words after the last HUFPAIR stream word (decoder lookahead)
constexpr int HUF_TAIL_WORDS = 16; // same for HUFFMAN

constexpr uint32_t FLAG_CHUNK_MAJOR = 1;
constexpr uint32_t FLAG_FRAG_ORDER = 2;

// First 80 of the 256 header bytes of every aux buffer; offsets are bytes from the aux start.
//   NIBBLE : off_a codes (rows*K/2) | off_b row tables (rows*16) | off_c esc_off u32[rows+1] | off_d escapes u32; n_a = #escapes
//   HUFFMAN: off_a LUT u32[1024] | off_b lane word offsets u32[units*32] | off_c stream; n_a units, n_b words
//   HUFPAIR: off_a LUT u32[4096] | off_b unit base u32[units] | off_c lane offsets u16[units*32] | off_d stream (16-B aligned)
struct AuxHeader {
    uint32_t magic, format, K, R;
    uint64_t rows;
    uint64_t off_a, off_b, off_c, off_d;
    uint64_t n_a, n_b;
    uint32_t flags, pad_;
};
static_assert(sizeof(AuxHeader) == 80, "aux header is 80 bytes");

// Column (inside a 512-weight chunk) of slot s (0..15) of lane l (0..31); the slot is stored at plane byte 16*l + s.
constexpr int chunk_col(int lane, int slot) { return 128 * (slot >> 2) + 4 * lane + (slot & 3); }

} // namespace b16
