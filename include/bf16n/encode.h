// bf16n::encode with the reference's signature (core/include/bf16n/encode.h:12-26) over the C ABI.
#pragma once

#include "../bf16n_c.h"
#include "format.h"

#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

namespace bf16n {

namespace detail {
inline void raise(int rc) {
    if (rc == BF16N_OK) { return; }
    const std::string msg = bf16n_last_error();
    if (rc == BF16N_EINVAL) { throw std::invalid_argument(msg); }
    throw std::runtime_error(msg);
}
} // namespace detail

struct encoded {
    std::vector<uint8_t> plane; // sign|mantissa byte per weight (rows * K)
    std::vector<uint8_t> aux;   // header + exponent data
    int format;                 // the format produced (FMT_HUFPAIR may fall back to FMT_HUFFMAN)
    int R;                      // rows per unit (0 for FMT_NIBBLE)
};

inline encoded encode(const uint16_t * w, int64_t rows, int64_t K, int format, int R, bool chunk_major, bool frag_order = false) {
    bf16n_encoded * h = nullptr;
    detail::raise(bf16n_encode(w, rows, K, format, R, chunk_major, frag_order, &h));
    encoded e;
    size_t n = 0;
    const uint8_t * p = bf16n_encoded_plane(h, &n);
    e.plane.assign(p, p + n);
    p = bf16n_encoded_aux(h, &n);
    e.aux.assign(p, p + n);
    e.format = bf16n_encoded_format(h);
    e.R = bf16n_encoded_R(h);
    bf16n_encoded_free(h);
    return e;
}

} // namespace bf16n
