// Host encoder of the BF16N format: BF16 bit patterns -> sign|mantissa plane + exponent "aux" buffer.
//
// Output is byte-for-byte what the reference encoder (core/src/encode.cpp:443-526) produces for the same input, so a
// tensor encoded here decodes with the reference kernels and the other way round; the layouts are documented in
// format.h.  The implementation is organised differently for throughput on large tensors:
//   * code lengths come from a boundary-counting package-merge (no per-item symbol lists): per level only the number
//     of leaves among the selected prefix is tracked, which gives the same lengths as the list form because leaves
//     keep their sorted order inside every merged level;
//   * bit streams are produced in two parallel passes over the units (sizes, then bits written in place into the final
//     aux buffer) instead of per-unit vectors that are concatenated afterwards;
//   * the plane is written directly in its final (lane-major, optionally chunk-major or fragment-order) position.
#include "encode.h"

#include <algorithm>
#include <atomic>
#include <cstring>
#include <stdexcept>
#include <string>
#include <thread>

namespace b16 {
namespace {

int host_threads() { return (int) std::max(1u, std::thread::hardware_concurrency()); }

// f(begin, end, thread) over [0, n) in contiguous grains, on all host threads (thread < host_threads())
template <typename F>
void parallel_ranges(int64_t n, int64_t grain, F && f) {
    const int64_t pieces = (n + grain - 1) / grain;
    const int nt = (int) std::min<int64_t>(host_threads(), pieces);
    if (nt <= 1) {
        if (n > 0) { f((int64_t) 0, n, 0); }
        return;
    }
    std::atomic<int64_t> next{0};
    std::vector<std::thread> pool;
    pool.reserve(nt);
    for (int t = 0; t < nt; t++) {
        pool.emplace_back([&, t] {
            for (int64_t p; (p = next.fetch_add(1)) < pieces;) { f(p * grain, std::min(n, (p + 1) * grain), t); }
        });
    }
    for (auto & th : pool) { th.join(); }
}

inline uint32_t expo(uint16_t v) { return (v >> 7) & 0xFFu; }
inline uint8_t sign_mant(uint16_t v) { return (uint8_t) (((v >> 15) << 7) | (v & 0x7F)); }

// fragment order: row and first column (inside a 16x16 tile) of register q of lane l (mma.m16n8k16 A operand)
inline void frag_rc(int l, int q, int & r, int & c) { r = (l >> 2) + 8 * (q & 1); c = 2 * (l & 3) + 8 * (q >> 1); }

[[noreturn]] void bad(const std::string & m) { throw std::invalid_argument("bf16n encode: " + m); }
void check(bool ok, const char * what) {
    if (!ok) { throw std::runtime_error(std::string("bf16n encode: check failed: ") + what); }
}

// ------------------------------------------------------------------ plane

// lane-major plane; unit_rows > 0: chunk-major inside units of unit_rows rows (chunk c of unit row r at (c*R + r)*512)
void write_plane(const uint16_t * w, int64_t rows, int64_t K, int unit_rows, uint8_t * sm) {
    const int64_t C = K / CHUNK;
    parallel_ranges(rows, 64, [&](int64_t r0, int64_t r1, int) {
        for (int64_t r = r0; r < r1; r++) {
            for (int64_t c = 0; c < C; c++) {
                const uint16_t * src = w + r * K + c * CHUNK;
                uint8_t * dst = unit_rows ? sm + (r / unit_rows) * unit_rows * K + (c * unit_rows + r % unit_rows) * CHUNK
                                          : sm + r * K + c * CHUNK;
                for (int j = 0; j < 4; j++) {
                    for (int l = 0; l < 32; l++) {
                        for (int t = 0; t < 4; t++) { dst[16 * l + 4 * j + t] = sign_mant(src[128 * j + 4 * l + t]); }
                    }
                }
            }
        }
    });
}

void write_plane_frag(const uint16_t * w, int64_t rows, int64_t K, uint8_t * sm) {
    parallel_ranges(rows / 16, 4, [&](int64_t b0, int64_t b1, int) {
        for (int64_t b = b0; b < b1; b++) {
            for (int64_t p = 0; p < K / 32; p++) {
                for (int l = 0; l < 32; l++) {
                    uint8_t * o = sm + b * 16 * K + p * 512 + l * 16;
                    for (int kk = 0; kk < 2; kk++) {
                        for (int q = 0; q < 4; q++) {
                            int r, c;
                            frag_rc(l, q, r, c);
                            const uint16_t * s = w + (b * 16 + r) * K + (2 * p + kk) * 16 + c;
                            o[8 * kk + 2 * q] = sign_mant(s[0]);
                            o[8 * kk + 2 * q + 1] = sign_mant(s[1]);
                        }
                    }
                }
            }
        }
    });
}

// ------------------------------------------------------------------ length-limited code lengths

// Package-merge with maximum length L over the non-zero frequencies. Tie rules (they decide which of two equally
// frequent symbols gets the longer code, hence the bytes): leaves are put in order by std::sort comparing weights only,
// starting from ascending symbol order; when a package and a leaf weigh the same the package comes first.
std::vector<uint8_t> code_lengths(const std::vector<uint64_t> & freq, int L) {
    struct leaf { uint64_t w; int sym; };
    std::vector<leaf> lv;
    for (int i = 0; i < (int) freq.size(); i++) {
        if (freq[i]) { lv.push_back({freq[i], i}); }
    }
    std::vector<uint8_t> len(freq.size(), 0);
    const size_t n = lv.size();
    if (n == 0) { return len; }
    if (n == 1) { len[lv[0].sym] = 1; return len; }
    std::sort(lv.begin(), lv.end(), [](const leaf & a, const leaf & b) { return a.w < b.w; });

    // level d holds the merged list's weights and, per item, whether it is a leaf
    std::vector<std::vector<uint64_t>> wt(L);
    std::vector<std::vector<uint8_t>> is_leaf(L);
    wt[0].resize(n);
    is_leaf[0].assign(n, 1);
    for (size_t i = 0; i < n; i++) { wt[0][i] = lv[i].w; }
    for (int d = 1; d < L; d++) {
        const std::vector<uint64_t> & prev = wt[d - 1];
        const size_t np = prev.size() / 2;
        wt[d].reserve(np + n);
        is_leaf[d].reserve(np + n);
        size_t a = 0, b = 0; // a: next package, b: next leaf
        while (a < np || b < n) {
            const bool take_pkg = a < np && (b >= n || !(lv[b].w < prev[2 * a] + prev[2 * a + 1]));
            if (take_pkg) {
                wt[d].push_back(prev[2 * a] + prev[2 * a + 1]);
                is_leaf[d].push_back(0);
                a++;
            } else {
                wt[d].push_back(lv[b].w);
                is_leaf[d].push_back(1);
                b++;
            }
        }
    }
    // walk back: the first m items of a level contain c leaves (the c lightest) and m - c packages, i.e. the first
    // 2(m - c) items of the level below
    size_t m = 2 * n - 2;
    for (int d = L - 1; d >= 0; d--) {
        check(m <= wt[d].size(), "package-merge prefix");
        size_t c = 0;
        for (size_t i = 0; i < m; i++) { c += is_leaf[d][i]; }
        for (size_t j = 0; j < c; j++) { len[lv[j].sym]++; }
        m = 2 * (m - c);
    }
    return len;
}

// canonical codes: ascending by (length, symbol)
std::vector<uint32_t> canonical_codes(const std::vector<uint8_t> & len, int L) {
    std::vector<uint32_t> code(len.size(), 0);
    uint32_t next = 0;
    for (int l = 1; l <= L; l++) {
        for (size_t s = 0; s < len.size(); s++) {
            if (len[s] == l) { code[s] = next++; }
        }
        next <<= 1;
    }
    return code;
}

// MSB-first bit sink writing whole little-endian u32 words in place
struct bit_sink {
    uint32_t * out;
    uint64_t acc = 0;
    int nb = 0;
    inline void put(uint32_t code, int len) {
        acc = (acc << len) | code;
        nb += len;
        if (nb >= 32) {
            nb -= 32;
            *out++ = (uint32_t) (acc >> nb);
            acc &= (1ull << nb) - 1;
        }
    }
    inline void finish() { if (nb) { *out++ = (uint32_t) (acc << (32 - nb)); } }
};

template <typename T> void put_at(std::vector<uint8_t> & buf, uint64_t off, const T * src, size_t n) {
    if (n) { memcpy(buf.data() + off, src, n * sizeof(T)); }
}

// ------------------------------------------------------------------ NIBBLE

std::vector<uint8_t> encode_nibble(const uint16_t * w, int64_t rows, int64_t K, uint8_t * plane) {
    const int64_t C = K / CHUNK;
    constexpr int64_t BLK = 256;
    const int64_t nblk = (rows + BLK - 1) / BLK;
    std::vector<std::vector<uint32_t>> esc_blk(nblk);
    std::vector<uint32_t> esc_off(rows + 1, 0);
    AuxHeader h = {};
    h.magic = MAGIC; h.format = FMT_NIBBLE; h.K = (uint32_t) K; h.rows = (uint64_t) rows;
    h.off_a = HEADER_BYTES;
    h.off_b = h.off_a + (uint64_t) rows * K / 2;
    h.off_c = h.off_b + (uint64_t) rows * 16;
    h.off_d = h.off_c + (uint64_t) (rows + 1) * 4;
    std::vector<uint8_t> head(h.off_d, 0); // everything but the escape list, whose size is known last
    parallel_ranges(nblk, 1, [&](int64_t b0, int64_t b1, int) {
        for (int64_t b = b0; b < b1; b++) {
            for (int64_t r = b * BLK; r < std::min(rows, (b + 1) * BLK); r++) {
                const uint16_t * row = w + r * K;
                int hist[256] = {0};
                for (int64_t k = 0; k < K; k++) { hist[expo(row[k])]++; }
                // table: entry 0 = exponent 0, then the 15 most frequent exponents in 1..127 (ties: smaller first)
                int order[127];
                for (int i = 0; i < 127; i++) { order[i] = i + 1; }
                std::stable_sort(order, order + 127, [&](int a, int c) { return hist[a] > hist[c]; });
                int code_of[256];
                std::fill(code_of, code_of + 256, -1);
                code_of[0] = 0;
                uint8_t * tab = head.data() + h.off_b + r * 16;
                for (int i = 0, n = 1; i < 127 && n < 16 && hist[order[i]] > 0; i++, n++) {
                    tab[n] = (uint8_t) order[i];
                    code_of[order[i]] = n;
                }
                uint32_t n_esc = 0;
                for (int64_t c = 0; c < C; c++) {
                    uint8_t * codes = head.data() + h.off_a + (r * C + c) * 256;
                    uint8_t * pl = plane + r * K + c * CHUNK;
                    for (int l = 0; l < 32; l++) {
                        uint64_t packed = 0;
                        for (int s = 0; s < 16; s++) {
                            const int col = (int) (c * CHUNK) + chunk_col(l, s);
                            const uint16_t v = row[col];
                            int code = code_of[expo(v)];
                            uint8_t sm = sign_mant(v);
                            if (code < 0) { // escape: exact value in the list, slot reads as +0
                                esc_blk[b].push_back((uint32_t) col | ((uint32_t) sm << 12) | (expo(v) << 20));
                                n_esc++;
                                code = 0;
                                sm = 0;
                            }
                            packed |= (uint64_t) code << (4 * s);
                            pl[16 * l + s] = sm;
                        }
                        memcpy(codes + 8 * l, &packed, 8);
                    }
                }
                esc_off[r + 1] = n_esc; // per-row count; prefix-summed below
            }
        }
    });
    for (int64_t r = 0; r < rows; r++) { esc_off[r + 1] += esc_off[r]; }
    h.n_a = esc_off[rows];
    std::vector<uint8_t> aux(h.off_d + std::max<uint64_t>(h.n_a, 1) * 4, 0);
    memcpy(aux.data(), head.data(), head.size());
    memcpy(aux.data(), &h, sizeof h);
    put_at(aux, h.off_c, esc_off.data(), esc_off.size());
    uint64_t o = h.off_d;
    for (auto & v : esc_blk) {
        put_at(aux, o, v.data(), v.size());
        o += v.size() * 4;
    }
    return aux;
}

// ------------------------------------------------------------------ HUFFMAN / HUFPAIR streams

} // namespace

Encoded encode(const uint16_t * w, int64_t rows, int64_t K, int format, int R, bool chunk_major, bool frag_order) {
    if (K % CHUNK != 0 || K < CHUNK || K > K_MAX) { bad("K must be a multiple of 512 in [512, 4096], got " + std::to_string(K)); }
    if (rows <= 0) { bad("rows must be positive"); }
    if (format == FMT_NIBBLE) {
        if (R != 0 || chunk_major || frag_order) { bad("NIBBLE takes R = 0 and no chunk-major or fragment-order layout"); }
    } else if (format == FMT_HUFFMAN || format == FMT_HUFPAIR) {
        if (R != 1 && R != 2 && R != 4 && R != 8 && R != 16) { bad("R must be one of 1, 2, 4, 8, 16, got " + std::to_string(R)); }
        if (rows % R != 0) { bad("rows (" + std::to_string(rows) + ") must be a multiple of R (" + std::to_string(R) + ")"); }
        if (format == FMT_HUFFMAN && chunk_major) { bad("chunk-major units exist only for HUFPAIR"); }
        if (chunk_major && (K == CHUNK || (R != 4 && R != 8 && R != 16))) { bad("chunk-major units need K > 512 and R in {4, 8, 16}"); }
        if (frag_order && (format != FMT_HUFPAIR || chunk_major || R != 16)) {
            bad("fragment order exists only for HUFPAIR with R = 16, without chunk-major units");
        }
    } else {
        bad("unknown format " + std::to_string(format));
    }

    Encoded out;
    out.plane.resize((size_t) (rows * K));
    out.R = format == FMT_NIBBLE ? 0 : R;
    if (format == FMT_NIBBLE) {
        out.aux = encode_nibble(w, rows, K, out.plane.data());
        out.format = FMT_NIBBLE;
        return out;
    }

    const int64_t C = K / CHUNK;
    bool pair = format == FMT_HUFPAIR;
    std::vector<uint8_t> len;
    std::vector<uint32_t> code;
    if (pair) {
        // histogram of (even, odd) exponent pairs
        std::vector<uint64_t> freq(65536, 0);
        std::vector<std::vector<uint32_t>> part(host_threads()); // one private histogram per thread
        parallel_ranges(rows, std::max<int64_t>(1, (1 << 22) / K), [&](int64_t r0, int64_t r1, int t) {
            std::vector<uint32_t> & hgram = part[t];
            if (hgram.empty()) { hgram.assign(65536, 0); }
            for (int64_t i = r0 * K; i < r1 * K; i += 2) { hgram[expo(w[i]) | expo(w[i + 1]) << 8]++; }
        });
        for (auto & hgram : part) {
            for (size_t i = 0; i < hgram.size(); i++) { freq[i] += hgram[i]; }
        }
        int nsym = 0;
        for (uint64_t f : freq) { nsym += f != 0; }
        if (nsym > HP_MAX_PAIRS) {
            pair = false; // more distinct pairs than the pair table holds: single-exponent code, no special layout
        } else {
            len = code_lengths(freq, HP_LMAX);
            code = canonical_codes(len, HP_LMAX);
        }
    }
    if (!pair) {
        std::vector<uint64_t> freq(256, 0);
        for (int64_t i = 0; i < rows * K; i++) { freq[expo(w[i])]++; }
        len = code_lengths(freq, HUF_LMAX);
        code = canonical_codes(len, HUF_LMAX);
        chunk_major = false;
        frag_order = false;
    }
    out.format = pair ? FMT_HUFPAIR : FMT_HUFFMAN;

    // decode table: every slot whose top bits equal a code holds that code's payload
    const int LM = pair ? HP_LMAX : HUF_LMAX;
    std::vector<uint32_t> lut((size_t) 1 << LM, 0);
    std::vector<uint32_t> cl(len.size()); // code << 4 | len, one load per symbol in the packing loops
    for (size_t s = 0; s < len.size(); s++) {
        cl[s] = code[s] << 4 | len[s];
        if (!len[s]) { continue; }
        const uint32_t payload = pair ? ((uint32_t) (s >> 8) << 23 | (uint32_t) (s & 0xFF) << 7 | len[s])
                                      : ((uint32_t) len[s] | (uint32_t) s << 7);
        const uint32_t lo = code[s] << (LM - len[s]), hi = (code[s] + 1) << (LM - len[s]);
        std::fill(lut.begin() + lo, lut.begin() + hi, payload);
    }

    const int64_t units = frag_order ? rows / 16 * C : rows / R;
    // symbols of lane l of unit u, in stream order
    auto for_lane = [&](int64_t u, int l, auto && emit) {
        if (!pair) {
            for (int64_t r = u * R; r < (u + 1) * R; r++) {
                for (int64_t c = 0; c < C; c++) {
                    const uint16_t * p = w + r * K + c * CHUNK;
                    for (int s = 0; s < 16; s++) { emit(expo(p[chunk_col(l, s)])); }
                }
            }
        } else if (frag_order) {
            const int64_t band = u / C, slab = u % C;
            for (int64_t kt = slab * 32; kt < slab * 32 + 32; kt++) {
                for (int q = 0; q < 4; q++) {
                    int r, c;
                    frag_rc(l, q, r, c);
                    const uint16_t * p = w + (band * 16 + r) * K + kt * 16 + c;
                    emit(expo(p[0]) | expo(p[1]) << 8);
                }
            }
        } else {
            for (int64_t o = 0; o < R * C; o++) {
                const int64_t r = u * R + (chunk_major ? o % R : o / C), c = chunk_major ? o / R : o % C;
                const uint16_t * p = w + r * K + c * CHUNK;
                for (int s = 0; s < 16; s += 2) {
                    const uint16_t * q = p + chunk_col(l, s);
                    emit(expo(q[0]) | expo(q[1]) << 8);
                }
            }
        }
    };

    // pass 1: words per lane stream
    std::vector<uint32_t> lane_words((size_t) units * 32);
    parallel_ranges(units, 8, [&](int64_t u0, int64_t u1, int) {
        for (int64_t u = u0; u < u1; u++) {
            for (int l = 0; l < 32; l++) {
                uint64_t bits = 0;
                for_lane(u, l, [&](uint32_t sym) { bits += cl[sym] & 15u; });
                lane_words[u * 32 + l] = (uint32_t) ((bits + 31) / 32);
            }
        }
    });
    std::vector<uint64_t> unit_start(units + 1, 0);
    for (int64_t u = 0; u < units; u++) {
        uint64_t n = 0;
        for (int l = 0; l < 32; l++) { n += lane_words[u * 32 + l]; }
        unit_start[u + 1] = unit_start[u] + n;
    }
    const uint64_t n_words = unit_start[units];
    const int tail = pair ? HP_TAIL_WORDS : HUF_TAIL_WORDS;
    check(n_words + tail < (1ull << 32), "stream words fit 32 bits");

    AuxHeader h = {};
    h.magic = MAGIC; h.format = (uint32_t) out.format; h.K = (uint32_t) K; h.R = (uint32_t) R; h.rows = (uint64_t) rows;
    h.off_a = HEADER_BYTES;
    h.off_b = h.off_a + lut.size() * 4;
    uint64_t stream_off;
    if (pair) {
        h.off_c = h.off_b + (uint64_t) units * 4;                       // u16 lane offsets relative to the unit
        h.off_d = (h.off_c + (uint64_t) units * 32 * 2 + 15) & ~15ull;  // stream, 16-byte aligned
        h.flags = (chunk_major ? FLAG_CHUNK_MAJOR : 0) | (frag_order ? FLAG_FRAG_ORDER : 0);
        stream_off = h.off_d;
    } else {
        h.off_c = h.off_b + (uint64_t) units * 32 * 4;                  // stream
        stream_off = h.off_c;
    }
    h.n_a = (uint64_t) units; h.n_b = n_words;
    out.aux.assign(stream_off + (n_words + tail) * 4, 0);
    memcpy(out.aux.data(), &h, sizeof h);
    put_at(out.aux, h.off_a, lut.data(), lut.size());

    // offsets
    if (pair) {
        uint32_t * ub = (uint32_t *) (out.aux.data() + h.off_b);
        uint16_t * lr = (uint16_t *) (out.aux.data() + h.off_c);
        for (int64_t u = 0; u < units; u++) {
            ub[u] = (uint32_t) unit_start[u];
            uint32_t rel = 0;
            for (int l = 0; l < 32; l++) {
                check(rel <= 0xFFFF, "lane offset fits 16 bits");
                lr[u * 32 + l] = (uint16_t) rel;
                rel += lane_words[u * 32 + l];
            }
        }
    } else {
        uint32_t * lo = (uint32_t *) (out.aux.data() + h.off_b);
        for (int64_t u = 0; u < units; u++) {
            uint64_t at = unit_start[u];
            for (int l = 0; l < 32; l++) {
                lo[u * 32 + l] = (uint32_t) at;
                at += lane_words[u * 32 + l];
            }
        }
    }

    // pass 2: the bits, in place
    uint32_t * stream = (uint32_t *) (out.aux.data() + stream_off);
    parallel_ranges(units, 8, [&](int64_t u0, int64_t u1, int) {
        for (int64_t u = u0; u < u1; u++) {
            uint32_t * at = stream + unit_start[u];
            for (int l = 0; l < 32; l++) {
                bit_sink sink{at};
                for_lane(u, l, [&](uint32_t sym) { sink.put(cl[sym] >> 4, (int) (cl[sym] & 15u)); });
                sink.finish();
                at += lane_words[u * 32 + l];
            }
        }
    });

    if (h.flags & FLAG_FRAG_ORDER) {
        write_plane_frag(w, rows, K, out.plane.data());
    } else {
        write_plane(w, rows, K, (h.flags & FLAG_CHUNK_MAJOR) ? R : 0, out.plane.data());
    }
    return out;
}

} // namespace b16
