// BF16N CPU oracle.  TEST INFRASTRUCTURE ONLY: nothing the library ships links, imports or calls this file; only the
// tests, the smoke check and the CPU-baseline leg of the benchmark load it, and only as the checker / the timed CPU arm.
//
// It restates, in straight single-purpose C++ (extern "C" entry points, no dependencies), the algorithm of the
// reference project's BF16N path:
//   * the host encoder            core/src/encode.cpp:48-62 (plane), :94-180 (NIBBLE), :182-218 (package-merge),
//                                 :220-312 (HUFFMAN), :321-439 (HUFPAIR), :443-526 (argument rules, escape zeroing,
//                                 chunk-major plane permutation)
//   * the independent decoder     core/tests/test_encode.cpp:36-164 (bit reader, plane addressing, all formats)
//   * the GEMV reference          FP64 dot products over the exact weights (engines/llamacpp/bench/moe_prefill.cpp:172-202)
//                                 and an FP32 emulation of the kernels' summation order (core/include/bf16n/kernels.cuh:
//                                 498-535 row-major, :119-125 warp butterfly, :958-986 chunk-major, :178-186 NIBBLE escapes)
// Parity is pinned: tests/test_oracle_pin.py checks every encoder output byte for byte against the reference encoder
// itself (compiled from its own sources into oracle/_ref by oracle/Makefile) and against the committed golden vectors.
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <vector>

namespace {

constexpr uint32_t kMagic = 0x4e363142u;
constexpr int kNibble = 1, kHuffman = 2, kHufpair = 3;
constexpr int kHufL = 10, kPairL = 12;
constexpr uint32_t kFlagCm = 1, kFlagFo = 2;

struct Header { // format.h:41-47
    uint32_t magic, format, K, R;
    uint64_t rows, off_a, off_b, off_c, off_d, n_a, n_b;
    uint32_t flags, pad;
};
static_assert(sizeof(Header) == 80, "header");

inline int pos_of(int l, int s) { return 128 * (s >> 2) + 4 * l + (s & 3); } // format.h:51
inline int expo(uint16_t v) { return (v >> 7) & 0xFF; }
inline uint8_t smbyte(uint16_t v) { return (uint8_t) (((v >> 15) << 7) | (v & 0x7F)); }
inline uint16_t join(uint8_t sm, int ex) { return (uint16_t) (((sm >> 7) << 15) | (ex << 7) | (sm & 0x7F)); }

// fragment order: first weight of register q of lane l in a 16x16 tile (encode.cpp:66-69)
inline void fo_pair(int l, int q, int & r, int & c) { r = (l >> 2) + 8 * (q & 1); c = 2 * (l & 3) + 8 * (q >> 1); }

// ------------------------------------------------------------------ package-merge (encode.cpp:182-218)
// Items carry explicit symbol lists, as the reference does; ties: leaves are ordered by std::sort on the weight
// alone from symbol-ascending input, packages precede leaves of equal weight (std::merge takes the first range on ties).
std::vector<int> limited_lengths(const std::vector<uint64_t> & freq, int L) {
    struct item { uint64_t w; std::vector<int> s; };
    std::vector<item> leaves;
    for (int i = 0; i < (int) freq.size(); i++) {
        if (freq[i]) { leaves.push_back({freq[i], {i}}); }
    }
    std::vector<int> len(freq.size(), 0);
    if (leaves.size() == 1) { len[leaves[0].s[0]] = 1; return len; }
    auto lt = [](const item & a, const item & b) { return a.w < b.w; };
    std::sort(leaves.begin(), leaves.end(), lt);
    std::vector<item> cur = leaves;
    for (int d = 1; d < L; d++) {
        std::vector<item> pk, mg;
        for (size_t i = 0; i + 1 < cur.size(); i += 2) {
            item m{cur[i].w + cur[i + 1].w, cur[i].s};
            m.s.insert(m.s.end(), cur[i + 1].s.begin(), cur[i + 1].s.end());
            pk.push_back(std::move(m));
        }
        std::merge(pk.begin(), pk.end(), leaves.begin(), leaves.end(), std::back_inserter(mg), lt);
        cur.swap(mg);
    }
    for (size_t i = 0; i < 2 * leaves.size() - 2; i++) {
        for (int s : cur[i].s) { len[s]++; }
    }
    return len;
}

std::vector<uint32_t> canonical(const std::vector<int> & len, int L) { // encode.cpp:239-250 / 348-359
    std::vector<uint32_t> code(len.size(), 0);
    uint32_t c = 0;
    for (int l = 1; l <= L; l++) {
        for (size_t s = 0; s < len.size(); s++) {
            if (len[s] == l) { code[s] = c++; }
        }
        c <<= 1;
    }
    return code;
}

struct BitWriter { // MSB-first into u32 words (encode.cpp:266-284)
    std::vector<uint32_t> & out;
    uint64_t acc = 0;
    int nb = 0;
    void put(uint32_t code, int len) {
        acc = (acc << len) | code;
        nb += len;
        if (nb >= 32) {
            out.push_back((uint32_t) (acc >> (nb - 32)));
            nb -= 32;
            acc &= nb ? ((1ull << nb) - 1) : 0;
        }
    }
    void flush() { if (nb) { out.push_back((uint32_t) (acc << (32 - nb))); } }
};

void plane_lane_major(const uint16_t * w, int64_t rows, int64_t K, uint8_t * sm) { // encode.cpp:48-62
    for (int64_t r = 0; r < rows; r++) {
        for (int64_t c = 0; c < K / 512; c++) {
            for (int l = 0; l < 32; l++) {
                for (int s = 0; s < 16; s++) {
                    sm[r * K + c * 512 + 16 * l + s] = smbyte(w[r * K + c * 512 + pos_of(l, s)]);
                }
            }
        }
    }
}

void plane_frag_order(const uint16_t * w, int64_t rows, int64_t K, uint8_t * sm) { // encode.cpp:73-92
    for (int64_t b = 0; b < rows / 16; b++) {
        for (int64_t p = 0; p < K / 32; p++) {
            for (int l = 0; l < 32; l++) {
                uint8_t * o = sm + b * 16 * K + p * 512 + l * 16;
                for (int kk = 0; kk < 2; kk++) {
                    for (int q = 0; q < 4; q++) {
                        int r, c;
                        fo_pair(l, q, r, c);
                        const int64_t i = (b * 16 + r) * K + (2 * p + kk) * 16 + c;
                        o[8 * kk + 2 * q] = smbyte(w[i]);
                        o[8 * kk + 2 * q + 1] = smbyte(w[i + 1]);
                    }
                }
            }
        }
    }
}

std::vector<uint8_t> enc_nibble(const uint16_t * w, int64_t rows, int64_t K) { // encode.cpp:94-180
    const int64_t C = K / 512;
    std::vector<uint8_t> nib(rows * K / 2), lut(rows * 16, 0);
    std::vector<uint32_t> esc, esc_off(rows + 1, 0);
    for (int64_t r = 0; r < rows; r++) {
        const uint16_t * row = w + r * K;
        int hist[256] = {0}, order[256], code_of[256];
        for (int64_t k = 0; k < K; k++) { hist[expo(row[k])]++; }
        for (int i = 0; i < 256; i++) { order[i] = i; code_of[i] = -1; }
        std::sort(order, order + 256, [&](int a, int b) { return hist[a] > hist[b] || (hist[a] == hist[b] && a < b); });
        code_of[0] = 0;
        int n = 1;
        for (int i = 0; i < 256 && n < 16; i++) {
            const int x = order[i];
            if (hist[x] == 0) { break; }
            if (x == 0 || x >= 128) { continue; }
            lut[r * 16 + n] = (uint8_t) x;
            code_of[x] = n++;
        }
        for (int64_t c = 0; c < C; c++) {
            for (int l = 0; l < 32; l++) {
                uint32_t nw[2] = {0, 0};
                for (int s = 0; s < 16; s++) {
                    const int col = (int) (c * 512 + pos_of(l, s));
                    const uint16_t v = row[col];
                    int code = code_of[expo(v)];
                    if (code < 0) {
                        esc.push_back((uint32_t) col | ((uint32_t) smbyte(v) << 12) | ((uint32_t) expo(v) << 20));
                        code = 0;
                    }
                    nw[s >> 3] |= (uint32_t) code << (4 * (s & 7));
                }
                memcpy(&nib[(r * C + c) * 256 + 8 * l], nw, 8);
            }
        }
        esc_off[r + 1] = (uint32_t) esc.size();
    }
    Header h = {};
    h.magic = kMagic; h.format = kNibble; h.K = (uint32_t) K; h.rows = rows;
    h.off_a = 256;
    h.off_b = h.off_a + nib.size();
    h.off_c = h.off_b + lut.size();
    h.off_d = h.off_c + esc_off.size() * 4;
    h.n_a = esc.size();
    std::vector<uint8_t> aux(h.off_d + std::max<uint64_t>(esc.size(), 1) * 4, 0);
    memcpy(aux.data(), &h, sizeof h);
    memcpy(aux.data() + h.off_a, nib.data(), nib.size());
    memcpy(aux.data() + h.off_b, lut.data(), lut.size());
    memcpy(aux.data() + h.off_c, esc_off.data(), esc_off.size() * 4);
    if (!esc.empty()) { memcpy(aux.data() + h.off_d, esc.data(), esc.size() * 4); }
    return aux;
}

std::vector<uint8_t> enc_huffman(const uint16_t * w, int64_t rows, int64_t K, int R) { // encode.cpp:220-312
    const int64_t C = K / 512, units = rows / R;
    std::vector<uint64_t> freq(256, 0);
    for (int64_t i = 0; i < rows * K; i++) { freq[expo(w[i])]++; }
    const std::vector<int> len = limited_lengths(freq, kHufL);
    const std::vector<uint32_t> code = canonical(len, kHufL);
    std::vector<uint32_t> lut(1 << kHufL, 0);
    for (int s = 0; s < 256; s++) {
        if (!len[s]) { continue; }
        for (uint32_t i = code[s] << (kHufL - len[s]); i < (code[s] + 1) << (kHufL - len[s]); i++) {
            lut[i] = (uint32_t) len[s] | ((uint32_t) s << 7);
        }
    }
    std::vector<uint32_t> stream, lane_off(units * 32);
    for (int64_t u = 0; u < units; u++) {
        for (int l = 0; l < 32; l++) {
            lane_off[u * 32 + l] = (uint32_t) stream.size();
            BitWriter bw{stream};
            for (int64_t r = u * R; r < (u + 1) * R; r++) {
                for (int64_t c = 0; c < C; c++) {
                    for (int s = 0; s < 16; s++) {
                        const int e = expo(w[r * K + c * 512 + pos_of(l, s)]);
                        bw.put(code[e], len[e]);
                    }
                }
            }
            bw.flush();
        }
    }
    Header h = {};
    h.magic = kMagic; h.format = kHuffman; h.K = (uint32_t) K; h.R = (uint32_t) R; h.rows = rows;
    h.off_a = 256;
    h.off_b = h.off_a + lut.size() * 4;
    h.off_c = h.off_b + lane_off.size() * 4;
    h.n_a = units; h.n_b = stream.size();
    std::vector<uint8_t> aux(h.off_c + (stream.size() + 16) * 4, 0);
    memcpy(aux.data(), &h, sizeof h);
    memcpy(aux.data() + h.off_a, lut.data(), lut.size() * 4);
    memcpy(aux.data() + h.off_b, lane_off.data(), lane_off.size() * 4);
    memcpy(aux.data() + h.off_c, stream.data(), stream.size() * 4);
    return aux;
}

std::vector<uint8_t> enc_hufpair(const uint16_t * w, int64_t rows, int64_t K, int R, bool cm, bool fo) { // encode.cpp:321-439
    const int64_t C = K / 512, units = fo ? rows / 16 * C : rows / R;
    std::vector<uint64_t> freq(65536, 0);
    for (int64_t i = 0; i < rows * K; i += 2) { freq[expo(w[i]) | expo(w[i + 1]) << 8]++; }
    int nsym = 0;
    for (uint64_t f : freq) { nsym += f != 0; }
    if (nsym > (1 << kPairL)) { return {}; }
    const std::vector<int> len = limited_lengths(freq, kPairL);
    const std::vector<uint32_t> code = canonical(len, kPairL);
    std::vector<uint32_t> lut(1 << kPairL, 0);
    for (int s = 0; s < 65536; s++) {
        if (!len[s]) { continue; }
        for (uint32_t i = code[s] << (kPairL - len[s]); i < (code[s] + 1) << (kPairL - len[s]); i++) {
            lut[i] = ((uint32_t) (s >> 8) << 23) | ((uint32_t) (s & 0xFF) << 7) | (uint32_t) len[s];
        }
    }
    std::vector<uint32_t> stream, unit_base(units);
    std::vector<uint16_t> lane_rel(units * 32);
    for (int64_t u = 0; u < units; u++) {
        unit_base[u] = (uint32_t) stream.size();
        for (int l = 0; l < 32; l++) {
            const uint64_t rel = stream.size() - unit_base[u];
            if (rel > 0xFFFF) { abort(); }
            lane_rel[u * 32 + l] = (uint16_t) rel;
            BitWriter bw{stream};
            auto put = [&](int64_t i) { const int sym = expo(w[i]) | expo(w[i + 1]) << 8; bw.put(code[sym], len[sym]); };
            if (fo) {
                const int64_t band = u / C, slab = u % C;
                for (int64_t kt = slab * 32; kt < slab * 32 + 32; kt++) {
                    for (int q = 0; q < 4; q++) {
                        int r, c;
                        fo_pair(l, q, r, c);
                        put((band * 16 + r) * K + kt * 16 + c);
                    }
                }
            } else {
                for (int64_t o = 0; o < R * C; o++) {
                    const int64_t r = u * R + (cm ? o % R : o / C), c = cm ? o / R : o % C;
                    for (int s = 0; s < 16; s += 2) { put(r * K + c * 512 + pos_of(l, s)); }
                }
            }
            bw.flush();
        }
    }
    Header h = {};
    h.magic = kMagic; h.format = kHufpair; h.K = (uint32_t) K; h.R = (uint32_t) R; h.rows = rows;
    h.off_a = 256;
    h.off_b = h.off_a + lut.size() * 4;
    h.off_c = h.off_b + unit_base.size() * 4;
    h.off_d = (h.off_c + lane_rel.size() * 2 + 15) & ~15ull;
    h.n_a = units; h.n_b = stream.size();
    h.flags = (cm ? kFlagCm : 0) | (fo ? kFlagFo : 0);
    std::vector<uint8_t> aux(h.off_d + (stream.size() + 32) * 4, 0);
    memcpy(aux.data(), &h, sizeof h);
    memcpy(aux.data() + h.off_a, lut.data(), lut.size() * 4);
    memcpy(aux.data() + h.off_b, unit_base.data(), unit_base.size() * 4);
    memcpy(aux.data() + h.off_c, lane_rel.data(), lane_rel.size() * 2);
    memcpy(aux.data() + h.off_d, stream.data(), stream.size() * 4);
    return aux;
}

// ------------------------------------------------------------------ decoder (test_encode.cpp:36-164)
struct BitReader {
    const uint8_t * base;
    uint64_t word;
    uint64_t acc = 0;
    int n = 0;
    uint32_t peek(int k) {
        while (n < k) {
            uint32_t v;
            memcpy(&v, base + 4 * word++, 4);
            acc = (acc << 32) | v;
            n += 32;
        }
        return (uint32_t) ((acc >> (n - k)) & ((1ull << k) - 1));
    }
    void skip(int k) { n -= k; acc &= n ? ((1ull << n) - 1) : 0; }
};

template <typename T> T rd(const uint8_t * p) { T v; memcpy(&v, p, sizeof v); return v; }

// exponents of units [u0, u1) into ex (row-major, row r at (r - row0) * K), from the aux streams only
void decode_exponents_hp(const uint8_t * aux, const Header & h, uint64_t u0, uint64_t u1, uint8_t * ex, int64_t row0 = 0) {
    const int64_t K = h.K, C = K / 512;
    const bool cm = h.flags & kFlagCm, fo = h.flags & kFlagFo;
    for (uint64_t u = u0; u < u1; u++) {
        const uint32_t ub = rd<uint32_t>(aux + h.off_b + 4 * u);
        for (int l = 0; l < 32; l++) {
            BitReader bs{aux + h.off_d, (uint64_t) ub + rd<uint16_t>(aux + h.off_c + 2 * (u * 32 + l))};
            auto take = [&](int64_t i0, int64_t i1) {
                const uint32_t v = rd<uint32_t>(aux + h.off_a + 4 * bs.peek(kPairL));
                bs.skip((int) (v & 0x7F));
                ex[i0] = (uint8_t) ((v >> 7) & 0xFF);
                ex[i1] = (uint8_t) ((v >> 23) & 0xFF);
            };
            if (fo) {
                const int64_t band = (int64_t) u / C, kt0 = (int64_t) (u % C) * 32;
                for (int64_t kt = kt0; kt < kt0 + 32; kt++) {
                    for (int q = 0; q < 4; q++) {
                        int r, c;
                        fo_pair(l, q, r, c);
                        const int64_t i = (band * 16 + r - row0) * K + kt * 16 + c;
                        take(i, i + 1);
                    }
                }
            } else {
                for (int64_t o = 0; o < (int64_t) h.R * C; o++) {
                    const int64_t r = u * h.R + (cm ? o % h.R : o / C), c = cm ? o / h.R : o % C;
                    for (int s = 0; s < 16; s += 2) {
                        take((r - row0) * K + c * 512 + pos_of(l, s), (r - row0) * K + c * 512 + pos_of(l, s + 1));
                    }
                }
            }
        }
    }
}

uint8_t sm_at(const uint8_t * plane, int64_t K, int R, int64_t r, int64_t col, bool cm, bool fo) { // test_encode.cpp:61-83
    if (fo) {
        const int64_t p = col / 32, kk = (col / 16) % 2, rr = r % 16, cc = col % 16;
        for (int l = 0; l < 32; l++) {
            for (int q = 0; q < 4; q++) {
                int rq, cq;
                fo_pair(l, q, rq, cq);
                if (rq == rr && (cc == cq || cc == cq + 1)) {
                    return plane[(r / 16) * 16 * K + p * 512 + 16 * l + 8 * kk + 2 * q + (cc - cq)];
                }
            }
        }
        return 0;
    }
    const int64_t c = col / 512, p = col % 512;
    const int64_t in_chunk = 16 * ((p % 128) / 4) + 4 * (p / 128) + (p % 4);
    if (cm) { return plane[(r / R) * R * K + (c * R + r % R) * 512 + in_chunk]; }
    return plane[r * K + c * 512 + in_chunk];
}

int decode_all(const uint8_t * plane, const uint8_t * aux, uint16_t * out) {
    const Header h = rd<Header>(aux);
    if (h.magic != kMagic) { return 1; }
    const int64_t K = h.K, rows = (int64_t) h.rows, C = K / 512;
    const bool cm = h.flags & kFlagCm, fo = h.flags & kFlagFo;
    std::vector<uint8_t> ex((size_t) (rows * K), 0);
    if (h.format == (uint32_t) kNibble) {
        for (int64_t r = 0; r < rows; r++) {
            for (int64_t c = 0; c < C; c++) {
                for (int l = 0; l < 32; l++) {
                    const uint64_t nw = rd<uint64_t>(aux + h.off_a + (r * C + c) * 256 + 8 * l);
                    for (int s = 0; s < 16; s++) {
                        ex[r * K + c * 512 + pos_of(l, s)] = aux[h.off_b + r * 16 + ((nw >> (4 * s)) & 0xF)];
                    }
                }
            }
        }
    } else if (h.format == (uint32_t) kHuffman) {
        for (uint64_t u = 0; u < h.n_a; u++) {
            for (int l = 0; l < 32; l++) {
                BitReader bs{aux + h.off_c, rd<uint32_t>(aux + h.off_b + 4 * (u * 32 + l))};
                for (int64_t r = u * h.R; r < (int64_t) ((u + 1) * h.R); r++) {
                    for (int64_t c = 0; c < C; c++) {
                        for (int s = 0; s < 16; s++) {
                            const uint32_t v = rd<uint32_t>(aux + h.off_a + 4 * bs.peek(kHufL));
                            bs.skip((int) (v & 0x7F));
                            ex[r * K + c * 512 + pos_of(l, s)] = (uint8_t) ((v >> 7) & 0xFF);
                        }
                    }
                }
            }
        }
    } else if (h.format == (uint32_t) kHufpair) {
        decode_exponents_hp(aux, h, 0, h.n_a, ex.data());
    } else {
        return 1;
    }
    for (int64_t r = 0; r < rows; r++) {
        for (int64_t k = 0; k < K; k++) {
            out[r * K + k] = join(sm_at(plane, K, (int) h.R, r, k, cm, fo), ex[r * K + k]);
        }
    }
    if (h.format == (uint32_t) kNibble) {
        for (int64_t r = 0; r < rows; r++) {
            for (uint32_t i = rd<uint32_t>(aux + h.off_c + 4 * r); i < rd<uint32_t>(aux + h.off_c + 4 * (r + 1)); i++) {
                const uint32_t x = rd<uint32_t>(aux + h.off_d + 4 * i);
                out[r * K + (x & 0xFFF)] = join((uint8_t) ((x >> 12) & 0xFF), (int) (x >> 20));
            }
        }
    }
    return 0;
}

inline float bf16_to_f32(uint16_t v) { uint32_t b = (uint32_t) v << 16; float f; memcpy(&f, &b, 4); return f; }

template <typename F> void par_for(int64_t n, int nthreads, F && f) {
    nthreads = std::max(1, nthreads);
    std::atomic<int64_t> next{0};
    std::vector<std::thread> th;
    for (int t = 0; t < nthreads; t++) {
        th.emplace_back([&] { for (int64_t i; (i = next.fetch_add(1)) < n;) { f(i); } });
    }
    for (auto & t : th) { t.join(); }
}

} // namespace

extern "C" {

// Encoder restatement. Returns 0, or 1 for arguments the reference rejects (encode.cpp:443-473). plane: rows*K bytes
// (caller), *aux: malloc'd (free with orc_free), *fmt_out: the format produced (HUFPAIR may fall back to HUFFMAN).
int orc_encode(const uint16_t * w, int64_t rows, int64_t K, int format, int R, int cm, int fo, uint8_t * plane,
               uint8_t ** aux, uint64_t * aux_len, int * fmt_out) {
    if (K % 512 != 0 || K < 512 || K > 4096 || rows <= 0) { return 1; }
    if (format == kNibble) {
        if (R != 0 || cm || fo) { return 1; }
    } else if (format == kHuffman || format == kHufpair) {
        if (R != 1 && R != 2 && R != 4 && R != 8 && R != 16) { return 1; }
        if (rows % R != 0) { return 1; }
        if (format == kHuffman && cm) { return 1; }
        if (cm && (K == 512 || (R != 4 && R != 8 && R != 16))) { return 1; }
        if (fo && (format != kHufpair || cm || R != 16)) { return 1; }
    } else {
        return 1;
    }
    std::vector<uint8_t> a;
    int fmt = format;
    if (format == kNibble) {
        plane_lane_major(w, rows, K, plane);
        a = enc_nibble(w, rows, K);
        const Header h = rd<Header>(a.data());
        for (int64_t r = 0; r < rows; r++) { // escaped slots read as +0 in the plane (encode.cpp:481-494)
            for (uint32_t i = rd<uint32_t>(a.data() + h.off_c + 4 * r); i < rd<uint32_t>(a.data() + h.off_c + 4 * (r + 1)); i++) {
                const int col = rd<uint32_t>(a.data() + h.off_d + 4 * i) & 0xFFF;
                const int p = col % 512;
                plane[r * K + (col / 512) * 512 + 16 * ((p % 128) / 4) + 4 * (p / 128) + p % 4] = 0;
            }
        }
    } else {
        if (format == kHufpair) { a = enc_hufpair(w, rows, K, R, cm, fo); }
        if (a.empty()) { a = enc_huffman(w, rows, K, R); fmt = kHuffman; }
        const uint32_t flags = fmt == kHufpair ? rd<Header>(a.data()).flags : 0;
        if (flags & kFlagFo) { plane_frag_order(w, rows, K, plane); } else { plane_lane_major(w, rows, K, plane); }
        if (flags & kFlagCm) { // encode.cpp:511-524
            std::vector<uint8_t> tmp((size_t) (R * K));
            for (int64_t u = 0; u < rows / R; u++) {
                uint8_t * ub = plane + u * R * K;
                memcpy(tmp.data(), ub, tmp.size());
                for (int r = 0; r < R; r++) {
                    for (int64_t c = 0; c < K / 512; c++) { memcpy(ub + (c * R + r) * 512, tmp.data() + r * K + c * 512, 512); }
                }
            }
        }
    }
    *aux = (uint8_t *) malloc(a.size());
    memcpy(*aux, a.data(), a.size());
    *aux_len = a.size();
    *fmt_out = fmt;
    return 0;
}

void orc_free(void * p) { free(p); }

// Decoder restatement: exact BF16 bits, row-major rows x K (sizes from the aux header). 0 ok, 1 bad header.
int orc_decode(const uint8_t * plane, const uint8_t * aux, uint16_t * out) { return decode_all(plane, aux, out); }

// FP64 reference: y[r] = sum_k w[r,k] x[k], s[r] = sum_k |w[r,k] x[k]| (the error scale of the reference's tests,
// tests/conftest.py:46-55). x as FP32 values (BF16 activations are passed widened).
void orc_gemv_f64(const uint16_t * w, int64_t rows, int64_t K, const float * x, double * y, double * s, int nthreads) {
    par_for(rows, nthreads, [&](int64_t r) {
        double a = 0, m = 0;
        for (int64_t k = 0; k < K; k++) {
            const double p = (double) bf16_to_f32(w[r * K + k]) * (double) x[k];
            a += p; m += std::fabs(p);
        }
        y[r] = a; if (s) { s[r] = m; }
    });
}

// FP32 emulation of the kernels' summation order over exact weights (row-major units, kernels.cuh:524-534 + 119-125;
// chunk_major != 0: per-chunk lane sums accumulated per row first, kernels.cuh:958-986). Escapes of NIBBLE matrices:
// esc_cols / esc_n per row list columns whose products are added after the dense pass (kernels.cuh:178-186); pass
// nullptr for Huffman formats.
void orc_gemv_f32_order(const uint16_t * w, int64_t rows, int64_t K, const float * x, float * y, int chunk_major,
                        const int32_t * esc_cols, const int64_t * esc_off) {
    const int64_t C = K / 512;
    for (int64_t r = 0; r < rows; r++) {
        float lane[32];
        for (int l = 0; l < 32; l++) {
            float acc = 0.f, a[4] = {0, 0, 0, 0};
            for (int64_t c = 0; c < C; c++) {
                if (chunk_major) { a[0] = a[1] = a[2] = a[3] = 0.f; }
                for (int j = 0; j < 4; j++) {
                    for (int t = 0; t < 4; t++) {
                        const int64_t k = c * 512 + 128 * j + 4 * l + t;
                        bool esc = false;
                        if (esc_cols) {
                            for (int64_t e = esc_off[r]; e < esc_off[r + 1]; e++) { esc |= esc_cols[e] == k; }
                        }
                        const float wv = esc ? 0.f : bf16_to_f32(w[r * K + k]);
                        a[t] = std::fmaf(wv, x[k], a[t]);
                    }
                }
                if (chunk_major) { acc += (a[0] + a[1]) + (a[2] + a[3]); }
            }
            if (!chunk_major) { acc = (a[0] + a[1]) + (a[2] + a[3]); }
            if (esc_cols) {
                for (int64_t e = esc_off[r] + l; e < esc_off[r + 1]; e += 32) {
                    acc = std::fmaf(bf16_to_f32(w[r * K + esc_cols[e]]), x[esc_cols[e]], acc);
                }
            }
            lane[l] = acc;
        }
        for (int o = 16; o; o >>= 1) {
            float nx[32];
            for (int l = 0; l < 32; l++) { nx[l] = lane[l] + lane[l ^ o]; }
            memcpy(lane, nx, sizeof nx);
        }
        y[r] = lane[0];
    }
}

// The timed CPU arm: decode HUFPAIR row-major / chunk-major units [u0, u1) from plane+aux and multiply by x with FP32
// accumulation, units spread over nthreads host threads. y indexed by row - u0*R. Returns 0, 1 on an unsupported header.
int orc_decode_gemv_mt(const uint8_t * plane, const uint8_t * aux, uint64_t u0, uint64_t u1, const float * x, float * y,
                       int nthreads) {
    const Header h = rd<Header>(aux);
    if (h.magic != kMagic || h.format != (uint32_t) kHufpair || (h.flags & kFlagFo)) { return 1; }
    const int64_t K = h.K, R = h.R;
    const bool cm = h.flags & kFlagCm;
    par_for((int64_t) (u1 - u0), nthreads, [&](int64_t i) {
        const uint64_t u = u0 + i;
        std::vector<uint8_t> ex((size_t) (R * K));
        decode_exponents_hp(aux, h, u, u + 1, ex.data(), (int64_t) u * R);
        for (int64_t rr = 0; rr < R; rr++) {
            const int64_t r = u * R + rr;
            float acc = 0.f;
            for (int64_t k = 0; k < K; k++) {
                const uint16_t b = join(sm_at(plane, K, (int) R, r, k, cm, false), ex[rr * K + k]);
                acc = std::fmaf(bf16_to_f32(b), x[k], acc);
            }
            y[(u - u0) * R + rr] = acc;
        }
    });
    return 0;
}

} // extern "C"
