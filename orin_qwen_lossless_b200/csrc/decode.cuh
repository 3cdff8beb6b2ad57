// Device-side building blocks shared by the BF16N kernels: bit-stream readers, weight assembly, reductions, output
// stores and the column descriptor. Layout facts (format.h): a warp owns one row-chunk of 512 weights at a time, lane l
// holds the 16 plane bytes of slots 0..15 (columns 128*(s>>2) + 4*l + (s&3)), i.e. one 32-bit plane word per column
// quad j = s>>2, whose bytes are the columns 128*j + 4*l + {0,1,2,3}.
#pragma once

#include "../../include/bf16n_c.h"
#include "format.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace b16 {
namespace dev {

constexpr uint32_t FULL = 0xffffffffu;

// ---------------------------------------------------------------- small PTX helpers

__device__ __forceinline__ uint32_t byte_perm(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

// (a & m) | (b & ~m) with m = 0x807F807F: sign and mantissa bits from a, exponent bits from b, for two BF16 halves
__device__ __forceinline__ uint32_t merge_sm_exp(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, 0x807F807F, 0xE4;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

// plane bytes (lo, hi) = bytes {0,1} or {2,3} of a plane word, each spread to a BF16 half with its sign bit copied to
// bit 15 (prmt sign-replication fills the upper byte); bits 7..14 are garbage and are masked by merge_sm_exp
__device__ __forceinline__ uint32_t spread_lo(uint32_t plane_word) { return byte_perm(plane_word, 0, 0x9180u); }
__device__ __forceinline__ uint32_t spread_hi(uint32_t plane_word) { return byte_perm(plane_word, 0, 0xB3A2u); }

// streaming 16-byte load that does not allocate in L1 (each plane byte is read once)
__device__ __forceinline__ uint4 ld_stream16(const void * p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ float bf16lo_f32(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi_f32(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) { v += __shfl_xor_sync(FULL, v, o); }
    return v;
}

// silu with the fast exponential and division the reference's fast-math build uses (core/include/bf16n/compat.cuh:29-31)
__device__ __forceinline__ float silu_f(float v) { return __fdividef(v, 1.0f + __expf(-v)); }

// ---------------------------------------------------------------- activations

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __uint_as_float((uint32_t) __bfloat16_as_ushort(v) << 16); }

// Activations may have been written by the kernel right before this one on the stream, which can still be running when
// this kernel starts (programmatic dependent launch). They are therefore read with ordinary coherent loads written as
// volatile asm: such a load stays behind the grid dependency wait (the read-only ld.global.nc path may be moved above it
// and may serve lines fetched before the producer's stores), and it still caches in L1 for the other rows of the block.
__device__ __forceinline__ uint4 ld_act16(const void * p) {
    uint4 v;
    asm volatile("ld.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint2 ld_act8(const void * p) {
    uint2 v;
    asm volatile("ld.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float ld_act_f32(const float * p) {
    float v;
    asm volatile("ld.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
    return v;
}
// x[i..i+3] as FP32 from global memory (i a multiple of 4; the caller guarantees 16-/8-byte alignment)
__device__ __forceinline__ float4 ldg_x4(const float * x, int i) {
    const uint4 v = ld_act16(x + i);
    return make_float4(__uint_as_float(v.x), __uint_as_float(v.y), __uint_as_float(v.z), __uint_as_float(v.w));
}
__device__ __forceinline__ float4 ldg_x4(const __nv_bfloat16 * x, int i) {
    const uint2 v = ld_act8(x + i);
    return make_float4(bf16lo_f32(v.x), bf16hi_f32(v.x), bf16lo_f32(v.y), bf16hi_f32(v.y));
}
__device__ __forceinline__ float ldg_x1(const float * x, int i) { return ld_act_f32(x + i); }
__device__ __forceinline__ float ldg_x1(const __nv_bfloat16 * x, int i) {
    unsigned short v;
    asm volatile("ld.global.u16 %0, [%1];" : "=h"(v) : "l"(x + i) : "memory");
    return __uint_as_float((uint32_t) v << 16);
}

// ---------------------------------------------------------------- output

struct OutVec { // one output column, FP32 or BF16 (round to nearest even)
    char * p;
    bool bf16;
    __device__ __forceinline__ void put(int64_t i, float v) const {
        if (bf16) { ((__nv_bfloat16 *) p)[i] = __float2bfloat16_rn(v); } else { ((float *) p)[i] = v; }
    }
};

// ---------------------------------------------------------------- columns (tokens, or (token, expert slot) pairs)

// Optional fan-out of a kernel's output to other GPUs (dense columns only): every value written to y is also stored at
// the same offset of each peer's buffer, and the last block to finish announces the launch in the peers' headers.
constexpr int MAX_PEERS = 7;
struct PeerOut {
    int n;                        // number of peers (0: none)
    char * y[MAX_PEERS];          // the peers' copies of y (peer memory mapped into this process)
    uint32_t * flag[MAX_PEERS];   // this rank's slot in each peer's exchange header
    uint32_t * hdr;               // this rank's own exchange header (block counter, epochs): words of bf16n_c.h's layout
    int wait_mask;                // ranks whose announcement of the same epoch the last block awaits before the kernel ends
    uint64_t wait_ns;             // how long that wait may take before the header's expired word is set (bf16n_set_peer_wait_limit_ms)
};
constexpr int XH_DONE = 16, XH_SENT = 17, XH_WAITED = 18, XH_EXPIRED = 19; // header words (0..7: the peers' flags)
// diagnostics of the last fan-out launch, %globaltimer nanoseconds of this GPU (64-bit, two words each): block 0 began,
// the last block saw every block's stores issued, the epoch was published to the peers, every peer's epoch was seen
constexpr int XH_T_BEGIN = 20, XH_T_STORED = 22, XH_T_PUBLISHED = 24, XH_T_SEEN = 26;

struct Cols {
    const char * x; char * y;
    int64_t x_tok, x_slot, y_tok, y_slot; // byte strides
    const char * ids; int64_t ids_s0, ids_s1;
    int n_used, x_per_slot;
    int64_t rows_per_matrix, row0, nrows;
    bool y_bf16;
    PeerOut peers;
};

// value i of the output column that starts `col_bytes` into y, to every peer
__device__ __forceinline__ void peers_put(const PeerOut & o, int64_t col_bytes, bool bf16, int64_t i, float v) {
    for (int r = 0; r < o.n; r++) {
        char * q = o.y[r] + col_bytes;
        if (bf16) { ((__nv_bfloat16 *) q)[i] = __float2bfloat16_rn(v); } else { ((float *) q)[i] = v; }
    }
}
// value i of dense column `col`, to every peer
__device__ __forceinline__ void peers_put(const Cols & c, int col, int64_t i, float v) {
    peers_put(c.peers, col * c.y_tok, c.y_bf16, i, v);
}
// End of a kernel that fans out: call with every thread of the block that is still running. Each block makes its
// stores visible system-wide and counts itself; the last one advances this rank's epoch and publishes it to the peers
// (release), whose bf16n_peer_wait acquires it.
__device__ __forceinline__ uint64_t global_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// start of a kernel that fans out: block 0 records when the launch began (header words 20, 21: diagnostics only)
__device__ __forceinline__ void peers_begin(const PeerOut & o) {
    if (o.n && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) { *(volatile uint64_t *) (o.hdr + XH_T_BEGIN) = global_ns(); }
}
__device__ __forceinline__ void peers_done(const PeerOut & o) {
    if (o.n == 0) { return; }
    __shared__ uint32_t last_epoch; // 0: this block is not the last one
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        const unsigned blocks = gridDim.x * gridDim.y * gridDim.z;
        uint32_t epoch = 0;
        if (atomicAdd(o.hdr + XH_DONE, 1u) == blocks - 1u) {
            o.hdr[XH_DONE] = 0u;
            epoch = o.hdr[XH_SENT] + 1u;
            o.hdr[XH_SENT] = epoch;
            *(volatile uint64_t *) (o.hdr + XH_T_STORED) = global_ns();
            // every block fenced before it counted itself; this fence (after the count was read) completes the
            // release of all of their stores, so the announcements themselves can be plain system-scope stores
            __threadfence_system();
            for (int r = 0; r < o.n; r++) {
                asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(o.flag[r]), "r"(epoch) : "memory");
            }
            *(volatile uint64_t *) (o.hdr + XH_T_PUBLISHED) = global_ns();
        }
        last_epoch = o.wait_mask ? epoch : 0u;
    }
    __syncthreads();
    // Optionally the kernel also stands in for the consumer's wait: it ends only when the peers' outputs of the same
    // epoch have arrived here. A peer publishes before it waits, so no rank waits for a rank that waits for it. One
    // thread per peer polls that peer's word (local memory); bounded: after wait_ns (two seconds by default) the
    // header's expired word is set and the kernel ends anyway.
    const uint32_t epoch = last_epoch;
    if (epoch != 0u && threadIdx.x < 32) {
        const int r = threadIdx.x;
        bool ok = true;
        if (r < 8 && (o.wait_mask >> r & 1)) {
            ok = false;
            uint64_t t0 = 0;
            for (uint32_t i = 0; i < (1u << 26); i++) {
                uint32_t seen;
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(o.hdr + r) : "memory");
                if ((int32_t) (seen - epoch) >= 0) { ok = true; break; }
                if ((i & 255u) == 255u) {
                    const uint64_t now = global_ns();
                    if (t0 == 0) { t0 = now; } else if (now - t0 > o.wait_ns) { break; }
                }
            }
        }
        const bool all = __all_sync(FULL, ok);
        if (r == 0) {
            if (!all) { o.hdr[XH_EXPIRED] = 1u; }
            o.hdr[XH_WAITED] = epoch;
            *(volatile uint64_t *) (o.hdr + XH_T_SEEN) = global_ns();
            __threadfence_system();
        }
    }
}
__device__ __forceinline__ void peers_done(const Cols & c) { peers_done(c.peers); }

// activation pointer, output column and first weight row of column `col`
template <typename TX>
__device__ __forceinline__ void column(const Cols & c, int col, const TX *& x, OutVec & out, int64_t & rbase) {
    out.bf16 = c.y_bf16;
    if (c.ids) {
        const int t = col / c.n_used, s = col - t * c.n_used;
        const int e = *(const int32_t *) (c.ids + t * c.ids_s1 + s * c.ids_s0);
        x = (const TX *) (c.x + t * c.x_tok + (s % c.x_per_slot) * c.x_slot);
        out.p = c.y + t * c.y_tok + s * c.y_slot;
        rbase = c.row0 + (int64_t) e * c.rows_per_matrix;
    } else {
        x = (const TX *) (c.x + col * c.x_tok);
        out.p = c.y + col * c.y_tok;
        rbase = c.row0;
    }
}

// ---------------------------------------------------------------- HUFPAIR lane stream

struct PairView { // device pointers of one HUFPAIR matrix
    const uint8_t * plane;
    const uint32_t * lut;     // 4096 entries: e_odd << 23 | e_even << 7 | len
    const uint32_t * ubase;   // per unit: first stream word
    const uint16_t * lrel;    // per (unit, lane): word offset inside the unit
    const uint32_t * stream;
};

// MSB-first reader of one lane's stream straight from global memory. `buf` holds `have` valid bits at the top; top_up()
// (call it before every second lookup) keeps at least 32 of them, enough for two codes of up to 12 bits.
struct PairReader {
    const uint32_t * next;
    uint64_t buf;
    uint32_t ahead; // the word after the buffered ones, already loaded
    int have;

    // start at `first` with its three first words already loaded by the caller
    __device__ __forceinline__ void open_loaded(const uint32_t * first, uint32_t w0, uint32_t w1, uint32_t w2) {
        next = first + 3;
        buf = (uint64_t) w0 << 32 | w1;
        ahead = w2;
        have = 64;
    }
    __device__ __forceinline__ void open(const PairView & w, int64_t unit, int lane) {
        const uint32_t * first = w.stream + (__ldg(w.ubase + unit) + __ldg(w.lrel + unit * 32 + lane));
        open_loaded(first, __ldg(first), __ldg(first + 1), __ldg(first + 2));
    }
    __device__ __forceinline__ void top_up() {
        if (have <= 32) {
            buf |= (uint64_t) ahead << (32 - have);
            have += 32;
            ahead = __ldg(next++);
        }
    }
    __device__ __forceinline__ uint32_t take(const uint32_t * lut) {
        const uint32_t e = lut[(uint32_t) (buf >> (64 - HP_LMAX))];
        const int n = e & 31;
        buf <<= n;
        have -= n;
        return e;
    }
    // the 8 entries of one row-chunk (this lane's 16 weights)
    __device__ __forceinline__ void take8(const uint32_t * lut, uint32_t (&e)[8]) {
#pragma unroll
        for (int q = 0; q < 8; q += 2) {
            top_up();
            e[q] = take(lut);
            e[q + 1] = take(lut);
        }
    }
};

// The same reader fed by 16-byte loads: a lane's stream is read as aligned groups of four words (one load request per
// group instead of one per word, which matters when the L1 cache is too small to keep every lane's line). `q0..q3`
// hold the `cnt` words not yet shifted into `buf`, oldest first; `pre` is the group after them, already loaded.
struct WidePairReader {
    const uint4 * next;
    uint64_t buf;
    uint32_t q0, q1, q2, q3;
    uint4 pre;
    int have, cnt;

    __device__ __forceinline__ uint32_t pop() {
        const uint32_t w = q0;
        q0 = q1; q1 = q2; q2 = q3;
        if (--cnt == 0) {
            q0 = pre.x; q1 = pre.y; q2 = pre.z; q3 = pre.w;
            cnt = 4;
            pre = __ldg(next++);
        }
        return w;
    }
    // the aligned group that holds the stream's first word
    static __device__ __forceinline__ const uint4 * group_of(const uint32_t * first) {
        return (const uint4 *) (first - (((uintptr_t) first >> 2) & 3));
    }
    // start at `first` with its two first groups (group_of(first)[0], [1]) already loaded by the caller
    __device__ __forceinline__ void open_loaded(const uint32_t * first, const uint4 & a, const uint4 & b) {
        const int skip = (int) (((uintptr_t) first >> 2) & 3); // words of the first aligned group before the stream
        next = group_of(first) + 2;
        pre = b;
        q0 = a.x; q1 = a.y; q2 = a.z; q3 = a.w;
        if (skip & 1) { q0 = q1; q1 = q2; q2 = q3; }
        if (skip & 2) { q0 = q2; q1 = q3; }
        cnt = 4 - skip;
        const uint32_t hi = pop();
        buf = (uint64_t) hi << 32 | pop();
        have = 64;
    }
    __device__ __forceinline__ void open(const PairView & w, int64_t unit, int lane) {
        const uint32_t * first = w.stream + (__ldg(w.ubase + unit) + __ldg(w.lrel + unit * 32 + lane));
        const uint4 * g = group_of(first);
        open_loaded(first, __ldg(g), __ldg(g + 1));
    }
    __device__ __forceinline__ void top_up() {
        if (have <= 32) {
            buf |= (uint64_t) pop() << (32 - have);
            have += 32;
        }
    }
    __device__ __forceinline__ uint32_t take(const uint32_t * lut) {
        const uint32_t e = lut[(uint32_t) (buf >> (64 - HP_LMAX))];
        const int n = e & 31;
        buf <<= n;
        have -= n;
        return e;
    }
    // the 8 entries of one row-chunk (this lane's 16 weights)
    __device__ __forceinline__ void take8(const uint32_t * lut, uint32_t (&e)[8]) {
#pragma unroll
        for (int q = 0; q < 8; q += 2) {
            top_up();
            e[q] = take(lut);
            e[q + 1] = take(lut);
        }
    }
};

// the four BF16x2 words (column pairs {0,1} and {2,3} of quads j = 0..3 ... in slot order) of a row-chunk
__device__ __forceinline__ void assemble8(const uint4 & sm, const uint32_t (&e)[8], uint32_t (&w)[8]) {
    const uint32_t q[4] = {sm.x, sm.y, sm.z, sm.w};
#pragma unroll
    for (int j = 0; j < 4; j++) {
        w[2 * j] = merge_sm_exp(spread_lo(q[j]), e[2 * j]);
        w[2 * j + 1] = merge_sm_exp(spread_hi(q[j]), e[2 * j + 1]);
    }
}

// ---------------------------------------------------------------- HUFFMAN (single exponent) lane stream

struct HufView {
    const uint8_t * plane;
    const uint32_t * lut;      // 1024 entries: len | exponent << 7
    const uint32_t * lane_off; // per (unit, lane): absolute word offset
    const uint32_t * stream;
};

struct HufReader { // same scheme, codes <= 10 bits, top_up() before every third lookup
    const uint32_t * next;
    uint64_t buf;
    uint32_t ahead;
    int have;
    __device__ __forceinline__ void open(const HufView & w, int64_t unit, int lane) {
        next = w.stream + __ldg(w.lane_off + unit * 32 + lane);
        buf = (uint64_t) __ldg(next) << 32 | __ldg(next + 1);
        ahead = __ldg(next + 2);
        next += 3;
        have = 64;
    }
    __device__ __forceinline__ void top_up() {
        if (have <= 32) {
            buf |= (uint64_t) ahead << (32 - have);
            have += 32;
            ahead = __ldg(next++);
        }
    }
    __device__ __forceinline__ uint32_t take(const uint32_t * lut) {
        const uint32_t e = lut[(uint32_t) (buf >> (64 - HUF_LMAX))];
        const int n = e & 31;
        buf <<= n;
        have -= n;
        return e;
    }
    // 16 exponents of a row-chunk, returned as 8 pair entries in the HUFPAIR table layout (e_odd<<23 | e_even<<7)
    __device__ __forceinline__ void take8(const uint32_t * lut, uint32_t (&e)[8]) {
#pragma unroll
        for (int s = 0; s < 16; s++) {
            if (s % 3 == 0) { top_up(); }
            const uint32_t ent = take(lut) & 0x7F80u;
            if (s & 1) { e[s >> 1] |= ent << 16; } else { e[s >> 1] = ent; }
        }
    }
};

// ---------------------------------------------------------------- NIBBLE rows

struct NibView {
    const uint8_t * plane;
    const uint8_t * codes;     // rows * K/2
    const uint4 * row_lut;     // 16 exponent bytes per row
    const uint32_t * esc_off;  // rows + 1
    const uint32_t * esc;      // col | sign_mantissa << 12 | exponent << 20
};

// The 8 BF16x2 words of a NIBBLE row-chunk. Exponent bytes come from two prmt lookups per 4 weights: a selector
// nibble 0..7 picks a byte of its 8-byte operand pair, 8..15 returns that byte's replicated sign bit, which is 0
// because table entries are < 128. So codes 0..7 read {L.x, L.y} and contribute 0 from {L.z, L.w} (looked up with
// the codes' bit 3 flipped), codes 8..15 the reverse, and the OR of both lookups is the exponent byte.
__device__ __forceinline__ void nib_assemble8(const uint4 & sm, const uint2 & codes, const uint4 & L, uint32_t (&w)[8]) {
    const uint32_t q[4] = {sm.x, sm.y, sm.z, sm.w};
    const uint32_t cw[2] = {codes.x, codes.y};
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const uint32_t sel = (j & 1) ? cw[j >> 1] >> 16 : cw[j >> 1]; // prmt reads the low four nibbles only
        const uint32_t e4 = byte_perm(L.x, L.y, sel) | byte_perm(L.z, L.w, sel ^ 0x8888u);
        w[2 * j] = (spread_lo(q[j]) & 0x807F807Fu) | (byte_perm(e4, 0, 0x4140u) << 7);
        w[2 * j + 1] = (spread_hi(q[j]) & 0x807F807Fu) | (byte_perm(e4, 0, 0x4342u) << 7);
    }
}

__device__ __forceinline__ uint32_t esc_bits(uint32_t rec) { // BF16 bit pattern of an escape record
    const uint32_t sm = (rec >> 12) & 0xFFu, ex = rec >> 20;
    return ((sm & 0x80u) << 8) | (ex << 7) | (sm & 0x7Fu);
}

// ---------------------------------------------------------------- host: views of a weight, column descriptor

inline PairView pair_view(const bf16n_weight & w) {
    return {w.plane, (const uint32_t *) (w.aux + w.off_a), (const uint32_t *) (w.aux + w.off_b),
            (const uint16_t *) (w.aux + w.off_c), (const uint32_t *) (w.aux + w.off_d)};
}
inline HufView huf_view(const bf16n_weight & w) {
    return {w.plane, (const uint32_t *) (w.aux + w.off_a), (const uint32_t *) (w.aux + w.off_b),
            (const uint32_t *) (w.aux + w.off_c)};
}
inline NibView nib_view(const bf16n_weight & w, int64_t shift_rows = 0) {
    // shifting every per-row array by `shift_rows` rows addresses the up half of a merged [gate; up] matrix: escape
    // offsets are absolute indices into the escape list, so the list itself does not move
    return {w.plane + shift_rows * w.K, w.aux + w.off_a + shift_rows * (w.K / 2), (const uint4 *) (w.aux + w.off_b) + shift_rows,
            (const uint32_t *) (w.aux + w.off_c) + shift_rows, (const uint32_t *) (w.aux + w.off_d)};
}

uint64_t peer_wait_limit_ns(); // capi.cu: the limit set by bf16n_set_peer_wait_limit_ms (default two seconds)

inline PeerOut make_peer_out(const bf16n_peer_out * peers) {
    PeerOut o = {};
    if (peers) {
        o.n = peers->n_peers;
        for (int r = 0; r < peers->n_peers && r < MAX_PEERS; r++) {
            o.y[r] = (char *) peers->y[r];
            o.flag[r] = peers->flag[r];
        }
        o.hdr = peers->local_header;
        o.wait_mask = peers->wait_mask;
        o.wait_ns = peer_wait_limit_ns();
    }
    return o;
}

inline Cols make_cols(const bf16n_mmv_args & a, const bf16n_peer_out * peers = nullptr) {
    Cols c = {};
    c.peers = make_peer_out(peers);
    c.x = (const char *) a.x; c.y = (char *) a.y;
    c.x_tok = a.x_tok; c.y_tok = a.y_tok; c.x_slot = a.x_slot; c.y_slot = a.y_slot;
    c.ids = (const char *) a.ids; c.ids_s0 = a.ids_s0; c.ids_s1 = a.ids_s1;
    c.n_used = a.ids ? a.n_used : 1;
    c.x_per_slot = a.x_per_slot > 0 ? a.x_per_slot : 1;
    c.rows_per_matrix = a.rows_per_matrix; c.row0 = a.row0; c.nrows = a.nrows;
    c.y_bf16 = a.y_bf16 != 0;
    return c;
}

} // namespace dev
} // namespace b16
