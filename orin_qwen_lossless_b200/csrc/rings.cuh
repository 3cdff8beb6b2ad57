// Per-lane shared-memory rings and the window reader over them: the lane-stream machinery of the large-matrix decode
// kernels (the decode+GEMV of gemv_rings.cu and the decode-to-operand-tiles pass of expand_tiles.cu).
//
// A chain's stream footprint is a 128-byte ring per lane (4 KB per warp) filled with cp.async 16-byte granules and
// topped up every 32 codes to more than 96 bytes ahead of the read pointer; 32 codes consume at most 48 bytes and
// everything copied before the previous top-up has landed (wait_group 0 at the top-up, 32 codes of work after the
// copies were issued), so the words being read are always complete. The ring is read as a window of three consecutive
// words and a bit offset: one funnel shift per view of the stream, no shift of the window per code, and a refill is
// two register moves and one load. Ring addressing: byte offset from the unit's 16-byte aligned start, modulo 128, XOR
// a per-lane constant that also carries the lane's ring base: one logic op per address. The code table is read from
// LUT_COPIES copies interleaved word by word (entry i of copy r at word LUT_COPIES * i + r; lane l reads copy
// l % LUT_COPIES): only the lanes that share a copy can collide on a bank.
#pragma once
#include "decode.cuh"

namespace b16 {
namespace ring {

using namespace dev;

struct Opaque { uint32_t one, four, minus_one, thirty_two, sixteen; }; // see gemv_staged.cu: keeps adds on the multiply pipe

constexpr int RING_BYTES = 128;
constexpr uint32_t RING_TARGET = 96; // fetch while at most this many bytes are ahead of the read pointer
constexpr int LUT_COPIES = 4;
constexpr int LUT_BYTES = 4 * HP_MAX_PAIRS * LUT_COPIES;

__device__ __forceinline__ uint32_t smem_u32(const void * p) { return (uint32_t) __cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t imad(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// Ring read. Not volatile, so that the instruction scheduler may move it; `token` is a value produced by the last
// cp.async wait, which keeps the read after that wait (the data dependency is the only ordering the compiler sees).
__device__ __forceinline__ uint32_t lds32(uint32_t addr, uint32_t token) {
    uint32_t v;
    asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr), "r"(token));
    return v;
}
__device__ __forceinline__ uint32_t lds32_ro(uint32_t addr) { // table reads: never written after the block barrier
    uint32_t v;
    asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 lds128_ro(uint32_t addr) {
    uint4 v;
    asm("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t shl_wrap_hi(uint32_t lo, uint32_t hi, uint32_t n) {
    uint32_t d;
    asm("shf.l.wrap.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(lo), "r"(hi), "r"(n));
    return d;
}
// (a & 127) ^ c
__device__ __forceinline__ uint32_t ring_addr(uint32_t off, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, 127, %2, 0x6A;" : "=r"(d) : "r"(off), "r"(c)); // (a & b) ^ c
    return d;
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void * src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ uint32_t cp_async_wait_all() { // returns the token ring reads depend on
    uint32_t token;
    asm volatile("cp.async.wait_group 0;\n\tmov.u32 %0, 0;" : "=r"(token) :: "memory");
    return token;
}

// One lane stream read through the lane's ring. Offsets are bytes from `base` (the unit's stream start rounded down to
// 16 bytes); only their low 7 bits address the ring. The stream is seen through a window of three consecutive words
// (hi, lo, ahead) and a bit offset `o` into hi whose low five bits position the view and whose bit 5 toggles when the
// offset passes a word. Only bits 0..5 of `o` are meaningful (table entries carry their length in the low bits and
// exponents above), which is all the funnel shifts and the word-crossing test read.
struct RingReader {
    const uint8_t * base; // global
    uint32_t key;         // ring base | lane swizzle
    uint32_t fetched;     // offset of the next granule to copy
    uint32_t next;        // offset of the next word to read
    uint32_t hi, lo, ahead, o;
    uint32_t token;       // from the last cp.async wait

    // copy granules until more than RING_TARGET bytes are ahead of the read pointer (at most ROUNDS granules)
    template <int ROUNDS>
    __device__ __forceinline__ void top_up(const Opaque & k) {
        int32_t avail = (int32_t) imad(next, k.minus_one, fetched); // negative right after open()
#pragma unroll
        for (int i = 0; i < ROUNDS; i++) {
            if (avail <= (int32_t) RING_TARGET) {
                cp_async16(ring_addr(fetched, key), base + fetched);
                fetched = imad(k.sixteen, k.one, fetched);
                avail = (int32_t) imad(k.sixteen, k.one, (uint32_t) avail);
            }
        }
    }
    // start of a unit: offset of this lane's first word; the caller commits, waits and then calls first_words()
    __device__ __forceinline__ void open(const uint8_t * unit_base, uint32_t first, uint32_t ring_key, const Opaque & k) {
        base = unit_base; key = ring_key;
        fetched = first & ~15u;
        next = first;
        top_up<7>(k);
    }
    __device__ __forceinline__ void first_words() {
        hi = lds32(ring_addr(next, key), token);
        lo = lds32(ring_addr(next + 4, key), token);
        ahead = lds32(ring_addr(next + 8, key), token);
        next += 12; o = 0;
    }
    // two codes: their table entries. `lut`: this lane's copy of the table (entries 16 bytes apart)
    __device__ __forceinline__ void take2(uint32_t lut, const Opaque & k, uint32_t & e0, uint32_t & e1) {
        const uint32_t v1 = shl_wrap_hi(lo, hi, o);          // 32 valid bits from the offset on: two codes are at most 24
        e0 = lds32_ro(imad(v1 >> (32 - HP_LMAX), k.sixteen, lut));
        const uint32_t v2 = shl_wrap_hi(0u, v1, e0);
        e1 = lds32_ro(imad(v2 >> (32 - HP_LMAX), k.sixteen, lut));
        const uint32_t o2 = o + e0 + e1;
        if ((o ^ o2) & 32u) {                                // the offset passed a word: slide the window
            hi = lo; lo = ahead;
            ahead = lds32(ring_addr(next, key), token);
            next = imad(k.four, k.one, next);
        }
        o = o2;
    }
};

} // namespace ring
} // namespace b16
