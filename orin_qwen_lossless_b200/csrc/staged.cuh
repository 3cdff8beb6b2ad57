// Building blocks of the kernels that stage a unit's exponent streams in shared memory with one bulk async copy:
// mbarrier / bulk-copy wrappers with bounded waits, the lane-stream reader over staged words, the lane's activations
// in registers. See gemv_staged.cu for the design notes.
#pragma once

#include "decode.cuh"

namespace b16 {
namespace dev {

using bf16 = __nv_bfloat16;

// Set when a bounded mbarrier wait ran out (one copy per translation unit; bf16n_fault_status reads and clears them).
// The outputs of the work item whose wait expired are written as NaN.
static __device__ unsigned int g_wait_expired;
// defines `unsigned int * NAME()`: the device address of this translation unit's word (device current, outside capture)
#define BF16N_DEFINE_FAULT_WORD(NAME)                                                           \
    unsigned int * NAME() {                                                                     \
        unsigned int * p = nullptr;                                                             \
        cuda_ok(cudaGetSymbolAddress((void **) &p, dev::g_wait_expired), "fault word address"); \
        return p;                                                                               \
    }

constexpr uint32_t WAIT_LIMIT = 1u << 20; // try_wait polls before a warp gives up on its bulk copy

__device__ __forceinline__ uint32_t smem_u32(const void * p) { return (uint32_t) __cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// returns 1 when the phase completed (the value doubles as the token staged reads depend on), 0 when the wait ran out
__device__ __forceinline__ uint32_t mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < WAIT_LIMIT; i++) {
        uint32_t done;
        asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) { return done; }
    }
    return 0;
}
// global -> shared bulk copy; dst/src 16-byte aligned, bytes a multiple of 16; completes on the mbarrier
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void * src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

__device__ __forceinline__ void prefetch_l2(const void * p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
__device__ __forceinline__ void bulk_prefetch_l2(const void * src, uint32_t bytes) { // 16-byte aligned, multiple of 16
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}

__device__ __forceinline__ uint32_t shl_wrap_hi(uint32_t lo, uint32_t hi, uint32_t n) { // high word of {hi:lo} << (n & 31)
    uint32_t d;
    asm("shf.l.wrap.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(lo), "r"(hi), "r"(n));
    return d;
}

// Integer constants the compiler must not see through: passed as kernel arguments so that "a * k + b" stays an integer
// multiply-add. On sm_100a shifts, logic ops and byte permutes issue at half rate on one pipe and integer multiply-adds
// at half rate on another; the decoder is bound by the first, so every add that can be phrased as a multiply-add by one
// of these constants runs on the second instead.
struct Opaque { uint32_t one, four, minus_one, thirty_two; };

__device__ __forceinline__ uint32_t imad(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// `token` is produced by the mbarrier wait of the bulk copy whose bytes are read: the data dependency keeps a read of
// staged stream words after that wait (table reads pass 0: the table is complete before the block barrier).
__device__ __forceinline__ uint32_t lds32(uint32_t addr, uint32_t token = 0) {
    uint32_t v;
    asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr), "r"(token));
    return v;
}

// Lane stream reader over words in shared memory (addresses are 32-bit shared-window addresses). {hi:lo} is the
// MSB-first bit buffer; `v` counts its valid bits in its low 7 bits (the rest is garbage left by subtracting whole
// table entries) and is kept in [32, 63] before every pair of codes; `t` is the sum of the last two entries, whose low
// bits are the bits they consumed.
struct StagedReader {
    uint32_t next, hi, lo, ahead, v, t, token;

    __device__ __forceinline__ void open(uint32_t addr, uint32_t wait_token) {
        token = wait_token;
        hi = lds32(addr, token); lo = 0; ahead = lds32(addr + 4, token); next = addr + 8; v = 32; t = 0;
    }
    // two codes: e0, e1 = their table entries
    __device__ __forceinline__ void take2(uint32_t lut, const Opaque & k, uint32_t & e0, uint32_t & e1) {
        v = imad(t, k.minus_one, v);
        const uint32_t place = __funnelshift_r(0u, 1u, v); // 2^(32 - v) for v in 1..31
        if (!(v & 32u)) {                                   // fewer than 32 valid bits: append the look-ahead word
            uint64_t b;
            asm("mov.b64 %0, {%1, %2};" : "=l"(b) : "r"(lo), "r"(hi));
            asm("mad.wide.u32 %0, %1, %2, %0;" : "+l"(b) : "r"(ahead), "r"(place));
            asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(b));
            ahead = lds32(next, token);
            next = imad(k.four, k.one, next);
            v = imad(k.thirty_two, k.one, v);
        }
        e0 = lds32(imad(hi >> (32 - HP_LMAX), k.four, lut));
        const uint32_t second = shl_wrap_hi(lo, hi, e0);
        e1 = lds32(imad(second >> (32 - HP_LMAX), k.four, lut));
        t = imad(e0, k.one, e1);
        hi = shl_wrap_hi(lo, hi, t);
        lo = shl_wrap_hi(0u, lo, t);
    }
    __device__ __forceinline__ void take8(uint32_t lut, const Opaque & k, uint32_t (&e)[8]) {
#pragma unroll
        for (int q = 0; q < 8; q += 2) { take2(lut, k, e[q], e[q + 1]); }
    }
};

// the same interface over the general reader (streams in global memory, table through a generic pointer)
struct GlobalReader {
    PairReader rd;
    const uint32_t * lut;
    __device__ __forceinline__ void take8(uint32_t, const Opaque &, uint32_t (&e)[8]) { rd.take8(lut, e); }
};

// this lane's activations of a K-column row, in registers
template <int C, typename TX> struct LaneX;
template <int C> struct LaneX<C, float> {
    float4 q[C * 4];
    __device__ __forceinline__ void load(const float * x, int lane) {
#pragma unroll
        for (int i = 0; i < C * 4; i++) { q[i] = ldg_x4(x, (i >> 2) * CHUNK + 128 * (i & 3) + 4 * lane); }
    }
    __device__ __forceinline__ void fma(int c, const uint32_t (&w)[8], float (&a)[4]) const {
#pragma unroll
        for (int j = 0; j < 4; j++) {
            a[0] = fmaf(bf16lo_f32(w[2 * j]), q[c * 4 + j].x, a[0]);
            a[1] = fmaf(bf16hi_f32(w[2 * j]), q[c * 4 + j].y, a[1]);
            a[2] = fmaf(bf16lo_f32(w[2 * j + 1]), q[c * 4 + j].z, a[2]);
            a[3] = fmaf(bf16hi_f32(w[2 * j + 1]), q[c * 4 + j].w, a[3]);
        }
    }
};
template <int C> struct LaneX<C, bf16> {
    uint2 q[C * 4]; // two BF16 pairs per column quad
    __device__ __forceinline__ void load(const bf16 * x, int lane) {
#pragma unroll
        for (int i = 0; i < C * 4; i++) { q[i] = ld_act8(x + (i >> 2) * CHUNK + 128 * (i & 3) + 4 * lane); }
    }
    // acc += w.lo * x.lo ; acc2 += w.hi * x.hi with BF16 operands and FP32 accumulate
    static __device__ __forceinline__ void fma2(uint32_t w, uint32_t x, float & lo, float & hi) {
        asm("{ .reg .b16 wl, wh, xl, xh;\n\t"
            "mov.b32 {wl, wh}, %2;\n\t"
            "mov.b32 {xl, xh}, %3;\n\t"
            "fma.rn.f32.bf16 %0, wl, xl, %0;\n\t"
            "fma.rn.f32.bf16 %1, wh, xh, %1; }"
            : "+f"(lo), "+f"(hi) : "r"(w), "r"(x));
    }
    __device__ __forceinline__ void fma(int c, const uint32_t (&w)[8], float (&a)[4]) const {
#pragma unroll
        for (int j = 0; j < 4; j++) {
            fma2(w[2 * j], q[c * 4 + j].x, a[0], a[1]);
            fma2(w[2 * j + 1], q[c * 4 + j].y, a[2], a[3]);
        }
    }
};

} // namespace dev
} // namespace b16
