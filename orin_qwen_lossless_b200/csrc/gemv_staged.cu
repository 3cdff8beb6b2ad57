// The large-matrix decode+GEMV (vocabulary projection, big dense projections): row-major HUFPAIR, one activation column.
//
// Persistent launch, one block per SM. Each warp owns one unit (R rows) at a time and
//   * stages the unit's whole exponent stream block - all 32 lane streams are contiguous in the aux buffer - into its
//     private shared-memory buffer with one bulk async copy (TMA, 1-D, no multicast) completing on an mbarrier, so
//     the HBM side of the streams is fully coalesced and costs no load/store-unit address work;
//   * keeps this lane's activations in registers for the whole kernel (the lane-major layout gives every lane the
//     same 16 columns of every chunk), packed as BF16 pairs when the activations are BF16, and multiplies with the
//     mixed-precision fma (BF16 x BF16 + FP32, exact products, one rounding: the same bits as FP32 fma of the widened
//     values);
//   * reads the sign|mantissa plane with 16-byte streaming loads, one row ahead;
//   * walks the bit streams with a 64-bit buffer, a one-word look-ahead and a refill test every second code whose
//     bookkeeping needs no masking: table entries carry the code length in their low bits and the funnel shifts use
//     only the low 5 bits of their shift operand.
// Units that do not fit the buffer (codes much longer than average) are decoded straight from global memory.
// Products are summed in the format's order (see gemv.cu), so results equal the general kernel's bit for bit.
#include "decode.cuh"
#include "launch.h"

namespace b16 {
namespace {

using namespace dev;
using bf16 = __nv_bfloat16;

__device__ unsigned int g_wait_expired; // a bounded mbarrier wait ran out (host-visible diagnostic)

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
        for (int i = 0; i < C * 4; i++) { q[i] = __ldg((const uint2 *) (x + (i >> 2) * CHUNK + 128 * (i & 3) + 4 * lane)); }
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

constexpr int PLANE_AHEAD = 4; // rows of plane prefetched into L2 ahead of the row being decoded

// the R rows of one unit: decode, multiply, reduce; lane r ends up holding row r's sum
template <int C, typename TX, typename Reader>
__device__ __forceinline__ float unit_rows(Reader & rd, uint32_t lut, const Opaque & k, const uint8_t * pl, int R, const LaneX<C, TX> & x, int lane) {
    constexpr int K = C * CHUNK;
    float mine = 0.f;
    uint4 nxt[C];
#pragma unroll
    for (int c = 0; c < C; c++) { nxt[c] = ld_stream16(pl + c * CHUNK); }
    for (int rr = 0; rr < R; rr++) {
        uint4 cur[C];
#pragma unroll
        for (int c = 0; c < C; c++) { cur[c] = nxt[c]; }
        if (rr + 1 < R) {
#pragma unroll
            for (int c = 0; c < C; c++) { nxt[c] = ld_stream16(pl + (rr + 1) * K + c * CHUNK); }
        }
        // pull a later row of the plane into L2 (one 128-byte line per lane), so the register loads above hit L2
        if (rr + PLANE_AHEAD < R && lane < K / 128) { prefetch_l2(pl - 16 * lane + (rr + PLANE_AHEAD) * K + 128 * lane); }
        float a[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < C; c++) {
            uint32_t e[8], wv[8];
            rd.take8(lut, k, e);
            assemble8(cur[c], e, wv);
            x.fma(c, wv, a);
        }
        const float s = warp_sum((a[0] + a[1]) + (a[2] + a[3]));
        if (lane == rr) { mine = s; }
    }
    return mine;
}

template <int C, typename TX>
__global__ void __launch_bounds__(512, 1) k_pair_gemv_staged(const PairView w, const AuxHeader * hdr, int R, Cols p, uint32_t cap_bytes,
                                                             const Opaque k) {
    extern __shared__ __align__(128) unsigned char smem[];
    uint32_t * lut = (uint32_t *) smem;                            // 16 KB
    uint64_t * bars = (uint64_t *) (smem + 4 * HP_MAX_PAIRS);      // one mbarrier per warp
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    unsigned char * buf = smem + 4 * HP_MAX_PAIRS + 128 + (size_t) warp * cap_bytes;
    const uint32_t bar = smem_u32(bars + warp);

    const TX * xg; OutVec out; int64_t rbase;
    column<TX>(p, blockIdx.y, xg, out, rbase);
    for (int i = threadIdx.x; i < HP_MAX_PAIRS / 4; i += blockDim.x) { ((uint4 *) lut)[i] = __ldg((const uint4 *) w.lut + i); }
    if (lane == 0) { mbar_init(bar, 1); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    LaneX<C, TX> x;
    x.load(xg, lane);
    const uint32_t n_units = (uint32_t) hdr->n_a, n_words = (uint32_t) hdr->n_b;
    __syncthreads();

    uint32_t parity = 0;
    const int64_t units = p.nrows / R, stride = (int64_t) gridDim.x * nwarp;
    // stream geometry of a unit: first word rounded down to 16 bytes, bytes to stage (with look-ahead words: the stream
    // is padded), this lane's first word inside the staged block
    struct Geo { uint32_t start, bytes, my; };
    auto geometry = [&](int64_t gu) {
        const uint32_t w0 = __ldg(w.ubase + gu);
        const uint32_t w1 = gu + 1 < (int64_t) n_units ? __ldg(w.ubase + gu + 1) : n_words;
        Geo g;
        g.start = w0 & ~3u;
        g.bytes = ((w1 - g.start + 4u + 3u) & ~3u) * 4u;
        g.my = w0 - g.start + __ldg(w.lrel + gu * 32 + lane);
        return g;
    };
    int64_t u = (int64_t) blockIdx.x * nwarp + warp;
    Geo cur = {0, 0, 0};
    if (u < units) { cur = geometry(rbase / R + u); }
    for (; u < units; u += stride) {
        const int64_t gu = rbase / R + u;
        const uint8_t * pl = w.plane + gu * R * (C * CHUNK) + 16 * lane;
        const bool staged = cur.bytes <= cap_bytes;
        if (staged) {
            __syncwarp(); // every lane is done with the previous unit's words
            if (lane == 0) {
                mbar_expect_tx(bar, cur.bytes);
                bulk_g2s(smem_u32(buf), w.stream + cur.start, cur.bytes, bar);
            }
        }
        // while the copy is in flight: the next unit's geometry, and its stream block and first plane rows into L2, so
        // that its own copy and first loads are short
        Geo nxt = {0, 0, 0};
        if (u + stride < units) {
            const int64_t gn = gu + stride;
            nxt = geometry(gn);
            if (lane == 0) { bulk_prefetch_l2(w.stream + nxt.start, nxt.bytes); }
            if (lane < PLANE_AHEAD * C * CHUNK / 128) { prefetch_l2(w.plane + gn * R * (C * CHUNK) + 128 * lane); }
        }
        float mine;
        if (staged) {
            const uint32_t landed = mbar_wait(bar, parity);
            if (!landed) {
                if (lane == 0) { atomicOr(&g_wait_expired, 1u); }
                return;
            }
            parity ^= 1u;
            StagedReader rd;
            rd.open(smem_u32(buf) + 4 * cur.my, landed);
            mine = unit_rows<C, TX>(rd, smem_u32(lut), k, pl, R, x, lane);
        } else {
            GlobalReader rd;
            rd.lut = lut;
            rd.rd.open(w, gu, lane);
            mine = unit_rows<C, TX>(rd, 0u, k, pl, R, x, lane);
        }
        if (lane < R) { out.put(u * R + lane, mine); }
        cur = nxt;
    }
}

constexpr int FIXED_SMEM = 4 * HP_MAX_PAIRS + 128;

// per-warp buffer: the unit's stream at 3 bits per weight (typical tensors need about 2.7) plus alignment slack
uint32_t buffer_bytes(const bf16n_weight & w) { return (uint32_t) ((w.R * w.K * 3 / 8 + 64 + 15) & ~15ll); }

} // namespace

void gemv_staged_init() {
    const int optin = device_info().smem_optin;
#define ATTR(KERNEL) cuda_ok(cudaFuncSetAttribute(KERNEL, cudaFuncAttributeMaxDynamicSharedMemorySize, optin), #KERNEL)
    ATTR((k_pair_gemv_staged<1, float>)); ATTR((k_pair_gemv_staged<2, float>)); ATTR((k_pair_gemv_staged<4, float>));
    ATTR((k_pair_gemv_staged<1, bf16>)); ATTR((k_pair_gemv_staged<2, bf16>)); ATTR((k_pair_gemv_staged<4, bf16>));
#undef ATTR
}

// Row-major HUFPAIR with K <= 2048 and enough units to give every SM several warps of work.
bool gemv_staged_applies(const bf16n_weight & w, const bf16n_mmv_args & a) {
    const int64_t C = w.K / CHUNK;
    if (w.format != FMT_HUFPAIR || w.cm || w.fo || !(C == 1 || C == 2 || C == 4) || a.nrows <= 0) { return false; }
    const int64_t units = a.nrows / w.R;
    const int64_t room = (device_info().smem_optin - FIXED_SMEM) / buffer_bytes(w);
    return room >= 8 && units >= (int64_t) device_info().sms * 8 * std::max(1, a.ncols);
}

void gemv_staged(const bf16n_weight & w, const bf16n_mmv_args & a, cudaStream_t st) {
    const Cols p = make_cols(a);
    const uint32_t cap = buffer_bytes(w);
    const int64_t units = a.nrows / w.R, sms = device_info().sms;
    const int max_warps = (int) std::min<int64_t>(16, (device_info().smem_optin - FIXED_SMEM) / cap);
    // static round-robin over sms * warps warps: take the warp count that wastes least of the last round
    int best = max_warps;
    double best_eff = 0.0;
    for (int nw = max_warps; nw >= std::max(8, max_warps - 4); nw--) {
        const int64_t slots = sms * nw, rounds = (units + slots - 1) / slots;
        const double eff = (double) units / (double) (rounds * slots) * (nw >= 12 ? 1.0 : 0.97);
        if (eff > best_eff + 1e-9) { best_eff = eff; best = nw; }
    }
    const dim3 grid((unsigned) sms, (unsigned) a.ncols);
    const size_t shm = FIXED_SMEM + (size_t) best * cap;
    const AuxHeader * hdr = (const AuxHeader *) w.aux;
    const PairView v = pair_view(w);
    const Opaque k = {1u, 4u, ~0u, 32u};
#define GO(CC, TX) k_pair_gemv_staged<CC, TX><<<grid, best * 32, shm, st>>>(v, hdr, w.R, p, cap, k)
    if (a.x_bf16) {
        switch (w.K / CHUNK) { case 1: GO(1, bf16); break; case 2: GO(2, bf16); break; default: GO(4, bf16); break; }
    } else {
        switch (w.K / CHUNK) { case 1: GO(1, float); break; case 2: GO(2, float); break; default: GO(4, float); break; }
    }
#undef GO
    check_launch();
}

} // namespace b16
