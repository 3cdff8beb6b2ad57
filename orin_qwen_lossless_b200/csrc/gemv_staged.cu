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
#include "staged.cuh"
#include <cstdlib>
#include "launch.h"

namespace b16 {
namespace {

using namespace dev;

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

template <int C, typename TX, bool PEERS = false> // PEERS: the output also goes to the other GPUs (separate instantiation)
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
    bool dead = false; // a bulk copy of this warp never arrived: no further copies, NaN outputs
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
        const bool staged = !dead && cur.bytes <= cap_bytes;
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
        float mine = __int_as_float(0x7fc00000);
        uint32_t landed = 0;
        if (staged) {
            landed = mbar_wait(bar, parity);
            if (!landed) { // the copy never arrived: report it; this unit and the warp's later units are written as NaN
                if (lane == 0) { atomicOr(&g_wait_expired, 1u); }
                dead = true;
            }
        }
        if (dead) {
            // nothing to compute; the block still reaches its end (and, with peers, its announcement)
        } else if (staged) {
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
        if (lane < R) {
            out.put(u * R + lane, mine);
            if (PEERS) { peers_put(p, blockIdx.y, u * R + lane, mine); }
        }
        cur = nxt;
    }
    if (PEERS) { peers_done(p); }
}

constexpr int FIXED_SMEM = 4 * HP_MAX_PAIRS + 128;

// per-warp buffer: the unit's stream at 3 bits per weight (typical tensors need about 2.7) plus alignment slack
uint32_t buffer_bytes(const bf16n_weight & w) { return (uint32_t) ((w.R * w.K * 3 / 8 + 64 + 15) & ~15ll); }

} // namespace

BF16N_DEFINE_FAULT_WORD(gemv_staged_fault_word)

void gemv_staged_init() {
    const int optin = device_info().smem_optin;
#define ATTR(KERNEL) allow_dynamic_smem((const void *) KERNEL, optin, optin, #KERNEL)
    ATTR((k_pair_gemv_staged<1, float>)); ATTR((k_pair_gemv_staged<2, float>)); ATTR((k_pair_gemv_staged<4, float>));
    ATTR((k_pair_gemv_staged<1, bf16>)); ATTR((k_pair_gemv_staged<2, bf16>)); ATTR((k_pair_gemv_staged<4, bf16>));
    ATTR((k_pair_gemv_staged<1, float, true>)); ATTR((k_pair_gemv_staged<2, float, true>)); ATTR((k_pair_gemv_staged<4, float, true>));
    ATTR((k_pair_gemv_staged<1, bf16, true>)); ATTR((k_pair_gemv_staged<2, bf16, true>)); ATTR((k_pair_gemv_staged<4, bf16, true>));
#undef ATTR
}

// Row-major HUFPAIR with K <= 2048 and enough units to give every SM several warps of work.
bool gemv_staged_applies(const bf16n_weight & w, const bf16n_mmv_args & a) {
    const int64_t C = w.K / CHUNK;
    if (w.format != FMT_HUFPAIR || w.cm || w.fo || !(C == 1 || C == 2 || C == 4) || a.nrows <= 0) { return false; }
    const int64_t units = a.nrows / w.R;
    const int64_t room = (device_info().smem_optin - FIXED_SMEM) / buffer_bytes(w);
    // from 256 units on: below 8 units per SM the kernel still pays, because a warp that reads its lane streams straight
    // from global memory stalls on every lane's cache line at a different moment (8192 x 2048, R = 16: 43 -> 16 us)
    constexpr int64_t min_units = 256;
    return room >= 8 && units >= min_units * std::max(1, a.ncols);
}

void gemv_staged(const bf16n_weight & w, const bf16n_mmv_args & a, cudaStream_t st, const bf16n_peer_out * peers) {
    const Cols p = make_cols(a, peers);
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
    if (units < sms * 8) { // few units: one per warp, spread over all SMs
        best = (int) std::max<int64_t>(1, std::min<int64_t>(max_warps, (units + sms - 1) / sms));
    }
    const dim3 grid((unsigned) std::min<int64_t>(sms, (units + best - 1) / best), (unsigned) a.ncols);
    const size_t shm = FIXED_SMEM + (size_t) best * cap;
    const AuxHeader * hdr = (const AuxHeader *) w.aux;
    const PairView v = pair_view(w);
    const Opaque k = {1u, 4u, ~0u, 32u};
#define GO(CC, TX) if (p.peers.n) { k_pair_gemv_staged<CC, TX, true><<<grid, best * 32, shm, st>>>(v, hdr, w.R, p, cap, k); } \
                   else { k_pair_gemv_staged<CC, TX, false><<<grid, best * 32, shm, st>>>(v, hdr, w.R, p, cap, k); }
    if (a.x_bf16) {
        switch (w.K / CHUNK) { case 1: GO(1, bf16); break; case 2: GO(2, bf16); break; default: GO(4, bf16); break; }
    } else {
        switch (w.K / CHUNK) { case 1: GO(1, float); break; case 2: GO(2, float); break; default: GO(4, float); break; }
    }
#undef GO
    check_launch();
}

} // namespace b16
