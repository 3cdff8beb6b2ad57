// Fragment-order HUFPAIR tensors (header flag 2, R = 16): exact reconstruction, row gather and the decode GEMV.
//
// Layout (core/src/encode.cpp:64-92, 387-394; docs/FORMAT.md "Fragment-order units"): rows come in bands of 16, a unit is
// one 512-column slab of a band (unit = band * K/512 + slab). Inside a slab the 16 x 16 tiles kt = 0..31 are walked in
// order; lane l owns, of every tile, the four column pairs q = 0..3 at row (l >> 2) + 8 * (q & 1), columns
// 2 * (l & 3) + 8 * (q >> 1) + {0, 1} (the A-operand registers of mma.m16n8k16). Its stream holds the pair symbols in the
// order tiles -> q; its plane bytes for the tile pair p = kt / 2 are the 16 bytes at band * 16 * K + p * 512 + l * 16
// (byte 8 * (kt & 1) + 2 * q + {0, 1}). Code tables and stream offsets are those of row-major units.
//
// The reference multiplies these fragments with mma.sync (core/include/bf16n/kernels.cuh:1507-2391). Here 2..8 dense BF16
// columns do the same (k_fo_gemv_mma: one decode and one mma.m16n8k16 per tile serve eight tokens; the tcgen05 path has
// no operand form for register fragments, so this small-N product stays on the warp-level instruction), while single
// columns, FP32 activations and routed columns use FMAs: a lane keeps two FP32 accumulators per column (its two rows)
// and the four lanes of a row quad are added at the end. Results are within FP32 rounding of FP64 either way (tested).
#include "staged.cuh"

#include <type_traits>
#include "launch.h"

namespace b16 {
namespace {

using namespace dev;
using bf16 = __nv_bfloat16;

constexpr int BAND = 16;

__device__ __forceinline__ void stage_lut(uint32_t * dst, const uint32_t * src) {
    for (int i = threadIdx.x; i < HP_MAX_PAIRS / 4; i += blockDim.x) { ((uint4 *) dst)[i] = __ldg((const uint4 *) src + i); }
}
// row (inside the band) and first column (inside the tile) of symbol q of lane l
__device__ __forceinline__ int frag_row(int l, int q) { return (l >> 2) + 8 * (q & 1); }
__device__ __forceinline__ int frag_col(int l, int q) { return 2 * (l & 3) + 8 * (q >> 1); }

// ---------------------------------------------------------------- exact reconstruction

struct FoStore { // row-major BF16 output, row 0 = row0
    uint16_t * out; int64_t K;
    __device__ __forceinline__ void pair(int64_t r, int64_t col, uint32_t w) { *(uint32_t *) (out + r * K + col) = w; }
    __device__ __forceinline__ void finish(int) {}
};
struct FoCompare { // count BF16 words that differ from src
    const uint16_t * src; int64_t K; unsigned long long * total; unsigned int bad;
    __device__ __forceinline__ void pair(int64_t r, int64_t col, uint32_t w) {
        const uint32_t d = __ldg((const uint32_t *) (src + r * K + col)) ^ w;
        bad += ((d & 0xFFFFu) != 0) + ((d >> 16) != 0);
    }
    __device__ __forceinline__ void finish(int lane) {
        unsigned int b = bad;
#pragma unroll
        for (int o = 16; o; o >>= 1) { b += __shfl_xor_sync(FULL, b, o); }
        if (lane == 0 && b) { atomicAdd(total, (unsigned long long) b); }
    }
};

// one warp per unit (band, slab) of rows [row0, row0 + nrows)
template <typename Sink>
__global__ void __launch_bounds__(256) k_fo_expand(const PairView w, int C, int64_t row0, int64_t nrows, const Sink sink_in) {
    Sink sink = sink_in;
    __shared__ uint32_t lut[HP_MAX_PAIRS];
    stage_lut(lut, w.lut);
    __syncthreads();
    const int64_t K = (int64_t) C * CHUNK;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t units = nrows / BAND * C;
    for (int64_t u = (int64_t) blockIdx.x * 8 + warp; u < units; u += (int64_t) gridDim.x * 8) {
        const int64_t band = u / C, slab = u - band * C, gband = row0 / BAND + band;
        PairReader rd;
        rd.open(w, gband * C + slab, lane);
        const uint8_t * pl = w.plane + gband * BAND * K + slab * (16 * 512) + 16 * lane;
        for (int p = 0; p < 16; p++) {
            uint32_t e[8], wv[8];
            rd.take8(lut, e);
            assemble8(ld_stream16(pl + p * 512), e, wv);
#pragma unroll
            for (int s = 0; s < 8; s++) {
                const int q = s & 3, kt = (int) slab * 32 + 2 * p + (s >> 2);
                sink.pair(band * BAND + frag_row(lane, q), (int64_t) kt * 16 + frag_col(lane, q), wv[s]);
            }
        }
    }
    sink.finish(lane);
}

// one warp per requested row: the four lanes of the row's quad decode their streams and keep the row's half
template <bool BF>
__global__ void __launch_bounds__(256) k_fo_rows(const PairView w, int C, const char * ids, int64_t ids_s0, int64_t n, int64_t row0,
                                                 char * dst, int64_t dst_s1) {
    __shared__ uint32_t lut[HP_MAX_PAIRS];
    stage_lut(lut, w.lut);
    __syncthreads();
    const int64_t K = (int64_t) C * CHUNK;
    const int j = threadIdx.x & 31;
    const int64_t i = (int64_t) blockIdx.x * 8 + (threadIdx.x >> 5);
    if (i >= n || j >= 4) { return; }
    const int64_t gr = row0 + *(const int32_t *) (ids + i * ids_s0);
    const int64_t band = gr / BAND;
    const int r = (int) (gr - band * BAND), l = 4 * (r & 7) + j, half = r >> 3;
    for (int slab = 0; slab < C; slab++) {
        PairReader rd;
        rd.open(w, band * C + slab, l);
        const uint8_t * pl = w.plane + band * BAND * K + (int64_t) slab * (16 * 512) + 16 * l;
        for (int p = 0; p < 16; p++) {
            uint32_t e[8], wv[8];
            rd.take8(lut, e);
            assemble8(ld_stream16(pl + p * 512), e, wv);
#pragma unroll
            for (int s = 0; s < 8; s++) {
                const int q = s & 3;
                if ((q & 1) != half) { continue; }
                const int64_t col = (int64_t) (slab * 32 + 2 * p + (s >> 2)) * 16 + frag_col(l, q);
                if (BF) { *(uint32_t *) (dst + i * dst_s1 + col * 2) = wv[s]; }
                else { *(float2 *) (dst + i * dst_s1 + col * 4) = make_float2(bf16lo_f32(wv[s]), bf16hi_f32(wv[s])); }
            }
        }
    }
}

// ---------------------------------------------------------------- decode GEMV

// NC dense columns (NC == 1: also routed columns, one per blockIdx.y); one warp per band, slabs in order
template <int NC, typename TX>
__global__ void __launch_bounds__(256) k_fo_gemv(const PairView w, int C, Cols p) {
    extern __shared__ __align__(16) unsigned char smem[];
    uint32_t * lut = (uint32_t *) smem;
    float * xs = (float *) (smem + 4 * HP_MAX_PAIRS);   // NC columns of K activations
    const int64_t K = (int64_t) C * CHUNK;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    stage_lut(lut, w.lut);
    grid_dependency_wait(); // activations (and expert ids) may come from the kernel before this one
    const TX * xg; OutVec out; int64_t rbase;
    column<TX>(p, NC == 1 ? blockIdx.y : 0, xg, out, rbase);
#pragma unroll
    for (int n = 0; n < NC; n++) {
        const TX * xn = (const TX *) ((const char *) xg + n * p.x_tok);
        for (int i = threadIdx.x; i < K; i += blockDim.x) { xs[n * K + i] = to_f32(xn[i]); }
    }
    __syncthreads();
    const int64_t bands = p.nrows / BAND;
    const int cq = 2 * (lane & 3); // this lane's columns inside a tile: cq + {0, 1} and cq + 8 + {0, 1}
    for (int64_t b = (int64_t) blockIdx.x * nwarp + warp; b < bands; b += (int64_t) gridDim.x * nwarp) {
        const int64_t gband = rbase / BAND + b;
        float acc[NC][2];
#pragma unroll
        for (int n = 0; n < NC; n++) { acc[n][0] = acc[n][1] = 0.f; }
        for (int slab = 0; slab < C; slab++) {
            PairReader rd;
            rd.open(w, gband * C + slab, lane);
            const uint8_t * pl = w.plane + gband * BAND * K + (int64_t) slab * (16 * 512) + 16 * lane;
            uint4 nxt = ld_stream16(pl);
            for (int pp = 0; pp < 16; pp++) {
                const uint4 cur = nxt;
                if (pp + 1 < 16) { nxt = ld_stream16(pl + (pp + 1) * 512); }
                uint32_t e[8], wv[8];
                rd.take8(lut, e);
                assemble8(cur, e, wv);
#pragma unroll
                for (int s = 0; s < 8; s++) {
                    const int q = s & 3;
                    const int col = (slab * 32 + 2 * pp + (s >> 2)) * 16 + cq + 8 * (q >> 1);
                    const float w0 = bf16lo_f32(wv[s]), w1 = bf16hi_f32(wv[s]);
#pragma unroll
                    for (int n = 0; n < NC; n++) {
                        const float2 xv = *(const float2 *) (xs + n * K + col);
                        acc[n][q & 1] = fmaf(w1, xv.y, fmaf(w0, xv.x, acc[n][q & 1]));
                    }
                }
            }
        }
#pragma unroll
        for (int n = 0; n < NC; n++) {
#pragma unroll
            for (int h = 0; h < 2; h++) {
                float v = acc[n][h];
                v += __shfl_xor_sync(FULL, v, 1);
                v += __shfl_xor_sync(FULL, v, 2);
                if ((lane & 3) == 0) {
                    OutVec o = out;
                    o.p += n * p.y_tok;
                    o.put(b * BAND + (lane >> 2) + 8 * h, v);
                }
            }
        }
    }
}

// One routed column per blockIdx.y for matrices of few bands (the routed experts of a decode step): the K / 512 slabs
// of a band go to as many warps, so that the dependent decode chain a warp walks is one unit long instead of K / 512;
// a block holds `nb` bands, a warp decodes exactly one unit. The slabs' partial sums meet in shared memory and are added
// in slab order. A warp here runs nearly alone on its SM and its unit comes cold from HBM; read lane by lane, every
// lane's stream line would stall the warp for a trip to L2 at a different moment. So the unit's stream block is copied
// into the warp's shared-memory buffer with one bulk copy and its plane pulled into L2, both started before the table
// and the activations are staged, and the plane is read four tile pairs ahead. A unit whose streams do not fit the
// buffer (more than 3 bits per weight) is read from global memory.
constexpr uint32_t FO_SPLIT_CAP = (BAND * CHUNK * 3 / 8 + 64 + 15) & ~15u;
constexpr int FO_GROUP = 2;      // routed columns of one expert that share a decode (4: 80 registers, a block fewer per SM: 96 against 81 us per layer when no experts are shared)
static_assert(FO_GROUP == 2 || FO_GROUP == 4, "k_fo_gemv_split specialises its loop for 1, 2, 3 and FO_GROUP members");
constexpr int FO_SPLIT_XPAD = 8; // BF16 elements of padding per activation row of the tensor-core form (as XPAD below)
// MMA = false: one column (routed or dense) on FMAs, FP32 or BF16 activations. MMA = true: up to 8 dense BF16 columns on
// mma.m16n8k16 (the activations are the B operand, columns beyond ncols are zero rows in shared memory).
// G > 1 (FMA form, routed columns of 4..8 tokens): columns that picked the same expert are multiplied by one decode. The
// block of column c first looks at the other columns' expert ids: if c is the first, G-th, 2G-th ... column with its
// expert it leads a group of up to G such columns (itself and the next ones) and the blocks of the group's other columns
// end at once. The leader's activations are staged in shared memory as before, the other members' are read from global
// memory in the loop, so a launch without shared experts keeps the occupancy of the ungrouped kernel. Every column keeps its own accumulators and the order of its additions, so a (token, slot) pair gets
// the same bits whatever else is in the batch (the reference's k_fo_mmv_grp / k_fo_mmv8_grp, core/include/bf16n/
// kernels.cuh:1839, 2003, group inside the kernel as well).
__device__ __forceinline__ float2 load_x2(const float * p) { return *(const float2 *) p; }
__device__ __forceinline__ float2 load_x2(const bf16 * p) {
    const uint32_t v = *(const uint32_t *) p;
    return make_float2(bf16lo_f32(v), bf16hi_f32(v));
}

template <typename TX, bool MMA, int G = 1>
__global__ void __launch_bounds__(256, G > 1 ? 4 : 1) k_fo_gemv_split(const PairView w, const AuxHeader * hdr, int C, Cols p, int nb, int ncols, const Opaque k) {
    static_assert(!MMA || G == 1, "grouping is for the FMA form");
    extern __shared__ __align__(128) unsigned char smem[];
    uint32_t * lut = (uint32_t *) smem;
    uint64_t * bars = (uint64_t *) (smem + 4 * HP_MAX_PAIRS); // one per warp
    const int64_t K = (int64_t) C * CHUNK;
    const int XS = (int) K + FO_SPLIT_XPAD;
    float * xs = (float *) (smem + 4 * HP_MAX_PAIRS + 128);              // MMA: 8 rows of XS BF16 values instead
    bf16 * xh = (bf16 *) xs;
    float * part = MMA ? (float *) (xh + 8 * XS) : xs + K;               // [band of the block][slab][16 rows | 32 lanes x 4 | G x 16 rows]
    constexpr int PART = MMA ? 128 : 16 * G;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned char * buf = (unsigned char *) (part + nb * C * PART) + (size_t) warp * FO_SPLIT_CAP;
    const int j = warp / C, slab = warp - j * C;
    const uint32_t bar = smem_u32(bars + warp);
    if (lane == 0) { mbar_init(bar, 1); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncwarp();
    grid_dependency_wait(); // activations and expert ids may come from the kernel before this one
    const TX * xg; OutVec out; int64_t rbase;
    column<TX>(p, MMA ? 0 : blockIdx.y, xg, out, rbase);
    int members[G];   // the columns this block multiplies ([0]: its own)
    int m = 1;
    members[0] = MMA ? 0 : (int) blockIdx.y;
    if constexpr (G > 1) {
        // expert id of column c: the same lookup as column(); lanes cover the (at most 64) columns
        auto expert_of = [&](int c) {
            const int t = c / p.n_used, sl = c - t * p.n_used;
            return *(const int32_t *) (p.ids + t * p.ids_s1 + sl * p.ids_s0);
        };
        const int c = (int) blockIdx.y, e = expert_of(c);
        const unsigned lo = __ballot_sync(FULL, lane < ncols && expert_of(lane) == e);
        const unsigned hi = __ballot_sync(FULL, lane + 32 < ncols && expert_of(lane + 32) == e);
        const unsigned long long same = (unsigned long long) hi << 32 | lo;
        const int before = __popcll(same & ((1ull << c) - 1ull));
        if (before % G != 0) { return; }    // another block leads this column's group (the whole block takes this branch)
        unsigned long long later = same >> c >> 1;
        for (int cc = c + 1; later && m < G; cc++, later >>= 1) {
            if (later & 1ull) { members[m++] = cc; }
        }
    }
    // where the other members' activations start (byte offsets from p.x: three registers), looked up once and here
    uint32_t xoff[G];
    xoff[0] = 0;
#pragma unroll
    for (int g = 1; g < G; g++) {
        xoff[g] = 0;
        if (g < m) {
            const TX * xm; OutVec om; int64_t rb;
            column<TX>(p, members[g], xm, om, rb);
            xoff[g] = (uint32_t) ((const char *) xm - p.x);
        }
    }
    const int64_t bands = p.nrows / BAND, b = (int64_t) blockIdx.x * nb + j;
    const bool active = b < bands;
    const int64_t unit = active ? (rbase / BAND + b) * C + slab : 0;
    uint32_t w0 = 0, my = 0, bytes = 0;
    if (active) {
        const uint32_t n_units = (uint32_t) hdr->n_a, n_words = (uint32_t) hdr->n_b;
        w0 = __ldg(w.ubase + unit);
        const uint32_t w1 = unit + 1 < (int64_t) n_units ? __ldg(w.ubase + unit + 1) : n_words, start = w0 & ~3u;
        bytes = ((w1 - start + 4u + 3u) & ~3u) * 4u;
        my = __ldg(w.lrel + unit * 32 + lane);
        if (lane == 0) {
            if (bytes <= FO_SPLIT_CAP) {
                mbar_expect_tx(bar, bytes);
                bulk_g2s(smem_u32(buf), w.stream + start, bytes, bar);
            }
            bulk_prefetch_l2(w.plane + unit * (BAND * CHUNK), BAND * CHUNK);
        }
    }
    stage_lut(lut, w.lut);
    if constexpr (MMA) {
        for (int i = threadIdx.x; i < 8 * (int) K; i += blockDim.x) {
            const int n = i / (int) K, c = i - n * (int) K;
            xh[n * XS + c] = n < ncols ? ((const bf16 *) (p.x + n * p.x_tok))[c] : __float2bfloat16(0.f);
        }
    } else {
        // the leader's activations are staged as FP32; further members of a group are read from global memory in the
        // loop (staging all of them would cost a block of every SM, grouped or not)
        for (int i = threadIdx.x; i < K; i += blockDim.x) { xs[i] = to_f32(xg[i]); }
    }
    __syncthreads();
    const int cq = 2 * (lane & 3), g8 = lane >> 2, t4 = lane & 3;
    float acc[MMA ? 4 : 2 * G]; // FMA form: [2 g], [2 g + 1] = rows g8, g8 + 8 of this lane's columns for member g; MMA form: the D fragment
#pragma unroll
    for (int i = 0; i < (MMA ? 4 : 2 * G); i++) { acc[i] = 0.f; }
    if (active) {
        const uint8_t * pl = w.plane + unit * (BAND * CHUNK) + 16 * lane;
        const bf16 * xl = xh + g8 * XS + 2 * t4; // B fragment: token g8, k = 2 t4, + 1 (and + 8) of every tile
        // mm: the number of grouped columns as a compile-time constant (no predicated-off FMAs for absent members)
        auto body = [&](auto & rd, uint32_t lut_arg, auto mm) {
            constexpr int M = decltype(mm)::value;
            uint4 ring[4];
#pragma unroll
            for (int i = 0; i < 4; i++) { ring[i] = ld_stream16(pl + i * 512); }
            for (int pp4 = 0; pp4 < 16; pp4 += 4) {
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int pp = pp4 + i;
                    const uint4 cur = ring[i];
                    if (pp + 4 < 16) { ring[i] = ld_stream16(pl + (pp + 4) * 512); }
                    uint32_t e[8], wv[8];
                    rd.take8(lut_arg, k, e);
                    assemble8(cur, e, wv);
                    if constexpr (MMA) {
#pragma unroll
                        for (int kk = 0; kk < 2; kk++) {
                            const int col = (slab * 32 + 2 * pp + kk) * 16;
                            const uint32_t b0 = *(const uint32_t *) (xl + col), b1 = *(const uint32_t *) (xl + col + 8);
                            asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
                                         "{%0, %1, %2, %3};"
                                         : "+f"(acc[0]), "+f"(acc[1]), "+f"(acc[2]), "+f"(acc[3])
                                         : "r"(wv[4 * kk]), "r"(wv[4 * kk + 1]), "r"(wv[4 * kk + 2]), "r"(wv[4 * kk + 3]), "r"(b0), "r"(b1));
                        }
                    } else {
#pragma unroll
                        for (int q8 = 0; q8 < 8; q8++) {
                            const int q = q8 & 3;
                            const float wl = bf16lo_f32(wv[q8]), wh = bf16hi_f32(wv[q8]);
                            const int xi = (slab * 32 + 2 * pp + (q8 >> 2)) * 16 + cq + 8 * (q >> 1);
                            const float2 x0 = *(const float2 *) (xs + xi);
                            acc[q & 1] = fmaf(wh, x0.y, fmaf(wl, x0.x, acc[q & 1]));
#pragma unroll
                            for (int g = 1; g < M; g++) { // the other members' activations come straight from global memory (L1)
                                const float2 xv = load_x2((const TX *) (p.x + xoff[g]) + xi);
                                acc[2 * g + (q & 1)] = fmaf(wh, xv.y, fmaf(wl, xv.x, acc[2 * g + (q & 1)]));
                            }
                        }
                    }
                }
            }
        };
        auto by_members = [&](auto & rd, uint32_t lut_arg) {
            if constexpr (G == 1) { body(rd, lut_arg, std::integral_constant<int, 1>{}); }
            else {
                if (m == 1) { body(rd, lut_arg, std::integral_constant<int, 1>{}); }
                else if (G == 2 || m == 2) { body(rd, lut_arg, std::integral_constant<int, 2>{}); }
                else if (m == 3) { body(rd, lut_arg, std::integral_constant<int, (G > 2 ? 3 : 2)>{}); }
                else { body(rd, lut_arg, std::integral_constant<int, G>{}); }
            }
        };
        if (bytes <= FO_SPLIT_CAP) {
            const uint32_t landed = mbar_wait(bar, 0u);
            if (landed) {
                StagedReader rd;
                rd.open(smem_u32(buf) + 4 * (w0 - (w0 & ~3u) + my), landed);
                by_members(rd, smem_u32(lut));
            } else { // the copy never arrived: the flag reports it and the band's outputs become NaN
                if (lane == 0) { atomicOr(&g_wait_expired, 1u); }
#pragma unroll
                for (int i = 0; i < (MMA ? 4 : 2 * G); i++) { acc[i] = __int_as_float(0x7fc00000); }
            }
        } else {
            GlobalReader rd;
            rd.lut = lut;
            rd.rd.open(w, unit, lane);
            by_members(rd, 0u);
        }
    }
    float * mine = part + (j * C + slab) * PART;
    if constexpr (MMA) {
#pragma unroll
        for (int i = 0; i < 4; i++) { mine[i * 32 + lane] = acc[i]; }
    } else {
#pragma unroll
        for (int h = 0; h < 2 * G; h++) {
            float v = acc[h];
            v += __shfl_xor_sync(FULL, v, 1);
            v += __shfl_xor_sync(FULL, v, 2);
            if ((lane & 3) == 0) { mine[(h >> 1) * 16 + (lane >> 2) + 8 * (h & 1)] = v; }
        }
    }
    __syncthreads();
    if (slab != 0 || !active) { return; }
    const float * sums = part + j * C * PART;
    if constexpr (MMA) { // D fragment: [0], [1] = row g8, tokens 2 t4, + 1; [2], [3] = row g8 + 8
#pragma unroll
        for (int i = 0; i < 4; i++) {
            float v = sums[i * 32 + lane];
            for (int s2 = 1; s2 < C; s2++) { v += sums[s2 * PART + i * 32 + lane]; }
            const int n = 2 * t4 + (i & 1);
            if (n < ncols) {
                const OutVec o = {p.y + n * p.y_tok, p.y_bf16};
                o.put(b * BAND + g8 + 8 * (i >> 1), v);
            }
        }
    } else if (lane < 16) {
#pragma unroll
        for (int g = 0; g < G; g++) {
            if (g < m) {
                float v = sums[g * 16 + lane];
                for (int s2 = 1; s2 < C; s2++) { v += sums[s2 * PART + g * 16 + lane]; }
                if (g == 0) { out.put(b * BAND + lane, v); }
                else {
                    const TX * xm; OutVec om; int64_t rb;
                    column<TX>(p, members[g], xm, om, rb);
                    om.put(b * BAND + lane, v);
                }
            }
        }
    }
}

// Up to 8 dense BF16 columns on the tensor cores: a lane's four symbols of a tile are exactly its A registers of
// mma.m16n8k16 (that is what the layout is for), the activations are the B operand (k x 8 tokens) and a band's
// D[16 rows, 8 tokens] accumulates in four registers per lane, so eight tokens cost one decode and one MMA per tile.
// Shared memory holds the 8 activation rows as BF16, each padded by 8 elements so that the B-fragment reads of a warp
// fall into 32 different banks; columns beyond ncols are zero.
constexpr int XPAD = 8;
constexpr int FO_BARS = 512; // room for two mbarriers per warp of the staged kernel (up to 32 warps)
__global__ void __launch_bounds__(512) k_fo_gemv_mma(const PairView w, int C, Cols p, int ncols, int64_t n_units) {
    extern __shared__ __align__(16) unsigned char smem[];
    uint32_t * lut = (uint32_t *) smem;
    bf16 * xs = (bf16 *) (smem + 4 * HP_MAX_PAIRS);
    const int K = C * CHUNK, XS = K + XPAD;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    stage_lut(lut, w.lut);
    grid_dependency_wait();
    for (int i = threadIdx.x; i < 8 * K; i += blockDim.x) {
        const int n = i / K, c = i - n * K;
        xs[n * XS + c] = n < ncols ? ((const bf16 *) (p.x + n * p.x_tok))[c] : __float2bfloat16(0.f);
    }
    __syncthreads();
    const int g = lane >> 2, t = lane & 3;
    const bf16 * xl = xs + g * XS + 2 * t; // B fragment: token g, k = 2t, 2t+1 (and + 8) of every tile
    const int64_t bands = p.nrows / BAND, stride = (int64_t) gridDim.x * nwarp;
    // while a unit is decoded, the next unit's stream start and first three words are loaded and its plane and stream
    // bytes are pulled into L2
    bool preloaded = false;
    const uint32_t * pfirst = nullptr;
    uint32_t p0 = 0, p1 = 0, p2 = 0;
    for (int64_t b = (int64_t) blockIdx.x * nwarp + warp; b < bands; b += stride) {
        const int64_t gband = p.row0 / BAND + b;
        float d[4] = {0.f, 0.f, 0.f, 0.f};
        for (int slab = 0; slab < C; slab++) {
            const int64_t unit = gband * C + slab;
            const int64_t nu = slab + 1 < C ? unit + 1 : b + stride < bands ? (gband + stride) * C : -1;
            uint32_t ub_n = 0, ub_n1 = 0, lr_n = 0;
            if (nu >= 0) {
                ub_n = __ldg(w.ubase + nu);
                ub_n1 = nu + 1 < n_units ? __ldg(w.ubase + nu + 1) : ub_n;
                lr_n = __ldg(w.lrel + nu * 32 + lane);
                if (lane == 0) { bulk_prefetch_l2(w.plane + nu * (BAND * CHUNK), BAND * CHUNK); }
            }
            PairReader rd;
            if (preloaded) { rd.open_loaded(pfirst, p0, p1, p2); } else { rd.open(w, unit, lane); }
            preloaded = false;
            const uint8_t * pl = w.plane + unit * (BAND * CHUNK) + 16 * lane;
            uint4 nxt = ld_stream16(pl);
#pragma unroll 1
            for (int pp = 0; pp < 16; pp++) {
                if (nu >= 0) {
                    if (pp == 3 && lane == 0 && ub_n1 > ub_n) {
                        const uint32_t first = ub_n & ~3u;
                        bulk_prefetch_l2(w.stream + first, ((ub_n1 - first + 3u) & ~3u) * 4u);
                    }
                    if (pp == 9) {
                        pfirst = w.stream + (ub_n + lr_n);
                        p0 = __ldg(pfirst);
                        p1 = __ldg(pfirst + 1);
                        p2 = __ldg(pfirst + 2);
                        preloaded = true;
                    }
                }
                const uint4 cur = nxt;
                if (pp + 1 < 16) { nxt = ld_stream16(pl + (pp + 1) * 512); }
                uint32_t e[8], a[8];
                rd.take8(lut, e);
                assemble8(cur, e, a);
#pragma unroll
                for (int kk = 0; kk < 2; kk++) {
                    const int col = (slab * 32 + 2 * pp + kk) * 16;
                    const uint32_t b0 = *(const uint32_t *) (xl + col), b1 = *(const uint32_t *) (xl + col + 8);
                    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
                                 "{%0, %1, %2, %3};"
                                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                                 : "r"(a[4 * kk]), "r"(a[4 * kk + 1]), "r"(a[4 * kk + 2]), "r"(a[4 * kk + 3]), "r"(b0), "r"(b1));
                }
            }
        }
        // d[0], d[1]: row g, tokens 2t, 2t+1; d[2], d[3]: row g + 8
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int n = 2 * t + (i & 1);
            if (n < ncols) {
                const OutVec o = {p.y + n * p.y_tok, p.y_bf16};
                o.put(b * BAND + g + 8 * (i >> 1), d[i]);
            }
        }
    }
}

// ---------------------------------------------------------------- batched routed product (prefill)

// dst[t, slot, :] = W_e x_t for every routed (token, slot) pair, optionally fused gate/up + SwiGLU, for fragment-order
// experts (replaces the reference's k_fo_mm_ids / k_fo_mm_glu, kernels.cuh:2070-2391). One persistent block of 16 warps
// per SM. An item is (expert, tile of up to 96 of its routed tokens, group of bands); a warp owns one band of the group
// (GLU: warps 0-7 the gate bands, warps 8-15 the same bands of up) and keeps D[16 rows, 96 tokens] in registers over the
// K / 512 slabs, so every weight is decoded once per (expert, token tile). The work is a sequence of steps (item, slab):
// while a step is multiplied, the next step's activation rows are gathered into the other of two shared-memory buffers
// with 16-byte asynchronous copies (one block barrier per step), the next unit's stream position and first three stream
// words are loaded, and its plane and stream bytes are pulled into L2. Activation rows are 1024 bytes, their 16-byte
// pieces XOR-swizzled by the row's low three bits so that ldmatrix reads eight rows without a bank conflict and no
// padding is spent. SwiGLU: gate and up warps swap halves of their sums through the buffer just consumed, each then
// finishes and stores half of the tile's tokens.
constexpr int FO_TOK = 96;                      // tokens per tile
constexpr int FO_NG = FO_TOK / 8;               // 8-token groups of a tile (multiplied in pairs)
constexpr int FO_WARPS = 16;
constexpr int FO_ROWB = CHUNK * 2;              // bytes of one staged activation row
constexpr int FO_BUF = FO_TOK * FO_ROWB;
static_assert(FO_NG % 2 == 0 && FO_WARPS * (FO_NG / 2) * 4 * 32 * 4 <= FO_BUF, "the swapped sums must fit one buffer");

struct FoBatch {
    PairView w0, w1;
    const bf16 * x; int64_t x_row;
    const int32_t * ids_src1; const int32_t * ids_dst; const int32_t * bounds;
    char * dst; int64_t dst_col; bool dst_bf16;
    int n_experts, C;
    int64_t rows_per_expert, n_units;
};

struct FoItem { int it, e, jb, ntok; int64_t band; bool valid, live; };

template <bool GLU>
__global__ void __launch_bounds__(FO_WARPS * 32, 1) k_fo_mm_ids(const FoBatch p) {
    constexpr int NB = GLU ? FO_WARPS / 2 : FO_WARPS; // bands of a group
    extern __shared__ __align__(16) unsigned char smem[];
    uint32_t * lut0 = (uint32_t *) smem;
    uint32_t * lut1 = lut0 + (GLU ? HP_MAX_PAIRS : 0);
    unsigned char * xb = (unsigned char *) (lut1 + HP_MAX_PAIRS);  // two buffers of FO_BUF
    int32_t * toff = (int32_t *) (xb + 2 * FO_BUF);                // first tile of each expert, E + 1
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, E = p.n_experts, C = p.C;
    const bool upw = GLU && warp >= NB;
    const PairView & w = upw ? p.w1 : p.w0;
    const uint32_t * lut = upw ? lut1 : lut0;
    stage_lut(lut0, p.w0.lut);
    if (GLU) { stage_lut(lut1, p.w1.lut); }
    {   // tiles per expert (parked in the first buffer), then their exclusive prefix
        int32_t * cnt = (int32_t *) xb;
        for (int e = threadIdx.x; e < E; e += blockDim.x) { cnt[e] = (p.bounds[e + 1] - p.bounds[e] + FO_TOK - 1) / FO_TOK; }
        __syncthreads();
        for (int e = threadIdx.x; e <= E; e += blockDim.x) {
            int run = 0;
            for (int i = 0; i < e; i++) { run += cnt[i]; }
            toff[e] = run;
        }
        __syncthreads();
    }
    const int64_t bands_e = p.rows_per_expert / BAND;
    const int nbg = (int) ((bands_e + NB - 1) / NB);
    const int n_items = toff[E] * nbg;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t xs_s = smem_u32(xb);
    const uint32_t xrow = xs_s + (uint32_t) (((lane >> 4) * 8 + (lane & 7)) * FO_ROWB);
    const uint32_t khalf = (lane >> 3) & 1, l7 = lane & 7;

    auto item_at = [&](int it) {
        FoItem r = {};
        r.it = it;
        r.valid = it < n_items;
        if (!r.valid) { return r; }
        const int tile = it / nbg;
        int lo = 0, hi = E; // the largest e with toff[e] <= tile: its tiles are toff[e] .. toff[e + 1] - 1
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (toff[mid] <= tile) { lo = mid; } else { hi = mid; }
        }
        r.e = lo;
        r.jb = __ldg(p.bounds + lo) + (tile - toff[lo]) * FO_TOK;
        r.ntok = min(FO_TOK, __ldg(p.bounds + lo + 1) - r.jb);
        r.band = (int64_t) (it - tile * nbg) * NB + (warp & (NB - 1));
        r.live = r.band < bands_e;
        return r;
    };
    // a thread copies one 16-byte piece of every 8th row: the row ids are all loaded before the first copy is issued
    auto stage = [&](const FoItem & im, int slab, int b) { // missing tokens of the last pair of groups: zero fill
        const int rows = ((im.ntok + 15) >> 4) << 4, row0 = threadIdx.x >> 6, piece = threadIdx.x & 63;
        int32_t tok[FO_TOK / 8];
#pragma unroll
        for (int i = 0; i < FO_TOK / 8; i++) {
            const int row = row0 + 8 * i;
            tok[i] = row < im.ntok ? __ldg(p.ids_src1 + im.jb + row) : -1;
        }
        const uint32_t to = xs_s + (uint32_t) (b * FO_BUF + row0 * FO_ROWB + ((piece ^ row0) << 4));
        const bf16 * from = p.x + slab * CHUNK + piece * 8;
#pragma unroll
        for (int i = 0; i < FO_TOK / 8; i++) {
            if (row0 + 8 * i < rows) {
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(to + (uint32_t) (8 * i * FO_ROWB)),
                             "l"(from + (tok[i] >= 0 ? (int64_t) tok[i] * p.x_row : 0)), "r"(tok[i] >= 0 ? 16u : 0u) : "memory");
            }
        }
    };

    FoItem cur = item_at(blockIdx.x);
    if (cur.valid) { stage(cur, 0, 0); }
    asm volatile("cp.async.commit_group;" ::: "memory");
    int step = 0;
    bool preloaded = false; // the next unit's stream start and first three words are in registers
    const uint32_t * pfirst = nullptr;
    uint32_t p0 = 0, p1 = 0, p2 = 0;
    while (cur.valid) {
        const FoItem nxt = item_at(cur.it + gridDim.x);
        const int ng = (cur.ntok + 7) >> 3;
        const int64_t unit0 = ((int64_t) cur.e * bands_e + cur.band) * C;
        float acc[FO_NG][4];
#pragma unroll
        for (int i = 0; i < FO_NG; i++) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }
        int b = 0;
        for (int slab = 0; slab < C; slab++, step++) {
            b = step & 1;
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            __syncthreads(); // this step's rows have landed; every warp is done with the other buffer
            if (slab + 1 < C) { stage(cur, slab + 1, b ^ 1); } else if (nxt.valid) { stage(nxt, 0, b ^ 1); }
            asm volatile("cp.async.commit_group;" ::: "memory");
            if (!cur.live) { continue; }
            int64_t nu = -1; // this warp's next unit
            if (slab + 1 < C) { nu = unit0 + slab + 1; } else if (nxt.valid && nxt.live) { nu = ((int64_t) nxt.e * bands_e + nxt.band) * C; }
            uint32_t ub_n = 0, ub_n1 = 0, lr_n = 0;
            if (nu >= 0) {
                ub_n = __ldg(w.ubase + nu);
                ub_n1 = nu + 1 < p.n_units ? __ldg(w.ubase + nu + 1) : ub_n;
                lr_n = __ldg(w.lrel + nu * 32 + lane);
                if (lane == 0) { bulk_prefetch_l2(w.plane + nu * (BAND * CHUNK), BAND * CHUNK); }
            }
            PairReader rd;
            if (preloaded) { rd.open_loaded(pfirst, p0, p1, p2); } else { rd.open(w, unit0 + slab, lane); }
            preloaded = false;
            const uint8_t * pl = w.plane + (unit0 + slab) * (BAND * CHUNK) + 16 * lane;
            const uint32_t xbuf = xrow + (uint32_t) (b * FO_BUF);
            uint4 nx = ld_stream16(pl);
#pragma unroll 1
            for (int pp = 0; pp < 16; pp++) {
                if (nu >= 0) {
                    if (pp == 3 && lane == 0 && ub_n1 > ub_n) {
                        const uint32_t first = ub_n & ~3u;
                        bulk_prefetch_l2(w.stream + first, ((ub_n1 - first + 3u) & ~3u) * 4u);
                    }
                    if (pp == 9) {
                        pfirst = w.stream + (ub_n + lr_n);
                        p0 = __ldg(pfirst);
                        p1 = __ldg(pfirst + 1);
                        p2 = __ldg(pfirst + 2);
                        preloaded = true;
                    }
                }
                const uint4 cu = nx;
                if (pp + 1 < 16) { nx = ld_stream16(pl + (pp + 1) * 512); }
                uint32_t en[8], a[8];
                rd.take8(lut, en);
                assemble8(cu, en, a);
#pragma unroll
                for (int kk = 0; kk < 2; kk++) {
                    // B fragments of two token groups per ldmatrix.x4: lane 8j + r addresses row r of 8x8 matrix j =
                    // (token group i + (j >> 1), k half j & 1); rows are tokens, 16 bytes of k each
                    const uint32_t xaddr = xbuf + ((((uint32_t) (4 * pp + 2 * kk) + khalf) ^ l7) << 4);
#pragma unroll
                    for (int i = 0; i < FO_NG; i += 2) {
                        if (i < ng) {
                            uint32_t b0, b1, b2, b3;
                            asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                                         : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(xaddr + (uint32_t) (i * 8 * FO_ROWB)));
                            asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
                                         "{%8, %9}, {%0, %1, %2, %3};"
                                         : "+f"(acc[i][0]), "+f"(acc[i][1]), "+f"(acc[i][2]), "+f"(acc[i][3])
                                         : "r"(a[4 * kk]), "r"(a[4 * kk + 1]), "r"(a[4 * kk + 2]), "r"(a[4 * kk + 3]), "r"(b0), "r"(b1));
                            asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
                                         "{%8, %9}, {%0, %1, %2, %3};"
                                         : "+f"(acc[i + 1][0]), "+f"(acc[i + 1][1]), "+f"(acc[i + 1][2]), "+f"(acc[i + 1][3])
                                         : "r"(a[4 * kk]), "r"(a[4 * kk + 1]), "r"(a[4 * kk + 2]), "r"(a[4 * kk + 3]), "r"(b2), "r"(b3));
                        }
                    }
                }
            }
        }
        // acc[i][0..1]: row g, tokens 8i + 2t, + 1; acc[i][2..3]: row g + 8
        auto put = [&](int i, int c, float v) {
            const int tok = 8 * i + 2 * t + (c & 1);
            if (cur.live && tok < cur.ntok) {
                const int64_t at = (int64_t) __ldg(p.ids_dst + cur.jb + tok) * p.dst_col + cur.band * BAND + g + 8 * (c >> 1);
                if (p.dst_bf16) { ((bf16 *) p.dst)[at] = __float2bfloat16_rn(v); } else { ((float *) p.dst)[at] = v; }
            }
        };
        if (GLU) {
            constexpr int H = FO_NG / 2; // the gate warp finishes groups 0 .. H - 1, the up warp the rest
            __syncthreads(); // every warp is done with this step's activations: the buffer now carries the swapped sums
            float * red = (float *) (xb + b * FO_BUF);
#pragma unroll
            for (int n = 0; n < H; n++) { // constant register indices on both sides of the branch
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    float * at = red + ((warp * H + n) * 4 + c) * 32 + lane;
                    if (upw) { *at = acc[n][c]; } else { *at = acc[H + n][c]; }
                }
            }
            __syncthreads();
            const float * theirs = red + (warp ^ NB) * H * 4 * 32 + lane;
#pragma unroll
            for (int n = 0; n < H; n++) {
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    const float other = theirs[(n * 4 + c) * 32];
                    if (upw) { put(H + n, c, silu_f(other) * acc[H + n][c]); } else { put(n, c, silu_f(acc[n][c]) * other); }
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < FO_NG; i++) {
                if (i < ng) {
#pragma unroll
                    for (int c = 0; c < 4; c++) { put(i, c, acc[i][c]); }
                }
            }
        }
        cur = nxt;
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// The same product with the streams staged: one persistent block per SM of up to 32 warps, a warp walks bands and copies each slab's
// stream block into its own shared-memory buffer with one bulk async copy (two buffers in turn, so the next slab's copy
// runs under the current slab's decoding; bounded wait, as in gemv_staged.cu), reads it with the staged reader and
// prefetches the plane bytes one tile pair ahead. Serves 1..8 dense BF16 columns. A slab whose streams do not fit the
// buffer (more than 3 bits per weight) is read straight from global memory.
constexpr uint32_t FO_CAP = (BAND * CHUNK * 3 / 8 + 64 + 15) & ~15u;

__global__ void __launch_bounds__(1024) k_fo_gemv_staged(const PairView w, const AuxHeader * hdr, int C, Cols p, int ncols, const Opaque k) {
    extern __shared__ __align__(128) unsigned char smem[];
    uint32_t * lut = (uint32_t *) smem;
    uint64_t * bars = (uint64_t *) (smem + 4 * HP_MAX_PAIRS);            // two per warp
    const int K = C * CHUNK, XS = K + XPAD;
    bf16 * xs = (bf16 *) (smem + 4 * HP_MAX_PAIRS + FO_BARS);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    unsigned char * buf = smem + 4 * HP_MAX_PAIRS + FO_BARS + (size_t) 8 * XS * 2 + (size_t) warp * 2 * FO_CAP;
    stage_lut(lut, w.lut);
    if (lane == 0) { mbar_init(smem_u32(bars + 2 * warp), 1); mbar_init(smem_u32(bars + 2 * warp + 1), 1); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    grid_dependency_wait();
    for (int i = threadIdx.x; i < 8 * (K / 8); i += blockDim.x) { // 16-byte pieces; columns beyond ncols are zero
        const int n = i / (K / 8), c = i - n * (K / 8);
        const uint4 v = n < ncols ? ld_act16((const uint4 *) (p.x + n * p.x_tok) + c) : make_uint4(0, 0, 0, 0);
        *(uint4 *) (xs + n * XS + c * 8) = v;
    }
    const uint32_t n_units = (uint32_t) hdr->n_a, n_words = (uint32_t) hdr->n_b;
    __syncthreads();
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
    auto stage = [&](const Geo & g, int b) { // one lane starts the copy of a slab's streams into buffer b
        if (g.bytes <= FO_CAP && lane == 0) {
            const uint32_t bar = smem_u32(bars + 2 * warp + b);
            mbar_expect_tx(bar, g.bytes);
            bulk_g2s(smem_u32(buf + b * FO_CAP), w.stream + g.start, g.bytes, bar);
        }
    };
    const int g8 = lane >> 2, t4 = lane & 3;
    const bf16 * xl = xs + g8 * XS + 2 * t4;
    uint32_t parity = 0u; // bit b: phase of buffer b's barrier
    bool dead = false;    // a bulk copy of this warp never arrived: no further copies, NaN outputs
    const int64_t bands = p.nrows / BAND;
    for (int64_t b = (int64_t) blockIdx.x * nwarp + warp; b < bands; b += (int64_t) gridDim.x * nwarp) {
        const int64_t gband = p.row0 / BAND + b;
        float d[4] = {0.f, 0.f, 0.f, 0.f};
        Geo cur = geometry(gband * C);
        __syncwarp(); // every lane is done with both buffers (previous band)
        if (!dead) { stage(cur, 0); }
        for (int slab = 0; slab < C && !dead; slab++) {
            Geo nxt = {0, 0, 0};
            if (slab + 1 < C) {
                nxt = geometry(gband * C + slab + 1);
                __syncwarp(); // the buffer about to be refilled was read two slabs ago by every lane
                stage(nxt, (slab + 1) & 1);
            }
            const uint8_t * pl = w.plane + gband * BAND * (int64_t) K + (int64_t) slab * (16 * 512) + 16 * lane;
            if (lane == 0) { // the next unit's plane bytes into L2 (the next slab, or the first slab of this warp's next band)
                const int64_t nb = b + (int64_t) gridDim.x * nwarp;
                if (slab + 1 < C) { bulk_prefetch_l2(pl + 16 * 512, 16 * 512); }
                else if (nb < bands) { bulk_prefetch_l2(w.plane + (p.row0 / BAND + nb) * BAND * (int64_t) K, 16 * 512); }
            }
            auto body = [&](auto & rd, uint32_t lut_arg) {
                uint4 nx = ld_stream16(pl);
                for (int pp = 0; pp < 16; pp++) {
                    const uint4 cu = nx;
                    if (pp + 1 < 16) { nx = ld_stream16(pl + (pp + 1) * 512); }
                    uint32_t e[8], a[8];
                    rd.take8(lut_arg, k, e);
                    assemble8(cu, e, a);
#pragma unroll
                    for (int kk = 0; kk < 2; kk++) {
                        const int col = (slab * 32 + 2 * pp + kk) * 16;
                        const uint32_t b0 = *(const uint32_t *) (xl + col), b1 = *(const uint32_t *) (xl + col + 8);
                        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
                                     "{%0, %1, %2, %3};"
                                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                                     : "r"(a[4 * kk]), "r"(a[4 * kk + 1]), "r"(a[4 * kk + 2]), "r"(a[4 * kk + 3]), "r"(b0), "r"(b1));
                    }
                }
            };
            if (cur.bytes <= FO_CAP) {
                const int bi = slab & 1;
                const uint32_t landed = mbar_wait(smem_u32(bars + 2 * warp + bi), (parity >> bi) & 1u);
                if (!landed) { // the copy never arrived: this band and the warp's later bands are written as NaN
                    if (lane == 0) { atomicOr(&g_wait_expired, 1u); }
                    dead = true;
                    break;
                }
                parity ^= 1u << bi;
                StagedReader rd;
                rd.open(smem_u32(buf + bi * FO_CAP) + 4 * cur.my, landed);
                body(rd, smem_u32(lut));
            } else {
                GlobalReader rd;
                rd.lut = lut;
                rd.rd.open(w, gband * C + slab, lane);
                body(rd, 0u);
            }
            cur = nxt;
        }
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int n = 2 * t4 + (i & 1);
            if (n < ncols) {
                const OutVec o = {p.y + n * p.y_tok, p.y_bf16};
                o.put(b * BAND + g8 + 8 * (i >> 1), dead ? __int_as_float(0x7fc00000) : d[i]);
            }
        }
    }
}

template <int NC, typename TX>
void launch_fo(const bf16n_weight & w, const Cols & p, int ncols_grid, cudaStream_t st) {
    const int C = (int) (w.K / CHUNK);
    const int64_t bands = p.nrows / BAND;
    const int64_t sms = device_info().sms;
    // small blocks while there are few bands, so that they spread over the SMs
    const int warps = bands * ncols_grid >= sms * 32 ? 8 : bands * ncols_grid >= sms * 8 ? 4 : 2;
    const dim3 grid((unsigned) std::min<int64_t>((bands + warps - 1) / warps, sms * 8), (unsigned) ncols_grid);
    const size_t shm = 4 * HP_MAX_PAIRS + (size_t) NC * w.K * 4;
    launch_chained(k_fo_gemv<NC, TX>, grid, dim3(warps * 32), shm, st, pair_view(w), C, p);
}

template <typename TX>
void fo_gemv_t(const bf16n_weight & w, const bf16n_mmv_args & a, cudaStream_t st) {
    Cols p = make_cols(a);
    // routed columns, and a single dense column of a small matrix: the kernels with one decode per column
    // From 16 bands per SM on, BF16 activations take the persistent kernel; below, it was measured level with or behind
    // the split kernels (16384 x 2048: 34.6 against 22.4 us at one token, 35.9 against 35.6 at eight).
    constexpr int64_t big_per_sm = 16;
    if (a.ids || (a.ncols == 1 && (p.nrows / BAND < (int64_t) device_info().sms * big_per_sm || !a.x_bf16))) {
        const int C = (int) (w.K / CHUNK);
        const int64_t bands = p.nrows / BAND;
        if (C <= 8 && bands * a.ncols < (int64_t) device_info().sms * 64) { // few bands: a band's slabs side by side
            const int nb = std::max(1, 8 / C);
            const Opaque k = {1u, 4u, ~0u, 32u};
            const dim3 grid((unsigned) ((bands + nb - 1) / nb), (unsigned) a.ncols);
            // routed columns of 4..8 whole tokens: columns with the same expert share one decode (same bits per column).
            // Measured on one MoE layer whose tokens all pick the same 8 experts: 4 tokens 88.5 us grouped against 93.3
            // per column; 2 tokens 63.1 against 60.7 (half as many blocks, each with twice the multiply work, on a GPU
            // that two tokens do not fill), so fewer than four tokens go per column, as in the reference.
            const bool grouped = a.ids && a.n_used > 0 && a.ncols % a.n_used == 0 && a.ncols >= 4 * a.n_used && a.ncols <= 64;
            const int g = grouped ? FO_GROUP : 1;
            const size_t shm = 4 * HP_MAX_PAIRS + 128 + (size_t) w.K * 4 + (size_t) nb * C * 16 * g * 4 + (size_t) nb * C * FO_SPLIT_CAP;
            if (grouped) {
                launch_chained(k_fo_gemv_split<TX, false, FO_GROUP>, grid, dim3(nb * C * 32), shm, st, pair_view(w), (const AuxHeader *) w.aux, C, p,
                               nb, a.ncols, k);
            } else {
                launch_chained(k_fo_gemv_split<TX, false>, grid, dim3(nb * C * 32), shm, st, pair_view(w), (const AuxHeader *) w.aux, C, p, nb, 1, k);
            }
        } else {
            launch_fo<1, TX>(w, p, a.ids ? a.ncols : 1, st);
        }
        return;
    }
    if (a.x_bf16 && (a.ncols >= 2 || p.nrows / BAND >= (int64_t) device_info().sms * big_per_sm)) {
        // BF16 activations: the tensor-core kernels, 8 columns per decode. Large matrices (at least 16 bands per SM) take
        // the persistent kernel with staged streams, also for a single column.
        const int C = (int) (w.K / CHUNK);
        const int64_t bands = p.nrows / BAND, sms = device_info().sms;
        const size_t x_bytes = (size_t) 8 * (w.K + XPAD) * 2;
        // One persistent block per SM with as many warps as the shared memory holds stream buffers for (28 with K = 2048;
        // the decode chains need the occupancy), then the fewest warps that still finish in the same number of bands
        // per warp, so that no warp slows the others down for nothing.
        const size_t shm_fixed = 4 * HP_MAX_PAIRS + FO_BARS + x_bytes;
        const size_t optin = (size_t) device_info().smem_optin;
        int staged_warps = optin > shm_fixed ? (int) std::min<size_t>(32, (optin - shm_fixed) / (2 * FO_CAP)) : 0;
        if (staged_warps > 0) {
            const int64_t rounds = (bands + sms * staged_warps - 1) / (sms * staged_warps);
            staged_warps = (int) ((bands + sms * rounds - 1) / (sms * rounds));
        }
        const size_t shm_staged = shm_fixed + (size_t) staged_warps * 2 * FO_CAP;
        const bool big = bands >= sms * big_per_sm && (uintptr_t) p.x % 16 == 0 && p.x_tok % 16 == 0 && staged_warps >= 1 &&
                         shm_staged <= optin;
        for (int c0 = 0; c0 < a.ncols; c0 += 8) {
            Cols q = p;
            q.x += c0 * p.x_tok;
            q.y += c0 * p.y_tok;
            const int nc = std::min(8, a.ncols - c0);
            if (big) {
                const Opaque k = {1u, 4u, ~0u, 32u};
                launch_chained(k_fo_gemv_staged, dim3((unsigned) sms), dim3(staged_warps * 32), shm_staged, st, pair_view(w),
                               (const AuxHeader *) w.aux, C, q, nc, k);
            } else if (C <= 8) { // small and mid-size matrices: a band's slabs on separate warps, streams staged
                if constexpr (sizeof(TX) == 2) {
                    const int nb = std::max(1, 8 / C);
                    const size_t shm = 4 * HP_MAX_PAIRS + 128 + (size_t) 8 * (w.K + FO_SPLIT_XPAD) * 2 + (size_t) nb * C * 128 * 4 +
                                       (size_t) nb * C * FO_SPLIT_CAP;
                    const Opaque k = {1u, 4u, ~0u, 32u};
                    launch_chained(k_fo_gemv_split<bf16, true>, dim3((unsigned) ((bands + nb - 1) / nb)), dim3(nb * C * 32), shm, st,
                                   pair_view(w), (const AuxHeader *) w.aux, C, q, nb, nc, k);
                }
            } else {
                const int warps = bands >= sms * 32 ? 8 : bands >= sms * 8 ? 4 : 2;
                const dim3 grid((unsigned) std::min<int64_t>((bands + warps - 1) / warps, sms * 8));
                launch_chained(k_fo_gemv_mma, grid, dim3(warps * 32), 4 * HP_MAX_PAIRS + x_bytes, st, pair_view(w), C, q, nc, w.rows / BAND * C);
            }
        }
        return;
    }
    for (int c0 = 0; c0 < a.ncols;) { // groups of 8, 4, 2, 1 columns, each decoding the matrix once
        const int left = a.ncols - c0, nc = left >= 8 ? 8 : left >= 4 ? 4 : left >= 2 ? 2 : 1;
        Cols q = p;
        q.x += c0 * p.x_tok;
        q.y += c0 * p.y_tok;
        switch (nc) {
            case 8: launch_fo<8, TX>(w, q, 1, st); break;
            case 4: launch_fo<4, TX>(w, q, 1, st); break;
            case 2: launch_fo<2, TX>(w, q, 1, st); break;
            default: launch_fo<1, TX>(w, q, 1, st); break;
        }
        c0 += nc;
    }
}

} // namespace

BF16N_DEFINE_FAULT_WORD(fo_fault_word)

void fo_init() {
    const int optin = device_info().smem_optin;
#define ATTR(KERNEL) cuda_ok(cudaFuncSetAttribute(KERNEL, cudaFuncAttributeMaxDynamicSharedMemorySize, optin), #KERNEL)
    ATTR((k_fo_gemv<1, float>)); ATTR((k_fo_gemv<2, float>)); ATTR((k_fo_gemv<4, float>)); ATTR((k_fo_gemv<8, float>));
    ATTR((k_fo_gemv<1, bf16>)); ATTR((k_fo_gemv<2, bf16>)); ATTR((k_fo_gemv<4, bf16>)); ATTR((k_fo_gemv<8, bf16>));
    ATTR(k_fo_gemv_mma);
    ATTR((k_fo_gemv_split<float, false>)); ATTR((k_fo_gemv_split<bf16, false>)); ATTR((k_fo_gemv_split<bf16, true>));
    ATTR((k_fo_gemv_split<float, false, FO_GROUP>)); ATTR((k_fo_gemv_split<bf16, false, FO_GROUP>));
    ATTR(k_fo_gemv_staged);
    ATTR(k_fo_mm_ids<false>); ATTR(k_fo_mm_ids<true>);
#undef ATTR
}

// K up to 4096 columns with 8 activation columns staged as FP32 beside the table
bool fo_supported(const bf16n_weight & w) {
    return w.fo && w.format == FMT_HUFPAIR && w.R == BAND && !w.cm && w.K % CHUNK == 0 && w.rows % BAND == 0 &&
           4 * HP_MAX_PAIRS + 8 * w.K * 4 <= device_info().smem_optin;
}

static size_t fo_mm_shm(bool glu, int n_experts) {
    return (size_t) (glu ? 2 : 1) * 4 * HP_MAX_PAIRS + 2 * (size_t) FO_BUF + ((size_t) n_experts + 1) * 4;
}

bool fo_mm_ids_supported(const bf16n_weight & w, const bf16n_weight * up) {
    if (!fo_supported(w)) { return false; }
    return !up || (fo_supported(*up) && up->K == w.K && up->rows == w.rows);
}

void fo_mm_ids(const bf16n_weight & w, const bf16n_weight * up, const void * x_bf16, int64_t x_row, const int32_t * ids_src1,
               const int32_t * ids_dst, const int32_t * bounds, void * dst, bool dst_bf16, int64_t dst_col, int n_experts,
               cudaStream_t st) {
    FoBatch a = {};
    a.w0 = pair_view(w);
    a.w1 = up ? pair_view(*up) : a.w0;
    a.x = (const bf16 *) x_bf16; a.x_row = x_row;
    a.ids_src1 = ids_src1; a.ids_dst = ids_dst; a.bounds = bounds;
    a.dst = (char *) dst; a.dst_col = dst_col; a.dst_bf16 = dst_bf16;
    a.n_experts = n_experts; a.C = (int) (w.K / CHUNK);
    a.rows_per_expert = w.rows / n_experts;
    require(((uintptr_t) x_bf16 % 16) == 0 && (x_row * 2) % 16 == 0, "batched activations must be 16-byte aligned rows");
    require(a.rows_per_expert % BAND == 0, "rows per expert must be whole 16-row bands");
    a.n_units = w.rows / BAND * a.C;
    const size_t shm = fo_mm_shm(up != nullptr, n_experts);
    require(shm <= (size_t) device_info().smem_optin, "too many experts for the fragment-order batched kernel's shared memory");
    const unsigned grid = (unsigned) device_info().sms; // persistent: the items are counted on the device from the bounds
    if (up) { k_fo_mm_ids<true><<<grid, FO_WARPS * 32, shm, st>>>(a); } else { k_fo_mm_ids<false><<<grid, FO_WARPS * 32, shm, st>>>(a); }
    check_launch();
}

void fo_gemv(const bf16n_weight & w, const bf16n_mmv_args & a, cudaStream_t st) {
    if (a.x_bf16) { fo_gemv_t<bf16>(w, a, st); } else { fo_gemv_t<float>(w, a, st); }
}

void fo_expand_store(const bf16n_weight & w, int64_t row0, int64_t nrows, uint16_t * out, cudaStream_t st) {
    const int C = (int) (w.K / CHUNK);
    const int64_t units = nrows / BAND * C;
    const unsigned gx = (unsigned) std::max<int64_t>(1, std::min<int64_t>((units + 7) / 8, (int64_t) device_info().sms * 16));
    k_fo_expand<FoStore><<<gx, 256, 0, st>>>(pair_view(w), C, row0, nrows, FoStore{out, w.K});
    check_launch();
}

void fo_expand_compare(const bf16n_weight & w, int64_t row0, int64_t nrows, const uint16_t * src, unsigned long long * total,
                       cudaStream_t st) {
    const int C = (int) (w.K / CHUNK);
    const int64_t units = nrows / BAND * C;
    const unsigned gx = (unsigned) std::max<int64_t>(1, std::min<int64_t>((units + 7) / 8, (int64_t) device_info().sms * 16));
    k_fo_expand<FoCompare><<<gx, 256, 0, st>>>(pair_view(w), C, row0, nrows, FoCompare{src, w.K, total, 0u});
    check_launch();
}

void fo_gather_rows(const bf16n_weight & w, const void * ids, int64_t ids_s0, int64_t n, void * dst, bool dst_bf16, int64_t dst_s1,
                    int64_t row0, cudaStream_t st) {
    const int C = (int) (w.K / CHUNK);
    const unsigned gx = (unsigned) ((n + 7) / 8);
    if (dst_bf16) { k_fo_rows<true><<<gx, 256, 0, st>>>(pair_view(w), C, (const char *) ids, ids_s0, n, row0, (char *) dst, dst_s1); }
    else { k_fo_rows<false><<<gx, 256, 0, st>>>(pair_view(w), C, (const char *) ids, ids_s0, n, row0, (char *) dst, dst_s1); }
    check_launch();
}

} // namespace b16
