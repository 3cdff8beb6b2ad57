// Decode-inside-GEMV kernels for 1..4 activation columns, exact dequantisation / verification and row gather, for the
// three BF16N exponent formats. One warp owns one unit (R rows) of a Huffman-coded matrix or one row of a NIBBLE
// matrix; every lane walks its own bit stream; products are accumulated in FP32 in the order the format's lane layout
// implies (four accumulators per lane by column & 3, chunks in order, then a xor butterfly), which makes the results
// independent of the launch geometry and equal, bit for bit, to the reference kernels' order
// (core/include/bf16n/kernels.cuh:498-535, 958-986, 139-187).
#include "decode.cuh"
#include "launch.h"
#include <cstdlib>

namespace b16 {
namespace {

using namespace dev;
using bf16 = __nv_bfloat16;

// FP32 products of one row-chunk (this lane's 16 weights, as 8 BF16x2 words) with the matching activations
__device__ __forceinline__ void fma_chunk(const uint32_t (&w)[8], const float4 (&x)[4], float (&a)[4]) {
#pragma unroll
    for (int j = 0; j < 4; j++) {
        a[0] = fmaf(bf16lo_f32(w[2 * j]), x[j].x, a[0]);
        a[1] = fmaf(bf16hi_f32(w[2 * j]), x[j].y, a[1]);
        a[2] = fmaf(bf16lo_f32(w[2 * j + 1]), x[j].z, a[2]);
        a[3] = fmaf(bf16hi_f32(w[2 * j + 1]), x[j].w, a[3]);
    }
}

template <typename TX>
__device__ __forceinline__ void stage_x(float * xs, const TX * xg, int K) {
    for (int i = threadIdx.x; i < K; i += blockDim.x) { xs[i] = to_f32(xg[i]); }
}
__device__ __forceinline__ void stage_lut(uint32_t * dst, const uint32_t * src, int n) {
    for (int i = threadIdx.x; i < n / 4; i += blockDim.x) { ((uint4 *) dst)[i] = __ldg((const uint4 *) src + i); }
}

// ---------------------------------------------------------------- HUFPAIR, row-major units

// NC dense columns (NC == 1: also routed columns, one per blockIdx.y). XR: the lane's activations live in registers.
template <int C, int NC, typename TX, bool XR, bool PEERS = false>
__global__ void __launch_bounds__(512) k_pair_gemv(const PairView w, int R, Cols p) {
    constexpr int K = C * CHUNK;
    extern __shared__ __align__(16) unsigned char smem[];
    uint32_t * lut = (uint32_t *) smem;
    float * xs = (float *) (smem + 4 * HP_MAX_PAIRS);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;

    const TX * xg; OutVec out; int64_t rbase;
    column<TX>(p, NC == 1 ? blockIdx.y : 0, xg, out, rbase);
    stage_lut(lut, w.lut, HP_MAX_PAIRS);
#pragma unroll
    for (int n = 0; n < NC; n++) { stage_x<TX>(xs + n * K, (const TX *) ((const char *) xg + n * p.x_tok), K); }
    __syncthreads();

    float4 xr[XR ? C * 4 : 1];
    if (XR) {
#pragma unroll
        for (int i = 0; i < C * 4; i++) { xr[i] = *(const float4 *) (xs + (i >> 2) * CHUNK + 128 * (i & 3) + 4 * lane); }
    }

    const int64_t units = p.nrows / R;
    for (int64_t u = (int64_t) blockIdx.x * nwarp + warp; u < units; u += (int64_t) gridDim.x * nwarp) {
        const int64_t gu = rbase / R + u;
        PairReader rd;
        rd.open(w, gu, lane);
        const uint8_t * pl = w.plane + gu * R * K + 16 * lane;
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
            float a[NC][4];
#pragma unroll
            for (int n = 0; n < NC; n++) { a[n][0] = a[n][1] = a[n][2] = a[n][3] = 0.f; }
#pragma unroll
            for (int c = 0; c < C; c++) {
                uint32_t e[8], wv[8];
                rd.take8(lut, e);
                assemble8(cur[c], e, wv);
#pragma unroll
                for (int n = 0; n < NC; n++) {
                    float4 xq[4];
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        xq[j] = XR ? xr[c * 4 + j] : *(const float4 *) (xs + n * K + c * CHUNK + 128 * j + 4 * lane);
                    }
                    fma_chunk(wv, xq, a[n]);
                }
            }
#pragma unroll
            for (int n = 0; n < NC; n++) {
                const float s = warp_sum((a[n][0] + a[n][1]) + (a[n][2] + a[n][3]));
                if (lane == 0) {
                    OutVec o = out;
                    o.p += n * p.y_tok;
                    o.put(u * R + rr, s);
                    if (PEERS) { peers_put(p, blockIdx.y, u * R + rr, s); }
                }
            }
        }
    }
    if (PEERS) { peers_done(p); }
}

// y = silu(gate x) * (up x), separate row-major gate / up matrices with the same geometry
template <int C, typename TX>
__global__ void __launch_bounds__(512) k_pair_glu(const PairView g, const PairView v, int R, Cols p) {
    constexpr int K = C * CHUNK;
    extern __shared__ __align__(16) unsigned char smem[];
    uint32_t * lut_g = (uint32_t *) smem;
    uint32_t * lut_v = lut_g + HP_MAX_PAIRS;
    float * xs = (float *) (lut_v + HP_MAX_PAIRS);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    const TX * xg; OutVec out; int64_t rbase;
    column<TX>(p, blockIdx.y, xg, out, rbase);
    stage_lut(lut_g, g.lut, HP_MAX_PAIRS);
    stage_lut(lut_v, v.lut, HP_MAX_PAIRS);
    stage_x<TX>(xs, xg, K);
    __syncthreads();
    const int64_t units = p.nrows / R;
    for (int64_t u = (int64_t) blockIdx.x * nwarp + warp; u < units; u += (int64_t) gridDim.x * nwarp) {
        const int64_t gu = rbase / R + u;
        PairReader rg, rv;
        rg.open(g, gu, lane);
        rv.open(v, gu, lane);
        for (int rr = 0; rr < R; rr++) {
            const int64_t row = gu * R + rr;
            float ag[4] = {0.f, 0.f, 0.f, 0.f}, av[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int c = 0; c < C; c++) {
                const uint4 sg = ld_stream16(g.plane + row * K + c * CHUNK + 16 * lane);
                const uint4 sv = ld_stream16(v.plane + row * K + c * CHUNK + 16 * lane);
                float4 xq[4];
#pragma unroll
                for (int j = 0; j < 4; j++) { xq[j] = *(const float4 *) (xs + c * CHUNK + 128 * j + 4 * lane); }
                uint32_t e[8], wv[8];
                rg.take8(lut_g, e);
                assemble8(sg, e, wv);
                fma_chunk(wv, xq, ag);
                rv.take8(lut_v, e);
                assemble8(sv, e, wv);
                fma_chunk(wv, xq, av);
            }
            const float gs = warp_sum((ag[0] + ag[1]) + (ag[2] + ag[3]));
            const float vs = warp_sum((av[0] + av[1]) + (av[2] + av[3]));
            if (lane == 0) { out.put(u * R + rr, vs * silu_f(gs)); }
        }
    }
}

// ---------------------------------------------------------------- HUFPAIR, chunk-major units (expert stacks, K > 512)

// Streams and plane run chunk -> row inside a unit: per chunk the lane's 16 activations are read once and reused for
// the R rows; each row adds its per-chunk lane sum, lanes are reduced once per unit.
template <int C, int R, typename TX>
__global__ void __launch_bounds__(512) k_pair_gemv_cm(const PairView w, Cols p) {
    constexpr int K = C * CHUNK;
    extern __shared__ __align__(16) unsigned char smem[];
    uint32_t * lut = (uint32_t *) smem;
    float * xs = (float *) (smem + 4 * HP_MAX_PAIRS);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    const TX * xg; OutVec out; int64_t rbase;
    column<TX>(p, blockIdx.y, xg, out, rbase);
    stage_lut(lut, w.lut, HP_MAX_PAIRS);
    stage_x<TX>(xs, xg, K);
    __syncthreads();
    const int64_t units = p.nrows / R;
    for (int64_t u = (int64_t) blockIdx.x * nwarp + warp; u < units; u += (int64_t) gridDim.x * nwarp) {
        const int64_t gu = rbase / R + u;
        PairReader rd;
        rd.open(w, gu, lane);
        const uint8_t * pl = w.plane + gu * R * K + 16 * lane;
        float acc[R];
#pragma unroll
        for (int rr = 0; rr < R; rr++) { acc[rr] = 0.f; }
#pragma unroll 1
        for (int c = 0; c < C; c++) {
            float4 xq[4];
#pragma unroll
            for (int j = 0; j < 4; j++) { xq[j] = *(const float4 *) (xs + c * CHUNK + 128 * j + 4 * lane); }
            uint4 sm[R];
#pragma unroll
            for (int rr = 0; rr < R; rr++) { sm[rr] = ld_stream16(pl + (c * R + rr) * CHUNK); }
#pragma unroll
            for (int rr = 0; rr < R; rr++) {
                uint32_t e[8], wv[8];
                rd.take8(lut, e);
                assemble8(sm[rr], e, wv);
                float a[4] = {0.f, 0.f, 0.f, 0.f};
                fma_chunk(wv, xq, a);
                acc[rr] += (a[0] + a[1]) + (a[2] + a[3]);
            }
        }
#pragma unroll
        for (int rr = 0; rr < R; rr++) {
            const float s = warp_sum(acc[rr]);
            if (lane == 0) { out.put(u * R + rr, s); }
        }
    }
}

// ---------------------------------------------------------------- HUFFMAN (single-exponent fallback), row-major units

template <typename TX, bool GLU>
__global__ void __launch_bounds__(256) k_huf_gemv(const HufView g, const HufView v, int C, int R, Cols p) {
    const int K = C * CHUNK;
    extern __shared__ __align__(16) unsigned char smem[];
    uint32_t * lut_g = (uint32_t *) smem;
    uint32_t * lut_v = lut_g + (1 << HUF_LMAX);
    float * xs = (float *) (lut_v + (GLU ? (1 << HUF_LMAX) : 0));
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    const TX * xg; OutVec out; int64_t rbase;
    column<TX>(p, blockIdx.y, xg, out, rbase);
    stage_lut(lut_g, g.lut, 1 << HUF_LMAX);
    if (GLU) { stage_lut(lut_v, v.lut, 1 << HUF_LMAX); }
    stage_x<TX>(xs, xg, K);
    __syncthreads();
    const int64_t units = p.nrows / R;
    for (int64_t u = (int64_t) blockIdx.x * nwarp + warp; u < units; u += (int64_t) gridDim.x * nwarp) {
        const int64_t gu = rbase / R + u;
        HufReader rg, rv;
        rg.open(g, gu, lane);
        if (GLU) { rv.open(v, gu, lane); }
        for (int rr = 0; rr < R; rr++) {
            const int64_t row = gu * R + rr;
            float ag[4] = {0.f, 0.f, 0.f, 0.f}, av[4] = {0.f, 0.f, 0.f, 0.f};
            for (int c = 0; c < C; c++) {
                float4 xq[4];
#pragma unroll
                for (int j = 0; j < 4; j++) { xq[j] = *(const float4 *) (xs + c * CHUNK + 128 * j + 4 * lane); }
                uint32_t e[8], wv[8];
                rg.take8(lut_g, e);
                assemble8(ld_stream16(g.plane + row * K + c * CHUNK + 16 * lane), e, wv);
                fma_chunk(wv, xq, ag);
                if (GLU) {
                    rv.take8(lut_v, e);
                    assemble8(ld_stream16(v.plane + row * K + c * CHUNK + 16 * lane), e, wv);
                    fma_chunk(wv, xq, av);
                }
            }
            const float gs = warp_sum((ag[0] + ag[1]) + (ag[2] + ag[3]));
            if (GLU) {
                const float vs = warp_sum((av[0] + av[1]) + (av[2] + av[3]));
                if (lane == 0) { out.put(u * R + rr, vs * silu_f(gs)); }
            } else if (lane == 0) {
                out.put(u * R + rr, gs);
            }
        }
    }
}

// ---------------------------------------------------------------- NIBBLE: one warp per row

template <int C>
struct NibRow { uint4 sm[C]; uint2 cd[C]; uint4 L; uint32_t e0, e1; };

template <int C>
__device__ __forceinline__ void nib_load(NibRow<C> & d, const NibView & w, int64_t row, int lane) {
    constexpr int K = C * CHUNK;
#pragma unroll
    for (int c = 0; c < C; c++) {
        d.sm[c] = __ldg((const uint4 *) (w.plane + row * K + c * CHUNK) + lane);
        d.cd[c] = __ldg((const uint2 *) (w.codes + row * (K / 2) + c * 256) + lane);
    }
    d.L = __ldg(w.row_lut + row);
    d.e0 = __ldg(w.esc_off + row);
    d.e1 = __ldg(w.esc_off + row + 1);
}

// dot(row, x): dense pass (escaped slots decode to +0), then the row's escapes, then the butterfly
template <int C, typename TX>
__device__ __forceinline__ float nib_dot(const NibRow<C> & d, const NibView & w, const TX * __restrict__ x, int lane) {
    float a[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int c = 0; c < C; c++) {
        uint32_t wv[8];
        nib_assemble8(d.sm[c], d.cd[c], d.L, wv);
        float4 xq[4];
#pragma unroll
        for (int j = 0; j < 4; j++) { xq[j] = ldg_x4(x, c * CHUNK + 128 * j + 4 * lane); }
        fma_chunk(wv, xq, a);
    }
    float acc = (a[0] + a[1]) + (a[2] + a[3]);
    for (uint32_t i = d.e0 + lane; i < d.e1; i += 32) {
        const uint32_t rec = __ldg(w.esc + i);
        acc = fmaf(__uint_as_float(esc_bits(rec) << 16), ldg_x1(x, rec & 0xFFF), acc);
    }
    return warp_sum(acc);
}

// GLU: g rows are the gate, v rows the up half (separate matrices, or the same matrix shifted by nrows rows)
template <int C, typename TX, bool GLU>
__global__ void __launch_bounds__(256) k_nib_gemv(const NibView g, const NibView v, Cols p) {
    // Launched as a programmatic dependent (launch_chained): a warp fetches its first row's weights while the kernel
    // before it on the stream is still draining, and waits for that kernel only before it reads activations or writes
    // outputs (expert ids, when there are any, belong to an earlier kernel too).
    bool waited = p.ids != nullptr;
    if (waited) { grid_dependency_wait(); }
    const TX * xg; OutVec out; int64_t rbase;
    column<TX>(p, blockIdx.y, xg, out, rbase);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int64_t r = (int64_t) blockIdx.x * 8 + warp; r < p.nrows; r += (int64_t) gridDim.x * 8) {
        NibRow<C> dg, dv;
        nib_load<C>(dg, g, rbase + r, lane);
        if (GLU) { nib_load<C>(dv, v, rbase + r, lane); }
        if (!waited) { grid_dependency_wait(); waited = true; }
        const float gs = nib_dot<C, TX>(dg, g, xg, lane);
        if (GLU) {
            const float vs = nib_dot<C, TX>(dv, v, xg, lane);
            if (lane == 0) { out.put(r, vs * silu_f(gs)); }
        } else if (lane == 0) {
            out.put(r, gs);
        }
    }
}

// ---------------------------------------------------------------- exact reconstruction (dequant / verify / gather)

struct StoreBF16 { // row-major BF16 output
    uint16_t * out;
    int64_t K;
    __device__ __forceinline__ void chunk(int64_t r, int c, int lane, const uint32_t (&w)[8]) {
        uint16_t * o = out + r * K + c * CHUNK + 4 * lane;
#pragma unroll
        for (int j = 0; j < 4; j++) { *(uint2 *) (o + 128 * j) = make_uint2(w[2 * j], w[2 * j + 1]); }
    }
    __device__ __forceinline__ void one(int64_t r, int col, uint32_t bits) { out[r * K + col] = (uint16_t) bits; }
    __device__ __forceinline__ void finish(int) {}
};

struct CompareBF16 { // count words that differ from src
    const uint16_t * src;
    int64_t K;
    unsigned long long * total;
    unsigned int bad;
    __device__ __forceinline__ void chunk(int64_t r, int c, int lane, const uint32_t (&w)[8]) {
        const uint16_t * o = src + r * K + c * CHUNK + 4 * lane;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint2 s = __ldg((const uint2 *) (o + 128 * j));
            const uint32_t d0 = s.x ^ w[2 * j], d1 = s.y ^ w[2 * j + 1];
            bad += ((d0 & 0xFFFFu) != 0) + ((d0 >> 16) != 0) + ((d1 & 0xFFFFu) != 0) + ((d1 >> 16) != 0);
        }
    }
    // NIBBLE escapes: the dense pass saw +0 where src holds the escaped value, so every escape that matches its source
    // takes back one counted difference (and a wrong one keeps it)
    __device__ __forceinline__ void one(int64_t r, int col, uint32_t bits) {
        const uint32_t s = src[r * K + col];
        if (s != 0) { bad -= 1; }
        if (s != bits) { bad += 1; }
    }
    __device__ __forceinline__ void finish(int lane) {
        unsigned int b = bad;
#pragma unroll
        for (int o = 16; o; o >>= 1) { b += __shfl_xor_sync(FULL, b, o); }
        if (lane == 0 && b) { atomicAdd(total, (unsigned long long) b); }
    }
};

template <typename Sink>
__global__ void __launch_bounds__(256) k_pair_expand(const PairView w, int C, int R, bool cm, int64_t row0, int64_t nrows, const Sink sink_in) {
    Sink sink = sink_in;
    __shared__ uint32_t lut[HP_MAX_PAIRS];
    stage_lut(lut, w.lut, HP_MAX_PAIRS);
    __syncthreads();
    const int64_t K = (int64_t) C * CHUNK;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int64_t u = (int64_t) blockIdx.x * 8 + warp; u < nrows / R; u += (int64_t) gridDim.x * 8) {
        const int64_t gu = row0 / R + u;
        PairReader rd;
        rd.open(w, gu, lane);
        const uint8_t * pl = w.plane + gu * R * K + 16 * lane;
        for (int o = 0; o < R * C; o++) {
            const int rr = cm ? o % R : o / C, c = cm ? o / R : o % C;
            const uint4 sm = ld_stream16(pl + (cm ? (int64_t) (c * R + rr) * CHUNK : rr * K + (int64_t) c * CHUNK));
            uint32_t e[8], wv[8];
            rd.take8(lut, e);
            assemble8(sm, e, wv);
            sink.chunk(u * R + rr, c, lane, wv);
        }
    }
    sink.finish(lane);
}

template <typename Sink>
__global__ void __launch_bounds__(256) k_huf_expand(const HufView w, int C, int R, int64_t row0, int64_t nrows, const Sink sink_in) {
    Sink sink = sink_in;
    __shared__ uint32_t lut[1 << HUF_LMAX];
    stage_lut(lut, w.lut, 1 << HUF_LMAX);
    __syncthreads();
    const int64_t K = (int64_t) C * CHUNK;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int64_t u = (int64_t) blockIdx.x * 8 + warp; u < nrows / R; u += (int64_t) gridDim.x * 8) {
        const int64_t gu = row0 / R + u;
        HufReader rd;
        rd.open(w, gu, lane);
        for (int o = 0; o < R * C; o++) {
            const int rr = o / C, c = o % C;
            const uint4 sm = ld_stream16(w.plane + (gu * R + rr) * K + (int64_t) c * CHUNK + 16 * lane);
            uint32_t e[8], wv[8];
            rd.take8(lut, e);
            assemble8(sm, e, wv);
            sink.chunk(u * R + rr, c, lane, wv);
        }
    }
    sink.finish(lane);
}

template <typename Sink>
__global__ void __launch_bounds__(256) k_nib_expand(const NibView w, int C, int64_t row0, int64_t nrows, const Sink sink_in) {
    Sink sink = sink_in;
    const int64_t K = (int64_t) C * CHUNK;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int64_t r = (int64_t) blockIdx.x * 8 + warp; r < nrows; r += (int64_t) gridDim.x * 8) {
        const int64_t gr = row0 + r;
        const uint4 L = __ldg(w.row_lut + gr);
        for (int c = 0; c < C; c++) {
            const uint4 sm = __ldg((const uint4 *) (w.plane + gr * K + (int64_t) c * CHUNK) + lane);
            const uint2 cd = __ldg((const uint2 *) (w.codes + gr * (K / 2) + (int64_t) c * 256) + lane);
            uint32_t wv[8];
            nib_assemble8(sm, cd, L, wv);
            sink.chunk(r, c, lane, wv);
        }
        __syncwarp();
        for (uint32_t i = __ldg(w.esc_off + gr) + lane; i < __ldg(w.esc_off + gr + 1); i += 32) {
            const uint32_t rec = __ldg(w.esc + i);
            sink.one(r, rec & 0xFFF, esc_bits(rec));
        }
    }
    sink.finish(lane);
}

// gather: dst[i] = W[row0 + ids[i]], FP32 or BF16. A Huffman-coded row is reached by decoding its unit from the start.
template <bool BF>
__device__ __forceinline__ void put_row_chunk(char * o, int c, int lane, const uint32_t (&w)[8]) {
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int i = c * CHUNK + 128 * j + 4 * lane;
        if (BF) {
            *(uint2 *) (o + 2 * i) = make_uint2(w[2 * j], w[2 * j + 1]);
        } else {
            *(float4 *) (o + 4 * i) = make_float4(bf16lo_f32(w[2 * j]), bf16hi_f32(w[2 * j]), bf16lo_f32(w[2 * j + 1]), bf16hi_f32(w[2 * j + 1]));
        }
    }
}

template <bool BF>
__global__ void __launch_bounds__(256) k_pair_rows(const PairView w, int C, int R, const char * ids, int64_t ids_s0, int64_t n,
                                                    int64_t row0, char * dst, int64_t dst_s1) {
    __shared__ uint32_t lut[HP_MAX_PAIRS];
    stage_lut(lut, w.lut, HP_MAX_PAIRS);
    __syncthreads();
    const int64_t K = (int64_t) C * CHUNK;
    const int lane = threadIdx.x & 31;
    const int64_t i = (int64_t) blockIdx.x * 8 + (threadIdx.x >> 5);
    if (i >= n) { return; }
    const int64_t gr = row0 + *(const int32_t *) (ids + i * ids_s0);
    const int64_t gu = gr / R;
    PairReader rd;
    rd.open(w, gu, lane);
    for (int64_t r = gu * R; r <= gr; r++) {
        for (int c = 0; c < C; c++) {
            uint32_t e[8];
            rd.take8(lut, e);
            if (r == gr) {
                uint32_t wv[8];
                assemble8(ld_stream16(w.plane + r * K + (int64_t) c * CHUNK + 16 * lane), e, wv);
                put_row_chunk<BF>(dst + i * dst_s1, c, lane, wv);
            }
        }
    }
}

template <bool BF>
__global__ void __launch_bounds__(256) k_nib_rows(const NibView w, int C, const char * ids, int64_t ids_s0, int64_t n, int64_t row0,
                                                   char * dst, int64_t dst_s1) {
    const int64_t K = (int64_t) C * CHUNK;
    const int lane = threadIdx.x & 31;
    const int64_t i = (int64_t) blockIdx.x * 8 + (threadIdx.x >> 5);
    if (i >= n) { return; }
    const int64_t gr = row0 + *(const int32_t *) (ids + i * ids_s0);
    char * o = dst + i * dst_s1;
    const uint4 L = __ldg(w.row_lut + gr);
    for (int c = 0; c < C; c++) {
        const uint4 sm = __ldg((const uint4 *) (w.plane + gr * K + (int64_t) c * CHUNK) + lane);
        const uint2 cd = __ldg((const uint2 *) (w.codes + gr * (K / 2) + (int64_t) c * 256) + lane);
        uint32_t wv[8];
        nib_assemble8(sm, cd, L, wv);
        put_row_chunk<BF>(o, c, lane, wv);
    }
    __syncwarp();
    for (uint32_t k = __ldg(w.esc_off + gr) + lane; k < __ldg(w.esc_off + gr + 1); k += 32) {
        const uint32_t rec = __ldg(w.esc + k);
        if (BF) { ((uint16_t *) o)[rec & 0xFFF] = (uint16_t) esc_bits(rec); }
        else { ((float *) o)[rec & 0xFFF] = __uint_as_float(esc_bits(rec) << 16); }
    }
}

// ---------------------------------------------------------------- views and geometry

// warps per block and blocks for `units` warp-sized work items per column: spread few units over all SMs with small
// blocks, fill the machine with 16-warp blocks otherwise
void unit_geometry(int64_t units, int ncols, int max_warps, dim3 & grid, int & threads) {
    const int64_t sms = device_info().sms;
    const int64_t per_col = std::max<int64_t>(1, sms / std::max(1, ncols));
    const int64_t wpb = std::min<int64_t>(std::max<int64_t>((units + per_col - 1) / per_col, 2), max_warps);
    threads = (int) wpb * 32;
    grid = dim3((unsigned) std::max<int64_t>(1, std::min<int64_t>((units + wpb - 1) / wpb, per_col)), (unsigned) ncols);
}

dim3 row_geometry(int64_t work, int ncols) { // 8 warps per block, one work item per warp
    const int64_t cap = std::max<int64_t>(1, (int64_t) device_info().sms * 8 / std::min(ncols, 8));
    return dim3((unsigned) std::max<int64_t>(1, std::min<int64_t>((work + 7) / 8, cap)), (unsigned) ncols);
}

// Mid-size dense HUFPAIR matrices (256 units up to 4 per SM) with several columns: one staged decode per column over all
// SMs instead of the general kernel's shared decode, whose warps read their lane streams straight from global memory
// (4096 x 2048, R = 8: 29 -> 19 us at 4 tokens, 54 -> 33 us at 8; from 1024 units on the two forms are level).
static bool mid_size_by_column(const bf16n_weight & w, const bf16n_mmv_args & a, int64_t units) {
    if (units > (int64_t) device_info().sms * 4) { return false; }
    bf16n_mmv_args one = a;
    one.ncols = 1;
    return gemv_staged_applies(w, one);
}

template <typename TX>
void launch_gemv(const bf16n_weight & w, const bf16n_mmv_args & a, cudaStream_t st, bool multi_col, const bf16n_peer_out * peers) {
    const Cols p = make_cols(a, peers);
    if (peers && peers->n_peers > 0) {
        require(w.format == FMT_HUFPAIR && !w.cm && !a.ids, "peer outputs need a dense row-major HUFPAIR product");
        multi_col = false; // one column per blockIdx.y: the kernels that fan out
    }
    const int C = (int) (w.K / CHUNK);
    if (w.format == FMT_HUFPAIR) {
        const int64_t units = a.nrows / w.R;
        dim3 grid; int threads;
        if (w.cm) {
            unit_geometry(units, a.ncols, 16, grid, threads);
            const size_t shm = 4 * HP_MAX_PAIRS + w.K * 4;
#define CM(CC, RR) case CC * 100 + RR: k_pair_gemv_cm<CC, RR, TX><<<grid, threads, shm, st>>>(pair_view(w), p); break;
            switch (C * 100 + w.R) {
                CM(2, 4) CM(2, 8) CM(2, 16) CM(4, 4) CM(4, 8) CM(4, 16) CM(8, 4) CM(8, 8) CM(8, 16)
                default: fail_invalid("unsupported chunk-major K/R");
            }
#undef CM
        } else if (gemv_rings_enabled() && gemv_rings_applies(w, a)) {
            gemv_rings(w, a, st, multi_col, peers); // large matrices, BF16 activations: 1, 2 or 4 columns per decode
            return;
        } else if (!a.ids && a.ncols > 1 && multi_col && !mid_size_by_column(w, a, units)) {
            unit_geometry(units, 1, 16, grid, threads);
            for (int c0 = 0; c0 < a.ncols; c0 += 4) {
                const int nc = std::min(4, a.ncols - c0);
                Cols q = p;
                q.x += c0 * p.x_tok;
                q.y += c0 * p.y_tok;
                const size_t shm = 4 * HP_MAX_PAIRS + (size_t) nc * w.K * 4;
#define MC(CC, NN) case CC * 10 + NN: k_pair_gemv<CC, NN, TX, false><<<grid, threads, shm, st>>>(pair_view(w), w.R, q); break;
                switch (C * 10 + nc) {
                    MC(1, 1) MC(1, 2) MC(1, 3) MC(1, 4) MC(2, 1) MC(2, 2) MC(2, 3) MC(2, 4)
                    MC(4, 1) MC(4, 2) MC(4, 3) MC(4, 4) MC(8, 1) MC(8, 2) MC(8, 3) MC(8, 4)
                    default: fail_invalid("unsupported K");
                }
#undef MC
            }
        } else if (gemv_staged_applies(w, a) || (!a.ids && a.ncols > 1 && mid_size_by_column(w, a, units))) {
            gemv_staged(w, a, st, peers);
            return;
        } else {
            unit_geometry(units, a.ncols, 16, grid, threads);
            const size_t shm = 4 * HP_MAX_PAIRS + w.K * 4;
            if (p.peers.n) {
                switch (C) {
                    case 1: k_pair_gemv<1, 1, TX, true, true><<<grid, threads, shm, st>>>(pair_view(w), w.R, p); break;
                    case 2: k_pair_gemv<2, 1, TX, true, true><<<grid, threads, shm, st>>>(pair_view(w), w.R, p); break;
                    case 4: k_pair_gemv<4, 1, TX, true, true><<<grid, threads, shm, st>>>(pair_view(w), w.R, p); break;
                    case 8: k_pair_gemv<8, 1, TX, false, true><<<grid, threads, shm, st>>>(pair_view(w), w.R, p); break;
                    default: fail_invalid("unsupported K");
                }
            } else {
                switch (C) {
                    case 1: k_pair_gemv<1, 1, TX, true><<<grid, threads, shm, st>>>(pair_view(w), w.R, p); break;
                    case 2: k_pair_gemv<2, 1, TX, true><<<grid, threads, shm, st>>>(pair_view(w), w.R, p); break;
                    case 4: k_pair_gemv<4, 1, TX, true><<<grid, threads, shm, st>>>(pair_view(w), w.R, p); break;
                    case 8: k_pair_gemv<8, 1, TX, false><<<grid, threads, shm, st>>>(pair_view(w), w.R, p); break;
                    default: fail_invalid("unsupported K");
                }
            }
        }
    } else if (w.format == FMT_NIBBLE) {
        const dim3 grid = row_geometry(a.nrows, a.ncols);
        const NibView v = nib_view(w);
        switch (C) {
            case 1: launch_chained(k_nib_gemv<1, TX, false>, grid, dim3(256), 0, st, v, v, p); break;
            case 2: launch_chained(k_nib_gemv<2, TX, false>, grid, dim3(256), 0, st, v, v, p); break;
            case 4: launch_chained(k_nib_gemv<4, TX, false>, grid, dim3(256), 0, st, v, v, p); break;
            case 8: launch_chained(k_nib_gemv<8, TX, false>, grid, dim3(256), 0, st, v, v, p); break;
            default: fail_invalid("unsupported K");
        }
    } else {
        const dim3 grid = row_geometry(a.nrows / w.R, a.ncols);
        const size_t shm = (4u << HUF_LMAX) + w.K * 4;
        k_huf_gemv<TX, false><<<grid, 256, shm, st>>>(huf_view(w), huf_view(w), C, w.R, p);
    }
    check_launch();
}

template <typename TX>
void launch_glu(const bf16n_weight & g, const NibView * up_nib, const bf16n_weight * u, const bf16n_mmv_args & a, cudaStream_t st) {
    const Cols p = make_cols(a);
    const int C = (int) (g.K / CHUNK);
    if (g.format == FMT_NIBBLE) {
        const dim3 grid = row_geometry(a.nrows, a.ncols);
        const NibView gv = nib_view(g), uv = up_nib ? *up_nib : nib_view(*u);
        switch (C) {
            case 1: launch_chained(k_nib_gemv<1, TX, true>, grid, dim3(256), 0, st, gv, uv, p); break;
            case 2: launch_chained(k_nib_gemv<2, TX, true>, grid, dim3(256), 0, st, gv, uv, p); break;
            case 4: launch_chained(k_nib_gemv<4, TX, true>, grid, dim3(256), 0, st, gv, uv, p); break;
            case 8: launch_chained(k_nib_gemv<8, TX, true>, grid, dim3(256), 0, st, gv, uv, p); break;
            default: fail_invalid("unsupported K");
        }
    } else if (g.format == FMT_HUFPAIR) {
        dim3 grid; int threads;
        unit_geometry(a.nrows / g.R, a.ncols, 16, grid, threads);
        const size_t shm = 8 * HP_MAX_PAIRS + g.K * 4;
        switch (C) {
            case 1: k_pair_glu<1, TX><<<grid, threads, shm, st>>>(pair_view(g), pair_view(*u), g.R, p); break;
            case 2: k_pair_glu<2, TX><<<grid, threads, shm, st>>>(pair_view(g), pair_view(*u), g.R, p); break;
            case 4: k_pair_glu<4, TX><<<grid, threads, shm, st>>>(pair_view(g), pair_view(*u), g.R, p); break;
            case 8: k_pair_glu<8, TX><<<grid, threads, shm, st>>>(pair_view(g), pair_view(*u), g.R, p); break;
            default: fail_invalid("unsupported K");
        }
    } else {
        const dim3 grid = row_geometry(a.nrows / g.R, a.ncols);
        const size_t shm = (8u << HUF_LMAX) + g.K * 4;
        k_huf_gemv<TX, true><<<grid, 256, shm, st>>>(huf_view(g), huf_view(*u), C, g.R, p);
    }
    check_launch();
}

template <typename Sink>
void launch_expand(const bf16n_weight & w, int64_t row0, int64_t nrows, const Sink & sink, cudaStream_t st) {
    const int C = (int) (w.K / CHUNK);
    const int64_t work = w.format == FMT_NIBBLE ? nrows : nrows / w.R;
    const unsigned gx = (unsigned) std::max<int64_t>(1, std::min<int64_t>((work + 7) / 8, (int64_t) device_info().sms * 16));
    if (w.format == FMT_NIBBLE) {
        k_nib_expand<Sink><<<gx, 256, 0, st>>>(nib_view(w), C, row0, nrows, sink);
    } else if (w.format == FMT_HUFPAIR) {
        k_pair_expand<Sink><<<gx, 256, 0, st>>>(pair_view(w), C, w.R, w.cm != 0, row0, nrows, sink);
    } else {
        k_huf_expand<Sink><<<gx, 256, 0, st>>>(huf_view(w), C, w.R, row0, nrows, sink);
    }
    check_launch();
}

} // namespace

// ---------------------------------------------------------------- entry points used by the C ABI (capi.cu)

void gemv_init() {
    const int optin = device_info().smem_optin;
#define ATTR(KERNEL, BYTES) allow_dynamic_smem((const void *) KERNEL, (int) (BYTES), optin, #KERNEL)
#define MC_ATTR(TX, CC) \
    ATTR((k_pair_gemv<CC, 1, TX, false>), 4 * HP_MAX_PAIRS + 1 * CC * CHUNK * 4); ATTR((k_pair_gemv<CC, 2, TX, false>), 4 * HP_MAX_PAIRS + 2 * CC * CHUNK * 4); \
    ATTR((k_pair_gemv<CC, 3, TX, false>), 4 * HP_MAX_PAIRS + 3 * CC * CHUNK * 4); ATTR((k_pair_gemv<CC, 4, TX, false>), 4 * HP_MAX_PAIRS + 4 * CC * CHUNK * 4);
    MC_ATTR(float, 1) MC_ATTR(float, 2) MC_ATTR(float, 4) MC_ATTR(float, 8)
    MC_ATTR(bf16, 1) MC_ATTR(bf16, 2) MC_ATTR(bf16, 4) MC_ATTR(bf16, 8)
#undef MC_ATTR
    ATTR((k_pair_glu<8, float>), 8 * HP_MAX_PAIRS + 8 * CHUNK * 4);
    ATTR((k_pair_glu<8, bf16>), 8 * HP_MAX_PAIRS + 8 * CHUNK * 4);
    ATTR((k_pair_glu<4, float>), 8 * HP_MAX_PAIRS + 4 * CHUNK * 4);
    ATTR((k_pair_glu<4, bf16>), 8 * HP_MAX_PAIRS + 4 * CHUNK * 4);
#undef ATTR
    gemv_staged_init();
    gemv_rings_init();
}

void gemv(const bf16n_weight & w, const bf16n_mmv_args & a, cudaStream_t st, bool multi_col, const bf16n_peer_out * peers) {
    if (a.x_bf16) { launch_gemv<bf16>(w, a, st, multi_col, peers); } else { launch_gemv<float>(w, a, st, multi_col, peers); }
}

// ---------------------------------------------------------------- several independent small products in one launch

namespace {

constexpr int GROUP_MAX = 8;
struct NibItem { // one dense NIBBLE product of a group
    NibView v;
    const char * x; char * y;
    int64_t x_tok, y_tok, row0, nrows;
    int ncols, chunks, first_block, blocks; // blocks [first_block, first_block + blocks) of the grid serve this item
    bool x_bf16, y_bf16;
};
struct NibGroup { int n; NibItem item[GROUP_MAX]; };

template <int C, typename TX>
__device__ __forceinline__ void nib_item_rows(const NibItem & it, int block, int col) {
    const TX * xg = (const TX *) (it.x + col * it.x_tok);
    const OutVec out = {it.y + col * it.y_tok, it.y_bf16};
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    bool waited = false;
    for (int64_t r = (int64_t) block * 8 + warp; r < it.nrows; r += (int64_t) it.blocks * 8) {
        NibRow<C> d;
        nib_load<C>(d, it.v, it.row0 + r, lane);
        if (!waited) { grid_dependency_wait(); waited = true; } // weights first, then the activations an earlier kernel may have written
        const float s = nib_dot<C, TX>(d, it.v, xg, lane);
        if (lane == 0) { out.put(r, s); }
    }
    if (!waited) { grid_dependency_wait(); }
}

// Every block belongs to one item of the group (a prefix table of block ranges); within its item it is a block of the
// single-product kernel: same loads, same order of operations, so the results are the same bits.
__global__ void __launch_bounds__(256) k_nib_gemv_group(const NibGroup g) {
    int m = 0;
    while (m + 1 < g.n && (int) blockIdx.x >= g.item[m + 1].first_block) { m++; }
    const NibItem & it = g.item[m];
    const int local = (int) blockIdx.x - it.first_block;
    const int col = local / (it.blocks / it.ncols), block = local % (it.blocks / it.ncols);
    NibItem one = it;
    one.blocks = it.blocks / it.ncols;
    const int key = it.chunks * 2 + (it.x_bf16 ? 1 : 0);
    switch (key) {
        case 2: nib_item_rows<1, float>(one, block, col); break;
        case 3: nib_item_rows<1, bf16>(one, block, col); break;
        case 4: nib_item_rows<2, float>(one, block, col); break;
        case 5: nib_item_rows<2, bf16>(one, block, col); break;
        case 8: nib_item_rows<4, float>(one, block, col); break;
        case 9: nib_item_rows<4, bf16>(one, block, col); break;
        case 16: nib_item_rows<8, float>(one, block, col); break;
        case 17: nib_item_rows<8, bf16>(one, block, col); break;
        default: grid_dependency_wait(); break;
    }
}

} // namespace

// dense NIBBLE products of up to 8 columns can share a grid
bool gemv_groupable(const bf16n_weight & w, const bf16n_mmv_args & a) {
    const int C = (int) (w.K / CHUNK);
    return w.format == FMT_NIBBLE && !a.ids && a.nrows > 0 && a.ncols >= 1 && a.ncols <= 8 && (C == 1 || C == 2 || C == 4 || C == 8);
}

// n independent groupable products (different matrices, activations and outputs) on one stream: one grid per eight.
void gemv_group(const bf16n_weight * w, const bf16n_mmv_args * a, int n, cudaStream_t st) {
    int i = 0;
    while (i < n) {
        NibGroup g = {};
        int blocks = 0;
        while (i < n && g.n < GROUP_MAX) {
            NibItem & it = g.item[g.n++];
            it.v = nib_view(w[i]);
            it.x = (const char *) a[i].x; it.y = (char *) a[i].y;
            it.x_tok = a[i].x_tok; it.y_tok = a[i].y_tok; it.row0 = a[i].row0; it.nrows = a[i].nrows;
            it.ncols = a[i].ncols; it.chunks = (int) (w[i].K / CHUNK);
            it.x_bf16 = a[i].x_bf16 != 0; it.y_bf16 = a[i].y_bf16 != 0;
            const dim3 geo = row_geometry(a[i].nrows, a[i].ncols);
            it.first_block = blocks;
            it.blocks = (int) geo.x * a[i].ncols;
            blocks += it.blocks;
            i++;
        }
        launch_chained(k_nib_gemv_group, dim3((unsigned) blocks), dim3(256), 0, st, g);
        check_launch();
    }
}

void gemv_glu_merged(const bf16n_weight & w, const bf16n_mmv_args & a, cudaStream_t st) {
    const NibView up = nib_view(w, a.nrows);
    if (a.x_bf16) { launch_glu<bf16>(w, &up, nullptr, a, st); } else { launch_glu<float>(w, &up, nullptr, a, st); }
}

void gemv_glu(const bf16n_weight & g, const bf16n_weight & u, const bf16n_mmv_args & a, cudaStream_t st) {
    if (a.x_bf16) { launch_glu<bf16>(g, nullptr, &u, a, st); } else { launch_glu<float>(g, nullptr, &u, a, st); }
}

void expand_store(const bf16n_weight & w, int64_t row0, int64_t nrows, uint16_t * out, cudaStream_t st) {
    launch_expand(w, row0, nrows, StoreBF16{out, w.K}, st);
}

void expand_compare(const bf16n_weight & w, int64_t row0, int64_t nrows, const uint16_t * src, unsigned long long * total,
                    cudaStream_t st) {
    launch_expand(w, row0, nrows, CompareBF16{src, w.K, total, 0u}, st);
}

void gather_rows(const bf16n_weight & w, const void * ids, int64_t ids_s0, int64_t n, void * dst, bool dst_bf16, int64_t dst_s1,
                 int64_t row0, cudaStream_t st) {
    const int C = (int) (w.K / CHUNK);
    const unsigned gx = (unsigned) ((n + 7) / 8);
    const char * ip = (const char *) ids;
    char * dp = (char *) dst;
    if (w.format == FMT_NIBBLE) {
        if (dst_bf16) { k_nib_rows<true><<<gx, 256, 0, st>>>(nib_view(w), C, ip, ids_s0, n, row0, dp, dst_s1); }
        else { k_nib_rows<false><<<gx, 256, 0, st>>>(nib_view(w), C, ip, ids_s0, n, row0, dp, dst_s1); }
    } else {
        if (dst_bf16) { k_pair_rows<true><<<gx, 256, 0, st>>>(pair_view(w), C, w.R, ip, ids_s0, n, row0, dp, dst_s1); }
        else { k_pair_rows<false><<<gx, 256, 0, st>>>(pair_view(w), C, w.R, ip, ids_s0, n, row0, dp, dst_s1); }
    }
    check_launch();
}

} // namespace b16
