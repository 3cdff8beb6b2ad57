// Draft-only k-bit copies of an output head (the reference's core/include/bf16n/draft_head.cuh:22-281, declared for its
// op shim at core/torch/torch_bindings.cpp:22-29): a 4-bit or 2-bit copy of a BF16 matrix with one FP32 scale per 128
// weights scores candidates, which the caller re-scores exactly from the lossless rows. The stored formats are the
// reference's, so copies made by either library serve either GEMV:
//   4 bit: q[r][k / 2], column k in the low (k even) or high nibble, value + 8; scale = amax / 7 (1 for a zero group)
//   2 bit: bits 2 (k % 16) of 32-bit word k / 16 of row r hold n in 0..3, value (n - 1.5) s, s = amax / 1.5 correctly
//          rounded; floor(w / s) clamped to [-2, 1], so ties go to the upper level; an all-zero group has s = 0
// The products are approximate by design (FP16 partial sums over one 32-bit word of weights); every column takes the
// same operations in the same order whatever the batch, so a column's scores do not depend on its neighbours.
//
// Built for B200 rather than carried over: quantisation is warp-cooperative (a warp per 128-weight group: coalesced
// 8-byte loads, shuffle reductions, packing by shuffles), and the GEMV is a persistent grid of one-warp-per-row loops
// with the next row's 16 bytes per lane in flight while the current one is multiplied.
#include "decode.cuh"
#include "launch.h"

#include <cuda_fp16.h>

namespace b16 {
namespace {

using namespace dev;
using bf16 = __nv_bfloat16;
constexpr int G = 128; // weights per scale

// One warp per (row, group): lane l holds columns 4 l .. 4 l + 3 of the group.
template <int BITS>
__global__ void __launch_bounds__(256) k_kbit_quantize(const bf16 * __restrict__ w, int64_t rows, int K, uint8_t * __restrict__ q,
                                                       float * __restrict__ s) {
    const int lane = threadIdx.x & 31;
    const int groups = K / G;
    const int64_t total = rows * groups;
    for (int64_t i = (blockIdx.x * (int64_t) blockDim.x + threadIdx.x) >> 5; i < total; i += ((int64_t) gridDim.x * blockDim.x) >> 5) {
        const int64_t r = i / groups;
        const int g = (int) (i - r * groups);
        const uint2 raw = __ldg((const uint2 *) (w + r * K + g * G) + lane);
        const float v[4] = {bf16lo_f32(raw.x), bf16hi_f32(raw.x), bf16lo_f32(raw.y), bf16hi_f32(raw.y)};
        float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
        for (int o = 16; o; o >>= 1) { amax = fmaxf(amax, __shfl_xor_sync(FULL, amax, o)); }
        if (BITS == 4) {
            const float scale = amax > 0.f ? __fdiv_rn(amax, 7.f) : 1.f;
            uint32_t nib = 0; // four nibbles: columns 4 l .. 4 l + 3 = two bytes
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const int a = (int) fminf(fmaxf(rintf(__fdiv_rn(v[c], scale)), -8.f), 7.f) + 8;
                nib |= (uint32_t) a << (4 * c);
            }
            ((uint16_t *) (q + r * (K / 2) + g * (G / 2)))[lane] = (uint16_t) nib;
            if (lane == 0) { s[i] = scale; }
        } else {
            const float scale = __fdiv_rn(amax, 1.5f);
            uint32_t bits = 0; // four 2-bit levels = one byte: columns 4 l .. 4 l + 3 are bits 8 (l % 4) .. of word l / 4
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const int n = scale > 0.f ? (int) fminf(fmaxf(floorf(__fdiv_rn(v[c], scale)), -2.f), 1.f) + 2 : 2;
                bits |= (uint32_t) n << (2 * c);
            }
            (q + r * (K / 4) + g * (G / 4))[lane] = (uint8_t) bits;
            if (lane == 0) { s[i] = scale; }
        }
    }
}

__device__ __forceinline__ __half2 magic_half2(uint32_t fields) { // two small integers in bits 0.. and 16.. -> (1024 + a, 1024 + b)
    const uint32_t p = fields | 0x64006400u;
    return *(const __half2 *) &p;
}

// 4 bit: one warp per row; per 1024 columns a lane owns 16 contiguous bytes (columns 32 l .. 32 l + 31 of the slab: a
// quarter of a scale group). Word w of them holds columns 8 w .. 8 w + 7, nibble m = column 8 w + m; a half2 pairs
// nibbles j and j + 4 (one shift and one mask). x in registers as half2 in that order.
template <int T, int NIT>
__global__ void __launch_bounds__(256) k_int4_gemv(const bf16 * __restrict__ x, const uint8_t * __restrict__ q, const float * __restrict__ s,
                                                   int64_t rows, float * __restrict__ y) {
    constexpr int K = NIT * 1024;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __half2 xr[T][NIT][16];
#pragma unroll
    for (int t = 0; t < T; t++) {
#pragma unroll
        for (int it = 0; it < NIT; it++) {
            const bf16 * xp = x + (int64_t) t * K + it * 1024 + lane * 32;
#pragma unroll
            for (int w = 0; w < 4; w++) {
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    xr[t][it][4 * w + j] = __floats2half2_rn(__bfloat162float(xp[8 * w + j]), __bfloat162float(xp[8 * w + j + 4]));
                }
            }
        }
    }
    const __half2 bias = __float2half2_rn(1032.f); // 1024 + 8
    const int64_t stride = (int64_t) gridDim.x * 8;
    int64_t r = blockIdx.x * 8 + warp;
    uint4 v[NIT]; float sc[NIT];
    auto load = [&](int64_t row, uint4 (&vv)[NIT], float (&ss)[NIT]) {
#pragma unroll
        for (int it = 0; it < NIT; it++) {
            vv[it] = ld_stream16(q + row * (K / 2) + it * 512 + lane * 16);
            ss[it] = __ldg(s + row * (K / G) + it * 8 + lane / 4);
        }
    };
    if (r < rows) { load(r, v, sc); }
    for (; r < rows; r += stride) {
        uint4 vn[NIT]; float scn[NIT];
#pragma unroll
        for (int it = 0; it < NIT; it++) { vn[it] = make_uint4(0, 0, 0, 0); scn[it] = 0.f; }
        if (r + stride < rows) { load(r + stride, vn, scn); }
        float acc[T];
#pragma unroll
        for (int t = 0; t < T; t++) { acc[t] = 0.f; }
#pragma unroll
        for (int it = 0; it < NIT; it++) {
            const uint32_t words[4] = {v[it].x, v[it].y, v[it].z, v[it].w};
            __half2 h[T];
#pragma unroll
            for (int t = 0; t < T; t++) { h[t] = __float2half2_rn(0.f); }
#pragma unroll
            for (int w = 0; w < 4; w++) {
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const __half2 wv = __hsub2(magic_half2((words[w] >> (4 * j)) & 0x000F000Fu), bias);
#pragma unroll
                    for (int t = 0; t < T; t++) { h[t] = __hfma2(wv, xr[t][it][4 * w + j], h[t]); }
                }
            }
#pragma unroll
            for (int t = 0; t < T; t++) {
                const float2 f = __half22float2(h[t]);
                acc[t] = fmaf(f.x + f.y, sc[it], acc[t]);
            }
        }
#pragma unroll
        for (int t = 0; t < T; t++) {
            const float val = warp_sum(acc[t]);
            if (lane == 0) { y[(int64_t) t * rows + r] = val; }
        }
#pragma unroll
        for (int it = 0; it < NIT; it++) { v[it] = vn[it]; sc[it] = scn[it]; }
    }
}

// 2 bit, K = 2048: a lane owns 16 contiguous bytes = 64 weights (half a scale group); a half2 pairs the fields at bits
// 2 j and 2 j + 16 of a word (columns 16 wd + j and 16 wd + j + 8). sum_k (n_k - 1.5) x_k = sum_k n_k x_k - 1.5 sum_k x_k:
// the second sum is a per-lane constant of the column.
template <int NC>
__global__ void __launch_bounds__(256, NC == 1 ? 3 : 1) k_int2_gemv(const bf16 * __restrict__ x, const uint8_t * __restrict__ q,
                                                                      const float * __restrict__ s, int64_t rows, float * __restrict__ y) {
    constexpr int K = 2048;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __half2 xr[NC][32];
    float xsum[NC];
#pragma unroll
    for (int c = 0; c < NC; c++) {
        const bf16 * xp = x + (int64_t) c * K + lane * 64;
        float sum = 0.f;
#pragma unroll
        for (int wd = 0; wd < 4; wd++) {
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const float a = __bfloat162float(xp[16 * wd + j]), b = __bfloat162float(xp[16 * wd + j + 8]);
                xr[c][8 * wd + j] = __floats2half2_rn(a, b);
                sum += a + b;
            }
        }
        xsum[c] = sum;
    }
    const __half2 bias = __float2half2_rn(1024.f);
    const int64_t stride = (int64_t) gridDim.x * 8;
    int64_t r = blockIdx.x * 8 + warp;
    uint4 v = make_uint4(0, 0, 0, 0);
    float sc = 0.f;
    if (r < rows) {
        v = ld_stream16(q + r * (K / 4) + lane * 16);
        sc = __ldg(s + r * (K / G) + lane / 2);
    }
    for (; r < rows; r += stride) {
        const int64_t rn = r + stride;
        uint4 vn = make_uint4(0, 0, 0, 0);
        float scn = 0.f;
        if (rn < rows) {
            vn = ld_stream16(q + rn * (K / 4) + lane * 16);
            scn = __ldg(s + rn * (K / G) + lane / 2);
        }
        const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int c = 0; c < NC; c++) {
            float nx = 0.f;
#pragma unroll
            for (int wd = 0; wd < 4; wd++) {
                __half2 h0 = __float2half2_rn(0.f), h1 = h0; // two chains of four products: half the dependent latency
#pragma unroll
                for (int j = 0; j < 8; j += 2) {
                    h0 = __hfma2(__hsub2(magic_half2((words[wd] >> (2 * j)) & 0x00030003u), bias), xr[c][8 * wd + j], h0);
                    h1 = __hfma2(__hsub2(magic_half2((words[wd] >> (2 * j + 2)) & 0x00030003u), bias), xr[c][8 * wd + j + 1], h1);
                }
                const float2 f = __half22float2(__hadd2(h0, h1));
                nx += f.x + f.y;
            }
            const float val = warp_sum(fmaf(fmaf(-1.5f, xsum[c], nx), sc, 0.f));
            if (lane == 0) { y[(int64_t) c * rows + r] = val; }
        }
        v = vn;
        sc = scn;
    }
}

unsigned quantize_blocks(int64_t rows, int K) { // 8 warps per block, a warp per group
    return (unsigned) std::max<int64_t>(1, std::min<int64_t>((rows * (K / G) + 7) / 8, (int64_t) device_info().sms * 32));
}

template <int T>
void int4_gemv_t(const bf16 * x, const uint8_t * q, const float * s, int64_t rows, int K, float * y, unsigned blocks, cudaStream_t st) {
    switch (K) {
        case 1024: k_int4_gemv<T, 1><<<blocks, 256, 0, st>>>(x, q, s, rows, y); break;
        case 2048: k_int4_gemv<T, 2><<<blocks, 256, 0, st>>>(x, q, s, rows, y); break;
        default: k_int4_gemv<T, 4><<<blocks, 256, 0, st>>>(x, q, s, rows, y); break;
    }
}

} // namespace

void draft_quantize(int bits, const void * w_bf16, int64_t rows, int K, uint8_t * q, float * s, cudaStream_t st) {
    require(bits == 2 || bits == 4, "draft head: 2 or 4 bits");
    require(K > 0 && K % G == 0, bits == 4 ? "int4_quantize: K must be a multiple of 128" : "int2_quantize: K must be a multiple of 128");
    require(rows >= 0 && (rows == 0 || (w_bf16 && q && s)), "draft head quantize: null argument");
    require((uintptr_t) w_bf16 % 8 == 0 && (uintptr_t) q % 4 == 0, "draft head quantize: w must be 8-byte and q 4-byte aligned");
    if (rows == 0) { return; }
    if (bits == 4) { k_kbit_quantize<4><<<quantize_blocks(rows, K), 256, 0, st>>>((const bf16 *) w_bf16, rows, K, q, s); }
    else { k_kbit_quantize<2><<<quantize_blocks(rows, K), 256, 0, st>>>((const bf16 *) w_bf16, rows, K, q, s); }
    check_launch();
}

void draft_gemv(int bits, const void * x_bf16, int T, const uint8_t * q, const float * s, int64_t rows, int K, float * y, cudaStream_t st) {
    require(bits == 2 || bits == 4, "draft head: 2 or 4 bits");
    if (bits == 4) { require(K == 1024 || K == 2048 || K == 4096, "int4_gemv: K must be 1024, 2048 or 4096"); }
    else { require(K == 2048, "int2_gemv: K must be 2048"); }
    require(T >= 1 && T <= 4, bits == 4 ? "int4_gemv: 1 to 4 columns" : "int2_gemv: 1 to 4 columns");
    require(rows >= 0 && (rows == 0 || (x_bf16 && q && s && y)), "draft head gemv: null argument");
    require((uintptr_t) q % 16 == 0, "draft head gemv: q must be 16-byte aligned");
    if (rows == 0) { return; }
    const bf16 * x = (const bf16 *) x_bf16;
    const int64_t sms = device_info().sms;
    if (bits == 4) {
        const unsigned blocks = (unsigned) std::min<int64_t>((rows + 7) / 8, sms * 8);
        switch (T) {
            case 1: int4_gemv_t<1>(x, q, s, rows, K, y, blocks, st); break;
            case 2: int4_gemv_t<2>(x, q, s, rows, K, y, blocks, st); break;
            case 3: int4_gemv_t<3>(x, q, s, rows, K, y, blocks, st); break;
            default: int4_gemv_t<4>(x, q, s, rows, K, y, blocks, st); break;
        }
    } else {
        for (int t = 0; t < T; t += 2) { // two columns per launch, an odd last one alone
            if (T - t >= 2) {
                const unsigned blocks = (unsigned) std::min<int64_t>((rows + 7) / 8, sms * 1 * 4);
                k_int2_gemv<2><<<blocks, 256, 0, st>>>(x + (int64_t) t * K, q, s, rows, y + (int64_t) t * rows);
            } else {
                const unsigned blocks = (unsigned) std::min<int64_t>((rows + 7) / 8, sms * 3 * 4);
                k_int2_gemv<1><<<blocks, 256, 0, st>>>(x + (int64_t) t * K, q, s, rows, y + (int64_t) t * rows);
            }
        }
    }
    check_launch();
}

} // namespace b16
