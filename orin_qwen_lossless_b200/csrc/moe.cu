// Small MoE-layer kernels around the expert GEMVs: the router (softmax top-k on the device), SwiGLU, the weighted
// combine of the expert outputs, and the routing sort that feeds the batched (prefill) kernel.
#include "decode.cuh"
#include "launch.h"

namespace b16 {
namespace {

using namespace dev;

// ---------------------------------------------------------------- router: softmax + top-k, one warp per token

// The k largest logits of a token (ties: lowest expert index), weights exp(z_i - max) renormalised over the selected
// ones, which equals softmax followed by renormalisation. Lane l holds experts l, l+32, ...; up to 1024 experts.
constexpr int TOPK_MAX_PER_LANE = 32;

template <int PER> // experts per lane: the register array and every scan are this long
__global__ void __launch_bounds__(32) k_topk(const float * __restrict__ logits, int n_experts, int k, int32_t * __restrict__ ids,
                                             float * __restrict__ weights) {
    grid_dependency_wait(); // the logits come from an earlier kernel
    const int t = blockIdx.x, lane = threadIdx.x;
    const float * z = logits + (int64_t) t * n_experts;
    float v[PER];
#pragma unroll
    for (int i = 0; i < PER; i++) {
        const int e = i * 32 + lane;
        v[i] = e < n_experts ? z[e] : -INFINITY;
    }
    float zmax = 0.f, denom = 0.f;
    for (int s = 0; s < k; s++) {
        // lane-local best (lowest index on ties: strict > while scanning upward)
        float best = -INFINITY;
        int bi = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < PER; i++) {
            if (v[i] > best) { best = v[i]; bi = i * 32 + lane; }
        }
        // warp arg-max with the same tie rule
#pragma unroll
        for (int o = 16; o; o >>= 1) {
            const float ob = __shfl_xor_sync(FULL, best, o);
            const int oi = __shfl_xor_sync(FULL, bi, o);
            if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
        }
        if (s == 0) { zmax = best; }
        const float pw = __expf(best - zmax);
        denom += pw;
        if (lane == 0) {
            ids[(int64_t) t * k + s] = bi;
            weights[(int64_t) t * k + s] = pw;
        }
        if ((bi & 31) == lane) { // retire the winner
#pragma unroll
            for (int i = 0; i < PER; i++) {
                if (i == (bi >> 5)) { v[i] = -INFINITY; }
            }
        }
    }
    __syncwarp();
    if (lane < k) { weights[(int64_t) t * k + lane] = __fdividef(weights[(int64_t) t * k + lane], denom); }
}

// ---------------------------------------------------------------- elementwise

__global__ void k_swiglu(const float * __restrict__ g, const float * __restrict__ u, float * __restrict__ y, int64_t n) {
    for (int64_t i = blockIdx.x * (int64_t) blockDim.x + threadIdx.x; i < n; i += (int64_t) gridDim.x * blockDim.x) {
        y[i] = silu_f(g[i]) * u[i];
    }
}

// y[t, i] = sum over slots k, in slot order, of w[t, k] * ys[t, k, i]
__global__ void k_combine(const float * __restrict__ ys, const char * __restrict__ w, bool w_bf16, char * __restrict__ y, bool y_bf16,
                          int n_used, int64_t n) {
    const int t = blockIdx.y;
    const OutVec out = {y + (int64_t) t * n * (y_bf16 ? 2 : 4), y_bf16};
    for (int64_t i = blockIdx.x * (int64_t) blockDim.x + threadIdx.x; i < n; i += (int64_t) gridDim.x * blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < n_used; k++) {
            const int64_t s = (int64_t) t * n_used + k;
            const float wk = w_bf16 ? to_f32(((const __nv_bfloat16 *) w)[s]) : ((const float *) w)[s];
            acc = fmaf(wk, ys[s * n + i], acc);
        }
        out.put(i, acc);
    }
}

// ---------------------------------------------------------------- routing sort (prefill)

// One block per expert. Pass 1 counts the routed pairs of lower-numbered experts (this expert's first output index);
// pass 2 walks the tokens in order, 256 at a time, and compacts the tokens that use this expert with a block-wide
// exclusive scan, so the expert's pairs come out sorted by token.
template <typename TI>
__global__ void __launch_bounds__(256) k_route(const TI * __restrict__ ids, int64_t row_stride, int32_t * __restrict__ ids_src1,
                                               int32_t * __restrict__ ids_dst, int32_t * __restrict__ bounds, int n_tok, int n_used,
                                               int nchannels_y, int sis1) {
    const int e = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    __shared__ int warp_tot[8];
    __shared__ int s_base;

    // int32 ids in contiguous rows of a multiple of four: four ids per load (the common case: 8 slots per token)
    const bool vec = sizeof(TI) == 4 && n_used % 4 == 0 && row_stride == n_used && ((uintptr_t) ids & 15) == 0;
    int lower = 0;
    if (vec) {
        const int4 * v = (const int4 *) ids;
        for (int64_t i = tid; i < (int64_t) n_tok * n_used / 4; i += 256) {
            const int4 q = __ldg(v + i);
            lower += (q.x < e) + (q.y < e) + (q.z < e) + (q.w < e);
        }
    } else {
        for (int64_t i = tid; i < (int64_t) n_tok * n_used; i += 256) {
            const int t = (int) (i / n_used), s = (int) (i - (int64_t) t * n_used);
            lower += (int) ids[t * row_stride + s] < e;
        }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) { lower += __shfl_xor_sync(FULL, lower, o); }
    if (lane == 0) { warp_tot[warp] = lower; }
    __syncthreads();
    if (tid == 0) {
        int b = 0;
        for (int i = 0; i < 8; i++) { b += warp_tot[i]; }
        s_base = b;
    }
    __syncthreads();
    const int base = s_base;
    int done = 0;
    for (int t0 = 0; t0 < n_tok; t0 += 256) {
        const int t = t0 + tid;
        int slot = -1;
        if (t < n_tok) {
            if (vec) {
                const int4 * v = (const int4 *) ids + (int64_t) t * (n_used / 4);
                for (int s4 = n_used / 4 - 1; s4 >= 0; s4--) { // downwards, so that the lowest matching slot wins
                    const int4 q = __ldg(v + s4);
                    slot = q.w == e ? 4 * s4 + 3 : slot;
                    slot = q.z == e ? 4 * s4 + 2 : slot;
                    slot = q.y == e ? 4 * s4 + 1 : slot;
                    slot = q.x == e ? 4 * s4 : slot;
                }
            } else {
                for (int s = 0; s < n_used; s++) {
                    if ((int) ids[t * row_stride + s] == e) { slot = s; break; }
                }
            }
        }
        const unsigned hit = __ballot_sync(FULL, slot >= 0);
        __syncthreads(); // warp_tot is reused
        if (lane == 0) { warp_tot[warp] = __popc(hit); }
        __syncthreads();
        int before = 0, total = 0;
        for (int i = 0; i < 8; i++) {
            before += i < warp ? warp_tot[i] : 0;
            total += warp_tot[i];
        }
        if (slot >= 0) {
            const int j = base + done + before + __popc(hit & ((1u << lane) - 1));
            ids_src1[j] = t * sis1 + slot % nchannels_y;
            ids_dst[j] = t * n_used + slot;
        }
        done += total;
    }
    if (tid == 0) {
        bounds[e] = base;
        if (e == (int) gridDim.x - 1) { bounds[e + 1] = base + done; }
    }
}

} // namespace

void moe_init() {}

void moe_topk(const float * logits, int n_tok, int n_experts, int k, int32_t * ids, float * weights, cudaStream_t st) {
    require(n_tok >= 0 && n_experts > 0 && n_experts <= 32 * TOPK_MAX_PER_LANE, "moe_topk: 1..1024 experts");
    require(k > 0 && k <= 32 && k <= n_experts, "moe_topk: k must be in 1..min(32, n_experts)");
    if (n_tok == 0) { return; }
    if (n_experts <= 256) {
        launch_chained(k_topk<8>, dim3(n_tok), dim3(32), 0, st, logits, n_experts, k, ids, weights);
    } else {
        launch_chained(k_topk<TOPK_MAX_PER_LANE>, dim3(n_tok), dim3(32), 0, st, logits, n_experts, k, ids, weights);
    }
}

void moe_combine(const float * ys, const void * w, bool w_bf16, void * y, bool y_bf16, int n_tok, int n_used, int64_t n,
                 cudaStream_t st) {
    if (n_tok == 0 || n == 0) { return; }
    require(n_tok <= 65535, "moe_combine: too many tokens for one launch");
    const dim3 grid((unsigned) std::min<int64_t>((n + 255) / 256, 64), (unsigned) n_tok);
    k_combine<<<grid, 256, 0, st>>>(ys, (const char *) w, w_bf16, (char *) y, y_bf16, n_used, n);
    check_launch();
}

void moe_swiglu(const float * g, const float * u, float * y, int64_t n, cudaStream_t st) {
    if (n == 0) { return; }
    const unsigned blocks = (unsigned) std::min<int64_t>((n + 255) / 256, (int64_t) device_info().sms * 8);
    k_swiglu<<<blocks, 256, 0, st>>>(g, u, y, n);
    check_launch();
}

void moe_route(const void * ids, bool ids_i64, int64_t ids_row_stride, int32_t * ids_src1, int32_t * ids_dst, int32_t * bounds,
               int n_experts, int n_tok, int n_used, int nchannels_y, int sis1, cudaStream_t st) {
    require(n_tok > 0 && n_tok < (1 << 22) && n_used > 0 && n_used < (1 << 10), "routing sizes out of range");
    require(n_experts > 0, "routing needs at least one expert");
    require((int64_t) n_tok * ids_row_stride < INT32_MAX, "routing ids too large for 32-bit indexing");
    if (ids_i64) {
        k_route<int64_t><<<n_experts, 256, 0, st>>>((const int64_t *) ids, ids_row_stride, ids_src1, ids_dst, bounds, n_tok, n_used,
                                                    nchannels_y, sis1);
    } else {
        k_route<int32_t><<<n_experts, 256, 0, st>>>((const int32_t *) ids, ids_row_stride, ids_src1, ids_dst, bounds, n_tok, n_used,
                                                    nchannels_y, sis1);
    }
    check_launch();
}

} // namespace b16
