// Routed-expert products of a MoE decode step (1..8 tokens): latency-oriented kernels for the stacked expert matrices.
//
// A column is one (token, slot) pair whose expert id is read on the device. Work is split as finely as the format
// allows: one warp decodes one unit (R rows) of one matrix for one column, so a gate/up launch at 1 token is
// 8 slots x 2 matrices x 64 units = 1024 independent warps. Every warp stages its unit's exponent streams with one bulk
// async copy (bounded wait), keeps its activations in registers and walks the streams as in gemv_staged.cu.
//   k_expert_units<C, R, CM, TX, GLU_IN>:
//     CM      chunk-major units (gate / up, K > 512): per chunk the R rows share the lane's activations
//     GLU_IN  the activation of the column is silu(g) * u formed while loading (the down product reads the gate and up
//             outputs directly: no separate activation kernel and no third buffer)
//   grid = (unit groups, columns, matrices): blockIdx.z picks gate or up so that one launch covers both.
// Columns whose expert lies outside [e_lo, e_lo + e_n) (expert-parallel ranks own a slice of the experts) write zeros.
// Summation order per row is the format's (chunk sums per row, then the xor butterfly), identical to the general
// kernels, so results are bit-identical to bf16n_mmv on the same expert.
#include "staged.cuh"
#include "launch.h"

#include <cstdlib>
#include <mutex>

namespace b16 {
namespace {

using namespace dev;

struct ExpertMat { // one stacked expert matrix (n_experts * rows_per_expert rows)
    PairView v;
    const AuxHeader * hdr;
    char * y;          // FP32 output [n_tok, n_used, rows_per_expert]
};

struct ExpertCols {
    const char * x;  int64_t x_tok, x_slot;   // activations: per token (x_slot = 0) or per (token, slot)
    const float * x2;                          // GLU_IN: second factor, same indexing as x (FP32)
    const char * ids; int64_t ids_s0, ids_s1;
    int n_used;
    int64_t rows_per_expert;
    int e_lo, e_n;                             // experts held by this weight: global ids [e_lo, e_lo + e_n)
    uint32_t cap_bytes;
    bool early_ids;                            // the expert ids were complete before the PREVIOUS kernel on the stream
                                               // began its dependent work (they come from a kernel before that one):
                                               // ids, unit geometry and the bulk copies need not wait for it; only the
                                               // activations do
};

template <int C, int R, bool CM, typename TX, bool GLU_IN, bool PLANE_STAGED>
__global__ void __launch_bounds__(256) k_expert_units(const ExpertMat m0, const ExpertMat m1, const ExpertCols p, const Opaque k) {
    constexpr int K = C * CHUNK;
    extern __shared__ __align__(128) unsigned char smem[];
    uint32_t * lut = (uint32_t *) smem;
    uint64_t * bars = (uint64_t *) (smem + 4 * HP_MAX_PAIRS);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    constexpr uint32_t PLANE_BYTES = PLANE_STAGED ? (uint32_t) (R * K) : 0u;   // the unit's sign|mantissa bytes, staged with its streams
    unsigned char * buf = smem + 4 * HP_MAX_PAIRS + 128 + (size_t) warp * (p.cap_bytes + PLANE_BYTES);
    const unsigned char * plane_s = buf + p.cap_bytes;
    const uint32_t bar = smem_u32(bars + warp);
    const ExpertMat & m = blockIdx.z ? m1 : m0;

    // independent prologue: the table and the barrier do not depend on earlier kernels
    for (int i = threadIdx.x; i < HP_MAX_PAIRS / 4; i += blockDim.x) { ((uint4 *) lut)[i] = __ldg((const uint4 *) m.v.lut + i); }
    if (lane == 0) { mbar_init(bar, 1); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncthreads();
    // Expert ids, activations and the output buffers belong to earlier kernels. Normally everything below waits for
    // them. With early_ids only the activations come from the kernel right before this one: that kernel's blocks let
    // this one start only after their own wait, i.e. after everything older (ids, the last reader of the outputs) was
    // complete and visible, so the ids, the unit geometry and the bulk copies of streams and plane run ahead of it.
    if (!p.early_ids) { grid_dependency_wait(); }

    const int col = blockIdx.y, t = col / p.n_used, s = col - t * p.n_used;
    const int e = *(const int32_t *) (p.ids + t * p.ids_s1 + s * p.ids_s0) - p.e_lo;
    const int64_t units = p.rows_per_expert / R;
    const int64_t u = (int64_t) blockIdx.x * nwarp + warp;
    float * y = (float *) m.y + ((int64_t) t * p.n_used + s) * p.rows_per_expert;
    if (e < 0 || e >= p.e_n) { // not this rank's expert: the combine adds exact zeros
        if (u < units && lane < R) { y[u * R + lane] = 0.f; }
        return;
    }
    if (u >= units) { return; }

    const int64_t gu = (int64_t) e * units + u;
    const uint32_t w0 = __ldg(m.v.ubase + gu);
    const uint32_t w1 = gu + 1 < (int64_t) m.hdr->n_a ? __ldg(m.v.ubase + gu + 1) : (uint32_t) m.hdr->n_b;
    const uint32_t start = w0 & ~3u, bytes = ((w1 - start + 4u + 3u) & ~3u) * 4u;
    const bool staged = bytes <= p.cap_bytes;
    const bool plane_staged = PLANE_STAGED && staged;
    if (staged && lane == 0) {
        mbar_expect_tx(bar, bytes + (plane_staged ? PLANE_BYTES : 0u));
        bulk_g2s(smem_u32(buf), m.v.stream + start, bytes, bar);
        if (plane_staged) { bulk_g2s(smem_u32(plane_s), m.v.plane + gu * R * K, PLANE_BYTES, bar); }
    }
    if (!plane_staged && lane == 0) { bulk_prefetch_l2(m.v.plane + gu * R * K, (uint32_t) (R * K)); } // later chunks then hit L2
    const uint32_t my = w0 - start + __ldg(m.v.lrel + gu * 32 + lane);

    if (p.early_ids) { grid_dependency_wait(); }
    // this lane's activations, in registers (FP32 values; BF16 inputs are widened exactly)
    float4 xr[C * 4];
    {
        const char * xp = p.x + t * p.x_tok + s * p.x_slot;
        const float * x2 = GLU_IN ? p.x2 + (xp - p.x) / 4 : nullptr;
#pragma unroll
        for (int i = 0; i < C * 4; i++) {
            const int at = (i >> 2) * CHUNK + 128 * (i & 3) + 4 * lane;
            float4 v = ldg_x4((const TX *) xp, at); // an ordered load: stays behind the dependency wait
            if (GLU_IN) {
                const float4 g = v, w2 = ldg_x4(x2, at);
                v = make_float4(silu_f(g.x) * w2.x, silu_f(g.y) * w2.y, silu_f(g.z) * w2.z, silu_f(g.w) * w2.w);
            }
            xr[i] = v;
        }
    }
    const uint8_t * pl = m.v.plane + gu * R * K + 16 * lane;
    // one lane's 16 bytes of a row-chunk: from the staged copy (after the wait below) or straight from global memory
    auto plane16 = [&](int64_t off) -> uint4 {
        if (plane_staged) { return *(const uint4 *) (plane_s + 16 * lane + off); }
        return ld_stream16(pl + off);
    };

    auto rows = [&](auto & rd, uint32_t lut_arg) {
        float mine = 0.f;
        if (CM) {
            float acc[R];
#pragma unroll
            for (int rr = 0; rr < R; rr++) { acc[rr] = 0.f; }
#pragma unroll
            for (int c = 0; c < C; c++) {
                uint4 sm[R];
#pragma unroll
                for (int rr = 0; rr < R; rr++) { sm[rr] = plane16((c * R + rr) * CHUNK); }
#pragma unroll
                for (int rr = 0; rr < R; rr++) {
                    uint32_t en[8], wv[8];
                    rd.take8(lut_arg, k, en);
                    assemble8(sm[rr], en, wv);
                    float a[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const float4 xv = xr[(C == 1 ? 0 : c) * 4 + j];
                        a[0] = fmaf(bf16lo_f32(wv[2 * j]), xv.x, a[0]);
                        a[1] = fmaf(bf16hi_f32(wv[2 * j]), xv.y, a[1]);
                        a[2] = fmaf(bf16lo_f32(wv[2 * j + 1]), xv.z, a[2]);
                        a[3] = fmaf(bf16hi_f32(wv[2 * j + 1]), xv.w, a[3]);
                    }
                    acc[rr] += (a[0] + a[1]) + (a[2] + a[3]);
                }
            }
#pragma unroll
            for (int rr = 0; rr < R; rr++) {
                const float sum = warp_sum(acc[rr]);
                if (lane == rr) { mine = sum; }
            }
        } else {
            for (int rr = 0; rr < R; rr++) {
                float a[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int c = 0; c < C; c++) {
                    const uint4 sm = plane16(rr * K + c * CHUNK);
                    uint32_t en[8], wv[8];
                    rd.take8(lut_arg, k, en);
                    assemble8(sm, en, wv);
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const float4 xv = xr[c * 4 + j];
                        a[0] = fmaf(bf16lo_f32(wv[2 * j]), xv.x, a[0]);
                        a[1] = fmaf(bf16hi_f32(wv[2 * j]), xv.y, a[1]);
                        a[2] = fmaf(bf16lo_f32(wv[2 * j + 1]), xv.z, a[2]);
                        a[3] = fmaf(bf16hi_f32(wv[2 * j + 1]), xv.w, a[3]);
                    }
                }
                const float sum = warp_sum((a[0] + a[1]) + (a[2] + a[3]));
                if (lane == rr) { mine = sum; }
            }
        }
        return mine;
    };

    float mine;
    if (staged) {
        const uint32_t landed = mbar_wait(bar, 0);
        if (!landed) { // the copy never arrived: report it and leave NaN where the unit's rows go
            if (lane == 0) { atomicOr(&g_wait_expired, 1u); }
            mine = __int_as_float(0x7fc00000);
        } else {
            StagedReader rd;
            rd.open(smem_u32(buf) + 4 * my, landed);
            mine = rows(rd, smem_u32(lut));
        }
    } else {
        GlobalReader rd;
        rd.lut = lut;
        rd.rd.open(m.v, gu, lane);
        mine = rows(rd, 0u);
    }
    if (lane < R) { y[u * R + lane] = mine; }
}

// y[t, i] = sum over slots, in slot order, of w[t, k] * ys[t, k, i]
__global__ void k_combine_f32(const float * __restrict__ ys, const float * __restrict__ w, char * __restrict__ y, bool y_bf16, int n_used,
                              int64_t n, const PeerOut peers) {
    grid_dependency_wait();
    const int t = blockIdx.y;
    const OutVec out = {y + (int64_t) t * n * (y_bf16 ? 2 : 4), y_bf16};
    for (int64_t i = blockIdx.x * (int64_t) blockDim.x + threadIdx.x; i < n; i += (int64_t) gridDim.x * blockDim.x) {
        float acc = 0.f;
        for (int kx = 0; kx < n_used; kx++) { // the slot outputs come from the launch right before this one: ordered loads
            const int64_t s = (int64_t) t * n_used + kx;
            acc = fmaf(w[s], ld_act_f32(ys + s * n + i), acc);
        }
        out.put(i, acc);
        peers_put(peers, (int64_t) t * n * (y_bf16 ? 2 : 4), y_bf16, i, acc);
    }
    peers_done(peers); // expert-parallel ranks: the partial output also went to every peer; announce it and await theirs
}

// y[i] = parts[0][i] + parts[1][i] + ... (+ extra[i]): the ranks' partial outputs in rank order, the same on every rank
__global__ void k_peer_sum(const float * __restrict__ parts, int n_parts, int64_t n, const float * __restrict__ extra,
                           char * __restrict__ y, bool y_bf16) {
    grid_dependency_wait();
    const OutVec out = {y, y_bf16};
    for (int64_t i = blockIdx.x * (int64_t) blockDim.x + threadIdx.x; i < n; i += (int64_t) gridDim.x * blockDim.x) {
        float acc = ld_act_f32(parts + i); // stored by the launch before this one and by the peers' kernels: ordered loads
        for (int r = 1; r < n_parts; r++) { acc += ld_act_f32(parts + (int64_t) r * n + i); }
        if (extra) { acc += ld_act_f32(extra + i); }
        out.put(i, acc);
    }
}

ExpertMat expert_mat(const bf16n_weight & w, float * y) { return {pair_view(w), (const AuxHeader *) w.aux, (char *) y}; }

uint32_t unit_cap(const bf16n_weight & w) { return (uint32_t) ((w.R * w.K * 3 / 8 + 64 + 15) & ~15ll); }

int g_plane_staged_warps_per_sm = 8; // stage the plane too while the launch has at most this many warps per SM

template <int C, int R, bool CM, typename TX, bool GLU_IN>
void launch_units(const ExpertMat & m0, const ExpertMat & m1, int n_mats, const ExpertCols & p, int ncols, cudaStream_t st) {
    const int64_t units = p.rows_per_expert / R;
    const int64_t all_warps = ncols * n_mats * units;
    // few tokens: small blocks so that the units of one column spread over many SMs
    const int warps = all_warps >= (int64_t) device_info().sms * 16 ? 8 : 4;
    // When the launch leaves most of an SM idle anyway, every warp also stages its unit's plane bytes, so that it waits
    // for memory once instead of once per chunk; with more warps per SM the shared memory is better spent on residency.
    const bool plane = all_warps <= (int64_t) device_info().sms * g_plane_staged_warps_per_sm;
    const dim3 grid((unsigned) ((units + warps - 1) / warps), (unsigned) ncols, (unsigned) n_mats);
    const size_t shm = 4 * HP_MAX_PAIRS + 128 + (size_t) warps * (p.cap_bytes + (plane ? R * C * CHUNK : 0));
    const Opaque k = {1u, 4u, ~0u, 32u};
    static bool attr_done = false; // set once per instantiation, during bf16n_init's warm-up call (before any capture)
    if (!attr_done) {
        cuda_ok(cudaFuncSetAttribute(k_expert_units<C, R, CM, TX, GLU_IN, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024),
                "k_expert_units attribute");
        cuda_ok(cudaFuncSetAttribute(k_expert_units<C, R, CM, TX, GLU_IN, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024),
                "k_expert_units attribute");
        attr_done = true;
    }
    if (ncols == 0) { return; }
    if (plane && shm <= 128 * 1024) {
        launch_chained(k_expert_units<C, R, CM, TX, GLU_IN, true>, grid, dim3(warps * 32), shm, st, m0, m1, p, k);
    } else {
        launch_chained(k_expert_units<C, R, CM, TX, GLU_IN, false>, grid, dim3(warps * 32), 4 * HP_MAX_PAIRS + 128 + (size_t) warps * p.cap_bytes, st,
                       m0, m1, p, k);
    }
    check_launch();
}

using bf16 = __nv_bfloat16;

bool gate_shape_ok(const bf16n_weight & w) {
    return w.format == FMT_HUFPAIR && !w.fo && w.cm && w.K == 2048 && w.R == 8;
}
bool down_shape_ok(const bf16n_weight & w) {
    return w.format == FMT_HUFPAIR && !w.fo && !w.cm && w.K == 512 && w.R == 16;
}

} // namespace

bool moe_decode_supported(const bf16n_weight & gate, const bf16n_weight & up, const bf16n_weight & down) {
    return gate_shape_ok(gate) && gate_shape_ok(up) && down_shape_ok(down) && gate.rows == up.rows;
}

BF16N_DEFINE_FAULT_WORD(moe_decode_fault_word)

void moe_decode_init() {
    // instantiate and set the shared-memory attribute of every variant outside of any stream capture
    ExpertMat none = {};
    ExpertCols p = {};
    p.rows_per_expert = 16; p.cap_bytes = 16;
    launch_units<4, 8, true, bf16, false>(none, none, 2, p, 0, nullptr);
    launch_units<4, 8, true, float, false>(none, none, 2, p, 0, nullptr);
    launch_units<1, 16, false, float, true>(none, none, 1, p, 0, nullptr);
    launch_units<1, 16, false, float, false>(none, none, 1, p, 0, nullptr);
    launch_units<1, 16, false, bf16, false>(none, none, 1, p, 0, nullptr);
}

// bf16n_mmv with expert ids on the expert shapes of the decode step takes the unit kernel too (one warp per unit, bulk-copy
// staged), so the reference's own operator chain (mmv gate, mmv up, swiglu, mmv down) gets it without calling the fused
// entry point. Results are bit-identical to the general routed kernels.
bool expert_units_applies(const bf16n_weight & w, const bf16n_mmv_args & a) {
    if (!a.ids || a.y_bf16 || !(gate_shape_ok(w) || down_shape_ok(w)) || a.n_used <= 0 || a.ncols % a.n_used) { return false; }
    const bool whole = a.row0 == 0 && a.nrows == a.rows_per_matrix && a.nrows > 0 && w.rows % a.rows_per_matrix == 0;
    const bool dense_y = a.y_slot == a.nrows * 4 && a.y_tok == (int64_t) a.n_used * a.nrows * 4;
    const bool x_ok = a.x_per_slot == 1 || a.x_per_slot == a.n_used;
    return whole && dense_y && x_ok && a.ncols <= 65535;
}

void expert_units_mmv(const bf16n_weight & w, const bf16n_mmv_args & a, cudaStream_t st) {
    ExpertCols p = {};
    p.x = (const char *) a.x; p.x_tok = a.x_tok; p.x_slot = a.x_per_slot == 1 ? 0 : a.x_slot;
    p.ids = (const char *) a.ids; p.ids_s0 = a.ids_s0; p.ids_s1 = a.ids_s1;
    p.n_used = a.n_used; p.rows_per_expert = a.rows_per_matrix; p.e_lo = 0; p.e_n = (int) (w.rows / a.rows_per_matrix);
    p.cap_bytes = unit_cap(w);
    const ExpertMat m = expert_mat(w, (float *) a.y);
    if (w.cm) {
        if (a.x_bf16) { launch_units<4, 8, true, bf16, false>(m, m, 1, p, a.ncols, st); }
        else { launch_units<4, 8, true, float, false>(m, m, 1, p, a.ncols, st); }
    } else {
        if (a.x_bf16) { launch_units<1, 16, false, bf16, false>(m, m, 1, p, a.ncols, st); }
        else { launch_units<1, 16, false, float, false>(m, m, 1, p, a.ncols, st); }
    }
}

// gate/up (chunk-major R = 8, K = 2048) -> silu(g) * u -> down (row-major R = 16, K = 512) -> weighted sum over slots.
// scratch: FP32 [2 * n_tok * n_used * N + n_tok * n_used * H] (N, H = rows per expert of gate and down).
void moe_decode(const bf16n_weight & gate, const bf16n_weight & up, const bf16n_weight & down, const void * x, bool x_bf16,
                int64_t x_tok, const int32_t * ids, const float * weights, int n_tok, int n_used, int n_experts_local, int e_lo,
                float * scratch, void * y, bool y_bf16, cudaStream_t st, const bf16n_peer_out * peers) {
    const int64_t N = gate.rows / n_experts_local, H = down.rows / n_experts_local;
    const int ncols = n_tok * n_used;
    float * g = scratch, * u = g + (int64_t) ncols * N, * ys = u + (int64_t) ncols * N;
    ExpertCols p = {};
    p.x = (const char *) x; p.x_tok = x_tok; p.x_slot = 0;
    p.ids = (const char *) ids; p.ids_s0 = 4; p.ids_s1 = 4ll * n_used;
    p.n_used = n_used; p.rows_per_expert = N; p.e_lo = e_lo; p.e_n = n_experts_local;
    p.cap_bytes = unit_cap(gate);
    if (x_bf16) {
        launch_units<4, 8, true, bf16, false>(expert_mat(gate, g), expert_mat(up, u), 2, p, ncols, st);
    } else {
        launch_units<4, 8, true, float, false>(expert_mat(gate, g), expert_mat(up, u), 2, p, ncols, st);
    }
    ExpertCols q = p;
    q.x = (const char *) g; q.x2 = u; q.x_tok = 4ll * n_used * N; q.x_slot = 4ll * N;
    q.rows_per_expert = H; q.cap_bytes = unit_cap(down);
    q.early_ids = true; // the ids precede the gate / up launch, whose outputs are the only thing this launch waits for
    launch_units<1, 16, false, float, true>(expert_mat(down, ys), expert_mat(down, ys), 1, q, ncols, st);
    const dim3 grid((unsigned) std::min<int64_t>((H + 255) / 256, 64), (unsigned) n_tok);
    launch_chained(k_combine_f32, grid, dim3(256), 0, st, ys, weights, (char *) y, y_bf16, n_used, H, make_peer_out(peers));
}

// The same step over fragment-order experts (the layout the vLLM policy gives expert stacks): routed products through the
// fragment-order GEMV (one decode per (token, slot) column, a band's slabs on separate warps), SwiGLU in place, the
// slot-order combine. All experts on this GPU (no expert slice). Same scratch layout as moe_decode.
void moe_decode_frag_order(const bf16n_weight & gate, const bf16n_weight & up, const bf16n_weight & down, const void * x, bool x_bf16,
                           int64_t x_tok, const int32_t * ids, const float * weights, int n_tok, int n_used, int n_experts,
                           float * scratch, void * y, bool y_bf16, cudaStream_t st) {
    const int64_t N = gate.rows / n_experts, H = down.rows / n_experts;
    const int ncols = n_tok * n_used;
    float * g = scratch, * u = g + (int64_t) ncols * N, * ys = u + (int64_t) ncols * N;
    bf16n_mmv_args a = {};
    a.x = x; a.x_bf16 = x_bf16; a.y_bf16 = 0; a.ncols = ncols; a.n_used = n_used; a.x_per_slot = 1;
    a.x_tok = x_tok; a.x_slot = 0;
    a.ids = ids; a.ids_s0 = 4; a.ids_s1 = 4ll * n_used;
    a.rows_per_matrix = N; a.row0 = 0; a.nrows = N;
    a.y_tok = 4ll * n_used * N; a.y_slot = 4ll * N;
    a.y = g; fo_gemv(gate, a, st);
    a.y = u; fo_gemv(up, a, st);
    moe_swiglu(g, u, g, (int64_t) ncols * N, st);            // g := silu(g) * u
    bf16n_mmv_args d = a;
    d.x = g; d.x_bf16 = 0; d.x_per_slot = n_used; d.x_tok = 4ll * n_used * N; d.x_slot = 4ll * N;
    d.rows_per_matrix = H; d.nrows = H; d.y = ys; d.y_tok = 4ll * n_used * H; d.y_slot = 4ll * H;
    fo_gemv(down, d, st);
    const dim3 grid((unsigned) std::min<int64_t>((H + 255) / 256, 64), (unsigned) n_tok);
    launch_chained(k_combine_f32, grid, dim3(256), 0, st, ys, weights, (char *) y, y_bf16, n_used, H, PeerOut{});
    check_launch();
}

void peer_sum(const float * parts, int n_parts, int64_t n, const float * extra, void * y, bool y_bf16, cudaStream_t st) {
    const unsigned blocks = (unsigned) std::min<int64_t>((n + 255) / 256, 256);
    launch_chained(k_peer_sum, dim3(blocks), dim3(256), 0, st, parts, n_parts, n, extra, (char *) y, y_bf16);
    check_launch();
}


// ---------------------------------------------------------------- the same step without caller-provided scratch

// Some callers are not allowed to allocate device memory at the point where they run a decode step: an engine that
// handed out all of its device memory to a fixed arena when the model was loaded, or a decode loop that must not reach
// cudaMalloc because an allocation synchronises the whole device. For them the intermediate buffers of the step (gate
// and up outputs and the per-slot down outputs, FP32) live in this array, which is part of the library image: every
// GPU that loads the library holds these 768 KB until the process exits.
constexpr size_t STATIC_SCRATCH_FLOATS = (size_t) BF16N_MOE_DECODE_STATIC_MAX_FLOATS;
static __device__ __align__(256) float g_static_scratch[STATIC_SCRATCH_FLOATS];

namespace {

// Device address of g_static_scratch on the current device. In host code the array's name is only a handle, not a
// pointer a kernel could use, so the address is asked for once per device (with that device current) and remembered.
float * static_scratch_of_current_device() {
    constexpr int MAX_DEVICES = 64;
    static std::mutex lock;
    static float * address[MAX_DEVICES] = {};
    int dev = 0;
    cuda_ok(cudaGetDevice(&dev), "cudaGetDevice");
    require(dev >= 0 && dev < MAX_DEVICES, "moe_decode_static: device index out of range");
    std::lock_guard<std::mutex> guard(lock);
    if (!address[dev]) {
        float * p = nullptr;
        cuda_ok(cudaGetSymbolAddress((void **) &p, g_static_scratch), "cudaGetSymbolAddress(static MoE scratch)");
        address[dev] = p;
    }
    return address[dev];
}

} // namespace

size_t moe_decode_static_capacity_floats() { return STATIC_SCRATCH_FLOATS; }

// moe_decode with the library's own scratch. Nothing in the array has to start at zero: the gate/up launch writes every
// element the down launch reads (zeros for slots of other ranks' experts) and the down launch every element the
// combine reads, so whatever an earlier call left behind is overwritten before it is used.
void moe_decode_static(const bf16n_weight & gate, const bf16n_weight & up, const bf16n_weight & down, const void * x, bool x_bf16,
                       int64_t x_tok, const int32_t * ids, const float * weights, int n_tok, int n_used, int n_experts_local,
                       int e_lo, void * y, bool y_bf16, cudaStream_t st) {
    moe_decode(gate, up, down, x, x_bf16, x_tok, ids, weights, n_tok, n_used, n_experts_local, e_lo,
               static_scratch_of_current_device(), y, y_bf16, st);
}

} // namespace b16
