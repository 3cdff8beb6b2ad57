// Large-matrix decode+GEMV for BF16 activations (the vocabulary projection): per-lane shared-memory rings, activations
// in tensor memory.
//
// Decoding a lane stream is a serial chain (table lookup -> code length -> next lookup) of about 16 instructions per
// pair of weights. The kernel is bound by the shared-memory pipe (a random 4-byte lookup in the table costs three to
// four bank-conflict wavefronts) and by instruction issue, not by HBM. What helps is many independent chains per SM,
// few registers per chain, and everything that is not a table lookup kept off the shared-memory pipe:
//   * one unit per warp and up to 28 warps per block (72 registers per thread);
//   * the activations a lane multiplies with are the same for every row, so they sit in tensor memory (tcgen05.st once,
//     tcgen05.ld of four words per half chunk into two register sets in turn): TMEM is read through its own pipe, which
//     this kernel otherwise leaves idle, and the reads cost the shared-memory pipe nothing;
//   * four copies of the code table, interleaved word by word (entry i of copy r at word 4 i + r; lane l reads copy
//     l % 4): only the eight lanes that share a copy can collide on a bank;
//   * a chain's stream footprint is a 128-byte ring per lane (4 KB per warp) filled with cp.async 16-byte granules,
//     topped up at every row start to more than 96 bytes ahead of the read pointer; a row consumes at most 48 bytes
//     (32 codes of up to 12 bits) and everything copied before the previous row start has landed (wait_group 0 at the
//     row start, a row of work after the copies were issued), so the words a row reads are always complete;
//   * the ring is read as a window of three consecutive words and a bit offset: one funnel shift per view of the
//     stream, no shift of the window per code, and a refill is two register moves and one load;
//   * ring addressing: byte offset from the unit's 16-byte aligned start, modulo 128, XOR a per-lane constant that also
//     carries the lane's ring base: one logic op per address;
//   * 2 or 4 dense columns share one decode (each column's activations in its own TMEM columns, four accumulators per
//     column), bitwise equal to the single-column results;
//   * the same summation order as every other kernel of the format (four accumulators per lane by column mod 4,
//     (a0 + a1) + (a2 + a3), xor butterfly), FP32 fma of exact BF16 products.
#include "launch.h"
#include "rings.cuh"


namespace b16 {
namespace {

using namespace dev;
using namespace ring;
using bf16 = __nv_bfloat16;

// Tensor memory as a per-lane register file extension: lane l of a warp reads columns [col, col + 4) of TMEM lane
// 32 * (warp % 4) + l.
__device__ __forceinline__ void tmem_alloc(uint32_t slot, uint32_t cols) { // cols: a power of two, 32..512
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_free(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_st4(uint32_t addr, const uint4 & v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld4(uint32_t addr, uint4 & v) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
}
// the loaded registers are operands of the wait, so no use of them can be scheduled above it
__device__ __forceinline__ void tmem_ld_wait(uint4 & v) {
    asm volatile("tcgen05.wait::ld.sync.aligned;" : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w) :: "memory");
}
__device__ __forceinline__ void tmem_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void fma_bf16x2(uint32_t w, uint32_t x, float & lo, float & hi) {
    asm("{ .reg .b16 wl, wh, xl, xh;\n\t"
        "mov.b32 {wl, wh}, %2;\n\t"
        "mov.b32 {xl, xh}, %3;\n\t"
        "fma.rn.f32.bf16 %0, wl, xl, %0;\n\t"
        "fma.rn.f32.bf16 %1, wh, xh, %1; }"
        : "+f"(lo), "+f"(hi) : "r"(w), "r"(x));
}

// Measured alternatives that lost (248320 x 2048, one column, 174 us as built): activations widened to FP32 in tensor
// memory with plain fma 183 us (three more instructions per pair of weights); 32 warps of 64 registers 192 us; plane
// bytes prefetched two chunks ahead instead of a row 179 us; activations read from shared memory 184 us; one table 178 us.
__host__ __device__ constexpr int tmem_cols(int C, int NC) { // per lane: 8 C words of BF16 pairs per column, rounded up to a power of two >= 32
    int need = NC * C * 8, cols = 32;
    while (cols < need) { cols *= 2; }
    return cols;
}

// One unit per warp. NC dense columns share the decode (NC = 1 also serves routed columns: blockIdx.y picks the column).
template <int C, int NT, int NC, bool PEERS = false> // PEERS: the output also goes to the other GPUs (a separate instantiation: the plain kernel carries none of it)
__global__ void __launch_bounds__(NT, 1) k_pair_gemv_rings(const PairView w, int R, Cols p, const Opaque k) {
    constexpr int K = C * CHUNK;
    constexpr int XW = C * 8;           // TMEM words per column and lane
    constexpr int STEPS = 2 * C * NC;   // four-word TMEM loads per row: one per (half chunk, column)
    constexpr uint32_t TCOLS = tmem_cols(C, NC);
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ uint32_t tmem_slot;
    uint32_t * lut = (uint32_t *) smem; // four interleaved tables | NC x K BF16 activations | one 4 KB ring set per warp
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    const uint32_t lut_s = smem_u32(lut);
    const uint32_t lut_l = lut_s + (lane & 3) * 4;
    const uint32_t xs = lut_s + LUT_BYTES + lane * 16;
    // ring of lane l: 128 bytes at l * 128; granule index XOR (l & 7) spreads lanes that read in step over the banks
    const uint32_t key = (lut_s + LUT_BYTES + NC * 2 * K + (uint32_t) warp * (32 * RING_BYTES) + lane * RING_BYTES) | ((lane & 7) << 4);

    const bf16 * xg; OutVec out; int64_t rbase;
    column<bf16>(p, NC == 1 ? blockIdx.y : 0, xg, out, rbase);
    if (PEERS) { peers_begin(p.peers); }
    if (warp == 0) { tmem_alloc(smem_u32(&tmem_slot), TCOLS); }
    for (int i = threadIdx.x; i < HP_MAX_PAIRS; i += blockDim.x) { const uint32_t e = __ldg(w.lut + i); ((uint4 *) lut)[i] = make_uint4(e, e, e, e); }
    // 16 bytes per (column n, chunk c, half h, lane l): the lane's activations of column quads 2h and 2h+1 of the chunk
    for (int i = threadIdx.x; i < NC * (K / 4); i += blockDim.x) {
        const int n = i / (K / 4), r = i - n * (K / 4);
        const int c = r >> 7, j = (r >> 5) & 3, l = r & 31; // quad j of chunk c, lane l: columns c*512 + 128*j + 4*l + {0..3}
        const uint2 v = __ldg((const uint2 *) ((const char *) xg + n * p.x_tok) + (c * CHUNK + 128 * j + 4 * l) / 4);
        *(uint2 *) (smem + LUT_BYTES + n * 2 * K + ((c * 2 + (j >> 1)) * 32 + l) * 16 + (j & 1) * 8) = v;
    }
    tmem_fence_before();
    __syncthreads();
    tmem_fence_after();
    // activations into tensor memory: warps 0..3 fill the four lane quarters (a warp reads the quarter warp % 4)
    const uint32_t tmem_base = tmem_slot;
    const uint32_t tmem_x = tmem_base + ((uint32_t) (warp & 3) << 21); // lane field (bits 16 and up): 32 * (warp % 4)
    if (warp < 4) {
#pragma unroll
        for (int i = 0; i < NC * 2 * C; i++) {
            tmem_st4(tmem_x + 4 * i, lds128_ro(xs + i * 512));
        }
        tmem_st_wait();
    }
    tmem_fence_before();
    __syncthreads();
    tmem_fence_after();

    // step s of a row = (half chunk, column n): its four words are at TMEM column n * XW + 4 * (half chunk index)
    auto x_addr = [&](int s) { return tmem_x + (s % NC) * XW + 4 * (s / NC); };
    uint4 xa, xb = make_uint4(0, 0, 0, 0);
    tmem_ld4(x_addr(0), xa);

    const int64_t units = p.nrows / R;
    // warp w of block b takes units w * blocks + b, + blocks * warps, ...: a matrix with few units still reaches every SM
    for (int64_t u = (int64_t) warp * gridDim.x + blockIdx.x; u < units; u += (int64_t) gridDim.x * nwarp) {
        const int64_t g = rbase / R + u;
        RingReader rd;
        {
            const uint32_t w0 = __ldg(w.ubase + g), l0 = __ldg(w.lrel + g * 32 + lane);
            rd.open((const uint8_t *) (w.stream + (w0 & ~3u)), ((w0 & 3u) + l0) * 4u, key, k);
        }
        cp_async_commit();
        const uint8_t * pl = w.plane + g * R * K + 16 * lane;
        uint4 nx[C]; // plane bytes one row ahead of the decode
#pragma unroll
        for (int c = 0; c < C; c++) { nx[c] = ld_stream16(pl + c * CHUNK); }
        rd.token = cp_async_wait_all();
        rd.first_words();
        float mine[NC];
#pragma unroll
        for (int n = 0; n < NC; n++) { mine[n] = 0.f; }
        for (int rr = 0; rr < R; rr++) {
            if (rr) {
                rd.token = cp_async_wait_all(); // copies issued one row ago
                rd.template top_up<3>(k);
                cp_async_commit();
            }
            float a[NC][4];
#pragma unroll
            for (int n = 0; n < NC; n++) { a[n][0] = a[n][1] = a[n][2] = a[n][3] = 0.f; }
            const uint8_t * nrow = pl + (rr + 1 < R ? rr + 1 : rr) * K;
#pragma unroll
            for (int c = 0; c < C; c++) {
                const uint4 sm = nx[c];
                nx[c] = ld_stream16(nrow + c * CHUNK); // the last row re-reads itself: one harmless L2 hit per chunk
                const uint32_t pw[4] = {sm.x, sm.y, sm.z, sm.w};
#pragma unroll
                for (int half = 0; half < 2; half++) {
                    uint32_t e[4];
                    rd.take2(lut_l, k, e[0], e[1]);
                    rd.take2(lut_l, k, e[2], e[3]);
                    uint32_t wv[4]; // BF16 pairs: columns {0, 1} and {2, 3} of quads 2 half and 2 half + 1
#pragma unroll
                    for (int jj = 0; jj < 2; jj++) {
                        wv[2 * jj] = merge_sm_exp(spread_lo(pw[2 * half + jj]), e[2 * jj]);
                        wv[2 * jj + 1] = merge_sm_exp(spread_hi(pw[2 * half + jj]), e[2 * jj + 1]);
                    }
#pragma unroll
                    for (int n = 0; n < NC; n++) { // two register sets in turn: wait for this step's, start the next step's load, use this one
                        const int s = (c * 2 + half) * NC + n;
                        uint4 & cur = (s & 1) ? xb : xa;
                        uint4 & nxt = (s & 1) ? xa : xb;
                        tmem_ld_wait(cur);
                        tmem_ld4(x_addr((s + 1) % STEPS), nxt);
                        fma_bf16x2(wv[0], cur.x, a[n][0], a[n][1]);
                        fma_bf16x2(wv[1], cur.y, a[n][2], a[n][3]);
                        fma_bf16x2(wv[2], cur.z, a[n][0], a[n][1]);
                        fma_bf16x2(wv[3], cur.w, a[n][2], a[n][3]);
                    }
                }
            }
#pragma unroll
            for (int n = 0; n < NC; n++) {
                const float s = warp_sum((a[n][0] + a[n][1]) + (a[n][2] + a[n][3]));
                if (lane == rr) { mine[n] = s; }
            }
        }
        if (lane < R) {
#pragma unroll
            for (int n = 0; n < NC; n++) {
                const OutVec o = {out.p + n * p.y_tok, out.bf16};
                o.put(u * R + lane, mine[n]);
                if (PEERS) { peers_put(p, (NC == 1 ? (int) blockIdx.y : 0) + n, u * R + lane, mine[n]); }
            }
        }
    }
    tmem_ld_wait(xa);
    tmem_fence_before();
    __syncthreads();
    if (warp == 0) { tmem_free(tmem_base, TCOLS); }
    if (PEERS) { peers_done(p); }
}

constexpr int RING_SET = 32 * RING_BYTES;
int fixed_smem(int64_t K, int nc) { return LUT_BYTES + nc * 2 * (int) K; }

} // namespace

constexpr int g_warps = 28; // most warps per block (72 registers per thread)

// (chunks, threads per block the register budget is set for, columns per decode)
#define RINGS_FOR_EACH(X) X(1, 896, 1) X(2, 896, 1) X(4, 896, 1) X(4, 768, 1) X(4, 768, 2) X(4, 640, 4) X(2, 768, 2) X(2, 640, 4) X(1, 768, 2) X(1, 640, 4)

void gemv_rings_init() {
    const int optin = device_info().smem_optin;
#define ATTR(CC, NT, NC) allow_dynamic_smem((const void *) k_pair_gemv_rings<CC, NT, NC>, optin, optin, "rings"); \
                         allow_dynamic_smem((const void *) k_pair_gemv_rings<CC, NT, NC, true>, optin, optin, "rings");
    RINGS_FOR_EACH(ATTR)
#undef ATTR
}

bool gemv_rings_enabled() { return g_warps > 0; }

// Row-major HUFPAIR, BF16 activations, K <= 2048, enough units to give every SM a full set of chains
bool gemv_rings_applies(const bf16n_weight & w, const bf16n_mmv_args & a) {
    const int64_t C = w.K / CHUNK;
    if (w.format != FMT_HUFPAIR || w.cm || w.fo || !(C == 1 || C == 2 || C == 4) || a.nrows <= 0 || !a.x_bf16) { return false; }
    const int groups = a.ids ? a.ncols : (a.ncols + 3) / 4; // dense columns share a decode four at a time
    // Several dense columns over a mid-size matrix (from 12 M weights and one unit per SM on): sharing the decode among
    // up to four columns beats one staged decode per column (8192 x 2048, R = 16: 33 / 64 us at 4 / 8 tokens against
    // 51 / 78; 16384 x 2048: 37 / 73 against 65 / 121), while a single column is faster there with the staged kernel's
    // short prologue (23 against 30 us) and 4096 x 2048 is level.
    if (!a.ids && a.ncols >= 2 && a.nrows * w.K >= (12ll << 20)) { return a.nrows / w.R >= (int64_t) device_info().sms; }
    return a.nrows / w.R >= (int64_t) device_info().sms * 16 * std::max(1, groups);
}

namespace {

// nc dense columns starting at p.x / p.y (nc = 1: also `ncols_grid` routed or dense columns, one decode each)
void launch_rings(const bf16n_weight & w, const Cols & p, int nc, int ncols_grid, cudaStream_t st) {
    const int64_t units = p.nrows / w.R, sms = device_info().sms;
    const int cap = nc == 1 ? (w.K == 2048 ? g_warps : std::min(g_warps, 28)) : nc == 2 ? std::min(g_warps, 24) : std::min(g_warps, 20);
    const int max_warps = std::max(4, cap);
    int best = max_warps;
    double best_eff = 0.0;
    if (units <= sms * max_warps) { // one round: as many warps as there are units per SM (four fill the tensor-memory quarters)
        best = (int) std::max<int64_t>(4, (units + sms - 1) / sms);
        best_eff = 1.0;
    }
    for (int nw = max_warps; best_eff < 1.0 && nw >= std::max(4, max_warps - 3); nw--) { // static round-robin: waste least of the last round
        const int64_t slots = sms * nw, rounds = (units + slots - 1) / slots;
        const double eff = (double) units / (double) (rounds * slots) * (1.0 - 0.01 * (max_warps - nw));
        if (eff > best_eff + 1e-9) { best_eff = eff; best = nw; }
    }
    const dim3 grid((unsigned) sms, (unsigned) ncols_grid);
    const size_t shm = fixed_smem(w.K, nc) + (size_t) best * RING_SET;
    const Opaque k = {1u, 4u, ~0u, 32u, 16u};
    const PairView v = pair_view(w);
#define GO(CC, NT, NC) if (p.peers.n) { k_pair_gemv_rings<CC, NT, NC, true><<<grid, best * 32, shm, st>>>(v, w.R, p, k); } \
                       else { k_pair_gemv_rings<CC, NT, NC, false><<<grid, best * 32, shm, st>>>(v, w.R, p, k); }
    const int C = (int) (w.K / CHUNK);
    if (nc == 4) { switch (C) { case 1: GO(1, 640, 4); break; case 2: GO(2, 640, 4); break; default: GO(4, 640, 4); break; } }
    else if (nc == 2) { switch (C) { case 1: GO(1, 768, 2); break; case 2: GO(2, 768, 2); break; default: GO(4, 768, 2); break; } }
    else if (C == 4 && best <= 24) { GO(4, 768, 1); }
    else { switch (C) { case 1: GO(1, 896, 1); break; case 2: GO(2, 896, 1); break; default: GO(4, 896, 1); break; } }
#undef GO
    check_launch();
}

} // namespace

void gemv_rings(const bf16n_weight & w, const bf16n_mmv_args & a, cudaStream_t st, bool multi_col, const bf16n_peer_out * peers) {
    const Cols p = make_cols(a, peers);
    if (a.ids || a.ncols == 1 || !multi_col || (peers && peers->n_peers > 0)) { // one decode per column
        launch_rings(w, p, 1, a.ncols, st);
        return;
    }
    for (int c0 = 0; c0 < a.ncols;) { // dense columns: four, two or one per decode
        const int left = a.ncols - c0, nc = left >= 4 ? 4 : left >= 2 ? 2 : 1;
        Cols q = p;
        q.x += c0 * p.x_tok;
        q.y += c0 * p.y_tok;
        launch_rings(w, q, nc, 1, st);
        c0 += nc;
    }
}

} // namespace b16
