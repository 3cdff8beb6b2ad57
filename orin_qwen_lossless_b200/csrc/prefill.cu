// Batched (prefill) routed product on the 5th-generation tensor cores: dst[t, slot, :] = W_e x_t for every routed
// (token, slot) pair, optionally fused gate/up + SwiGLU. Replaces the reference's persistent mma.sync kernel
// (core/include/bf16n/kernels.cuh:1162-1505) with a warp-specialised tcgen05 / TMEM design.
//
// One persistent block per SM walks work items (expert, block of weight rows, pass of up to G x 128 of the expert's
// tokens). Its 20 warps have three roles that run concurrently and meet only through mbarriers:
//
//   * 16 decoder warps. Each owns one unit of the item (SwiGLU: 8 gate units + the 8 matching up units) and walks its
//     exponent streams once, four rows at a time: a "weight tile" is 64 weight rows (4 per decoder warp) x one 512-column
//     chunk, written straight into shared memory in the canonical K-major 128-byte-swizzled operand layout (8 k-tiles of
//     64 rows x 64 columns; a lane's 4 consecutive weights are one 8-byte store: the lane-major plane maps lanes 0..15 /
//     16..31 of column quad j to k-tiles 2j / 2j+1). Two weight tiles alternate, so decoding runs up to two tiles ahead
//     of the tensor core. The bit-stream state stays in registers across chunks, which is what chunk-major units are for.
//   * 3 gather warps. They copy the routed activation rows of the pass (cp.async, 16-byte pieces, a full 128-byte line
//     per 8 threads) into a ring of 128-token x 64-column operand slots; each slot's mbarrier completes when the
//     copies of all gather threads have landed (cp.async.mbarrier.arrive), so the threads never wait for their copies.
//   * 1 MMA warp. One thread waits for a slot and (at each tile's first k-tile) for the weight tile, then issues four
//     tcgen05.mma (M = 128 tokens, N = 64 weight rows, K = 16) that accumulate D[token, weight row] in TMEM;
//     tcgen05.commit releases the slot and the weight tile to their producers and announces the finished accumulators.
//
// After the last chunk of a pass the four non-decoder warps read the accumulators back (tcgen05.ld: warp w reads TMEM
// lanes 32w..32w+31 = tokens) and scatter them through ids_dst. A thread holds gate and up of the same (token, row), so
// SwiGLU needs no exchange. Activations are the M operand, so an expert with few tokens costs no extra decoding and one
// with many is decoded once per G x 128 tokens; experts without tokens are skipped.
// Every wait is bounded. A wait that expires sets a block-wide flag; from then on every role runs through the rest of
// its loops without waiting, multiplying or decoding, so that all barriers still see all their threads; the block then
// lets the tensor core drain, records the fault, frees its TMEM and returns. No cluster launch, no multicast.
#include "decode.cuh"
#include "launch.h"

namespace b16 {
namespace {

using namespace dev;
using bf16 = __nv_bfloat16;

__device__ unsigned int g_prefill_fault; // a bounded wait expired (bf16n_fault_status reads and clears it)

constexpr int DEC_WARPS = 16, GATHER_WARPS = 3, GATHERERS = GATHER_WARPS * 32;
constexpr int MMA_WARP = DEC_WARPS + GATHER_WARPS;   // the last warp
constexpr int HELPERS = (GATHER_WARPS + 1) * 32;     // the epilogue is done by the gather warps and the MMA warp
constexpr int NTHREADS = DEC_WARPS * 32 + HELPERS;
constexpr int SUB = 4;                           // rows a decoder warp adds to a weight tile
constexpr int N_TILE = DEC_WARPS * SUB;          // weight rows per tile = N of the MMA
constexpr int M_TOK = 128;                       // tokens per group = M of the MMA
constexpr int W_KTILE_BYTES = N_TILE * 128;      // 64 rows x 64 columns of BF16
constexpr int W_TILE_BYTES = 8 * W_KTILE_BYTES;  // one 512-column chunk
constexpr int X_SLOT_BYTES = M_TOK * 128;        // 128 tokens x 64 columns
constexpr int TMEM_COLS = 512;
constexpr uint32_t POLL_LIMIT = 1u << 20;
static_assert(HELPERS == 128, "four warps read the 128 TMEM lanes");

__device__ __forceinline__ uint32_t smem_u32(const void * p) { return (uint32_t) __cvta_generic_to_shared(p); }

// ---- mbarrier / tcgen05 wrappers
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("{ .reg .b64 st; mbarrier.arrive.shared::cta.b64 st, [%0]; }" ::"r"(bar) : "memory");
}
// bounded wait: gives up after POLL_LIMIT probes or two seconds, whichever comes first
__device__ __forceinline__ bool mbar_poll(uint32_t bar, uint32_t parity) {
    uint64_t t0 = 0;
    for (uint32_t i = 0; i < POLL_LIMIT; i++) {
        uint32_t done;
        asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) { return true; }
        if ((i & 255u) == 255u) {
            uint64_t now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (t0 == 0) { t0 = now; } else if (now - t0 > 2000000000ull) { return false; }
        }
    }
    return false;
}
// the wait every role uses: nothing is waited for once the block has failed, and an expired wait fails the block
__device__ __forceinline__ void wait_on(uint64_t * bar, uint32_t parity, volatile int * failed) {
    if (*failed) { return; }
    if (!mbar_poll(smem_u32(bar), parity)) { *failed = 1; }
}
__device__ __forceinline__ void tmem_alloc(uint32_t slot, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_free(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t * bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void proxy_fence() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void helper_bar() { asm volatile("bar.sync 1, %0;" ::"n"(HELPERS) : "memory"); }
__device__ __forceinline__ void tmem_ld32(uint32_t addr, uint32_t (&v)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,"
                 "%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                   "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
                   "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
                   "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                 : "r"(addr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void * src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
// asynchronous arrival on an mbarrier, triggered when all earlier cp.async of this thread are complete; the arrival is
// one of the count the barrier was initialised with
__device__ __forceinline__ void cp_async_arrive(uint64_t * bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// asks the L2 cache for `bytes` (a multiple of 16) at a 16-byte aligned address; nothing waits for it
__device__ __forceinline__ void bulk_prefetch_l2(const void * src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// shared-memory matrix descriptor of a K-major, 128-byte-swizzled tile: rows 128 bytes apart, 8-row groups 1024 bytes
// apart (stride byte offset), descriptor version 1, layout type 2; `addr` may point 32*k bytes into the first row
__device__ __forceinline__ uint64_t tile_desc(uint32_t addr) {
    return (uint64_t) ((addr >> 4) & 0x3FFFu) | (uint64_t) 1 << 16 | (uint64_t) (1024 >> 4) << 32 | (uint64_t) 1 << 46 | (uint64_t) 2 << 61;
}
// kind::f16 instruction descriptor: FP32 accumulate, BF16 A and B, both K-major, N = 64, M = 128 or 64. With M = 64 the
// accumulator row m lives in TMEM lane 32 * (m / 16) + m % 16 (measured: the other lanes are not written).
__host__ __device__ constexpr uint32_t instr_desc(int m) {
    return 1u << 4 | 1u << 7 | 1u << 10 | (uint32_t) (N_TILE >> 3) << 17 | (uint32_t) (m >> 4) << 24;
}

struct PrefillArgs {
    PairView w0, w1;                    // w1: the up matrix (GLU)
    const bf16 * x; int64_t x_row;      // activations: row ids_src1[j] * x_row
    const int32_t * ids_src1; const int32_t * ids_dst; const int32_t * bounds;
    char * dst; int64_t dst_col; bool dst_bf16;
    bool vec_ok;                        // dst rows allow 4-element vector stores
    int n_experts;
    int64_t rows_per_expert;
};

// four consecutive output elements of one (token, slot) row
__device__ __forceinline__ void store4(char * dst, bool dst_bf16, bool vec_ok, int64_t at, float a, float b, float c, float d) {
    if (dst_bf16) {
        bf16 * o = (bf16 *) dst + at;
        if (vec_ok) {
            const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
            *(uint2 *) o = make_uint2(*(const uint32_t *) &lo, *(const uint32_t *) &hi);
        } else {
            o[0] = __float2bfloat16_rn(a); o[1] = __float2bfloat16_rn(b); o[2] = __float2bfloat16_rn(c); o[3] = __float2bfloat16_rn(d);
        }
    } else {
        float * o = (float *) dst + at;
        if (vec_ok) { *(float4 *) o = make_float4(a, b, c, d); }
        else { o[0] = a; o[1] = b; o[2] = c; o[3] = d; }
    }
}
__device__ __forceinline__ void store4(const PrefillArgs & p, int64_t at, float a, float b, float c, float d) {
    store4(p.dst, p.dst_bf16, p.vec_ok, at, a, b, c, d);
}

// C chunks per row, R rows per unit, CM chunk-major units, GLU fused gate/up + SwiGLU, G token groups of 128 per pass,
// SLOTS activation operand slots in the ring
template <int C, int R, bool CM, bool GLU, int G, int SLOTS>
__global__ void __launch_bounds__(NTHREADS, 1) k_prefill(const PrefillArgs p) {
    static_assert(CM || C == 1, "row-major units are walked in row order: one chunk per row only");
    static_assert(R % SUB == 0, "unit rows are split into groups of SUB");
    constexpr int K = C * CHUNK;
    constexpr int Q = R / SUB;                                 // weight tiles per chunk
    constexpr int TILES = C * Q;                               // weight tiles per pass
    constexpr int UNITS_PER_MAT = GLU ? DEC_WARPS / 2 : DEC_WARPS;
    constexpr int ROWS_OUT = UNITS_PER_MAT * R;                // output rows per item
    static_assert(G * Q * N_TILE <= TMEM_COLS, "accumulators of a pass must fit TMEM");
    extern __shared__ unsigned char smem_raw[];
    unsigned char * smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u); // operand tiles need 1024-byte alignment
    unsigned char * wbuf = smem;                                     // 2 weight tiles
    unsigned char * xbuf = wbuf + 2 * W_TILE_BYTES;                  // SLOTS activation slots
    uint32_t * lut0 = (uint32_t *) (xbuf + SLOTS * X_SLOT_BYTES);
    uint32_t * lut1 = lut0 + (GLU ? HP_MAX_PAIRS : 0);
    uint64_t * bars = (uint64_t *) (lut1 + HP_MAX_PAIRS);
    uint64_t * w_full = bars, * w_empty = bars + 2, * x_full = bars + 4, * x_free = x_full + SLOTS;
    uint64_t * acc_done = x_free + SLOTS, * drained = acc_done + 1;
    uint32_t * tmem_slot = (uint32_t *) (drained + 1);
    volatile int * failed = (volatile int *) (tmem_slot + 1);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int i = tid; i < HP_MAX_PAIRS / 4; i += NTHREADS) {
        ((uint4 *) lut0)[i] = __ldg((const uint4 *) p.w0.lut + i);
        if (GLU) { ((uint4 *) lut1)[i] = __ldg((const uint4 *) p.w1.lut + i); }
    }
    if (tid == 0) {
        for (int i = 0; i < 2; i++) { mbar_init(smem_u32(w_full + i), DEC_WARPS); mbar_init(smem_u32(w_empty + i), 1); }
        for (int i = 0; i < SLOTS; i++) { mbar_init(smem_u32(x_full + i), GATHERERS); mbar_init(smem_u32(x_free + i), 1); }
        mbar_init(smem_u32(acc_done), 1);
        mbar_init(smem_u32(drained), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        *failed = 0;
    }
    if (warp == 0) { tmem_alloc(smem_u32(tmem_slot), TMEM_COLS); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    const int m_blocks = (int) (p.rows_per_expert / ROWS_OUT);
    const int64_t units_per_expert = p.rows_per_expert / R;
    const int n_items = p.n_experts * m_blocks;

    if (warp < DEC_WARPS) {
        // ------------------------------------------------------------------ decoders
        const bool second = GLU && warp >= DEC_WARPS / 2;                // up half
        const PairView & wv = second ? p.w1 : p.w0;
        const uint32_t * lut = second ? lut1 : lut0;
        const int uw = second ? warp - DEC_WARPS / 2 : warp;             // unit inside this item's row block
        const int n_row0 = GLU ? (second ? N_TILE / 2 : 0) + uw * SUB : warp * SUB; // first of this warp's rows in a weight tile
        const uint32_t lane_part = (uint32_t) (lane >> 4) * W_KTILE_BYTES + (uint32_t) (lane & 1) * 8;
        const uint32_t piece = (uint32_t) (lane & 15) >> 1;
        uint32_t n = 0;                                                  // weight tiles produced
        for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
            const int e = item / m_blocks, mb = item - e * m_blocks;
            const int j0 = p.bounds[e], j1 = p.bounds[e + 1];
            const int64_t gu = (int64_t) e * units_per_expert + (int64_t) mb * UNITS_PER_MAT + uw;
            // the unit this warp decodes next: its plane and streams are requested into L2 now, a whole item ahead, so that
            // the short read-ahead of the stream reader only has to cover L2 latency
            int64_t gun = -1;
            uint32_t ns0 = 0, ns1 = 0;
            if (j1 > j0 && item + (int) gridDim.x < n_items) {
                const int e2 = (item + (int) gridDim.x) / m_blocks, mb2 = item + (int) gridDim.x - e2 * m_blocks;
                if (p.bounds[e2 + 1] > p.bounds[e2]) {
                    gun = (int64_t) e2 * units_per_expert + (int64_t) mb2 * UNITS_PER_MAT + uw;
                    if (lane == 0) { bulk_prefetch_l2(wv.plane + gun * R * K, R * K); }
                    ns0 = __ldg(wv.ubase + gun);
                    ns1 = gun + 1 < (int64_t) p.n_experts * units_per_expert ? __ldg(wv.ubase + gun + 1) : ns0; // the very last unit: skipped
                }
            }
            for (int jp = j0; jp < j1; jp += G * M_TOK) {
                if (*failed) { n += TILES; continue; }
                WidePairReader rd;
                rd.open(wv, gu, lane);
                const uint8_t * pl = wv.plane + gu * R * K + 16 * lane;
                uint4 cur[SUB];
#pragma unroll
                for (int r = 0; r < SUB; r++) { cur[r] = ld_stream16(pl + r * CHUNK); }
                for (int t = 0; t < TILES; t++) {
                    // rows t*SUB .. t*SUB+3 of the unit in stream order (chunk-major: chunk t / Q, rows (t % Q) * SUB ..)
                    uint4 nxt[SUB];
                    if (t + 1 < TILES) {
#pragma unroll
                        for (int r = 0; r < SUB; r++) { nxt[r] = ld_stream16(pl + ((t + 1) * SUB + r) * CHUNK); }
                    }
                    const uint32_t b = n & 1, use = n >> 1;
                    if (use >= 1) { // the MMAs that read this buffer's previous contents must be complete
                        if (lane == 0) { wait_on(w_empty + b, (use - 1) & 1, failed); }
                        __syncwarp();
                    }
                    unsigned char * wb = wbuf + b * W_TILE_BYTES + lane_part;
#pragma unroll
                    for (int r = 0; r < SUB; r++) {
                        uint32_t en[8], w8[8];
                        rd.take8(lut, en);
                        assemble8(cur[r], en, w8);
                        const uint32_t row = (uint32_t) (n_row0 + r);
                        unsigned char * rp = wb + row * 128 + ((piece ^ (row & 7)) << 4);
#pragma unroll
                        for (int j = 0; j < 4; j++) { *(uint2 *) (rp + 2 * j * W_KTILE_BYTES) = make_uint2(w8[2 * j], w8[2 * j + 1]); }
                    }
                    proxy_fence();
                    __syncwarp();
                    if (lane == 0) { mbar_arrive(smem_u32(w_full + b)); }
                    n++;
                    if (t == 0 && jp == j0 && gun >= 0 && lane == 0) { // by now the two offsets have arrived
                        // codes are at most 12 bits per pair: a unit's streams hold at most R*K*3/16 words plus one partial word per lane
                        const uint32_t first = ns0 & ~3u, words = min(ns1 - first, (uint32_t) (R * K * 3 / 16 + 64));
                        if (ns1 > ns0) { bulk_prefetch_l2(wv.stream + first, ((words + 3u) & ~3u) * 4u); }
                    }
                    if (t + 1 < TILES) {
#pragma unroll
                        for (int r = 0; r < SUB; r++) { cur[r] = nxt[r]; }
                    }
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ gather warps, MMA warp; epilogue by all four
        const int ht = tid - DEC_WARPS * 32, hw = warp - DEC_WARPS;
        const bool mma_warp = warp == MMA_WARP;
        uint32_t n = 0;        // weight tiles consumed
        uint32_t vv = 0;       // activation slots used
        uint32_t passes = 0;
        for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
            const int e = item / m_blocks, mb = item - e * m_blocks;
            const int j0 = p.bounds[e], j1 = p.bounds[e + 1];
            for (int jp = j0; jp < j1; jp += G * M_TOK) {
                const int ntok = min(G * M_TOK, j1 - jp), ng = (ntok + M_TOK - 1) / M_TOK;
                // up to 64 tokens: M = 64 and a slot holds two k-tiles of 64 rows, so that the ring stays densely filled
                const bool small = ntok <= M_TOK / 2;
                const int kslots = small ? 4 : 8;        // slots per weight tile and token group
                const int total = TILES * kslots * ng;   // slots of the pass: for each weight tile, each k position, each token group
                int64_t my_dst[G];                       // output row of the token whose accumulators this thread reads
#pragma unroll
                for (int tg = 0; tg < G; tg++) {
                    const int ti = small ? (lane < 16 ? 16 * hw + lane : ntok) : tg * M_TOK + ht;
                    my_dst[tg] = ti < ntok ? (int64_t) p.ids_dst[jp + ti] : -1;
                }
                if (!mma_warp) {
                    // ---- gather: this thread copies 16-byte piece pc of rows r0, r0 + 12, ... of every slot
                    const int pc = ht & 7, r0 = ht >> 3;
                    constexpr int RSTEP = GATHERERS / 8, RMAX = (M_TOK + RSTEP - 1) / RSTEP;
                    const bf16 * src[G][RMAX]; // the rows' activations at piece pc (nullptr: no such token)
#pragma unroll
                    for (int tg = 0; tg < G; tg++) {
#pragma unroll
                        for (int i = 0; i < RMAX; i++) {
                            const int row = r0 + i * RSTEP, ti = tg * M_TOK + row;
                            src[tg][i] = (row < M_TOK && ti < ntok) ? p.x + (int64_t) p.ids_src1[jp + ti] * p.x_row + pc * 8 : nullptr;
                        }
                    }
                    for (int si = 0; si < total; si++) {
                        const int tile = si / ng, tg = si - tile * ng, kpos = tile % kslots, c = tile / kslots / Q;
                        const int kcol = (c * 8 + (small ? 2 * kpos : kpos)) * 64;
                        const uint32_t vs = vv + (uint32_t) si, slot = vs % SLOTS, use = vs / SLOTS;
                        if (use >= 1) { wait_on(x_free + slot, (use - 1) & 1, failed); }
                        const uint32_t dst0 = smem_u32(xbuf + slot * X_SLOT_BYTES) + (uint32_t) r0 * 128;
#pragma unroll
                        for (int g2 = 0; g2 < G; g2++) {
                            if (g2 == tg) {
#pragma unroll
                                for (int i = 0; i < RMAX; i++) {
                                    const int row = r0 + i * RSTEP;
                                    if (src[g2][i]) {
                                        const uint32_t at = dst0 + i * RSTEP * 128 + ((pc ^ (row & 7)) << 4);
                                        cp_async16(at, src[g2][i] + kcol);
                                        if (small) { cp_async16(at + X_SLOT_BYTES / 2, src[g2][i] + kcol + 64); } // rows < 64: second k-tile
                                    }
                                }
                            }
                        }
                        cp_async_arrive(x_full + slot); // arrives once this thread's copies so far have landed
                    }
                } else if (lane == 0) {
                    // ---- MMA issue
                    for (int si = 0; si < total; si++) {
                        const int tile = si / ng, tg = si - tile * ng, kpos = tile % kslots, cq = tile / kslots, c = cq / Q, q = cq - c * Q;
                        const bool last_of_tile = kpos == kslots - 1 && tg == ng - 1;
                        const uint32_t b = n & 1;
                        const uint32_t vs = vv + (uint32_t) si, slot = vs % SLOTS, use = vs / SLOTS;
                        if (kpos == 0 && tg == 0) { wait_on(w_full + b, (n >> 1) & 1, failed); }
                        wait_on(x_full + slot, use & 1, failed);
                        if (!*failed) {
                            proxy_fence(); // the copies (generic proxy) before the tensor core's reads (async proxy)
                            tc_fence_after();
                            const uint32_t d = tmem + (uint32_t) ((tg * Q + q) * N_TILE);
                            const uint32_t idesc = small ? instr_desc(M_TOK / 2) : instr_desc(M_TOK);
                            for (int j = 0; j < (small ? 2 : 1); j++) {
                                const int kb = small ? 2 * kpos + j : kpos;
                                const uint32_t a0 = smem_u32(xbuf + slot * X_SLOT_BYTES + j * (X_SLOT_BYTES / 2));
                                const uint32_t b0 = smem_u32(wbuf + b * W_TILE_BYTES + kb * W_KTILE_BYTES);
#pragma unroll
                                for (int s2 = 0; s2 < 4; s2++) {
                                    umma_bf16(d, tile_desc(a0 + s2 * 32), tile_desc(b0 + s2 * 32), idesc, (c | kb | s2) != 0);
                                }
                            }
                        }
                        umma_commit(x_free + slot);
                        if (last_of_tile) { umma_commit(w_empty + b); n++; }
                        if (si == total - 1) { umma_commit(acc_done); }
                    }
                }
                if (!mma_warp || lane != 0) { n += TILES; } // the issuing thread counted its tiles itself
                vv += (uint32_t) total;
                __syncwarp();
                // ---- epilogue: TMEM -> registers -> dst
                wait_on(acc_done, passes & 1, failed);
                passes++;
                tc_fence_after();
                for (int tg = 0; tg < ng; tg++) {
                    const int64_t drow = my_dst[tg];
#pragma unroll 1
                    for (int q = 0; q < Q; q++) {
                        __syncwarp(); // the TMEM loads are warp-wide: rejoin the lanes that skipped the stores
                        const uint32_t taddr = tmem + ((uint32_t) (32 * hw) << 16) + (uint32_t) ((tg * Q + q) * N_TILE);
                        uint32_t v0[32], v1[32];
                        tmem_ld32(taddr, v0);
                        tmem_ld32(taddr + 32, v1);
                        if (drow < 0 || *failed) { continue; }
                        const int64_t at0 = drow * p.dst_col + (int64_t) mb * ROWS_OUT + q * SUB;
                        if (GLU) { // v0: gate rows of units 0..7, v1: the matching up rows
#pragma unroll
                            for (int u = 0; u < 8; u++) {
                                float r4[4];
#pragma unroll
                                for (int r = 0; r < 4; r++) { r4[r] = silu_f(__uint_as_float(v0[u * 4 + r])) * __uint_as_float(v1[u * 4 + r]); }
                                store4(p, at0 + u * R, r4[0], r4[1], r4[2], r4[3]);
                            }
                        } else {
#pragma unroll
                            for (int u = 0; u < 8; u++) {
                                store4(p, at0 + u * R, __uint_as_float(v0[u * 4]), __uint_as_float(v0[u * 4 + 1]),
                                       __uint_as_float(v0[u * 4 + 2]), __uint_as_float(v0[u * 4 + 3]));
                                store4(p, at0 + (u + 8) * R, __uint_as_float(v1[u * 4]), __uint_as_float(v1[u * 4 + 1]),
                                       __uint_as_float(v1[u * 4 + 2]), __uint_as_float(v1[u * 4 + 3]));
                            }
                        }
                    }
                }
                tc_fence_before();
                helper_bar(); // the accumulators are read: the next pass may overwrite them
            }
        }
        cp_async_wait_all();
        if (mma_warp && lane == 0 && *failed) {
            // MMAs may still be in flight: wait (bounded) until the tensor core has drained before TMEM is freed
            umma_commit(drained);
            mbar_poll(smem_u32(drained), 0);
            atomicOr(&g_prefill_fault, 1u);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) { tmem_free(tmem, TMEM_COLS); }
}

// ---------------------------------------------------------------- second pass of the two-pass product
//
// k_tile_mm multiplies routed activation rows with weights that expand_tiles.cu has already decoded into operand-tile
// images ([k-tile][256 rows][128 bytes], 128-byte swizzled, 32 KB per k-tile). Without decoders the block is ten warps:
//   * warps 0..7 gather the routed activation rows (cp.async into a ring of 128-token x 64-column slots, each slot's
//     mbarrier completed by cp.async.mbarrier.arrive; eight warps because one slot per 472 MMA cycles is more copy
//     instructions than four warps issue) and afterwards read the accumulators (tcgen05.ld: warp w reads TMEM lanes
//     32 (w % 4) .. + 31 = tokens, warps 4..7 the second half of the columns) and store them, SwiGLU in registers;
//   * warp 8, one thread: tcgen05.mma with M = 128 tokens, N = 256 weight rows, K = 16; per (k-tile, token group) four of
//     them; tcgen05.commit hands activation slots and weight stages back and announces the finished accumulators;
//   * warp 9, one thread: one 32 KB bulk copy per k-tile of the item's image into a ring of four weight stages
//     (mbarrier expect_tx / complete_tx).
// A work item is (expert, row block of 256 image rows); a pass covers up to TM_G x 128 of the expert's tokens, whose
// accumulators (TM_G x 256 columns) fill tensor memory. The activations of a pass cross L2 -> shared memory once per
// 256 weight rows, and a weight k-tile is copied once per pass.
constexpr int TM_N = 256, TM_G = 2, TM_WST = 4, TM_XSL = 6;
constexpr int TM_GATHERERS = 256, TM_THREADS = 320, TM_MMA_WARP = 8, TM_W_WARP = 9;
constexpr int TM_W_STAGE = TM_N * 128;       // one k-tile of a row block
constexpr int TM_STAGE_ROW = 256 + 16;       // epilogue staging: 256 output bytes per thread, padded so that 16-byte stores of a quarter warp miss each other's banks
static_assert(TM_GATHERERS * TM_STAGE_ROW <= TM_XSL * X_SLOT_BYTES, "the epilogue stages its output rows in the activation ring");
__host__ __device__ constexpr uint32_t tm_instr_desc() { return 1u << 4 | 1u << 7 | 1u << 10 | (uint32_t) (TM_N >> 3) << 17 | (uint32_t) (M_TOK >> 4) << 24; }
static_assert(TM_G * TM_N <= TMEM_COLS, "accumulators of a pass must fit TMEM");

struct TileMmArgs {
    const unsigned char * images;       // [expert][row block][k-tile][256][128 bytes]
    const bf16 * x; int64_t x_row;
    const int32_t * ids_src1; const int32_t * ids_dst; const int32_t * bounds;
    char * dst; int64_t dst_col; bool dst_bf16;
    bool vec_ok;                        // dst rows allow 4-element vector stores
    bool bulk_ok;                       // dst rows are 16-byte aligned: BF16 rows may leave as 256-byte bulk stores
    int n_experts, blocks_per_expert, ktiles;
};

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void * src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// shared -> global bulk store (16-byte aligned addresses, size a multiple of 16), tracked by the thread's bulk groups
__device__ __forceinline__ void bulk_s2g(void * dst, uint32_t src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void tm_helper_bar() { asm volatile("bar.sync 1, %0;" ::"n"(TM_GATHERERS) : "memory"); }

template <bool GLU>
__global__ void __launch_bounds__(TM_THREADS, 1) k_tile_mm(const TileMmArgs p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char * smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u); // operand tiles need 1024-byte alignment
    unsigned char * wbuf = smem;                                   // TM_WST weight stages
    unsigned char * xbuf = wbuf + TM_WST * TM_W_STAGE;             // TM_XSL activation slots
    uint64_t * bars = (uint64_t *) (xbuf + TM_XSL * X_SLOT_BYTES);
    uint64_t * w_full = bars, * w_empty = bars + TM_WST, * x_full = w_empty + TM_WST, * x_free = x_full + TM_XSL;
    uint64_t * acc_done = x_free + TM_XSL, * drained = acc_done + 1, * fin = drained + 1;
    uint32_t * tmem_slot = (uint32_t *) (fin + 1);
    volatile int * failed = (volatile int *) (tmem_slot + 1);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        for (int i = 0; i < TM_WST; i++) { mbar_init(smem_u32(w_full + i), 1); mbar_init(smem_u32(w_empty + i), 1); }
        for (int i = 0; i < TM_XSL; i++) { mbar_init(smem_u32(x_full + i), TM_GATHERERS); mbar_init(smem_u32(x_free + i), 1); }
        mbar_init(smem_u32(acc_done), 1);
        mbar_init(smem_u32(drained), 1);
        mbar_init(smem_u32(fin), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        *failed = 0;
    }
    if (warp == 0) { tmem_alloc(smem_u32(tmem_slot), TMEM_COLS); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const int n_items = p.n_experts * p.blocks_per_expert, KT = p.ktiles;

    if (warp == TM_W_WARP) {
        // ------------------------------------------------------------------ weight stages: one bulk copy per k-tile
        if (lane == 0) {
            uint32_t n = 0, issued = 0; // stages of the walk, copies actually started (equal until a wait fails)
            // (Asking each k-tile into L2 eight k-tiles before its bulk copy was measured and lost: 988 / 1631 us per layer
            // at 2048 / 8192 tokens against 952 / 1567 without.)
            for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
                const int e = item / p.blocks_per_expert;
                const int j0 = p.bounds[e], j1 = p.bounds[e + 1];
                const unsigned char * img = p.images + (int64_t) item * KT * TM_W_STAGE;
                for (int jp = j0; jp < j1; jp += TM_G * M_TOK) {
                    for (int kt = 0; kt < KT; kt++, n++) {
                        const uint32_t s = n % TM_WST, use = n / TM_WST;
                        if (use >= 1) { wait_on(w_empty + s, (use - 1) & 1, failed); }
                        if (*failed) { continue; }
                        mbar_expect_tx(smem_u32(w_full + s), TM_W_STAGE);
                        bulk_g2s(smem_u32(wbuf + s * TM_W_STAGE), img + (int64_t) kt * TM_W_STAGE, TM_W_STAGE, smem_u32(w_full + s));
                        issued++;
                    }
                }
            }
            if (*failed) { // copies may still be in flight: wait (bounded) for every stage's last one before the block ends
                for (uint32_t back = 1; back <= (uint32_t) TM_WST && back <= issued; back++) {
                    const uint32_t m = issued - back;
                    mbar_poll(smem_u32(w_full + m % TM_WST), (m / TM_WST) & 1);
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ gather warps + epilogue, MMA warp
        const int ht = tid;                     // gather thread index (warps 0..7)
        const int hw = warp & 3, part = warp >> 2; // epilogue: TMEM lane quarter, and which half of the output columns
        const bool mma_warp = warp == TM_MMA_WARP;
        uint32_t n = 0;        // weight stages consumed
        uint32_t vv = 0;       // activation slots used
        uint32_t passes = 0;
        for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
            const int e = item / p.blocks_per_expert, nb = item - e * p.blocks_per_expert;
            const int j0 = p.bounds[e], j1 = p.bounds[e + 1];
            for (int jp = j0; jp < j1; jp += TM_G * M_TOK) {
                const int ntok = min(TM_G * M_TOK, j1 - jp), ng = (ntok + M_TOK - 1) / M_TOK;
                const int total = KT * ng;   // slots of the pass: for each k-tile, each token group
                if (!mma_warp) {
                    int64_t my_dst[TM_G];    // output row of the token whose accumulators this thread reads
#pragma unroll
                    for (int tg = 0; tg < TM_G; tg++) {
                        const int ti = tg * M_TOK + (ht & (M_TOK - 1));
                        my_dst[tg] = ti < ntok ? (int64_t) p.ids_dst[jp + ti] : -1;
                    }
                    // ---- gather: this thread copies 16-byte piece pc of rows r0, r0 + 32, ... of every slot
                    const int pc = ht & 7, r0 = ht >> 3;
                    constexpr int RSTEP = TM_GATHERERS / 8, RMAX = M_TOK / RSTEP;
                    const bf16 * src[TM_G][RMAX]; // the rows' activations at piece pc (nullptr: no such token)
#pragma unroll
                    for (int tg = 0; tg < TM_G; tg++) {
#pragma unroll
                        for (int i = 0; i < RMAX; i++) {
                            const int ti = tg * M_TOK + r0 + i * RSTEP;
                            src[tg][i] = ti < ntok ? p.x + (int64_t) p.ids_src1[jp + ti] * p.x_row + pc * 8 : nullptr;
                        }
                    }
                    for (int si = 0; si < total; si++) {
                        const int kt = si / ng, tg = si - kt * ng;
                        const uint32_t vs = vv + (uint32_t) si, slot = vs % TM_XSL, use = vs / TM_XSL;
                        if (use >= 1) { wait_on(x_free + slot, (use - 1) & 1, failed); }
                        const uint32_t dst0 = smem_u32(xbuf + slot * X_SLOT_BYTES) + (uint32_t) r0 * 128;
#pragma unroll
                        for (int g2 = 0; g2 < TM_G; g2++) {
                            if (g2 == tg) {
#pragma unroll
                                for (int i = 0; i < RMAX; i++) {
                                    const int row = r0 + i * RSTEP;
                                    if (src[g2][i]) { cp_async16(dst0 + i * RSTEP * 128 + ((pc ^ (row & 7)) << 4), src[g2][i] + kt * 64); }
                                }
                            }
                        }
                        cp_async_arrive(x_full + slot); // arrives once this thread's copies so far have landed
                    }
                    vv += (uint32_t) total;
                    // ---- epilogue: TMEM -> registers -> dst
                    wait_on(acc_done, passes & 1, failed);
                    passes++;
                    tc_fence_after();
                    // A thread holds one token's accumulators; written row by row from there, a store instruction would touch
                    // 32 different lines. Instead a thread stages a piece of its token's output row in shared memory (the
                    // activation ring is idle now: every MMA of the pass is complete) and sends it with one bulk store:
                    // 64 BF16 SwiGLU outputs (128 bytes) or 64 FP32 outputs (256 bytes). Warps 0..3 take the first half of
                    // the output columns, warps 4..7 the second. (Measured at 8192 tokens per layer with four helper
                    // warps: direct stores 1.91 ms, bulk stores 1.64 ms, a warp-level transposition through shared memory
                    // with four whole lines per store instruction 1.68 ms.)
                    const bool bulk_out = GLU && p.dst_bf16 && p.bulk_ok;
                    unsigned char * row = xbuf + ht * TM_STAGE_ROW;
                    for (int tg = 0; tg < ng; tg++) {
                        static_assert(TM_G == 2, "two token groups per pass");
                        const int64_t drow = tg ? my_dst[1] : my_dst[0];
                        const uint32_t taddr = tmem + ((uint32_t) (32 * hw) << 16) + (uint32_t) (tg * TM_N);
                        const bool live = drow >= 0 && !*failed;
                        if (GLU) { // image rows 0..127: gate, 128..255: the same rows of up
                            const int o0 = part * (TM_N / 4);   // this warp's 64 outputs
                            const int64_t at0 = drow * p.dst_col + (int64_t) nb * (TM_N / 2) + o0;
                            if (bulk_out) { bulk_wait_read<0>(); } // the previous store has read the staging row
#pragma unroll 1
                            for (int cc = 0; cc < TM_N / 4; cc += 32) {
                                __syncwarp(); // the TMEM loads are warp-wide
                                uint32_t v0[32], v1[32];
                                tmem_ld32(taddr + o0 + cc, v0);
                                tmem_ld32(taddr + TM_N / 2 + o0 + cc, v1);
                                if (!live) { continue; }
                                float r[32];
#pragma unroll
                                for (int u = 0; u < 32; u++) { r[u] = silu_f(__uint_as_float(v0[u])) * __uint_as_float(v1[u]); }
                                if (bulk_out) {
#pragma unroll
                                    for (int u = 0; u < 32; u += 8) {
                                        uint32_t o[4];
#pragma unroll
                                        for (int j = 0; j < 4; j++) {
                                            const __nv_bfloat162 h = __floats2bfloat162_rn(r[u + 2 * j], r[u + 2 * j + 1]);
                                            o[j] = *(const uint32_t *) &h;
                                        }
                                        *(uint4 *) (row + (cc + u) * 2) = make_uint4(o[0], o[1], o[2], o[3]);
                                    }
                                } else {
#pragma unroll
                                    for (int u = 0; u < 32; u += 4) { store4(p.dst, p.dst_bf16, p.vec_ok, at0 + cc + u, r[u], r[u + 1], r[u + 2], r[u + 3]); }
                                }
                            }
                            if (bulk_out) {
                                if (live) { proxy_fence(); bulk_s2g((bf16 *) p.dst + at0, smem_u32(row), 128); }
                                bulk_commit();
                            }
                        } else if (!p.dst_bf16 && p.bulk_ok) {   // this warp's 128 FP32 outputs = two pieces of 64
                            const int64_t at0 = drow * p.dst_col + (int64_t) nb * TM_N;
#pragma unroll 1
                            for (int c0 = part * (TM_N / 2); c0 < (part + 1) * (TM_N / 2); c0 += 64) {
                                bulk_wait_read<0>();
#pragma unroll 1
                                for (int cc = c0; cc < c0 + 64; cc += 32) {
                                    __syncwarp();
                                    uint32_t v0[32];
                                    tmem_ld32(taddr + cc, v0);
                                    if (!live) { continue; }
#pragma unroll
                                    for (int u = 0; u < 32; u += 4) { *(uint4 *) (row + (cc - c0 + u) * 4) = make_uint4(v0[u], v0[u + 1], v0[u + 2], v0[u + 3]); }
                                }
                                if (live) { proxy_fence(); bulk_s2g((float *) p.dst + at0 + c0, smem_u32(row), 256); }
                                bulk_commit();
                            }
                        } else {
                            const int64_t at0 = drow * p.dst_col + (int64_t) nb * TM_N;
#pragma unroll 1
                            for (int cc = part * (TM_N / 2); cc < (part + 1) * (TM_N / 2); cc += 32) {
                                __syncwarp();
                                uint32_t v0[32];
                                tmem_ld32(taddr + cc, v0);
                                if (!live) { continue; }
#pragma unroll
                                for (int u = 0; u < 32; u += 4) {
                                    store4(p.dst, p.dst_bf16, p.vec_ok, at0 + cc + u, __uint_as_float(v0[u]), __uint_as_float(v0[u + 1]),
                                           __uint_as_float(v0[u + 2]), __uint_as_float(v0[u + 3]));
                                }
                            }
                        }
                    }
                    bulk_wait_read<0>(); // the staging rows are activation slots again from the next pass on
                    __syncwarp();
                    tc_fence_before();
                    tm_helper_bar(); // every helper warp has read its part
                    if (tid == 0) { mbar_arrive(smem_u32(drained)); } // the next pass may overwrite the accumulators
                } else if (lane == 0) {
                    // ---- MMA issue
                    if (passes >= 1) { wait_on(drained, (passes - 1) & 1, failed); tc_fence_after(); }
                    passes++;
                    for (int si = 0; si < total; si++) {
                        const int kt = si / ng, tg = si - kt * ng;
                        const uint32_t s = n % TM_WST;
                        const uint32_t vs = vv + (uint32_t) si, slot = vs % TM_XSL, use = vs / TM_XSL;
                        if (tg == 0) { wait_on(w_full + s, (n / TM_WST) & 1, failed); }
                        wait_on(x_full + slot, use & 1, failed);
                        if (!*failed) {
                            proxy_fence(); // the gather's copies (generic proxy) before the tensor core's reads (async proxy)
                            tc_fence_after();
                            const uint32_t d = tmem + (uint32_t) (tg * TM_N);
                            const uint32_t a0 = smem_u32(xbuf + slot * X_SLOT_BYTES), b0 = smem_u32(wbuf + s * TM_W_STAGE);
#pragma unroll
                            for (int s2 = 0; s2 < 4; s2++) {
                                umma_bf16(d, tile_desc(a0 + s2 * 32), tile_desc(b0 + s2 * 32), tm_instr_desc(), (kt | s2) != 0);
                            }
                        }
                        umma_commit(x_free + slot);
                        if (tg == ng - 1) { umma_commit(w_empty + s); n++; }
                        if (si == total - 1) { umma_commit(acc_done); }
                    }
                    vv += (uint32_t) total;
                }
            }
        }
        if (!mma_warp) { cp_async_wait_all(); }
        if (mma_warp && lane == 0 && *failed) {
            // MMAs may still be in flight: wait (bounded) until the tensor core has drained before TMEM is freed
            umma_commit(fin);
            mbar_poll(smem_u32(fin), 0);
            atomicOr(&g_prefill_fault, 1u);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) { tmem_free(tmem, TMEM_COLS); }
}

constexpr size_t TM_SMEM = (size_t) TM_WST * TM_W_STAGE + (size_t) TM_XSL * X_SLOT_BYTES + 256 + 1024;

PairView view_of(const bf16n_weight & w) {
    return {w.plane, (const uint32_t *) (w.aux + w.off_a), (const uint32_t *) (w.aux + w.off_b),
            (const uint16_t *) (w.aux + w.off_c), (const uint32_t *) (w.aux + w.off_d)};
}

template <bool GLU, int SLOTS> constexpr size_t smem_bytes() {
    return 2 * W_TILE_BYTES + SLOTS * X_SLOT_BYTES + (GLU ? 2 : 1) * 4 * HP_MAX_PAIRS + 256 + 1024;
}

constexpr int G_TOK = 2;                      // token groups per pass
constexpr int SLOTS_GLU = 3, SLOTS_ONE = 4;   // what fits beside two tables / one table

} // namespace

unsigned int * prefill_fault_word() {
    unsigned int * p = nullptr;
    cuda_ok(cudaGetSymbolAddress((void **) &p, g_prefill_fault), "fault word address");
    return p;
}

void prefill_init() {
    cuda_ok(cudaFuncSetAttribute(k_prefill<4, 8, true, true, G_TOK, SLOTS_GLU>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int) smem_bytes<true, SLOTS_GLU>()), "k_prefill glu");
    cuda_ok(cudaFuncSetAttribute(k_prefill<4, 8, true, false, G_TOK, SLOTS_ONE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int) smem_bytes<false, SLOTS_ONE>()), "k_prefill gate");
    cuda_ok(cudaFuncSetAttribute(k_prefill<1, 16, false, false, G_TOK, SLOTS_ONE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int) smem_bytes<false, SLOTS_ONE>()), "k_prefill down");
    cuda_ok(cudaFuncSetAttribute(k_tile_mm<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) TM_SMEM), "k_tile_mm glu");
    cuda_ok(cudaFuncSetAttribute(k_tile_mm<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) TM_SMEM), "k_tile_mm");
    expand_tiles_init();
}

bool prefill_supported(const bf16n_weight & w, const bf16n_weight * up) {
    const int C = (int) (w.K / CHUNK);
    const bool shape = w.format == FMT_HUFPAIR && !w.fo && (w.cm || w.K == CHUNK) && ((C == 4 && w.R == 8) || (C == 1 && w.R == 16));
    if (!up) { return shape; }
    const bool same = up->format == w.format && up->K == w.K && up->R == w.R && up->cm == w.cm && up->fo == w.fo && up->rows == w.rows;
    return same && w.format == FMT_HUFPAIR && w.K == 2048 && w.cm && w.R == 8;
}

// The caller's buffer for the decoded operand tiles of the two-pass product (bf16n_set_workspace): one per process, used
// by one stream at a time.
static void * g_workspace = nullptr;
static size_t g_workspace_bytes = 0;

void prefill_set_workspace(void * p, size_t bytes) {
    g_workspace = p;
    g_workspace_bytes = p ? bytes : 0;
}

size_t prefill_workspace_bytes(const bf16n_weight & w, const bf16n_weight * up) {
    if (!expand_tiles_supported(w) || (up && !expand_tiles_supported(*up))) { return 0; }
    return (size_t) w.rows * (size_t) w.K * 2 * (up ? 2 : 1);
}

namespace {

// decode pass (expand_tiles.cu) + tensor-core pass over the decoded tiles
bool two_pass(const bf16n_weight & w, const bf16n_weight * up, const PrefillArgs & a, int n_experts, cudaStream_t st) {
    const size_t need = prefill_workspace_bytes(w, up);
    const int rows_per_block = up ? TM_N / 2 : TM_N;
    if (need == 0 || need > g_workspace_bytes || a.rows_per_expert % rows_per_block || ((uintptr_t) g_workspace % 1024)) { return false; }
    expand_tiles(w, up, n_experts, a.bounds, g_workspace, st);
    TileMmArgs t = {};
    t.images = (const unsigned char *) g_workspace;
    t.x = a.x; t.x_row = a.x_row;
    t.ids_src1 = a.ids_src1; t.ids_dst = a.ids_dst; t.bounds = a.bounds;
    t.dst = a.dst; t.dst_col = a.dst_col; t.dst_bf16 = a.dst_bf16;
    t.vec_ok = a.vec_ok;
    t.bulk_ok = ((uintptr_t) a.dst % 16) == 0 && (a.dst_col * (a.dst_bf16 ? 2 : 4)) % 16 == 0;
    t.n_experts = n_experts;
    t.blocks_per_expert = (int) (a.rows_per_expert / rows_per_block);
    t.ktiles = (int) (w.K / 64);
    const unsigned grid = (unsigned) std::min<int64_t>(device_info().sms, (int64_t) n_experts * t.blocks_per_expert);
    if (up) { k_tile_mm<true><<<grid, TM_THREADS, TM_SMEM, st>>>(t); }
    else { k_tile_mm<false><<<grid, TM_THREADS, TM_SMEM, st>>>(t); }
    check_launch();
    return true;
}

} // namespace

void prefill_mm_ids(const bf16n_weight & w, const bf16n_weight * up, const void * x_bf16, int64_t x_row, const int32_t * ids_src1,
                    const int32_t * ids_dst, const int32_t * bounds, void * dst, bool dst_bf16, int64_t dst_col, int n_experts,
                    int n_tok, int n_used, cudaStream_t st) {
    (void) n_tok; (void) n_used;
    PrefillArgs a = {};
    a.w0 = view_of(w);
    a.w1 = up ? view_of(*up) : a.w0;
    a.x = (const bf16 *) x_bf16; a.x_row = x_row;
    a.ids_src1 = ids_src1; a.ids_dst = ids_dst; a.bounds = bounds;
    a.dst = (char *) dst; a.dst_col = dst_col; a.dst_bf16 = dst_bf16;
    a.vec_ok = ((uintptr_t) dst % 16) == 0 && dst_col % 4 == 0;
    a.n_experts = n_experts;
    a.rows_per_expert = w.rows / n_experts;
    require(((uintptr_t) x_bf16 % 16) == 0 && (x_row * 2) % 16 == 0, "batched activations must be 16-byte aligned rows");
    const int rows_out = (up ? DEC_WARPS / 2 : DEC_WARPS) * w.R;
    require(a.rows_per_expert % rows_out == 0, "rows per expert must be a multiple of the batched kernel's row block");
    if (g_workspace && two_pass(w, up, a, n_experts, st)) { return; }
    const unsigned grid = (unsigned) std::min<int64_t>(device_info().sms, (int64_t) n_experts * (a.rows_per_expert / rows_out));
    if (up) {
        k_prefill<4, 8, true, true, G_TOK, SLOTS_GLU><<<grid, NTHREADS, smem_bytes<true, SLOTS_GLU>(), st>>>(a);
    } else if (w.K == 2048) {
        k_prefill<4, 8, true, false, G_TOK, SLOTS_ONE><<<grid, NTHREADS, smem_bytes<false, SLOTS_ONE>(), st>>>(a);
    } else {
        k_prefill<1, 16, false, false, G_TOK, SLOTS_ONE><<<grid, NTHREADS, smem_bytes<false, SLOTS_ONE>(), st>>>(a);
    }
    check_launch();
}

} // namespace b16
