// Batched (prefill) routed product on the 5th-generation tensor cores: dst[t, slot, :] = W_e x_t for every routed
// (token, slot) pair, optionally fused gate/up + SwiGLU. Replaces the reference's persistent mma.sync kernel
// (core/include/bf16n/kernels.cuh:1162-1505) with a tcgen05 / TMEM design.
//
// One persistent block of 16 warps per SM walks work items (expert, block of 128 weight rows, pass of up to NT of the
// expert's tokens). For an item it loops over the 512-column chunks of K:
//   1. decode: each warp owns one unit and decodes this chunk of its rows straight into the A operand tile in shared
//      memory, in the canonical K-major 128-byte-swizzled layout the tensor core reads (8 tiles of 128 rows x 64 columns;
//      a lane's 4 consecutive weights are one 8-byte store: the lane-major plane maps lanes 0..15 / 16..31 of column
//      quad j to the 64-column tiles 2j / 2j+1). The bit-stream state stays in registers across chunks, which is what
//      chunk-major units are for. With SwiGLU the tile holds 64 gate rows and the 64 matching up rows.
//   2. multiply: per 64-column tile the routed activation rows are gathered (cp.async, zero-filled padding) into a
//      double-buffered swizzled B tile while the previous tile is multiplied: one elected thread issues four
//      tcgen05.mma (M = 128, N = tokens rounded to 16, K = 16) per tile, accumulating in TMEM, and commits to an
//      mbarrier that releases the B buffer.
// After the last chunk the accumulators are read back with tcgen05.ld (warp w reads TMEM lanes 32*(w%4)..+31) and
// scattered through ids_dst; the SwiGLU variant first moves the up half next to the gate half through shared memory.
// The gathered activation tiles run STAGES deep so that the gather latency is hidden behind the MMAs of earlier tiles.
// Every wait on an mbarrier is bounded: a thread whose wait expires clears a flag in shared memory, the block reads the
// flag after its next barrier, records the fault, frees its TMEM and returns. No cluster launch, no multicast.
#include "decode.cuh"
#include "launch.h"

namespace b16 {
namespace {

using namespace dev;
using bf16 = __nv_bfloat16;

__device__ unsigned int g_prefill_fault; // a bounded wait expired (diagnostic)

constexpr int NTHREADS = 512;
constexpr int M_TILE = 128;              // weight rows per item (GLU: 64 gate + 64 up)
constexpr int KB = 64;                   // columns per operand tile (128 bytes of BF16: one swizzle row)
constexpr int A_TILE_BYTES = M_TILE * 128;
constexpr int A_SLAB_BYTES = 8 * A_TILE_BYTES; // one 512-column chunk
constexpr uint32_t POLL_LIMIT = 1u << 20;

__device__ __forceinline__ uint32_t smem_u32(const void * p) { return (uint32_t) __cvta_generic_to_shared(p); }

// ---- mbarrier / tcgen05 wrappers
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ bool mbar_poll(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < POLL_LIMIT; i++) {
        uint32_t done;
        asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) { return true; }
    }
    return false;
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
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void proxy_fence() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
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
// 16-byte async copy global -> shared; bytes = 0 writes zeros (padding rows)
__device__ __forceinline__ void cp_async16_zfill(uint32_t dst, const void * src, uint32_t bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// shared-memory matrix descriptor of a K-major, 128-byte-swizzled tile: rows 128 bytes apart, 8-row groups 1024 bytes
// apart (stride byte offset), descriptor version 1, layout type 2; `addr` may point 32*k bytes into the first row
__device__ __forceinline__ uint64_t tile_desc(uint32_t addr) {
    return (uint64_t) ((addr >> 4) & 0x3FFFu) | (uint64_t) 1 << 16 | (uint64_t) (1024 >> 4) << 32 | (uint64_t) 1 << 46 | (uint64_t) 2 << 61;
}
// kind::f16 instruction descriptor: FP32 accumulate, BF16 A and B, both K-major, M = 128, N = n
__device__ __forceinline__ uint32_t instr_desc(uint32_t n) {
    return 1u << 4 | 1u << 7 | 1u << 10 | (n >> 3) << 17 | (uint32_t) (M_TILE >> 4) << 24;
}

struct PrefillArgs {
    PairView w0, w1;                    // w1: the up matrix (GLU)
    const bf16 * x; int64_t x_row;      // activations: row ids_src1[j] * x_row
    const int32_t * ids_src1; const int32_t * ids_dst; const int32_t * bounds;
    char * dst; int64_t dst_col; bool dst_bf16;
    int n_experts;
    int64_t rows_per_expert;
};

// C chunks per row, R rows per unit, CM chunk-major units, GLU fused gate/up + SwiGLU, NT tokens per pass, STAGES
// gathered activation tiles in flight
template <int C, int R, bool CM, bool GLU, int NT, int STAGES>
__global__ void __launch_bounds__(NTHREADS, 1) k_prefill(const PrefillArgs p) {
    constexpr int K = C * CHUNK;
    constexpr int B_TILE_BYTES = NT * 128;
    constexpr int UNITS = M_TILE / R;                  // units decoded per item (GLU: half gate, half up)
    constexpr int ROWS_OUT = GLU ? M_TILE / 2 : M_TILE; // output rows per item
    extern __shared__ unsigned char smem_raw[];
    unsigned char * smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u); // operand tiles need 1024-byte alignment
    unsigned char * a_slab = smem;                                   // 128 KB
    unsigned char * b_buf = smem + A_SLAB_BYTES;                     // STAGES x NT x 128 B
    uint32_t * lut0 = (uint32_t *) (b_buf + STAGES * B_TILE_BYTES);
    uint32_t * lut1 = lut0 + (GLU ? HP_MAX_PAIRS : 0);
    int32_t * tok_src = (int32_t *) (lut1 + HP_MAX_PAIRS);            // activation row of each token of the pass
    int32_t * tok_dst = tok_src + NT;
    uint64_t * bars = (uint64_t *) (tok_dst + NT);                    // one per B stage: its MMAs are complete
    uint32_t * tmem_slot = (uint32_t *) (bars + STAGES);
    volatile int * verdict = (volatile int *) (tmem_slot + 1);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int i = tid; i < HP_MAX_PAIRS / 4; i += NTHREADS) {
        ((uint4 *) lut0)[i] = __ldg((const uint4 *) p.w0.lut + i);
        if (GLU) { ((uint4 *) lut1)[i] = __ldg((const uint4 *) p.w1.lut + i); }
    }
    if (tid == 0) {
        for (int i = 0; i < STAGES; i++) { mbar_init(smem_u32(bars + i), 1); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (tid == 0) { *verdict = 1; }
    if (warp == 0) { tmem_alloc(smem_u32(tmem_slot), NT); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    uint32_t uses[STAGES]; // commits so far on each B stage's barrier
#pragma unroll
    for (int i = 0; i < STAGES; i++) { uses[i] = 0; }
    bool ok = true;

    const int m_blocks = (int) (p.rows_per_expert / ROWS_OUT);
    const int64_t units_per_expert = p.rows_per_expert / R;
    for (int item = blockIdx.x; ok && item < p.n_experts * m_blocks; item += gridDim.x) {
        const int e = item / m_blocks, mb = item - e * m_blocks;
        const int j0 = p.bounds[e], j1 = p.bounds[e + 1];
        for (int jp = j0; ok && jp < j1; jp += NT) {
            const int ntok = min(NT, j1 - jp);
            const uint32_t n_mma = (uint32_t) ((ntok + 15) & ~15);
            for (int i = tid; i < NT; i += NTHREADS) {
                tok_src[i] = i < ntok ? p.ids_src1[jp + i] : 0;
                tok_dst[i] = i < ntok ? p.ids_dst[jp + i] : 0;
            }
            // this warp's unit: its matrix, table, first row inside the A tile
            const bool second = GLU && warp >= UNITS / 2;                 // up half
            const bool decoder = warp < UNITS;
            const PairView & wv = second ? p.w1 : p.w0;
            const uint32_t * lut = second ? lut1 : lut0;
            const int uw = GLU ? (second ? warp - UNITS / 2 : warp) : warp; // unit inside this item's row block
            const int64_t gu = (int64_t) e * units_per_expert + (int64_t) mb * (GLU ? UNITS / 2 : UNITS) + uw;
            const int row_base = (second ? M_TILE / 2 : 0) + uw * R;
            DeepPairReader rd;
            const uint8_t * pl = nullptr;
            if (decoder) {
                rd.open(wv, gu, lane);
                pl = wv.plane + gu * R * K + 16 * lane;
            }
            __syncthreads(); // tok_src / tok_dst visible

            // gather of B tile g (global tile counter over the item) into buffer g & 1
            auto load_b = [&](int g) {
                const int kcol = g * KB;
                unsigned char * dstb = b_buf + (g % STAGES) * B_TILE_BYTES;
                for (int i = tid; i < (int) n_mma * 8; i += NTHREADS) {
                    const int t = i >> 3, piece = i & 7;
                    const bf16 * src = p.x + (int64_t) tok_src[t] * p.x_row + kcol + piece * 8;
                    cp_async16_zfill(smem_u32(dstb + t * 128 + ((piece ^ (t & 7)) << 4)), src, t < ntok ? 16u : 0u);
                }
                cp_async_commit();
            };
            constexpr int TILES = C * 8;
#pragma unroll
            for (int g = 0; g < STAGES - 1; g++) {
                if (g < TILES) { load_b(g); } else { cp_async_commit(); }
            }
            for (int c = 0; ok && c < C; c++) {
                // 1. decode chunk c of the unit's rows into the A slab (the wait that ended the previous chunk made
                //    sure every MMA that read the slab is complete)
                if (decoder) {
                    for (int rr = 0; rr < R; rr++) {
                        const int64_t off = CM ? (int64_t) (c * R + rr) * CHUNK : (int64_t) rr * K + (int64_t) c * CHUNK;
                        const uint4 sm = ld_stream16(pl + off);
                        uint32_t en[8], wv8[8];
                        rd.take8(lut, en);
                        assemble8(sm, en, wv8);
                        const int row = row_base + rr;
                        unsigned char * rp = a_slab + row * 128 + (((lane & 15) >> 1) ^ (row & 7)) * 16 + (lane & 1) * 8;
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            *(uint2 *) (rp + (2 * j + (lane >> 4)) * A_TILE_BYTES) = make_uint2(wv8[2 * j], wv8[2 * j + 1]);
                        }
                    }
                }
                // 2. the eight 64-column tiles of the chunk; the block barrier of the first tile also publishes the slab
                for (int kb = 0; kb < 8; kb++) {
                    const int g = c * 8 + kb, st = g % STAGES;
                    // tile g + STAGES - 1 goes into the stage tile g - 1 used: its MMAs must be complete
                    if (g + STAGES - 1 < TILES) {
                        if (g >= 1) {
                            const int ps = (g - 1) % STAGES;
                            if (!mbar_poll(smem_u32(bars + ps), (uses[ps] - 1) & 1)) { *verdict = 0; }
                        }
                        load_b(g + STAGES - 1);
                    } else {
                        cp_async_commit(); // keeps the group count in step
                    }
                    cp_async_wait<STAGES - 1>(); // tile g has landed (this thread's copies)
                    proxy_fence();
                    __syncthreads();
                    if (*verdict == 0) { ok = false; break; }
                    if (tid == 0) {
                        tc_fence_after();
                        const uint32_t idesc = instr_desc(n_mma);
                        const uint32_t a0 = smem_u32(a_slab + kb * A_TILE_BYTES), b0 = smem_u32(b_buf + st * B_TILE_BYTES);
#pragma unroll
                        for (int s2 = 0; s2 < 4; s2++) {
                            umma_bf16(tmem, tile_desc(a0 + s2 * 32), tile_desc(b0 + s2 * 32), idesc, (g | s2) != 0);
                        }
                        umma_commit(smem_u32(bars + st));
                    }
                    uses[st]++;
                }
                if (!ok) { break; }
                // all MMAs of this chunk complete before the slab is rewritten / the accumulators are read
                {
                    const int ls = (c * 8 + 7) % STAGES;
                    if (!mbar_poll(smem_u32(bars + ls), (uses[ls] - 1) & 1)) { *verdict = 0; }
                    __syncthreads();
                    if (*verdict == 0) { ok = false; }
                }
            }
            if (!ok) { break; }
            // 3. epilogue: TMEM -> registers -> dst
            tc_fence_after();
            const int q = warp & 3, cg = warp >> 2;            // TMEM lane quadrant, column group
            constexpr int COLS_PER_WARP = NT / 4;
            const int m = 32 * q + lane;                       // row of the A tile held by this thread
            float * xchg = (float *) b_buf;                    // GLU: up half moved next to the gate half
            for (int c0 = cg * COLS_PER_WARP; c0 < (cg + 1) * COLS_PER_WARP; c0 += 32) {
                if (c0 >= (int) n_mma) { break; }
                uint32_t v[32];
                tmem_ld32(tmem + ((uint32_t) (32 * q) << 16) + (uint32_t) c0, v);
                if (!GLU) {
                    const int64_t row = (int64_t) mb * ROWS_OUT + m;
#pragma unroll
                    for (int i = 0; i < 32; i++) {
                        if (c0 + i < ntok) {
                            const int64_t at = (int64_t) tok_dst[c0 + i] * p.dst_col + row;
                            if (p.dst_bf16) { ((bf16 *) p.dst)[at] = __float2bfloat16_rn(__uint_as_float(v[i])); }
                            else { ((float *) p.dst)[at] = __uint_as_float(v[i]); }
                        }
                    }
                } else if (q >= 2) {
#pragma unroll
                    for (int i = 0; i < 32; i++) { xchg[(c0 + i) * 64 + (m - 64)] = __uint_as_float(v[i]); }
                }
                if (GLU) {
                    // gate warps wait for the matching up warps (same column group): named barrier per column group
                    asm volatile("bar.sync %0, 128;" ::"r"(1 + cg) : "memory");
                    if (q < 2) {
                        const int64_t row = (int64_t) mb * ROWS_OUT + m;
#pragma unroll
                        for (int i = 0; i < 32; i++) {
                            if (c0 + i < ntok) {
                                const float gte = __uint_as_float(v[i]), up = xchg[(c0 + i) * 64 + m];
                                const float r = silu_f(gte) * up;
                                const int64_t at = (int64_t) tok_dst[c0 + i] * p.dst_col + row;
                                if (p.dst_bf16) { ((bf16 *) p.dst)[at] = __float2bfloat16_rn(r); } else { ((float *) p.dst)[at] = r; }
                            }
                        }
                    }
                    asm volatile("bar.sync %0, 128;" ::"r"(1 + cg) : "memory");
                }
            }
            tc_fence_before();
            __syncthreads(); // accumulators read, exchange area free: the next pass may overwrite both
        }
    }
    if (!ok && tid == 0) { atomicOr(&g_prefill_fault, 1u); }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) { tmem_free(tmem, NT); }
}

PairView view_of(const bf16n_weight & w) {
    return {w.plane, (const uint32_t *) (w.aux + w.off_a), (const uint32_t *) (w.aux + w.off_b),
            (const uint16_t *) (w.aux + w.off_c), (const uint32_t *) (w.aux + w.off_d)};
}

template <bool GLU, int NT, int STAGES> constexpr size_t smem_bytes() {
    return A_SLAB_BYTES + STAGES * NT * 128 + (GLU ? 2 : 1) * 4 * HP_MAX_PAIRS + 2 * NT * 4 + STAGES * 8 + 16 + 1024;
}

} // namespace

void prefill_init() {
    cuda_ok(cudaFuncSetAttribute(k_prefill<4, 8, true, true, 128, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem_bytes<true, 128, 4>()), "k_prefill glu");
    cuda_ok(cudaFuncSetAttribute(k_prefill<4, 8, true, false, 256, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem_bytes<false, 256, 2>()), "k_prefill gate");
    cuda_ok(cudaFuncSetAttribute(k_prefill<1, 16, false, false, 256, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem_bytes<false, 256, 2>()), "k_prefill down");
}

bool prefill_supported(const bf16n_weight & w, const bf16n_weight * up) {
    const int C = (int) (w.K / CHUNK);
    const bool shape = w.format == FMT_HUFPAIR && !w.fo && (w.cm || w.K == CHUNK) && ((C == 4 && w.R == 8) || (C == 1 && w.R == 16));
    if (!up) { return shape; }
    const bool same = up->format == w.format && up->K == w.K && up->R == w.R && up->cm == w.cm && up->fo == w.fo && up->rows == w.rows;
    return same && w.format == FMT_HUFPAIR && w.K == 2048 && w.cm && w.R == 8;
}

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
    a.n_experts = n_experts;
    a.rows_per_expert = w.rows / n_experts;
    require(((uintptr_t) x_bf16 % 16) == 0 && (x_row * 2) % 16 == 0, "batched activations must be 16-byte aligned rows");
    const int rows_out = up ? M_TILE / 2 : M_TILE;
    require(a.rows_per_expert % rows_out == 0, "rows per expert must be a multiple of the batched kernel's row block");
    const unsigned grid = (unsigned) std::min<int64_t>(device_info().sms, (int64_t) n_experts * (a.rows_per_expert / rows_out));
    if (up) {
        k_prefill<4, 8, true, true, 128, 4><<<grid, NTHREADS, smem_bytes<true, 128, 4>(), st>>>(a);
    } else if (w.K == 2048) {
        k_prefill<4, 8, true, false, 256, 2><<<grid, NTHREADS, smem_bytes<false, 256, 2>(), st>>>(a);
    } else {
        k_prefill<1, 16, false, false, 256, 2><<<grid, NTHREADS, smem_bytes<false, 256, 2>(), st>>>(a);
    }
    check_launch();
}

} // namespace b16
