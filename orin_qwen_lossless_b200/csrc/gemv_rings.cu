// Large-matrix decode+GEMV for BF16 activations (the vocabulary projection): per-lane shared-memory rings.
//
// Decoding a lane stream is a serial chain (table lookup -> code length -> next lookup) of about 18 instructions per
// pair of weights, most of them on the half-rate integer pipes, so the kernel is bound by instruction issue and by the
// shared-memory pipe (random table lookups conflict about 4 ways), not by HBM. What helps is many independent chains per
// SM and few registers per chain:
//   * one unit per warp and up to 28 warps per block (72 registers per thread): the activations live in shared memory
//     (BF16, natural order, conflict-free 8-byte reads at base + immediate) and the plane is prefetched one row ahead;
//   * a chain's stream footprint is a 128-byte ring per lane (4 KB per warp) filled with cp.async 16-byte granules,
//     topped up at every row start to more than 96 bytes ahead of the read pointer; a row consumes at most 48 bytes
//     (32 codes of up to 12 bits) and everything copied before the previous row start has landed (wait_group 0 at the
//     row start, a row of work after the copies were issued), so the words a row reads are always complete;
//   * ring addressing: byte offset from the unit's 16-byte aligned start, modulo 128, XOR a per-lane constant that also
//     carries the lane's ring base: one logic op per address, and lanes that read in step hit different banks;
//   * BF16 x BF16 + FP32 fma on the activations and the merged weights (exact products, one rounding: the same bits as
//     an FP32 fma of the widened values), the same summation order as every other kernel of the format.
#include "decode.cuh"
#include "launch.h"

#include <cstdlib>

namespace b16 {
namespace {

using namespace dev;
using bf16 = __nv_bfloat16;

struct Opaque { uint32_t one, four, minus_one, thirty_two, sixteen; }; // see gemv_staged.cu: keeps adds on the multiply pipe

constexpr int RING_BYTES = 128;
constexpr uint32_t RING_TARGET = 96; // fetch while at most this many bytes are ahead of the read pointer

__device__ __forceinline__ uint32_t smem_u32(const void * p) { return (uint32_t) __cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t imad(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// Ring read. Not volatile, so that the two chains of a warp can be interleaved by the instruction scheduler; `token`
// is a value produced by the last cp.async wait, which keeps the read after that wait (the data dependency is the
// only ordering the compiler sees).
__device__ __forceinline__ uint32_t lds32(uint32_t addr, uint32_t token) {
    uint32_t v;
    asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr), "r"(token));
    return v;
}
__device__ __forceinline__ uint32_t lds32_ro(uint32_t addr) { // table reads: never written after the block barrier
    uint32_t v;
    asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t shl_wrap_hi(uint32_t lo, uint32_t hi, uint32_t n) {
    uint32_t d;
    asm("shf.l.wrap.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(lo), "r"(hi), "r"(n));
    return d;
}
// (a & 127) ^ c
__device__ __forceinline__ uint32_t ring_addr(uint32_t off, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, 127, %2, 0x6A;" : "=r"(d) : "r"(off), "r"(c)); // (a & b) ^ c
    return d;
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void * src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ uint32_t cp_async_wait_all() { // returns the token ring reads depend on
    uint32_t token;
    asm volatile("cp.async.wait_group 0;\n\tmov.u32 %0, 0;" : "=r"(token) :: "memory");
    return token;
}

// One lane stream read through the lane's ring. Offsets are bytes from `base` (the unit's stream start rounded down to
// 16 bytes); only their low 7 bits address the ring.
struct RingReader {
    const uint8_t * base; // global
    uint32_t key;         // ring base | lane swizzle
    uint32_t fetched;     // offset of the next granule to copy
    uint32_t next;        // offset of the next word to read
    uint32_t hi, lo, ahead, v, t;
    uint32_t token;       // from the last cp.async wait

    // copy granules until more than RING_TARGET bytes are ahead of the read pointer (at most `rounds` granules)
    template <int ROUNDS>
    __device__ __forceinline__ void top_up(const Opaque & k) {
        int32_t avail = (int32_t) imad(next, k.minus_one, fetched); // negative right after open()
#pragma unroll
        for (int i = 0; i < ROUNDS; i++) {
            if (avail <= (int32_t) RING_TARGET) {
                cp_async16(ring_addr(fetched, key), base + fetched);
                fetched = imad(k.sixteen, k.one, fetched);
                avail = (int32_t) imad(k.sixteen, k.one, (uint32_t) avail);
            }
        }
    }
    // start of a unit: offset of this lane's first word; the caller commits, waits and then calls first_words()
    __device__ __forceinline__ void open(const uint8_t * unit_base, uint32_t first, uint32_t ring_key, const Opaque & k) {
        base = unit_base; key = ring_key;
        fetched = first & ~15u;
        next = first;
        top_up<7>(k);
    }
    __device__ __forceinline__ void first_words() {
        hi = lds32(ring_addr(next, key), token);
        ahead = lds32(ring_addr(next + 4, key), token);
        next += 8; lo = 0; v = 32; t = 0;
    }
    __device__ __forceinline__ void take2(uint32_t lut, const Opaque & k, uint32_t & e0, uint32_t & e1) {
        v = imad(t, k.minus_one, v);
        const uint32_t place = __funnelshift_r(0u, 1u, v);
        if (!(v & 32u)) {
            uint64_t b;
            asm("mov.b64 %0, {%1, %2};" : "=l"(b) : "r"(lo), "r"(hi));
            asm("mad.wide.u32 %0, %1, %2, %0;" : "+l"(b) : "r"(ahead), "r"(place));
            asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(b));
            ahead = lds32(ring_addr(next, key), token);
            next = imad(k.four, k.one, next);
            v = imad(k.thirty_two, k.one, v);
        }
        e0 = lds32_ro(imad(hi >> (32 - HP_LMAX), k.four, lut));
        const uint32_t second = shl_wrap_hi(lo, hi, e0);
        e1 = lds32_ro(imad(second >> (32 - HP_LMAX), k.four, lut));
        t = imad(e0, k.one, e1);
        hi = shl_wrap_hi(lo, hi, t);
        lo = shl_wrap_hi(0u, lo, t);
    }
};

__device__ __forceinline__ void fma_bf16x2(uint32_t w, uint32_t x, float & lo, float & hi) {
    asm("{ .reg .b16 wl, wh, xl, xh;\n\t"
        "mov.b32 {wl, wh}, %2;\n\t"
        "mov.b32 {xl, xh}, %3;\n\t"
        "fma.rn.f32.bf16 %0, wl, xl, %0;\n\t"
        "fma.rn.f32.bf16 %1, wh, xh, %1; }"
        : "+f"(lo), "+f"(hi) : "r"(w), "r"(x));
}
__device__ __forceinline__ uint2 lds64_ro(uint32_t addr) {
    uint2 v;
    asm("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}

// One unit per warp, as many warps as the register file allows: the activations live in shared memory (BF16, natural
// order: lane l's four activations of column quad j of chunk c are the 8 bytes at ((c*4 + j)*32 + l)*8, so every read
// is base + immediate and conflict-free) and the plane is prefetched one row ahead chunk by chunk.
template <int C, int NT, bool PEERS = false> // PEERS: the output also goes to the other GPUs (a separate instantiation: the plain kernel carries none of it)
__global__ void __launch_bounds__(NT, 1) k_pair_gemv_rings(const PairView w, int R, Cols p, const Opaque k) {
    constexpr int K = C * CHUNK;
    extern __shared__ __align__(128) unsigned char smem[];
    uint32_t * lut = (uint32_t *) smem; // 16 KB table | K BF16 activations | one 4 KB ring set per warp
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    const uint32_t lut_s = smem_u32(lut);
    const uint32_t xs = lut_s + 4 * HP_MAX_PAIRS + lane * 8;
    // ring of lane l: 128 bytes at l * 128; granule index XOR (l & 7) spreads lanes that read in step over the banks
    const uint32_t key = (lut_s + 4 * HP_MAX_PAIRS + 2 * K + (uint32_t) warp * (32 * RING_BYTES) + lane * RING_BYTES) | ((lane & 7) << 4);

    const bf16 * xg; OutVec out; int64_t rbase;
    column<bf16>(p, blockIdx.y, xg, out, rbase);
    for (int i = threadIdx.x; i < HP_MAX_PAIRS / 4; i += blockDim.x) { ((uint4 *) lut)[i] = __ldg((const uint4 *) w.lut + i); }
    for (int i = threadIdx.x; i < K / 8; i += blockDim.x) { ((uint4 *) (smem + 4 * HP_MAX_PAIRS))[i] = __ldg((const uint4 *) xg + i); }
    __syncthreads();

    const int64_t units = p.nrows / R;
    for (int64_t u = (int64_t) blockIdx.x * nwarp + warp; u < units; u += (int64_t) gridDim.x * nwarp) {
        const int64_t g = rbase / R + u;
        RingReader rd;
        {
            const uint32_t w0 = __ldg(w.ubase + g), l0 = __ldg(w.lrel + g * 32 + lane);
            rd.open((const uint8_t *) (w.stream + (w0 & ~3u)), ((w0 & 3u) + l0) * 4u, key, k);
        }
        cp_async_commit();
        const uint8_t * pl = w.plane + g * R * K + 16 * lane;
        uint4 nx[C];
#pragma unroll
        for (int c = 0; c < C; c++) { nx[c] = ld_stream16(pl + c * CHUNK); }
        rd.token = cp_async_wait_all();
        rd.first_words();
        float mine = 0.f;
        for (int rr = 0; rr < R; rr++) {
            if (rr) {
                rd.token = cp_async_wait_all(); // copies issued one row ago
                rd.template top_up<3>(k);
                cp_async_commit();
            }
            float a[4] = {0.f, 0.f, 0.f, 0.f};
            const uint8_t * nrow = pl + (rr + 1 < R ? rr + 1 : rr) * K;
#pragma unroll
            for (int c = 0; c < C; c++) {
                const uint4 sm = nx[c];
                nx[c] = ld_stream16(nrow + c * CHUNK); // the last row re-reads itself: one harmless L2 hit per chunk
                const uint32_t pw[4] = {sm.x, sm.y, sm.z, sm.w};
#pragma unroll
                for (int half = 0; half < 2; half++) {
                    uint32_t e[4];
                    rd.take2(lut_s, k, e[0], e[1]);
                    rd.take2(lut_s, k, e[2], e[3]);
#pragma unroll
                    for (int jj = 0; jj < 2; jj++) {
                        const int j = 2 * half + jj;
                        const uint2 xq = lds64_ro(xs + (c * 4 + j) * 256);
                        fma_bf16x2(merge_sm_exp(spread_lo(pw[j]), e[2 * jj]), xq.x, a[0], a[1]);
                        fma_bf16x2(merge_sm_exp(spread_hi(pw[j]), e[2 * jj + 1]), xq.y, a[2], a[3]);
                    }
                }
            }
            const float s = warp_sum((a[0] + a[1]) + (a[2] + a[3]));
            if (lane == rr) { mine = s; }
        }
        if (lane < R) {
            out.put(u * R + lane, mine);
            if (PEERS) { peers_put(p, blockIdx.y, u * R + lane, mine); }
        }
    }
    if (PEERS) { peers_done(p); }
}

constexpr int RING_SET = 32 * RING_BYTES;
int fixed_smem(int64_t K) { return 4 * HP_MAX_PAIRS + 2 * (int) K; }

} // namespace

static int g_warps = 28; // most warps per block; BF16N_RINGS_WARPS overrides it (0: off, the bulk-copy kernel takes over)

void gemv_rings_init() {
    const int optin = device_info().smem_optin;
#define ATTR(KERNEL) cuda_ok(cudaFuncSetAttribute(KERNEL, cudaFuncAttributeMaxDynamicSharedMemorySize, optin), #KERNEL)
    ATTR((k_pair_gemv_rings<1, 896>)); ATTR((k_pair_gemv_rings<2, 896>)); ATTR((k_pair_gemv_rings<4, 896>));
    ATTR((k_pair_gemv_rings<4, 768>)); ATTR((k_pair_gemv_rings<4, 1024>));
    ATTR((k_pair_gemv_rings<1, 896, true>)); ATTR((k_pair_gemv_rings<2, 896, true>)); ATTR((k_pair_gemv_rings<4, 896, true>));
    ATTR((k_pair_gemv_rings<4, 768, true>)); ATTR((k_pair_gemv_rings<4, 1024, true>));
#undef ATTR
    if (const char * e = getenv("BF16N_RINGS_WARPS")) { g_warps = atoi(e); }
}

bool gemv_rings_enabled() { return g_warps > 0; }

// Row-major HUFPAIR, BF16 activations, K <= 2048, enough units to give every SM a full set of chains
bool gemv_rings_applies(const bf16n_weight & w, const bf16n_mmv_args & a) {
    const int64_t C = w.K / CHUNK;
    if (w.format != FMT_HUFPAIR || w.cm || w.fo || !(C == 1 || C == 2 || C == 4) || a.nrows <= 0 || !a.x_bf16) { return false; }
    return a.nrows / w.R >= (int64_t) device_info().sms * 16 * std::max(1, a.ncols);
}

void gemv_rings(const bf16n_weight & w, const bf16n_mmv_args & a, cudaStream_t st, const bf16n_peer_out * peers) {
    const Cols p = make_cols(a, peers);
    const int64_t units = a.nrows / w.R, sms = device_info().sms;
    const int max_warps = std::min(g_warps, w.K == 2048 ? 32 : 28);
    int best = max_warps;
    double best_eff = 0.0;
    for (int nw = max_warps; nw >= max_warps - 3; nw--) { // static round-robin: waste least of the last round
        const int64_t slots = sms * nw, rounds = (units + slots - 1) / slots;
        const double eff = (double) units / (double) (rounds * slots) * (1.0 - 0.01 * (max_warps - nw));
        if (eff > best_eff + 1e-9) { best_eff = eff; best = nw; }
    }
    const dim3 grid((unsigned) sms, (unsigned) a.ncols);
    const size_t shm = fixed_smem(w.K) + (size_t) best * RING_SET;
    const Opaque k = {1u, 4u, ~0u, 32u, 16u};
    const PairView v = pair_view(w);
#define GO(CC, NT) if (p.peers.n) { k_pair_gemv_rings<CC, NT, true><<<grid, best * 32, shm, st>>>(v, w.R, p, k); } \
                   else { k_pair_gemv_rings<CC, NT, false><<<grid, best * 32, shm, st>>>(v, w.R, p, k); }
    if (w.K == 2048 && best > 28) { GO(4, 1024); }
    else if (w.K == 2048 && best <= 24) { GO(4, 768); }
    else { switch (w.K / CHUNK) { case 1: GO(1, 896); break; case 2: GO(2, 896); break; default: GO(4, 896); break; } }
#undef GO
    check_launch();
}

} // namespace b16
