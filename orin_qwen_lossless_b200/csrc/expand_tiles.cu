// First pass of the two-pass batched (prefill) product: decode whole expert matrices, at full occupancy, into BF16
// operand tiles that the tensor-core pass (k_tile_mm in prefill.cu) copies into shared memory with one bulk copy each.
//
// The fused prefill kernel decodes inside the block that multiplies; its 16 decoder warps per SM are register-bound and
// their dependent table lookups set the pace of the layer. Here one unit per warp and 28 warps per SM decode with the
// ring reader of the large-matrix GEMV (per-lane cp.async rings, window reader, four interleaved table copies), and
// what they write is already the shared-memory image of the B operand:
//
//   image of (expert e, row block nb) = [K / 64 k-tiles][256 rows][128 bytes], K-major, 128-byte swizzled
//   (16-byte piece p of row r is stored at piece p ^ (r & 7)); a k-tile of a row block is 32 KB, contiguous.
//
// Row block of a plain matrix: its rows 256 nb .. 256 nb + 255. Row block of a gate/up pair (SwiGLU): gate rows
// 128 nb .. 128 nb + 127 as image rows 0..127 and the same rows of up as image rows 128..255, so that the thread that
// reads a token's accumulators holds gate and up of the same output.
//
// A lane's 4 consecutive weights (lane-major chunk: column 128 j + 4 l + {0..3} of quad j) are one 8-byte store; the 32
// lanes of a store instruction fill two whole 128-byte lines (k-tiles 2 j and 2 j + 1 of the chunk). Both unit layouts
// are one linear walk over (row, chunk) steps of 512 weights: row-major units step chunks fastest, chunk-major units
// rows fastest; the plane and the streams are in step order either way.
#include "launch.h"
#include "rings.cuh"

namespace b16 {
namespace {

using namespace dev;
using namespace ring;

constexpr int EXPAND_WARPS = 28;              // 72 registers per thread: four steps of plane bytes in flight per lane
constexpr int AHEAD = 4;                     // plane bytes are loaded this many steps (of 512 weights) before they are decoded
constexpr int IMG_ROWS = 256;                 // rows of a row block = N of the tensor-core pass
constexpr int IMG_KTILE_BYTES = IMG_ROWS * 128;

struct ExpandArgs {
    PairView w[2];               // [1]: the up matrix of a gate/up pair (blockIdx.y picks the matrix)
    unsigned char * images;      // row-block images of the experts (see the layout above)
    const int32_t * bounds;      // per expert: first routed pair (n_experts + 1 entries); experts without pairs are skipped; may be null
    int64_t units;               // units of the whole (expert-stacked) matrix
    int rows_per_expert;
    int rows_per_block;          // 256 (plain) or 128 (one half of a gate/up pair; the up half fills image rows 128..255)
    int blocks_per_expert;
};

template <int C, int R, bool CM>
__global__ void __launch_bounds__(EXPAND_WARPS * 32, 1) k_expand_tiles(const ExpandArgs p, const Opaque k) {
    constexpr int K = C * CHUNK, STEPS = R * C, KT = K / 64;
    static_assert(AHEAD == 4 && STEPS % AHEAD == 0, "the rings are topped up every four steps (32 codes), which is also the plane read-ahead");
    extern __shared__ __align__(128) unsigned char smem[];
    uint32_t * lut = (uint32_t *) smem; // four interleaved tables | one 4 KB ring set per warp
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    const uint32_t lut_s = smem_u32(lut);
    const uint32_t lut_l = lut_s + (lane & 3) * 4;
    const uint32_t key = (lut_s + LUT_BYTES + (uint32_t) warp * (32 * RING_BYTES) + lane * RING_BYTES) | ((lane & 7) << 4);
    const PairView w = blockIdx.y ? p.w[1] : p.w[0];
    const int row_offset = blockIdx.y ? IMG_ROWS / 2 : 0;
    for (int i = threadIdx.x; i < HP_MAX_PAIRS; i += blockDim.x) { const uint32_t e = __ldg(w.lut + i); ((uint4 *) lut)[i] = make_uint4(e, e, e, e); }
    __syncthreads();

    const uint32_t piece = (uint32_t) (lane & 15) >> 1;
    const uint32_t lane_part = (uint32_t) (lane >> 4) * IMG_KTILE_BYTES + (uint32_t) (lane & 1) * 8;
    for (int64_t u = (int64_t) blockIdx.x * nwarp + warp; u < p.units; u += (int64_t) gridDim.x * nwarp) {
        const int64_t row0 = u * R;
        const int e = (int) (row0 / p.rows_per_expert), ri = (int) (row0 - (int64_t) e * p.rows_per_expert);
        if (p.bounds && __ldg(p.bounds + e + 1) == __ldg(p.bounds + e)) { continue; }
        const int nb = ri / p.rows_per_block, img_row0 = ri - nb * p.rows_per_block + row_offset;
        unsigned char * img = p.images + ((int64_t) e * p.blocks_per_expert + nb) * ((int64_t) KT * IMG_KTILE_BYTES) + lane_part;
        RingReader rd;
        {
            const uint32_t w0 = __ldg(w.ubase + u), l0 = __ldg(w.lrel + u * 32 + lane);
            rd.open((const uint8_t *) (w.stream + (w0 & ~3u)), ((w0 & 3u) + l0) * 4u, key, k);
        }
        cp_async_commit();
        const uint8_t * pl = w.plane + u * R * K + 16 * lane;
        // Plane bytes AHEAD steps ahead of the decode: with every SM writing tiles at the same time a load takes several
        // microseconds, more than one step of decoding hides.
        uint4 nx[AHEAD];
#pragma unroll
        for (int i = 0; i < AHEAD; i++) { nx[i] = ld_stream16(pl + i * CHUNK); }
        rd.token = cp_async_wait_all();
        rd.first_words();
#pragma unroll 1
        for (int t0 = 0; t0 < STEPS; t0 += AHEAD) {
            if (t0) {
                rd.token = cp_async_wait_all(); // copies issued four steps ago
                rd.template top_up<3>(k);
                cp_async_commit();
            }
#pragma unroll
            for (int i = 0; i < AHEAD; i++) {
                const int t = t0 + i;
                const int rr = CM ? t % R : t / C, c = CM ? t / R : t % C;
                const uint4 sm = nx[i];
                nx[i] = ld_stream16(pl + (t + AHEAD < STEPS ? t + AHEAD : t) * CHUNK); // the last steps re-read themselves: harmless L2 hits
                const uint32_t pw[4] = {sm.x, sm.y, sm.z, sm.w};
                const uint32_t row = (uint32_t) (img_row0 + rr);
                unsigned char * rp = img + (size_t) c * 8 * IMG_KTILE_BYTES + row * 128 + ((piece ^ (row & 7)) << 4);
#pragma unroll
                for (int half = 0; half < 2; half++) {
                    uint32_t en[4];
                    rd.take2(lut_l, k, en[0], en[1]);
                    rd.take2(lut_l, k, en[2], en[3]);
#pragma unroll
                    for (int jj = 0; jj < 2; jj++) { // quad 2 half + jj of the chunk: k-tiles 2 (2 half + jj) and the next one
                        const uint32_t lo = merge_sm_exp(spread_lo(pw[2 * half + jj]), en[2 * jj]);
                        const uint32_t hi = merge_sm_exp(spread_hi(pw[2 * half + jj]), en[2 * jj + 1]);
                        *(uint2 *) (rp + (size_t) (2 * (2 * half + jj)) * IMG_KTILE_BYTES) = make_uint2(lo, hi);
                    }
                }
            }
        }
    }
}

constexpr size_t EXPAND_SMEM = LUT_BYTES + (size_t) EXPAND_WARPS * 32 * RING_BYTES;

} // namespace

void expand_tiles_init() {
    const int optin = device_info().smem_optin;
    allow_dynamic_smem((const void *) k_expand_tiles<4, 8, true>, (int) EXPAND_SMEM, optin, "expand tiles");
    allow_dynamic_smem((const void *) k_expand_tiles<1, 16, false>, (int) EXPAND_SMEM, optin, "expand tiles");
}

bool expand_tiles_supported(const bf16n_weight & w) {
    const int C = (int) (w.K / CHUNK);
    return w.format == FMT_HUFPAIR && !w.fo && w.K % CHUNK == 0 && ((C == 4 && w.R == 8 && w.cm) || (C == 1 && w.R == 16));
}

// Decodes every expert of `w` (and of `up`, the second matrix of a gate/up pair, in the same launch) that has routed
// pairs into its row-block images: 256-row blocks of a plain matrix, 128 + 128 rows of a pair.
void expand_tiles(const bf16n_weight & w, const bf16n_weight * up, int n_experts, const int32_t * bounds, void * images, cudaStream_t st) {
    ExpandArgs a = {};
    a.w[0] = pair_view(w);
    a.w[1] = up ? pair_view(*up) : a.w[0];
    a.images = (unsigned char *) images;
    a.bounds = bounds;
    a.units = w.rows / w.R;
    a.rows_per_expert = (int) (w.rows / n_experts);
    a.rows_per_block = up ? IMG_ROWS / 2 : IMG_ROWS;
    a.blocks_per_expert = a.rows_per_expert / a.rows_per_block;
    require(a.rows_per_expert % a.rows_per_block == 0, "rows per expert must be a multiple of the tensor-core pass's row block");
    const int n_mats = up ? 2 : 1;
    const unsigned gx = (unsigned) std::min<int64_t>(std::max(1, device_info().sms / n_mats), (a.units + EXPAND_WARPS - 1) / EXPAND_WARPS);
    const dim3 grid(gx, (unsigned) n_mats);
    const Opaque k = {1u, 4u, ~0u, 32u, 16u};
    if (w.K == 4 * CHUNK) { k_expand_tiles<4, 8, true><<<grid, EXPAND_WARPS * 32, EXPAND_SMEM, st>>>(a, k); }
    else { k_expand_tiles<1, 16, false><<<grid, EXPAND_WARPS * 32, EXPAND_SMEM, st>>>(a, k); }
    check_launch();
}

} // namespace b16
