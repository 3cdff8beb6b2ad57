// Expert-parallel prefill without the host in the loop (new: the reference is single-GPU). Tokens are split over the
// ranks of a node and every rank holds a slice of the experts. A routed (token, slot) row travels to the rank that
// owns its expert, is multiplied there by the batched kernels and its result travels back. All of it is device work on
// one stream, so a layer can be captured in a CUDA graph: no exchange of sizes through the host, no collective.
//
// Every rank owns one exchange buffer (bf16n_exchange_create) with the same layout, mapped into its peers:
//   counts  int32 [ranks]             rows source s sent to this rank in the current layer
//   expert  int32 [ranks][cap]        local expert id of each received row
//   pair    int32 [ranks][cap]        index of the row's (token, slot) pair at its source
//   rows    bf16  [ranks][cap][K]     the received activation rows
//   back    fp32  [pairs][H]          results of this rank's own pairs, stored by the owners (row = pair index)
// plan:      per pair its position among the pairs this rank sends to the same owner (by pair index, so the order is
//            deterministic), and the counts per owner
// dispatch:  a warp per pair copies the 2 K bytes of its activation row into the owner's `rows` with 16-byte peer stores
//            and writes expert and pair; the launch ends like every fan-out kernel (decode.cuh: each block fences, the last
//            one publishes an epoch in the peers' headers and, with a wait mask, waits for theirs)
// expert ids: slots beyond a source's count read as "no expert", so the routing sort and the batched kernels of the
//            single-GPU path run unchanged over the fixed-size inbox
// give back: a warp per received row stores its 4 H result bytes into the source's `back` at the pair's index.
// Plain peer stores over NVLink; no multicast, no TMA from peer memory.
#include "decode.cuh"
#include "launch.h"

namespace b16 {
namespace {

using namespace dev;

struct EpView { // one rank's view of every exchange buffer of the node (device pointers; own buffer included at [rank])
    int n_ranks, rank, cap, K, H, n_pairs_max;
    char * base[8];
    size_t off_counts, off_expert, off_pair, off_rows, off_back;
};

__device__ __forceinline__ int32_t * ep_counts(const EpView & v, int r) { return (int32_t *) (v.base[r] + v.off_counts); }
__device__ __forceinline__ int32_t * ep_expert(const EpView & v, int r, int src) { return (int32_t *) (v.base[r] + v.off_expert) + (int64_t) src * v.cap; }
__device__ __forceinline__ int32_t * ep_pair(const EpView & v, int r, int src) { return (int32_t *) (v.base[r] + v.off_pair) + (int64_t) src * v.cap; }
__device__ __forceinline__ char * ep_rows(const EpView & v, int r, int src) { return v.base[r] + v.off_rows + (int64_t) src * v.cap * v.K * 2; }
__device__ __forceinline__ float * ep_back(const EpView & v, int r) { return (float *) (v.base[r] + v.off_back); }

// One block. pos[j] = number of pairs i < j with the same owner; counts[w] = pairs owned by rank w.
__global__ void __launch_bounds__(1024) k_ep_plan(const int32_t * __restrict__ ids, int n_pairs, int n_local, int n_ranks,
                                                  int32_t * __restrict__ pos, int32_t * __restrict__ counts) {
    __shared__ int warp_tot[8][32];
    __shared__ int running[8];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    grid_dependency_wait();
    if (tid < 8) { running[tid] = 0; }
    __syncthreads();
    for (int c0 = 0; c0 < n_pairs; c0 += 1024) {
        const int j = c0 + tid;
        const int owner = j < n_pairs ? ids[j] / n_local : -1;
        int before = 0; // pairs of my owner in lower lanes of my warp
        for (int w = 0; w < n_ranks; w++) {
            const unsigned m = __ballot_sync(FULL, owner == w);
            if (owner == w) { before = __popc(m & ((1u << lane) - 1u)); }
            if (lane == 0) { warp_tot[w][warp] = __popc(m); }
        }
        __syncthreads();
        if (owner >= 0) {
            int p = running[owner] + before;
            for (int i = 0; i < warp; i++) { p += warp_tot[owner][i]; }
            pos[j] = p;
        }
        __syncthreads();
        if (tid < n_ranks) {
            int t = 0;
            for (int i = 0; i < 32; i++) { t += warp_tot[tid][i]; }
            running[tid] += t;
        }
        __syncthreads();
    }
    if (tid < n_ranks) { counts[tid] = running[tid]; }
}

__device__ __forceinline__ void st16(void * p, const uint4 & v) {
    asm volatile("st.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 ld16_cg(const void * p) {
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ int32_t ld32_cg(const int32_t * p) {
    int32_t v;
    asm volatile("ld.global.cg.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// x [n_tok, K] BF16 (row stride x_row bytes), ids [n_pairs] = [n_tok, n_used] flattened
__global__ void __launch_bounds__(256) k_ep_dispatch(const EpView v, const char * __restrict__ x, int64_t x_row, const int32_t * __restrict__ ids,
                                                     int n_pairs, int n_used, int n_local, const int32_t * __restrict__ pos,
                                                     const int32_t * __restrict__ counts, const PeerOut peers) {
    grid_dependency_wait();
    peers_begin(peers);
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    for (int j = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; j < n_pairs; j += warps) {
        const int e = ids[j], owner = e / n_local, p = pos[j];
        const uint4 * src = (const uint4 *) (x + (int64_t) (j / n_used) * x_row);
        uint4 * dst = (uint4 *) (ep_rows(v, owner, v.rank) + (int64_t) p * v.K * 2);
        for (int i = lane; i < v.K / 8; i += 32) { st16(dst + i, __ldg(src + i)); }
        if (lane == 0) {
            ep_expert(v, owner, v.rank)[p] = e - owner * n_local;
            ep_pair(v, owner, v.rank)[p] = j;
        }
    }
    if (blockIdx.x == 0 && threadIdx.x < v.n_ranks) { ep_counts(v, threadIdx.x)[v.rank] = counts[threadIdx.x]; }
    peers_done(peers);
}

// ids_out [n_ranks * cap]: the local expert of every inbox slot, 0x7fffffff (no expert) beyond a source's count
__global__ void __launch_bounds__(256) k_ep_inbox_ids(const EpView v, int32_t * __restrict__ ids_out) {
    grid_dependency_wait();
    const int64_t n = (int64_t) v.n_ranks * v.cap;
    for (int64_t i = blockIdx.x * (int64_t) blockDim.x + threadIdx.x; i < n; i += (int64_t) gridDim.x * blockDim.x) {
        const int src = (int) (i / v.cap), p = (int) (i - (int64_t) src * v.cap);
        const int cnt = ld32_cg(ep_counts(v, v.rank) + src);
        ids_out[i] = p < cnt ? ld32_cg(ep_expert(v, v.rank, src) + p) : 0x7fffffff;
    }
}

// ys [n_ranks * cap, H] FP32: row of inbox slot (src, p) goes to rank src's `back` at the pair's index
__global__ void __launch_bounds__(256) k_ep_give_back(const EpView v, const float * __restrict__ ys, const PeerOut peers) {
    grid_dependency_wait();
    peers_begin(peers);
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    const int64_t n = (int64_t) v.n_ranks * v.cap;
    for (int64_t i = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; i < n; i += warps) {
        const int src = (int) (i / v.cap), p = (int) (i - (int64_t) src * v.cap);
        if (p >= ld32_cg(ep_counts(v, v.rank) + src)) { continue; }
        const int j = ld32_cg(ep_pair(v, v.rank, src) + p);
        const uint4 * from = (const uint4 *) (ys + i * v.H);
        uint4 * to = (uint4 *) (ep_back(v, src) + (int64_t) j * v.H);
        for (int q = lane; q < v.H / 4; q += 32) { st16(to + q, ld16_cg(from + q)); }
    }
    peers_done(peers);
}

EpView view_of(const bf16n_ep_layout & l) {
    EpView v = {};
    v.n_ranks = l.n_ranks; v.rank = l.rank; v.cap = l.cap; v.K = l.K; v.H = l.H; v.n_pairs_max = l.n_pairs_max;
    for (int r = 0; r < l.n_ranks; r++) { v.base[r] = (char *) l.base[r] + BF16N_EXCHANGE_HEADER_BYTES; }
    v.off_counts = l.off_counts; v.off_expert = l.off_expert; v.off_pair = l.off_pair; v.off_rows = l.off_rows; v.off_back = l.off_back;
    return v;
}

PeerOut peers_of(const bf16n_ep_layout & l, bool wait) {
    PeerOut o = {};
    for (int r = 0; r < l.n_ranks; r++) {
        if (r == l.rank) { continue; }
        o.y[o.n] = nullptr;
        o.flag[o.n] = (uint32_t *) l.base[r] + l.rank;
        o.n++;
        if (wait) { o.wait_mask |= 1 << r; }
    }
    o.hdr = (uint32_t *) l.base[l.rank];
    o.wait_ns = peer_wait_limit_ns();
    return o;
}

void check_layout(const bf16n_ep_layout & l) {
    require(l.n_ranks >= 1 && l.n_ranks <= 8 && l.rank >= 0 && l.rank < l.n_ranks, "ep: 1..8 ranks");
    require(l.cap > 0 && l.K > 0 && l.K % 8 == 0 && l.H > 0 && l.H % 4 == 0 && l.n_pairs_max > 0, "ep: bad sizes");
    for (int r = 0; r < l.n_ranks; r++) { require(l.base[r] != nullptr, "ep: null exchange buffer"); }
    require((l.off_counts | l.off_expert | l.off_pair | l.off_rows | l.off_back) % 16 == 0, "ep: offsets must be 16-byte aligned");
}

} // namespace

size_t ep_layout_fill(bf16n_ep_layout & l) { // offsets of the payload areas; returns the payload bytes
    auto up = [](size_t n) { return (n + 255) / 256 * 256; };
    size_t o = 0;
    l.off_counts = o; o += up(4 * 8);
    l.off_expert = o; o += up((size_t) 4 * l.n_ranks * l.cap);
    l.off_pair = o; o += up((size_t) 4 * l.n_ranks * l.cap);
    l.off_rows = o; o += up((size_t) 2 * l.n_ranks * l.cap * l.K);
    l.off_back = o; o += up((size_t) 4 * l.n_pairs_max * l.H);
    return o;
}

void ep_dispatch(const bf16n_ep_layout & l, const void * x_bf16, int64_t x_row, const int32_t * ids, int n_tok, int n_used, int n_experts,
                 int32_t * plan, cudaStream_t st) {
    check_layout(l);
    const int n_pairs = n_tok * n_used;
    require(n_pairs > 0 && n_pairs <= l.n_pairs_max && n_pairs <= l.cap, "ep_dispatch: more pairs than the exchange buffers hold");
    require(n_experts % l.n_ranks == 0, "ep_dispatch: experts must split evenly over the ranks");
    require((uintptr_t) x_bf16 % 16 == 0 && x_row % 16 == 0, "ep_dispatch: x and its row stride must be 16-byte aligned");
    const int n_local = n_experts / l.n_ranks;
    int32_t * pos = plan, * counts = plan + n_pairs;
    launch_chained(k_ep_plan, dim3(1), dim3(1024), 0, st, ids, n_pairs, n_local, l.n_ranks, pos, counts);
    const unsigned blocks = (unsigned) std::min<int64_t>((n_pairs + 7) / 8, (int64_t) device_info().sms * 4);
    launch_chained(k_ep_dispatch, dim3(blocks), dim3(256), 0, st, view_of(l), (const char *) x_bf16, x_row, ids, n_pairs, n_used, n_local,
                   (const int32_t *) pos, (const int32_t *) counts, peers_of(l, true));
    check_launch();
}

void ep_inbox_ids(const bf16n_ep_layout & l, int32_t * ids_out, cudaStream_t st) {
    check_layout(l);
    const int64_t n = (int64_t) l.n_ranks * l.cap;
    launch_chained(k_ep_inbox_ids, dim3((unsigned) std::min<int64_t>((n + 255) / 256, (int64_t) device_info().sms * 4)), dim3(256), 0, st,
                   view_of(l), ids_out);
    check_launch();
}

void ep_give_back(const bf16n_ep_layout & l, const float * ys, cudaStream_t st) {
    check_layout(l);
    require((uintptr_t) ys % 16 == 0, "ep_give_back: ys must be 16-byte aligned");
    const int64_t n = (int64_t) l.n_ranks * l.cap;
    launch_chained(k_ep_give_back, dim3((unsigned) std::min<int64_t>((n + 7) / 8, (int64_t) device_info().sms * 4)), dim3(256), 0, st,
                   view_of(l), ys, peers_of(l, true));
    check_launch();
}

} // namespace b16
