// The C ABI (include/bf16n_c.h): argument validation with the reference's rules and messages
// (core/src/launch.cu:261-268, 313-365, 367-376, 404-413, 458-490), error translation, one-time initialisation.
#include "encode.h"
#include "launch.h"
#include "policy.h"

#include <atomic>
#include <cstring>
#include <mutex>

namespace b16 {
namespace {

thread_local std::string g_error;
DeviceInfo g_info;
std::once_flag g_once;
int g_init_status = BF16N_OK;
std::string g_init_error;
int g_device = -1;                         // the device bf16n_init ran on: the only one this process may launch on
unsigned int * g_fault_words[4] = {};      // bit i of bf16n_fault_status: gemv_staged, moe_decode, fragment order, prefill
std::atomic<uint64_t> g_peer_wait_ns{2000000000ull};

template <typename F>
int guarded(F && f) {
    try {
        f();
        return BF16N_OK;
    } catch (const std::invalid_argument & e) {
        g_error = e.what();
        return BF16N_EINVAL;
    } catch (const std::runtime_error & e) {
        g_error = e.what();
        return std::strstr(e.what(), "CUDA error") ? BF16N_ECUDA : BF16N_EINTERNAL;
    } catch (const std::exception & e) {
        g_error = e.what();
        return BF16N_EINTERNAL;
    }
}

void ensure_init() {
    std::call_once(g_once, [] {
        try {
            int dev = 0;
            cuda_ok(cudaGetDevice(&dev), "cudaGetDevice");
            g_device = dev;
            cuda_ok(cudaDeviceGetAttribute(&g_info.sms, cudaDevAttrMultiProcessorCount, dev), "SM count");
            cuda_ok(cudaDeviceGetAttribute(&g_info.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev), "shared memory limit");
            gemv_init();
            moe_init();
            moe_decode_init();
            prefill_init();
            fo_init();
            g_fault_words[0] = gemv_staged_fault_word();
            g_fault_words[1] = moe_decode_fault_word();
            g_fault_words[2] = fo_fault_word();
            g_fault_words[3] = prefill_fault_word();
        } catch (const std::exception & e) {
            g_init_status = BF16N_ECUDA;
            g_init_error = e.what();
        }
    });
    if (g_init_status != BF16N_OK) { throw std::runtime_error(g_init_error); }
    // The kernels' shared-memory limits, the SM count the grids are sized from and the fault words belong to the device
    // that was current at the first call: one process drives one GPU, and a launch from another device is refused.
    int dev = -1;
    cuda_ok(cudaGetDevice(&dev), "cudaGetDevice");
    if (dev != g_device) {
        fail_invalid("this process initialised device " + std::to_string(g_device) + " and the current device is " +
                     std::to_string(dev) + ": one device per process");
    }
}

void check_weight(const bf16n_weight & w) {
    require(w.K % CHUNK == 0 && w.K >= CHUNK && w.K <= K_MAX, "K must be a multiple of 512 in [512, 4096]");
    require(w.format == FMT_NIBBLE || w.format == FMT_HUFFMAN || w.format == FMT_HUFPAIR, "unknown format");
    require(w.format == FMT_NIBBLE || (w.R > 0 && w.rows % w.R == 0), "rows must be a multiple of R");
    require(!w.cm || w.format == FMT_HUFPAIR, "chunk-major units exist only for HUFPAIR");
    require(!w.fo || (w.format == FMT_HUFPAIR && !w.cm && w.R == 16),
            "fragment order exists only for HUFPAIR with R = 16, without chunk-major units");
    require(((uintptr_t) w.plane | (uintptr_t) w.aux) % 16 == 0, "plane and aux must be 16-byte aligned");
}
void no_frag_order(const bf16n_weight & w) {
    require(!w.fo, "this operation has no kernel for fragment-order matrices");
}
// fragment-order matrices go to their own kernels (fo.cu): true when w is one (and checks that they can take it)
bool frag_order(const bf16n_weight & w) {
    if (!w.fo) { return false; }
    require(fo_supported(w), "fragment order: HUFPAIR bands of 16 rows with K up to 4096");
    return true;
}
void whole_units(const bf16n_weight & w, const bf16n_mmv_args & a) {
    require(w.format == FMT_NIBBLE || (a.nrows % w.R == 0 && a.row0 % w.R == 0 && a.rows_per_matrix % w.R == 0),
            "rows of a product must be whole units");
}
void check_x(const bf16n_weight & w, const bf16n_mmv_args & a) {
    // vector loads: 16 bytes for FP32 activations, 8 for BF16 (the kernels read 4 activations at a time)
    const uintptr_t al = a.x_bf16 ? 8 : 16;
    require((uintptr_t) a.x % al == 0 && a.x_tok % (int64_t) al == 0 && a.x_slot % (int64_t) al == 0,
            "activation base and strides must be 16-byte aligned (8 for BF16)");
    (void) w;
}

} // namespace

const DeviceInfo & device_info() { return g_info; }
void set_last_error(const std::string & message) { g_error = message; }
namespace dev { uint64_t peer_wait_limit_ns() { return g_peer_wait_ns.load(std::memory_order_relaxed); } }

} // namespace b16

using namespace b16;

struct bf16n_encoded { Encoded e; };

extern "C" {

const char * bf16n_last_error(void) { return g_error.c_str(); }

int bf16n_encode(const uint16_t * w, int64_t rows, int64_t K, int format, int R, int chunk_major, int frag_order,
                 bf16n_encoded ** out) {
    return guarded([&] {
        require(w != nullptr && out != nullptr, "encode: null argument");
        auto * r = new bf16n_encoded;
        try {
            r->e = encode(w, rows, K, format, R, chunk_major != 0, frag_order != 0);
        } catch (...) {
            delete r;
            throw;
        }
        *out = r;
    });
}
const uint8_t * bf16n_encoded_plane(const bf16n_encoded * e, size_t * n) { if (n) { *n = e->e.plane.size(); } return e->e.plane.data(); }
const uint8_t * bf16n_encoded_aux(const bf16n_encoded * e, size_t * n) { if (n) { *n = e->e.aux.size(); } return e->e.aux.data(); }
int bf16n_encoded_format(const bf16n_encoded * e) { return e->e.format; }
int bf16n_encoded_R(const bf16n_encoded * e) { return e->e.R; }
void bf16n_encoded_free(bf16n_encoded * e) { delete e; }

int bf16n_parse_header(const uint8_t * aux_host, size_t nbytes, bf16n_weight * w) {
    return guarded([&] {
        require(aux_host && w && nbytes >= (size_t) HEADER_BYTES, "aux must hold at least the 256-byte header");
        AuxHeader h;
        memcpy(&h, aux_host, sizeof h);
        require(h.magic == MAGIC, "bad aux header (magic)");
        require(h.format == (uint32_t) FMT_NIBBLE || h.format == (uint32_t) FMT_HUFFMAN || h.format == (uint32_t) FMT_HUFPAIR,
                "bad aux header (format)");
        require((h.flags & ~(FLAG_CHUNK_MAJOR | FLAG_FRAG_ORDER)) == 0, "unknown layout flags");
        w->format = (int32_t) h.format; w->R = (int32_t) h.R; w->K = h.K; w->rows = (int64_t) h.rows;
        w->cm = (h.flags & FLAG_CHUNK_MAJOR) != 0; w->fo = (h.flags & FLAG_FRAG_ORDER) != 0;
        w->off_a = h.off_a; w->off_b = h.off_b; w->off_c = h.off_c; w->off_d = h.off_d;
    });
}

int bf16n_choose(int64_t rows, int64_t K, int64_t n_matrices, int engine, int mode, int64_t dense_min, int expert,
                 int dense_frag_order, int out[4]) {
    PolicyOptions o;
    o.engine = engine ? Engine::vllm : Engine::llama;
    o.mode = mode == 1 ? Mode::huffman : mode == 2 ? Mode::nibble : Mode::hybrid;
    o.dense_min = dense_min; o.expert = expert != 0; o.dense_frag_order = dense_frag_order != 0;
    PolicyChoice c;
    if (!choose(rows, K, n_matrices, o, &c)) { return 0; }
    out[0] = c.format; out[1] = c.R; out[2] = c.chunk_major; out[3] = c.frag_order;
    return 1;
}

int bf16n_choose_for_machine(int64_t rows, int64_t K, int64_t n_matrices, int engine, int mode, int64_t dense_min, int expert,
                             int dense_frag_order, int64_t min_units, int out[4]) {
    PolicyOptions o;
    o.engine = engine ? Engine::vllm : Engine::llama;
    o.mode = mode == 1 ? Mode::huffman : mode == 2 ? Mode::nibble : Mode::hybrid;
    o.dense_min = dense_min; o.expert = expert != 0; o.dense_frag_order = dense_frag_order != 0;
    o.min_units = min_units;
    PolicyChoice c;
    if (!choose(rows, K, n_matrices, o, &c)) { return 0; }
    out[0] = c.format; out[1] = c.R; out[2] = c.chunk_major; out[3] = c.frag_order;
    return 1;
}

int bf16n_init(void) { return guarded([] { ensure_init(); }); }

int bf16n_fault_status(unsigned int * flags, void * stream) {
    return guarded([&] {
        require(flags != nullptr, "fault_status: null argument");
        ensure_init();
        cudaStream_t st = (cudaStream_t) stream;
        unsigned int seen[4] = {0, 0, 0, 0};
        for (int i = 0; i < 4; i++) {
            cuda_ok(cudaMemcpyAsync(&seen[i], g_fault_words[i], sizeof(unsigned int), cudaMemcpyDeviceToHost, st), "fault word read");
            cuda_ok(cudaMemsetAsync(g_fault_words[i], 0, sizeof(unsigned int), st), "fault word clear");
        }
        cuda_ok(cudaStreamSynchronize(st), "fault word read");
        *flags = 0;
        for (int i = 0; i < 4; i++) { if (seen[i]) { *flags |= 1u << i; } }
    });
}

int bf16n_int4_quantize(const void * w_bf16, int64_t rows, int K, uint8_t * q, float * s, void * stream) {
    return guarded([&] { ensure_init(); draft_quantize(4, w_bf16, rows, K, q, s, (cudaStream_t) stream); });
}
int bf16n_int2_quantize(const void * w_bf16, int64_t rows, int K, uint8_t * q, float * s, void * stream) {
    return guarded([&] { ensure_init(); draft_quantize(2, w_bf16, rows, K, q, s, (cudaStream_t) stream); });
}
int bf16n_int4_gemv(const void * x_bf16, int T, const uint8_t * q, const float * s, int64_t rows, int K, float * y, void * stream) {
    return guarded([&] { ensure_init(); draft_gemv(4, x_bf16, T, q, s, rows, K, y, (cudaStream_t) stream); });
}
int bf16n_int2_gemv(const void * x_bf16, int T, const uint8_t * q, const float * s, int64_t rows, int K, float * y, void * stream) {
    return guarded([&] { ensure_init(); draft_gemv(2, x_bf16, T, q, s, rows, K, y, (cudaStream_t) stream); });
}

int bf16n_set_peer_wait_limit_ms(unsigned int ms) {
    return guarded([&] {
        require(ms >= 1 && ms <= 60000, "peer wait limit: 1..60000 ms");
        g_peer_wait_ns.store((uint64_t) ms * 1000000ull, std::memory_order_relaxed);
    });
}
int bf16n_sm_count(int * out) { return guarded([&] { ensure_init(); *out = g_info.sms; }); }

int bf16n_mmv(const bf16n_weight * w, const bf16n_mmv_args * a, void * stream, int multi_col) {
    return guarded([&] {
        ensure_init();
        check_weight(*w);
        require(a->ncols > 0 && a->ncols <= 65535, "ncols out of range");
        whole_units(*w, *a);
        check_x(*w, *a);
        if (a->nrows == 0) { return; }
        if (frag_order(*w)) { fo_gemv(*w, *a, (cudaStream_t) stream); return; }
        if (expert_units_applies(*w, *a)) { expert_units_mmv(*w, *a, (cudaStream_t) stream); return; }
        gemv(*w, *a, (cudaStream_t) stream, multi_col != 0);
    });
}

int bf16n_mmv_group(const bf16n_weight * w, const bf16n_mmv_args * a, int n, void * stream) {
    return guarded([&] {
        ensure_init();
        require(n >= 0 && (n == 0 || (w && a)), "mmv_group: null argument");
        for (int i = 0; i < n; i++) {
            check_weight(w[i]);
            require(a[i].ncols > 0 && a[i].ncols <= 65535, "ncols out of range");
            whole_units(w[i], a[i]);
            check_x(w[i], a[i]);
        }
        cudaStream_t st = (cudaStream_t) stream;
        for (int i = 0; i < n;) {
            int j = i;
            while (j < n && gemv_groupable(w[j], a[j])) { j++; }
            if (j > i) { gemv_group(w + i, a + i, j - i, st); i = j; continue; }
            if (a[i].nrows != 0) { // not a small dense NIBBLE product: launched as bf16n_mmv launches it
                if (frag_order(w[i])) { fo_gemv(w[i], a[i], st); }
                else if (expert_units_applies(w[i], a[i])) { expert_units_mmv(w[i], a[i], st); }
                else { gemv(w[i], a[i], st, true); }
            }
            i++;
        }
    });
}

int bf16n_mmv_glu_merged(const bf16n_weight * w, const bf16n_mmv_args * a, void * stream) {
    return guarded([&] {
        ensure_init();
        check_weight(*w);
        require(w->format == FMT_NIBBLE, "mmv_glu supports NIBBLE matrices only");
        require(a->rows_per_matrix == 2 * a->nrows, "mmv_glu: rows per matrix must be [gate; up] of nrows each");
        require(a->ncols > 0 && a->ncols <= 65535, "ncols out of range");
        check_x(*w, *a);
        if (a->nrows == 0) { return; }
        gemv_glu_merged(*w, *a, (cudaStream_t) stream);
    });
}

int bf16n_mmv_glu(const bf16n_weight * g, const bf16n_weight * u, const bf16n_mmv_args * a, void * stream) {
    return guarded([&] {
        ensure_init();
        check_weight(*g);
        check_weight(*u);
        require(g->format == u->format && g->K == u->K, "mmv_glu: gate/up format and K must match");
        require(g->rows == u->rows, "mmv_glu: gate/up row counts must match");
        require(a->row0 >= 0 && a->nrows >= 0 && a->row0 <= g->rows && a->nrows <= g->rows - a->row0, "mmv_glu: product rows out of range");
        require(!g->cm && !u->cm, "mmv_glu: chunk-major weights require separate mmv launches");
        require(!g->fo && !u->fo, "mmv_glu: fragment-order weights require separate mmv launches");
        require(g->format == FMT_NIBBLE || g->R == u->R, "mmv_glu: gate/up R must match");
        require(a->ncols > 0 && a->ncols <= 65535, "ncols out of range");
        whole_units(*g, *a);
        check_x(*g, *a);
        if (a->nrows == 0) { return; }
        gemv_glu(*g, *u, *a, (cudaStream_t) stream);
    });
}

int bf16n_dequant(const bf16n_weight * w, int64_t row0, int64_t nrows, uint16_t * out, void * stream) {
    return guarded([&] {
        ensure_init();
        check_weight(*w);
        if (nrows == 0) { return; }
        require(row0 >= 0 && nrows > 0 && row0 + nrows <= w->rows, "dequant rows out of range");
        require(w->format == FMT_NIBBLE || (nrows % w->R == 0 && row0 % w->R == 0), "dequant rows must be whole units");
        if (frag_order(*w)) { fo_expand_store(*w, row0, nrows, out, (cudaStream_t) stream); return; }
        expand_store(*w, row0, nrows, out, (cudaStream_t) stream);
    });
}

int bf16n_verify(const bf16n_weight * w, int64_t row0, int64_t nrows, const uint16_t * src, unsigned long long * mismatches,
                 void * stream) {
    return guarded([&] {
        ensure_init();
        check_weight(*w);
        if (nrows == 0) { return; }
        require(row0 >= 0 && nrows > 0 && row0 + nrows <= w->rows, "verify rows out of range");
        require(w->format == FMT_NIBBLE || (nrows % w->R == 0 && row0 % w->R == 0), "verify rows must be whole units");
        require((uintptr_t) src % 8 == 0, "verify source must be 8-byte aligned");
        if (frag_order(*w)) { fo_expand_compare(*w, row0, nrows, src, mismatches, (cudaStream_t) stream); return; }
        expand_compare(*w, row0, nrows, src, mismatches, (cudaStream_t) stream);
    });
}

int bf16n_get_rows(const bf16n_weight * w, const void * ids, int64_t ids_s0, int64_t n, void * dst, int dst_bf16, int64_t dst_s1,
                   void * stream, int64_t row0) {
    return guarded([&] {
        ensure_init();
        check_weight(*w);
        require(n >= 0, "get_rows: n must be nonnegative");
        require(row0 >= 0 && (n == 0 ? row0 <= w->rows : row0 < w->rows), "get_rows: row0 out of range");
        require(!w->cm, "get_rows of a chunk-major (expert) matrix");
        require(w->format != FMT_HUFFMAN, "get_rows is not implemented for the single-symbol Huffman format");
        if (n == 0) { return; }
        if (frag_order(*w)) { fo_gather_rows(*w, ids, ids_s0, n, dst, dst_bf16 != 0, dst_s1, row0, (cudaStream_t) stream); return; }
        gather_rows(*w, ids, ids_s0, n, dst, dst_bf16 != 0, dst_s1, row0, (cudaStream_t) stream);
    });
}

int bf16n_mm_ids_supported(const bf16n_weight * w, const bf16n_weight * up) {
    if (w->fo || (up && up->fo)) {
        // the fragment-order kernel's shared-memory need is checked against the device: that needs bf16n_init
        try { ensure_init(); } catch (...) { return 0; }
        return fo_mm_ids_supported(*w, up) ? 1 : 0;
    }
    return prefill_supported(*w, up) ? 1 : 0;
}

int bf16n_mm_ids_route(const void * ids, int ids_i64, int64_t ids_row_stride, int32_t * ids_src1, int32_t * ids_dst,
                       int32_t * bounds, int n_experts, int n_tok, int n_used, int nchannels_y, int sis1, void * stream) {
    return guarded([&] {
        ensure_init();
        moe_route(ids, ids_i64 != 0, ids_row_stride, ids_src1, ids_dst, bounds, n_experts, n_tok, n_used, nchannels_y, sis1,
                  (cudaStream_t) stream);
    });
}

int bf16n_mm_ids(const bf16n_weight * w, const bf16n_weight * up, const void * x_bf16, int64_t x_row, const int32_t * ids_src1,
                 const int32_t * ids_dst, const int32_t * bounds, void * dst, int dst_bf16, int64_t dst_col, int n_experts,
                 int n_tok, int n_used, void * stream) {
    return guarded([&] {
        ensure_init();
        check_weight(*w);
        if (up) { check_weight(*up); }
        require(n_experts > 0 && w->rows % n_experts == 0, "rows must split evenly into experts");
        if (w->fo || (up && up->fo)) {
            require(fo_mm_ids_supported(*w, up), "no batched kernel for this matrix");
            fo_mm_ids(*w, up, x_bf16, x_row, ids_src1, ids_dst, bounds, dst, dst_bf16 != 0, dst_col, n_experts, (cudaStream_t) stream);
            return;
        }
        require(prefill_supported(*w, up), "no batched kernel for this matrix");
        prefill_mm_ids(*w, up, x_bf16, x_row, ids_src1, ids_dst, bounds, dst, dst_bf16 != 0, dst_col, n_experts, n_tok, n_used,
                       (cudaStream_t) stream);
    });
}

size_t bf16n_mm_ids_workspace_bytes(const bf16n_weight * w, const bf16n_weight * up) {
    return w ? prefill_workspace_bytes(*w, up) : 0;
}

int bf16n_set_workspace(void * workspace, size_t bytes) {
    return guarded([&] {
        require(!workspace || ((uintptr_t) workspace % 1024) == 0, "set_workspace: the buffer must be 1024-byte aligned");
        prefill_set_workspace(workspace, bytes);
    });
}

int bf16n_moe_combine(const float * ys, const void * w, int w_bf16, void * y, int y_bf16, int n_tok, int n_used, int64_t n,
                      void * stream) {
    return guarded([&] {
        ensure_init();
        moe_combine(ys, w, w_bf16 != 0, y, y_bf16 != 0, n_tok, n_used, n, (cudaStream_t) stream);
    });
}

int bf16n_swiglu(const float * g, const float * u, float * y, int64_t n, void * stream) {
    return guarded([&] {
        ensure_init();
        moe_swiglu(g, u, y, n, (cudaStream_t) stream);
    });
}

int bf16n_moe_topk(const float * logits, int n_tok, int n_experts, int k, int32_t * ids, float * weights, void * stream) {
    return guarded([&] {
        ensure_init();
        moe_topk(logits, n_tok, n_experts, k, ids, weights, (cudaStream_t) stream);
    });
}

size_t bf16n_moe_decode_scratch_bytes(int n_tok, int n_used, int64_t rows_gate, int64_t rows_down) {
    return (size_t) n_tok * n_used * (2 * rows_gate + rows_down) * sizeof(float);
}

static void moe_decode_checked(const bf16n_weight * gate, const bf16n_weight * up, const bf16n_weight * down, const void * x, int x_bf16,
                               int64_t x_tok, const float * router_logits, int n_experts, int32_t * topk_ids, float * topk_weights,
                               int n_tok, int n_used, int expert_lo, int n_experts_local, float * scratch, size_t scratch_bytes,
                               void * y, int y_bf16, void * stream, const bf16n_peer_out * peers) {
    ensure_init();
    require(gate && up && down, "moe_decode: null weight");
    require(n_tok <= 0 || (x && y && topk_ids && topk_weights && scratch), "moe_decode: null argument");
    check_weight(*gate); check_weight(*up); check_weight(*down);
    const bool frag = gate->fo && up->fo && down->fo && fo_supported(*gate) && fo_supported(*up) && fo_supported(*down) &&
                      gate->rows == up->rows && gate->K == up->K;
    require(frag || moe_decode_supported(*gate, *up, *down),
            "moe_decode: gate/up must be chunk-major HUFPAIR R = 8 K = 2048 and down row-major HUFPAIR R = 16 K = 512, or all three "
            "in fragment order");
    require(n_tok >= 0 && n_tok <= 64 && n_used > 0 && n_used <= 32, "moe_decode: 0..64 tokens, 1..32 slots");
    require(n_experts_local > 0 && expert_lo >= 0 && expert_lo + n_experts_local <= n_experts, "moe_decode: expert slice out of range");
    require(gate->rows % n_experts_local == 0 && down->rows % n_experts_local == 0, "rows must split evenly into experts");
    const int64_t N = gate->rows / n_experts_local, H = down->rows / n_experts_local;
    require(N == down->K && H % down->R == 0 && N % gate->R == 0, "moe_decode: down's K must equal the gate/up rows per expert");
    require(scratch_bytes >= bf16n_moe_decode_scratch_bytes(n_tok, n_used, N, H), "moe_decode: scratch too small");
    require((uintptr_t) x % 16 == 0 && x_tok % 16 == 0 && (uintptr_t) scratch % 16 == 0, "moe_decode: x, its row stride and scratch must be 16-byte aligned");
    if (peers) {
        require(n_tok > 0, "moe_decode_peers: empty step (every rank must announce)");
        require(peers->n_peers >= 0 && peers->n_peers <= BF16N_MAX_PEERS && peers->wait_mask >= 0 && peers->wait_mask < 256,
                "moe_decode_peers: 0..7 peers, wait_mask over ranks 0..7");
        require(peers->n_peers == 0 || peers->local_header, "moe_decode_peers: the local exchange header is missing");
        for (int r = 0; r < peers->n_peers; r++) { require(peers->y[r] && peers->flag[r], "moe_decode_peers: null peer pointer"); }
    }
    if (frag) {
        require(!peers && expert_lo == 0 && n_experts_local == n_experts,
                "moe_decode: fragment-order experts run with all experts on one GPU (no expert slice, no peers)");
    }
    if (n_tok == 0) { return; }
    if (router_logits) { moe_topk(router_logits, n_tok, n_experts, n_used, topk_ids, topk_weights, (cudaStream_t) stream); }
    if (frag) {
        moe_decode_frag_order(*gate, *up, *down, x, x_bf16 != 0, x_tok, topk_ids, topk_weights, n_tok, n_used, n_experts, scratch, y,
                              y_bf16 != 0, (cudaStream_t) stream);
        return;
    }
    moe_decode(*gate, *up, *down, x, x_bf16 != 0, x_tok, topk_ids, topk_weights, n_tok, n_used, n_experts_local, expert_lo,
               scratch, y, y_bf16 != 0, (cudaStream_t) stream, peers);
}

int bf16n_moe_decode(const bf16n_weight * gate, const bf16n_weight * up, const bf16n_weight * down, const void * x, int x_bf16,
                     int64_t x_tok, const float * router_logits, int n_experts, int32_t * topk_ids, float * topk_weights, int n_tok,
                     int n_used, int expert_lo, int n_experts_local, float * scratch, size_t scratch_bytes, void * y, int y_bf16,
                     void * stream) {
    return guarded([&] {
        moe_decode_checked(gate, up, down, x, x_bf16, x_tok, router_logits, n_experts, topk_ids, topk_weights, n_tok, n_used, expert_lo,
                           n_experts_local, scratch, scratch_bytes, y, y_bf16, stream, nullptr);
    });
}

int bf16n_moe_decode_peers(const bf16n_weight * gate, const bf16n_weight * up, const bf16n_weight * down, const void * x, int x_bf16,
                           int64_t x_tok, const float * router_logits, int n_experts, int32_t * topk_ids, float * topk_weights,
                           int n_tok, int n_used, int expert_lo, int n_experts_local, float * scratch, size_t scratch_bytes,
                           void * y, int y_bf16, const bf16n_peer_out * peers, void * stream) {
    return guarded([&] {
        require(peers != nullptr, "moe_decode_peers: peers is null");
        moe_decode_checked(gate, up, down, x, x_bf16, x_tok, router_logits, n_experts, topk_ids, topk_weights, n_tok, n_used, expert_lo,
                           n_experts_local, scratch, scratch_bytes, y, y_bf16, stream, peers);
    });
}

int bf16n_peer_sum(const float * parts, int n_parts, int64_t n, const float * extra, void * y, int y_bf16, void * stream) {
    return guarded([&] {
        require(parts && y && n_parts >= 1 && n_parts <= 8 && n >= 0, "peer_sum: 1..8 parts");
        if (n == 0) { return; }
        peer_sum(parts, n_parts, n, extra, y, y_bf16 != 0, (cudaStream_t) stream);
    });
}

int bf16n_moe_decode_static(const bf16n_weight * gate, const bf16n_weight * up, const bf16n_weight * down, const void * x, int x_bf16,
                            int64_t x_tok, const float * router_logits, int n_experts, int32_t * topk_ids, float * topk_weights,
                            int n_tok, int n_used, int expert_lo, int n_experts_local, void * y, int y_bf16, void * stream) {
    return guarded([&] {
        ensure_init();
        require(gate && up && down, "moe_decode: null weight");
        require(n_tok <= 0 || (x && y && topk_ids && topk_weights), "moe_decode: null argument");
        check_weight(*gate); check_weight(*up); check_weight(*down);
        require(moe_decode_supported(*gate, *up, *down),
                "moe_decode: gate/up must be chunk-major HUFPAIR R = 8 K = 2048 and down row-major HUFPAIR R = 16 K = 512");
        require(n_tok >= 0 && n_tok <= 64 && n_used > 0 && n_used <= 32, "moe_decode: 0..64 tokens, 1..32 slots");
        require(n_experts_local > 0 && expert_lo >= 0 && expert_lo + n_experts_local <= n_experts, "moe_decode: expert slice out of range");
        require(gate->rows % n_experts_local == 0 && down->rows % n_experts_local == 0, "rows must split evenly into experts");
        const int64_t N = gate->rows / n_experts_local, H = down->rows / n_experts_local;
        require(N == down->K && H % down->R == 0 && N % gate->R == 0, "moe_decode: down's K must equal the gate/up rows per expert");
        const size_t need = bf16n_moe_decode_scratch_bytes(n_tok, n_used, N, H) / sizeof(float);
        if (need > moe_decode_static_capacity_floats()) {
            fail_invalid("moe_decode_static: the step needs " + std::to_string(need) + " floats of scratch, the built-in buffer holds " +
                         std::to_string(moe_decode_static_capacity_floats()) + " (BF16N_MOE_DECODE_STATIC_MAX_FLOATS); use bf16n_moe_decode");
        }
        require((uintptr_t) x % 16 == 0 && x_tok % 16 == 0, "moe_decode: x and its row stride must be 16-byte aligned");
        if (n_tok == 0) { return; }
        if (router_logits) { moe_topk(router_logits, n_tok, n_experts, n_used, topk_ids, topk_weights, (cudaStream_t) stream); }
        moe_decode_static(*gate, *up, *down, x, x_bf16 != 0, x_tok, topk_ids, topk_weights, n_tok, n_used, n_experts_local, expert_lo,
                          y, y_bf16 != 0, (cudaStream_t) stream);
    });
}


int bf16n_exchange_create(size_t payload_bytes, void ** base, unsigned char handle[BF16N_IPC_HANDLE_BYTES]) {
    return guarded([&] {
        static_assert(sizeof(cudaIpcMemHandle_t) == BF16N_IPC_HANDLE_BYTES, "IPC handle size");
        require(base && handle, "exchange_create: null output");
        void * p = nullptr;
        const size_t bytes = BF16N_EXCHANGE_HEADER_BYTES + ((payload_bytes + 255) & ~(size_t) 255);
        cuda_ok(cudaMalloc(&p, bytes), "exchange buffer");
        cuda_ok(cudaMemset(p, 0, bytes), "exchange buffer clear");
        cuda_ok(cudaDeviceSynchronize(), "exchange buffer clear");
        cudaIpcMemHandle_t h;
        cuda_ok(cudaIpcGetMemHandle(&h, p), "exchange buffer export");
        memcpy(handle, &h, sizeof h);
        *base = p;
    });
}

int bf16n_exchange_open(const unsigned char handle[BF16N_IPC_HANDLE_BYTES], void ** base) {
    return guarded([&] {
        require(base && handle, "exchange_open: null argument");
        cudaIpcMemHandle_t h;
        memcpy(&h, handle, sizeof h);
        void * p = nullptr;
        cuda_ok(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "exchange buffer import");
        *base = p;
    });
}

int bf16n_exchange_close(void * peer_base) {
    return guarded([&] { cuda_ok(cudaIpcCloseMemHandle(peer_base), "exchange buffer unmap"); });
}

int bf16n_exchange_destroy(void * base) {
    return guarded([&] { cuda_ok(cudaFree(base), "exchange buffer free"); });
}

int bf16n_mmv_peers(const bf16n_weight * w, const bf16n_mmv_args * a, const bf16n_peer_out * peers, void * stream) {
    return guarded([&] {
        ensure_init();
        check_weight(*w);
        no_frag_order(*w);
        require(a->ncols > 0 && a->ncols <= 65535, "ncols out of range");
        whole_units(*w, *a);
        check_x(*w, *a);
        require(peers && peers->n_peers >= 0 && peers->n_peers <= BF16N_MAX_PEERS, "mmv_peers: 0..7 peers");
        require(peers->n_peers == 0 || peers->local_header, "mmv_peers: the local exchange header is missing");
        require(peers->wait_mask >= 0 && peers->wait_mask < 256, "mmv_peers: wait_mask names ranks 0..7");
        for (int r = 0; r < peers->n_peers; r++) { require(peers->y[r] && peers->flag[r], "mmv_peers: null peer pointer"); }
        require(a->nrows > 0, "mmv_peers: empty product (every rank must announce)");
        gemv(*w, *a, (cudaStream_t) stream, false, peers);
    });
}

int bf16n_peer_wait(uint32_t * local_header, int rank_mask, void * stream) {
    return guarded([&] {
        require(local_header && rank_mask >= 0 && rank_mask < 256, "peer_wait: header and a mask of ranks 0..7");
        peer_wait(local_header, rank_mask, (cudaStream_t) stream);
    });
}

size_t bf16n_ep_layout_bytes(bf16n_ep_layout * l) { return l ? ep_layout_fill(*l) : 0; }
int bf16n_ep_dispatch(const bf16n_ep_layout * l, const void * x_bf16, int64_t x_row_bytes, const int32_t * topk_ids, int n_tok, int n_used,
                      int n_experts, int32_t * plan, void * stream) {
    return guarded([&] {
        ensure_init();
        require(l && x_bf16 && topk_ids && plan, "ep_dispatch: null argument");
        ep_dispatch(*l, x_bf16, x_row_bytes, topk_ids, n_tok, n_used, n_experts, plan, (cudaStream_t) stream);
    });
}
int bf16n_ep_inbox_ids(const bf16n_ep_layout * l, int32_t * ids_out, void * stream) {
    return guarded([&] {
        ensure_init();
        require(l && ids_out, "ep_inbox_ids: null argument");
        ep_inbox_ids(*l, ids_out, (cudaStream_t) stream);
    });
}
int bf16n_ep_give_back(const bf16n_ep_layout * l, const float * ys, void * stream) {
    return guarded([&] {
        ensure_init();
        require(l && ys, "ep_give_back: null argument");
        ep_give_back(*l, ys, (cudaStream_t) stream);
    });
}

int bf16n_peer_expired(const uint32_t * local_header, void * stream, int * expired) {
    return guarded([&] {
        require(local_header && expired, "peer_expired: null argument");
        uint32_t v = 0;
        cuda_ok(cudaMemcpyAsync(&v, local_header + 19, sizeof v, cudaMemcpyDeviceToHost, (cudaStream_t) stream), "exchange header read");
        cuda_ok(cudaStreamSynchronize((cudaStream_t) stream), "exchange header read");
        *expired = (int) v;
    });
}

} // extern "C"
