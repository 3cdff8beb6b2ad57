// The engine-independent half of the llama.cpp adapter (the reference's ggml-cuda/bf16n.cu, added by
// engines/llamacpp/patches/0002-ggml-cuda-thin-BF16N-adapter-over-the-shared-core.patch, patch lines 47-332): ownership
// of the auxiliary buffers, the address-range registry that turns a tensor's data pointer (or a view into it) back into
// its encoded matrix and first row, the shape-policy entry point of ggml's conversion ABI, and the loader
// (encode -> upload -> registry -> exhaustive bit-exact check in bounded chunks -> one log line per tensor).
// What stays in the engine is only what needs its types: reading ne[] / nb[] of a ggml_tensor into bf16n_mmv_args.
//
// Unlike the launchers this is load-time code: it allocates (the aux buffer, a bounded staging buffer for the check)
// and synchronises. The check compares on the device (bf16n_verify) instead of copying the decoded rows back.
#include "encode.h"
#include "launch.h"
#include "policy.h"

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <functional>
#include <mutex>
#include <vector>

namespace b16 {
namespace {

struct Entry {
    bf16n_weight w;
    size_t nbytes;        // plane bytes: rows * K
    const void * owner;   // the engine's buffer handle; its release frees the aux storage of everything it owns
    uint8_t * aux_dev;    // owned here
};

std::mutex g_mutex;
std::vector<Entry> g_entries; // sorted by plane address

std::vector<Entry>::iterator upper(const uint8_t * p) {
    const auto less = std::less<const uint8_t *>{};
    return std::upper_bound(g_entries.begin(), g_entries.end(), p, [&](const uint8_t * a, const Entry & e) { return less(a, e.w.plane); });
}

constexpr int TAG_NIBBLE = 1, TAG_HUFFMAN = 2; // ggml's conversion tags: 2 = pair Huffman with single-symbol fallback

} // namespace
} // namespace b16

using namespace b16;

extern "C" {

int bf16n_adapter_choose(int64_t rows, int64_t K, int64_t n_matrices, const char * mode, int64_t dense_min, int expert) {
    PolicyOptions o;
    o.engine = Engine::llama;
    o.mode = mode && strcmp(mode, "nibble") == 0 ? Mode::nibble : mode && strcmp(mode, "huffman") == 0 ? Mode::huffman : Mode::hybrid;
    o.dense_min = dense_min;
    o.expert = expert != 0;
    PolicyChoice c;
    if (!choose(rows, K, n_matrices, o, &c)) { return 0; }
    return c.format == FMT_NIBBLE ? TAG_NIBBLE : TAG_HUFFMAN;
}

int bf16n_adapter_lookup(const void * data, bf16n_weight * out, int64_t * row0) {
    std::lock_guard<std::mutex> lock(g_mutex);
    const auto * q = static_cast<const uint8_t *>(data);
    auto it = upper(q);
    if (it == g_entries.begin()) { return 0; }
    --it;
    const auto less = std::less<const uint8_t *>{};
    if (!less(q, it->w.plane + it->nbytes)) { return 0; }
    const size_t off = (size_t) (q - it->w.plane);
    if (off % (size_t) it->w.K) { return 0; } // a view starts on a row
    if (out) { *out = it->w; }                // by value: loading or unloading another model may move the entries
    if (row0) { *row0 = (int64_t) (off / (size_t) it->w.K); }
    return 1;
}

int bf16n_adapter_release(const void * owner) {
    std::lock_guard<std::mutex> lock(g_mutex);
    int n = 0;
    for (auto it = g_entries.begin(); it != g_entries.end();) {
        if (it->owner == owner) {
            cudaFree(it->aux_dev);
            it = g_entries.erase(it);
            n++;
        } else {
            ++it;
        }
    }
    return n;
}

int bf16n_adapter_convert(void * plane_dev, const void * bf16_host, int64_t K, int64_t rows_per_matrix, int64_t n_matrices, int format_tag,
                          const void * owner, const char * name, int * roundtrip_ok) {
    try {
        require(plane_dev && bf16_host && roundtrip_ok, "adapter_convert: null argument");
        require(format_tag == TAG_NIBBLE || format_tag == TAG_HUFFMAN, "adapter_convert: format tag must be 1 (nibble) or 2 (huffman)");
        require(K > 0 && rows_per_matrix > 0 && n_matrices > 0, "adapter_convert: empty tensor");
        if (bf16n_init() != BF16N_OK) { throw std::runtime_error(bf16n_last_error()); }
        const int64_t rows = rows_per_matrix * n_matrices;
        const auto * src = static_cast<const uint16_t *>(bf16_host);
        // the explicit format is part of the conversion ABI; the unit layout comes from the llama shape policy
        PolicyOptions o;
        o.engine = Engine::llama;
        o.mode = format_tag == TAG_NIBBLE ? Mode::nibble : Mode::huffman;
        PolicyChoice pc;
        require(choose(rows_per_matrix, K, n_matrices, o, &pc), "adapter_convert: the shape policy keeps this tensor in BF16");
        const Encoded enc = encode(src, rows, K, pc.format, pc.R, pc.chunk_major);
        cuda_ok(cudaMemcpy(plane_dev, enc.plane.data(), enc.plane.size(), cudaMemcpyHostToDevice), "plane upload");
        uint8_t * aux_dev = nullptr;
        cuda_ok(cudaMalloc(&aux_dev, enc.aux.size()), "aux allocation");
        if (cudaMemcpy(aux_dev, enc.aux.data(), enc.aux.size(), cudaMemcpyHostToDevice) != cudaSuccess) {
            cudaFree(aux_dev);
            throw std::runtime_error("bf16n: CUDA error at aux upload");
        }
        AuxHeader h;
        memcpy(&h, enc.aux.data(), sizeof h);
        Entry e = {};
        e.w.plane = static_cast<const uint8_t *>(plane_dev);
        e.w.aux = aux_dev;
        e.w.format = enc.format; e.w.R = enc.R; e.w.K = K; e.w.rows = rows;
        e.w.cm = (h.flags & FLAG_CHUNK_MAJOR) != 0; e.w.fo = 0;
        e.w.off_a = h.off_a; e.w.off_b = h.off_b; e.w.off_c = h.off_c; e.w.off_d = h.off_d;
        e.nbytes = enc.plane.size(); e.owner = owner; e.aux_dev = aux_dev;
        {
            std::lock_guard<std::mutex> lock(g_mutex);
            g_entries.insert(upper(e.w.plane), e);
        }
        // exhaustive bit-exact check, bounded to a 64 MiB device staging buffer of source rows (whole units)
        const int R = std::max(e.w.R, 1);
        const int64_t chunk_rows = std::max<int64_t>((64ll << 20) / (K * 2) / R * R, R);
        uint16_t * d_src = nullptr;
        unsigned long long * d_bad = nullptr;
        cuda_ok(cudaMalloc(&d_src, (size_t) chunk_rows * K * 2), "staging allocation");
        if (cudaMalloc(&d_bad, sizeof *d_bad) != cudaSuccess) { cudaFree(d_src); throw std::runtime_error("bf16n: CUDA error at counter allocation"); }
        unsigned long long bad = 0;
        int rc = BF16N_OK;
        cudaMemset(d_bad, 0, sizeof *d_bad);
        for (int64_t r0 = 0; r0 < rows && rc == BF16N_OK; r0 += chunk_rows) {
            const int64_t nr = std::min(chunk_rows, rows - r0);
            if (cudaMemcpy(d_src, src + r0 * K, (size_t) nr * K * 2, cudaMemcpyHostToDevice) != cudaSuccess) { rc = BF16N_ECUDA; break; }
            rc = bf16n_verify(&e.w, r0, nr, d_src, d_bad, nullptr);
        }
        if (rc == BF16N_OK && cudaMemcpy(&bad, d_bad, sizeof bad, cudaMemcpyDeviceToHost) != cudaSuccess) { rc = BF16N_ECUDA; }
        cudaFree(d_src);
        cudaFree(d_bad);
        if (rc != BF16N_OK) { throw std::runtime_error(rc == BF16N_ECUDA ? "bf16n: CUDA error during the load-time check" : bf16n_last_error()); }
        const bool ok = bad == 0;
        *roundtrip_ok = ok;
        const double ratio = double(enc.plane.size() + enc.aux.size()) / double(rows * K * 2);
        fprintf(stderr, "bf16n: %-32s %s K=%5lld rows=%7lld R=%2d ratio=%.4f roundtrip=%s\n", name ? name : "",
                e.w.format == FMT_HUFPAIR ? "hufpair" : e.w.format == FMT_HUFFMAN ? "huffman" : "nibble ", (long long) K, (long long) rows,
                e.w.R, ratio, ok ? "OK" : "FAIL");
        return BF16N_OK;
    } catch (const std::invalid_argument & ex) {
        set_last_error(ex.what());
        return BF16N_EINVAL;
    } catch (const std::exception & ex) {
        set_last_error(ex.what());
        return strstr(ex.what(), "CUDA error") ? BF16N_ECUDA : BF16N_EINTERNAL;
    }
}

int bf16n_adapter_count(void) {
    std::lock_guard<std::mutex> lock(g_mutex);
    return (int) g_entries.size();
}

} // extern "C"
