// One driver, two libraries: times the hot path through the reference's C++ operator interface (namespace bf16n:
// encode, init, mmv, swiglu, moe_combine, mm_ids_route, mm_ids). Compiled once against the reference's own headers and
// sources (the reference's kernels recompiled for sm_100a: the same-GPU baseline) and once against this repository's
// include/bf16n/*.h + libbf16n_b200.so, which shows that the interface is a drop-in and gives both numbers on identical
// inputs. Test and measurement infrastructure only; the build recipe is baseline/Makefile.
//
//   api_bench [lm_head|moe_decode|moe_prefill|small|all|frag_order] [reps]
//
// Synthetic inputs as in bench.py: weights N(0, 0.02) rounded to BF16 (mt19937_64, seed per tensor), activations N(0, 1)
// rounded to BF16. Every timing is the median of `reps` CUDA-event measurements after warm-up; working sets larger than
// L2 or rotated over several copies. Prints one JSON line per workload with a checksum of the result.
#include "bf16n/encode.h"
#include "bf16n/format.h"
#include "bf16n/launch.h"
#ifdef WITH_WORKSPACE
#include "bf16n_c.h"
#endif

#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <string>
#include <vector>

#ifndef IMPL_NAME
#define IMPL_NAME "unknown"
#endif

#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { fprintf(stderr, "CUDA error %s at %s:%d\n", cudaGetErrorString(e_), __FILE__, __LINE__); exit(1); } } while (0)

static uint16_t to_bf16(float f) { // round to nearest even
    uint32_t u;
    memcpy(&u, &f, 4);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t) (u >> 16);
}
static std::vector<uint16_t> normal_bf16(size_t n, float sigma, uint64_t seed) {
    std::mt19937_64 g(seed);
    std::normal_distribution<float> d(0.f, sigma);
    std::vector<uint16_t> v(n);
    for (auto & x : v) { x = to_bf16(d(g)); }
    return v;
}

struct Dev { // one encoded matrix on the device
    bf16n::weight w;
    size_t bytes = 0;
};
static Dev upload(const bf16n::encoded & e, int64_t rows, int64_t K) {
    Dev d;
    uint8_t * p, * a;
    CK(cudaMalloc(&p, e.plane.size()));
    CK(cudaMalloc(&a, e.aux.size()));
    CK(cudaMemcpy(p, e.plane.data(), e.plane.size(), cudaMemcpyHostToDevice));
    CK(cudaMemcpy(a, e.aux.data(), e.aux.size(), cudaMemcpyHostToDevice));
    const bf16n::aux_header * h = (const bf16n::aux_header *) e.aux.data();
    d.w.plane = p; d.w.aux = a; d.w.format = e.format; d.w.K = K; d.w.rows = rows; d.w.R = e.R;
    d.w.cm = (h->flags & 1u) != 0; d.w.fo = (h->flags & 2u) != 0;
    d.w.off_a = h->off_a; d.w.off_b = h->off_b; d.w.off_c = h->off_c; d.w.off_d = h->off_d;
    d.bytes = e.plane.size() + e.aux.size();
    return d;
}
static Dev make(int64_t rows, int64_t K, int format, int R, bool cm, uint64_t seed, bool fo = false) {
    const std::vector<uint16_t> w = normal_bf16((size_t) rows * K, 0.02f, seed);
    return upload(bf16n::encode(w.data(), rows, K, format, R, cm, fo), rows, K);
}
template <typename T> static T * dev_copy(const std::vector<T> & v) {
    T * p;
    CK(cudaMalloc(&p, v.size() * sizeof(T)));
    CK(cudaMemcpy(p, v.data(), v.size() * sizeof(T), cudaMemcpyHostToDevice));
    return p;
}
template <typename F> static double median_us(int reps, F && f) {
    cudaEvent_t a, b;
    CK(cudaEventCreate(&a)); CK(cudaEventCreate(&b));
    for (int i = 0; i < 5; i++) { f(i); }
    CK(cudaDeviceSynchronize());
    std::vector<float> t(reps);
    for (int i = 0; i < reps; i++) {
        CK(cudaEventRecord(a));
        f(i);
        CK(cudaEventRecord(b));
        CK(cudaEventSynchronize(b));
        CK(cudaEventElapsedTime(&t[i], a, b));
    }
    std::sort(t.begin(), t.end());
    return t[reps / 2] * 1e3;
}
// sum of |y|; with API_BENCH_DUMP=<prefix> in the environment the raw FP32 result also goes to <prefix><tag>.f32, so that
// the outputs of the two builds can be compared element by element (baseline/compare_dumps.py)
static double checksum(const float * dev, size_t n, const std::string & tag) {
    std::vector<float> h(n);
    CK(cudaMemcpy(h.data(), dev, n * 4, cudaMemcpyDeviceToHost));
    if (const char * prefix = getenv("API_BENCH_DUMP")) {
        FILE * f = fopen((std::string(prefix) + tag + ".f32").c_str(), "wb");
        if (f) { fwrite(h.data(), 4, n, f); fclose(f); }
    }
    double s = 0;
    for (size_t i = 0; i < n; i++) { s += std::fabs((double) h[i]); }
    return s;
}

// ---- config 1: lm_head 248320 x 2048, HUFPAIR R = 16, one BF16 activation, FP32 logits
static void lm_head(int reps) {
    const int64_t rows = 248320, K = 2048;
    const Dev d = make(rows, K, bf16n::FMT_HUFPAIR, 16, false, 1);
    const uint16_t * x = dev_copy(normal_bf16(K, 1.f, 2));
    float * y;
    CK(cudaMalloc(&y, rows * 4));
    bf16n::mmv_args a;
    a.x = x; a.x_bf16 = true; a.y = y; a.y_bf16 = false; a.ncols = 1; a.x_tok = K * 2; a.y_tok = rows * 4;
    a.rows_per_matrix = rows; a.row0 = 0; a.nrows = rows;
    const double us = median_us(reps, [&](int) { bf16n::mmv(d.w, a, 0); });
    printf("{\"impl\": \"%s\", \"workload\": \"lm_head 248320x2048 HUFPAIR R=16, batch-1 GEMV\", \"us\": %.2f, \"compressed_GBps\": %.1f, "
           "\"sum_abs_y\": %.6e}\n", IMPL_NAME, us, (double) d.bytes / us / 1e3, checksum(y, rows, "lm_head"));
}

// ---- config 2: 48 layers x {2048x512, 512x2048, 256x2048} NIBBLE, batch-1 GEMVs, captured into one CUDA graph
static void small(int reps) {
    struct L { Dev a, b, c; float * ya, * yb, * yc; };
    std::vector<L> layers(48);
    size_t bytes = 0;
    for (int l = 0; l < 48; l++) {
        L & s = layers[l];
        s.a = make(2048, 512, bf16n::FMT_NIBBLE, 0, false, 300 + 3 * l);
        s.b = make(512, 2048, bf16n::FMT_NIBBLE, 0, false, 301 + 3 * l);
        s.c = make(256, 2048, bf16n::FMT_NIBBLE, 0, false, 302 + 3 * l);
        CK(cudaMalloc(&s.ya, 2048 * 4)); CK(cudaMalloc(&s.yb, 512 * 4)); CK(cudaMalloc(&s.yc, 256 * 4));
        bytes += s.a.bytes + s.b.bytes + s.c.bytes;
    }
    const uint16_t * x512 = dev_copy(normal_bf16(512, 1.f, 3)), * x2048 = dev_copy(normal_bf16(2048, 1.f, 4));
    cudaStream_t st;
    CK(cudaStreamCreate(&st));
    auto one = [&](const Dev & d, const uint16_t * x, float * y, int64_t rows, int64_t K) {
        bf16n::mmv_args a;
        a.x = x; a.x_bf16 = true; a.y = y; a.y_bf16 = false; a.ncols = 1; a.x_tok = K * 2; a.y_tok = rows * 4;
        a.rows_per_matrix = rows; a.row0 = 0; a.nrows = rows;
        bf16n::mmv(d.w, a, st);
    };
    auto all = [&] { for (L & s : layers) { one(s.a, x512, s.ya, 2048, 512); one(s.b, x2048, s.yb, 512, 2048); one(s.c, x2048, s.yc, 256, 2048); } };
    all();
    CK(cudaStreamSynchronize(st));
    cudaGraph_t graph; cudaGraphExec_t exec;
    CK(cudaStreamBeginCapture(st, cudaStreamCaptureModeGlobal));
    all();
    CK(cudaStreamEndCapture(st, &graph));
    CK(cudaGraphInstantiate(&exec, graph, 0));
    cudaEvent_t e0, e1;
    CK(cudaEventCreate(&e0)); CK(cudaEventCreate(&e1));
    for (int i = 0; i < 5; i++) { CK(cudaGraphLaunch(exec, st)); }
    CK(cudaStreamSynchronize(st));
    std::vector<float> t(reps);
    for (int i = 0; i < reps; i++) {
        CK(cudaEventRecord(e0, st)); CK(cudaGraphLaunch(exec, st)); CK(cudaEventRecord(e1, st));
        CK(cudaEventSynchronize(e1)); CK(cudaEventElapsedTime(&t[i], e0, e1));
    }
    std::sort(t.begin(), t.end());
    const double us = t[reps / 2] * 1e3;
    printf("{\"impl\": \"%s\", \"workload\": \"small matrices: 48 layers x 3 NIBBLE GEMVs in one CUDA graph\", \"us\": %.1f, \"us_per_gemv\": %.2f, "
           "\"compressed_GBps\": %.1f, \"sum_abs_y\": %.6e}\n", IMPL_NAME, us, us / 144, (double) bytes / us / 1e3,
           checksum(layers[47].ya, 2048, "small"));
}

// ---- the fragment-order layout (what the reference's vLLM policy picks): projection at 1 and 8 tokens, prefill layer
static void frag_order(int reps) {
    {
        const int64_t rows = 248320, K = 2048;
        const Dev d = make(rows, K, bf16n::FMT_HUFPAIR, 16, false, 1, true);
        for (int T : {1, 8}) {
            const uint16_t * x = dev_copy(normal_bf16((size_t) T * K, 1.f, 2));
            float * y;
            CK(cudaMalloc(&y, (size_t) T * rows * 4));
            bf16n::mmv_args a;
            a.x = x; a.x_bf16 = true; a.y = y; a.y_bf16 = false; a.ncols = T; a.x_tok = K * 2; a.y_tok = rows * 4;
            a.rows_per_matrix = rows; a.row0 = 0; a.nrows = rows;
            const double us = median_us(reps, [&](int) { bf16n::mmv(d.w, a, 0); });
            printf("{\"impl\": \"%s\", \"workload\": \"lm_head 248320x2048 fragment order, %d token(s)\", \"us\": %.2f, \"sum_abs_y\": %.6e}\n",
                   IMPL_NAME, T, us, checksum(y, (size_t) T * rows, "fo_lm_head_" + std::to_string(T)));
            CK(cudaFree(y));
        }
        CK(cudaFree((void *) d.w.plane)); CK(cudaFree((void *) d.w.aux));
    }
    const int E = 256, k = 8, H = 2048, N = 512;
    const Dev gate = make((int64_t) E * N, H, bf16n::FMT_HUFPAIR, 16, false, 11, true);
    const Dev up = make((int64_t) E * N, H, bf16n::FMT_HUFPAIR, 16, false, 12, true);
    const Dev down = make((int64_t) E * H, N, bf16n::FMT_HUFPAIR, 16, false, 13, true);
    if (!bf16n::mm_ids_supported(gate.w, &up.w) || !bf16n::mm_ids_supported(down.w, nullptr)) {
        printf("{\"impl\": \"%s\", \"workload\": \"MoE prefill, fragment order\", \"unavailable\": \"no batched kernel\"}\n", IMPL_NAME);
        return;
    }
    for (int T : {2048, 8192}) {
        std::mt19937_64 g(200 + T);
        std::vector<int32_t> ids((size_t) T * k);
        for (int t = 0; t < T; t++) {
            std::vector<int> perm(E);
            for (int i = 0; i < E; i++) { perm[i] = i; }
            std::shuffle(perm.begin(), perm.end(), g);
            for (int s = 0; s < k; s++) { ids[(size_t) t * k + s] = perm[s]; }
        }
        const int32_t * d_ids = dev_copy(ids);
        const std::vector<float> wts((size_t) T * k, 1.f / k);
        const float * d_w = dev_copy(wts);
        const uint16_t * x = dev_copy(normal_bf16((size_t) T * H, 1.f, 30));
        int32_t * src1, * dst, * bounds;
        CK(cudaMalloc(&src1, (size_t) T * k * 4)); CK(cudaMalloc(&dst, (size_t) T * k * 4)); CK(cudaMalloc(&bounds, (E + 1) * 4));
        uint16_t * act; float * ys, * y;
        CK(cudaMalloc(&act, (size_t) T * k * N * 2)); CK(cudaMalloc(&ys, (size_t) T * k * H * 4)); CK(cudaMalloc(&y, (size_t) T * H * 4));
        auto step = [&](int) {
            bf16n::mm_ids_route(d_ids, false, k, src1, dst, bounds, E, T, k, 1, 1, 0);
            bf16n::mm_ids(gate.w, &up.w, x, H, src1, dst, bounds, act, true, N, E, T, k, 0);
            bf16n::mm_ids_route(d_ids, false, k, src1, dst, bounds, E, T, k, k, k, 0);
            bf16n::mm_ids(down.w, nullptr, act, N, src1, dst, bounds, ys, false, H, E, T, k, 0);
            bf16n::moe_combine(ys, d_w, false, y, false, T, k, H, 0);
        };
        const double us = median_us(std::max(5, reps / 4), step);
        printf("{\"impl\": \"%s\", \"workload\": \"MoE prefill layer, %d tokens, fragment-order experts\", \"us\": %.1f, \"TFLOPs\": %.1f, "
               "\"sum_abs_y\": %.6e}\n", IMPL_NAME, T, us, 6.0 * N * H * k * T / us / 1e6, checksum(y, (size_t) T * H, "fo_moe_prefill_" + std::to_string(T)));
        for (const void * q : {(const void *) d_ids, (const void *) d_w, (const void *) x, (const void *) src1, (const void *) dst, (const void *) bounds,
                               (const void *) act, (const void *) ys, (const void *) y}) {
            CK(cudaFree((void *) q));
        }
    }
}

// ---- config 3: MoE decode layer through the operator chain of the reference's Python layer
// (mmv gate, mmv up with expert ids, swiglu, mmv down, moe_combine): 256 experts, top-8, T tokens
static void moe_decode(int reps, bool fo = false) {
    const int E = 256, k = 8, H = 2048, N = 512;
    const Dev gate = make((int64_t) E * N, H, bf16n::FMT_HUFPAIR, fo ? 16 : 8, !fo, 11, fo);
    const Dev up = make((int64_t) E * N, H, bf16n::FMT_HUFPAIR, fo ? 16 : 8, !fo, 12, fo);
    const Dev down = make((int64_t) E * H, N, bf16n::FMT_HUFPAIR, 16, false, 13, fo);
    for (int T : {1, 2, 4}) {
        const int rot = 16; // routings rotated so that consecutive steps read different experts (weights exceed L2)
        std::mt19937_64 g(100 + T);
        std::vector<int32_t> ids((size_t) rot * T * k);
        for (int r = 0; r < rot * T; r++) {
            std::vector<int> perm(E);
            for (int i = 0; i < E; i++) { perm[i] = i; }
            std::shuffle(perm.begin(), perm.end(), g);
            for (int s = 0; s < k; s++) { ids[(size_t) r * k + s] = perm[s]; }
        }
        const int32_t * d_ids = dev_copy(ids);
        const std::vector<float> wts((size_t) T * k, 1.f / k);
        const float * d_w = dev_copy(wts);
        const uint16_t * x = dev_copy(normal_bf16((size_t) T * H, 1.f, 20 + T));
        float * gbuf, * ubuf, * abuf, * ys, * y;
        CK(cudaMalloc(&gbuf, (size_t) T * k * N * 4)); CK(cudaMalloc(&ubuf, (size_t) T * k * N * 4));
        CK(cudaMalloc(&abuf, (size_t) T * k * N * 4)); CK(cudaMalloc(&ys, (size_t) T * k * H * 4));
        CK(cudaMalloc(&y, (size_t) T * H * 4));
        auto step = [&](int i) {
            const int32_t * id = d_ids + (size_t) (i % rot) * T * k;
            bf16n::mmv_args a;
            a.x = x; a.x_bf16 = true; a.ncols = T * k; a.x_tok = H * 2; a.ids = id; a.ids_s0 = 4; a.ids_s1 = 4 * k;
            a.n_used = k; a.x_per_slot = 1; a.x_slot = 0; a.y_bf16 = false; a.y_tok = (int64_t) k * N * 4; a.y_slot = N * 4;
            a.rows_per_matrix = N; a.row0 = 0; a.nrows = N;
            a.y = gbuf; bf16n::mmv(gate.w, a, 0);
            a.y = ubuf; bf16n::mmv(up.w, a, 0);
            bf16n::swiglu(gbuf, ubuf, abuf, (int64_t) T * k * N, 0);
            bf16n::mmv_args b;
            b.x = abuf; b.x_bf16 = false; b.ncols = T * k; b.x_tok = (int64_t) k * N * 4; b.x_per_slot = k; b.x_slot = N * 4;
            b.ids = id; b.ids_s0 = 4; b.ids_s1 = 4 * k; b.n_used = k; b.y = ys; b.y_bf16 = false; b.y_tok = (int64_t) k * H * 4;
            b.y_slot = H * 4; b.rows_per_matrix = H; b.row0 = 0; b.nrows = H;
            bf16n::mmv(down.w, b, 0);
            bf16n::moe_combine(ys, d_w, false, y, false, T, k, H, 0);
        };
        const double us = median_us(reps, step);
        printf("{\"impl\": \"%s\", \"workload\": \"MoE decode, routed experts only%s, %d token(s), operator chain of 5 launches\", \"us\": %.2f, "
               "\"sum_abs_y\": %.6e}\n", IMPL_NAME, fo ? ", fragment-order experts" : "", T, us,
               checksum(y, (size_t) T * H, std::string(fo ? "fo_" : "") + "moe_decode_" + std::to_string(T)));
    }
}

// ---- config 4: MoE prefill layer: route, batched gate/up + SwiGLU (BF16 out), route, batched down (FP32 out), combine
static void moe_prefill(int reps) {
    const int E = 256, k = 8, H = 2048, N = 512;
    const Dev gate = make((int64_t) E * N, H, bf16n::FMT_HUFPAIR, 8, true, 11);
    const Dev up = make((int64_t) E * N, H, bf16n::FMT_HUFPAIR, 8, true, 12);
    const Dev down = make((int64_t) E * H, N, bf16n::FMT_HUFPAIR, 16, false, 13);
    if (!bf16n::mm_ids_supported(gate.w, &up.w) || !bf16n::mm_ids_supported(down.w, nullptr)) {
        printf("{\"impl\": \"%s\", \"workload\": \"MoE prefill\", \"unavailable\": \"no batched kernel for these layouts\"}\n", IMPL_NAME);
        return;
    }
    for (int T : {2048, 8192}) {
        std::mt19937_64 g(200 + T);
        std::vector<int32_t> ids((size_t) T * k);
        for (int t = 0; t < T; t++) {
            std::vector<int> perm(E);
            for (int i = 0; i < E; i++) { perm[i] = i; }
            std::shuffle(perm.begin(), perm.end(), g);
            for (int s = 0; s < k; s++) { ids[(size_t) t * k + s] = perm[s]; }
        }
        const int32_t * d_ids = dev_copy(ids);
        const std::vector<float> wts((size_t) T * k, 1.f / k);
        const float * d_w = dev_copy(wts);
        const uint16_t * x = dev_copy(normal_bf16((size_t) T * H, 1.f, 30));
        int32_t * src1, * dst, * bounds;
        CK(cudaMalloc(&src1, (size_t) T * k * 4)); CK(cudaMalloc(&dst, (size_t) T * k * 4)); CK(cudaMalloc(&bounds, (E + 1) * 4));
        uint16_t * act; float * ys, * y;
        CK(cudaMalloc(&act, (size_t) T * k * N * 2)); CK(cudaMalloc(&ys, (size_t) T * k * H * 4)); CK(cudaMalloc(&y, (size_t) T * H * 4));
        auto step = [&](int) {
            // gate/up: every slot of a token reads the token's row (sis1 = 0 in the reference's adapter: one x row per token)
            bf16n::mm_ids_route(d_ids, false, k, src1, dst, bounds, E, T, k, 1, 1, 0);
            bf16n::mm_ids(gate.w, &up.w, x, H, src1, dst, bounds, act, true, N, E, T, k, 0);
            // down: one activation row per (token, slot)
            bf16n::mm_ids_route(d_ids, false, k, src1, dst, bounds, E, T, k, k, k, 0);
            bf16n::mm_ids(down.w, nullptr, act, N, src1, dst, bounds, ys, false, H, E, T, k, 0);
            bf16n::moe_combine(ys, d_w, false, y, false, T, k, H, 0);
        };
        const double us = median_us(std::max(5, reps / 4), step);
        const double flops = 6.0 * N * H * k * T;
        printf("{\"impl\": \"%s\", \"workload\": \"MoE prefill layer, %d tokens\", \"us\": %.1f, \"TFLOPs\": %.1f, \"sum_abs_y\": %.6e}\n",
               IMPL_NAME, T, us, flops / us / 1e6, checksum(y, (size_t) T * H, "moe_prefill_" + std::to_string(T)));
#ifdef WITH_WORKSPACE
        {   // this library only: the same calls with a caller-owned workspace registered (two-pass form of mm_ids)
            const bf16n_weight cg = bf16n::detail::c(gate.w), cu = bf16n::detail::c(up.w);
            const size_t need = bf16n_mm_ids_workspace_bytes(&cg, &cu);
            void * ws = nullptr;
            CK(cudaMalloc(&ws, need));
            if (bf16n_set_workspace(ws, need) != BF16N_OK) { fprintf(stderr, "set_workspace: %s\n", bf16n_last_error()); exit(1); }
            const double us2 = median_us(std::max(5, reps / 4), step);
            printf("{\"impl\": \"%s\", \"workload\": \"MoE prefill layer, %d tokens, workspace registered (two-pass)\", \"us\": %.1f, \"TFLOPs\": %.1f, "
                   "\"sum_abs_y\": %.6e}\n", IMPL_NAME, T, us2, flops / us2 / 1e6, checksum(y, (size_t) T * H, "moe_prefill_ws_" + std::to_string(T)));
            CK(cudaDeviceSynchronize());
            bf16n_set_workspace(nullptr, 0);
            CK(cudaFree(ws));
        }
#endif
        CK(cudaFree(src1)); CK(cudaFree(dst)); CK(cudaFree(bounds)); CK(cudaFree(act)); CK(cudaFree(ys)); CK(cudaFree(y));
    }
}

int main(int argc, char ** argv) {
    const std::string what = argc > 1 ? argv[1] : "all";
    const int reps = argc > 2 ? atoi(argv[2]) : 50;
    bf16n::init();
    if (what == "lm_head" || what == "all") { lm_head(reps); }
    if (what == "moe_decode" || what == "all") { moe_decode(reps); }
    if (what == "moe_prefill" || what == "all") { moe_prefill(reps); }
    if (what == "small" || what == "all") { small(reps); }
    if (what == "frag_order" || what == "more") { frag_order(reps); }
    if (what == "frag_order_decode" || what == "more") { moe_decode(reps, true); }
    return 0;
}
