// The reference's launcher API (core/include/bf16n/launch.h:14-82) as inline wrappers over the C ABI: same struct
// fields, same signatures, std::invalid_argument / std::runtime_error as the reference throws.
#pragma once

#include "../bf16n_c.h"
#include "encode.h"

#include <cuda_runtime.h>

#include <cstdint>

namespace bf16n {

struct weight {
    const uint8_t * plane = nullptr;
    const uint8_t * aux = nullptr;
    int format = 0;
    int64_t K = 0, rows = 0;
    int R = 0;
    bool cm = false;
    bool fo = false;
    uint64_t off_a = 0, off_b = 0, off_c = 0, off_d = 0;
};

struct mmv_args {
    const void * x = nullptr; bool x_bf16 = false;
    void * y = nullptr;       bool y_bf16 = false;
    int ncols = 0;
    int64_t x_tok = 0, y_tok = 0;
    const void * ids = nullptr; int64_t ids_s0 = 0, ids_s1 = 0;
    int n_used = 1, x_per_slot = 1;
    int64_t x_slot = 0, y_slot = 0;
    int64_t rows_per_matrix = 0, row0 = 0, nrows = 0;
};

namespace detail {
inline bf16n_weight c(const weight & w) {
    return {w.plane, w.aux, w.format, w.R, w.K, w.rows, w.cm, w.fo, w.off_a, w.off_b, w.off_c, w.off_d};
}
inline bf16n_mmv_args c(const mmv_args & a) {
    bf16n_mmv_args r = {};
    r.x = a.x; r.x_bf16 = a.x_bf16; r.y = a.y; r.y_bf16 = a.y_bf16; r.ncols = a.ncols;
    r.n_used = a.n_used; r.x_per_slot = a.x_per_slot; r.x_tok = a.x_tok; r.y_tok = a.y_tok;
    r.ids = a.ids; r.ids_s0 = a.ids_s0; r.ids_s1 = a.ids_s1; r.x_slot = a.x_slot; r.y_slot = a.y_slot;
    r.rows_per_matrix = a.rows_per_matrix; r.row0 = a.row0; r.nrows = a.nrows;
    return r;
}
} // namespace detail

inline void init() { detail::raise(bf16n_init()); }
inline int sm_count() { int n = 0; detail::raise(bf16n_sm_count(&n)); return n; }

inline void mmv(const weight & w, const mmv_args & a, cudaStream_t stream, bool multi_col = true) {
    const bf16n_weight cw = detail::c(w); const bf16n_mmv_args ca = detail::c(a);
    detail::raise(bf16n_mmv(&cw, &ca, stream, multi_col));
}
inline void mmv_glu(const weight & w, const mmv_args & a, cudaStream_t stream) {
    const bf16n_weight cw = detail::c(w); const bf16n_mmv_args ca = detail::c(a);
    detail::raise(bf16n_mmv_glu_merged(&cw, &ca, stream));
}
inline void mmv_glu(const weight & gate, const weight & up, const mmv_args & a, cudaStream_t stream) {
    const bf16n_weight cg = detail::c(gate), cu = detail::c(up); const bf16n_mmv_args ca = detail::c(a);
    detail::raise(bf16n_mmv_glu(&cg, &cu, &ca, stream));
}
inline void dequant(const weight & w, int64_t row0, int64_t nrows, uint16_t * out, cudaStream_t stream) {
    const bf16n_weight cw = detail::c(w);
    detail::raise(bf16n_dequant(&cw, row0, nrows, out, stream));
}
inline void get_rows(const weight & w, const void * ids, int64_t ids_s0, int64_t n, void * dst, bool dst_bf16, int64_t dst_s1,
                     cudaStream_t stream, int64_t row0 = 0) {
    const bf16n_weight cw = detail::c(w);
    detail::raise(bf16n_get_rows(&cw, ids, ids_s0, n, dst, dst_bf16, dst_s1, stream, row0));
}
inline bool mm_ids_supported(const weight & w, const weight * up) {
    const bf16n_weight cw = detail::c(w);
    if (!up) { return bf16n_mm_ids_supported(&cw, nullptr) != 0; }
    const bf16n_weight cu = detail::c(*up);
    return bf16n_mm_ids_supported(&cw, &cu) != 0;
}
inline void mm_ids_route(const void * ids, bool ids_i64, int64_t ids_row_stride, int32_t * ids_src1, int32_t * ids_dst,
                         int32_t * bounds, int n_experts, int n_tok, int n_used, int nchannels_y, int sis1, cudaStream_t stream) {
    detail::raise(bf16n_mm_ids_route(ids, ids_i64, ids_row_stride, ids_src1, ids_dst, bounds, n_experts, n_tok, n_used, nchannels_y,
                                     sis1, stream));
}
inline void mm_ids(const weight & w, const weight * up, const void * x_bf16, int64_t x_row, const int32_t * ids_src1,
                   const int32_t * ids_dst, const int32_t * bounds, void * dst, bool dst_bf16, int64_t dst_col, int n_experts,
                   int n_tok, int n_used, cudaStream_t stream) {
    const bf16n_weight cw = detail::c(w);
    bf16n_weight cu = {};
    if (up) { cu = detail::c(*up); }
    detail::raise(bf16n_mm_ids(&cw, up ? &cu : nullptr, x_bf16, x_row, ids_src1, ids_dst, bounds, dst, dst_bf16, dst_col, n_experts,
                               n_tok, n_used, stream));
}
inline void moe_combine(const float * ys, const void * w, bool w_bf16, void * y, bool y_bf16, int n_tok, int n_used, int64_t n,
                        cudaStream_t stream) {
    detail::raise(bf16n_moe_combine(ys, w, w_bf16, y, y_bf16, n_tok, n_used, n, stream));
}
inline void swiglu(const float * g, const float * u, float * y, int64_t n, cudaStream_t stream) {
    detail::raise(bf16n_swiglu(g, u, y, n, stream));
}

// draft-only k-bit output head (core/include/bf16n/draft_head.cuh:224-281; the reference declares these in
// core/torch/torch_bindings.cpp:22-29 rather than in a header). sm_count is accepted for source compatibility.
inline void int4_quantize(const void * w_bf16, int64_t rows, int K, uint8_t * q, float * s, cudaStream_t stream) {
    detail::raise(bf16n_int4_quantize(w_bf16, rows, K, q, s, stream));
}
inline void int4_gemv(const void * x_bf16, int T, const uint8_t * q, const float * s, int64_t rows, int K, float * y, int /*sm_count*/,
                      cudaStream_t stream) {
    detail::raise(bf16n_int4_gemv(x_bf16, T, q, s, rows, K, y, stream));
}
inline void int2_quantize(const void * w_bf16, int64_t rows, int K, uint8_t * q, float * s, cudaStream_t stream) {
    detail::raise(bf16n_int2_quantize(w_bf16, rows, K, q, s, stream));
}
inline void int2_gemv(const void * x_bf16, int T, const uint8_t * q, const float * s, int64_t rows, int K, float * y, int /*sm_count*/,
                      cudaStream_t stream) {
    detail::raise(bf16n_int2_gemv(x_bf16, T, q, s, rows, K, y, stream));
}

} // namespace bf16n
