// Batched (prefill) routed product. Placeholder translation unit: the tensor-core kernel is added separately.
#include "launch.h"

namespace b16 {

void prefill_init() {}

bool prefill_supported(const bf16n_weight & w, const bf16n_weight * up) {
    const int C = (int) (w.K / CHUNK);
    const bool shape = w.format == FMT_HUFPAIR && !w.fo && (w.cm || w.K == CHUNK) && ((C == 4 && w.R == 8) || (C == 1 && w.R == 16));
    if (!up) { return shape; }
    const bool same = up->format == w.format && up->K == w.K && up->R == w.R && up->cm == w.cm && up->fo == w.fo && up->rows == w.rows;
    return same && w.format == FMT_HUFPAIR && w.K == 2048 && w.cm && w.R == 8;
}

void prefill_mm_ids(const bf16n_weight &, const bf16n_weight *, const void *, int64_t, const int32_t *, const int32_t *,
                    const int32_t *, void *, bool, int64_t, int, int, int, cudaStream_t) {
    throw std::runtime_error("bf16n: batched kernel not built");
}

} // namespace b16
