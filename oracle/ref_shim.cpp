// C entry points over the UNMODIFIED reference encoder and shape policy, for use as the byte-level oracle.
// TEST INFRASTRUCTURE ONLY. This file is compiled together with the reference project's own core/src/encode.cpp and
// core/src/policy.cpp, read in place from the reference checkout (see Makefile: REF=...), into oracle/_ref/. It
// contains no reference code: it only calls bf16n::encode (core/include/bf16n/encode.h:26) and bf16n::choose
// (core/include/bf16n/policy.h:37).
#include "bf16n/encode.h"
#include "bf16n/policy.h"

#include <cstdlib>
#include <cstring>
#include <stdexcept>

extern "C" {

// 0 ok; 1 std::invalid_argument; 2 any other exception. plane: rows*K bytes (caller); *aux malloc'd (ref_free).
int ref_encode(const uint16_t * w, int64_t rows, int64_t K, int format, int R, int cm, int fo, uint8_t * plane,
               uint8_t ** aux, uint64_t * aux_len, int * fmt_out, int * R_out) {
    try {
        const bf16n::encoded e = bf16n::encode(w, rows, K, format, R, cm != 0, fo != 0);
        memcpy(plane, e.plane.data(), e.plane.size());
        *aux = (uint8_t *) malloc(e.aux.size());
        memcpy(*aux, e.aux.data(), e.aux.size());
        *aux_len = e.aux.size();
        *fmt_out = e.format;
        *R_out = e.R;
        return 0;
    } catch (const std::invalid_argument &) {
        return 1;
    } catch (...) {
        return 2;
    }
}

void ref_free(void * p) { free(p); }

// out = {format, R, chunk_major, frag_order}; returns 1 when the policy picks a BF16N format, 0 for "stays BF16".
int ref_choose(int64_t rows, int64_t K, int64_t n_matrices, int engine, int mode, int64_t dense_min, int expert,
               int dense_frag_order, int * out) {
    bf16n::policy_options o;
    o.engine = engine ? bf16n::policy_engine::vllm : bf16n::policy_engine::llama;
    o.mode = mode == 0 ? bf16n::policy_mode::hybrid : mode == 1 ? bf16n::policy_mode::huffman : bf16n::policy_mode::nibble;
    o.dense_min = dense_min;
    o.expert = expert != 0;
    o.dense_frag_order = dense_frag_order != 0;
    const auto c = bf16n::choose(rows, K, n_matrices, o);
    if (!c) { return 0; }
    out[0] = c->format; out[1] = c->R; out[2] = c->chunk_major; out[3] = c->frag_order;
    return 1;
}

} // extern "C"
