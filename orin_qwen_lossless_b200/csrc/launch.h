// Internal interface between the C ABI (capi.cu) and the kernel translation units.
#pragma once

#include "../../include/bf16n_c.h"
#include "format.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <stdexcept>
#include <string>

namespace b16 {

void set_last_error(const std::string & message); // what bf16n_last_error() returns on this thread (capi.cu)

struct DeviceInfo { int sms = 0; int smem_optin = 0; };
const DeviceInfo & device_info(); // filled by bf16n_init

[[noreturn]] inline void fail_invalid(const std::string & m) { throw std::invalid_argument("bf16n: " + m); }
inline void require(bool ok, const char * m) { if (!ok) { fail_invalid(m); } }
inline void cuda_ok(cudaError_t e, const char * what) {
    if (e != cudaSuccess) { throw std::runtime_error(std::string("bf16n: CUDA error ") + cudaGetErrorString(e) + " at " + what); }
}
inline void check_launch() { cuda_ok(cudaGetLastError(), "kernel launch"); }
// Lets `kernel` use up to `bytes` of dynamic shared memory, capped at the device's opt-in limit less whatever the
// kernel declares statically (the limit covers both together).
inline void allow_dynamic_smem(const void * kernel, int bytes, int optin, const char * what) {
    cudaFuncAttributes fa;
    cuda_ok(cudaFuncGetAttributes(&fa, kernel), what);
    cuda_ok(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, std::min(bytes, optin - (int) fa.sharedSizeBytes)), what);
}

#ifdef __CUDACC__
// Launch of a kernel that may start while the kernel before it on the stream is still draining (programmatic dependent
// launch): such a kernel calls grid_dependency_wait() before it touches anything an earlier kernel wrote or still reads,
// and does only independent work (tables, barriers) above that line. Works under stream capture as well.
template <typename... KArgs, typename... Args>
void launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t shm, cudaStream_t st, Args &&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = shm; cfg.stream = st;
    cudaLaunchAttribute attr = {};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr; cfg.numAttrs = 1;
    cuda_ok(cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...), "kernel launch");
}
// Blocks until every kernel this one depends on has completed and its writes are visible; then lets the next kernel on
// the stream begin its own prologue.
__device__ __forceinline__ void grid_dependency_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
#endif

// gemv.cu
void gemv_init();
void gemv(const bf16n_weight & w, const bf16n_mmv_args & a, cudaStream_t st, bool multi_col, const bf16n_peer_out * peers = nullptr);
bool gemv_groupable(const bf16n_weight & w, const bf16n_mmv_args & a);
void gemv_group(const bf16n_weight * w, const bf16n_mmv_args * a, int n, cudaStream_t st);
void gemv_glu_merged(const bf16n_weight & w, const bf16n_mmv_args & a, cudaStream_t st);
void gemv_glu(const bf16n_weight & g, const bf16n_weight & u, const bf16n_mmv_args & a, cudaStream_t st);
void expand_store(const bf16n_weight & w, int64_t row0, int64_t nrows, uint16_t * out, cudaStream_t st);
void expand_compare(const bf16n_weight & w, int64_t row0, int64_t nrows, const uint16_t * src, unsigned long long * total,
                    cudaStream_t st);
void gather_rows(const bf16n_weight & w, const void * ids, int64_t ids_s0, int64_t n, void * dst, bool dst_bf16, int64_t dst_s1,
                 int64_t row0, cudaStream_t st);

// device addresses of the words the kernels set when one of their bounded waits runs out (bf16n_fault_status)
unsigned int * gemv_staged_fault_word();
unsigned int * moe_decode_fault_word();
unsigned int * fo_fault_word();
unsigned int * prefill_fault_word();

// gemv_staged.cu
void gemv_staged_init();
bool gemv_staged_applies(const bf16n_weight & w, const bf16n_mmv_args & a);
void gemv_staged(const bf16n_weight & w, const bf16n_mmv_args & a, cudaStream_t st, const bf16n_peer_out * peers = nullptr);

// gemv_rings.cu
void gemv_rings_init();
bool gemv_rings_enabled();
bool gemv_rings_applies(const bf16n_weight & w, const bf16n_mmv_args & a);
void gemv_rings(const bf16n_weight & w, const bf16n_mmv_args & a, cudaStream_t st, bool multi_col, const bf16n_peer_out * peers = nullptr);

// fo.cu: fragment-order HUFPAIR tensors
void fo_init();
bool fo_supported(const bf16n_weight & w);
void fo_gemv(const bf16n_weight & w, const bf16n_mmv_args & a, cudaStream_t st);
bool fo_mm_ids_supported(const bf16n_weight & w, const bf16n_weight * up);
void fo_mm_ids(const bf16n_weight & w, const bf16n_weight * up, const void * x_bf16, int64_t x_row, const int32_t * ids_src1,
               const int32_t * ids_dst, const int32_t * bounds, void * dst, bool dst_bf16, int64_t dst_col, int n_experts,
               cudaStream_t st);
void fo_expand_store(const bf16n_weight & w, int64_t row0, int64_t nrows, uint16_t * out, cudaStream_t st);
void fo_expand_compare(const bf16n_weight & w, int64_t row0, int64_t nrows, const uint16_t * src, unsigned long long * total,
                       cudaStream_t st);
void fo_gather_rows(const bf16n_weight & w, const void * ids, int64_t ids_s0, int64_t n, void * dst, bool dst_bf16, int64_t dst_s1,
                    int64_t row0, cudaStream_t st);

// peer.cu: exchange buffers shared between the GPUs of a node and the wait for the peers' announcements
void peer_wait(uint32_t * local_header, int n_peers_mask, cudaStream_t st);

// ep_prefill.cu: expert-parallel prefill, rows exchanged with peer stores
size_t ep_layout_fill(bf16n_ep_layout & l);
void ep_dispatch(const bf16n_ep_layout & l, const void * x_bf16, int64_t x_row, const int32_t * ids, int n_tok, int n_used, int n_experts,
                 int32_t * plan, cudaStream_t st);
void ep_inbox_ids(const bf16n_ep_layout & l, int32_t * ids_out, cudaStream_t st);
void ep_give_back(const bf16n_ep_layout & l, const float * ys, cudaStream_t st);

// moe.cu
void moe_init();
void moe_topk(const float * logits, int n_tok, int n_experts, int k, int32_t * ids, float * weights, cudaStream_t st);
void moe_combine(const float * ys, const void * w, bool w_bf16, void * y, bool y_bf16, int n_tok, int n_used, int64_t n, cudaStream_t st);
void moe_swiglu(const float * g, const float * u, float * y, int64_t n, cudaStream_t st);
void moe_route(const void * ids, bool ids_i64, int64_t ids_row_stride, int32_t * ids_src1, int32_t * ids_dst, int32_t * bounds,
               int n_experts, int n_tok, int n_used, int nchannels_y, int sis1, cudaStream_t st);

// moe_decode.cu
void moe_decode_init();
bool expert_units_applies(const bf16n_weight & w, const bf16n_mmv_args & a);
void expert_units_mmv(const bf16n_weight & w, const bf16n_mmv_args & a, cudaStream_t st);
bool moe_decode_supported(const bf16n_weight & gate, const bf16n_weight & up, const bf16n_weight & down);
void moe_decode(const bf16n_weight & gate, const bf16n_weight & up, const bf16n_weight & down, const void * x, bool x_bf16,
                int64_t x_tok, const int32_t * ids, const float * weights, int n_tok, int n_used, int n_experts_local, int e_lo,
                float * scratch, void * y, bool y_bf16, cudaStream_t st, const bf16n_peer_out * peers = nullptr);
void moe_decode_frag_order(const bf16n_weight & gate, const bf16n_weight & up, const bf16n_weight & down, const void * x, bool x_bf16,
                           int64_t x_tok, const int32_t * ids, const float * weights, int n_tok, int n_used, int n_experts,
                           float * scratch, void * y, bool y_bf16, cudaStream_t st);
void peer_sum(const float * parts, int n_parts, int64_t n, const float * extra, void * y, bool y_bf16, cudaStream_t st);

size_t moe_decode_static_capacity_floats();
void moe_decode_static(const bf16n_weight & gate, const bf16n_weight & up, const bf16n_weight & down, const void * x, bool x_bf16,
                       int64_t x_tok, const int32_t * ids, const float * weights, int n_tok, int n_used, int n_experts_local,
                       int e_lo, void * y, bool y_bf16, cudaStream_t st);

// draft.cu: draft-only 2-bit / 4-bit copies of an output head
void draft_quantize(int bits, const void * w_bf16, int64_t rows, int K, uint8_t * q, float * s, cudaStream_t st);
void draft_gemv(int bits, const void * x_bf16, int T, const uint8_t * q, const float * s, int64_t rows, int K, float * y, cudaStream_t st);

// prefill.cu
void prefill_init();
void expand_tiles_init();
bool expand_tiles_supported(const bf16n_weight & w);
void expand_tiles(const bf16n_weight & w, const bf16n_weight * up, int n_experts, const int32_t * bounds, void * images, cudaStream_t st);
void prefill_set_workspace(void * p, size_t bytes);
size_t prefill_workspace_bytes(const bf16n_weight & w, const bf16n_weight * up);
bool prefill_supported(const bf16n_weight & w, const bf16n_weight * up);
void prefill_mm_ids(const bf16n_weight & w, const bf16n_weight * up, const void * x_bf16, int64_t x_row, const int32_t * ids_src1,
                    const int32_t * ids_dst, const int32_t * bounds, void * dst, bool dst_bf16, int64_t dst_col, int n_experts,
                    int n_tok, int n_used, cudaStream_t st);

} // namespace b16
