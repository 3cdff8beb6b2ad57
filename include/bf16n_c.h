/* C ABI of the B200 (sm_100a) BF16N library: libbf16n_b200.so.
 *
 * Every entry point replaces one function of the reference project's C++ core (namespace bf16n); the comment on each
 * declaration names it by file:line inside the reference checkout.  Conventions:
 *   - plain C types only; device pointers are ordinary pointers into CUDA device memory owned by the caller;
 *   - `stream` is a cudaStream_t passed as void*; launchers only enqueue work on it: no allocation, no host
 *     synchronisation, no environment lookups, so every launch can be captured into a CUDA graph after bf16n_init();
 *   - return value: BF16N_OK, or an error code with a message in bf16n_last_error() (thread-local). The reference
 *     throws std::invalid_argument where this returns BF16N_EINVAL and std::runtime_error elsewhere; the C++ wrappers
 *     in include/bf16n/ re-throw exactly those.
 */
#ifndef BF16N_C_H
#define BF16N_C_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { BF16N_OK = 0, BF16N_EINVAL = 1, BF16N_ECUDA = 2, BF16N_EINTERNAL = 3 };

enum { BF16N_FMT_NIBBLE = 1, BF16N_FMT_HUFFMAN = 2, BF16N_FMT_HUFPAIR = 3 }; /* core/include/bf16n/format.h:12-14 */
enum { BF16N_FLAG_CHUNK_MAJOR = 1, BF16N_FLAG_FRAG_ORDER = 2 };             /* format.h:27-33 */

/* Device view of one encoded matrix; fields parsed once on the host from the aux header.
 * Replaces struct bf16n::weight (core/include/bf16n/launch.h:14-23). */
typedef struct bf16n_weight {
    const uint8_t * plane; /* rows*K sign|mantissa bytes (device) */
    const uint8_t * aux;   /* header + exponent data (device) */
    int32_t format;
    int32_t R;             /* rows per unit; 0 for NIBBLE */
    int64_t K;
    int64_t rows;
    int32_t cm;            /* HUFPAIR chunk-major units */
    int32_t fo;            /* HUFPAIR fragment-order bands */
    uint64_t off_a, off_b, off_c, off_d;
} bf16n_weight;

/* One matrix-vector product call: y[col] = W[rbase : rbase+nrows] x[col] for ncols columns.
 * Dense: column c = token c, rbase = row0.  With ids: column c = (token c / n_used, slot c % n_used), expert
 * e = ids[token, slot], rbase = row0 + e*rows_per_matrix; x of a column at x_tok*token + x_slot*(slot % x_per_slot),
 * y at y_tok*token + y_slot*slot.  Strides are signed byte counts; ids are int32, or int64 < 2^31 (low word read).
 * Replaces struct bf16n::mmv_args (launch.h:27-41). */
typedef struct bf16n_mmv_args {
    const void * x; int32_t x_bf16;
    void * y;       int32_t y_bf16;
    int32_t ncols;
    int32_t n_used, x_per_slot;
    int64_t x_tok, y_tok;
    const void * ids; int64_t ids_s0, ids_s1;
    int64_t x_slot, y_slot;
    int64_t rows_per_matrix, row0, nrows;
} bf16n_mmv_args;

const char * bf16n_last_error(void);

/* ---- host side ------------------------------------------------------------------------------------------------ */

/* Opaque result of bf16n_encode. Replaces struct bf16n::encoded (core/include/bf16n/encode.h:12-17). */
typedef struct bf16n_encoded bf16n_encoded;

/* Encode rows x K BF16 bit patterns (host memory, row-major) on all host threads.
 * Replaces bf16n::encode (encode.h:26, core/src/encode.cpp:443-526): same argument rules, same bytes. */
int bf16n_encode(const uint16_t * w, int64_t rows, int64_t K, int format, int R, int chunk_major, int frag_order,
                 bf16n_encoded ** out);
const uint8_t * bf16n_encoded_plane(const bf16n_encoded * e, size_t * nbytes);
const uint8_t * bf16n_encoded_aux(const bf16n_encoded * e, size_t * nbytes);
int bf16n_encoded_format(const bf16n_encoded * e);
int bf16n_encoded_R(const bf16n_encoded * e);
void bf16n_encoded_free(bf16n_encoded * e);

/* Fill every field of *w except the two device pointers from the first 256 bytes of a HOST copy of the aux buffer.
 * Replaces the header parse each engine does once per tensor (engines/vllm/vllm_bf16n/ops.py:54-63;
 * engines/llamacpp/patches/0002 bf16n.cu registry insert). */
int bf16n_parse_header(const uint8_t * aux_host, size_t nbytes, bf16n_weight * w);

/* Shape policy. engine: 0 llama, 1 vllm; mode: 0 hybrid, 1 huffman, 2 nibble. out = {format, R, chunk_major,
 * frag_order}. Returns 1 when a format was chosen, 0 when the shape stays BF16 (never fails).
 * Replaces bf16n::choose (core/include/bf16n/policy.h:37, core/src/policy.cpp:45-69). */
int bf16n_choose(int64_t rows, int64_t K, int64_t n_matrices, int engine, int mode, int64_t dense_min, int expert,
                 int dense_frag_order, int out[4]);

/* bf16n_choose with the machine size as an argument: a dense pair-Huffman matrix keeps at least min_units units (the
 * reference hard-codes 512, the warps of the GPU it was written for; bf16n_choose keeps that constant and its tables).
 * A loader that splits a matrix over several B200s asks with min_units of the order of SMs x warps per SM (e.g.
 * 148 x 24), so that a small shard gets shorter units and still fills the machine. */
int bf16n_choose_for_machine(int64_t rows, int64_t K, int64_t n_matrices, int engine, int mode, int64_t dense_min, int expert,
                             int dense_frag_order, int64_t min_units, int out[4]);

/* ---- device side ---------------------------------------------------------------------------------------------- */

/* Once per process, with the process's GPU current, before the first launch and before any graph capture: device
 * attributes and the kernels' shared-memory limits. One process drives one device (one process per GPU): every later
 * call checks that the device bf16n_init ran on is still the current one and returns BF16N_EINVAL otherwise.
 * Replaces bf16n::init / bf16n::sm_count (launch.h:45-46, core/src/launch.cu:270-311). */
int bf16n_init(void);
int bf16n_sm_count(int * out);

/* Every wait inside a kernel is bounded (bulk copies completing on an mbarrier, tensor-core commits). When one runs out
 * the kernel sets a status word, writes NaN where the affected work item's outputs go and finishes, so the context stays
 * usable. This call synchronises the stream, returns the status words since the last call as a bit mask and clears
 * them: bit 0 the bulk-copy staged GEMV, bit 1 the MoE decode unit kernels, bit 2 the fragment-order kernels, bit 3 the
 * batched (prefill) kernel. 0 means every launch so far wrote complete outputs. Not capturable (it synchronises).
 * The reference has no bounded waits and nothing like this. */
#define BF16N_FAULT_GEMV_STAGED 1u
#define BF16N_FAULT_MOE_DECODE 2u
#define BF16N_FAULT_FRAG_ORDER 4u
#define BF16N_FAULT_PREFILL 8u
int bf16n_fault_status(unsigned int * flags, void * stream);

/* GEMV (<= a few columns), dense or routed by expert ids. multi_col != 0: dense batches of 2..4 columns decode the
 * matrix once per group of 4. Replaces bf16n::mmv (launch.h:50, launch.cu:313-325). */
int bf16n_mmv(const bf16n_weight * w, const bf16n_mmv_args * a, void * stream, int multi_col);
/* n independent products on one stream, w[i] with a[i]: the small dense NIBBLE products among them (K 512..4096, up to
 * 8 columns; the per-layer projections and routers that are each too small to fill the GPU) share one grid, eight
 * products per launch, instead of one launch each; everything else is launched as bf16n_mmv would launch it. Results
 * are the bits bf16n_mmv gives for each product. The reference launches every product on its own
 * (core/src/launch.cu:313-325); this is the B200 answer to its launch-bound small-matrix path. */
int bf16n_mmv_group(const bf16n_weight * w, const bf16n_mmv_args * a, int n, void * stream);
/* y = silu(gate x) * (up x) for a NIBBLE matrix whose rows_per_matrix rows are [gate (nrows); up (nrows)].
 * Replaces bf16n::mmv_glu(w, a, stream) (launch.h:53, launch.cu:327-339). */
int bf16n_mmv_glu_merged(const bf16n_weight * w, const bf16n_mmv_args * a, void * stream);
/* Same with separate gate and up matrices (NIBBLE, row-major HUFPAIR, HUFFMAN).
 * Replaces bf16n::mmv_glu(gate, up, a, stream) (launch.h:60, launch.cu:341-365). */
int bf16n_mmv_glu(const bf16n_weight * gate, const bf16n_weight * up, const bf16n_mmv_args * a, void * stream);
/* Exact BF16 bits of rows [row0, row0+nrows) into out (device, row-major nrows x K).
 * Replaces bf16n::dequant (launch.h:62, launch.cu:367-402). */
int bf16n_dequant(const bf16n_weight * w, int64_t row0, int64_t nrows, uint16_t * out, void * stream);
/* Verify-at-load without materialising the tensor: decodes rows [row0, row0+nrows) and adds the number of BF16 words
 * that differ from src (device, row-major, row 0 = row0) to *mismatches (device, caller zeroes it).
 * Replaces the dequant + compare loop of engines/vllm/vllm_bf16n/ops.py:104-116 (roundtrip_equal). */
int bf16n_verify(const bf16n_weight * w, int64_t row0, int64_t nrows, const uint16_t * src, unsigned long long * mismatches,
                 void * stream);
/* dst[i] = W[row0 + ids[i]] as FP32 or BF16 (row gather for embeddings). Replaces bf16n::get_rows (launch.h:67-68,
 * launch.cu:404-443). */
int bf16n_get_rows(const bf16n_weight * w, const void * ids, int64_t ids_s0, int64_t n, void * dst, int dst_bf16,
                   int64_t dst_s1, void * stream, int64_t row0);

/* Batched (prefill) routed product. Replaces bf16n::mm_ids_supported / mm_ids_route / mm_ids (launch.h:73-78,
 * launch.cu:446-535; routing semantics core/src/mmid_helper.cu:4-8). */
int bf16n_mm_ids_supported(const bf16n_weight * w, const bf16n_weight * up);
int bf16n_mm_ids_route(const void * ids, int ids_i64, int64_t ids_row_stride, int32_t * ids_src1, int32_t * ids_dst,
                       int32_t * bounds, int n_experts, int n_tok, int n_used, int nchannels_y, int sis1, void * stream);
int bf16n_mm_ids(const bf16n_weight * w, const bf16n_weight * up, const void * x_bf16, int64_t x_row,
                 const int32_t * ids_src1, const int32_t * ids_dst, const int32_t * bounds, void * dst, int dst_bf16,
                 int64_t dst_col, int n_experts, int n_tok, int n_used, void * stream);


/* No reference counterpart: a caller-owned device buffer for the two-pass form of bf16n_mm_ids. With a workspace of at
 * least bf16n_mm_ids_workspace_bytes(w, up) bytes registered, bf16n_mm_ids on lane-major HUFPAIR experts first decodes the
 * experts that have routed pairs into BF16 operand tiles in the workspace (every SM's warps decoding, no tensor core)
 * and then multiplies from those tiles on the tensor cores (bulk copies into shared memory, tcgen05.mma with N = 256);
 * without one (the default), or when it is too small, the fused decode-and-multiply kernel runs. Results of the two
 * forms agree to FP32 accumulation order, not bitwise. The library never allocates or frees the buffer; it is used by
 * the launches of one stream at a time and must stay valid while they (or CUDA graphs captured from them) can run.
 * workspace = NULL withdraws it. bf16n_mm_ids_workspace_bytes returns 0 for matrices the two-pass form does not take
 * (fragment order, NIBBLE, other unit shapes): rows * K * 2 bytes for one matrix, twice that for a gate/up pair. */
size_t bf16n_mm_ids_workspace_bytes(const bf16n_weight * w, const bf16n_weight * up);
int bf16n_set_workspace(void * workspace, size_t bytes);
/* y[t, i] = sum_k w[t, k] * ys[t, k, i] in slot order (FP32). Replaces bf16n::moe_combine (launch.h:81-82,
 * launch.cu:539-572). */
int bf16n_moe_combine(const float * ys, const void * w, int w_bf16, void * y, int y_bf16, int n_tok, int n_used, int64_t n,
                      void * stream);
/* y = silu(g) * u elementwise. Replaces bf16n::swiglu (launch.h:84, launch.cu:554-582). */
int bf16n_swiglu(const float * g, const float * u, float * y, int64_t n, void * stream);

/* Draft-only k-bit copies of an output head: q / s are a 4-bit (q [rows, K / 2], value + 8 per nibble, even column
 * low) or 2-bit (q [rows, K / 4], level n of column c in bits 2 (c % 16) of 32-bit word c / 16, value (n - 1.5) s)
 * copy of a BF16 matrix with one FP32 scale per 128 weights (s [rows, K / 128]); the GEMVs return approximate FP32
 * scores y [T, rows] (T <= 4; int4: K 1024 / 2048 / 4096, int2: K = 2048) that only choose which rows the caller
 * re-scores exactly. Same stored formats and argument rules as the reference. Replaces bf16n::int4_quantize /
 * int4_gemv / int2_quantize / int2_gemv (core/include/bf16n/draft_head.cuh:224-281, declared at
 * core/torch/torch_bindings.cpp:22-29; sm_count is taken from bf16n_init). */
int bf16n_int4_quantize(const void * w_bf16, int64_t rows, int K, uint8_t * q, float * s, void * stream);
int bf16n_int4_gemv(const void * x_bf16, int T, const uint8_t * q, const float * s, int64_t rows, int K, float * y, void * stream);
int bf16n_int2_quantize(const void * w_bf16, int64_t rows, int K, uint8_t * q, float * s, void * stream);
int bf16n_int2_gemv(const void * x_bf16, int T, const uint8_t * q, const float * s, int64_t rows, int K, float * y, void * stream);

/* Router on the GPU: softmax over n_experts logits per token, the k largest (ties: lowest index), weights renormalised
 * to sum 1. The reference core takes ids and weights from its engines (tests/core/test_kernels.py:333-345 synthesise
 * them); this keeps the 1-4 token decode step on the device. logits FP32 [n_tok, n_experts]; ids int32 [n_tok, k];
 * weights FP32 [n_tok, k]. */
int bf16n_moe_topk(const float * logits, int n_tok, int n_experts, int k, int32_t * ids, float * weights, void * stream);

/* One MoE decode step (1..64 tokens) of the routed experts, entirely on the device:
 *   router (when router_logits != NULL: softmax top-n_used of n_experts logits per token into topk_ids / topk_weights;
 *   otherwise those two arrays are inputs) -> gate and up products of every (token, slot) in one launch -> down product
 *   reading silu(gate) * up directly -> weighted sum over the slots in slot order.
 * It replaces the five-launch sequence of the reference's Python layer (engines/vllm/vllm_bf16n/ops.py:267-271:
 * mmv, mmv, swiglu, mmv, moe_combine) and its host-side router; results are bit-identical to that sequence with an
 * FP32 combine. gate/up: chunk-major HUFPAIR R = 8, K = 2048; down: row-major HUFPAIR R = 16, K = rows per expert of
 * gate. Expert parallelism: the three weights hold experts [expert_lo, expert_lo + n_experts_local) of n_experts;
 * slots routed elsewhere contribute exact zeros, so ranks' outputs add up to the full layer.
 * scratch: device memory, bf16n_moe_decode_scratch_bytes(...) bytes, 16-byte aligned, owned by the caller. */
size_t bf16n_moe_decode_scratch_bytes(int n_tok, int n_used, int64_t rows_gate_per_expert, int64_t rows_down_per_expert);
int bf16n_moe_decode(const bf16n_weight * gate, const bf16n_weight * up, const bf16n_weight * down, const void * x, int x_bf16,
                     int64_t x_tok, const float * router_logits, int n_experts, int32_t * topk_ids, float * topk_weights, int n_tok,
                     int n_used, int expert_lo, int n_experts_local, float * scratch, size_t scratch_bytes, void * y, int y_bf16,
                     void * stream);

/* bf16n_moe_decode for callers that cannot allocate device memory. It has no counterpart in the reference.
 *
 * Who needs it: code that runs a decode step at a point where cudaMalloc is not an option - an engine whose device
 * memory was all committed to a fixed arena when the model was loaded, or a serving loop that must stay clear of the
 * allocator because an allocation synchronises the device. bf16n_moe_decode asks such a caller for a scratch buffer it
 * cannot provide; this entry point uses a buffer that is part of the library image instead and calls neither
 * cudaMalloc nor cudaFree nor any allocating library routine.
 *
 * Same arguments, checks and results as bf16n_moe_decode (bit for bit), without scratch / scratch_bytes. Limits:
 *   - the step must fit the built-in buffer: n_tok * n_used * (2 * rows_gate_per_expert + rows_down_per_expert) <=
 *     BF16N_MOE_DECODE_STATIC_MAX_FLOATS (8 tokens x 8 slots of 512-row gate/up and 2048-row down experts); larger steps
 *     are rejected with BF16N_EINVAL and a message naming both sizes;
 *   - the buffer (768 KB) is held by every GPU that loads the library until the process exits;
 *   - the first call on a device looks up the buffer's device address (the device must be current); make that first
 *     call before any stream capture begins;
 *   - all calls on a device share the one buffer, which keeps whatever the last call wrote. Nothing in it needs to be
 *     cleared (each launch overwrites what the next one reads), but two calls whose kernels overlap on the GPU -
 *     different streams, or graphs replayed concurrently - race on it: serialise them, or use bf16n_moe_decode with
 *     one scratch buffer per stream. */
#define BF16N_MOE_DECODE_STATIC_MAX_FLOATS 196608
int bf16n_moe_decode_static(const bf16n_weight * gate, const bf16n_weight * up, const bf16n_weight * down, const void * x, int x_bf16,
                            int64_t x_tok, const float * router_logits, int n_experts, int32_t * topk_ids, float * topk_weights,
                            int n_tok, int n_used, int expert_lo, int n_experts_local, void * y, int y_bf16, void * stream);

/* ---- loader side of the llama.cpp adapter -------------------------------------------------------------------------
 * The engine-independent half of ggml-cuda/bf16n.cu (engines/llamacpp/patches/0002-ggml-cuda-thin-BF16N-adapter-over-
 * the-shared-core.patch, patch lines 47-332): a registry keyed by the device address range of every converted tensor's
 * plane, so that a tensor's data pointer, or a view that starts on a later row, finds its encoded matrix again.
 * Load-time calls: they allocate and synchronise.
 *
 * choose   ggml's conversion ABI (patch lines 274-283, ggml_backend_cuda_bf16n_choose): 0 = stays BF16, 1 = NIBBLE,
 *          2 = Huffman (pairs with single-symbol fallback), by the llama shape policy; mode "hybrid" | "huffman" | "nibble".
 * convert  patch lines 285-332 (ggml_backend_cuda_bf16n_convert): encodes the host BF16 tensor [n_matrices,
 *          rows_per_matrix, K] with the layout the llama policy picks for format_tag (1 or 2), copies the plane into
 *          plane_dev (the tensor's own device storage, rows * K bytes), allocates the aux buffer, registers the range
 *          for `owner` (the engine's buffer handle) and decodes every row on the device against the source in chunks
 *          of at most 64 MiB; prints one line per tensor to stderr in the reference's format; *roundtrip_ok = 1 when
 *          every weight came back bit-exact.
 * lookup   patch lines 69-87: 1 and the matrix (by value) plus the first row of the view when `data` lies inside a
 *          registered plane on a row boundary, else 0.
 * release  patch lines 118-129 (ggml_cuda_bf16n_free): frees the aux buffers of everything `owner` registered; returns
 *          how many. Call before the owning buffer is freed. */
int bf16n_adapter_choose(int64_t rows, int64_t K, int64_t n_matrices, const char * mode, int64_t dense_min, int expert);
int bf16n_adapter_convert(void * plane_dev, const void * bf16_host, int64_t K, int64_t rows_per_matrix, int64_t n_matrices,
                          int format_tag, const void * owner, const char * name, int * roundtrip_ok);
int bf16n_adapter_lookup(const void * data, bf16n_weight * out, int64_t * row0);
int bf16n_adapter_release(const void * owner);
int bf16n_adapter_count(void);

/* ---- multi-GPU: outputs written straight into the other GPUs of the node ------------------------------------------
 * New: the reference is single-GPU and has nothing like this. A row-sharded projection normally ends with a collective
 * that gathers the shards; here the GEMV kernel itself stores every logit it produces into each peer's buffer as well
 * (plain stores to peer memory over NVLink), and the last block to finish publishes an epoch number in the peers'
 * headers. A consumer waits for the epochs of all its peers with bf16n_peer_wait (one tiny kernel) instead of running a
 * collective. No multicast, no library collective on this path.
 *
 * An exchange buffer is [256-byte header | payload]. Header words (uint32): 0..7 epoch announced by rank r (written by
 * rank r), 16 finished-block counter, 17 epochs sent, 18 epochs waited for, 19 set when a wait expired; diagnostics of
 * the last fan-out launch as 64-bit %globaltimer nanoseconds of this GPU: words 20-21 its first block began, 22-23 the
 * last block saw every block's stores issued, 24-25 the epoch was published, 26-27 every awaited peer's epoch was seen. The counters
 * live on the device, so launches captured in a CUDA graph keep working when replayed; every rank must issue the same
 * sequence of fan-out launches and waits. Use two payload areas in turn when a step may start before every peer has
 * consumed the previous one. */
#define BF16N_EXCHANGE_HEADER_BYTES 256
#define BF16N_MAX_PEERS 7
#define BF16N_IPC_HANDLE_BYTES 64
typedef struct bf16n_peer_out {
    int n_peers;                         /* 0..7 other GPUs */
    void * y[BF16N_MAX_PEERS];           /* where the same output goes in each peer's exchange buffer (mapped here) */
    uint32_t * flag[BF16N_MAX_PEERS];    /* header word [my rank] of each peer's exchange buffer (mapped here) */
    uint32_t * local_header;             /* this GPU's own exchange buffer */
    int wait_mask;                       /* 0, or the ranks (bit r) whose output of the same epoch must have arrived here
                                          * before the kernel ends: the kernel then replaces bf16n_peer_wait as well */
} bf16n_peer_out;
/* Allocates a zeroed exchange buffer of header + payload_bytes on the current device and exports it for the other
 * processes of the node (cudaIpcGetMemHandle). */
int bf16n_exchange_create(size_t payload_bytes, void ** base, unsigned char handle[BF16N_IPC_HANDLE_BYTES]);
/* Maps a peer's exchange buffer into this process (peer access is enabled on demand). */
int bf16n_exchange_open(const unsigned char handle[BF16N_IPC_HANDLE_BYTES], void ** base);
int bf16n_exchange_close(void * peer_base);
int bf16n_exchange_destroy(void * base);
/* bf16n_mmv whose output also goes to the peers (dense row-major HUFPAIR matrices; one kernel does the product, the
 * peer stores and the announcement). a->y must point into this GPU's exchange payload at the offset the peers use. */
int bf16n_mmv_peers(const bf16n_weight * w, const bf16n_mmv_args * a, const bf16n_peer_out * peers, void * stream);
/* Waits on the stream until every peer in rank_mask (bit r = rank r) has announced its next epoch; bounded (two
 * seconds unless bf16n_set_peer_wait_limit_ms changed it), after which header word 19 is set and the stream continues. */
int bf16n_peer_wait(uint32_t * local_header, int rank_mask, void * stream);
/* How long bf16n_peer_wait and the kernels that wait for their peers themselves (wait_mask) may spin, 1..60000 ms. The
 * limit is a launch argument: it applies to launches made (or captured) after this call. */
int bf16n_set_peer_wait_limit_ms(unsigned int ms);
/* bf16n_moe_decode on an expert-parallel rank whose last kernel (the slot-order combine) also stores the rank's partial
 * [n_tok, H] output into every peer (y and peers->y[r] are this rank's slot in the exchange payloads), announces it and,
 * with peers->wait_mask, ends only when the peers' partial outputs have arrived. */
int bf16n_moe_decode_peers(const bf16n_weight * gate, const bf16n_weight * up, const bf16n_weight * down, const void * x, int x_bf16,
                           int64_t x_tok, const float * router_logits, int n_experts, int32_t * topk_ids, float * topk_weights,
                           int n_tok, int n_used, int expert_lo, int n_experts_local, float * scratch, size_t scratch_bytes,
                           void * y, int y_bf16, const bf16n_peer_out * peers, void * stream);
/* y[i] = parts[0][i] + ... + parts[n_parts-1][i] (+ extra[i] when extra is not null): the ranks' partial outputs added
 * in rank order, so that every rank gets the same bits. parts: n_parts consecutive arrays of n floats. */
int bf16n_peer_sum(const float * parts, int n_parts, int64_t n, const float * extra, void * y, int y_bf16, void * stream);
/* Synchronises the stream and returns header word 19 (non-zero: a wait expired since the buffer was created). */
int bf16n_peer_expired(const uint32_t * local_header, void * stream, int * expired);

/* Expert-parallel prefill on the device: tokens split over the ranks of a node, experts sharded; every routed
 * (token, slot) row is stored into the exchange buffer of the rank that owns its expert, multiplied there by the batched
 * kernels and its result stored back into the source's buffer. No host round trip and no collective: the three calls
 * enqueue kernels on the caller's stream and a layer can be captured in a CUDA graph. Every rank issues the same
 * sequence of calls per layer:
 *     bf16n_ep_dispatch    plan + row copies into the owners' inboxes; ends when every peer's rows have arrived here
 *     bf16n_ep_inbox_ids   expert id of every inbox slot ([n_ranks * cap], 0x7fffffff = empty) for bf16n_mm_ids_route /
 *                          bf16n_mm_ids over the inbox rows (n_tok = n_ranks * cap, n_used = 1)
 *     bf16n_ep_give_back   results [n_ranks * cap, H] FP32 of the inbox rows into their sources' `back` areas (row = pair
 *                          index, i.e. [n_tok, n_used, H] for bf16n_moe_combine); ends when every owner's results are here
 * The buffers are bf16n_exchange_create buffers of bf16n_ep_layout_bytes(l) payload bytes with one layout on all ranks. */
typedef struct bf16n_ep_layout {
    int n_ranks, rank;
    int cap;             /* rows one source can send to one owner: at least the largest n_tok * n_used of any rank */
    int K, H;            /* activation columns (BF16) and result columns (FP32) */
    int n_pairs_max;     /* the most (token, slot) pairs this rank itself routes in a layer */
    void * base[8];      /* the exchange buffers of all ranks as mapped into this process ([rank] = the own one) */
    size_t off_counts, off_expert, off_pair, off_rows, off_back;   /* payload areas, set by bf16n_ep_layout_bytes */
} bf16n_ep_layout;
size_t bf16n_ep_layout_bytes(bf16n_ep_layout * l);
/* plan: device scratch of n_tok * n_used + 8 int32 */
int bf16n_ep_dispatch(const bf16n_ep_layout * l, const void * x_bf16, int64_t x_row_bytes, const int32_t * topk_ids, int n_tok, int n_used,
                      int n_experts, int32_t * plan, void * stream);
int bf16n_ep_inbox_ids(const bf16n_ep_layout * l, int32_t * ids_out, void * stream);
int bf16n_ep_give_back(const bf16n_ep_layout * l, const float * ys, void * stream);

#ifdef __cplusplus
}
#endif
#endif /* BF16N_C_H */
