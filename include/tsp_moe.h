/*
 * tsp_moe.h — C ABI of the B200 (sm_100a) routed-MoE FFN hot path.
 *
 * This is the boundary a tokspur maintainer binds in place of the Metal operator methods of
 * `MetalGraph` (native/include/tokspur/graph.hpp) that `encode_moe`, `encode_moe_mm_many` and
 * `encode_verify_nax_moe` dispatch to. Each entry point names the reference operator it replaces.
 *
 * Conventions
 *  - Every pointer prefixed `d_` is a DEVICE pointer owned by the caller. Nothing here allocates,
 *    frees, copies weights or reads results back, unless the entry point says so.
 *  - `stream` is a `cudaStream_t` passed as an opaque pointer (NULL = the legacy default stream).
 *    Launches are asynchronous and ordered on that stream.
 *  - Activations are FP32 rows with a byte stride (the reference's `GpuRowsF32`), ids are uint32.
 *  - Return value: TSP_OK or a negative TSP_E_* code; `tsp_last_error()` gives the message of the
 *    last refusal on the calling thread. Host-side contract violations are refused BEFORE any launch
 *    (the reference throws `FormatError` there).
 *  - Device-side numerical / index failures never trap: kernels OR bits into the caller's sticky
 *    error word `d_error` (the reference's buffer index 7, graph.mm:3977) and write zeros for the
 *    affected rows; the host reads the word once per batch with `tsp_error_word_read`.
 *  - No CPU fallback exists. On a machine without a usable CUDA device every launch entry point
 *    returns TSP_E_CUDA.
 */
#ifndef TSP_MOE_H
#define TSP_MOE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TSP_OK 0
#define TSP_E_ARG (-1)      /* shape / size / alignment / aliasing contract violation */
#define TSP_E_TYPE (-2)     /* encoding or layout without a kernel */
#define TSP_E_CUDA (-3)     /* CUDA runtime refused (message holds the CUDA error string) */
#define TSP_E_DEVICE (-4)   /* sticky device error word was non-zero at read time */

/* Sticky error word bits (same meaning as the reference's kernels, planar_moe_v3.metal:100-105). */
#define TSP_ERR_NONFINITE 2u /* non-finite scale, input or result */
#define TSP_ERR_INDEX 4u     /* expert id / route geometry out of range, or an expert named twice by one token */
#define TSP_ERR_TIMEOUT 8u   /* a bounded in-kernel wait gave up (pipeline barrier) */

/* GGUF tensor type ids (gguf.cpp:21-32). */
#define TSP_TYPE_F32 0u
#define TSP_TYPE_Q5_1 7u   /* decode-size kernels only, GGUF layout (the reference model's down tensors) */
#define TSP_TYPE_Q8_0 8u
#define TSP_TYPE_Q4_K 12u
#define TSP_TYPE_Q5_K 13u  /* decode-size kernels only, GGUF layout (some of the reference model's gate / up tensors) */

/* Weight byte layouts. */
#define TSP_LAYOUT_GGUF 0u    /* GGUF array-of-blocks rows (144 B / 256 weights Q4_K, 34 B / 32 weights Q8_0) */
#define TSP_LAYOUT_PLANAR 1u  /* Pack v3 planar expert: planes qs | sm | dm (planar_pack_v3.cpp:601-716) */

/* Router activation (routing.hpp: RouterMode). */
#define TSP_ROUTER_SOFTMAX 0u
#define TSP_ROUTER_SIGMOID 1u

/* A set of `experts` equally shaped quantised matrices [rows x cols], row-major, one per expert.
 *   GGUF layout  : expert e at base + e * expert_stride, rows of cols/block blocks.
 *   PLANAR layout: expert e at (e < split ? base + e*expert_stride : base_hi + (e-split)*expert_stride),
 *                  each a complete planar expert. Co-located gate/up pairs (planar_moe_v3.metal:549-553)
 *                  are described by split = experts/2, expert_stride = 2*planar_expert_bytes, with the up
 *                  matrix set using base + planar_expert_bytes.
 * A dense matrix is a set with experts = 1. All bases must be 16-byte aligned. */
typedef struct tsp_matrix_set {
    const void* base;
    const void* base_hi;     /* used only when split < experts */
    uint64_t expert_stride;  /* bytes between consecutive experts in one half */
    uint32_t split;          /* first expert id stored under base_hi; == experts when unused */
    uint32_t experts;
    uint32_t rows, cols;
    uint32_t type;           /* TSP_TYPE_Q4_K or TSP_TYPE_Q8_0; TSP_TYPE_Q5_K / TSP_TYPE_Q5_1 on the decode-size entries */
    uint32_t layout;         /* TSP_LAYOUT_* */
} tsp_matrix_set;

/* Per-thread message of the last refused call. Never NULL. */
const char* tsp_last_error(void);

/* Library / device facts: writes the SM count and returns TSP_OK when a CUDA device is usable. */
int tsp_device_info(int* sm_count, int* cc_major, int* cc_minor);

/* Sticky error word helpers (graph.mm:3977-3978: checked once per batch at submit).
 * `tsp_error_word_read` synchronises `stream`, copies the word to *host_word and returns
 * TSP_E_DEVICE when it is non-zero. `tsp_error_word_reset` zeroes it asynchronously. */
int tsp_error_word_read(const uint32_t* d_error, void* stream, uint32_t* host_word);
int tsp_error_word_reset(uint32_t* d_error, void* stream);

/* Bytes per expert of a [rows x cols] matrix in the given type/layout; 0 when unsupported.
 * (planar: make_expert_spec, planar_pack_v3.cpp:601-650.) */
uint64_t tsp_expert_bytes(uint32_t type, uint32_t layout, uint32_t rows, uint32_t cols);

/* Test hook: decode one expert of a matrix set to FP32 [rows x cols], bit-identical to the
 * reference's `dequantize` (numeric.cpp:97-148) / `dequantize_expert_planar_v3` (planar_pack_v3.cpp:760). */
int tsp_dequant_f32(const tsp_matrix_set* m, uint32_t expert, float* d_out, uint32_t* d_error, void* stream);

/* Replaces `MetalGraph::route` / `prefill_route_batch` / `moe_route_rows` (graph.mm:7929,5957,5863;
 * CPU: route_reference, routing.cpp:11-40). Per token row: top-`selected` ids by descending logit,
 * ties to the lower id; weights per `mode`, renormalised over the selection when `normalize_selected`.
 * d_logits: [tokens] rows of `experts` floats, `logits_stride_bytes` apart. experts <= 4096, selected <= 64. */
int tsp_moe_route(const float* d_logits, uint64_t logits_stride_bytes, uint32_t tokens, uint32_t experts,
                  uint32_t selected, uint32_t mode, int normalize_selected,
                  uint32_t* d_ids, float* d_weights, uint32_t* d_error, void* stream);

/* The same with the router-margin audit (graph.hpp:162-172, moe_route_rows' margin buffer graph.mm:5877): d_margins[t] = logit of the
 * last selected expert minus the best logit left out, i.e. how large a perturbation of the FP32 logits the selection of
 * row t survives (+inf when every expert is selected, 0 for a row with a non-finite logit).
 * tsp_router_margin_evaluate replaces `evaluate_router_margin` (graph.mm:4931-4985): it synchronises `stream`, reads the
 * margins back and folds them into the running telemetry; a row counts as a violation when its margin is <= 2*epsilon, and
 * *fallback (optional) tells whether this batch had any (the reference then re-projects the batch on its exact path). */
typedef struct tsp_router_margin_telemetry {
    float min_margin;          /* valid once total_tokens > 0 */
    double sum_margin;
    uint64_t total_tokens, violation_count, fallback_layers, total_layers;
} tsp_router_margin_telemetry;
int tsp_moe_route_audit(const float* d_logits, uint64_t logits_stride_bytes, uint32_t tokens, uint32_t experts, uint32_t selected,
                        uint32_t mode, int normalize_selected, uint32_t* d_ids, float* d_weights, float* d_margins,
                        uint32_t* d_error, void* stream);
int tsp_router_margin_evaluate(const float* d_margins, uint32_t tokens, float epsilon, void* stream, tsp_router_margin_telemetry* telemetry,
                               int* fallback);

/* Replaces `graph_grouped_routes` + `graph_grouped_tasks` (grouped_mpp.metal:12-66; host
 * grouped_mm_routes, graph.mm:4608). Builds the stable per-expert token permutation:
 *   d_token_map[e*tokens + j] = token*selected + slot of the j-th (ascending) token routed to e,
 *   d_counts[e], and d_tasks = {live_tiles, routes, (expert,start)*live_tiles, 0xffffffff padding}
 *   with tiles of `tile` routes in ascending expert order; d_tasks has tsp_moe_tasks_words() words. */
int tsp_moe_permute(const uint32_t* d_ids, uint32_t tokens, uint32_t experts, uint32_t selected, uint32_t tile,
                    uint32_t* d_token_map, uint32_t* d_counts, uint32_t* d_tasks, uint32_t* d_error, void* stream);
uint64_t tsp_moe_tasks_words(uint32_t tokens, uint32_t experts, uint32_t selected, uint32_t tile);

/* Expert-parallel form of tsp_moe_permute (no reference counterpart: the reference is single-GPU). d_ids holds GLOBAL
 * expert ids; the tables cover only the experts [first_expert, first_expert + local_experts) this GPU owns, indexed
 * locally (row 0 of d_token_map = expert first_expert). Routes to other owners are skipped, not errors; route ids keep
 * the global numbering token*selected + slot. d_tasks needs tsp_moe_tasks_words(tokens, local_experts, selected, tile). */
int tsp_moe_permute_local(const uint32_t* d_ids, uint32_t tokens, uint32_t first_expert, uint32_t local_experts, uint32_t selected,
                          uint32_t tile, uint32_t* d_token_map, uint32_t* d_counts, uint32_t* d_tasks, uint32_t* d_error, void* stream);

/* Decode-size routed projection with the weight bytes streamed once per tile of routes.
 * Replaces `planar_moe_gate_up_swiglu_m8` (graph.mm:9134), `routed_gemv`x2 + `swiglu` (moe.cpp:62-66),
 * and for a dense set (token map NULL) `gemv`/`gemv_rows`/`q8_matvec_many` + `swiglu` of the shared expert.
 *   h[route][r] = silu(sum_c G_e[r][c] x[token][c]) * (sum_c U_e[r][c] x[token][c]),  route = token*selected+slot
 * gate/up: matrix sets [hidden x channels] with identical shape/type/layout.
 * d_x: FP32 rows [tokens x channels]; d_h: FP32 rows [tokens*selected x hidden] (dense: [tokens x hidden]).
 * d_token_map/d_counts/d_tasks: from tsp_moe_permute with tile == TSP_GEMV_TILE; all NULL for a dense set.
 * x_is_f16_exact: non-zero promises every x value is exactly representable in binary16 (skips the
 * low-half correction pass); zero is always safe. */
#define TSP_GEMV_TILE 8u
int tsp_moe_gate_up_swiglu(const tsp_matrix_set* gate, const tsp_matrix_set* up,
                           const float* d_x, uint64_t x_stride_bytes, uint32_t tokens, uint32_t selected,
                           const uint32_t* d_token_map, const uint32_t* d_counts, const uint32_t* d_tasks,
                           float* d_h, uint64_t h_stride_bytes, int x_is_f16_exact,
                           uint32_t* d_error, void* stream);

/* Routed (or dense) plain projection y[route][r] = sum_j W_e[r][j] h[route][j].
 * Replaces `planar_moe_routed_m8`'s down stage (graph.mm:9205), `routed_gemv(broadcast=false)` (moe.cpp:68),
 * and for a dense set `gemv`/`q8_matvec_many`/`verify_nax_dense_q8` (shared down, vocabulary head).
 * in_div: input row of a route is route / in_div (1 for down; `selected` to broadcast token rows). */
int tsp_moe_project(const tsp_matrix_set* w, const float* d_in, uint64_t in_stride_bytes, uint32_t in_div,
                    uint32_t tokens, uint32_t selected,
                    const uint32_t* d_token_map, const uint32_t* d_counts, const uint32_t* d_tasks,
                    float* d_out, uint64_t out_stride_bytes, int in_is_f16_exact,
                    uint32_t* d_error, void* stream);

/* The two projections above for the routed experts AND the layer's dense shared expert in one launch each, as the decode
 * layer runs them: `encode_moe` issues the routed projections (moe.cpp:62-68) and the shared expert's `gemv`s
 * (moe.cpp:70-77) back to back on the same input rows. When the shared expert has the routed experts' shape, encoding
 * and layout (Q4_K), its token tiles are appended to the routed tiles of the same launch; otherwise these entries fall
 * back to two launches.
 * d_x16 (optional, may be NULL): the same token rows as binary16, [tokens x channels]; used instead of d_x when
 * x_is_f16_exact is set, so that staging the rows needs no conversion.
 * d_shared_h: FP32 rows [tokens x hidden]; d_shared_in / d_shared_out: the shared expert's hidden rows and output rows. */
int tsp_moe_gate_up_swiglu_shared(const tsp_matrix_set* gate, const tsp_matrix_set* up, const tsp_matrix_set* shared_gate,
                                  const tsp_matrix_set* shared_up, const float* d_x, uint64_t x_stride_bytes, const void* d_x16,
                                  uint64_t x16_stride_bytes, uint32_t tokens, uint32_t selected, const uint32_t* d_token_map,
                                  const uint32_t* d_counts, const uint32_t* d_tasks, float* d_h, uint64_t h_stride_bytes,
                                  float* d_shared_h, uint64_t shared_h_stride_bytes, int x_is_f16_exact, uint32_t* d_error, void* stream);
int tsp_moe_project_shared(const tsp_matrix_set* w, const tsp_matrix_set* shared_w, const float* d_in, uint64_t in_stride_bytes,
                           const float* d_shared_in, uint64_t shared_in_stride_bytes, uint32_t tokens, uint32_t selected,
                           const uint32_t* d_token_map, const uint32_t* d_counts, const uint32_t* d_tasks, float* d_out,
                           uint64_t out_stride_bytes, float* d_shared_out, uint64_t shared_out_stride_bytes, uint32_t* d_error, void* stream);

/* The same two launches where the dense shared expert works on OTHER rows than the routed experts (no reference counterpart: the
 * expert-parallel layer runs the routed experts over the rows it received and the shared expert over the rank's own rows).
 * d_shared_x / d_shared_in: FP32 rows [shared_tokens x cols] of the shared expert. d_x16 may only be given when both row sets
 * are the same rows. */
int tsp_moe_gate_up_swiglu_shared_rows(const tsp_matrix_set* gate, const tsp_matrix_set* up, const tsp_matrix_set* shared_gate,
                                       const tsp_matrix_set* shared_up, const float* d_x, uint64_t x_stride_bytes, const void* d_x16,
                                       uint64_t x16_stride_bytes, uint32_t tokens, uint32_t selected, const uint32_t* d_token_map,
                                       const uint32_t* d_counts, const uint32_t* d_tasks, float* d_h, uint64_t h_stride_bytes,
                                       const float* d_shared_x, uint64_t shared_x_stride_bytes, uint32_t shared_tokens, float* d_shared_h,
                                       uint64_t shared_h_stride_bytes, int x_is_f16_exact, uint32_t* d_error, void* stream);
int tsp_moe_project_shared_rows(const tsp_matrix_set* w, const tsp_matrix_set* shared_w, const float* d_in, uint64_t in_stride_bytes,
                                const float* d_shared_in, uint64_t shared_in_stride_bytes, uint32_t shared_tokens, uint32_t tokens,
                                uint32_t selected, const uint32_t* d_token_map, const uint32_t* d_counts, const uint32_t* d_tasks, float* d_out,
                                uint64_t out_stride_bytes, float* d_shared_out, uint64_t shared_out_stride_bytes, uint32_t* d_error, void* stream);

/* Replaces `gemv(shared_router, rows=1)` + `mixture` / `prefill_mixture_batch` (moe.cpp:79-81,
 * graph.mm:8023,5975; CPU mixture_reference, routing.cpp:42-61):
 *   out[t][c] = sigmoid(s_t) * shared[t][c] + sum_{r<selected} w[t][r] * routed[t*selected+r][c]
 * accumulated in route-rank order starting from the shared term. s_t = dot(d_shared_router, x[t]) when
 * d_shared_router != NULL (and is stored to d_shared_logit when that is non-NULL), else d_shared_logit[t].
 * routed_dtype / x_dtype: 0 = FP32 rows, 1 = binary16 rows (the prefill path keeps its route rows as binary16).
 * d_shared == NULL leaves the shared term out (partial sums over the routes only: expert parallelism); a route whose weight
 * is exactly zero is skipped without reading its row.
 * d_out_f16 (optional) receives the same rows rounded to binary16. */
int tsp_moe_combine(const void* d_routed, uint64_t routed_stride_bytes, uint32_t routed_dtype, const float* d_weights,
                    const float* d_shared, uint64_t shared_stride_bytes,
                    const float* d_shared_router, const void* d_x, uint64_t x_stride_bytes, uint32_t x_dtype,
                    float* d_shared_logit, uint32_t tokens, uint32_t channels, uint32_t selected,
                    float* d_out, uint64_t out_stride_bytes, void* d_out_f16, uint64_t out_f16_stride_bytes,
                    uint32_t* d_error, void* stream);

/* `q8_lanes_v1` rows (the layout the Pack v3 container keeps dense Q8_0 matrices such as the vocabulary head in,
 * planar_pack_v3.cpp:467-470; `lanes::pack_rows` / `unpack_rows`, expert_lanes.cpp:92-130) to GGUF Q8_0 rows and back. A
 * lossless re-layout of whole rows (34 bytes per 32 weights either way), meant to run once when the tensor is uploaded: the
 * projection kernels read GGUF rows. rows x cols weights, cols a multiple of 32; the two buffers must not overlap. */
int tsp_q8_lanes_unpack(const void* d_lanes, void* d_gguf, uint64_t rows, uint32_t cols, void* stream);
int tsp_q8_lanes_pack(const void* d_gguf, void* d_lanes, uint64_t rows, uint32_t cols, void* stream);

/* Self test of the bounded waits (no reference counterpart): one thread waits at most `polls` (1..65536) polls on a barrier
 * that nothing arrives on, then sets TSP_ERR_TIMEOUT in *d_error and the kernel returns normally; the context stays usable.
 * Every pipeline wait of the library gives up the same way (after 2^24 polls). */
int tsp_selftest_bounded_wait(uint32_t polls, uint32_t* d_error, void* stream);

/* Top-64 rows of the sampler behind the vocabulary head. Replaces `MetalGraph::logit_topk` (graph.hpp:1030-1033, graph.mm:9443-9478)
 * and its size helpers; one output row per logits row in the layout of `GpuLogitTopKRow` (sampling.hpp:21-29, 528 bytes):
 * u32 vocabulary, count, first_nonfinite_col, first_subnormal_col (0xffffffff: none), u32 ids[64], f32 logits[64].
 * Order as `cpu_logit_topk_row` (sampling.cpp:473-515): value descending with -0 == +0, ties to the lower column; non-finite
 * logits are left out, subnormal ones compete; raw bits are returned; unused slots hold id 0 and -infinity.
 * d_logits: FP32 rows [rows x vocabulary] with a byte stride; d_partial: scratch of tsp_logit_topk_scratch_bytes() (one row per
 * tile of 4096 columns); both buffers 4-byte aligned and disjoint from the logits. rows 1..2048, vocabulary 1..2^20. */
#define TSP_TOPK_CAPACITY 64u
#define TSP_TOPK_TILE_SPAN 4096u
#define TSP_TOPK_ROW_BYTES 528u
uint64_t tsp_logit_topk_scratch_bytes(uint32_t rows, uint32_t vocabulary);
uint64_t tsp_logit_topk_output_bytes(uint32_t rows);
int tsp_logit_topk(const float* d_logits, uint64_t logits_stride_bytes, uint32_t rows, uint32_t vocabulary, void* d_partial,
                   uint64_t partial_bytes, void* d_rows_out, uint64_t out_bytes, void* stream);

/* Hyper-connection residual read / write, the steps either side of the FFN sub-layer in every layer (mtp_head.cpp:206-208).
 * Replace `MetalGraph::residual_read` / `residual_write` (graph.hpp:1056-1058; CPU: gated_residual_reference's last step and
 * residual_write_reference, operators.cpp:79-96), batched over `tokens` rows; all buffers FP32, row-major, densely packed:
 *   read:  output[t][c] = sum_b normalized[t][b][c] * sigmoid(scores[t][b][c]) / branches,  scales[t][b] = 2 sigmoid(inject_logits[t][b] / branches)
 *   write: destination[t][b][c] = streams[t][b][c] + scales[t][b] * output[t][c]   (destination may be the streams themselves) */
int tsp_residual_read(const float* d_normalized, const float* d_scores, const float* d_inject_logits, uint32_t branches, uint32_t channels,
                      uint32_t tokens, float* d_output, float* d_scales, uint32_t* d_error, void* stream);
int tsp_residual_write(const float* d_streams, const float* d_output, const float* d_scales, uint32_t branches, uint32_t channels,
                       uint32_t tokens, float* d_destination, uint32_t* d_error, void* stream);

/* ---- data preparation (device side) ----------------------------------------------------------------
 * tsp_synth_weights: seeded N(0, sigma) values quantised to GGUF blocks of `type` (Q4_K, Q8_0) or written
 * as FP32 (type F32, `blocks` = element count), `blocks` blocks starting at stream block `first_block`
 * (any slice of a tensor can be produced independently). No reference counterpart: the reference has
 * no quantizer; the benchmark's synthetic weights come from here.
 * tsp_pack_planar: GGUF rows -> Pack v3 planar experts on the device; replaces `pack_expert_planar_v3`
 * (planar_pack_v3.cpp:676-716). `planar_expert_stride` lets gate and up experts interleave into the
 * co-located pair tensors (stride 2 * planar_expert_bytes, up offset by one expert). */
int tsp_synth_weights(uint32_t type, uint64_t seed, uint64_t first_block, uint64_t blocks, float sigma, void* d_out, void* stream);
int tsp_pack_planar(uint32_t type, uint32_t rows, uint32_t cols, uint32_t experts, const void* d_gguf, uint64_t gguf_expert_stride,
                    void* d_planar, uint64_t planar_expert_stride, void* stream);

/* Replaces `gemv(type 0)` / `gemv_rows` / `moe_router_f32_batch` on F32 matrices (graph.mm:4182, 4271, 5729): the router and
 * shared-router projections, out[t][r] = sum_c W[r][c] x[t][c], W row-major F32 [rows x cols], FP32 accumulation. */
int tsp_gemv_f32(const float* d_w, uint32_t rows, uint32_t cols, const float* d_x, uint64_t x_stride_bytes, uint32_t tokens,
                 float* d_out, uint64_t out_stride_bytes, uint32_t* d_error, void* stream);
/* Replaces `moe_router_f32_window` + `moe_shared_router_rows` (graph.mm:5812, 5884): the router projection of a batch with the
 * shared-router vector as one extra matrix row of the same pass, d_extra_out[t] = sum_c d_extra_row[c] x[t][c] (both NULL: none).
 * From 32 token rows on this is a tiled FP32 GEMM that reads W once per 64 rows; FP32 FMA only (no reduced-precision tensor
 * path: the ids chosen from these logits have to follow the reference's double-precision logits; tsp_moe_route_audit tells
 * how close each row's selection is to changing). */
int tsp_router_project(const float* d_w, uint32_t rows, uint32_t cols, const float* d_extra_row, const float* d_x, uint64_t x_stride_bytes,
                       uint32_t tokens, float* d_out, uint64_t out_stride_bytes, float* d_extra_out, uint32_t* d_error, void* stream);

/* binary16 rows -> FP32 rows (exact) and back (round to nearest even); activation edge of the layer. */
int tsp_rows_f16_to_f32(const void* d_in, uint64_t in_stride_bytes, float* d_out, uint64_t out_stride_bytes,
                        uint32_t rows, uint32_t cols, void* stream);

/* Caller-owned scratch of one MoE layer call, sized for `capacity` token rows.
 * Mirrors MoeScratch / MoeMmManyScratch (moe.hpp:14-17, moe_mm_many.hpp:50-55). */
typedef struct tsp_moe_scratch {
    uint32_t* d_ids;        /* [capacity x selected] */
    float* d_weights;       /* [capacity x selected] */
    float* d_hidden;        /* [capacity*selected x hidden]   (MoeScratch.gate after swiglu) */
    float* d_routed;        /* [capacity*selected x channels] (MoeScratch.down) */
    float* d_shared_hidden; /* [capacity x hidden] */
    float* d_shared_out;    /* [capacity x channels] */
    float* d_shared_logit;  /* [capacity] */
    float* d_x32;           /* [capacity x channels] staging when the input is binary16 */
    uint32_t* d_token_map;  /* [experts x capacity] */
    uint32_t* d_counts;     /* [experts] */
    uint32_t* d_tasks;      /* tsp_moe_tasks_words(capacity, experts, selected, TSP_GEMV_TILE) */
    uint32_t capacity;
} tsp_moe_scratch;

typedef struct tsp_moe_weights {
    tsp_matrix_set gate, up, down;                      /* routed experts */
    tsp_matrix_set shared_gate, shared_up, shared_down; /* dense shared expert (experts = 1) */
    const float* d_shared_router;                       /* F32 [channels]; NULL: gate logit 0 is NOT assumed, see below */
} tsp_moe_weights;

/* One whole MoE FFN sub-layer for `tokens` <= scratch.capacity rows with router logits supplied:
 * route -> permute -> gate-up+SwiGLU -> down -> shared expert -> gated combine.
 * Replaces `encode_moe` after its router GEMV (moe.cpp:37-83) and `encode_verify_nax_moe`
 * (verify_nax.cpp:436-575) for small batches. x_dtype/out_dtype: 0 = FP32 rows, 1 = binary16 rows.
 * When d_shared_router is NULL the shared expert is added ungated (gate = 1). */
int tsp_moe_layer_decode(const tsp_moe_weights* w, const tsp_moe_scratch* s,
                         const void* d_x, uint64_t x_stride_bytes, uint32_t x_dtype,
                         const float* d_logits, uint64_t logits_stride_bytes,
                         uint32_t tokens, uint32_t channels, uint32_t hidden, uint32_t experts, uint32_t selected,
                         uint32_t mode, int normalize_selected,
                         void* d_out, uint64_t out_stride_bytes, uint32_t out_dtype,
                         uint32_t* d_error, void* stream);

/* ---- prefill-size path: grouped per-expert GEMMs on the tcgen05 tensor cores --------------------------
 * Replaces `planar_nax_grouped_moe` (graph.mm:9293-9420) = `graph_grouped_routes` -> `nax_grouped_tasks_indirect` ->
 * `nax_moe_gather_bf16_v3` -> `nax_grouped_moe_gate_up_swiglu_v3` -> `nax_grouped_moe_down_v3`
 * (planar_moe_v3.metal:2406-2621). Weights: Q4_K, Pack v3 planar (one copy per plane) or plain GGUF super-blocks (the tensor
 * maps then walk the 144-byte blocks: codes from byte 16, the 16-byte header beside them; same staged operands, so the same
 * result bits); gate, up and their shared expert in one layout; hidden a multiple of 64, channels of 256.
 *   1. tsp_moe_rows_f16k                                       binary16 copy of the input rows in the K order the tensor-core tiles use
 *   2. tsp_moe_permute(..., tile = TSP_GROUPED_TILE)           token_map / counts / tasks (tasks of 256 routes = two sub-tiles of 128)
 *   3. tsp_moe_route_offsets                                   offsets[e] = first permuted position of expert e; experts+5 words: the last
 *                                                              four are item counters, cleared here (steps 5 and 6, and the
 *                                                              two dense launches of a shared expert in another encoding)
 *   4. tsp_moe_gather_rows16                                   the routed copy of the rows of step 1, in permuted position order
 *   5. tsp_moe_grouped_gate_up                                 H[pos][hidden] binary16, SwiGLU applied, FP32 accumulate in tensor memory
 *   6. tsp_moe_grouped_down                                    routed[route][channel], FP32 or binary16, scattered by route id
 * Steps 5 and 6 hand their work items out through the counters step 3 cleared: run step 3 before every pair of them.
 * Row buffers in permuted position order (d_xp, d_hp) hold tokens*selected rows. Values inside each aligned run of 8 along a
 * row of d_xk / d_xp / d_hp are stored in the order 0,2,1,3,4,6,5,7 (the order the dequantised weight tiles use), which only
 * these kernels read. Operands are binary16, accumulation FP32. The route id of a route is row*selected + slot.
 *
 * Weights of steps 5 and 6 may also be Q8_0 GGUF blocks (the Q8_0 expert sets of the MTP block).
 * Both GEMMs take the layer's dense shared expert in the same launch when shared_* is non-NULL (same shape, encoding and
 * layout as a routed expert): its tasks cover every one of `tokens` rows in row order and follow the routed ones, as
 * `encode_moe_mm_many` runs the shared expert's dense projections right after the routed ones (moe_mm_many.cpp:189-214).
 * It reads the rows of step 1 (d_xk) directly; d_s_hp: its binary16 hidden rows [shared_tokens x hidden]; d_shared_out: FP32
 * [shared_tokens x channels]. shared_tokens is the layer's own row count (equal to `tokens` on one GPU; under expert
 * parallelism the routed rows are the rows received from every rank while the shared expert serves this rank's rows). */
#define TSP_GROUPED_TILE 256u
int tsp_moe_route_offsets(const uint32_t* d_counts, uint32_t experts, uint32_t* d_offsets, void* stream);
int tsp_moe_rows_f16k(const void* d_x, uint64_t x_stride_bytes, uint32_t x_dtype, uint32_t rows, uint32_t cols, void* d_xk,
                      uint64_t xk_stride_bytes, uint32_t* d_error, void* stream);
int tsp_moe_gather_rows16(const void* d_xk, uint64_t xk_stride_bytes, const uint32_t* d_token_map, const uint32_t* d_offsets, uint32_t experts,
                          uint32_t tokens, uint32_t selected, uint32_t cols, void* d_xp, uint64_t xp_stride_bytes, void* stream);
int tsp_moe_grouped_gate_up(const tsp_matrix_set* gate, const tsp_matrix_set* up, const tsp_matrix_set* shared_gate,
                            const tsp_matrix_set* shared_up, const void* d_xp, uint64_t xp_stride_bytes, const void* d_xk,
                            uint64_t xk_stride_bytes, uint32_t shared_tokens, uint32_t tokens, uint32_t selected, const uint32_t* d_token_map,
                            const uint32_t* d_counts, const uint32_t* d_tasks, uint32_t* d_offsets, void* d_hp, uint64_t hp_stride_bytes,
                            void* d_s_hp, uint64_t s_hp_stride_bytes, uint32_t* d_error, void* stream);
int tsp_moe_grouped_down(const tsp_matrix_set* down, const tsp_matrix_set* shared_down, const void* d_hp, uint64_t hp_stride_bytes,
                         uint32_t tokens, uint32_t selected, const uint32_t* d_token_map, const uint32_t* d_counts, const uint32_t* d_tasks,
                         uint32_t* d_offsets, void* d_routed, uint64_t routed_stride_bytes, uint32_t routed_dtype, const void* d_s_hp,
                         uint64_t s_hp_stride_bytes, uint32_t shared_tokens, float* d_shared_out, uint64_t shared_out_stride_bytes,
                         uint32_t* d_error, void* stream);

/* Dense projections of row batches through the same tensor-core kernel (no routing tables): the shared expert when its
 * encoding or layout differs from the routed experts', i.e. the reference's dense Q8_0 shared expert beside Q4_K experts.
 * Replace `nax_dense_q8_swiglu` (gate + up + SwiGLU in one dispatch) and `dense_mm_q8` as `encode_moe_mm_many` uses them
 * (moe_mm_many.cpp:236-259; kernels nax_prefill.metal:1506-1636). Matrices: single [rows x cols] Q8_0 GGUF blocks or Q4_K
 * (planar or GGUF), rows a multiple of 64 (gate/up) or 128, cols of 256.
 *   tsp_dense_mm_swiglu: d_xk binary16 input rows in tile K order (tsp_moe_rows_f16k) -> d_h binary16 silu(gate.x) * (up.x), in
 *                        the K order the next projection reads;
 *   tsp_dense_mm:        d_xk binary16 rows in tile K order (e.g. the rows tsp_dense_mm_swiglu wrote) -> d_out FP32 rows.
 * d_counter: one device word holding 0 when the launch starts (the item hand-out counter; tsp_moe_route_offsets clears words
 * experts+3 and experts+4 of its buffer for this use). */
int tsp_dense_mm_swiglu(const tsp_matrix_set* gate, const tsp_matrix_set* up, const void* d_xk, uint64_t xk_stride_bytes, uint32_t rows,
                        void* d_h, uint64_t h_stride_bytes, uint32_t* d_counter, uint32_t* d_error, void* stream);
int tsp_dense_mm(const tsp_matrix_set* matrix, const void* d_xk, uint64_t xk_stride_bytes, uint32_t rows, float* d_out,
                 uint64_t out_stride_bytes, uint32_t* d_counter, uint32_t* d_error, void* stream);

/* Test hook: the binary16 values the grouped kernels stage for one Q4_K planar expert, [rows x cols] in natural K order.
 * Per weight this is RN16((q - 8) * RN16(d*sc) + RN16(8*d*sc - dmin*mn)), three roundings instead of the one rounding of
 * the exact value the reference's tensor-op path stages (planar_moe_v3.metal:165); the tests bound the deviation. */
int tsp_moe_staged_f16(const tsp_matrix_set* m, uint32_t expert, void* d_out, void* stream);

/* One whole MoE FFN sub-layer at prefill size: K-ordered rows -> route -> permute (tasks of TSP_GROUPED_TILE) -> offsets ->
 * routed copy of the rows -> grouped gate-up + SwiGLU -> grouped down (the dense shared expert rides in both launches) -> gated mixture.
 * Replaces `encode_moe_mm_many` after its router projection (moe_mm_many.cpp:126-220) on the `planar_nax_grouped_moe`
 * path (graph.mm:9293-9420). Weights: Q4_K, Pack v3 planar or plain GGUF super-blocks, hidden a multiple of 64 and channels
 * of 256. A shared expert in the routed experts' form rides in the routed launches; in another form (dense Q8_0 GGUF blocks
 * beside Q4_K experts, as the reference's model has it) it is computed by tsp_dense_mm_swiglu / tsp_dense_mm in launches of
 * its own (11 launches instead of 9). Arguments as tsp_moe_layer_decode; `tokens` <= s->base.capacity.
 * Caller-owned scratch, all device memory, nothing has to start at zero:
 *   base: as for the decode layer, except d_tasks sized tsp_moe_tasks_words(capacity, experts, selected, TSP_GROUPED_TILE);
 *         d_routed is used as binary16 rows [capacity*selected x channels]; d_hidden, d_shared_hidden and d_x32 are not
 *         used and may be NULL;
 *   d_xk: binary16 copy of the input rows in tile K order, [capacity x channels];
 *   d_xp / d_hp: binary16 rows in permuted position order, [capacity*selected x channels] / [capacity*selected x hidden];
 *   d_offsets [experts + 5]; d_s_hp: the shared expert's binary16 hidden rows, [capacity x hidden]. */
typedef struct tsp_moe_prefill_scratch {
    tsp_moe_scratch base;
    void* d_xk;
    void* d_xp;
    void* d_hp;
    uint32_t* d_offsets;
    void* d_s_hp;
} tsp_moe_prefill_scratch;
int tsp_moe_layer_prefill(const tsp_moe_weights* w, const tsp_moe_prefill_scratch* s, const void* d_x, uint64_t x_stride_bytes,
                          uint32_t x_dtype, const float* d_logits, uint64_t logits_stride_bytes, uint32_t tokens,
                          uint32_t channels, uint32_t hidden, uint32_t experts, uint32_t selected, uint32_t mode,
                          int normalize, void* d_out, uint64_t out_stride_bytes, uint32_t out_dtype, uint32_t* d_error, void* stream);

/* No counterpart in the reference (its graph always works out of caller-allocated buffers).
 *
 * The same layer as tsp_moe_layer_decode, for callers that have nowhere to get scratch from: code that runs
 * where device allocation is forbidden or unavailable -- inside a host callback or another library's plugin
 * hook, under an allocator the embedding application owns exclusively, or late in a process whose memory
 * pool is already fully handed out. The caller passes only weights, inputs and outputs; every intermediate
 * buffer lives in one array of TSP_STATIC_SCRATCH_BYTES that is part of the library image, so each GPU that
 * loads the library gives up that much memory until the process exits.
 *
 *  - Limit: the layer shape and token count must fit the array; tsp_moe_layer_decode_static_bytes() tells what
 *    a call needs (0 for an invalid shape). At hidden 2048 / FFN 512 / 512 experts / top-10 that is 34 token
 *    rows (4 187 904 of the 4 194 304 bytes; 35 rows need 4 310 784). Anything larger is refused with TSP_E_ARG and a message naming both sizes; nothing is launched.
 *  - The first call on each device looks up the array's device address (with that device current). Make that
 *    first call during start-up, before any stream capture begins.
 *  - No cudaMalloc / cudaFree / allocating library routine is called, on the first call or later.
 *  - All calls on one device share the one array, which simply keeps what the last call left there; nothing in
 *    it needs clearing between calls. Two calls whose kernels overlap on the GPU (different streams, or
 *    different host threads) would overwrite each other's intermediates: keep calls on one device ordered. */
#define TSP_STATIC_SCRATCH_BYTES (4ull << 20)
uint64_t tsp_moe_layer_decode_static_bytes(uint32_t tokens, uint32_t channels, uint32_t hidden, uint32_t experts, uint32_t selected);
int tsp_moe_layer_decode_static(const tsp_moe_weights* w,
                                const void* d_x, uint64_t x_stride_bytes, uint32_t x_dtype,
                                const float* d_logits, uint64_t logits_stride_bytes,
                                uint32_t tokens, uint32_t channels, uint32_t hidden, uint32_t experts, uint32_t selected,
                                uint32_t mode, int normalize_selected,
                                void* d_out, uint64_t out_stride_bytes, uint32_t out_dtype,
                                uint32_t* d_error, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TSP_MOE_H */
