/*
 * CPU oracle for the block-quantised routed-MoE FFN path. TEST INFRASTRUCTURE ONLY.
 *
 * This is a plain-C restatement of the reference's scalar, double-accumulating CPU
 * algorithm. It exists to check the CUDA path and to serve as the timed CPU baseline.
 * Nothing in the product library links, loads or calls it; only the test-suite, the
 * smoke check and the benchmark's cpu-baseline / reference arms may.
 *
 * Parity pins: every function is checked against the reference's own known-answer
 * vectors (restated in tests/test_oracle_pins.py) and, where the reference's CPU sources
 * compile, against those sources themselves (oracle/_ref, see oracle/Makefile), with the
 * resulting outputs committed as fixtures under tests/golden/.
 *
 * All functions return 0 on success and a negative code on refusal; they never abort.
 */
#ifndef TSP_ORACLE_H
#define TSP_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    TSO_OK = 0,
    TSO_E_SHAPE = -1,     /* size / shape mismatch */
    TSO_E_TYPE = -2,      /* encoding without a decoder */
    TSO_E_NONFINITE = -3, /* non-finite weight, input or result */
    TSO_E_RANGE = -4,     /* index or factor out of range */
};

/* GGUF type ids handled here: 0 F32, 1 F16, 7 Q5_1, 8 Q8_0, 12 Q4_K, 13 Q5_K, 14 Q6_K, 20 IQ4_NL, 30 BF16 (every encoding
 * numeric.cpp decodes; the CUDA kernels cover 7, 8, 12 and 13). */
int tso_block_geometry(uint32_t type, uint32_t* elements_per_block, uint32_t* bytes_per_block);

/* binary16 -> binary32, all 65536 patterns (numeric.cpp:81-91). */
float tso_binary16(uint16_t bits);

/* Exact logical value of element `index` of one encoded block (numeric.cpp:33-68). */
double tso_value(uint32_t type, const uint8_t* block, uint32_t index);

/* Whole-tensor decode to FP32, one rounding from the exact double (numeric.cpp:97-148). */
int tso_dequantize(uint32_t type, const uint8_t* bytes, size_t nbytes, float* out, size_t elements);

/* Scalar double-accumulating matrix-vector product (numeric.cpp:150-184). */
int tso_gemv_f64(uint32_t type, const uint8_t* matrix, size_t nbytes, uint32_t columns, uint32_t rows,
                 const double* input, double* output);
int tso_gemv_f32(uint32_t type, const uint8_t* matrix, size_t nbytes, uint32_t columns, uint32_t rows,
                 const float* input, double* output);

/* operators.cpp:28-40 */
double tso_sigmoid(double v);
double tso_silu(double v);
double tso_softplus(double v);

/* Hyper-connection residual read / write around the FFN sub-layer (operators.cpp:42-96).
 * tso_gated_residual: streams [branches x channels] -> grouped RMS (per branch, gains elementwise) -> bottleneck
 * silu(down . normalized / branches) [rank] -> scores = up . bottleneck [branches x channels], inject logits =
 * inject . normalized [branches]; input[c] = sum_b normalized[b][c] * sigmoid(scores[b][c]) / branches,
 * write_scales[b] = 2 * sigmoid(inject_logit[b] / branches). The intermediates are returned too (any may be NULL).
 * tso_residual_write: out[b][c] = streams[b][c] + scales[b] * output[c]. */
int tso_gated_residual(const double* streams, const double* gains, const double* down, const double* up, const double* inject,
                       size_t branches, size_t channels, size_t rank, double epsilon, double* input, double* write_scales,
                       double* normalized, double* scores, double* inject_logits);
int tso_residual_write(const double* streams, const double* output, const double* scales, size_t branches, size_t channels, double* out);

/* Top-k by descending logit, ties to the lower id; mode 0 softmax, 1 sigmoid (routing.cpp:11-40). */
int tso_route(const double* logits, size_t experts, size_t selected, uint32_t mode, int normalize_selected,
              uint32_t* indices, double* weights);

/* out[c] = sigmoid(shared_logit)*shared[c] + sum_r w[r]*experts[r][c] in route order (routing.cpp:42-61). */
int tso_mixture(const double* experts, const double* weights, size_t selected, const double* shared,
                size_t channels, double shared_logit, double* out);

/* Top-64 of a row of logits for the sampler (sampling.cpp:473-515; row type sampling.hpp:21-29, 528 bytes). Non-finite values
 * are left out and the first such column is recorded; the first subnormal column is recorded too (the value still competes).
 * Order: value descending with -0 == +0, ties to the lower column; the raw bits of the logits are kept. Unused slots hold
 * -infinity and id 0. */
#define TSO_TOPK_CAPACITY 64
typedef struct {
    uint32_t vocabulary, count, first_nonfinite_col, first_subnormal_col;
    uint32_t ids[TSO_TOPK_CAPACITY];
    float logits[TSO_TOPK_CAPACITY];
} tso_topk_row;
int tso_logit_topk_row(const float* logits, size_t vocabulary, tso_topk_row* out);

/* Lane layouts of whole rows (expert_lanes.cpp:75-130), lossless: a row keeps its byte count; the block headers move to a leading
 * run and the quant bytes are regrouped so that one lane's bytes of consecutive blocks are adjacent. type 8 (Q8_0, layout
 * `q8_lanes_v1`): 2-byte scales first, then runs of up to 16 blocks, byte i of block b at meta + run*512 + i*width + b%16.
 * type 12 (Q4_K): 16-byte headers first, runs of up to 4 blocks, quant byte (pair p, lane l) at meta + run*512 + l*width*... as
 * packed_quant_offset states. nbytes must hold whole rows. */
int tso_lanes_pack_rows(uint32_t type, uint32_t columns, const uint8_t* original, uint8_t* packed, size_t nbytes);
int tso_lanes_unpack_rows(uint32_t type, uint32_t columns, const uint8_t* packed, uint8_t* original, size_t nbytes);

/* ---- Pack v3 planar expert layout (planar_pack_v3.cpp:601-896): types 12 (Q4_K), 8 (Q8_0), 13 (Q5_K), 7 (Q5_1) ---- */
typedef struct {
    uint32_t source_type, columns, rows, blocks_per_row;
    uint64_t source_row_bytes, planar_row_bytes, source_expert_bytes, planar_expert_bytes;
    uint64_t qs_offset, sm_offset, dm_offset;
    uint64_t qh_offset;   /* fifth-bit plane of the five-bit encodings (types 13 and 7), 0 otherwise */
} tso_planar_spec;

int tso_make_expert_spec(uint32_t source_type, uint32_t columns, uint32_t rows, tso_planar_spec* spec);
void tso_pack_sm16(const uint8_t s12[12], uint8_t sm[16]);
int tso_unpack_sm16(const uint8_t sm[16], uint8_t s12[12]);
int tso_pack_expert_planar(const tso_planar_spec* spec, const uint8_t* gguf, uint8_t* planar);
int tso_unpack_expert_planar(const tso_planar_spec* spec, const uint8_t* planar, uint8_t* gguf);
int tso_dequantize_expert_planar(const tso_planar_spec* spec, const uint8_t* planar, float* out);

/* ---- token permutation tables (grouped_mpp.metal:12-66 semantics) ---- */
/* token_map[e*tokens + j] = token*selected + slot of the j-th token (ascending) routed to e; counts[e]. */
int tso_grouped_routes(const uint32_t* indices, uint32_t tokens, uint32_t experts, uint32_t selected,
                       uint32_t* token_map, uint32_t* counts);
/* tasks = {live_tiles, routes, (expert,start)*, UINT32_MAX padding}; length 2 + 2*(tokens*selected/tile + experts). */
int tso_grouped_tasks(const uint32_t* counts, uint32_t tokens, uint32_t experts, uint32_t selected,
                      uint32_t tile, uint32_t* tasks);

/* ---- one whole MoE FFN layer, composed as ffn_check.cpp:104-139 ---- */
typedef struct {
    uint32_t channels, hidden, experts, selected;
    uint32_t expert_type;           /* encoding of gate/up/down expert tensors (12, 13, 8 or 7) */
    uint32_t shared_type;           /* encoding of the shared expert tensors */
    const uint8_t* gate;            /* [experts][hidden x channels] GGUF bytes, expert-major */
    const uint8_t* up;
    const uint8_t* down;            /* [experts][channels x hidden] */
    const uint8_t* shared_gate;     /* [hidden x channels] */
    const uint8_t* shared_up;
    const uint8_t* shared_down;     /* [channels x hidden] */
    const float* shared_router;     /* F32 [channels], may be NULL: gate logit supplied as +inf-like "always on" is NOT assumed; NULL means logit 0 */
    const float* router;            /* F32 [experts x channels] or NULL when logits are supplied */
    uint32_t mode;                  /* 0 softmax, 1 sigmoid */
    int normalize_selected;
    uint32_t down_type;             /* encoding of the down expert tensors when it differs from gate/up (0: expert_type) */
} tso_layer;

typedef struct {
    uint32_t* indices;   /* [tokens x selected] or NULL */
    double* weights;     /* [tokens x selected] or NULL */
    double* activated;   /* [tokens x selected x hidden] or NULL */
    double* routed;      /* [tokens x selected x channels] or NULL */
    double* shared_act;  /* [tokens x hidden] or NULL */
    double* shared_out;  /* [tokens x channels] or NULL */
    double* shared_logit;/* [tokens] or NULL */
} tso_layer_stages;

/* x: [tokens x channels] FP32; logits: [tokens x experts] FP32 or NULL (then layer.router is used);
 * out: [tokens x channels] double. Rows are independent; `threads` host threads split the token range. */
int tso_moe_layer(const tso_layer* layer, const float* x, const float* logits, uint32_t tokens,
                  double* out, const tso_layer_stages* stages, uint32_t threads);

#ifdef __cplusplus
}
#endif
#endif
