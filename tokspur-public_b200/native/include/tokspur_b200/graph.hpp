// CUDA-backed execution context with the ownership and batch rules of the reference's graph
// (native/include/tokspur/graph.hpp:427-495, 709-717): buffers are opaque checked capabilities, allocation / upload /
// read / release happen only between batches, weights are immutable registered imports, encode calls never allocate
// or read back, one host thread owns the graph, and a batch's device-side failures surface once, at submit().
#pragma once

#include <cstddef>
#include <cstdint>
#include <optional>
#include <span>
#include <stdexcept>
#include <string>
#include <vector>

#include "tsp_moe.h"

namespace tokspur_b200 {

class FormatError : public std::runtime_error {
public:
    using std::runtime_error::runtime_error;
};

// Opaque, checked capability: a released or foreign view is never silently rebound. Offsets/lengths are bytes.
struct GpuView {
    uint64_t owner = 0;
    size_t slot = 0;
    uint64_t offset = 0;
    uint64_t bytes = 0;
};
struct GpuRowsF32 {
    GpuView view;
    uint32_t rows = 0, columns = 0;
    uint64_t stride_bytes = 0;
};
struct PlanarMatrixShape {
    uint32_t source_type = 0;  // 8 (Q8_0), 12 (Q4_K)
    uint32_t kind = 0;         // PlanarKind: 2/3 q4k co-located gate/up, 6/7 q8 co-located, 9 q8 planar, 10 q4k planar (this build's down extension)
    uint32_t columns = 0, rows = 0, experts = 0;
};
enum class RouterMode : uint32_t { softmax, sigmoid };
// Registered identity of a weight tensor on the prefill path (native/include/tokspur/moe_mm_many.hpp:7-10): raw GGUF blocks or
// a registered Pack v3 planar matrix.
enum class PrefillWeightLayout : uint32_t { gguf = 0, planar = 1 };
struct BatchResult { uint64_t dispatches = 0; double wall_ms = 0, gpu_ms = 0; };

class CudaGraph {
public:
    explicit CudaGraph(int device, uint64_t byte_budget);
    ~CudaGraph();
    CudaGraph(const CudaGraph&) = delete;
    CudaGraph& operator=(const CudaGraph&) = delete;

    [[nodiscard]] GpuView zeros(uint64_t bytes, std::string label);
    [[nodiscard]] GpuView upload(std::span<const std::byte> data, std::string label, bool immutable = true);
    [[nodiscard]] GpuView slice(GpuView buffer, uint64_t offset, uint64_t bytes) const;
    void write(GpuView destination, std::span<const std::byte> data);
    [[nodiscard]] std::vector<std::byte> read(GpuView source) const;
    void release(GpuView full_buffer);
    [[nodiscard]] uint64_t live_bytes() const noexcept { return live_bytes_; }
    [[nodiscard]] uint64_t allocations() const noexcept { return allocations_; }

    // Lossless Pack v3 planar registration (graph.mm:9021-9059): immutable, 16-byte aligned, size == planar bytes * experts.
    void register_planar_matrix(GpuView matrix, PlanarMatrixShape shape);
    [[nodiscard]] std::optional<PlanarMatrixShape> planar_matrix_shape(GpuView matrix) const;

    void begin();
    void abort();                          // discards an unsubmitted batch
    [[nodiscard]] BatchResult submit();    // waits once, checks the sticky error word, throws FormatError if it is set

    // operators (each is one or two launches through the C ABI; all require an open batch)
    void gemv_f32(GpuView matrix, GpuView input, GpuView output, uint32_t columns, uint32_t rows);   // gemv(type 0)
    // the same projection for `tokens` strided input rows (moe_router_f32_batch): output rows of `rows` values at out_stride_bytes
    void gemv_f32_rows(GpuView matrix, GpuView input, uint64_t in_stride_bytes, uint32_t tokens, GpuView output, uint64_t out_stride_bytes,
                       uint32_t columns, uint32_t rows);
    void route(GpuView logits, GpuView indices, GpuView weights, uint32_t selected, RouterMode mode, bool normalize_selected);
    // Dense projections through the decode-size kernels (graph.hpp:730-746, 780): encoding 0 (F32 rows), 8 (Q8_0) or 12 (Q4_K); a
    // quantised matrix is GGUF rows unless it was registered as a planar matrix. out[t][r] = sum_c W[r][c] in[t][c].
    void gemv(uint32_t encoding, GpuView matrix, GpuView input, GpuView output, uint32_t columns, uint32_t rows);
    void gemv_rows(uint32_t encoding, GpuView matrix, GpuRowsF32 input, GpuRowsF32 output);
    // `width` token-major input rows of `columns` values, output rows of `rows` values, both densely packed (q8_many.cpp:20-29)
    void q8_matvec_many(GpuView matrix, GpuView input, GpuView output, uint32_t columns, uint32_t rows, uint32_t width);
    void verify_nax_dense_q8(GpuView matrix, GpuRowsF32 input, GpuRowsF32 output);
    // Dense Q8_0 projection of a prefill-size row batch on the tensor cores (graph.hpp:859-860, 767): binary16 operands, FP32
    // accumulate, FP32 rows out. prepare_dense_mm_q8 (between batches) sizes the staging of the binary16 input rows; the encode
    // call never allocates. `reuse_staged` skips the conversion when the previous dense_mm_q8 staged the same input rows.
    // Matrix: raw Q8_0 blocks [rows x columns], rows a multiple of 128, columns of 256.
    void prepare_dense_mm_q8(PrefillWeightLayout layout, uint32_t max_rows, uint32_t max_columns);
    void dense_mm_q8(PrefillWeightLayout layout, GpuView matrix, GpuRowsF32 input, GpuRowsF32 output, bool reuse_staged = false);
    [[nodiscard]] static uint32_t dense_mm_q8_dispatches(bool reuse_staged = false) { return reuse_staged ? 1u : 2u; }
    // Batched routing and mixture (graph.hpp:852-853): `tokens` rows of `experts` logits; expert outputs [tokens*selected x channels]
    void prefill_route_batch(GpuView logits, GpuView indices, GpuView weights, uint32_t experts, uint32_t selected, uint32_t tokens,
                             RouterMode mode, bool normalize_selected);
    void prefill_mixture_batch(GpuView experts, GpuView weights, GpuView shared, GpuView shared_logit, GpuRowsF32 output, uint32_t selected);
    void mixture(GpuView expert_outputs, GpuView weights, GpuView shared_output, GpuView shared_logit, GpuView output);   // graph.hpp:1102
    // Router projection of a batch with the shared-router row in the same pass (moe_router_f32_window + moe_shared_router_rows,
    // graph.mm:5812, 5884) and the router-margin audit (graph.hpp:162-172, graph.mm:4911-4985)
    void moe_router_rows(GpuView router, GpuView shared_router, GpuRowsF32 input, GpuView logits, GpuView shared_logits, uint32_t experts);
    void configure_router_margin_audit(bool enabled) { require_idle(); margin_audit_ = enabled; }
    void configure_router_margin_epsilon(float epsilon);
    [[nodiscard]] bool router_margin_audit() const noexcept { return margin_audit_; }
    [[nodiscard]] tsp_router_margin_telemetry router_margin_telemetry() const noexcept { return margin_telemetry_; }
    void reset_router_margin_telemetry() noexcept { margin_telemetry_ = {}; }
    // routes `tokens` (<= 2048) rows; with the audit enabled it also records each row's top-k margin into the scratch that
    // prepare_router_margin_scratch() allocated between batches (encode calls never allocate)
    void prepare_router_margin_scratch();
    void moe_route_rows(GpuView logits, GpuView indices, GpuView weights, uint32_t experts, uint32_t selected, uint32_t tokens, RouterMode mode,
                        bool normalize_selected);
    [[nodiscard]] bool evaluate_router_margin(uint32_t tokens);   // waits for the stream; true when a row's margin is within 2 epsilon
    // The sampler's top-64 rows of a batch of logits rows (graph.hpp:1030-1033): scratch of logit_topk_scratch_bytes(), one
    // 528-byte row (GpuLogitTopKRow, sampling.hpp:21-29) per logits row in `out_rows`
    static uint64_t logit_topk_scratch_bytes(uint32_t max_rows, uint32_t max_vocabulary = 1u << 20) { return tsp_logit_topk_scratch_bytes(max_rows, max_vocabulary); }
    static uint64_t logit_topk_output_bytes(uint32_t max_rows) { return tsp_logit_topk_output_bytes(max_rows); }
    void logit_topk(GpuRowsF32 logits, GpuView partial_scratch, GpuView out_rows);
    // Hyper-connection residual read / write around the FFN sub-layer (graph.hpp:1056-1058)
    void residual_read(GpuView normalized, GpuView scores, GpuView inject_logits, GpuView output, GpuView scales, uint32_t branches, uint32_t channels);
    void residual_write(GpuView streams, GpuView output, GpuView scales, GpuView destination);

    // raw access for the composed encoders in moe.cpp
    [[nodiscard]] void* device_pointer(GpuView view, bool for_write = false) const;
    [[nodiscard]] uint32_t* error_word() const noexcept { return error_; }
    [[nodiscard]] void* stream() const noexcept { return stream_; }
    void count_dispatches(uint64_t n) { require_batch(); dispatches_ += n; }
    void require_batch() const;

private:
    struct Buffer { void* ptr = nullptr; uint64_t bytes = 0; bool immutable = false; bool live = false; std::string label; };
    struct Planar { size_t slot; uint64_t offset; PlanarMatrixShape shape; };
    const Buffer& checked(GpuView view) const;
    void require_idle() const;
    void select_device() const;
    void check(int rc) const;

    uint64_t owner_;
    int device_;
    uint64_t budget_, live_bytes_ = 0, allocations_ = 0;
    std::vector<Buffer> buffers_;
    std::vector<Planar> planar_;
    uint32_t* error_ = nullptr;
    void* stream_ = nullptr;
    void *ev0_ = nullptr, *ev1_ = nullptr;
    bool in_batch_ = false, frozen_ = false, margin_audit_ = false;
    float margin_epsilon_ = 1.0e-4f;
    void* dense_staging_ = nullptr;       // binary16 input rows of dense_mm_q8 in tile K order, then 256 item-counter words
    uint64_t dense_staging_rows_ = 0, dense_staging_cols_ = 0;
    uint32_t dense_counter_ = 0;          // next unused counter word
    float* margins_ = nullptr;            // per-row top-k margins of the last moe_route_rows (2048 rows, as the reference's scratch)
    tsp_router_margin_telemetry margin_telemetry_{};
    tsp_matrix_set dense_set(uint32_t encoding, GpuView matrix, uint32_t columns, uint32_t rows) const;
    uint64_t dispatches_ = 0;
    double batch_start_ = 0;
};

}  // namespace tokspur_b200
