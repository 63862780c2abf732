// CUDA-backed graph: capability-checked buffers, batch begin/submit with the sticky error word, operator forwarding
// to the C ABI. Mirrors the contract of the reference's MetalGraph for the MoE path (graph.mm:990, 3366, 3822, 3977, 9021).
#include "tokspur_b200/graph.hpp"

#include <cuda_runtime.h>

#include <atomic>
#include <chrono>

namespace tokspur_b200 {
namespace {
std::atomic<uint64_t> next_owner{1};
void cuda(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw FormatError(std::string(what) + ": " + cudaGetErrorString(e));
}
double now_ms() { return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now().time_since_epoch()).count(); }
}

CudaGraph::CudaGraph(int device, uint64_t byte_budget) : owner_(next_owner++), device_(device), budget_(byte_budget) {
    cuda(cudaSetDevice(device), "cudaSetDevice");
    cudaStream_t st;
    cuda(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking), "cudaStreamCreate");
    stream_ = st;
    cuda(cudaMalloc(reinterpret_cast<void**>(&error_), sizeof(uint32_t)), "error word");
    cuda(cudaMemsetAsync(error_, 0, sizeof(uint32_t), st), "error word");
    cuda(cudaStreamSynchronize(st), "error word");
    cudaEvent_t a, b;
    cuda(cudaEventCreate(&a), "event"); cuda(cudaEventCreate(&b), "event");
    ev0_ = a; ev1_ = b;
}

CudaGraph::~CudaGraph() {
    cudaSetDevice(device_);
    cudaStreamSynchronize(static_cast<cudaStream_t>(stream_));
    for (auto& b : buffers_) if (b.live) cudaFree(b.ptr);
    cudaFree(error_);
    if (margins_) cudaFree(margins_);
    if (dense_staging_) cudaFree(dense_staging_);
    cudaEventDestroy(static_cast<cudaEvent_t>(ev0_));
    cudaEventDestroy(static_cast<cudaEvent_t>(ev1_));
    cudaStreamDestroy(static_cast<cudaStream_t>(stream_));
}

// one host thread may own graphs on several devices: every entry that touches the device selects this graph's own first
void CudaGraph::select_device() const { cuda(cudaSetDevice(device_), "cudaSetDevice"); }
void CudaGraph::require_idle() const { if (in_batch_) throw FormatError("operation is permitted only between batches"); }
void CudaGraph::require_batch() const {
    if (!in_batch_) throw FormatError("no batch is open");
    select_device();   // every operator and composed encoder passes here before its launches
}
void CudaGraph::check(int rc) const { if (rc != TSP_OK) throw FormatError(tsp_last_error()); }

const CudaGraph::Buffer& CudaGraph::checked(GpuView v) const {
    if (v.owner != owner_ || v.slot >= buffers_.size() || !buffers_[v.slot].live) throw FormatError("foreign or released buffer view");
    const auto& b = buffers_[v.slot];
    if (v.offset > b.bytes || v.bytes > b.bytes - v.offset) throw FormatError("buffer view out of range");
    return b;
}

GpuView CudaGraph::zeros(uint64_t bytes, std::string label) {
    require_idle();
    if (!bytes || bytes > budget_ - live_bytes_) throw FormatError("allocation exceeds the graph's byte budget");
    void* p = nullptr;
    select_device();
    cuda(cudaMalloc(&p, bytes), "cudaMalloc");
    // fills and copies run on the graph's own (non-blocking) stream and are waited for: a non-blocking stream does not
    // order itself after the legacy default stream, so a fill issued there could still be in flight at the first launch
    cuda(cudaMemsetAsync(p, 0, bytes, static_cast<cudaStream_t>(stream_)), "cudaMemset");
    cuda(cudaStreamSynchronize(static_cast<cudaStream_t>(stream_)), "cudaMemset");
    buffers_.push_back({p, bytes, false, true, std::move(label)});
    live_bytes_ += bytes; ++allocations_;
    return {owner_, buffers_.size() - 1, 0, bytes};
}

GpuView CudaGraph::upload(std::span<const std::byte> data, std::string label, bool immutable) {
    const auto v = zeros(data.size(), std::move(label));
    cuda(cudaMemcpyAsync(buffers_[v.slot].ptr, data.data(), data.size(), cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream_)), "upload");
    cuda(cudaStreamSynchronize(static_cast<cudaStream_t>(stream_)), "upload");
    buffers_[v.slot].immutable = immutable;
    return v;
}

GpuView CudaGraph::slice(GpuView buffer, uint64_t offset, uint64_t bytes) const {
    checked(buffer);
    if (offset > buffer.bytes || bytes > buffer.bytes - offset || !bytes) throw FormatError("slice out of range");
    return {buffer.owner, buffer.slot, buffer.offset + offset, bytes};
}

void CudaGraph::write(GpuView dst, std::span<const std::byte> data) {
    require_idle();
    const auto& b = checked(dst);
    if (b.immutable || data.size() != dst.bytes) throw FormatError("write to an immutable buffer or size mismatch");
    select_device();
    cuda(cudaMemcpyAsync(static_cast<char*>(b.ptr) + dst.offset, data.data(), data.size(), cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream_)), "write");
    cuda(cudaStreamSynchronize(static_cast<cudaStream_t>(stream_)), "write");
}

std::vector<std::byte> CudaGraph::read(GpuView src) const {
    require_idle();
    const auto& b = checked(src);
    std::vector<std::byte> out(src.bytes);
    select_device();
    cuda(cudaMemcpyAsync(out.data(), static_cast<const char*>(b.ptr) + src.offset, src.bytes, cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream_)), "read");
    cuda(cudaStreamSynchronize(static_cast<cudaStream_t>(stream_)), "read");
    return out;
}

void CudaGraph::release(GpuView full) {
    require_idle();
    const auto& b = checked(full);
    select_device();
    if (full.offset || full.bytes != b.bytes) throw FormatError("release needs the full buffer view");
    for (const auto& p : planar_) if (p.slot == full.slot) throw FormatError("a registered planar matrix cannot be released");
    cuda(cudaFree(b.ptr), "cudaFree");
    live_bytes_ -= b.bytes;
    buffers_[full.slot].live = false;
}

void CudaGraph::register_planar_matrix(GpuView matrix, PlanarMatrixShape shape) {
    require_idle();
    if (frozen_) throw FormatError("planar matrices are registered before the first batch");
    const auto& b = checked(matrix);
    if (!b.immutable) throw FormatError("planar matrix must be an immutable import");
    if (shape.source_type != TSP_TYPE_Q4_K && shape.source_type != TSP_TYPE_Q8_0) throw FormatError("unsupported planar source type");
    const bool q4 = shape.source_type == TSP_TYPE_Q4_K;
    const bool kind_ok = q4 ? (shape.kind == 2 || shape.kind == 3 || shape.kind == 10) : (shape.kind == 6 || shape.kind == 7 || shape.kind == 9);
    if (!kind_ok) throw FormatError("planar kind does not match its source type");
    const uint64_t per = tsp_expert_bytes(shape.source_type, TSP_LAYOUT_PLANAR, shape.rows, shape.columns);
    const bool coloc = shape.kind == 2 || shape.kind == 3 || shape.kind == 6 || shape.kind == 7;
    // a co-located tensor holds half the experts as [gate, up] pairs: as many expert-sized blocks as `experts`
    if (!per || !shape.experts || (coloc && shape.experts % 2) || matrix.bytes != per * shape.experts) throw FormatError("planar matrix byte size mismatch");
    if ((reinterpret_cast<uintptr_t>(b.ptr) + matrix.offset) % 16) throw FormatError("planar matrix must be 16-byte aligned");
    if (planar_.size() >= 2048) throw FormatError("too many planar matrices");
    for (const auto& p : planar_)
        if (p.slot == matrix.slot && p.offset == matrix.offset) throw FormatError("planar matrix registered twice");
    planar_.push_back({matrix.slot, matrix.offset, shape});
}

std::optional<PlanarMatrixShape> CudaGraph::planar_matrix_shape(GpuView matrix) const {
    for (const auto& p : planar_) if (p.slot == matrix.slot && p.offset == matrix.offset && matrix.owner == owner_) return p.shape;
    return std::nullopt;
}

void CudaGraph::begin() {
    require_idle();
    select_device();
    frozen_ = true;
    dispatches_ = 0;
    batch_start_ = now_ms();
    check(tsp_error_word_reset(error_, stream_));
    cuda(cudaEventRecord(static_cast<cudaEvent_t>(ev0_), static_cast<cudaStream_t>(stream_)), "event record");
    in_batch_ = true;   // only once everything that can throw has succeeded
}

void CudaGraph::abort() {
    if (!in_batch_) return;
    cudaStreamSynchronize(static_cast<cudaStream_t>(stream_));   // launches are asynchronous: let what was encoded drain, publish nothing
    in_batch_ = false;
}

BatchResult CudaGraph::submit() {
    require_batch();
    in_batch_ = false;   // whatever happens below, the batch is over: a throwing submit must not leave the graph stuck in a batch
    select_device();
    cuda(cudaEventRecord(static_cast<cudaEvent_t>(ev1_), static_cast<cudaStream_t>(stream_)), "event record");
    uint32_t word = 0;
    const int rc = tsp_error_word_read(error_, stream_, &word);
    if (rc == TSP_E_DEVICE) throw FormatError(tsp_last_error());
    check(rc);
    float gpu_ms = 0;
    cuda(cudaEventElapsedTime(&gpu_ms, static_cast<cudaEvent_t>(ev0_), static_cast<cudaEvent_t>(ev1_)), "event time");
    return {dispatches_, now_ms() - batch_start_, gpu_ms};
}

void* CudaGraph::device_pointer(GpuView view, bool for_write) const {
    const auto& b = checked(view);
    if (for_write && b.immutable) throw FormatError("operator output is an immutable buffer");
    return static_cast<char*>(b.ptr) + view.offset;
}

void CudaGraph::gemv_f32(GpuView matrix, GpuView input, GpuView output, uint32_t columns, uint32_t rows) {
    require_batch();
    if (matrix.bytes != uint64_t(columns) * rows * 4 || input.bytes != uint64_t(columns) * 4 || output.bytes != uint64_t(rows) * 4)
        throw FormatError("GEMV shape mismatch");
    check(tsp_gemv_f32(static_cast<const float*>(device_pointer(matrix)), rows, columns, static_cast<const float*>(device_pointer(input)),
                       uint64_t(columns) * 4, 1, static_cast<float*>(device_pointer(output, true)), uint64_t(rows) * 4, error_, stream_));
    ++dispatches_;
}

void CudaGraph::gemv_f32_rows(GpuView matrix, GpuView input, uint64_t in_stride_bytes, uint32_t tokens, GpuView output, uint64_t out_stride_bytes,
                              uint32_t columns, uint32_t rows) {
    require_batch();
    if (!tokens || matrix.bytes != uint64_t(columns) * rows * 4 || in_stride_bytes < uint64_t(columns) * 4 || out_stride_bytes < uint64_t(rows) * 4 ||
        input.bytes < uint64_t(tokens - 1) * in_stride_bytes + uint64_t(columns) * 4 ||
        output.bytes < uint64_t(tokens - 1) * out_stride_bytes + uint64_t(rows) * 4)
        throw FormatError("GEMV shape mismatch");
    check(tsp_gemv_f32(static_cast<const float*>(device_pointer(matrix)), rows, columns, static_cast<const float*>(device_pointer(input)),
                       in_stride_bytes, tokens, static_cast<float*>(device_pointer(output, true)), out_stride_bytes, error_, stream_));
    ++dispatches_;
}

void CudaGraph::route(GpuView logits, GpuView indices, GpuView weights, uint32_t selected, RouterMode mode, bool normalize_selected) {
    require_batch();
    const uint32_t experts = static_cast<uint32_t>(logits.bytes / 4);
    if (logits.bytes % 4 || indices.bytes != uint64_t(selected) * 4 || weights.bytes != uint64_t(selected) * 4) throw FormatError("invalid router shape/mode");
    check(tsp_moe_route(static_cast<const float*>(device_pointer(logits)), logits.bytes, 1, experts, selected, uint32_t(mode), normalize_selected,
                        static_cast<uint32_t*>(device_pointer(indices, true)), static_cast<float*>(device_pointer(weights, true)), error_, stream_));
    ++dispatches_;
}


// ---- dense projections --------------------------------------------------------------------------------------------------
tsp_matrix_set CudaGraph::dense_set(uint32_t encoding, GpuView matrix, uint32_t columns, uint32_t rows) const {
    if (encoding != TSP_TYPE_Q8_0 && encoding != TSP_TYPE_Q4_K) throw FormatError("unsupported GEMV encoding");
    const auto planar = planar_matrix_shape(matrix);
    const uint32_t layout = planar ? TSP_LAYOUT_PLANAR : TSP_LAYOUT_GGUF;
    const uint64_t bytes = tsp_expert_bytes(encoding, layout, rows, columns);
    if (!bytes || matrix.bytes != bytes) throw FormatError("GEMV shape mismatch");
    return tsp_matrix_set{device_pointer(matrix), nullptr, bytes, 1, 1, rows, columns, encoding, layout};
}

void CudaGraph::gemv(uint32_t encoding, GpuView matrix, GpuView input, GpuView output, uint32_t columns, uint32_t rows) {
    gemv_rows(encoding, matrix, {input, 1, columns, uint64_t(columns) * 4}, {output, 1, rows, uint64_t(rows) * 4});
}

void CudaGraph::gemv_rows(uint32_t encoding, GpuView matrix, GpuRowsF32 input, GpuRowsF32 output) {
    require_batch();
    if (!input.rows || input.rows != output.rows || input.view.bytes < uint64_t(input.rows - 1) * input.stride_bytes + uint64_t(input.columns) * 4 ||
        output.view.bytes < uint64_t(output.rows - 1) * output.stride_bytes + uint64_t(output.columns) * 4)
        throw FormatError("GEMV shape mismatch");
    if (encoding == 0) { gemv_f32_rows(matrix, input.view, input.stride_bytes, input.rows, output.view, output.stride_bytes, input.columns, output.columns); return; }
    const auto set = dense_set(encoding, matrix, input.columns, output.columns);
    check(tsp_moe_project(&set, static_cast<const float*>(device_pointer(input.view)), input.stride_bytes, 1, input.rows, 1, nullptr, nullptr, nullptr,
                          static_cast<float*>(device_pointer(output.view, true)), output.stride_bytes, 0, error_, stream_));
    ++dispatches_;
}

void CudaGraph::q8_matvec_many(GpuView matrix, GpuView input, GpuView output, uint32_t columns, uint32_t rows, uint32_t width) {
    if (!width || width > 64 || input.bytes != uint64_t(columns) * width * 4 || output.bytes != uint64_t(rows) * width * 4) throw FormatError("Q8 many-row shape mismatch");
    gemv_rows(TSP_TYPE_Q8_0, matrix, {input, width, columns, uint64_t(columns) * 4}, {output, width, rows, uint64_t(rows) * 4});
}

void CudaGraph::verify_nax_dense_q8(GpuView matrix, GpuRowsF32 input, GpuRowsF32 output) {
    if (input.rows < 1 || input.rows > 16) throw FormatError("verify batch must hold 1..16 rows");
    gemv_rows(TSP_TYPE_Q8_0, matrix, input, output);
}

// ---- dense Q8_0 row batches on the tensor cores (dense_mm_q8, graph.mm:5009-5100) -------------------------------------------
namespace { constexpr uint32_t kDenseCounters = 256; }

void CudaGraph::prepare_dense_mm_q8(PrefillWeightLayout layout, uint32_t max_rows, uint32_t max_columns) {
    require_idle();
    select_device();
    if (layout != PrefillWeightLayout::gguf) throw FormatError("dense Q8_0 GEMM reads raw GGUF blocks only");
    if (!max_rows || !max_columns || max_columns % 256) throw FormatError("dense Q8_0 GEMM staging shape");
    if (dense_staging_ && dense_staging_rows_ * dense_staging_cols_ >= uint64_t(max_rows) * max_columns) return;
    if (dense_staging_) { cuda(cudaFree(dense_staging_), "dense staging"); dense_staging_ = nullptr; }
    const uint64_t bytes = uint64_t(max_rows) * max_columns * 2 + kDenseCounters * 4;
    cuda(cudaMalloc(&dense_staging_, bytes), "dense staging");
    cuda(cudaMemset(dense_staging_, 0, bytes), "dense staging");
    dense_staging_rows_ = max_rows; dense_staging_cols_ = max_columns; dense_counter_ = 0;
}

void CudaGraph::dense_mm_q8(PrefillWeightLayout layout, GpuView matrix, GpuRowsF32 input, GpuRowsF32 output, bool reuse_staged) {
    require_batch();
    if (layout != PrefillWeightLayout::gguf || planar_matrix_shape(matrix)) throw FormatError("dense Q8_0 GEMM reads raw GGUF blocks only");
    if (!input.rows || input.rows != output.rows || !input.columns || input.columns % 256 || !output.columns || output.columns % 128 ||
        input.stride_bytes < uint64_t(input.columns) * 4 || input.stride_bytes % 16 || output.stride_bytes < uint64_t(output.columns) * 4 || output.stride_bytes % 16 ||
        input.view.bytes < uint64_t(input.rows - 1) * input.stride_bytes + uint64_t(input.columns) * 4 ||
        output.view.bytes < uint64_t(output.rows - 1) * output.stride_bytes + uint64_t(output.columns) * 4)
        throw FormatError("dense Q8_0 GEMM shape mismatch");
    if (!dense_staging_ || uint64_t(input.rows) * input.columns > dense_staging_rows_ * dense_staging_cols_)
        throw FormatError("dense Q8_0 GEMM: call prepare_dense_mm_q8() between batches with at least this many rows and columns");
    const uint64_t bytes = tsp_expert_bytes(TSP_TYPE_Q8_0, TSP_LAYOUT_GGUF, output.columns, input.columns);
    if (!bytes || matrix.bytes != bytes) throw FormatError("dense Q8_0 GEMM matrix extent");
    const tsp_matrix_set set{device_pointer(matrix), nullptr, bytes, 1, 1, output.columns, input.columns, TSP_TYPE_Q8_0, TSP_LAYOUT_GGUF};
    const uint64_t xk_stride = uint64_t(input.columns) * 2;
    auto* counters = reinterpret_cast<uint32_t*>(static_cast<char*>(dense_staging_) + dense_staging_rows_ * dense_staging_cols_ * 2);
    if (dense_counter_ == kDenseCounters) {   // every word has been used once: clear them in stream order
        cuda(cudaMemsetAsync(counters, 0, kDenseCounters * 4, static_cast<cudaStream_t>(stream_)), "dense counters");
        dense_counter_ = 0;
    }
    if (!reuse_staged) {
        check(tsp_moe_rows_f16k(device_pointer(input.view), input.stride_bytes, 0, input.rows, input.columns, dense_staging_, xk_stride, error_, stream_));
        ++dispatches_;
    }
    check(tsp_dense_mm(&set, dense_staging_, xk_stride, input.rows, static_cast<float*>(device_pointer(output.view, true)), output.stride_bytes,
                       counters + dense_counter_++, error_, stream_));
    ++dispatches_;
}

// ---- batched routing, mixture, router projection with the margin audit -----------------------------------------------------
void CudaGraph::prefill_route_batch(GpuView logits, GpuView indices, GpuView weights, uint32_t experts, uint32_t selected, uint32_t tokens,
                                    RouterMode mode, bool normalize_selected) {
    require_batch();
    if (!tokens || logits.bytes != uint64_t(tokens) * experts * 4 || indices.bytes != uint64_t(tokens) * selected * 4 || weights.bytes != indices.bytes)
        throw FormatError("invalid router shape/mode");
    check(tsp_moe_route(static_cast<const float*>(device_pointer(logits)), uint64_t(experts) * 4, tokens, experts, selected, uint32_t(mode), normalize_selected,
                        static_cast<uint32_t*>(device_pointer(indices, true)), static_cast<float*>(device_pointer(weights, true)), error_, stream_));
    ++dispatches_;
}

void CudaGraph::prefill_mixture_batch(GpuView experts, GpuView weights, GpuView shared, GpuView shared_logit, GpuRowsF32 output, uint32_t selected) {
    require_batch();
    const uint32_t tokens = output.rows, channels = output.columns;
    if (!tokens || !selected || experts.bytes != uint64_t(tokens) * selected * channels * 4 || weights.bytes != uint64_t(tokens) * selected * 4 ||
        shared.bytes != uint64_t(tokens) * channels * 4 || shared_logit.bytes != uint64_t(tokens) * 4 ||
        output.view.bytes < uint64_t(tokens - 1) * output.stride_bytes + uint64_t(channels) * 4)
        throw FormatError("mixture shape mismatch");
    check(tsp_moe_combine(device_pointer(experts), uint64_t(channels) * 4, 0, static_cast<const float*>(device_pointer(weights)),
                          static_cast<const float*>(device_pointer(shared)), uint64_t(channels) * 4, nullptr, nullptr, 0, 0,
                          static_cast<float*>(device_pointer(shared_logit)), tokens, channels, selected, static_cast<float*>(device_pointer(output.view, true)),
                          output.stride_bytes, nullptr, 0, error_, stream_));
    ++dispatches_;
}

void CudaGraph::mixture(GpuView expert_outputs, GpuView weights, GpuView shared_output, GpuView shared_logit, GpuView output) {
    const uint32_t channels = static_cast<uint32_t>(output.bytes / 4), selected = static_cast<uint32_t>(weights.bytes / 4);
    if (output.bytes % 4 || !channels) throw FormatError("mixture shape mismatch");
    prefill_mixture_batch(expert_outputs, weights, shared_output, shared_logit, {output, 1, channels, uint64_t(channels) * 4}, selected);
}

void CudaGraph::moe_router_rows(GpuView router, GpuView shared_router, GpuRowsF32 input, GpuView logits, GpuView shared_logits, uint32_t experts) {
    require_batch();
    const uint32_t tokens = input.rows, columns = input.columns;
    if (!tokens || router.bytes != uint64_t(experts) * columns * 4 || shared_router.bytes != uint64_t(columns) * 4 ||
        logits.bytes != uint64_t(tokens) * experts * 4 || shared_logits.bytes != uint64_t(tokens) * 4 ||
        input.view.bytes < uint64_t(tokens - 1) * input.stride_bytes + uint64_t(columns) * 4)
        throw FormatError("router projection shape mismatch");
    check(tsp_router_project(static_cast<const float*>(device_pointer(router)), experts, columns, static_cast<const float*>(device_pointer(shared_router)),
                             static_cast<const float*>(device_pointer(input.view)), input.stride_bytes, tokens, static_cast<float*>(device_pointer(logits, true)),
                             uint64_t(experts) * 4, static_cast<float*>(device_pointer(shared_logits, true)), error_, stream_));
    ++dispatches_;
}

void CudaGraph::configure_router_margin_epsilon(float epsilon) {
    require_idle();
    if (!(epsilon > 0) || epsilon > 1e30f) throw FormatError("router margin epsilon must be positive finite");
    margin_epsilon_ = epsilon;
}

void CudaGraph::moe_route_rows(GpuView logits, GpuView indices, GpuView weights, uint32_t experts, uint32_t selected, uint32_t tokens, RouterMode mode,
                               bool normalize_selected) {
    if (!margin_audit_) { prefill_route_batch(logits, indices, weights, experts, selected, tokens, mode, normalize_selected); return; }
    require_batch();
    if (!tokens || tokens > 2048 || logits.bytes != uint64_t(tokens) * experts * 4 || indices.bytes != uint64_t(tokens) * selected * 4 || weights.bytes != indices.bytes)
        throw FormatError("router row top-k geometry/mode mismatch");
    if (!margins_) throw FormatError("router margin audit: enable it and call prepare_router_margin_scratch() between batches first");
    check(tsp_moe_route_audit(static_cast<const float*>(device_pointer(logits)), uint64_t(experts) * 4, tokens, experts, selected, uint32_t(mode), normalize_selected,
                              static_cast<uint32_t*>(device_pointer(indices, true)), static_cast<float*>(device_pointer(weights, true)), margins_, error_, stream_));
    ++dispatches_;
}

void CudaGraph::prepare_router_margin_scratch() {
    require_idle();
    select_device();
    if (!margins_) cuda(cudaMalloc(reinterpret_cast<void**>(&margins_), 2048 * sizeof(float)), "router margin scratch");
}

bool CudaGraph::evaluate_router_margin(uint32_t tokens) {
    if (!margins_ || !tokens) return false;
    select_device();
    int fallback = 0;
    check(tsp_router_margin_evaluate(margins_, tokens, margin_epsilon_, stream_, &margin_telemetry_, &fallback));
    return fallback != 0;
}

void CudaGraph::logit_topk(GpuRowsF32 logits, GpuView partial_scratch, GpuView out_rows) {
    require_batch();
    if (!logits.rows || logits.rows > 2048 || !logits.columns || logits.columns > (1u << 20) || logits.stride_bytes < uint64_t(logits.columns) * 4 ||
        logits.stride_bytes % 4)
        throw FormatError("GPU logit top-k geometry mismatch");
    if (logits.view.bytes < uint64_t(logits.rows - 1) * logits.stride_bytes + uint64_t(logits.columns) * 4 ||
        partial_scratch.bytes < tsp_logit_topk_scratch_bytes(logits.rows, logits.columns) || out_rows.bytes < tsp_logit_topk_output_bytes(logits.rows))
        throw FormatError("GPU logit top-k buffer span or alignment mismatch");
    check(tsp_logit_topk(static_cast<const float*>(device_pointer(logits.view)), logits.stride_bytes, logits.rows, logits.columns,
                         device_pointer(partial_scratch, true), partial_scratch.bytes, device_pointer(out_rows, true), out_rows.bytes, stream_));
    dispatches_ += 2;
}

// ---- residual read / write ---------------------------------------------------------------------------------------------------
void CudaGraph::residual_read(GpuView normalized, GpuView scores, GpuView inject_logits, GpuView output, GpuView scales, uint32_t branches, uint32_t channels) {
    require_batch();
    const uint64_t wide = uint64_t(branches) * channels * 4;
    if (!branches || !channels || normalized.bytes != wide || scores.bytes != wide || inject_logits.bytes != uint64_t(branches) * 4 ||
        output.bytes != uint64_t(channels) * 4 || scales.bytes != uint64_t(branches) * 4) throw FormatError("residual read shape mismatch");
    check(tsp_residual_read(static_cast<const float*>(device_pointer(normalized)), static_cast<const float*>(device_pointer(scores)),
                            static_cast<const float*>(device_pointer(inject_logits)), branches, channels, 1, static_cast<float*>(device_pointer(output, true)),
                            static_cast<float*>(device_pointer(scales, true)), error_, stream_));
    ++dispatches_;
}

void CudaGraph::residual_write(GpuView streams, GpuView output, GpuView scales, GpuView destination) {
    require_batch();
    const uint64_t channels = output.bytes / 4, branches = scales.bytes / 4;
    if (!channels || !branches || output.bytes % 4 || scales.bytes % 4 || streams.bytes != branches * channels * 4 || destination.bytes != streams.bytes)
        throw FormatError("residual write shape mismatch");
    check(tsp_residual_write(static_cast<const float*>(device_pointer(streams)), static_cast<const float*>(device_pointer(output)),
                             static_cast<const float*>(device_pointer(scales)), uint32_t(branches), uint32_t(channels), 1,
                             static_cast<float*>(device_pointer(destination, true)), error_, stream_));
    ++dispatches_;
}

}  // namespace tokspur_b200
