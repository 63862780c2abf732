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

}  // namespace tokspur_b200
