// C ABI of the MoE hot path: argument validation (refused before any launch, as the reference's
// FormatError checks are), then the launches. No entry point allocates, frees or reads results back
// except tsp_error_word_read, which is the once-per-batch readback of the sticky error word.
#include <atomic>
#include <cstdarg>
#include <cstdio>

#include "tsp_common.cuh"

namespace tsp {

static thread_local char g_message[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_message, sizeof g_message, fmt, ap);
    va_end(ap);
    return code;
}

int cuda_fail(cudaError_t e, const char* what) {
    snprintf(g_message, sizeof g_message, "CUDA error %d (%s) at %s", static_cast<int>(e), cudaGetErrorString(e), what);
    return TSP_E_CUDA;
}

int sm_count() {
    static thread_local int cached_device = -1, cached = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (dev != cached_device) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
        cached = n;
        cached_device = dev;
    }
    return cached;
}

// launchers implemented in the kernel files
int launch_route(const float*, uint64_t, uint32_t, uint32_t, uint32_t, uint32_t, int, uint32_t*, float*, uint32_t*, cudaStream_t, float* = nullptr);
int launch_permute(const uint32_t*, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, int, uint32_t*, uint32_t*, uint32_t*, uint32_t*, cudaStream_t);
int launch_combine(const void*, uint64_t, uint32_t, const float*, const float*, uint64_t, const float*, const void*, uint64_t, uint32_t, float*,
                   uint32_t, uint32_t, uint32_t, float*, uint64_t, void*, uint64_t, uint32_t*, cudaStream_t);
int launch_decode_prologue(const float*, uint64_t, uint32_t, uint32_t, uint32_t, uint32_t, int, uint32_t, uint32_t*, float*, uint32_t*, uint32_t*,
                           uint32_t*, const void*, uint64_t, float*, uint64_t, uint32_t, uint32_t*, cudaStream_t);
int launch_f16_to_f32(const void*, uint64_t, float*, uint64_t, uint32_t, uint32_t, cudaStream_t);
int launch_dequant(uint32_t, uint32_t, const uint8_t*, uint64_t, float*, uint32_t*, cudaStream_t);
int launch_gemv(const tsp_matrix_set*, const tsp_matrix_set*, bool, const float*, uint64_t, uint32_t, uint32_t,
                const uint32_t*, const uint32_t*, const uint32_t*, float*, uint64_t, int, int, uint32_t*, cudaStream_t, const GemvShared* = nullptr);

int launch_route_offsets(const uint32_t*, uint32_t, uint32_t*, cudaStream_t);
int launch_bounded_wait_selftest(uint32_t, uint32_t*, cudaStream_t);
int launch_q8_lanes(const void*, void*, uint64_t, uint32_t, bool, cudaStream_t);
int launch_logit_topk(const float*, uint64_t, uint32_t, uint32_t, uint32_t*, uint32_t*, cudaStream_t);
int launch_rows_f16k(const void*, uint64_t, uint32_t, uint32_t, uint32_t, void*, uint64_t, uint32_t*, cudaStream_t);
int launch_grouped(const tsp_matrix_set*, const tsp_matrix_set*, bool, const void*, uint64_t, uint32_t, uint32_t, uint32_t, const uint32_t*,
                   const uint32_t*, const uint32_t*, const uint32_t*, uint32_t*, void*, uint64_t, uint32_t, uint32_t*, cudaStream_t, const GroupedShared* = nullptr);
int launch_gather_rows16(const void*, uint64_t, const uint32_t*, const uint32_t*, uint32_t, uint32_t, uint32_t, uint32_t, void*, uint64_t, cudaStream_t);
int launch_staged_f16(const uint8_t*, uint32_t, uint32_t, void*, cudaStream_t);
int launch_residual_read(const float*, const float*, const float*, uint32_t, uint32_t, uint32_t, float*, float*, uint32_t*, cudaStream_t);
int launch_residual_write(const float*, const float*, const float*, uint32_t, uint32_t, uint32_t, float*, uint32_t*, cudaStream_t);
int launch_gemv_f32(const float*, uint32_t, uint32_t, const float*, const float*, uint64_t, uint32_t, float*, uint64_t, float*, uint32_t*, cudaStream_t);
int launch_synth(uint32_t, uint64_t, uint64_t, uint64_t, float, void*, cudaStream_t);
int launch_dequant_k5(uint32_t, const uint8_t*, uint64_t, float*, uint32_t*, cudaStream_t);
int launch_pack_planar(uint32_t, const void*, uint64_t, void*, uint64_t, uint64_t, uint32_t, cudaStream_t);

static int check_matrix(const tsp_matrix_set* m, const char* name) {
    TSP_REQUIRE(m != nullptr, "%s: null matrix set", name);
    const bool five = m->type == TSP_TYPE_Q5_K || m->type == TSP_TYPE_Q5_1;
    if (m->type != TSP_TYPE_Q4_K && m->type != TSP_TYPE_Q8_0 && !five) return fail(TSP_E_TYPE, "%s: encoding %u has no kernel", name, m->type);
    if (m->layout != TSP_LAYOUT_GGUF && m->layout != TSP_LAYOUT_PLANAR) return fail(TSP_E_TYPE, "%s: unknown layout %u", name, m->layout);
    if (five && m->layout != TSP_LAYOUT_GGUF) return fail(TSP_E_TYPE, "%s: the five-bit encodings are read as plain GGUF rows only", name);
    TSP_REQUIRE(m->base && aligned16(m->base), "%s: base must be a 16-byte aligned device pointer", name);
    TSP_REQUIRE(m->experts >= 1 && m->experts <= 4096, "%s: experts out of range", name);
    TSP_REQUIRE(m->rows >= 8 && m->rows % 8 == 0 && m->rows <= 1u << 20, "%s: rows must be a multiple of 8", name);
    const uint32_t block = (m->type == TSP_TYPE_Q4_K || m->type == TSP_TYPE_Q5_K) ? 256u : 32u;
    TSP_REQUIRE(m->cols >= block && m->cols % block == 0 && m->cols <= 65536, "%s: columns must be a multiple of %u", name, block);
    const uint64_t bytes = tsp_expert_bytes(m->type, m->layout, m->rows, m->cols);
    TSP_REQUIRE(bytes != 0, "%s: shape not representable in this layout", name);
    if (m->experts > 1 || m->split < m->experts) {
        TSP_REQUIRE(m->expert_stride >= bytes && m->expert_stride % 16 == 0, "%s: expert stride too small or unaligned", name);
    }
    if (m->split < m->experts) TSP_REQUIRE(m->base_hi && aligned16(m->base_hi), "%s: base_hi must be a 16-byte aligned device pointer", name);
    return TSP_OK;
}

static int check_rows(const void* p, uint64_t stride, uint32_t cols, uint32_t elem, const char* name) {
    TSP_REQUIRE(p && aligned16(p), "%s: rows must be 16-byte aligned", name);
    TSP_REQUIRE(stride >= static_cast<uint64_t>(cols) * elem && stride % 16 == 0, "%s: row stride must cover the row and be a multiple of 16", name);
    return TSP_OK;
}

static bool overlap(const void* a, uint64_t abytes, const void* b, uint64_t bbytes) {
    const uintptr_t x = reinterpret_cast<uintptr_t>(a), y = reinterpret_cast<uintptr_t>(b);
    return x < y + bbytes && y < x + abytes;
}

}  // namespace tsp

using namespace tsp;

extern "C" {

const char* tsp_last_error(void) { return g_message; }

int tsp_device_info(int* sms, int* major, int* minor) {
    int dev = 0;
    TSP_CUDA(cudaGetDevice(&dev));
    int n = 0, ma = 0, mi = 0;
    TSP_CUDA(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
    TSP_CUDA(cudaDeviceGetAttribute(&ma, cudaDevAttrComputeCapabilityMajor, dev));
    TSP_CUDA(cudaDeviceGetAttribute(&mi, cudaDevAttrComputeCapabilityMinor, dev));
    if (sms) *sms = n;
    if (major) *major = ma;
    if (minor) *minor = mi;
    return TSP_OK;
}

int tsp_error_word_read(const uint32_t* d_error, void* stream, uint32_t* host_word) {
    TSP_REQUIRE(d_error && host_word, "error word pointers must not be null");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    TSP_CUDA(cudaMemcpyAsync(host_word, d_error, sizeof(uint32_t), cudaMemcpyDeviceToHost, st));
    TSP_CUDA(cudaStreamSynchronize(st));
    if (*host_word) return fail(TSP_E_DEVICE, "device error word 0x%x:%s%s%s", *host_word,
                                (*host_word & TSP_ERR_NONFINITE) ? " non-finite value" : "",
                                (*host_word & TSP_ERR_INDEX) ? " bad index/geometry" : "",
                                (*host_word & TSP_ERR_TIMEOUT) ? " bounded wait expired" : "");
    return TSP_OK;
}

int tsp_error_word_reset(uint32_t* d_error, void* stream) {
    TSP_REQUIRE(d_error, "error word pointer must not be null");
    TSP_CUDA(cudaMemsetAsync(d_error, 0, sizeof(uint32_t), static_cast<cudaStream_t>(stream)));
    return TSP_OK;
}

uint64_t tsp_expert_bytes(uint32_t type, uint32_t layout, uint32_t rows, uint32_t cols) {
    if (!rows || !cols) return 0;
    if (type == TSP_TYPE_Q4_K) {
        if (cols % 256) return 0;
        if (layout == TSP_LAYOUT_PLANAR && rows % 4) return 0;
        return static_cast<uint64_t>(rows) * (cols / 256) * (layout == TSP_LAYOUT_PLANAR ? 148u : 144u);
    }
    if (type == TSP_TYPE_Q8_0) {
        if (cols % 32) return 0;
        const uint64_t blocks = static_cast<uint64_t>(rows) * (cols / 32);
        if (layout == TSP_LAYOUT_PLANAR && (rows % 4 || blocks % 8)) return 0;
        return blocks * 34u;
    }
    if (layout != TSP_LAYOUT_GGUF) return 0;
    if (type == TSP_TYPE_Q5_K) return cols % 256 ? 0 : static_cast<uint64_t>(rows) * (cols / 256) * 176u;
    if (type == TSP_TYPE_Q5_1) return cols % 32 ? 0 : static_cast<uint64_t>(rows) * (cols / 32) * 24u;
    return 0;
}

int tsp_dequant_f32(const tsp_matrix_set* m, uint32_t expert, float* d_out, uint32_t* d_error, void* stream) {
    if (int rc = check_matrix(m, "dequant")) return rc;
    TSP_REQUIRE(expert < m->experts, "dequant: expert %u out of range", expert);
    TSP_REQUIRE(d_out, "dequant: null output");
    const uint8_t* base = static_cast<const uint8_t*>(expert < m->split ? m->base : m->base_hi);
    const uint32_t local = expert < m->split ? expert : expert - m->split;
    if (m->type == TSP_TYPE_Q5_K || m->type == TSP_TYPE_Q5_1)
        return launch_dequant_k5(m->type, base + local * m->expert_stride, static_cast<uint64_t>(m->rows) * m->cols, d_out, d_error,
                                 static_cast<cudaStream_t>(stream));
    const uint64_t blocks = static_cast<uint64_t>(m->rows) * (m->cols / (m->type == TSP_TYPE_Q4_K ? 256 : 32));
    TSP_REQUIRE(blocks < (1ull << 31), "dequant: matrix too large");
    return launch_dequant(m->type, m->layout, base + local * m->expert_stride, blocks, d_out, d_error, static_cast<cudaStream_t>(stream));
}

int tsp_moe_route(const float* d_logits, uint64_t stride, uint32_t tokens, uint32_t experts, uint32_t selected,
                  uint32_t mode, int normalize, uint32_t* d_ids, float* d_weights, uint32_t* d_error, void* stream) {
    TSP_REQUIRE(d_logits && d_ids && d_weights, "route: null buffer");
    TSP_REQUIRE(tokens >= 1, "route: no token rows");
    TSP_REQUIRE(experts >= 1 && experts <= 4096 && selected >= 1 && selected <= 64 && selected <= experts && mode <= 1,
                "route: invalid router shape/mode");
    TSP_REQUIRE(stride >= static_cast<uint64_t>(experts) * 4 && stride % 4 == 0, "route: logits stride too small");
    return launch_route(d_logits, stride, tokens, experts, selected, mode, normalize, d_ids, d_weights, d_error,
                        static_cast<cudaStream_t>(stream));
}

int tsp_moe_route_audit(const float* d_logits, uint64_t stride, uint32_t tokens, uint32_t experts, uint32_t selected, uint32_t mode,
                        int normalize, uint32_t* d_ids, float* d_weights, float* d_margins, uint32_t* d_error, void* stream) {
    TSP_REQUIRE(d_logits && d_ids && d_weights && d_margins, "route: null buffer");
    TSP_REQUIRE(tokens >= 1, "route: no token rows");
    TSP_REQUIRE(experts >= 1 && experts <= 4096 && selected >= 1 && selected <= 64 && selected <= experts && mode <= 1,
                "route: invalid router shape/mode");
    TSP_REQUIRE(stride >= static_cast<uint64_t>(experts) * 4 && stride % 4 == 0, "route: logits stride too small");
    return launch_route(d_logits, stride, tokens, experts, selected, mode, normalize, d_ids, d_weights, d_error,
                        static_cast<cudaStream_t>(stream), d_margins);
}

int tsp_router_margin_evaluate(const float* d_margins, uint32_t tokens, float epsilon, void* stream, tsp_router_margin_telemetry* t, int* fallback) {
    TSP_REQUIRE(d_margins && t && tokens >= 1 && tokens <= (1u << 20), "margin audit: null buffer or row count out of range");
    TSP_REQUIRE(epsilon > 0.f && epsilon < 1e30f, "margin audit: epsilon must be positive and finite");
    static thread_local float host[4096];
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    float min_m = t->total_tokens ? t->min_margin : INFINITY;
    double sum = 0;
    uint64_t violations = 0;
    const float threshold = 2.f * epsilon;
    for (uint32_t at = 0; at < tokens; at += 4096) {
        const uint32_t n = tokens - at < 4096 ? tokens - at : 4096;
        TSP_CUDA(cudaMemcpyAsync(host, d_margins + at, n * sizeof(float), cudaMemcpyDeviceToHost, st));
        TSP_CUDA(cudaStreamSynchronize(st));
        for (uint32_t i = 0; i < n; ++i) {
            const float m = host[i];
            if (m < min_m) min_m = m;
            sum += m;
            if (!(m > threshold)) ++violations;
        }
    }
    t->min_margin = min_m;
    t->sum_margin += sum;
    t->total_tokens += tokens;
    t->violation_count += violations;
    t->total_layers += 1;
    if (violations) t->fallback_layers += 1;
    if (fallback) *fallback = violations != 0;
    return TSP_OK;
}

uint64_t tsp_moe_tasks_words(uint32_t tokens, uint32_t experts, uint32_t selected, uint32_t tile) {
    if (!tile) return 0;
    return 2 + 2 * ((static_cast<uint64_t>(tokens) * selected) / tile + experts);
}

int tsp_moe_permute(const uint32_t* d_ids, uint32_t tokens, uint32_t experts, uint32_t selected, uint32_t tile,
                    uint32_t* d_token_map, uint32_t* d_counts, uint32_t* d_tasks, uint32_t* d_error, void* stream) {
    TSP_REQUIRE(d_ids && d_token_map && d_counts && d_tasks, "permute: null buffer");
    TSP_REQUIRE(tokens >= 1 && experts >= 1 && experts <= 4096 && selected >= 1 && selected <= 64 && selected <= experts,
                "permute: invalid shape");
    TSP_REQUIRE(tile >= 1 && tile <= 1024, "permute: tile out of range");
    TSP_REQUIRE(static_cast<uint64_t>(tokens) * selected < (1ull << 31), "permute: too many routes");
    return launch_permute(d_ids, tokens, experts, selected, tile, 0, 0, d_token_map, d_counts, d_tasks, d_error,
                          static_cast<cudaStream_t>(stream));
}

int tsp_moe_permute_local(const uint32_t* d_ids, uint32_t tokens, uint32_t first_expert, uint32_t local_experts, uint32_t selected,
                          uint32_t tile, uint32_t* d_token_map, uint32_t* d_counts, uint32_t* d_tasks, uint32_t* d_error, void* stream) {
    TSP_REQUIRE(d_ids && d_token_map && d_counts && d_tasks, "permute: null buffer");
    TSP_REQUIRE(tokens >= 1 && local_experts >= 1 && local_experts <= 4096 && selected >= 1 && selected <= 64, "permute: invalid shape");
    TSP_REQUIRE(tile >= 1 && tile <= 1024, "permute: tile out of range");
    TSP_REQUIRE(static_cast<uint64_t>(tokens) * selected < (1ull << 31), "permute: too many routes");
    return launch_permute(d_ids, tokens, local_experts, selected, tile, first_expert, 1, d_token_map, d_counts, d_tasks, d_error,
                          static_cast<cudaStream_t>(stream));
}

int tsp_moe_gate_up_swiglu(const tsp_matrix_set* gate, const tsp_matrix_set* up, const float* d_x, uint64_t x_stride,
                           uint32_t tokens, uint32_t selected, const uint32_t* d_token_map, const uint32_t* d_counts,
                           const uint32_t* d_tasks, float* d_h, uint64_t h_stride, int f16_exact, uint32_t* d_error, void* stream) {
    if (int rc = check_matrix(gate, "gate")) return rc;
    if (int rc = check_matrix(up, "up")) return rc;
    TSP_REQUIRE(gate->type == up->type && gate->layout == up->layout && gate->rows == up->rows && gate->cols == up->cols &&
                gate->experts == up->experts && gate->expert_stride == up->expert_stride && gate->split == up->split,
                "gate/up matrix sets must share shape, encoding, layout and addressing");
    TSP_REQUIRE(tokens >= 1, "gate-up: no token rows");
    if (int rc = check_rows(d_x, x_stride, gate->cols, 4, "gate-up input")) return rc;
    if (int rc = check_rows(d_h, h_stride, gate->rows, 4, "gate-up output")) return rc;
    const bool routed = d_token_map != nullptr;
    TSP_REQUIRE(routed == (d_counts != nullptr) && routed == (d_tasks != nullptr), "gate-up: token map, counts and tasks go together");
    TSP_REQUIRE(routed || gate->experts == 1, "gate-up: an expert set needs the route tables");
    if (routed) TSP_REQUIRE(selected >= 1 && selected <= 64, "gate-up: selected out of range");
    const uint64_t out_rows = routed ? static_cast<uint64_t>(tokens) * selected : tokens;
    TSP_REQUIRE(!overlap(d_x, tokens * x_stride, d_h, out_rows * h_stride), "gate-up: input and output overlap");
    const int nc = (!routed && tokens > 8) ? 2 : 1;
    return launch_gemv(gate, up, true, d_x, x_stride, routed ? selected : 1, tokens, d_token_map, d_counts, d_tasks, d_h, h_stride,
                       f16_exact, nc, d_error, static_cast<cudaStream_t>(stream));
}

int tsp_moe_project(const tsp_matrix_set* w, const float* d_in, uint64_t in_stride, uint32_t in_div, uint32_t tokens,
                    uint32_t selected, const uint32_t* d_token_map, const uint32_t* d_counts, const uint32_t* d_tasks,
                    float* d_out, uint64_t out_stride, int f16_exact, uint32_t* d_error, void* stream) {
    if (int rc = check_matrix(w, "project")) return rc;
    TSP_REQUIRE(tokens >= 1, "project: no token rows");
    TSP_REQUIRE(w->rows % 16 == 0, "project: rows must be a multiple of 16");
    if (int rc = check_rows(d_in, in_stride, w->cols, 4, "project input")) return rc;
    if (int rc = check_rows(d_out, out_stride, w->rows, 4, "project output")) return rc;
    const bool routed = d_token_map != nullptr;
    TSP_REQUIRE(routed == (d_counts != nullptr) && routed == (d_tasks != nullptr), "project: token map, counts and tasks go together");
    TSP_REQUIRE(routed || w->experts == 1, "project: an expert set needs the route tables");
    if (routed) TSP_REQUIRE(selected >= 1 && selected <= 64 && (in_div == 1 || in_div == selected), "project: selected / in_div out of range");
    const uint64_t out_rows = routed ? static_cast<uint64_t>(tokens) * selected : tokens;
    const uint64_t in_rows = routed ? out_rows / (in_div ? in_div : 1) : tokens;
    TSP_REQUIRE(!overlap(d_in, in_rows * in_stride, d_out, out_rows * out_stride), "project: input and output overlap");
    const int nc = (!routed && tokens > 8) ? 2 : 1;
    return launch_gemv(w, nullptr, false, d_in, in_stride, routed ? (in_div ? in_div : 1) : 1, tokens, d_token_map, d_counts, d_tasks,
                       d_out, out_stride, f16_exact, nc, d_error, static_cast<cudaStream_t>(stream));
}

int tsp_moe_combine(const void* d_routed, uint64_t routed_stride, uint32_t routed_dtype, const float* d_weights, const float* d_shared,
                    uint64_t shared_stride, const float* d_shared_router, const void* d_x, uint64_t x_stride, uint32_t x_dtype,
                    float* d_shared_logit, uint32_t tokens, uint32_t channels, uint32_t selected, float* d_out,
                    uint64_t out_stride, void* d_out_f16, uint64_t out_f16_stride, uint32_t* d_error, void* stream) {
    TSP_REQUIRE(d_routed && d_weights && (d_out || d_out_f16), "combine: null buffer");
    TSP_REQUIRE(tokens >= 1 && channels >= 1 && channels <= 65536 && selected >= 1 && selected <= 64, "combine: mixture shape mismatch");
    TSP_REQUIRE(routed_dtype <= 1 && x_dtype <= 1, "combine: row dtype must be 0 (FP32) or 1 (binary16)");
    const uint64_t relem = routed_dtype ? 2 : 4, xelem = x_dtype ? 2 : 4;
    TSP_REQUIRE(routed_stride >= channels * relem && routed_stride % relem == 0, "combine: row stride too small");
    if (d_shared) TSP_REQUIRE(shared_stride >= channels * 4ull && shared_stride % 4 == 0, "combine: shared row stride too small");
    if (d_out) TSP_REQUIRE(out_stride >= channels * 4ull && out_stride % 4 == 0, "combine: output row stride too small");
    if (d_shared_router) TSP_REQUIRE(d_x && x_stride >= channels * xelem && x_stride % xelem == 0, "combine: the shared router needs the input rows");
    if (d_out_f16) TSP_REQUIRE(out_f16_stride >= channels * 2ull && out_f16_stride % 2 == 0, "combine: binary16 output stride too small");
    if (d_out) TSP_REQUIRE(!overlap(d_out, tokens * out_stride, d_routed, static_cast<uint64_t>(tokens) * selected * routed_stride) &&
                           (!d_shared || !overlap(d_out, tokens * out_stride, d_shared, tokens * shared_stride)), "combine: output overlaps an input");
    return launch_combine(d_routed, routed_stride, routed_dtype, d_weights, d_shared, shared_stride, d_shared_router, d_x, x_stride, x_dtype,
                          d_shared_logit, tokens, channels, selected, d_out, out_stride, d_out_f16, out_f16_stride, d_error,
                          static_cast<cudaStream_t>(stream));
}

int tsp_residual_read(const float* d_normalized, const float* d_scores, const float* d_inject_logits, uint32_t branches, uint32_t channels,
                      uint32_t tokens, float* d_output, float* d_scales, uint32_t* d_error, void* stream) {
    TSP_REQUIRE(d_normalized && d_scores && d_inject_logits && d_output && d_scales, "residual read: null buffer");
    TSP_REQUIRE(branches >= 1 && branches <= 64 && channels >= 1 && channels <= 65536 && tokens >= 1 && tokens <= 65535, "residual read shape mismatch");
    const uint64_t wide = static_cast<uint64_t>(tokens) * branches * channels * 4, narrow = static_cast<uint64_t>(tokens) * channels * 4;
    TSP_REQUIRE(!overlap(d_output, narrow, d_normalized, wide) && !overlap(d_output, narrow, d_scores, wide), "residual read: output overlaps an input");
    return launch_residual_read(d_normalized, d_scores, d_inject_logits, branches, channels, tokens, d_output, d_scales, d_error,
                                static_cast<cudaStream_t>(stream));
}

int tsp_residual_write(const float* d_streams, const float* d_output, const float* d_scales, uint32_t branches, uint32_t channels, uint32_t tokens,
                       float* d_destination, uint32_t* d_error, void* stream) {
    TSP_REQUIRE(d_streams && d_output && d_scales && d_destination, "residual write: null buffer");
    TSP_REQUIRE(branches >= 1 && branches <= 64 && channels >= 1 && channels <= 65536 && tokens >= 1 && tokens <= 65535, "residual write shape mismatch");
    const uint64_t wide = static_cast<uint64_t>(tokens) * branches * channels * 4, narrow = static_cast<uint64_t>(tokens) * channels * 4;
    // in place over the streams is allowed (each element is read once, then written); the FFN output must not be clobbered
    TSP_REQUIRE(!overlap(d_destination, wide, d_output, narrow), "residual write: destination overlaps the FFN output");
    return launch_residual_write(d_streams, d_output, d_scales, branches, channels, tokens, d_destination, d_error, static_cast<cudaStream_t>(stream));
}

int tsp_synth_weights(uint32_t type, uint64_t seed, uint64_t first_block, uint64_t blocks, float sigma, void* d_out, void* stream) {
    if (type != TSP_TYPE_Q4_K && type != TSP_TYPE_Q8_0 && type != TSP_TYPE_F32 && type != TSP_TYPE_Q5_K && type != TSP_TYPE_Q5_1)
        return fail(TSP_E_TYPE, "synth: encoding %u has no generator", type);
    TSP_REQUIRE(d_out && blocks >= 1 && blocks < (1ull << 38), "synth: null output or block count out of range");
    TSP_REQUIRE(sigma > 0.f && sigma < 1e4f, "synth: sigma out of range");
    return launch_synth(type, seed, first_block, blocks, sigma, d_out, static_cast<cudaStream_t>(stream));
}

int tsp_pack_planar(uint32_t type, uint32_t rows, uint32_t cols, uint32_t experts, const void* d_gguf, uint64_t gguf_stride,
                    void* d_planar, uint64_t planar_stride, void* stream) {
    const uint64_t pb = tsp_expert_bytes(type, TSP_LAYOUT_PLANAR, rows, cols), gb = tsp_expert_bytes(type, TSP_LAYOUT_GGUF, rows, cols);
    if (!pb || !gb) return fail(TSP_E_TYPE, "pack: shape %ux%u of encoding %u has no planar layout", rows, cols, type);
    TSP_REQUIRE(d_gguf && d_planar && aligned16(d_gguf) && aligned16(d_planar), "pack: buffers must be 16-byte aligned");
    TSP_REQUIRE(experts >= 1 && gguf_stride >= gb && planar_stride >= pb && planar_stride % 16 == 0 && gguf_stride % 16 == 0,
                "pack: expert strides too small or unaligned");
    const uint64_t blocks = static_cast<uint64_t>(rows) * (cols / (type == TSP_TYPE_Q4_K ? 256 : 32));
    return launch_pack_planar(type, d_gguf, gguf_stride, d_planar, planar_stride, blocks, experts, static_cast<cudaStream_t>(stream));
}

int tsp_gemv_f32(const float* d_w, uint32_t rows, uint32_t cols, const float* d_x, uint64_t x_stride, uint32_t tokens, float* d_out,
                 uint64_t out_stride, uint32_t* d_error, void* stream) {
    return tsp_router_project(d_w, rows, cols, nullptr, d_x, x_stride, tokens, d_out, out_stride, nullptr, d_error, stream);
}

int tsp_router_project(const float* d_w, uint32_t rows, uint32_t cols, const float* d_extra_row, const float* d_x, uint64_t x_stride,
                       uint32_t tokens, float* d_out, uint64_t out_stride, float* d_extra_out, uint32_t* d_error, void* stream) {
    TSP_REQUIRE(d_w && d_x && d_out, "gemv: null buffer");
    TSP_REQUIRE((d_extra_row != nullptr) == (d_extra_out != nullptr), "gemv: the extra row and its output go together");
    TSP_REQUIRE(rows >= 1 && cols >= 1 && tokens >= 1 && static_cast<uint64_t>(rows) * tokens < (1ull << 28), "GEMV shape mismatch");
    TSP_REQUIRE(x_stride >= cols * 4ull && x_stride % 4 == 0 && out_stride >= rows * 4ull && out_stride % 4 == 0, "gemv: row stride too small");
    return launch_gemv_f32(d_w, rows, cols, d_extra_row, d_x, x_stride, tokens, d_out, out_stride, d_extra_out, d_error,
                           static_cast<cudaStream_t>(stream));
}

int tsp_rows_f16_to_f32(const void* d_in, uint64_t in_stride, float* d_out, uint64_t out_stride, uint32_t rows,
                        uint32_t cols, void* stream) {
    TSP_REQUIRE(d_in && d_out && rows >= 1 && cols >= 1, "convert: null buffer or empty shape");
    TSP_REQUIRE(in_stride >= cols * 2ull && in_stride % 2 == 0 && out_stride >= cols * 4ull && out_stride % 4 == 0, "convert: row stride too small");
    TSP_REQUIRE(rows <= 65535, "convert: too many rows");
    return launch_f16_to_f32(d_in, in_stride, d_out, out_stride, rows, cols, static_cast<cudaStream_t>(stream));
}

// Routed experts and the layer's dense shared expert in one launch when the shared expert looks like a routed one (same
// shape, encoding and layout, Q4_K); otherwise the shared expert gets a launch of its own.
int tsp_moe_gate_up_swiglu_shared_rows(const tsp_matrix_set* gate, const tsp_matrix_set* up, const tsp_matrix_set* shared_gate,
                                       const tsp_matrix_set* shared_up, const float* d_x, uint64_t x_stride, const void* d_x16,
                                       uint64_t x16_stride, uint32_t tokens, uint32_t selected, const uint32_t* d_token_map,
                                       const uint32_t* d_counts, const uint32_t* d_tasks, float* d_h, uint64_t h_stride,
                                       const float* d_shared_x, uint64_t shared_x_stride, uint32_t shared_tokens, float* d_shared_h,
                                       uint64_t shared_h_stride, int x_is_f16_exact, uint32_t* d_error, void* stream) {
    TSP_REQUIRE(gate && up && shared_gate && shared_up && d_token_map && d_counts && d_tasks && d_shared_h && d_shared_x && shared_tokens >= 1,
                "gate-up with shared expert: null argument");
    TSP_REQUIRE(!d_x16 || (d_shared_x == d_x && shared_tokens == tokens), "gate-up with shared expert: binary16 rows serve both row sets only when they are the same rows");
    const bool same_shape = shared_gate->type == gate->type && shared_gate->layout == gate->layout && shared_up->type == gate->type &&
                            shared_up->layout == gate->layout && shared_gate->rows == gate->rows && shared_gate->cols == gate->cols &&
                            shared_up->rows == gate->rows && shared_up->cols == gate->cols && shared_gate->experts == 1 && shared_up->experts == 1;
    if (same_shape && check_matrix(gate, "gate") == TSP_OK && check_matrix(up, "up") == TSP_OK && check_matrix(shared_gate, "shared gate") == TSP_OK &&
        check_matrix(shared_up, "shared up") == TSP_OK && gate->type == up->type && gate->layout == up->layout && up->rows == gate->rows &&
        up->cols == gate->cols && up->experts == gate->experts && gate->expert_stride == up->expert_stride && gate->split == up->split &&
        tokens >= 1 && selected >= 1 && selected <= 64 && check_rows(d_x, x_stride, gate->cols, 4, "gate-up input") == TSP_OK &&
        check_rows(d_shared_x, shared_x_stride, gate->cols, 4, "shared gate-up input") == TSP_OK &&
        check_rows(d_h, h_stride, gate->rows, 4, "gate-up output") == TSP_OK &&
        check_rows(d_shared_h, shared_h_stride, gate->rows, 4, "shared gate-up output") == TSP_OK && aligned16(d_x) && x_stride % 16 == 0 &&
        aligned16(d_shared_x) && shared_x_stride % 16 == 0 &&
        (!d_x16 || check_rows(d_x16, x16_stride, gate->cols, 2, "binary16 input") == TSP_OK)) {
        GemvShared sh{shared_gate, shared_up, d_shared_x, shared_x_stride, d_shared_h, shared_h_stride};
        sh.tokens = shared_tokens;
        if (d_x16 && x_is_f16_exact) { sh.x16 = d_x16; sh.x16_stride_bytes = x16_stride; }   // the binary16 rows themselves: staged without conversion
        const int rc = launch_gemv(gate, up, true, d_x, x_stride, selected, tokens, d_token_map, d_counts, d_tasks, d_h, h_stride,
                                   x_is_f16_exact, 1, d_error, static_cast<cudaStream_t>(stream), &sh);
        if (rc <= 0) return rc;
    }
    if (int rc = tsp_moe_gate_up_swiglu(gate, up, d_x, x_stride, tokens, selected, d_token_map, d_counts, d_tasks, d_h, h_stride, x_is_f16_exact,
                                        d_error, stream)) return rc;
    return tsp_moe_gate_up_swiglu(shared_gate, shared_up, d_shared_x, shared_x_stride, shared_tokens, 1, nullptr, nullptr, nullptr, d_shared_h, shared_h_stride,
                                  x_is_f16_exact, d_error, stream);
}

int tsp_moe_gate_up_swiglu_shared(const tsp_matrix_set* gate, const tsp_matrix_set* up, const tsp_matrix_set* shared_gate,
                                  const tsp_matrix_set* shared_up, const float* d_x, uint64_t x_stride, const void* d_x16,
                                  uint64_t x16_stride, uint32_t tokens, uint32_t selected, const uint32_t* d_token_map,
                                  const uint32_t* d_counts, const uint32_t* d_tasks, float* d_h, uint64_t h_stride, float* d_shared_h,
                                  uint64_t shared_h_stride, int x_is_f16_exact, uint32_t* d_error, void* stream) {
    return tsp_moe_gate_up_swiglu_shared_rows(gate, up, shared_gate, shared_up, d_x, x_stride, d_x16, x16_stride, tokens, selected, d_token_map, d_counts,
                                              d_tasks, d_h, h_stride, d_x, x_stride, tokens, d_shared_h, shared_h_stride, x_is_f16_exact, d_error, stream);
}

int tsp_moe_project_shared_rows(const tsp_matrix_set* w, const tsp_matrix_set* shared_w, const float* d_in, uint64_t in_stride,
                                const float* d_shared_in, uint64_t shared_in_stride, uint32_t shared_tokens, uint32_t tokens, uint32_t selected,
                                const uint32_t* d_token_map, const uint32_t* d_counts, const uint32_t* d_tasks, float* d_out, uint64_t out_stride,
                                float* d_shared_out, uint64_t shared_out_stride, uint32_t* d_error, void* stream) {
    TSP_REQUIRE(w && shared_w && d_token_map && d_counts && d_tasks && d_shared_in && d_shared_out && shared_tokens >= 1, "project with shared expert: null argument");
    const bool same_shape = shared_w->type == w->type && shared_w->layout == w->layout && shared_w->rows == w->rows && shared_w->cols == w->cols &&
                            shared_w->experts == 1;
    if (same_shape && w->rows % 16 == 0 && check_matrix(w, "project") == TSP_OK && check_matrix(shared_w, "shared project") == TSP_OK &&
        tokens >= 1 && selected >= 1 && selected <= 64 && check_rows(d_in, in_stride, w->cols, 4, "project input") == TSP_OK &&
        check_rows(d_shared_in, shared_in_stride, w->cols, 4, "shared project input") == TSP_OK &&
        check_rows(d_out, out_stride, w->rows, 4, "project output") == TSP_OK &&
        check_rows(d_shared_out, shared_out_stride, w->rows, 4, "shared project output") == TSP_OK) {
        GemvShared sh{shared_w, nullptr, d_shared_in, shared_in_stride, d_shared_out, shared_out_stride};
        sh.tokens = shared_tokens;
        const int rc = launch_gemv(w, nullptr, false, d_in, in_stride, 1, tokens, d_token_map, d_counts, d_tasks, d_out, out_stride, 0, 1, d_error,
                                   static_cast<cudaStream_t>(stream), &sh);
        if (rc <= 0) return rc;
    }
    if (int rc = tsp_moe_project(w, d_in, in_stride, 1, tokens, selected, d_token_map, d_counts, d_tasks, d_out, out_stride, 0, d_error, stream)) return rc;
    return tsp_moe_project(shared_w, d_shared_in, shared_in_stride, 1, shared_tokens, 1, nullptr, nullptr, nullptr, d_shared_out, shared_out_stride, 0,
                           d_error, stream);
}

int tsp_moe_project_shared(const tsp_matrix_set* w, const tsp_matrix_set* shared_w, const float* d_in, uint64_t in_stride,
                           const float* d_shared_in, uint64_t shared_in_stride, uint32_t tokens, uint32_t selected,
                           const uint32_t* d_token_map, const uint32_t* d_counts, const uint32_t* d_tasks, float* d_out, uint64_t out_stride,
                           float* d_shared_out, uint64_t shared_out_stride, uint32_t* d_error, void* stream) {
    return tsp_moe_project_shared_rows(w, shared_w, d_in, in_stride, d_shared_in, shared_in_stride, tokens, tokens, selected, d_token_map, d_counts, d_tasks,
                                       d_out, out_stride, d_shared_out, shared_out_stride, d_error, stream);
}

int tsp_moe_layer_decode(const tsp_moe_weights* w, const tsp_moe_scratch* s, const void* d_x, uint64_t x_stride,
                         uint32_t x_dtype, const float* d_logits, uint64_t logits_stride, uint32_t tokens,
                         uint32_t channels, uint32_t hidden, uint32_t experts, uint32_t selected, uint32_t mode,
                         int normalize, void* d_out, uint64_t out_stride, uint32_t out_dtype, uint32_t* d_error, void* stream) {
    TSP_REQUIRE(w && s && d_x && d_logits && d_out, "layer: null argument");
    TSP_REQUIRE(tokens >= 1 && tokens <= s->capacity, "layer: %u token rows exceed the scratch capacity %u", tokens, s->capacity);
    TSP_REQUIRE(x_dtype <= 1 && out_dtype <= 1, "layer: activation dtype must be 0 (FP32) or 1 (binary16)");
    TSP_REQUIRE(w->gate.rows == hidden && w->gate.cols == channels && w->gate.experts == experts &&
                w->down.rows == channels && w->down.cols == hidden && w->down.experts == experts &&
                w->shared_gate.rows == hidden && w->shared_gate.cols == channels && w->shared_gate.experts == 1 &&
                w->shared_up.experts == 1 && w->shared_down.rows == channels && w->shared_down.cols == hidden &&
                w->shared_down.experts == 1, "layer: weight shapes do not match the layer shape");
    TSP_REQUIRE(s->d_ids && s->d_weights && s->d_hidden && s->d_routed && s->d_shared_hidden && s->d_shared_out &&
                s->d_token_map && s->d_counts && s->d_tasks, "layer: incomplete scratch");
    TSP_REQUIRE(x_dtype == 0 || s->d_x32, "layer: binary16 input needs the d_x32 staging rows");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    TSP_REQUIRE(experts >= 1 && experts <= 4096 && selected >= 1 && selected <= 64 && selected <= experts && mode <= 1, "layer: invalid router shape/mode");
    TSP_REQUIRE(logits_stride >= static_cast<uint64_t>(experts) * 4 && logits_stride % 4 == 0, "layer: logits stride too small");
    const float* x32 = static_cast<const float*>(d_x);
    uint64_t x32_stride = x_stride;
    if (x_dtype == 1) { x32 = s->d_x32; x32_stride = channels * 4ull; }
    const int exact = x_dtype == 1;
    // small batches: route, permutation, tile table and the binary16 -> FP32 copy of the rows in ONE launch
    int fused = launch_decode_prologue(d_logits, logits_stride, tokens, experts, selected, mode, normalize, TSP_GEMV_TILE, s->d_ids, s->d_weights,
                                       s->d_token_map, s->d_counts, s->d_tasks, x_dtype == 1 ? d_x : nullptr, x_stride, s->d_x32, channels * 4ull,
                                       channels, d_error, st);
    if (fused < 0) return fused;
    if (fused == 1) {
        if (x_dtype == 1) { if (int rc = tsp_rows_f16_to_f32(d_x, x_stride, s->d_x32, channels * 4ull, tokens, channels, st)) return rc; }
        if (int rc = tsp_moe_route(d_logits, logits_stride, tokens, experts, selected, mode, normalize, s->d_ids, s->d_weights, d_error, st)) return rc;
        if (int rc = tsp_moe_permute(s->d_ids, tokens, experts, selected, TSP_GEMV_TILE, s->d_token_map, s->d_counts, s->d_tasks, d_error, st)) return rc;
    }
    if (int rc = tsp_moe_gate_up_swiglu_shared(&w->gate, &w->up, &w->shared_gate, &w->shared_up, x32, x32_stride, x_dtype == 1 ? d_x : nullptr,
                                               x_dtype == 1 ? x_stride : 0, tokens, selected, s->d_token_map, s->d_counts, s->d_tasks, s->d_hidden,
                                               hidden * 4ull, s->d_shared_hidden, hidden * 4ull, exact, d_error, stream)) return rc;
    if (int rc = tsp_moe_project_shared(&w->down, &w->shared_down, s->d_hidden, hidden * 4ull, s->d_shared_hidden, hidden * 4ull, tokens, selected,
                                        s->d_token_map, s->d_counts, s->d_tasks, s->d_routed, channels * 4ull, s->d_shared_out, channels * 4ull,
                                        d_error, stream)) return rc;
    // binary16 output rows are written straight from the FP32 mixture; no FP32 copy of the output is kept
    return tsp_moe_combine(s->d_routed, channels * 4ull, 0, s->d_weights, s->d_shared_out, channels * 4ull, w->d_shared_router, x32,
                           x32_stride, 0, s->d_shared_logit, tokens, channels, selected,
                           out_dtype == 0 ? static_cast<float*>(d_out) : nullptr, out_dtype == 0 ? out_stride : 0,
                           out_dtype == 1 ? d_out : nullptr, out_dtype == 1 ? out_stride : 0, d_error, st);
}

static int q8_lanes(const void* d_in, void* d_out, uint64_t rows, uint32_t cols, bool unpack, void* stream) {
    TSP_REQUIRE(d_in && d_out && rows >= 1 && cols >= 32 && cols % 32 == 0 && cols <= 65536, "q8 lanes: null buffer or invalid shape");
    TSP_REQUIRE(reinterpret_cast<uintptr_t>(d_in) % 2 == 0 && reinterpret_cast<uintptr_t>(d_out) % 2 == 0, "q8 lanes: buffers must be 2-byte aligned");
    const uint64_t bytes = rows * (cols / 32u) * 34ull;
    TSP_REQUIRE(!overlap(d_in, bytes, d_out, bytes), "q8 lanes: input and output overlap");
    return launch_q8_lanes(d_in, d_out, rows, cols, unpack, static_cast<cudaStream_t>(stream));
}
int tsp_q8_lanes_unpack(const void* d_lanes, void* d_gguf, uint64_t rows, uint32_t cols, void* stream) { return q8_lanes(d_lanes, d_gguf, rows, cols, true, stream); }
int tsp_q8_lanes_pack(const void* d_gguf, void* d_lanes, uint64_t rows, uint32_t cols, void* stream) { return q8_lanes(d_gguf, d_lanes, rows, cols, false, stream); }

int tsp_selftest_bounded_wait(uint32_t polls, uint32_t* d_error, void* stream) {
    TSP_REQUIRE(d_error && polls >= 1 && polls <= (1u << 16), "bounded-wait self test: null error word or poll limit outside 1..65536");
    return launch_bounded_wait_selftest(polls, d_error, static_cast<cudaStream_t>(stream));
}

uint64_t tsp_logit_topk_scratch_bytes(uint32_t rows, uint32_t vocabulary) {
    if (!rows || rows > 2048 || !vocabulary || vocabulary > (1u << 20)) return 0;
    return static_cast<uint64_t>(rows) * ((vocabulary + TSP_TOPK_TILE_SPAN - 1) / TSP_TOPK_TILE_SPAN) * TSP_TOPK_ROW_BYTES;
}
uint64_t tsp_logit_topk_output_bytes(uint32_t rows) { return rows && rows <= 2048 ? static_cast<uint64_t>(rows) * TSP_TOPK_ROW_BYTES : 0; }

int tsp_logit_topk(const float* d_logits, uint64_t stride, uint32_t rows, uint32_t vocabulary, void* d_partial, uint64_t partial_bytes,
                   void* d_rows_out, uint64_t out_bytes, void* stream) {
    TSP_REQUIRE(d_logits && d_partial && d_rows_out, "logit top-k: null buffer");
    TSP_REQUIRE(rows >= 1 && rows <= 2048 && vocabulary >= 1 && vocabulary <= (1u << 20) && stride >= static_cast<uint64_t>(vocabulary) * 4 && stride % 4 == 0,
                "logit top-k geometry mismatch");
    const uint64_t need_partial = tsp_logit_topk_scratch_bytes(rows, vocabulary), need_out = tsp_logit_topk_output_bytes(rows);
    const uint64_t in_bytes = static_cast<uint64_t>(rows - 1) * stride + static_cast<uint64_t>(vocabulary) * 4;
    TSP_REQUIRE(partial_bytes >= need_partial && out_bytes >= need_out && reinterpret_cast<uintptr_t>(d_logits) % 4 == 0 &&
                reinterpret_cast<uintptr_t>(d_partial) % 4 == 0 && reinterpret_cast<uintptr_t>(d_rows_out) % 4 == 0,
                "logit top-k buffer span or alignment mismatch");
    TSP_REQUIRE(!overlap(d_logits, in_bytes, d_partial, need_partial) && !overlap(d_logits, in_bytes, d_rows_out, need_out) &&
                !overlap(d_partial, need_partial, d_rows_out, need_out), "logit top-k buffers overlap");
    return launch_logit_topk(d_logits, stride, rows, vocabulary, static_cast<uint32_t*>(d_partial), static_cast<uint32_t*>(d_rows_out),
                             static_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------------------------------------
// Prefill-size path: grouped per-expert GEMMs on the tcgen05 tensor cores
// ---------------------------------------------------------------------------------------------
int tsp_moe_route_offsets(const uint32_t* d_counts, uint32_t experts, uint32_t* d_offsets, void* stream) {
    TSP_REQUIRE(d_counts && d_offsets && experts >= 1 && experts <= 4096, "offsets: null buffer or experts out of range");
    return launch_route_offsets(d_counts, experts, d_offsets, static_cast<cudaStream_t>(stream));
}

int tsp_moe_rows_f16k(const void* d_x, uint64_t x_stride, uint32_t x_dtype, uint32_t rows, uint32_t cols, void* d_xk, uint64_t xk_stride,
                      uint32_t* d_error, void* stream) {
    TSP_REQUIRE(x_dtype <= 1 && rows >= 1 && cols >= 8 && cols % 8 == 0, "K-ordered rows: invalid shape or dtype");
    if (int rc = check_rows(d_x, x_stride, cols, x_dtype ? 2 : 4, "K-ordered rows input")) return rc;
    if (int rc = check_rows(d_xk, xk_stride, cols, 2, "K-ordered rows output")) return rc;
    TSP_REQUIRE(!overlap(d_x, rows * x_stride, d_xk, rows * xk_stride), "K-ordered rows: input and output overlap");
    return launch_rows_f16k(d_x, x_stride, x_dtype, rows, cols, d_xk, xk_stride, d_error, static_cast<cudaStream_t>(stream));
}

static int check_shared_set(const tsp_matrix_set* s, const tsp_matrix_set* like, const char* name) {
    if (int rc = check_matrix(s, name)) return rc;
    TSP_REQUIRE(s->experts == 1 && s->type == like->type && s->layout == like->layout && s->rows == like->rows && s->cols == like->cols,
                "%s: the shared expert must have the routed experts' shape, encoding and layout", name);
    return TSP_OK;
}

int tsp_moe_gather_rows16(const void* d_xk, uint64_t xk_stride, const uint32_t* d_token_map, const uint32_t* d_offsets, uint32_t experts,
                          uint32_t tokens, uint32_t selected, uint32_t cols, void* d_xp, uint64_t xp_stride, void* stream) {
    TSP_REQUIRE(d_token_map && d_offsets && experts >= 1 && experts <= 4096 && tokens >= 1 && selected >= 1 && selected <= 64 && cols >= 8 && cols % 8 == 0,
                "gather: null table or invalid shape");
    TSP_REQUIRE(static_cast<uint64_t>(tokens) * selected < (1ull << 31), "gather: too many routes");
    if (int rc = check_rows(d_xk, xk_stride, cols, 2, "gather input")) return rc;
    if (int rc = check_rows(d_xp, xp_stride, cols, 2, "gather output")) return rc;
    return launch_gather_rows16(d_xk, xk_stride, d_token_map, d_offsets, experts, tokens, selected, cols, d_xp, xp_stride, static_cast<cudaStream_t>(stream));
}

int tsp_moe_grouped_gate_up(const tsp_matrix_set* gate, const tsp_matrix_set* up, const tsp_matrix_set* shared_gate, const tsp_matrix_set* shared_up,
                            const void* d_xp, uint64_t xp_stride, const void* d_xk, uint64_t xk_stride, uint32_t shared_tokens, uint32_t tokens,
                            uint32_t selected, const uint32_t* d_token_map, const uint32_t* d_counts, const uint32_t* d_tasks, uint32_t* d_offsets,
                            void* d_hp, uint64_t hp_stride, void* d_s_hp, uint64_t s_hp_stride, uint32_t* d_error, void* stream) {
    if (int rc = check_matrix(gate, "gate")) return rc;
    if (int rc = check_matrix(up, "up")) return rc;
    TSP_REQUIRE(gate->type == up->type && gate->layout == up->layout && gate->rows == up->rows && gate->cols == up->cols &&
                gate->experts == up->experts && gate->expert_stride == up->expert_stride && gate->split == up->split,
                "gate/up matrix sets must share shape, encoding, layout and addressing");
    TSP_REQUIRE(d_token_map && d_tasks && d_counts && d_offsets && tokens >= 1 && selected >= 1 && selected <= 64, "grouped gate-up: null table or empty batch");
    TSP_REQUIRE(static_cast<uint64_t>(tokens) * selected < (1ull << 31), "grouped gate-up: too many routes");
    TSP_REQUIRE((shared_gate != nullptr) == (shared_up != nullptr), "grouped gate-up: shared gate and up go together");
    if (int rc = check_rows(d_xp, xp_stride, gate->cols, 2, "grouped gate-up input")) return rc;
    if (int rc = check_rows(d_hp, hp_stride, gate->rows, 2, "grouped gate-up output")) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    uint32_t* counter = d_offsets + gate->experts + 1;
    if (!shared_gate)
        return launch_grouped(gate, up, true, d_xp, xp_stride, tokens * selected, tokens, selected, d_token_map, d_tasks, d_counts, d_offsets, counter,
                              d_hp, hp_stride, 0, d_error, st);
    if (int rc = check_shared_set(shared_gate, gate, "shared gate")) return rc;
    if (int rc = check_shared_set(shared_up, gate, "shared up")) return rc;
    if (int rc = check_rows(d_xk, xk_stride, gate->cols, 2, "shared gate-up input")) return rc;
    if (int rc = check_rows(d_s_hp, s_hp_stride, gate->rows, 2, "shared gate-up output")) return rc;
    TSP_REQUIRE(shared_tokens >= 1, "grouped gate-up: the shared expert needs at least one row");
    const GroupedShared sh{shared_gate, shared_up, d_xk, xk_stride, shared_tokens, d_s_hp, s_hp_stride};
    return launch_grouped(gate, up, true, d_xp, xp_stride, tokens * selected, tokens, selected, d_token_map, d_tasks, d_counts, d_offsets, counter,
                          d_hp, hp_stride, 0, d_error, st, &sh);
}

int tsp_moe_grouped_down(const tsp_matrix_set* down, const tsp_matrix_set* shared_down, const void* d_hp, uint64_t hp_stride, uint32_t tokens,
                         uint32_t selected, const uint32_t* d_token_map, const uint32_t* d_counts, const uint32_t* d_tasks, uint32_t* d_offsets,
                         void* d_routed, uint64_t routed_stride, uint32_t routed_dtype, const void* d_s_hp, uint64_t s_hp_stride,
                         uint32_t shared_tokens, float* d_shared_out, uint64_t shared_out_stride, uint32_t* d_error, void* stream) {
    if (int rc = check_matrix(down, "down")) return rc;
    TSP_REQUIRE(d_token_map && d_tasks && d_counts && d_offsets && tokens >= 1 && selected >= 1 && selected <= 64 && routed_dtype <= 1,
                "grouped down: null table, empty batch or bad row dtype");
    TSP_REQUIRE(static_cast<uint64_t>(tokens) * selected < (1ull << 31), "grouped down: too many routes");
    if (int rc = check_rows(d_hp, hp_stride, down->cols, 2, "grouped down input")) return rc;
    if (int rc = check_rows(d_routed, routed_stride, down->rows, routed_dtype ? 2 : 4, "grouped down output")) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    uint32_t* counter = d_offsets + down->experts + 2;
    if (!shared_down)
        return launch_grouped(down, nullptr, false, d_hp, hp_stride, tokens * selected, tokens, selected, d_token_map, d_tasks, d_counts, d_offsets,
                              counter, d_routed, routed_stride, routed_dtype, d_error, st);
    if (int rc = check_shared_set(shared_down, down, "shared down")) return rc;
    if (int rc = check_rows(d_s_hp, s_hp_stride, down->cols, 2, "shared down input")) return rc;
    if (int rc = check_rows(d_shared_out, shared_out_stride, down->rows, 4, "shared down output")) return rc;
    TSP_REQUIRE(shared_tokens >= 1, "grouped down: the shared expert needs at least one row");
    const GroupedShared sh{shared_down, nullptr, d_s_hp, s_hp_stride, shared_tokens, d_shared_out, shared_out_stride};
    return launch_grouped(down, nullptr, false, d_hp, hp_stride, tokens * selected, tokens, selected, d_token_map, d_tasks, d_counts, d_offsets,
                          counter, d_routed, routed_stride, routed_dtype, d_error, st, &sh);
}

int tsp_dense_mm_swiglu(const tsp_matrix_set* gate, const tsp_matrix_set* up, const void* d_xk, uint64_t xk_stride, uint32_t rows,
                        void* d_h, uint64_t h_stride, uint32_t* d_counter, uint32_t* d_error, void* stream) {
    if (int rc = check_matrix(gate, "dense gate")) return rc;
    if (int rc = check_matrix(up, "dense up")) return rc;
    TSP_REQUIRE(gate->experts == 1 && up->experts == 1 && gate->type == up->type && gate->layout == up->layout && gate->rows == up->rows &&
                gate->cols == up->cols, "dense gate/up must be single matrices of one shape, encoding and layout");
    TSP_REQUIRE(rows >= 1 && d_counter, "dense gate-up: no rows or no item counter");
    if (int rc = check_rows(d_xk, xk_stride, gate->cols, 2, "dense gate-up input")) return rc;
    if (int rc = check_rows(d_h, h_stride, gate->rows, 2, "dense gate-up output")) return rc;
    const GroupedShared sh{gate, up, d_xk, xk_stride, rows, d_h, h_stride};
    return launch_grouped(gate, up, true, d_xk, xk_stride, rows, rows, 1, nullptr, nullptr, nullptr, nullptr, d_counter, d_h, h_stride, 0, d_error,
                          static_cast<cudaStream_t>(stream), &sh);
}

int tsp_dense_mm(const tsp_matrix_set* m, const void* d_xk, uint64_t xk_stride, uint32_t rows, float* d_out, uint64_t out_stride,
                 uint32_t* d_counter, uint32_t* d_error, void* stream) {
    if (int rc = check_matrix(m, "dense matrix")) return rc;
    TSP_REQUIRE(m->experts == 1, "dense projection: one matrix");
    TSP_REQUIRE(rows >= 1 && d_counter, "dense projection: no rows or no item counter");
    if (int rc = check_rows(d_xk, xk_stride, m->cols, 2, "dense projection input")) return rc;
    if (int rc = check_rows(d_out, out_stride, m->rows, 4, "dense projection output")) return rc;
    const GroupedShared sh{m, nullptr, d_xk, xk_stride, rows, d_out, out_stride};
    return launch_grouped(m, nullptr, false, d_xk, xk_stride, rows, rows, 1, nullptr, nullptr, nullptr, nullptr, d_counter, d_out, out_stride, 0, d_error,
                          static_cast<cudaStream_t>(stream), &sh);
}

int tsp_moe_staged_f16(const tsp_matrix_set* m, uint32_t expert, void* d_out, void* stream) {
    if (int rc = check_matrix(m, "staged tile")) return rc;
    if (m->type != TSP_TYPE_Q4_K || m->layout != TSP_LAYOUT_PLANAR) return fail(TSP_E_TYPE, "staged tile: only Q4_K Pack v3 planar weights go through the tensor-core kernels");
    TSP_REQUIRE(expert < m->experts && d_out, "staged tile: expert out of range or null output");
    const uint8_t* base = static_cast<const uint8_t*>(expert < m->split ? m->base : m->base_hi);
    const uint32_t local = expert < m->split ? expert : expert - m->split;
    return launch_staged_f16(base + local * m->expert_stride, m->rows, m->cols, d_out, static_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------------------------------------
// Entry point that needs no caller scratch and performs no device allocation.
// ---------------------------------------------------------------------------------------------
// All intermediate buffers of one layer call live in this array. Every device that loads the library
// carries it from load until process exit.
static __device__ __align__(256) unsigned char g_static_scratch[TSP_STATIC_SCRATCH_BYTES];

namespace {
// The array's name is only a host-side handle; kernels need its device address, which is looked up once per
// device (with that device current) and remembered here.
constexpr int kMaxDevices = 64;
std::atomic<unsigned char*> g_static_scratch_addr[kMaxDevices] = {};   // two host threads may make a device's first call at once

struct StaticPlan {
    uint64_t ids, weights, hidden, routed, shared_hidden, shared_out, shared_logit, x32, token_map, counts, tasks, total;
};

StaticPlan plan_static(uint32_t tokens, uint32_t channels, uint32_t hidden, uint32_t experts, uint32_t selected) {
    StaticPlan pl{};
    uint64_t at = 0;
    auto take = [&](uint64_t bytes) { const uint64_t here = at; at += (bytes + 255) & ~uint64_t(255); return here; };
    const uint64_t T = tokens, K = selected;
    pl.ids = take(T * K * 4);
    pl.weights = take(T * K * 4);
    pl.hidden = take(T * K * hidden * 4);
    pl.routed = take(T * K * channels * 4);
    pl.shared_hidden = take(T * hidden * 4);
    pl.shared_out = take(T * channels * 4);
    pl.shared_logit = take(T * 4);
    pl.x32 = take(T * channels * 4);
    pl.token_map = take(uint64_t(experts) * T * 4);
    pl.counts = take(uint64_t(experts) * 4);
    pl.tasks = take(tsp_moe_tasks_words(tokens, experts, selected, TSP_GEMV_TILE) * 4);
    pl.total = at;
    return pl;
}
}  // namespace

int tsp_moe_layer_prefill(const tsp_moe_weights* w, const tsp_moe_prefill_scratch* ps, const void* d_x, uint64_t x_stride,
                          uint32_t x_dtype, const float* d_logits, uint64_t logits_stride, uint32_t tokens, uint32_t channels,
                          uint32_t hidden, uint32_t experts, uint32_t selected, uint32_t mode, int normalize, void* d_out,
                          uint64_t out_stride, uint32_t out_dtype, uint32_t* d_error, void* stream) {
    TSP_REQUIRE(w && ps && d_x && d_logits && d_out, "prefill layer: null argument");
    const tsp_moe_scratch* s = &ps->base;
    TSP_REQUIRE(tokens >= 1 && tokens <= s->capacity, "prefill layer: %u token rows exceed the scratch capacity %u", tokens, s->capacity);
    TSP_REQUIRE(x_dtype <= 1 && out_dtype <= 1, "prefill layer: activation dtype must be 0 (FP32) or 1 (binary16)");
    TSP_REQUIRE(selected >= 1 && selected <= 64, "prefill layer: selected out of range");
    TSP_REQUIRE(w->gate.rows == hidden && w->gate.cols == channels && w->gate.experts == experts &&
                w->down.rows == channels && w->down.cols == hidden && w->down.experts == experts &&
                w->shared_gate.rows == hidden && w->shared_gate.cols == channels && w->shared_gate.experts == 1 &&
                w->shared_up.experts == 1 && w->shared_down.rows == channels && w->shared_down.cols == hidden &&
                w->shared_down.experts == 1, "prefill layer: weight shapes do not match the layer shape");
    TSP_REQUIRE(s->d_ids && s->d_weights && s->d_routed && s->d_shared_out && s->d_token_map && s->d_counts && s->d_tasks && ps->d_xk &&
                ps->d_xp && ps->d_hp && ps->d_offsets && ps->d_s_hp, "prefill layer: incomplete scratch");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (int rc = tsp_moe_rows_f16k(d_x, x_stride, x_dtype, tokens, channels, ps->d_xk, channels * 2ull, d_error, st)) return rc;
    if (int rc = tsp_moe_route(d_logits, logits_stride, tokens, experts, selected, mode, normalize, s->d_ids, s->d_weights, d_error, st)) return rc;
    if (int rc = tsp_moe_permute(s->d_ids, tokens, experts, selected, TSP_GROUPED_TILE, s->d_token_map, s->d_counts, s->d_tasks, d_error, st)) return rc;
    if (int rc = tsp_moe_route_offsets(s->d_counts, experts, ps->d_offsets, st)) return rc;
    if (int rc = tsp_moe_gather_rows16(ps->d_xk, channels * 2ull, s->d_token_map, ps->d_offsets, experts, tokens, selected, channels, ps->d_xp,
                                       channels * 2ull, st)) return rc;
    // the dense shared expert rides in both launches when it has the routed experts' encoding and layout; in another form (the
    // reference's dense Q8_0 shared expert beside Q4_K experts) it gets the same kernel in launches of its own.
    // The route rows are kept as binary16 (half the traffic of the mixture)
    auto same_form = [](const tsp_matrix_set& a, const tsp_matrix_set& b) { return a.type == b.type && a.layout == b.layout; };
    const bool ride_up = same_form(w->shared_gate, w->gate) && same_form(w->shared_up, w->gate);
    const bool ride_down = same_form(w->shared_down, w->down);
    if (int rc = tsp_moe_grouped_gate_up(&w->gate, &w->up, ride_up ? &w->shared_gate : nullptr, ride_up ? &w->shared_up : nullptr, ps->d_xp, channels * 2ull,
                                         ps->d_xk, channels * 2ull, tokens, tokens, selected, s->d_token_map,
                                         s->d_counts, s->d_tasks, ps->d_offsets, ps->d_hp, hidden * 2ull, ps->d_s_hp, hidden * 2ull, d_error, st)) return rc;
    if (!ride_up)
        if (int rc = tsp_dense_mm_swiglu(&w->shared_gate, &w->shared_up, ps->d_xk, channels * 2ull, tokens, ps->d_s_hp, hidden * 2ull,
                                         ps->d_offsets + experts + 3, d_error, st)) return rc;
    if (int rc = tsp_moe_grouped_down(&w->down, ride_down ? &w->shared_down : nullptr, ps->d_hp, hidden * 2ull, tokens, selected, s->d_token_map, s->d_counts,
                                      s->d_tasks, ps->d_offsets, s->d_routed, channels * 2ull, 1, ps->d_s_hp, hidden * 2ull, tokens, s->d_shared_out,
                                      channels * 4ull, d_error, st)) return rc;
    if (!ride_down)
        if (int rc = tsp_dense_mm(&w->shared_down, ps->d_s_hp, hidden * 2ull, tokens, s->d_shared_out, channels * 4ull, ps->d_offsets + experts + 4,
                                  d_error, st)) return rc;
    return tsp_moe_combine(s->d_routed, channels * 2ull, 1, s->d_weights, s->d_shared_out, channels * 4ull, w->d_shared_router, d_x, x_stride, x_dtype,
                           s->d_shared_logit, tokens, channels, selected, out_dtype == 0 ? static_cast<float*>(d_out) : nullptr,
                           out_dtype == 0 ? out_stride : 0, out_dtype == 1 ? d_out : nullptr, out_dtype == 1 ? out_stride : 0, d_error, st);
}

uint64_t tsp_moe_layer_decode_static_bytes(uint32_t tokens, uint32_t channels, uint32_t hidden, uint32_t experts, uint32_t selected) {
    if (!tokens || !channels || !hidden || !experts || !selected || selected > 64) return 0;
    return plan_static(tokens, channels, hidden, experts, selected).total;
}

int tsp_moe_layer_decode_static(const tsp_moe_weights* w, const void* d_x, uint64_t x_stride, uint32_t x_dtype,
                                const float* d_logits, uint64_t logits_stride, uint32_t tokens, uint32_t channels,
                                uint32_t hidden, uint32_t experts, uint32_t selected, uint32_t mode, int normalize,
                                void* d_out, uint64_t out_stride, uint32_t out_dtype, uint32_t* d_error, void* stream) {
    TSP_REQUIRE(tokens >= 1 && channels >= 1 && hidden >= 1 && experts >= 1 && selected >= 1 && selected <= 64 && experts <= 4096,
                "static layer: invalid layer shape");
    const StaticPlan pl = plan_static(tokens, channels, hidden, experts, selected);
    if (pl.total > TSP_STATIC_SCRATCH_BYTES)
        return fail(TSP_E_ARG, "static layer: %u tokens of this layer shape need %llu bytes of scratch, the built-in array holds %llu; "
                               "use tsp_moe_layer_decode with caller scratch", tokens, static_cast<unsigned long long>(pl.total),
                    static_cast<unsigned long long>(TSP_STATIC_SCRATCH_BYTES));
    int dev = 0;
    TSP_CUDA(cudaGetDevice(&dev));
    TSP_REQUIRE(dev >= 0 && dev < kMaxDevices, "static layer: device ordinal %d out of range", dev);
    unsigned char* base = g_static_scratch_addr[dev].load(std::memory_order_acquire);
    if (!base) {   // first call on this device: resolve the array's device address (every racing thread resolves the same value)
        TSP_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&base), g_static_scratch));
        TSP_REQUIRE(base != nullptr, "static layer: the scratch array has no device address");
        g_static_scratch_addr[dev].store(base, std::memory_order_release);
    }
    tsp_moe_scratch s{};
    s.d_ids = reinterpret_cast<uint32_t*>(base + pl.ids);
    s.d_weights = reinterpret_cast<float*>(base + pl.weights);
    s.d_hidden = reinterpret_cast<float*>(base + pl.hidden);
    s.d_routed = reinterpret_cast<float*>(base + pl.routed);
    s.d_shared_hidden = reinterpret_cast<float*>(base + pl.shared_hidden);
    s.d_shared_out = reinterpret_cast<float*>(base + pl.shared_out);
    s.d_shared_logit = reinterpret_cast<float*>(base + pl.shared_logit);
    s.d_x32 = reinterpret_cast<float*>(base + pl.x32);
    s.d_token_map = reinterpret_cast<uint32_t*>(base + pl.token_map);
    s.d_counts = reinterpret_cast<uint32_t*>(base + pl.counts);
    s.d_tasks = reinterpret_cast<uint32_t*>(base + pl.tasks);
    s.capacity = tokens;
    // Nothing in the scratch has to start at zero: every region is fully written by the launch that produces it
    // before any launch reads it, so the previous call's contents are simply overwritten.
    return tsp_moe_layer_decode(w, &s, d_x, x_stride, x_dtype, d_logits, logits_stride, tokens, channels, hidden, experts, selected,
                                mode, normalize, d_out, out_stride, out_dtype, d_error, stream);
}

}  // extern "C"
