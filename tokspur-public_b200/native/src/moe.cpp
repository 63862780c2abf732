// encode_moe over the CUDA graph: the reference's composition (native/src/moe.cpp:37-83) with the routed / shared expert
// stages and the mixture forwarded to the C ABI's layer entry point. Shape and extent checks happen before anything is encoded.
#include "tokspur_b200/moe.hpp"

namespace tokspur_b200 {
namespace {
void shape_check(MoeShape s) {
    if (!s.channels || s.channels > 65536 || !s.hidden || s.hidden > 65536 || !s.experts || s.experts > 4096 || !s.selected ||
        s.selected > 64 || s.selected > s.experts) throw FormatError("invalid mixture shape");
}

// matrix set of `experts` matrices [rows x cols] behind one view: GGUF rows, or a registered planar tensor
tsp_matrix_set matrix_set(const CudaGraph& g, GpuMatrix m, uint32_t rows, uint32_t cols, uint32_t experts) {
    tsp_matrix_set s{};
    s.base = g.device_pointer(m.view);
    s.rows = rows; s.cols = cols; s.experts = experts; s.split = experts; s.type = m.encoding;
    const auto planar = g.planar_matrix_shape(m.view);
    s.layout = planar ? TSP_LAYOUT_PLANAR : TSP_LAYOUT_GGUF;
    s.expert_stride = tsp_expert_bytes(s.type, s.layout, rows, cols);
    if (!s.expert_stride || m.view.bytes != s.expert_stride * experts) throw FormatError("weight view does not match the layer shape");
    return s;
}
}

std::array<GpuView, 13> MoeScratch::views() const {
    return {logits, indices, weights, gate, up, down, shared_gate, shared_up, shared_down, shared_logit, token_map, counts, tasks};
}

MoeScratch allocate_moe_rows_scratch(CudaGraph& graph, MoeShape s, uint32_t rows) {
    shape_check(s);
    if (!rows || rows > 64) throw FormatError("invalid row count for the mixture scratch");
    const uint64_t n = rows, tasks_words = tsp_moe_tasks_words(rows, s.experts, s.selected, TSP_GEMV_TILE);
    const std::array<uint64_t, 13> counts{n * s.experts, n * s.selected, n * s.selected, n * s.hidden * s.selected, n * s.hidden * s.selected,
                                          n * s.channels * s.selected, n * s.hidden, n * s.hidden, n * s.channels, n, n * s.experts, s.experts,
                                          tasks_words};
    std::array<GpuView, 13> v{};
    size_t made = 0;
    try {
        for (; made < counts.size(); ++made) v[made] = graph.zeros(counts[made] * 4, "mixture scratch");
    } catch (...) {
        for (size_t i = 0; i < made; ++i) graph.release(v[i]);
        throw;
    }
    return {v[0], v[1], v[2], v[3], v[4], v[5], v[6], v[7], v[8], v[9], v[10], v[11], v[12]};
}

MoeScratch allocate_moe_scratch(CudaGraph& graph, MoeShape s) { return allocate_moe_rows_scratch(graph, s, 1); }

void release_moe_scratch(CudaGraph& graph, const MoeScratch& scratch) {
    for (const auto view : scratch.views()) graph.release(view);
}

bool is_planar_gate_up(const CudaGraph& g, const MoeWeights& w, MoeShape s) {
    const auto lo = g.planar_matrix_shape(w.gate.view), hi = g.planar_matrix_shape(w.up.view);
    if (!lo || !hi) return false;
    return (lo->kind == 2u || lo->kind == 6u) && (hi->kind == 3u || hi->kind == 7u) && lo->source_type == w.gate.encoding &&
           hi->source_type == w.up.encoding && lo->source_type == hi->source_type && lo->columns == s.channels && lo->rows == s.hidden &&
           lo->experts == s.experts && hi->columns == s.channels && hi->rows == s.hidden && hi->experts == s.experts;
}

bool is_planar_moe(const CudaGraph& g, const MoeWeights& w, MoeShape s) {
    const auto dn = g.planar_matrix_shape(w.down.view);
    return is_planar_gate_up(g, w, s) && dn && (dn->kind == 9u || dn->kind == 10u) && dn->source_type == w.down.encoding &&
           dn->columns == s.hidden && dn->rows == s.channels && dn->experts == s.experts;
}

namespace {
void encode_rows(CudaGraph& g, const MoeWeights& w, const MoeScratch& s, GpuView input, GpuView output, MoeShape shape, RouterMode mode,
                 bool normalize_selected, uint32_t rows);
}

void encode_moe(CudaGraph& g, const MoeWeights& w, const MoeScratch& s, GpuView input, GpuView output, MoeShape shape,
                RouterMode mode, bool normalize_selected) {
    encode_rows(g, w, s, input, output, shape, mode, normalize_selected, 1);
}

MoeManyScratch allocate_moe_many_scratch(CudaGraph& graph, MoeShape shape, uint32_t capacity) {
    return {allocate_moe_rows_scratch(graph, shape, capacity), capacity};
}

void release_moe_many_scratch(CudaGraph& graph, const MoeManyScratch& scratch) { release_moe_scratch(graph, scratch.rows); }

void prepare_moe_many(CudaGraph& g, const MoeWeights& w, MoeShape shape) {
    shape_check(shape);
    if (w.router.encoding != 0 || w.shared_router.encoding != 0) throw FormatError("router projections must be F32");
    if (w.router.view.bytes != uint64_t(shape.channels) * shape.experts * 4 || w.shared_router.view.bytes != uint64_t(shape.channels) * 4)
        throw FormatError("router shape mismatch");
    if (!is_planar_gate_up(g, w, shape)) {
        (void)matrix_set(g, w.gate, shape.hidden, shape.channels, shape.experts);
        (void)matrix_set(g, w.up, shape.hidden, shape.channels, shape.experts);
    }
    (void)matrix_set(g, w.down, shape.channels, shape.hidden, shape.experts);
    (void)matrix_set(g, w.shared_gate, shape.hidden, shape.channels, 1);
    (void)matrix_set(g, w.shared_up, shape.hidden, shape.channels, 1);
    (void)matrix_set(g, w.shared_down, shape.channels, shape.hidden, 1);
}

uint64_t moe_many_dispatches(const CudaGraph&, const MoeWeights&, MoeShape shape, uint32_t steps) {
    shape_check(shape);
    if (!steps || steps > 64) throw FormatError("invalid row count for the mixture");
    return 6;   // router GEMV, routing (+ row conversion), permutation + tile table, gate-up, down, mixture
}

void encode_moe_many(CudaGraph& g, const MoeWeights& w, const MoeManyScratch& s, GpuView input, GpuView output, MoeShape shape, RouterMode mode,
                     bool normalize_selected, uint32_t steps) {
    if (!steps || steps > s.capacity) throw FormatError("mixture rows beyond the scratch capacity");
    encode_rows(g, w, s.rows, input, output, shape, mode, normalize_selected, steps);
}

void encode_verify_nax_moe(CudaGraph& g, const MoeWeights& w, const MoeScratch& s, const VerifyNaxMoeScratch&, GpuView input, GpuView output,
                           MoeShape shape, RouterMode mode, bool normalize_selected, uint32_t steps) {
    if (steps < 2 || steps > 8) throw FormatError("verify batch must hold 2..8 rows");
    encode_rows(g, w, s, input, output, shape, mode, normalize_selected, steps);
}

namespace {
void encode_rows(CudaGraph& g, const MoeWeights& w, const MoeScratch& s, GpuView input, GpuView output, MoeShape shape, RouterMode mode,
                 bool normalize_selected, uint32_t rows) {
    shape_check(shape);
    if (input.bytes != uint64_t(shape.channels) * 4 * rows || output.bytes != uint64_t(shape.channels) * 4 * rows) throw FormatError("mixture shape mismatch");
    if (w.router.encoding != 0 || w.shared_router.encoding != 0) throw FormatError("router projections must be F32");
    tsp_moe_weights tw{};
    if (is_planar_gate_up(g, w, shape)) {
        // co-located pairs: the "gate" tensor holds experts [0, E/2) as [gate_e, up_e], the "up" tensor experts [E/2, E)
        const uint64_t pb = tsp_expert_bytes(w.gate.encoding, TSP_LAYOUT_PLANAR, shape.hidden, shape.channels);
        const auto lo = static_cast<const char*>(g.device_pointer(w.gate.view)), hi = static_cast<const char*>(g.device_pointer(w.up.view));
        tw.gate = {lo, hi, 2 * pb, shape.experts / 2, shape.experts, shape.hidden, shape.channels, w.gate.encoding, TSP_LAYOUT_PLANAR};
        tw.up = {lo + pb, hi + pb, 2 * pb, shape.experts / 2, shape.experts, shape.hidden, shape.channels, w.up.encoding, TSP_LAYOUT_PLANAR};
    } else {
        tw.gate = matrix_set(g, w.gate, shape.hidden, shape.channels, shape.experts);
        tw.up = matrix_set(g, w.up, shape.hidden, shape.channels, shape.experts);
    }
    tw.down = matrix_set(g, w.down, shape.channels, shape.hidden, shape.experts);
    tw.shared_gate = matrix_set(g, w.shared_gate, shape.hidden, shape.channels, 1);
    tw.shared_up = matrix_set(g, w.shared_up, shape.hidden, shape.channels, 1);
    tw.shared_down = matrix_set(g, w.shared_down, shape.channels, shape.hidden, 1);
    tw.d_shared_router = static_cast<const float*>(g.device_pointer(w.shared_router.view));
    if (w.shared_router.view.bytes != uint64_t(shape.channels) * 4) throw FormatError("shared router shape mismatch");

    tsp_moe_scratch ts{};
    ts.d_ids = static_cast<uint32_t*>(g.device_pointer(s.indices, true));
    ts.d_weights = static_cast<float*>(g.device_pointer(s.weights, true));
    ts.d_hidden = static_cast<float*>(g.device_pointer(s.gate, true));
    ts.d_routed = static_cast<float*>(g.device_pointer(s.down, true));
    ts.d_shared_hidden = static_cast<float*>(g.device_pointer(s.shared_gate, true));
    ts.d_shared_out = static_cast<float*>(g.device_pointer(s.shared_down, true));
    ts.d_shared_logit = static_cast<float*>(g.device_pointer(s.shared_logit, true));
    ts.d_token_map = static_cast<uint32_t*>(g.device_pointer(s.token_map, true));
    ts.d_counts = static_cast<uint32_t*>(g.device_pointer(s.counts, true));
    ts.d_tasks = static_cast<uint32_t*>(g.device_pointer(s.tasks, true));
    ts.capacity = rows;
    const uint64_t n = rows;
    if (s.token_map.bytes < n * shape.experts * 4 || s.counts.bytes < uint64_t(shape.experts) * 4 ||
        s.tasks.bytes < tsp_moe_tasks_words(rows, shape.experts, shape.selected, TSP_GEMV_TILE) * 4 ||
        s.gate.bytes < n * shape.hidden * shape.selected * 4 || s.down.bytes < n * shape.channels * shape.selected * 4 ||
        s.logits.bytes < n * shape.experts * 4 || s.indices.bytes < n * shape.selected * 4 || s.weights.bytes < n * shape.selected * 4 ||
        s.shared_gate.bytes < n * shape.hidden * 4 || s.shared_down.bytes < n * shape.channels * 4 || s.shared_logit.bytes < n * 4)
        throw FormatError("mixture scratch too small");

    g.gemv_f32_rows(w.router.view, input, uint64_t(shape.channels) * 4, rows, s.logits, uint64_t(shape.experts) * 4, shape.channels, shape.experts);
    const int rc = tsp_moe_layer_decode(&tw, &ts, g.device_pointer(input), uint64_t(shape.channels) * 4, 0,
                                        static_cast<const float*>(g.device_pointer(s.logits)), uint64_t(shape.experts) * 4, rows, shape.channels,
                                        shape.hidden, shape.experts, shape.selected, uint32_t(mode), normalize_selected,
                                        g.device_pointer(output, true), uint64_t(shape.channels) * 4, 0, g.error_word(), g.stream());
    if (rc != TSP_OK) throw FormatError(tsp_last_error());
    g.count_dispatches(5);   // routing (+ row conversion), permutation + tile table, gate-up, down, combine (the shared expert rides in the routed launches)
}
}  // namespace

}  // namespace tokspur_b200
