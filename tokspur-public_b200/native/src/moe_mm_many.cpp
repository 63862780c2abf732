// encode_moe_mm_many over the CUDA graph: the reference's composition (native/src/moe_mm_many.cpp:126-220) with everything
// after the router projection forwarded to the C ABI's prefill layer entry point (grouped tcgen05 GEMMs).
#include "tokspur_b200/moe_mm_many.hpp"

#include <algorithm>
#include <utility>

namespace tokspur_b200 {
namespace {
void need(bool ok, const char* what) { if (!ok) throw FormatError(what); }
}

std::array<GpuView, kMoeMmManyViews> MoeMmManyScratch::views() const {
    return {logits, indices, weights, routed, shared_out, shared_logit, token_map, counts, tasks, offsets, xk, xp, hp, s_hp};
}

MoeMmManyBytes moe_mm_many_bytes(MoeShape s, uint32_t capacity) {
    need(s.channels && s.hidden && s.experts && s.selected && s.selected <= 64 && s.selected <= s.experts && capacity, "tiled MoE shape/capacity");
    const uint64_t n = capacity, r = n * s.selected;
    MoeMmManyBytes b;
    // logits, indices, weights, binary16 route rows, FP32 shared-expert rows, gate logits | token_map, counts, tasks, offsets |
    // binary16 input rows in tile K order, their routed copy and the hidden rows in permuted order, the shared expert's hidden rows
    b.views = {n * s.experts * 4, r * 4, r * 4, r * s.channels * 2, n * s.channels * 4, n * 4,
               uint64_t(s.experts) * n * 4, uint64_t(s.experts) * 4, tsp_moe_tasks_words(capacity, s.experts, s.selected, TSP_GROUPED_TILE) * 4,
               (uint64_t(s.experts) + 5) * 4, n * s.channels * 2, r * s.channels * 2, r * s.hidden * 2, n * s.hidden * 2};
    for (const auto v : b.views) b.total += v;
    return b;
}

MoeMmManyScratch allocate_moe_mm_many_scratch(CudaGraph& graph, MoeShape shape, uint32_t capacity) {
    const auto bytes = moe_mm_many_bytes(shape, capacity);
    std::array<GpuView, kMoeMmManyViews> v{};
    size_t made = 0;
    try {
        for (; made < v.size(); ++made) v[made] = graph.zeros(bytes.views[made], "tiled mixture scratch");
    } catch (...) {
        for (size_t i = 0; i < made; ++i) graph.release(v[i]);
        throw;
    }
    return {v[0], v[1], v[2], v[3], v[4], v[5], v[6], v[7], v[8], v[9], v[10], v[11], v[12], v[13], capacity};
}

void release_moe_mm_many_scratch(CudaGraph& graph, const MoeMmManyScratch& scratch) {
    for (const auto view : scratch.views()) graph.release(view);
}

namespace {
constexpr uint64_t kLaunchesPerChunk = 10;   // router GEMM, K-ordered rows, route, routes, tasks, offsets, routed copy, gate-up, down, mixture
// a shared expert that cannot ride in the routed launches adds one launch per projection
uint64_t extra_launches(const tsp_moe_weights& tw) {
    auto same = [](const tsp_matrix_set& a, const tsp_matrix_set& b) { return a.type == b.type && a.layout == b.layout; };
    return (same(tw.shared_gate, tw.gate) && same(tw.shared_up, tw.gate) ? 0u : 1u) + (same(tw.shared_down, tw.down) ? 0u : 1u);
}
tsp_moe_weights checked_weights(const CudaGraph& g, const MoeWeights& w, MoeShape shape, MoeMmLayouts l) {
    // gate and up go through one launch: one identity for the pair (routed, and shared). A shared expert whose encoding or
    // identity differs from the routed experts' gets launches of its own
    need(l.gate == l.up && l.shared_gate == l.shared_up, "tiled MoE: gate and up must be registered in the same layout");
    need(w.router.encoding == 0 && w.shared_router.encoding == 0, "router projections must be F32");
    need(w.router.view.bytes == uint64_t(shape.channels) * shape.experts * 4 && w.shared_router.view.bytes == uint64_t(shape.channels) * 4,
         "router shape mismatch");
    need(w.gate.encoding == TSP_TYPE_Q4_K && w.up.encoding == TSP_TYPE_Q4_K, "tiled MoE reads Q4_K gate / up expert tensors only");
    need(w.down.encoding == TSP_TYPE_Q4_K || (w.down.encoding == TSP_TYPE_Q8_0 && l.down == PrefillWeightLayout::gguf),
         "tiled MoE down experts: Q4_K (planar or raw blocks) or raw Q8_0 blocks");
    need(w.shared_gate.encoding == w.shared_up.encoding, "tiled MoE: shared gate and up must share an encoding");
    for (const auto& [m, layout] : {std::pair{w.shared_gate, l.shared_gate}, std::pair{w.shared_up, l.shared_up}, std::pair{w.shared_down, l.shared_down}})
        need(m.encoding == TSP_TYPE_Q4_K || (m.encoding == TSP_TYPE_Q8_0 && layout == PrefillWeightLayout::gguf),
             "tiled MoE shared expert: Q4_K (planar or raw blocks) or raw Q8_0 blocks");
    // a tensor declared `gguf` must be raw blocks of the layer's extent and must not be a registered planar matrix, one declared
    // `planar` must be registered with the matching shape: the declared identity is checked, never guessed
    auto set = [&](GpuMatrix m, PrefillWeightLayout layout, uint32_t rows, uint32_t cols, uint32_t experts) {
        const bool planar = layout == PrefillWeightLayout::planar;
        need(g.planar_matrix_shape(m.view).has_value() == planar, "tiled MoE explicit registered layout mismatch");
        const uint32_t tl = planar ? TSP_LAYOUT_PLANAR : TSP_LAYOUT_GGUF;
        const uint64_t eb = tsp_expert_bytes(m.encoding, tl, rows, cols);
        need(eb && m.view.bytes == eb * experts, "tiled MoE weight extent");
        return tsp_matrix_set{g.device_pointer(m.view), nullptr, eb, experts, experts, rows, cols, m.encoding, tl};
    };
    tsp_moe_weights tw{};
    if (l.gate == PrefillWeightLayout::planar) {
        // co-located pairs: the "gate" tensor holds experts [0, E/2) as [gate_e, up_e], the "up" tensor experts [E/2, E)
        need(is_planar_gate_up(g, w, shape), "tiled MoE needs the registered co-located gate / up pair tensors");
        const uint64_t pb = tsp_expert_bytes(TSP_TYPE_Q4_K, TSP_LAYOUT_PLANAR, shape.hidden, shape.channels);
        need(pb && shape.experts % 2 == 0, "tiled MoE weight extent");
        const auto lo = static_cast<const char*>(g.device_pointer(w.gate.view)), hi = static_cast<const char*>(g.device_pointer(w.up.view));
        tw.gate = {lo, hi, 2 * pb, shape.experts / 2, shape.experts, shape.hidden, shape.channels, TSP_TYPE_Q4_K, TSP_LAYOUT_PLANAR};
        tw.up = {lo + pb, hi + pb, 2 * pb, shape.experts / 2, shape.experts, shape.hidden, shape.channels, TSP_TYPE_Q4_K, TSP_LAYOUT_PLANAR};
    } else {
        tw.gate = set(w.gate, l.gate, shape.hidden, shape.channels, shape.experts);
        tw.up = set(w.up, l.up, shape.hidden, shape.channels, shape.experts);
    }
    tw.down = set(w.down, l.down, shape.channels, shape.hidden, shape.experts);
    tw.shared_gate = set(w.shared_gate, l.shared_gate, shape.hidden, shape.channels, 1);
    tw.shared_up = set(w.shared_up, l.shared_up, shape.hidden, shape.channels, 1);
    tw.shared_down = set(w.shared_down, l.shared_down, shape.channels, shape.hidden, 1);
    tw.d_shared_router = static_cast<const float*>(g.device_pointer(w.shared_router.view));
    return tw;
}
}  // namespace

void prepare_moe_mm_many(CudaGraph& g, const MoeWeights& w, MoeShape shape, MoeMmLayouts layouts) {
    (void)moe_mm_many_bytes(shape, 1);
    (void)checked_weights(g, w, shape, layouts);
}

uint64_t moe_mm_many_dispatches(const CudaGraph& g, const MoeWeights& w, MoeShape shape, uint32_t rows, uint32_t capacity, MoeMmLayouts layouts) {
    (void)moe_mm_many_bytes(shape, capacity);
    need(rows > 0, "tiled MoE active rows");
    const tsp_moe_weights tw = checked_weights(g, w, shape, layouts);
    return (kLaunchesPerChunk + extra_launches(tw)) * ((uint64_t(rows) + capacity - 1) / capacity);
}

void encode_moe_mm_many(CudaGraph& g, const MoeWeights& w, const MoeMmManyScratch& s, GpuRowsF32 input, GpuRowsF32 output, MoeShape shape,
                        RouterMode mode, bool normalize_selected, MoeMmLayouts layouts) {
    need(s.capacity > 0 && input.rows > 0 && input.rows == output.rows && input.columns == shape.channels && output.columns == shape.channels &&
         uint32_t(mode) <= 1, "tiled MoE active rows/router mode");
    for (const auto r : {input, output})
        need(r.stride_bytes >= uint64_t(shape.channels) * 4 && r.stride_bytes % 16 == 0 &&
             r.view.bytes >= uint64_t(r.rows - 1) * r.stride_bytes + uint64_t(shape.channels) * 4, "tiled MoE strided row extent");
    if (input.rows > s.capacity) {   // longer batches: chunks of `capacity` rows
        for (uint32_t r0 = 0; r0 < input.rows; r0 += s.capacity) {
            const uint32_t n = std::min(s.capacity, input.rows - r0);
            const uint64_t span_in = uint64_t(n - 1) * input.stride_bytes + uint64_t(input.columns) * 4;
            const uint64_t span_out = uint64_t(n - 1) * output.stride_bytes + uint64_t(output.columns) * 4;
            encode_moe_mm_many(g, w, s, {g.slice(input.view, uint64_t(r0) * input.stride_bytes, span_in), n, input.columns, input.stride_bytes},
                               {g.slice(output.view, uint64_t(r0) * output.stride_bytes, span_out), n, output.columns, output.stride_bytes}, shape,
                               mode, normalize_selected, layouts);
        }
        return;
    }
    const auto bytes = moe_mm_many_bytes(shape, s.capacity);
    const auto all = s.views();
    for (size_t i = 0; i < all.size(); ++i) need(all[i].bytes == bytes.views[i], "tiled MoE scratch capacity extent");
    const tsp_moe_weights tw = checked_weights(g, w, shape, layouts);
    auto u32p = [&](GpuView v) { return static_cast<uint32_t*>(g.device_pointer(v, true)); };
    auto f32p = [&](GpuView v) { return static_cast<float*>(g.device_pointer(v, true)); };
    tsp_moe_prefill_scratch ps{};
    ps.base.d_ids = u32p(s.indices); ps.base.d_weights = f32p(s.weights); ps.base.d_routed = f32p(s.routed);
    ps.base.d_shared_out = f32p(s.shared_out); ps.base.d_shared_logit = f32p(s.shared_logit);
    ps.base.d_token_map = u32p(s.token_map); ps.base.d_counts = u32p(s.counts); ps.base.d_tasks = u32p(s.tasks);
    ps.base.capacity = s.capacity;
    ps.d_xk = g.device_pointer(s.xk, true); ps.d_xp = g.device_pointer(s.xp, true); ps.d_hp = g.device_pointer(s.hp, true);
    ps.d_offsets = u32p(s.offsets); ps.d_s_hp = g.device_pointer(s.s_hp, true);

    const uint32_t n = input.rows;
    g.gemv_f32_rows(w.router.view, input.view, input.stride_bytes, n, s.logits, uint64_t(shape.experts) * 4, shape.channels, shape.experts);
    const int rc = tsp_moe_layer_prefill(&tw, &ps, g.device_pointer(input.view), input.stride_bytes, 0, static_cast<const float*>(g.device_pointer(s.logits)),
                                         uint64_t(shape.experts) * 4, n, shape.channels, shape.hidden, shape.experts, shape.selected, uint32_t(mode),
                                         normalize_selected, g.device_pointer(output.view, true), output.stride_bytes, 0, g.error_word(), g.stream());
    if (rc != TSP_OK) throw FormatError(tsp_last_error());
    g.count_dispatches(kLaunchesPerChunk - 1 + extra_launches(tw));   // the router GEMM counted itself
}

}  // namespace tokspur_b200
