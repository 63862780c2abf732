// MoE FFN sub-layer encoders with the reference's entry points (native/include/tokspur/moe.hpp:9-45): same descriptor
// structs, same argument meaning, same refusal behaviour (FormatError before anything is encoded).
#pragma once

#include <array>

#include "tokspur_b200/graph.hpp"

namespace tokspur_b200 {

struct GpuMatrix { GpuView view; uint32_t encoding; };
struct MoeShape { uint32_t channels, hidden, experts, selected; };
struct MoeWeights {
    GpuMatrix router, gate, up, down, shared_gate, shared_up, shared_down, shared_router;
};
// The reference's ten views plus the three permutation tables its prefill scratch carries (moe_mm_many.hpp:50-55).
struct MoeScratch {
    GpuView logits, indices, weights, gate, up, down, shared_gate, shared_up, shared_down, shared_logit;
    GpuView token_map, counts, tasks;
    [[nodiscard]] std::array<GpuView, 13> views() const;
};

MoeScratch allocate_moe_scratch(CudaGraph& graph, MoeShape shape);
void release_moe_scratch(CudaGraph& graph, const MoeScratch& scratch);

// True when gate/up are registered co-located planar pairs and down a registered planar set of matching shape (moe.hpp:22-35).
[[nodiscard]] bool is_planar_moe(const CudaGraph& g, const MoeWeights& w, MoeShape s);
// The gate / up half of that test alone: the "gate" tensor holds experts [0, E/2) as [gate_e, up_e] pairs, the "up" tensor the rest.
// The encoders address such pairs whatever form the down tensor has (a pack's planar Q8_0 down may be kept as raw rows).
[[nodiscard]] bool is_planar_gate_up(const CudaGraph& g, const MoeWeights& w, MoeShape s);

// One token row: F32 router projection, top-k, routed gate-up + SwiGLU and down, shared expert, gated mixture.
// Neither allocates, reads back nor commits; `input`/`output` are FP32 rows of `channels` values.
void encode_moe(CudaGraph& graph, const MoeWeights& weights, const MoeScratch& scratch, GpuView input, GpuView output,
                MoeShape shape, RouterMode mode, bool normalize_selected);

// Speculative-verify batches (native/include/tokspur/verify_nax.hpp:12-14, 70): `steps` (2..8) token rows, contiguous FP32 rows
// of `channels` values in and out, through the decode kernels: the experts the rows share are read once per tile of 8 routes.
// The scratch is the row scratch for `steps` rows (allocate_moe_rows_scratch); the reference's extra scratch type carries no
// views and is kept for signature parity.
struct VerifyNaxMoeScratch {
    [[nodiscard]] std::array<GpuView, 0> views() const { return {}; }
};
MoeScratch allocate_moe_rows_scratch(CudaGraph& graph, MoeShape shape, uint32_t rows);
void encode_verify_nax_moe(CudaGraph& graph, const MoeWeights& weights, const MoeScratch& scratch, const VerifyNaxMoeScratch& nax_moe,
                           GpuView input, GpuView output, MoeShape shape, RouterMode mode, bool normalize_selected, uint32_t steps);

// Known-input FFN over up to 64 densely packed rows through the decode-size kernels (native/include/tokspur/moe_many.hpp:5-19): the
// scratch is the row scratch for `capacity` rows, encode only; `steps` beyond the capacity or the views is refused.
struct MoeManyScratch {
    MoeScratch rows;
    uint32_t capacity = 0;
};
MoeManyScratch allocate_moe_many_scratch(CudaGraph& graph, MoeShape shape, uint32_t capacity);
void release_moe_many_scratch(CudaGraph& graph, const MoeManyScratch& scratch);
// Checks the weights against the shape between batches, so that a wrong tensor is refused before the first token (prepare_moe_many,
// moe_many.hpp:16). Kernels here need no pipeline objects, so nothing else is prepared.
void prepare_moe_many(CudaGraph& graph, const MoeWeights& weights, MoeShape shape);
// Launches one encode_moe_many of `steps` rows issues (the figure CommandBatch::dispatches grows by)
uint64_t moe_many_dispatches(const CudaGraph& graph, const MoeWeights& weights, MoeShape shape, uint32_t steps);
void encode_moe_many(CudaGraph& graph, const MoeWeights& weights, const MoeManyScratch& scratch, GpuView input, GpuView output, MoeShape shape,
                     RouterMode mode, bool normalize_selected, uint32_t steps);

}  // namespace tokspur_b200
