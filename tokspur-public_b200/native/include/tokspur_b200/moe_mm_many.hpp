// Prefill-size MoE FFN encoder with the reference's entry points (native/include/tokspur/moe_mm_many.hpp:52-66): caller-owned
// scratch for `capacity` token rows, strided FP32 row batches in and out, encode only. Longer batches are walked in chunks
// of `capacity` rows, as the reference does (moe_mm_many.cpp:133-143).
#pragma once

#include <array>

#include "tokspur_b200/moe.hpp"

namespace tokspur_b200 {


// Registered identity of each weight tensor on the prefill path (native/include/tokspur/moe_mm_many.hpp:7-10). The grouped tensor-core
// GEMMs read Q4_K in both forms: Pack v3 planar (a registered planar matrix; the default here, the faster walk) and raw GGUF
// super-blocks (the reference's default), and a dense shared expert also as raw Q8_0 blocks (the reference model's form,
// moe_mm_many.cpp:236-259). The declared identity must be the tensor's real one (a registered planar matrix declared `gguf`, or
// the reverse, is refused), gate and up share one identity, and nothing is repacked behind the caller's back. A shared expert in
// the routed experts' encoding and identity rides in their launches; otherwise it costs one more launch per projection.
struct MoeMmLayouts {
    PrefillWeightLayout gate = PrefillWeightLayout::planar, up = PrefillWeightLayout::planar, down = PrefillWeightLayout::planar;
    PrefillWeightLayout shared_gate = PrefillWeightLayout::planar, shared_up = PrefillWeightLayout::planar, shared_down = PrefillWeightLayout::planar;
};

constexpr size_t kMoeMmManyViews = 14;
struct MoeMmManyBytes {
    std::array<uint64_t, kMoeMmManyViews> views{};
    uint64_t total = 0;
};
struct MoeMmManyScratch {
    // router logits and routing results of the rows, binary16 route outputs, shared expert output and gate logit
    GpuView logits, indices, weights, routed, shared_out, shared_logit;
    // stable per-expert permutation (tasks of 256 routes) and the first permuted position of every expert
    GpuView token_map, counts, tasks, offsets;
    // binary16 rows: the input rows in tile K order, their routed copy and the hidden rows in permuted position order, and the
    // dense shared expert's hidden rows in row order (it rides in the routed launches)
    GpuView xk, xp, hp, s_hp;
    uint32_t capacity = 0;
    [[nodiscard]] std::array<GpuView, kMoeMmManyViews> views() const;
};
MoeMmManyBytes moe_mm_many_bytes(MoeShape shape, uint32_t capacity);
MoeMmManyScratch allocate_moe_mm_many_scratch(CudaGraph& graph, MoeShape shape, uint32_t capacity);
void release_moe_mm_many_scratch(CudaGraph& graph, const MoeMmManyScratch& scratch);

// Encode only. The caller owns allocation, the batch and the committed state. Gate / up expert tensors must be Q4_K in the declared
// layout (planar: the co-located pair tensors; gguf: raw blocks of the layer's extent), the down experts Q4_K in either layout or
// raw Q8_0 blocks (the reference model's down encoding), the shared expert Q4_K in either layout or raw Q8_0 blocks; anything
// else is refused before the first launch.
void encode_moe_mm_many(CudaGraph& graph, const MoeWeights& weights, const MoeMmManyScratch& scratch, GpuRowsF32 input, GpuRowsF32 output,
                        MoeShape shape, RouterMode mode, bool normalize_selected, MoeMmLayouts layouts = {});
// The weight checks of the encoder, run between batches (prepare_moe_mm_many, moe_mm_many.hpp:59): a tensor of the wrong form or
// extent is refused before the first token instead of in the middle of a prompt.
void prepare_moe_mm_many(CudaGraph& graph, const MoeWeights& weights, MoeShape shape, MoeMmLayouts layouts = {});
// Launches one encode_moe_mm_many of `rows` rows issues with a scratch of `capacity` rows (moe_mm_many_dispatches, moe_mm_many.hpp:60;
// the reference's chunk is fixed, here it is the scratch capacity).
uint64_t moe_mm_many_dispatches(const CudaGraph& graph, const MoeWeights& weights, MoeShape shape, uint32_t rows, uint32_t capacity,
                                MoeMmLayouts layouts = {});

}  // namespace tokspur_b200
