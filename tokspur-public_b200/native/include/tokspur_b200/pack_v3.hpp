// Reader of the reference's weight container "tokspur-pack-v3" (native/include/tokspur/planar_pack_v3.hpp:22-104,
// native/src/planar_pack_v3.cpp:120-153, 502-553, 898-920): a GGUF v3 file whose five metadata keys carry the pack identity
// and a JSON manifest, whose tensor directory gives the packed extents, and whose payload holds every tensor at a 16 KiB
// aligned offset. The index part has no CUDA dependency; load_pack_v3_moe_layer puts one layer's FFN tensors on a CudaGraph
// in the form the MoE encoders take them (registered planar matrices, lane-packed dense Q8_0 matrices unpacked to rows).
#pragma once

#include <cstdint>
#include <filesystem>
#include <string>
#include <string_view>
#include <vector>

namespace tokspur_b200 {

class CudaGraph;
struct MoeWeights;
struct MoeShape;
struct GpuMatrix;

// planar_pack_v3.hpp:29-40; kind 10 is this build's extension (Q4_K down tensors in planar form), never written by the reference
enum class PlanarKind : uint32_t {
    plain = 0, q8_lanes_v1 = 1, q4k_coloc_gate_v3 = 2, q4k_coloc_up_v3 = 3, q5k_coloc_gate_v3 = 4, q5k_coloc_up_v3 = 5,
    q8_coloc_gate_v3 = 6, q8_coloc_up_v3 = 7, q51_planar_v3 = 8, q8_planar_v3 = 9,
};
[[nodiscard]] const char* planar_kind_name(PlanarKind kind);
[[nodiscard]] PlanarKind parse_planar_kind(std::string_view name);   // throws FormatError on an unknown layout string

struct PackTensorV3 {
    std::string name;
    uint32_t type = 0;          // directory type: 24 (I8) when the packed extent differs from the source's, else source_type
    uint32_t source_type = 0;   // original GGUF encoding
    PlanarKind kind = PlanarKind::plain;
    std::string layout;
    std::vector<uint64_t> dimensions, source_dimensions;   // first dimension contiguous
    uint64_t source_bytes = 0, bytes = 0;
    uint64_t offset = 0;        // relative to data_offset, a multiple of the alignment
    std::string partner_name;   // the other tensor of a co-located gate / up pair
    std::string source_sha256, packed_sha256;
};

struct PackIndexV3 {
    uint32_t version = 0, alignment = 0;
    std::string architecture, recipe;
    uint64_t data_offset = 0, payload_bytes = 0, file_bytes = 0;
    std::vector<PackTensorV3> tensors;
    [[nodiscard]] const PackTensorV3* find(std::string_view name) const;
    [[nodiscard]] const PackTensorV3& at(std::string_view name) const;   // throws FormatError when absent
};

// Parses the header of `path` and checks it the way the reference's adopter does: exactly the five metadata keys with their
// types and values ("tokspur_pack", alignment 16384, version 3, the recipe), a manifest entry per directory entry with equal
// name / type / extent / offset, known layout strings, 64-digit digests, offsets aligned and ascending without overlap, and a
// file of exactly data_offset + aligned payload bytes. Throws FormatError; reads nothing but the header.
[[nodiscard]] PackIndexV3 read_pack_v3_index(const std::filesystem::path& path);
// The index as one line of JSON (tests and tools)
[[nodiscard]] std::string describe_pack_v3(const PackIndexV3& index);
// The layer prefixes ("blk.0.", "blk.1.", ...) whose routed-expert tensors the pack holds, in ascending layer order
[[nodiscard]] std::vector<std::string> pack_v3_moe_layers(const PackIndexV3& index);
// The packed bytes of one tensor
[[nodiscard]] std::vector<std::byte> read_pack_v3_tensor(const std::filesystem::path& path, const PackIndexV3& index, const PackTensorV3& tensor);

// Planar expert images back to plain GGUF blocks on the host, lossless (the plane order of planar_pack_v3.cpp:601-650: Q4_K nibbles |
// factor records | (d, dmin); Q5_K nibbles | fifth bits | factor records | (d, dmin); Q5_1 nibbles | fifth-bit words | (d, m);
// Q8_0 codes | scales). `planar` holds `experts` images of planar_expert_bytes_v3() each, `gguf` receives as many of
// gguf_expert_bytes_v3(). A factor record with a value above 63 is refused (FormatError).
[[nodiscard]] uint64_t planar_expert_bytes_v3(uint32_t source_type, uint64_t columns, uint64_t rows);   // 0: no planar form of this shape
[[nodiscard]] uint64_t gguf_expert_bytes_v3(uint32_t source_type, uint64_t columns, uint64_t rows);
void unpack_planar_experts_v3(uint32_t source_type, uint64_t columns, uint64_t rows, uint64_t experts, const std::byte* planar, std::byte* gguf);
// The two tensors of a co-located pair ("gate" = experts [0, E/2) as [gate_e, up_e] images, "up" = the rest; planar_pack_v3.cpp:1076-1093)
// to separate gate and up tensors of E plain GGUF experts each.
void split_coloc_pair_v3(uint32_t source_type, uint64_t columns, uint64_t rows, uint64_t experts, const std::byte* pair_lo, const std::byte* pair_hi,
                         std::byte* gate_gguf, std::byte* up_gguf);

// One layer's FFN tensors (`prefix` + ffn_gate_inp, ffn_gate_inp_shexp, ffn_{gate,up,down}_exps, ffn_{gate,up,down}_shexp,
// model.cpp:50-57) uploaded as immutable buffers of `graph`, between batches: co-located Q4_K / Q8_0 pairs and planar Q8_0 down
// tensors are registered as planar matrices, lane-packed dense Q8_0 matrices are unpacked to GGUF rows on the device, plain
// tensors are taken as they are. The five-bit planar forms (co-located Q5_K pairs, planar Q5_1 down) have no planar kernel here: they
// are re-laid as plain GGUF blocks on the host while loading and then run through the decode-size five-bit kernel. The shape is
// read from the directory. Returns the weights and fills `shape` (selected is left to the caller).
// q8_down_as_rows: a planar Q8_0 down tensor is re-laid as raw GGUF blocks on the host while loading (lossless) instead of being
// registered as a planar matrix: the prefill encoder (encode_moe_mm_many) reads Q8_0 experts as raw blocks only.
struct PackLoadOptions { bool q8_down_as_rows = false; };
// One dense two-dimensional tensor (the vocabulary head `output.weight`, a shared-expert matrix, a router) as the projection
// kernels read it: plain tensors as they are, lane-packed Q8_0 (`q8_lanes_v1`) unpacked to GGUF rows on the device.
GpuMatrix load_pack_v3_dense_matrix(CudaGraph& graph, const std::filesystem::path& path, const PackIndexV3& index, std::string_view name);
MoeWeights load_pack_v3_moe_layer(CudaGraph& graph, const std::filesystem::path& path, const PackIndexV3& index, std::string_view prefix,
                                  MoeShape& shape, PackLoadOptions options = {});

}  // namespace tokspur_b200
