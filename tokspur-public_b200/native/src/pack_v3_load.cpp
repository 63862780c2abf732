// One layer's FFN tensors from a "tokspur-pack-v3" container onto a CudaGraph (tensor names and encodings: model.cpp:50-57;
// packed forms: planar_pack_v3.cpp:354-470). Runs between batches; the encoders then use the returned weights as they use any
// registered weights.
#include <cuda_runtime.h>

#include <cstring>

#include "tokspur_b200/moe.hpp"
#include "tokspur_b200/pack_v3.hpp"

namespace tokspur_b200 {
namespace {
void need(bool ok, const char* what) { if (!ok) throw FormatError(what); }

GpuView upload_tensor(CudaGraph& g, const std::filesystem::path& path, const PackIndexV3& index, const PackTensorV3& t) {
    const auto bytes = read_pack_v3_tensor(path, index, t);
    return g.upload(bytes, t.name, true);
}

// a dense 2-D matrix [columns x rows] of the shared expert or a router
GpuMatrix dense(CudaGraph& g, const std::filesystem::path& path, const PackIndexV3& index, const std::string& name, uint64_t columns, uint64_t rows) {
    const auto& t = index.at(name);
    const auto& d = t.source_dimensions;
    const bool vector_ok = rows == 1 && (d == std::vector<uint64_t>{columns} || d == std::vector<uint64_t>{columns, 1});
    need(vector_ok || d == std::vector<uint64_t>{columns, rows}, "pack v3: dense tensor shape does not match the layer");
    if (t.kind == PlanarKind::plain) {
        need(t.bytes == t.source_bytes, "pack v3: plain tensor extent");
        return {upload_tensor(g, path, index, t), t.source_type};
    }
    need(t.kind == PlanarKind::q8_lanes_v1 && t.source_type == TSP_TYPE_Q8_0 && t.bytes == t.source_bytes && columns % 32 == 0 &&
         t.bytes == rows * (columns / 32) * 34, "pack v3: dense tensor in a layout without a kernel here");
    // lane-packed rows -> GGUF rows, once, on the device (the projection kernels read GGUF rows)
    const GpuView packed = upload_tensor(g, path, index, t);
    const GpuView rows_view = g.zeros(t.bytes, t.name + " (rows)");
    const int rc = tsp_q8_lanes_unpack(g.device_pointer(packed), g.device_pointer(rows_view, true), rows, uint32_t(columns), g.stream());
    if (rc != TSP_OK) throw FormatError(tsp_last_error());
    if (cudaStreamSynchronize(static_cast<cudaStream_t>(g.stream())) != cudaSuccess) throw FormatError("pack v3: lane unpack failed on the device");
    g.release(packed);
    return {rows_view, TSP_TYPE_Q8_0};
}
}  // namespace

GpuMatrix load_pack_v3_dense_matrix(CudaGraph& g, const std::filesystem::path& path, const PackIndexV3& index, std::string_view name) {
    const auto& t = index.at(name);
    need(t.source_dimensions.size() == 2 && t.source_dimensions[0] >= 1 && t.source_dimensions[1] >= 1, "pack v3: not a two-dimensional tensor");
    return dense(g, path, index, std::string(name), t.source_dimensions[0], t.source_dimensions[1]);
}

MoeWeights load_pack_v3_moe_layer(CudaGraph& g, const std::filesystem::path& path, const PackIndexV3& index, std::string_view prefix, MoeShape& shape,
                                  PackLoadOptions options) {
    const std::string p(prefix);
    const auto& gate = index.at(p + "ffn_gate_exps.weight");
    const auto& up = index.at(p + "ffn_up_exps.weight");
    const auto& down = index.at(p + "ffn_down_exps.weight");
    need(gate.source_dimensions.size() == 3 && gate.source_dimensions == up.source_dimensions && gate.source_type == up.source_type &&
         down.source_dimensions.size() == 3, "pack v3: expert tensors must be three-dimensional and gate / up alike");
    const uint64_t C = gate.source_dimensions[0], H = gate.source_dimensions[1], E = gate.source_dimensions[2];
    need(down.source_dimensions[0] == H && down.source_dimensions[1] == C && down.source_dimensions[2] == E, "pack v3: down tensor does not match gate / up");
    need(C <= 65536 && H <= 65536 && E >= 1 && E <= 4096, "pack v3: layer shape out of range");
    shape.channels = uint32_t(C); shape.hidden = uint32_t(H); shape.experts = uint32_t(E);

    MoeWeights w{};
    w.router = dense(g, path, index, p + "ffn_gate_inp.weight", C, E);
    w.shared_router = dense(g, path, index, p + "ffn_gate_inp_shexp.weight", C, 1);
    need(w.router.encoding == TSP_TYPE_F32 && w.shared_router.encoding == TSP_TYPE_F32, "pack v3: router projections must be F32");
    w.shared_gate = dense(g, path, index, p + "ffn_gate_shexp.weight", C, H);
    w.shared_up = dense(g, path, index, p + "ffn_up_shexp.weight", C, H);
    w.shared_down = dense(g, path, index, p + "ffn_down_shexp.weight", H, C);

    // gate / up: a co-located pair (two tensors of [gate_e, up_e] expert pairs, planar_pack_v3.cpp:1076-1093) or plain GGUF experts
    const bool coloc_q4 = gate.kind == PlanarKind::q4k_coloc_gate_v3 && up.kind == PlanarKind::q4k_coloc_up_v3;
    const bool coloc_q8 = gate.kind == PlanarKind::q8_coloc_gate_v3 && up.kind == PlanarKind::q8_coloc_up_v3;
    const bool coloc_q5 = gate.kind == PlanarKind::q5k_coloc_gate_v3 && up.kind == PlanarKind::q5k_coloc_up_v3;
    if (coloc_q5) {
        // no planar five-bit kernel: the pair tensors become separate gate / up tensors of plain Q5_K blocks on the host
        need(gate.source_type == TSP_TYPE_Q5_K && gate.partner_name == up.name && up.partner_name == gate.name && gate.bytes == up.bytes &&
             gate.bytes == planar_expert_bytes_v3(TSP_TYPE_Q5_K, C, H) * E, "pack v3: co-located Q5_K pair extent");
        const auto lo = read_pack_v3_tensor(path, index, gate), hi = read_pack_v3_tensor(path, index, up);
        std::vector<std::byte> gg(gguf_expert_bytes_v3(TSP_TYPE_Q5_K, C, H) * E), ug(gg.size());
        split_coloc_pair_v3(TSP_TYPE_Q5_K, C, H, E, lo.data(), hi.data(), gg.data(), ug.data());
        w.gate = {g.upload(gg, gate.name + " (rows)", true), TSP_TYPE_Q5_K};
        w.up = {g.upload(ug, up.name + " (rows)", true), TSP_TYPE_Q5_K};
    } else if (coloc_q4 || coloc_q8) {
        need(gate.partner_name == up.name && up.partner_name == gate.name && gate.bytes == up.bytes, "pack v3: co-located pair does not name its partner");
        w.gate = {upload_tensor(g, path, index, gate), gate.source_type};
        w.up = {upload_tensor(g, path, index, up), up.source_type};
        g.register_planar_matrix(w.gate.view, {gate.source_type, uint32_t(gate.kind), uint32_t(C), uint32_t(H), uint32_t(E)});
        g.register_planar_matrix(w.up.view, {up.source_type, uint32_t(up.kind), uint32_t(C), uint32_t(H), uint32_t(E)});
    } else {
        need(gate.kind == PlanarKind::plain && up.kind == PlanarKind::plain && gate.bytes == gate.source_bytes && up.bytes == up.source_bytes,
             "pack v3: gate / up tensors in a layout without a kernel here");
        w.gate = {upload_tensor(g, path, index, gate), gate.source_type};
        w.up = {upload_tensor(g, path, index, up), up.source_type};
    }
    if ((down.kind == PlanarKind::q8_planar_v3 && options.q8_down_as_rows) || down.kind == PlanarKind::q51_planar_v3) {
        // planar Q8_0 on request, planar Q5_1 always (no planar five-bit kernel): plain GGUF blocks, re-laid on the host
        const uint32_t type = down.kind == PlanarKind::q51_planar_v3 ? TSP_TYPE_Q5_1 : TSP_TYPE_Q8_0;
        need(down.source_type == type && down.bytes == planar_expert_bytes_v3(type, H, C) * E && down.bytes, "pack v3: planar down extent");
        std::vector<std::byte> rows(gguf_expert_bytes_v3(type, H, C) * E);
        unpack_planar_experts_v3(type, H, C, E, read_pack_v3_tensor(path, index, down).data(), rows.data());
        w.down = {g.upload(rows, down.name + " (rows)", true), type};
    } else if (down.kind == PlanarKind::q8_planar_v3) {
        w.down = {upload_tensor(g, path, index, down), down.source_type};
        g.register_planar_matrix(w.down.view, {down.source_type, uint32_t(down.kind), uint32_t(H), uint32_t(C), uint32_t(E)});
    } else {
        need(down.kind == PlanarKind::plain && down.bytes == down.source_bytes, "pack v3: down tensor in a layout without a kernel here");
        w.down = {upload_tensor(g, path, index, down), down.source_type};
    }
    return w;
}

}  // namespace tokspur_b200
