// Test-side writer of a "tokspur-pack-v3" container: restates the header and manifest the reference's pack builder emits
// (planar_pack_v3.cpp:103-153, 486-495, 898-920) so that the reader can be exercised without the 80 GiB model pack.
// TEST INFRASTRUCTURE ONLY: nothing in the library writes packs.
#pragma once

#include <cstdint>
#include <filesystem>
#include <fstream>
#include <string>
#include <vector>

namespace pack_v3_test {

struct Entry {
    std::string name;
    uint32_t type, source_type;
    std::string layout;
    std::vector<uint64_t> dimensions, source_dimensions;
    uint64_t source_bytes;
    std::string partner_name;
    std::vector<uint8_t> payload;   // the packed bytes
    uint64_t offset = 0;
};

inline void push_number(std::vector<uint8_t>& b, uint64_t v, unsigned bytes) { for (unsigned i = 0; i < bytes; ++i) b.push_back(uint8_t(v >> (8 * i))); }
inline void push_string(std::vector<uint8_t>& b, const std::string& s) { push_number(b, s.size(), 8); b.insert(b.end(), s.begin(), s.end()); }
inline uint64_t aligned(uint64_t v, uint64_t a = 16384) { return (v + a - 1) / a * a; }

inline std::string manifest(const std::vector<Entry>& tensors, const std::string& recipe) {
    auto dims = [](const std::vector<uint64_t>& d) { std::string s = "["; for (size_t i = 0; i < d.size(); ++i) s += (i ? "," : "") + std::to_string(d[i]); return s + "]"; };
    uint64_t src = 0, packed = 0;
    std::string ts;
    for (size_t i = 0; i < tensors.size(); ++i) {
        const auto& t = tensors[i];
        src += t.source_bytes; packed += t.payload.size();
        ts += std::string(i ? "," : "") + "{\"name\":\"" + t.name + "\",\"type\":" + std::to_string(t.type) + ",\"source_type\":" + std::to_string(t.source_type) +
              ",\"layout\":\"" + t.layout + "\",\"dimensions\":" + dims(t.dimensions) + ",\"source_dimensions\":" + dims(t.source_dimensions) +
              ",\"source_bytes\":" + std::to_string(t.source_bytes) + ",\"bytes\":" + std::to_string(t.payload.size()) + ",\"offset\":" + std::to_string(t.offset) +
              ",\"partner_name\":\"" + t.partner_name + "\",\"source_sha256\":\"" + std::string(64, '0') + "\",\"packed_sha256\":\"" + std::string(64, '0') + "\"}";
    }
    return "{\"schema\":3,\"recipe\":\"" + recipe + "\",\"source_architecture\":\"qwen4exp\",\"target_revision\":\"" + std::string(40, '0') +
           "\",\"mtp_sidecar_sha256\":\"" + std::string(64, '0') + "\",\"source_payload_bytes\":" + std::to_string(src) + ",\"payload_bytes\":" + std::to_string(packed) +
           ",\"tensors\":[" + ts + "]}";
}

// lays the tensors out (16 KiB aligned relative offsets in the given order), builds the header and writes the file
inline void write(const std::filesystem::path& path, std::vector<Entry> tensors, const std::string& recipe = "tokspur-pack-v3", uint32_t alignment = 16384,
                  uint32_t version = 3, const std::string& architecture = "tokspur_pack") {
    uint64_t rel = 0;
    for (auto& t : tensors) { rel = aligned(rel); t.offset = rel; rel += t.payload.size(); }
    std::vector<uint8_t> b;
    push_number(b, 0x46554747, 4);
    push_number(b, 3, 4);
    push_number(b, tensors.size(), 8);
    push_number(b, 5, 8);
    push_string(b, "general.architecture"); push_number(b, 8, 4); push_string(b, architecture);
    push_string(b, "general.alignment"); push_number(b, 4, 4); push_number(b, alignment, 4);
    push_string(b, "tokspur_pack.version"); push_number(b, 4, 4); push_number(b, version, 4);
    push_string(b, "tokspur_pack.recipe"); push_number(b, 8, 4); push_string(b, recipe);
    push_string(b, "tokspur_pack.manifest"); push_number(b, 8, 4); push_string(b, manifest(tensors, recipe));
    for (const auto& t : tensors) {
        push_string(b, t.name);
        push_number(b, t.dimensions.size(), 4);
        for (const uint64_t d : t.dimensions) push_number(b, d, 8);
        push_number(b, t.type, 4);
        push_number(b, t.offset, 8);
    }
    b.resize(aligned(b.size(), 16384), 0);
    std::ofstream out(path, std::ios::binary | std::ios::trunc);
    out.write(reinterpret_cast<const char*>(b.data()), std::streamsize(b.size()));
    uint64_t at = 0;
    for (const auto& t : tensors) {
        const std::vector<char> pad(size_t(t.offset - at), 0);
        out.write(pad.data(), std::streamsize(pad.size()));
        out.write(reinterpret_cast<const char*>(t.payload.data()), std::streamsize(t.payload.size()));
        at = t.offset + t.payload.size();
    }
}

}  // namespace pack_v3_test

// ---- one MoE FFN layer as the reference's pack builder would lay it out (needs the CPU oracle's packers) ----
#ifdef TSP_ORACLE_H
namespace pack_v3_test {

inline std::vector<uint8_t> planar_experts(uint32_t type, const std::vector<uint8_t>& gguf, uint32_t cols, uint32_t rows, uint32_t experts) {
    tso_planar_spec spec;
    if (tso_make_expert_spec(type, cols, rows, &spec) != TSO_OK) throw std::runtime_error("planar spec");
    std::vector<uint8_t> out(spec.planar_expert_bytes * experts);
    for (uint32_t e = 0; e < experts; ++e)
        if (tso_pack_expert_planar(&spec, gguf.data() + e * spec.source_expert_bytes, out.data() + e * spec.planar_expert_bytes) != TSO_OK) throw std::runtime_error("pack");
    return out;
}

// gate / up of Q4_K or Q8_0 experts -> the co-located pair tensors: "gate" = experts [0, E/2) as [gate_e, up_e], "up" = the rest
inline void colocate(uint32_t type, const std::vector<uint8_t>& gate, const std::vector<uint8_t>& up, uint32_t C, uint32_t H, uint32_t E,
                     std::vector<uint8_t>& lo, std::vector<uint8_t>& hi) {
    const auto pg = planar_experts(type, gate, C, H, E), pu = planar_experts(type, up, C, H, E);
    const size_t pb = pg.size() / E;
    lo.assign(pb * E, 0); hi.assign(pb * E, 0);
    for (uint32_t e = 0; e < E; ++e) {
        auto& dst = e < E / 2 ? lo : hi;
        const size_t at = size_t(e % (E / 2)) * 2 * pb;
        std::memcpy(dst.data() + at, pg.data() + e * pb, pb);
        std::memcpy(dst.data() + at + pb, pu.data() + e * pb, pb);
    }
}

struct LayerBytes {   // GGUF bytes of one layer: experts Q4_K, Q5_K or Q8_0 (gate / up), down Q8_0 or Q5_1, shared expert Q8_0, routers F32
    uint32_t C, H, E, gate_type;
    std::vector<uint8_t> gate, up, down, sgate, sup, sdown;
    std::vector<float> router, srouter;
    uint32_t down_type = 8;
};

inline std::vector<Entry> layer_entries(const LayerBytes& L, const std::string& prefix) {
    const uint32_t C = L.C, H = L.H, E = L.E, gt = L.gate_type;
    std::vector<uint8_t> lo, hi;
    colocate(gt, L.gate, L.up, C, H, E, lo, hi);
    const bool expanded = lo.size() != L.gate.size();
    const uint64_t planar_row = lo.size() / E / H;
    const std::vector<uint64_t> gdims{C, H, E}, pdims = expanded ? std::vector<uint64_t>{planar_row, H, E} : gdims;
    const std::string gname = prefix + "ffn_gate_exps.weight", uname = prefix + "ffn_up_exps.weight";
    auto lanes = [&](const std::vector<uint8_t>& m, uint32_t cols) {
        std::vector<uint8_t> out(m.size());
        if (tso_lanes_pack_rows(8, cols, m.data(), out.data(), m.size()) != TSO_OK) throw std::runtime_error("lanes");
        return out;
    };
    auto f32 = [](const std::vector<float>& v) { std::vector<uint8_t> b(v.size() * 4); std::memcpy(b.data(), v.data(), b.size()); return b; };
    const char* gl = gt == 12 ? "q4k_coloc_gate_v3" : gt == 13 ? "q5k_coloc_gate_v3" : "q8_coloc_gate_v3";
    const char* ul = gt == 12 ? "q4k_coloc_up_v3" : gt == 13 ? "q5k_coloc_up_v3" : "q8_coloc_up_v3";
    const uint32_t dt = L.down_type;
    return {
        {prefix + "ffn_gate_inp.weight", 0, 0, "plain", {C, E}, {C, E}, uint64_t(C) * E * 4, "", f32(L.router)},
        {prefix + "ffn_gate_inp_shexp.weight", 0, 0, "plain", {C}, {C}, uint64_t(C) * 4, "", f32(L.srouter)},
        {gname, expanded ? 24u : gt, gt, gl, pdims, gdims, L.gate.size(), uname, lo},
        {uname, expanded ? 24u : gt, gt, ul, pdims, gdims, L.up.size(), gname, hi},
        {prefix + "ffn_down_exps.weight", dt, dt, dt == 7 ? "q51_planar_v3" : "q8_planar_v3", {H, C, E}, {H, C, E}, L.down.size(), "", planar_experts(dt, L.down, H, C, E)},
        {prefix + "ffn_gate_shexp.weight", 8, 8, "q8_lanes_v1", {C, H}, {C, H}, L.sgate.size(), "", lanes(L.sgate, C)},
        {prefix + "ffn_up_shexp.weight", 8, 8, "q8_lanes_v1", {C, H}, {C, H}, L.sup.size(), "", lanes(L.sup, C)},
        {prefix + "ffn_down_shexp.weight", 8, 8, "q8_lanes_v1", {H, C}, {H, C}, L.sdown.size(), "", lanes(L.sdown, H)},
    };
}

}  // namespace pack_v3_test
#endif
