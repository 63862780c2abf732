// CPU checks of the "tokspur-pack-v3" container reader: a small layer written with the test-side writer, read back field by
// field; refusals of damaged files; and, where the reference's own CPU sources were compiled (oracle/_ref), the same file
// bytes parsed by the reference's GGUF reader with the directories compared. No GPU.
#include <dlfcn.h>
#include <unistd.h>

#include <cstring>
#include <functional>
#include <iostream>
#include <stdexcept>

#include "tokspur_b200/graph.hpp"
#include "tokspur_b200/pack_v3.hpp"
#include "tsp_oracle.h"
#include "pack_v3_writer.hpp"

using namespace tokspur_b200;
namespace fs = std::filesystem;

namespace {
int checks = 0;
void require(bool ok, const char* what) { ++checks; if (!ok) throw std::runtime_error(what); }
void refuses(const std::function<void()>& f, const char* what) {
    ++checks;
    try { f(); } catch (const FormatError&) { return; }
    throw std::runtime_error(what);
}
std::vector<uint8_t> blocks(uint32_t type, uint64_t weights, uint32_t seed) {
    const uint32_t epb = (type == 8 || type == 7) ? 32 : 256, bpb = type == 8 ? 34 : type == 7 ? 24 : type == 13 ? 176 : 144;
    std::vector<uint8_t> raw(weights / epb * bpb);
    uint32_t rng = seed;
    for (size_t at = 0; at < raw.size(); at += bpb) {
        for (uint32_t i = 0; i < bpb; ++i) { rng = rng * 1664525u + 1013904223u; raw[at + i] = uint8_t(rng >> 24); }
        raw[at] = 1; raw[at + 1] = 0x0c;
        if (type == 12 || type == 13 || type == 7) { raw[at + 2] = 1; raw[at + 3] = 4; }
    }
    return raw;
}
std::vector<uint8_t> slurp(const fs::path& p) {
    std::ifstream in(p, std::ios::binary);
    return std::vector<uint8_t>((std::istreambuf_iterator<char>(in)), std::istreambuf_iterator<char>());
}
void spit(const fs::path& p, const std::vector<uint8_t>& b) {
    std::ofstream out(p, std::ios::binary | std::ios::trunc);
    out.write(reinterpret_cast<const char*>(b.data()), std::streamsize(b.size()));
}
}  // namespace

int main(int argc, char** argv) {
    try {
        const fs::path dir = fs::temp_directory_path() / ("tokspur_b200_pack_v3_" + std::to_string(::getpid()));
        fs::create_directories(dir);
        const fs::path path = dir / "layer.gguf";
        const uint32_t C = 256, H = 64, E = 4;
        pack_v3_test::LayerBytes L{C, H, E, 12, blocks(12, uint64_t(C) * H * E, 1), blocks(12, uint64_t(C) * H * E, 2), blocks(8, uint64_t(C) * H * E, 3),
                                   blocks(8, uint64_t(C) * H, 4), blocks(8, uint64_t(C) * H, 5), blocks(8, uint64_t(C) * H, 6),
                                   std::vector<float>(size_t(C) * E, 0.25f), std::vector<float>(C, -0.5f)};
        const auto entries = pack_v3_test::layer_entries(L, "blk.7.");
        pack_v3_test::write(path, entries);

        const PackIndexV3 index = read_pack_v3_index(path);
        require(index.version == 3 && index.alignment == 16384 && index.architecture == "tokspur_pack" && index.recipe == "tokspur-pack-v3", "pack identity");
        require(index.tensors.size() == 8 && index.data_offset % 16384 == 0 && index.file_bytes == fs::file_size(path), "directory size / extents");
        uint64_t expected = 0;
        for (size_t i = 0; i < entries.size(); ++i) {
            const auto& t = index.tensors[i];
            const auto& e = entries[i];
            expected = (expected + 16383) / 16384 * 16384;
            require(t.name == e.name && t.type == e.type && t.source_type == e.source_type && t.layout == e.layout && t.dimensions == e.dimensions &&
                    t.source_dimensions == e.source_dimensions && t.source_bytes == e.source_bytes && t.bytes == e.payload.size() && t.offset == expected &&
                    t.partner_name == e.partner_name && planar_kind_name(t.kind) == e.layout, "tensor entry");
            expected += t.bytes;
            const auto back = read_pack_v3_tensor(path, index, t);
            require(back.size() == e.payload.size() && std::memcmp(back.data(), e.payload.data(), back.size()) == 0, "tensor payload");
        }
        // planar Q4_K experts are 148 bytes per super-block against 144: the directory says I8 with the planar row extent
        const auto& gate = index.at("blk.7.ffn_gate_exps.weight");
        require(gate.type == 24 && gate.kind == PlanarKind::q4k_coloc_gate_v3 && gate.dimensions == std::vector<uint64_t>{148, H, E} &&
                gate.bytes == uint64_t(148) * H * E && gate.partner_name == "blk.7.ffn_up_exps.weight", "co-located gate entry");
        require(index.at("blk.7.ffn_down_exps.weight").kind == PlanarKind::q8_planar_v3 && index.at("blk.7.ffn_gate_shexp.weight").kind == PlanarKind::q8_lanes_v1 &&
                index.find("blk.8.ffn_gate_exps.weight") == nullptr, "kinds and lookup");
        refuses([&] { (void)index.at("missing"); }, "lookup of a missing tensor did not throw");
        require(pack_v3_moe_layers(index) == std::vector<std::string>{"blk.7."}, "layer prefixes of the pack");
        {   // several layers, written out of order: ascending layer numbers come back
            auto many = pack_v3_test::layer_entries(L, "blk.12.");
            for (auto& e : pack_v3_test::layer_entries(L, "blk.3.")) many.push_back(e);
            for (auto& e : pack_v3_test::layer_entries(L, "blk.48.")) many.push_back(e);
            const fs::path pm = dir / "layers.gguf";
            pack_v3_test::write(pm, many);
            require(pack_v3_moe_layers(read_pack_v3_index(pm)) == std::vector<std::string>{"blk.3.", "blk.12.", "blk.48."}, "layer order");
        }
        refuses([&] { (void)parse_planar_kind("q4k_planar_v9"); }, "unknown layout string accepted");
        const std::string text = describe_pack_v3(index);
        require(text.find("\"layout\":\"q4k_coloc_up_v3\"") != std::string::npos && text.find("\"alignment\":16384") != std::string::npos, "description text");

        // ---- damaged files ----
        const auto good = slurp(path);
        const fs::path bad = dir / "bad.gguf";
        auto damaged = [&](const std::function<void(std::vector<uint8_t>&)>& edit, const char* what) {
            auto b = good;
            edit(b);
            spit(bad, b);
            refuses([&] { (void)read_pack_v3_index(bad); }, what);
        };
        damaged([](auto& b) { b[0] ^= 1; }, "bad magic accepted");
        damaged([](auto& b) { b[4] = 2; }, "GGUF version 2 accepted");
        damaged([](auto& b) { b.push_back(0); }, "a longer file accepted");
        damaged([](auto& b) { b.resize(b.size() - 1); }, "a shorter file accepted");
        damaged([](auto& b) { b.resize(100); }, "a truncated header accepted");
        auto patch = [&](std::vector<uint8_t>& b, const std::string& from, const std::string& to, size_t nth) {
            size_t at = 0, seen = 0;
            const std::string hay(b.begin(), b.begin() + std::min<size_t>(b.size(), 65536));
            while ((at = hay.find(from, at)) != std::string::npos) { if (seen++ == nth) { std::memcpy(b.data() + at, to.data(), to.size()); return; } ++at; }
            throw std::runtime_error("patch target not found");
        };
        damaged([&](auto& b) { patch(b, "tokspur_pack", "tokspur_pick", 0); }, "foreign architecture accepted");   // the first occurrence is the architecture value
        damaged([&](auto& b) { patch(b, "q8_planar_v3", "q8_planar_v4", 0); }, "unknown layout in the manifest accepted");
        damaged([&](auto& b) { patch(b, "\"offset\":16384", "\"offset\":16385", 0); }, "manifest offset different from the directory accepted");
        damaged([&](auto& b) { patch(b, "blk.7.ffn_up_shexp.weight", "blk.7.ffn_ap_shexp.weight", 0); }, "manifest / directory name mismatch accepted");
        {   // wrong alignment and wrong version in the metadata
            pack_v3_test::write(bad, entries, "tokspur-pack-v3", 4096);
            refuses([&] { (void)read_pack_v3_index(bad); }, "alignment 4096 accepted");
            pack_v3_test::write(bad, entries, "tokspur-pack-v3", 16384, 2);
            refuses([&] { (void)read_pack_v3_index(bad); }, "pack version 2 accepted");
            pack_v3_test::write(bad, entries, "tokspur-pack-v2");
            refuses([&] { (void)read_pack_v3_index(bad); }, "foreign recipe accepted");
            pack_v3_test::write(bad, entries, "tokspur-pack-v3-block-7");   // the reference's per-block recipes share the prefix
            require(read_pack_v3_index(bad).recipe == "tokspur-pack-v3-block-7", "per-block recipe");
        }

        // ---- planar images back to GGUF blocks on the host: every encoding, against the oracle's packer and unpacker ----
        for (const uint32_t type : {12u, 13u, 7u, 8u}) {
            const uint32_t cols = 512, rows = 24, experts = 4;
            const auto src = blocks(type, uint64_t(cols) * rows * experts, 40 + type);
            const auto planar = pack_v3_test::planar_experts(type, src, cols, rows, experts);
            require(planar.size() == planar_expert_bytes_v3(type, cols, rows) * experts && src.size() == gguf_expert_bytes_v3(type, cols, rows) * experts, "planar / GGUF extents");
            std::vector<std::byte> back(src.size());
            unpack_planar_experts_v3(type, cols, rows, experts, reinterpret_cast<const std::byte*>(planar.data()), back.data());
            require(std::memcmp(back.data(), src.data(), src.size()) == 0, "planar experts do not come back as their GGUF blocks");
            tso_planar_spec spec;
            require(tso_make_expert_spec(type, cols, rows, &spec) == TSO_OK, "oracle spec");
            std::vector<uint8_t> want(spec.source_expert_bytes);
            require(tso_unpack_expert_planar(&spec, planar.data() + spec.planar_expert_bytes, want.data()) == TSO_OK &&
                    std::memcmp(reinterpret_cast<const uint8_t*>(back.data()) + spec.source_expert_bytes, want.data(), want.size()) == 0, "differs from the oracle's unpacker");
            if (type != 7) {   // co-located pairs exist for Q4_K, Q5_K and Q8_0
                const auto other = blocks(type, uint64_t(cols) * rows * experts, 50 + type);
                std::vector<uint8_t> lo, hi;
                pack_v3_test::colocate(type, src, other, cols, rows, experts, lo, hi);
                std::vector<std::byte> g2(src.size()), u2(src.size());
                split_coloc_pair_v3(type, cols, rows, experts, reinterpret_cast<const std::byte*>(lo.data()), reinterpret_cast<const std::byte*>(hi.data()), g2.data(), u2.data());
                require(std::memcmp(g2.data(), src.data(), src.size()) == 0 && std::memcmp(u2.data(), other.data(), other.size()) == 0, "co-located pair does not split into its gate and up tensors");
            }
            if (type == 12 || type == 13) {   // a factor byte above 63 in the factor-record plane
                auto bad_planar = planar;
                bad_planar[uint64_t(rows) * (cols / 256) * (type == 13 ? 160 : 128) + 5] |= 0x40;
                refuses([&] { unpack_planar_experts_v3(type, cols, rows, 1, reinterpret_cast<const std::byte*>(bad_planar.data()), back.data()); }, "a factor above 63 was accepted");
            }
        }
        refuses([&] { (void)planar_expert_bytes_v3(5, 256, 8); }, "an encoding without a planar form was accepted");
        require(planar_expert_bytes_v3(12, 300, 8) == 0 && planar_expert_bytes_v3(8, 32, 4) == 0 && planar_expert_bytes_v3(13, 512, 6) == 0, "shapes without a planar form");
        {   // the reference model's other pairing in a pack: co-located Q5_K gate / up, planar Q5_1 down
            pack_v3_test::LayerBytes L5{C, H, E, 13, blocks(13, uint64_t(C) * H * E, 11), blocks(13, uint64_t(C) * H * E, 12), blocks(7, uint64_t(C) * H * E, 13),
                                        blocks(8, uint64_t(C) * H, 14), blocks(8, uint64_t(C) * H, 15), blocks(8, uint64_t(C) * H, 16),
                                        std::vector<float>(size_t(C) * E, 0.5f), std::vector<float>(C, 0.25f), 7};
            const fs::path p5 = dir / "layer5.gguf";
            pack_v3_test::write(p5, pack_v3_test::layer_entries(L5, "blk.0."));
            const PackIndexV3 i5 = read_pack_v3_index(p5);
            const auto& g5 = i5.at("blk.0.ffn_gate_exps.weight");
            const auto& d5 = i5.at("blk.0.ffn_down_exps.weight");
            require(g5.kind == PlanarKind::q5k_coloc_gate_v3 && g5.type == 24 && g5.dimensions == std::vector<uint64_t>{180, H, E} && g5.source_type == 13 &&
                    d5.kind == PlanarKind::q51_planar_v3 && d5.type == 7 && d5.bytes == d5.source_bytes, "five-bit pack entries");
            const auto lo = read_pack_v3_tensor(p5, i5, g5), hi = read_pack_v3_tensor(p5, i5, i5.at("blk.0.ffn_up_exps.weight"));
            std::vector<std::byte> gg(L5.gate.size()), ug(L5.up.size()), dd(L5.down.size());
            split_coloc_pair_v3(13, C, H, E, lo.data(), hi.data(), gg.data(), ug.data());
            unpack_planar_experts_v3(7, H, C, E, read_pack_v3_tensor(p5, i5, d5).data(), dd.data());
            require(std::memcmp(gg.data(), L5.gate.data(), gg.size()) == 0 && std::memcmp(ug.data(), L5.up.data(), ug.size()) == 0 &&
                    std::memcmp(dd.data(), L5.down.data(), dd.size()) == 0, "five-bit pack tensors do not come back as their GGUF blocks");
        }

        // ---- the reference's own GGUF parser on the same bytes ----
        const fs::path here = fs::path(argc > 0 ? argv[0] : ".").parent_path();
        const char* env = std::getenv("TSP_REF_LIB");
        const fs::path lib = env ? fs::path(env) : here / "../../../oracle/_ref/libtokspur_ref.so";
        if (void* h = fs::exists(lib) ? dlopen(lib.c_str(), RTLD_NOW) : nullptr) {
            using Fn = long (*)(const uint8_t*, size_t, char*, size_t);
            const auto fn = reinterpret_cast<Fn>(dlsym(h, "ref_gguf_describe"));
            require(fn != nullptr, "ref_gguf_describe missing from the reference shim");
            std::vector<char> out(1 << 16);
            require(fn(good.data(), good.size(), out.data(), out.size()) > 0, "the reference's GGUF parser refused the written pack");
            std::string want = "16384|3|tokspur_pack|tokspur-pack-v3|" + std::to_string(index.data_offset) + "|";
            const std::string got(out.data());
            require(got.rfind(want, 0) == 0, "pack metadata differ from the reference parser's");
            size_t line = got.find('\n') + 1;
            for (const auto& t : index.tensors) {
                std::string w = t.name + "|" + std::to_string(t.type) + "|" + std::to_string(index.data_offset + t.offset) + "|" + std::to_string(t.bytes) + "|";
                for (size_t i = 0; i < t.dimensions.size(); ++i) w += (i ? "," : "") + std::to_string(t.dimensions[i]);
                const size_t end = got.find('\n', line);
                require(got.substr(line, end - line) == w, "tensor directory differs from the reference parser's");
                line = end + 1;
            }
            std::cout << "reference GGUF parser agrees on " << index.tensors.size() << " tensors\n";
        } else {
            std::cout << "reference shim not present: directory comparison skipped\n";
        }
        fs::remove_all(dir);
        std::cout << "pack v3 reader checks passed: " << checks << "\n";
        return 0;
    } catch (const std::exception& e) {
        std::cerr << "pack v3 reader check failed after " << checks << " checks: " << e.what() << "\n";
        return 1;
    }
}
