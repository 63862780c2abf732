// Index reader of the "tokspur-pack-v3" container: GGUF v3 header, five metadata keys, JSON manifest, tensor directory.
// Restates what the reference's writer emits (planar_pack_v3.cpp:103-153, 898-920) and what its adopter checks
// (planar_pack_v3.cpp:502-553). No CUDA in this file.
#include "tokspur_b200/pack_v3.hpp"

#include <algorithm>
#include <cstring>
#include <fstream>
#include <map>
#include <memory>
#include <variant>

#include "tokspur_b200/graph.hpp"   // FormatError

namespace tokspur_b200 {
namespace {

constexpr uint64_t kMaxHeaderBytes = 64ull << 20;   // bound on what is read before the directory is known
constexpr uint32_t kPackAlignment = 16384;          // derived_pack.hpp:18
constexpr uint32_t kPackVersion = 3;                // planar_pack_v3.hpp:24
constexpr const char* kPackArchitecture = "tokspur_pack";
constexpr const char* kRecipePrefix = "tokspur-pack-v3";

void need(bool ok, const char* what) { if (!ok) throw FormatError(what); }
uint64_t aligned(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }

// ---- bounded little-endian reader over the header bytes ----
struct Cursor {
    const unsigned char* p; size_t n, at = 0;
    uint64_t number(unsigned bytes) {
        need(bytes <= n - at && at <= n, "pack v3 header truncated");
        uint64_t v = 0;
        for (unsigned i = 0; i < bytes; ++i) v |= uint64_t(p[at + i]) << (8 * i);
        at += bytes;
        return v;
    }
    std::string string() {
        const uint64_t len = number(8);
        need(len <= n - at, "pack v3 header string runs past the header");
        std::string s(reinterpret_cast<const char*>(p + at), size_t(len));
        at += size_t(len);
        return s;
    }
};

// ---- a small JSON reader: objects, arrays, strings, non-negative integers (all the manifest uses), true / false / null ----
struct Json;
using JsonObject = std::vector<std::pair<std::string, Json>>;
using JsonArray = std::vector<Json>;
struct Json {
    std::variant<std::nullptr_t, bool, uint64_t, std::string, std::shared_ptr<JsonArray>, std::shared_ptr<JsonObject>> v;
    const Json* find(std::string_view key) const {
        const auto* o = std::get_if<std::shared_ptr<JsonObject>>(&v);
        if (!o) return nullptr;
        for (const auto& [k, val] : **o) if (k == key) return &val;
        return nullptr;
    }
    const std::string& str() const { const auto* s = std::get_if<std::string>(&v); need(s, "pack v3 manifest: string expected"); return *s; }
    uint64_t num() const { const auto* u = std::get_if<uint64_t>(&v); need(u, "pack v3 manifest: unsigned integer expected"); return *u; }
    const JsonArray& arr() const { const auto* a = std::get_if<std::shared_ptr<JsonArray>>(&v); need(a, "pack v3 manifest: array expected"); return **a; }
};
struct JsonParser {
    std::string_view s; size_t at = 0; int depth = 0;
    void ws() { while (at < s.size() && (s[at] == ' ' || s[at] == '\n' || s[at] == '\t' || s[at] == '\r')) ++at; }
    char peek() { ws(); need(at < s.size(), "pack v3 manifest: unexpected end"); return s[at]; }
    void expect(char c) { need(peek() == c, "pack v3 manifest: malformed JSON"); ++at; }
    std::string string() {
        expect('"');
        std::string out;
        while (true) {
            need(at < s.size(), "pack v3 manifest: unterminated string");
            const char c = s[at++];
            if (c == '"') return out;
            if (c != '\\') { out.push_back(c); continue; }
            need(at < s.size(), "pack v3 manifest: unterminated escape");
            const char e = s[at++];
            if (e == '"' || e == '\\' || e == '/') out.push_back(e);
            else if (e == 'n') out.push_back('\n');
            else if (e == 't') out.push_back('\t');
            else if (e == 'r') out.push_back('\r');
            else if (e == 'b') out.push_back('\b');
            else if (e == 'f') out.push_back('\f');
            else if (e == 'u') {
                need(at + 4 <= s.size(), "pack v3 manifest: short \\u escape");
                unsigned code = 0;
                for (int i = 0; i < 4; ++i) {
                    const char h = s[at++];
                    code = code * 16 + (h >= '0' && h <= '9' ? h - '0' : h >= 'a' && h <= 'f' ? h - 'a' + 10 : h >= 'A' && h <= 'F' ? h - 'A' + 10 : 99);
                    need(code < 0x10000, "pack v3 manifest: bad \\u escape");
                }
                need(code < 0x80, "pack v3 manifest: only ASCII escapes occur in a pack manifest");
                out.push_back(char(code));
            } else need(false, "pack v3 manifest: unknown escape");
        }
    }
    Json value() {
        need(++depth <= 16, "pack v3 manifest: nesting too deep");
        Json j;
        const char c = peek();
        if (c == '{') {
            ++at;
            auto o = std::make_shared<JsonObject>();
            if (peek() == '}') ++at;
            else while (true) {
                std::string k = (ws(), string());
                expect(':');
                o->emplace_back(std::move(k), value());
                if (peek() == ',') { ++at; continue; }
                expect('}');
                break;
            }
            j.v = std::move(o);
        } else if (c == '[') {
            ++at;
            auto a = std::make_shared<JsonArray>();
            if (peek() == ']') ++at;
            else while (true) {
                a->push_back(value());
                if (peek() == ',') { ++at; continue; }
                expect(']');
                break;
            }
            j.v = std::move(a);
        } else if (c == '"') j.v = string();
        else if (c >= '0' && c <= '9') {
            uint64_t n = 0;
            while (at < s.size() && s[at] >= '0' && s[at] <= '9') {
                need(n <= (UINT64_MAX - uint64_t(s[at] - '0')) / 10, "pack v3 manifest: integer overflow");
                n = n * 10 + uint64_t(s[at++] - '0');
            }
            need(at >= s.size() || (s[at] != '.' && s[at] != 'e' && s[at] != 'E'), "pack v3 manifest: only integers occur in a pack manifest");
            j.v = n;
        } else if (s.substr(at, 4) == "true") { at += 4; j.v = true; }
        else if (s.substr(at, 5) == "false") { at += 5; j.v = false; }
        else if (s.substr(at, 4) == "null") { at += 4; j.v = nullptr; }
        else need(false, "pack v3 manifest: malformed JSON value");
        --depth;
        return j;
    }
};

std::vector<uint64_t> dims_of(const Json* a) {
    need(a != nullptr, "pack v3 manifest tensor dimensions missing");
    std::vector<uint64_t> out;
    for (const auto& d : a->arr()) out.push_back(d.num());
    need(!out.empty() && out.size() <= 4, "pack v3 manifest tensor dimensions missing");
    return out;
}

void escape_into(std::string& out, std::string_view s) {
    out.push_back('"');
    for (const char c : s) { if (c == '"' || c == '\\') out.push_back('\\'); out.push_back(c); }
    out.push_back('"');
}

}  // namespace

const char* planar_kind_name(PlanarKind kind) {
    switch (kind) {
        case PlanarKind::plain: return "plain";
        case PlanarKind::q8_lanes_v1: return "q8_lanes_v1";
        case PlanarKind::q4k_coloc_gate_v3: return "q4k_coloc_gate_v3";
        case PlanarKind::q4k_coloc_up_v3: return "q4k_coloc_up_v3";
        case PlanarKind::q5k_coloc_gate_v3: return "q5k_coloc_gate_v3";
        case PlanarKind::q5k_coloc_up_v3: return "q5k_coloc_up_v3";
        case PlanarKind::q8_coloc_gate_v3: return "q8_coloc_gate_v3";
        case PlanarKind::q8_coloc_up_v3: return "q8_coloc_up_v3";
        case PlanarKind::q51_planar_v3: return "q51_planar_v3";
        case PlanarKind::q8_planar_v3: return "q8_planar_v3";
    }
    throw FormatError("unknown PlanarKind");
}

PlanarKind parse_planar_kind(std::string_view name) {
    for (uint32_t k = 0; k <= 9; ++k)
        if (name == planar_kind_name(PlanarKind(k))) return PlanarKind(k);
    throw FormatError("unrecognised planar v3 layout string: " + std::string(name));
}

namespace {
struct PlaneSpec { uint32_t per_block, block_bytes, planar_bytes, qs, qh, sm, dm; };   // weights per block; bytes per GGUF / planar block; plane widths
PlaneSpec plane_spec(uint32_t type) {
    switch (type) {
        case 12: return {256, 144, 148, 128, 0, 16, 4};
        case 13: return {256, 176, 180, 128, 32, 16, 4};
        case 7: return {32, 24, 24, 16, 4, 0, 4};
        case 8: return {32, 34, 34, 32, 0, 0, 2};
        default: throw FormatError("pack v3: encoding without a planar form");
    }
}
// sixteen factor bytes sc[0..7], mn[0..7] -> the twelve packed bytes of a K-quant header (numeric.cpp:25-31 read the other way)
void factors_to_packed(const unsigned char* sm, unsigned char* s12) {
    for (int i = 0; i < 16; ++i) need((sm[i] & 0xc0u) == 0, "corrupt planar v3 scale/min factor exceeds 6 bits");
    for (int k = 0; k < 4; ++k) {
        s12[k] = (unsigned char)(sm[k] | ((sm[4 + k] >> 4) << 6));
        s12[4 + k] = (unsigned char)(sm[8 + k] | ((sm[12 + k] >> 4) << 6));
        s12[8 + k] = (unsigned char)((sm[4 + k] & 15u) | ((sm[12 + k] & 15u) << 4));
    }
}
}  // namespace

uint64_t gguf_expert_bytes_v3(uint32_t type, uint64_t columns, uint64_t rows) {
    const PlaneSpec s = plane_spec(type);
    return columns % s.per_block ? 0 : rows * (columns / s.per_block) * s.block_bytes;
}
uint64_t planar_expert_bytes_v3(uint32_t type, uint64_t columns, uint64_t rows) {
    const PlaneSpec s = plane_spec(type);
    if (!columns || columns % s.per_block || rows < 4 || rows % 4) return 0;
    const uint64_t blocks = rows * (columns / s.per_block);
    if (type == 8 && blocks % 8) return 0;
    const uint64_t bytes = blocks * s.planar_bytes;
    return bytes % 16 ? 0 : bytes;
}

void unpack_planar_experts_v3(uint32_t type, uint64_t columns, uint64_t rows, uint64_t experts, const std::byte* planar, std::byte* gguf) {
    const PlaneSpec s = plane_spec(type);
    const uint64_t pb = planar_expert_bytes_v3(type, columns, rows), gb = gguf_expert_bytes_v3(type, columns, rows);
    need(pb && gb, "pack v3: shape without a planar form");
    const uint64_t n = rows * (columns / s.per_block);
    const uint64_t at_qh = n * s.qs, at_sm = at_qh + n * s.qh, at_dm = at_sm + n * s.sm;   // planes follow one another
    for (uint64_t e = 0; e < experts; ++e) {
        const auto* src = reinterpret_cast<const unsigned char*>(planar) + e * pb;
        auto* dst = reinterpret_cast<unsigned char*>(gguf) + e * gb;
        for (uint64_t b = 0; b < n; ++b) {
            unsigned char* blk = dst + b * s.block_bytes;
            std::memcpy(blk, src + at_dm + b * s.dm, s.dm);                       // scales first in every GGUF block
            if (type == 12 || type == 13) {
                factors_to_packed(src + at_sm + b * 16, blk + 4);
                if (type == 13) std::memcpy(blk + 16, src + at_qh + b * 32, 32);
                std::memcpy(blk + (type == 13 ? 48 : 16), src + b * 128, 128);
            } else if (type == 7) {
                std::memcpy(blk + 4, src + at_qh + b * 4, 4);
                std::memcpy(blk + 8, src + b * 16, 16);
            } else {
                std::memcpy(blk + 2, src + b * 32, 32);
            }
        }
    }
}

void split_coloc_pair_v3(uint32_t type, uint64_t columns, uint64_t rows, uint64_t experts, const std::byte* pair_lo, const std::byte* pair_hi,
                         std::byte* gate_gguf, std::byte* up_gguf) {
    need(experts >= 2 && experts % 2 == 0, "pack v3: a co-located pair holds an even number of experts");
    const uint64_t pb = planar_expert_bytes_v3(type, columns, rows), gb = gguf_expert_bytes_v3(type, columns, rows);
    need(pb && gb, "pack v3: shape without a planar form");
    for (uint64_t e = 0; e < experts; ++e) {
        const std::byte* pair = (e < experts / 2 ? pair_lo : pair_hi) + (e % (experts / 2)) * 2 * pb;
        unpack_planar_experts_v3(type, columns, rows, 1, pair, gate_gguf + e * gb);
        unpack_planar_experts_v3(type, columns, rows, 1, pair + pb, up_gguf + e * gb);
    }
}

const PackTensorV3* PackIndexV3::find(std::string_view name) const {
    for (const auto& t : tensors) if (t.name == name) return &t;
    return nullptr;
}
const PackTensorV3& PackIndexV3::at(std::string_view name) const {
    const auto* t = find(name);
    if (!t) throw FormatError("pack v3: no tensor named " + std::string(name));
    return *t;
}

PackIndexV3 read_pack_v3_index(const std::filesystem::path& path) {
    std::error_code ec;
    const uint64_t file_bytes = std::filesystem::file_size(path, ec);
    need(!ec, "pack v3: cannot stat the file");
    std::ifstream in(path, std::ios::binary);
    need(bool(in), "pack v3: cannot open the file");
    std::vector<unsigned char> head(size_t(std::min<uint64_t>(file_bytes, kMaxHeaderBytes)));
    in.read(reinterpret_cast<char*>(head.data()), std::streamsize(head.size()));
    need(size_t(in.gcount()) == head.size(), "pack v3: short read");

    Cursor c{head.data(), head.size()};
    need(c.number(4) == 0x46554747u, "pack v3: not a GGUF file");
    need(c.number(4) == 3, "pack v3: GGUF version 3 expected");
    const uint64_t n_tensors = c.number(8), n_meta = c.number(8);
    need(n_meta == 5, "unexpected metadata entries in pack v3 GGUF");
    need(n_tensors >= 1 && n_tensors <= 1u << 20, "pack v3: tensor count out of range");

    PackIndexV3 index;
    std::string manifest;
    std::map<std::string, int> seen;
    for (uint64_t i = 0; i < n_meta; ++i) {
        const std::string key = c.string();
        const uint64_t type = c.number(4);
        need(++seen[key] == 1, "pack v3: duplicate metadata key");
        if (key == "general.architecture") { need(type == 8, "wrong pack v3 GGUF metadata type"); index.architecture = c.string(); }
        else if (key == "general.alignment") { need(type == 4, "wrong pack v3 GGUF metadata type"); index.alignment = uint32_t(c.number(4)); }
        else if (key == "tokspur_pack.version") { need(type == 4, "wrong pack v3 GGUF metadata type"); index.version = uint32_t(c.number(4)); }
        else if (key == "tokspur_pack.recipe") { need(type == 8, "wrong pack v3 GGUF metadata type"); index.recipe = c.string(); }
        else if (key == "tokspur_pack.manifest") { need(type == 8, "wrong pack v3 GGUF metadata type"); manifest = c.string(); }
        else need(false, "unexpected metadata entries in pack v3 GGUF");
    }
    need(index.architecture == kPackArchitecture && index.alignment == kPackAlignment && index.version == kPackVersion &&
         index.recipe.rfind(kRecipePrefix, 0) == 0, "stale or incompatible pack v3 metadata");

    index.tensors.resize(size_t(n_tensors));
    for (auto& t : index.tensors) {
        t.name = c.string();
        need(!t.name.empty() && t.name.size() <= 1024, "pack v3: tensor name length");
        const uint64_t nd = c.number(4);
        need(nd >= 1 && nd <= 4, "pack v3: tensor rank");
        for (uint64_t d = 0; d < nd; ++d) t.dimensions.push_back(c.number(8));
        t.type = uint32_t(c.number(4));
        t.offset = c.number(8);
    }
    index.data_offset = aligned(c.at, index.alignment);

    JsonParser jp{manifest};
    const Json root = jp.value();
    jp.ws();
    need(jp.at == manifest.size(), "pack v3 manifest: trailing bytes");
    const Json* schema = root.find("schema");
    need(schema && schema->num() == index.version, "pack v3 manifest schema mismatch");
    const Json* recipe = root.find("recipe");
    need(recipe && recipe->str() == index.recipe, "pack v3 manifest recipe mismatch");
    const Json* entries = root.find("tensors");
    need(entries && entries->arr().size() == index.tensors.size(), "pack v3 manifest tensor count mismatch");
    uint64_t expected_offset = 0;
    for (size_t i = 0; i < index.tensors.size(); ++i) {
        auto& t = index.tensors[i];
        const Json& e = entries->arr()[i];
        const Json *name = e.find("name"), *type = e.find("type"), *src_type = e.find("source_type"), *layout = e.find("layout"),
                   *src_bytes = e.find("source_bytes"), *bytes = e.find("bytes"), *offset = e.find("offset"), *partner = e.find("partner_name"),
                   *sh = e.find("source_sha256"), *ph = e.find("packed_sha256");
        need(name && name->str() == t.name, "pack v3 manifest tensor name mismatch");
        need(type && type->num() == t.type, "pack v3 manifest tensor type mismatch");
        need(src_type && layout && src_bytes && bytes, "incomplete pack v3 tensor manifest entry");
        need(offset && offset->num() == t.offset, "pack v3 manifest offset mismatch");
        need(sh && ph && sh->str().size() == 64 && ph->str().size() == 64, "pack v3 manifest missing SHA-256 digests");
        need(dims_of(e.find("dimensions")) == t.dimensions, "pack v3 manifest tensor dimensions mismatch");
        t.source_type = uint32_t(src_type->num());
        t.layout = layout->str();
        t.kind = parse_planar_kind(t.layout);
        t.source_dimensions = dims_of(e.find("source_dimensions"));
        t.source_bytes = src_bytes->num();
        t.bytes = bytes->num();
        t.partner_name = partner ? partner->str() : std::string();
        t.source_sha256 = sh->str();
        t.packed_sha256 = ph->str();
        // the directory type is I8 (24) exactly when the packed extent differs from the source's (planar_pack_v3.cpp:375-379)
        need(t.type == (t.bytes != t.source_bytes ? 24u : t.source_type), "pack v3 directory type does not match the packed extent");
        need(t.bytes >= 1 && t.offset == aligned(expected_offset, index.alignment), "pack v3 tensor offsets must be aligned, ascending and gap-free");
        expected_offset = t.offset + t.bytes;
        need(expected_offset >= t.offset, "pack v3 tensor extent overflow");
    }
    index.payload_bytes = expected_offset;
    index.file_bytes = index.data_offset + expected_offset;
    need(index.file_bytes == file_bytes, "pack v3 must be a file of exactly the planned size");
    const Json* payload = root.find("payload_bytes");
    uint64_t sum = 0;
    for (const auto& t : index.tensors) sum += t.bytes;
    need(payload && payload->num() == sum, "pack v3 manifest payload_bytes mismatch");
    return index;
}

std::vector<std::string> pack_v3_moe_layers(const PackIndexV3& index) {
    constexpr std::string_view prefix = "blk.", suffix = ".ffn_gate_exps.weight";
    std::vector<std::pair<uint64_t, std::string>> found;
    for (const auto& t : index.tensors) {
        const std::string_view n = t.name;
        if (n.size() <= prefix.size() + suffix.size() || n.substr(0, prefix.size()) != prefix || n.substr(n.size() - suffix.size()) != suffix) continue;
        const std::string_view digits = n.substr(prefix.size(), n.size() - prefix.size() - suffix.size());
        if (digits.empty() || digits.size() > 6 || !std::all_of(digits.begin(), digits.end(), [](char ch) { return ch >= '0' && ch <= '9'; })) continue;
        found.emplace_back(std::stoull(std::string(digits)), std::string(n.substr(0, n.size() - suffix.size() + 1)));
    }
    std::sort(found.begin(), found.end());
    std::vector<std::string> out;
    for (auto& f : found) out.push_back(std::move(f.second));
    return out;
}

std::string describe_pack_v3(const PackIndexV3& index) {
    std::string out = "{\"version\":" + std::to_string(index.version) + ",\"alignment\":" + std::to_string(index.alignment) + ",\"architecture\":";
    escape_into(out, index.architecture);
    out += ",\"recipe\":";
    escape_into(out, index.recipe);
    out += ",\"data_offset\":" + std::to_string(index.data_offset) + ",\"file_bytes\":" + std::to_string(index.file_bytes) + ",\"tensors\":[";
    for (size_t i = 0; i < index.tensors.size(); ++i) {
        const auto& t = index.tensors[i];
        if (i) out += ",";
        out += "{\"name\":";
        escape_into(out, t.name);
        out += ",\"type\":" + std::to_string(t.type) + ",\"source_type\":" + std::to_string(t.source_type) + ",\"layout\":";
        escape_into(out, t.layout);
        out += ",\"dimensions\":[";
        for (size_t d = 0; d < t.dimensions.size(); ++d) out += (d ? "," : "") + std::to_string(t.dimensions[d]);
        out += "],\"source_dimensions\":[";
        for (size_t d = 0; d < t.source_dimensions.size(); ++d) out += (d ? "," : "") + std::to_string(t.source_dimensions[d]);
        out += "],\"source_bytes\":" + std::to_string(t.source_bytes) + ",\"bytes\":" + std::to_string(t.bytes) + ",\"offset\":" + std::to_string(t.offset) +
               ",\"absolute_offset\":" + std::to_string(index.data_offset + t.offset) + ",\"partner_name\":";
        escape_into(out, t.partner_name);
        out += "}";
    }
    return out + "]}";
}

std::vector<std::byte> read_pack_v3_tensor(const std::filesystem::path& path, const PackIndexV3& index, const PackTensorV3& tensor) {
    need(index.data_offset + tensor.offset + tensor.bytes <= index.file_bytes, "pack v3 tensor extent beyond the file");
    std::ifstream in(path, std::ios::binary);
    need(bool(in), "pack v3: cannot open the file");
    in.seekg(std::streamoff(index.data_offset + tensor.offset));
    std::vector<std::byte> out(size_t(tensor.bytes));
    in.read(reinterpret_cast<char*>(out.data()), std::streamsize(out.size()));
    need(size_t(in.gcount()) == out.size(), "pack v3: short tensor read");
    return out;
}

}  // namespace tokspur_b200

// C entry for tools and tests that have no C++: the index of `path` as JSON text. Returns the text length (the text is cut
// to cap - 1 bytes), or -1 with the refusal message in `out`.
extern "C" long tokspur_b200_pack_v3_describe(const char* path, char* out, unsigned long cap) {
    auto put = [&](const std::string& s) {
        if (out && cap) { const size_t n = std::min<size_t>(s.size(), cap - 1); std::memcpy(out, s.data(), n); out[n] = 0; }
    };
    try {
        const std::string text = tokspur_b200::describe_pack_v3(tokspur_b200::read_pack_v3_index(path));
        put(text);
        return long(text.size());
    } catch (const std::exception& e) {
        put(e.what());
        return -1;
    }
}
