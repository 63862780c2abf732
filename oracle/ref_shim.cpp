// C entry points over the reference's own CPU sources, compiled where they lie in the
// read-only reference tree (see oracle/Makefile). TEST INFRASTRUCTURE ONLY: used to
// validate the plain-C restatement in tsp_oracle.c, to generate the golden fixtures
// under tests/golden/, and as the timed "reference" CPU arm of the benchmark.
// Nothing here is reference source: it only calls the reference's public functions.
#include "tokspur/expert_lanes.hpp"
#include "tokspur/gguf.hpp"
#include "tokspur/numeric.hpp"
#include "tokspur/operators.hpp"
#include "tokspur/routing.hpp"

#include <cstring>
#include <string>
#include <thread>
#include <vector>

using namespace tokspur;

namespace {
template <class F> int guarded(F&& f) {
    try { f(); return 0; }
    catch (const FormatError&) { return -1; }
    catch (...) { return -2; }
}
std::span<const std::byte> bytes(const uint8_t* p, size_t n) { return {reinterpret_cast<const std::byte*>(p), n}; }
size_t tensor_bytes(uint32_t type, uint64_t elements) {
    const auto& e = encoding(type);
    return size_t(elements / e.elements_per_block) * e.bytes_per_block;
}
}

extern "C" {

float ref_binary16(uint16_t bits) { return binary16(bits); }

int ref_dequantize(uint32_t type, const uint8_t* data, size_t nbytes, float* out, size_t elements) {
    return guarded([&] { dequantize(type, bytes(data, nbytes), std::span<float>(out, elements)); });
}

int ref_gemv_f64(uint32_t type, const uint8_t* matrix, size_t nbytes, uint32_t columns, uint32_t rows,
                 const double* input, double* output) {
    return guarded([&] {
        const auto r = reference_gemv_doubleinput(type, bytes(matrix, nbytes), columns, rows, std::span<const double>(input, columns));
        std::memcpy(output, r.data(), sizeof(double) * rows);
    });
}

int ref_gemv_f32(uint32_t type, const uint8_t* matrix, size_t nbytes, uint32_t columns, uint32_t rows,
                 const float* input, double* output) {
    return guarded([&] {
        const auto r = reference_gemv(type, bytes(matrix, nbytes), columns, rows, std::span<const float>(input, columns));
        std::memcpy(output, r.data(), sizeof(double) * rows);
    });
}

int ref_lanes_pack_rows(uint32_t type, uint32_t columns, const uint8_t* original, uint8_t* packed, size_t nbytes) {
    return guarded([&] { lanes::pack_rows(lanes::row_layout(type, columns), bytes(original, nbytes), {reinterpret_cast<std::byte*>(packed), nbytes}); });
}
int ref_lanes_unpack_rows(uint32_t type, uint32_t columns, const uint8_t* packed, uint8_t* original, size_t nbytes) {
    return guarded([&] { lanes::unpack_rows(lanes::row_layout(type, columns), bytes(packed, nbytes), {reinterpret_cast<std::byte*>(original), nbytes}); });
}

double ref_sigmoid(double v) { return stable_sigmoid(v); }
double ref_silu(double v) { return stable_silu(v); }
double ref_softplus(double v) { return stable_softplus(v); }

int ref_route(const double* logits, size_t experts, size_t selected, uint32_t mode, int normalize,
              uint32_t* indices, double* weights) {
    return guarded([&] {
        const auto r = route_reference(std::span<const double>(logits, experts), selected, static_cast<RouterMode>(mode), normalize != 0);
        std::memcpy(indices, r.indices.data(), 4 * selected);
        std::memcpy(weights, r.weights.data(), sizeof(double) * selected);
    });
}

int ref_mixture(const double* experts, const double* weights, size_t selected, const double* shared,
                size_t channels, double shared_logit, double* out) {
    return guarded([&] {
        const auto r = mixture_reference(std::span<const double>(experts, selected * channels), std::span<const double>(weights, selected),
                                         std::span<const double>(shared, channels), shared_logit);
        std::memcpy(out, r.data(), sizeof(double) * channels);
    });
}

// One MoE FFN layer composed from the reference functions in the order its ffn-check tool uses:
// route, per selected expert gate/up -> silu*up -> down, shared expert, shared gate logit, mixture.
struct RefLayer {
    uint32_t channels, hidden, experts, selected, expert_type, shared_type;
    const uint8_t *gate, *up, *down, *shared_gate, *shared_up, *shared_down;
    const float* shared_router;
    const float* router;
    uint32_t mode;
    int normalize_selected;
    uint32_t down_type;   // 0: expert_type
};

int ref_moe_layer(const RefLayer* L, const float* x, const float* logits, uint32_t tokens, double* out,
                  uint32_t* indices_out, uint32_t threads) {
    if (!threads) threads = 1;
    if (threads > tokens) threads = tokens;
    std::vector<int> rcs(threads, 0);
    const uint32_t C = L->channels, H = L->hidden, E = L->experts, K = L->selected;
    const size_t eb = tensor_bytes(L->expert_type, uint64_t(C) * H), sb = tensor_bytes(L->shared_type, uint64_t(C) * H);
    const uint32_t down_type = L->down_type ? L->down_type : L->expert_type;
    const size_t db = tensor_bytes(down_type, uint64_t(C) * H);
    auto work = [&](uint32_t id) {
        rcs[id] = guarded([&] {
            for (uint32_t t = uint64_t(tokens) * id / threads; t < uint64_t(tokens) * (id + 1) / threads; ++t) {
                std::vector<double> xd(x + size_t(t) * C, x + size_t(t) * C + C), lg;
                if (logits) lg.assign(logits + size_t(t) * E, logits + size_t(t) * E + E);
                else lg = reference_gemv_doubleinput(0, bytes(reinterpret_cast<const uint8_t*>(L->router), size_t(E) * C * 4), C, E, xd);
                const auto routes = route_reference(lg, K, static_cast<RouterMode>(L->mode), L->normalize_selected != 0);
                std::vector<double> routed;
                for (const auto e : routes.indices) {
                    auto g = reference_gemv_doubleinput(L->expert_type, bytes(L->gate + size_t(e) * eb, eb), C, H, xd);
                    const auto u = reference_gemv_doubleinput(L->expert_type, bytes(L->up + size_t(e) * eb, eb), C, H, xd);
                    for (size_t i = 0; i < g.size(); ++i) g[i] = stable_silu(g[i]) * u[i];
                    const auto d = reference_gemv_doubleinput(down_type, bytes(L->down + size_t(e) * db, db), H, C, g);
                    routed.insert(routed.end(), d.begin(), d.end());
                }
                auto sg = reference_gemv_doubleinput(L->shared_type, bytes(L->shared_gate, sb), C, H, xd);
                const auto su = reference_gemv_doubleinput(L->shared_type, bytes(L->shared_up, sb), C, H, xd);
                for (size_t i = 0; i < sg.size(); ++i) sg[i] = stable_silu(sg[i]) * su[i];
                const auto sd = reference_gemv_doubleinput(L->shared_type, bytes(L->shared_down, sb), H, C, sg);
                double slogit = 0;
                if (L->shared_router)
                    slogit = reference_gemv_doubleinput(0, bytes(reinterpret_cast<const uint8_t*>(L->shared_router), size_t(C) * 4), C, 1, xd)[0];
                const auto y = mixture_reference(routed, routes.weights, sd, slogit);
                std::memcpy(out + size_t(t) * C, y.data(), sizeof(double) * C);
                if (indices_out) std::memcpy(indices_out + size_t(t) * K, routes.indices.data(), 4 * K);
            }
        });
    };
    std::vector<std::thread> pool;
    for (uint32_t i = 1; i < threads; ++i) pool.emplace_back(work, i);
    work(0);
    for (auto& th : pool) th.join();
    for (const int rc : rcs) if (rc) return rc;
    return 0;
}

int ref_gated_residual(const double* streams, const double* gains, const double* down, const double* up, const double* inject,
                       size_t branches, size_t channels, size_t rank, double epsilon, double* input, double* write_scales,
                       double*, double*, double*) {
    return guarded([&] {
        const size_t width = branches * channels;
        const auto r = gated_residual_reference({streams, width}, {gains, width}, {down, rank * width}, {up, width * rank}, {inject, branches * width},
                                                branches, channels, rank, epsilon);
        std::memcpy(input, r.input.data(), sizeof(double) * channels);
        std::memcpy(write_scales, r.write_scales.data(), sizeof(double) * branches);
    });
}

int ref_residual_write(const double* streams, const double* output, const double* scales, size_t branches, size_t channels, double* out) {
    return guarded([&] {
        const auto r = residual_write_reference({streams, branches * channels}, {output, channels}, {scales, branches});
        std::memcpy(out, r.data(), sizeof(double) * r.size());
    });
}

// The reference's own GGUF parser on borrowed file bytes (gguf.hpp:97, gguf.cpp): the tensor directory and the pack metadata as
// text lines, for checking this build's container reader and test writer. Line 1: alignment, version, architecture, recipe,
// data offset, manifest length; then one line per tensor: name|type|absolute offset|bytes|dimensions.
long ref_gguf_describe(const uint8_t* file, size_t nbytes, char* out, size_t cap) {
    std::string text;
    const int rc = guarded([&] {
        const Gguf g(bytes(file, nbytes));
        text = std::to_string(g.unsigned_value("general.alignment")) + "|" + std::to_string(g.unsigned_value("tokspur_pack.version")) + "|" +
               std::string(g.string_value("general.architecture")) + "|" + std::string(g.string_value("tokspur_pack.recipe")) + "|" +
               std::to_string(g.data_offset()) + "|" + std::to_string(g.string_value("tokspur_pack.manifest").size()) + "\n";
        for (const auto& t : g.tensors()) {
            text += t.name + "|" + std::to_string(t.type) + "|" + std::to_string(t.offset) + "|" + std::to_string(t.bytes) + "|";
            for (size_t i = 0; i < t.dimensions.size(); ++i) text += (i ? "," : "") + std::to_string(t.dimensions[i]);
            text += "\n";
        }
    });
    if (rc) return rc;
    if (out && cap) { const size_t n = text.size() < cap - 1 ? text.size() : cap - 1; std::memcpy(out, text.data(), n); out[n] = 0; }
    return long(text.size());
}

} // extern "C"
