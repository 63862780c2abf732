// encode_moe and encode_moe_mm_many on the CUDA graph against the CPU oracle, in the style of the reference's native/tests/test_moe.cpp:
// generated weights, route ids bit-equal, every stage within 5e-5 scaled error, refusals before encoding, sticky-error
// recovery, allocation invariants. The oracle (oracle/tsp_oracle.h) is test infrastructure and is linked only here.
#include <unistd.h>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <filesystem>
#include <functional>
#include <iostream>
#include <stdexcept>
#include <vector>

#include "tokspur_b200/moe.hpp"
#include "tokspur_b200/moe_mm_many.hpp"
#include "tokspur_b200/pack_v3.hpp"
#include "tsp_oracle.h"
#include "pack_v3_writer.hpp"

using namespace tokspur_b200;
namespace {
size_t checks = 0;
double worst = 0;
void require(bool v, const char* message) { ++checks; if (!v) throw std::runtime_error(message); }
void refuses(const std::function<void()>& action, const char* message) {
    ++checks;
    try { action(); } catch (const FormatError&) { return; }
    throw std::runtime_error(message);
}
template <class T> std::vector<T> read(CudaGraph& g, GpuView v) {
    const auto bytes = g.read(v);
    std::vector<T> out(bytes.size() / sizeof(T));
    std::memcpy(out.data(), bytes.data(), bytes.size());
    return out;
}
void close(const std::vector<float>& actual, const double* expected, size_t n, double tolerance = 5e-5) {
    require(actual.size() >= n, "result shape mismatch");
    for (size_t i = 0; i < n; ++i) {
        const double e = std::abs(actual[i] - expected[i]) / std::max(1.0, std::abs(expected[i]));
        worst = std::max(worst, e);
        require(std::isfinite(actual[i]) && e <= tolerance, "MoE numerical tolerance exceeded");
    }
}
// the reference's "bounded nonzero quant domain" generator (native/tests/test_moe_mm_many_gpu.cpp:30-47), Q4_K and Q8_0
std::vector<uint8_t> generated(uint32_t type, uint32_t k, uint32_t r, uint32_t e, uint32_t seed) {
    // Q5_1 (7): d, m, fifth bits, nibbles; Q5_K (13): the Q4_K header, 32 bytes of fifth bits, 128 bytes of nibbles
    const uint32_t epb = (type == 8 || type == 7) ? 32 : 256, bpb = type == 8 ? 34 : type == 7 ? 24 : type == 13 ? 176 : 144;
    std::vector<uint8_t> raw(uint64_t(k / epb) * bpb * r * e);
    uint32_t rng = seed;
    for (size_t at = 0; at < raw.size(); at += bpb) {
        for (uint32_t i = 0; i < bpb; ++i) { rng = rng * 1664525u + 1013904223u; raw[at + i] = uint8_t(rng >> 24); }
        raw[at] = 1; raw[at + 1] = 0x0c;
        if (type == 8) { for (unsigned i = 0; i < 32; ++i) { rng = rng * 1664525u + 1013904223u; raw[at + 2 + i] = uint8_t(int(rng % 31) - 15); } }
        else if (type == 7) { raw[at + 2] = 1; raw[at + 3] = 0x84; }   // m = -0x0401: the 32 codes centre near zero
        else {
            raw[at + 2] = 1; raw[at + 3] = 4;
            for (unsigned i = 0; i < 8; ++i) raw[at + 4 + i] = 1;
            for (unsigned i = 8; i < 12; ++i) raw[at + 4 + i] = 0x11;
            if (type == 12) for (unsigned i = 0; i < 128; ++i) raw[at + 16 + i] &= 0x77;
        }
    }
    return raw;
}
std::vector<float> activations(uint32_t seed, size_t n, float scale) {
    std::vector<float> out(n);
    uint32_t rng = seed;
    for (auto& x : out) { rng = rng * 1664525u + 1013904223u; x = scale * float(int(rng % 1993) - 996) / 997; }
    return out;
}
std::span<const std::byte> bytes(const std::vector<uint8_t>& v) { return {reinterpret_cast<const std::byte*>(v.data()), v.size()}; }
template <class T> std::span<const std::byte> bytes_of(const std::vector<T>& v) { return {reinterpret_cast<const std::byte*>(v.data()), v.size() * sizeof(T)}; }

std::vector<uint8_t> planar(uint32_t type, const std::vector<uint8_t>& gguf, uint32_t cols, uint32_t rows, uint32_t experts) {
    tso_planar_spec spec;
    require(tso_make_expert_spec(type, cols, rows, &spec) == TSO_OK, "planar spec");
    std::vector<uint8_t> out(spec.planar_expert_bytes * experts);
    for (uint32_t e = 0; e < experts; ++e)
        require(tso_pack_expert_planar(&spec, gguf.data() + e * spec.source_expert_bytes, out.data() + e * spec.planar_expert_bytes) == TSO_OK, "pack");
    return out;
}

// down_type / shared_type 0: the encoding of gate and up
void layer(CudaGraph& g, uint32_t type, bool use_planar, MoeShape shape, uint32_t seed, uint32_t down_type = 0, uint32_t shared_type = 0) {
    const uint32_t C = shape.channels, H = shape.hidden, E = shape.experts, K = shape.selected;
    const uint32_t dt = down_type ? down_type : type, st = shared_type ? shared_type : type;
    const auto gate = generated(type, C, H, E, seed + 1), up = generated(type, C, H, E, seed + 2), down = generated(dt, H, C, E, seed + 3);
    const auto sgate = generated(st, C, H, 1, seed + 4), sup = generated(st, C, H, 1, seed + 5), sdown = generated(st, H, C, 1, seed + 6);
    const auto router = activations(seed + 7, size_t(E) * C, 0.25f), srouter = activations(seed + 8, C, 0.125f);
    MoeWeights w{};
    w.router = {g.upload(bytes_of(router), "router"), 0};
    w.shared_router = {g.upload(bytes_of(srouter), "shared router"), 0};
    w.shared_gate = {g.upload(bytes(sgate), "sg"), st}; w.shared_up = {g.upload(bytes(sup), "su"), st}; w.shared_down = {g.upload(bytes(sdown), "sd"), st};
    if (use_planar) {
        // co-located pairs: lo = experts [0, E/2) as [gate_e, up_e], hi = the rest (planar_pack_v3.cpp:1076-1093)
        const auto pg = planar(type, gate, C, H, E), pu = planar(type, up, C, H, E);
        const size_t pb = pg.size() / E;
        std::vector<uint8_t> lo(pb * E), hi(pb * E);
        for (uint32_t e = 0; e < E; ++e) {
            auto& dst = e < E / 2 ? lo : hi;
            const size_t at = size_t(e % (E / 2)) * 2 * pb;
            std::memcpy(dst.data() + at, pg.data() + e * pb, pb);
            std::memcpy(dst.data() + at + pb, pu.data() + e * pb, pb);
        }
        w.gate = {g.upload(bytes(lo), "pair lo"), type}; w.up = {g.upload(bytes(hi), "pair hi"), type};
        w.down = {g.upload(bytes(planar(type, down, H, C, E)), "down planar"), type};
        const uint32_t gk = type == 12 ? 2 : 6, dk = type == 12 ? 10 : 9;
        g.register_planar_matrix(w.gate.view, {type, gk, C, H, E});
        g.register_planar_matrix(w.up.view, {type, gk + 1, C, H, E});
        g.register_planar_matrix(w.down.view, {type, dk, H, C, E});
        require(is_planar_moe(g, w, shape), "registered pairs are recognised as a planar MoE");
    } else {
        w.gate = {g.upload(bytes(gate), "gate"), type}; w.up = {g.upload(bytes(up), "up"), type}; w.down = {g.upload(bytes(down), "down"), dt};
        require(!is_planar_moe(g, w, shape), "raw GGUF tensors are not planar");
    }
    const auto scratch = allocate_moe_scratch(g, shape);
    const auto input = g.zeros(C * 4, "input"), output = g.zeros(C * 4, "output");
    const auto allocations = g.allocations();

    tso_layer L{C, H, E, K, type, st, gate.data(), up.data(), down.data(), sgate.data(), sup.data(), sdown.data(), srouter.data(), router.data(), 0, 1, dt};
    for (uint32_t token = 0; token < 3; ++token) {
        const auto x = activations(100 + token + seed, C, 8.f);
        std::vector<double> expected(C), ew(K), act(size_t(K) * H), routed(size_t(K) * C), sact(H), sout(C);
        std::vector<uint32_t> eids(K);
        double slog = 0;
        tso_layer_stages st{eids.data(), ew.data(), act.data(), routed.data(), sact.data(), sout.data(), &slog};
        require(tso_moe_layer(&L, x.data(), nullptr, 1, expected.data(), &st, 1) == TSO_OK, "oracle layer");
        g.write(input, bytes_of(x));
        for (int run = 0; run < 2; ++run) {
            g.begin();
            encode_moe(g, w, scratch, input, output, shape, RouterMode::softmax, true);
            const auto batch = g.submit();
            require(batch.dispatches >= 5 && g.allocations() == allocations, "dispatch / allocation invariant");
            require(read<uint32_t>(g, scratch.indices) == eids, "route ids differ");
            close(read<float>(g, scratch.weights), ew.data(), K);
            close(read<float>(g, scratch.gate), act.data(), act.size());
            close(read<float>(g, scratch.down), routed.data(), routed.size());
            close(read<float>(g, scratch.shared_gate), sact.data(), H);
            close(read<float>(g, scratch.shared_down), sout.data(), C);
            close(read<float>(g, output), expected.data(), C);
        }
    }
    // refusals happen before anything is encoded; the batch is then discarded and the graph stays usable
    g.begin();
    refuses([&] { encode_moe(g, w, scratch, g.slice(input, 0, C * 2), output, shape, RouterMode::softmax, true); }, "short input accepted");
    refuses([&] { encode_moe(g, w, scratch, input, output, {C, H, E, E + 1}, RouterMode::softmax, true); }, "selected > experts accepted");
    g.abort();
    refuses([&] { encode_moe(g, w, scratch, input, output, shape, RouterMode::softmax, true); }, "encode outside a batch accepted");
    // sticky error word: a non-finite input is reported at submit, and the next batch is clean again
    auto bad = activations(5, C, 1.f);
    bad[3] = std::numeric_limits<float>::infinity();
    g.write(input, bytes_of(bad));
    g.begin();
    encode_moe(g, w, scratch, input, output, shape, RouterMode::softmax, true);
    refuses([&] { (void)g.submit(); }, "non-finite input was not reported at submit");
    const auto x = activations(100 + seed, C, 8.f);
    g.write(input, bytes_of(x));
    g.begin();
    encode_moe(g, w, scratch, input, output, shape, RouterMode::softmax, true);
    (void)g.submit();
    release_moe_scratch(g, scratch);
}
// encode_verify_nax_moe: a verify batch of `steps` rows through the decode kernels, every stage against the oracle.
void verify_rows(CudaGraph& g, uint32_t type, MoeShape shape, uint32_t steps, uint32_t seed) {
    const uint32_t C = shape.channels, H = shape.hidden, E = shape.experts, K = shape.selected;
    const auto gate = generated(type, C, H, E, seed + 1), up = generated(type, C, H, E, seed + 2), down = generated(type, H, C, E, seed + 3);
    const auto sgate = generated(type, C, H, 1, seed + 4), sup = generated(type, C, H, 1, seed + 5), sdown = generated(type, H, C, 1, seed + 6);
    const auto router = activations(seed + 7, size_t(E) * C, 0.25f), srouter = activations(seed + 8, C, 0.125f);
    MoeWeights w{};
    w.router = {g.upload(bytes_of(router), "router"), 0};
    w.shared_router = {g.upload(bytes_of(srouter), "shared router"), 0};
    w.shared_gate = {g.upload(bytes(sgate), "sg"), type}; w.shared_up = {g.upload(bytes(sup), "su"), type}; w.shared_down = {g.upload(bytes(sdown), "sd"), type};
    w.gate = {g.upload(bytes(gate), "gate"), type}; w.up = {g.upload(bytes(up), "up"), type}; w.down = {g.upload(bytes(down), "down"), type};
    const auto scratch = allocate_moe_rows_scratch(g, shape, steps);
    const auto input = g.zeros(uint64_t(C) * 4 * steps, "rows in"), output = g.zeros(uint64_t(C) * 4 * steps, "rows out");
    const auto x = activations(900 + seed, size_t(C) * steps, 8.f);
    g.write(input, bytes_of(x));
    tso_layer L{C, H, E, K, type, type, gate.data(), up.data(), down.data(), sgate.data(), sup.data(), sdown.data(), srouter.data(), router.data(), 0, 1, 0};
    std::vector<double> expected(size_t(C) * steps), ew(size_t(K) * steps);
    std::vector<uint32_t> eids(size_t(K) * steps);
    tso_layer_stages st{eids.data(), ew.data(), nullptr, nullptr, nullptr, nullptr, nullptr};
    require(tso_moe_layer(&L, x.data(), nullptr, steps, expected.data(), &st, 2) == TSO_OK, "oracle layer");
    const VerifyNaxMoeScratch none{};
    g.begin();
    encode_verify_nax_moe(g, w, scratch, none, input, output, shape, RouterMode::softmax, true, steps);
    (void)g.submit();
    require(read<uint32_t>(g, scratch.indices) == eids, "verify batch: route ids differ");
    close(read<float>(g, scratch.weights), ew.data(), ew.size());
    close(read<float>(g, output), expected.data(), expected.size());
    // the same rows through encode_moe_many with its own capacity scratch
    prepare_moe_many(g, w, shape);
    const auto ms = allocate_moe_many_scratch(g, shape, steps);
    g.write(output, std::vector<std::byte>(output.bytes));
    g.begin();
    encode_moe_many(g, w, ms, input, output, shape, RouterMode::softmax, true, steps);
    const auto batch = g.submit();
    require(batch.dispatches == moe_many_dispatches(g, w, shape, steps), "known-input FFN dispatch count");
    require(read<uint32_t>(g, ms.rows.indices) == eids, "known-input FFN: route ids differ");
    close(read<float>(g, output), expected.data(), expected.size());
    g.begin();
    refuses([&] { encode_moe_many(g, w, ms, input, output, shape, RouterMode::softmax, true, steps + 1); }, "rows beyond the scratch capacity accepted");
    g.abort();
    release_moe_many_scratch(g, ms);
    g.begin();
    refuses([&] { encode_verify_nax_moe(g, w, scratch, none, input, output, shape, RouterMode::softmax, true, 1); }, "one-row verify batch accepted");
    refuses([&] { encode_verify_nax_moe(g, w, scratch, none, input, output, shape, RouterMode::softmax, true, steps + 1); }, "rows beyond the views accepted");
    g.abort();
    release_moe_scratch(g, scratch);
}

// encode_moe_mm_many (grouped tensor-core GEMMs): strided row batches longer than the scratch capacity, against the oracle.
// Operands are binary16 there, so the layer bar is the relative L2 error of 2e-3, not the decode path's 5e-5.
void many(CudaGraph& g, MoeShape shape, uint32_t rows, uint32_t capacity, uint32_t seed) {
    const uint32_t type = 12, C = shape.channels, H = shape.hidden, E = shape.experts, K = shape.selected;
    const auto gate = generated(type, C, H, E, seed + 1), up = generated(type, C, H, E, seed + 2), down = generated(type, H, C, E, seed + 3);
    const auto sgate = generated(type, C, H, 1, seed + 4), sup = generated(type, C, H, 1, seed + 5), sdown = generated(type, H, C, 1, seed + 6);
    const auto router = activations(seed + 7, size_t(E) * C, 0.25f), srouter = activations(seed + 8, C, 0.125f);
    MoeWeights w{};
    w.router = {g.upload(bytes_of(router), "router"), 0};
    w.shared_router = {g.upload(bytes_of(srouter), "shared router"), 0};
    const auto pg = planar(type, gate, C, H, E), pu = planar(type, up, C, H, E);
    const size_t pb = pg.size() / E;
    std::vector<uint8_t> lo(pb * E), hi(pb * E);
    for (uint32_t e = 0; e < E; ++e) {
        auto& dst = e < E / 2 ? lo : hi;
        const size_t at = size_t(e % (E / 2)) * 2 * pb;
        std::memcpy(dst.data() + at, pg.data() + e * pb, pb);
        std::memcpy(dst.data() + at + pb, pu.data() + e * pb, pb);
    }
    w.gate = {g.upload(bytes(lo), "pair lo"), type}; w.up = {g.upload(bytes(hi), "pair hi"), type};
    w.down = {g.upload(bytes(planar(type, down, H, C, E)), "down planar"), type};
    w.shared_gate = {g.upload(bytes(planar(type, sgate, C, H, 1)), "sg planar"), type};
    w.shared_up = {g.upload(bytes(planar(type, sup, C, H, 1)), "su planar"), type};
    w.shared_down = {g.upload(bytes(planar(type, sdown, H, C, 1)), "sd planar"), type};
    g.register_planar_matrix(w.gate.view, {type, 2, C, H, E});
    g.register_planar_matrix(w.up.view, {type, 3, C, H, E});
    g.register_planar_matrix(w.down.view, {type, 10, H, C, E});
    g.register_planar_matrix(w.shared_gate.view, {type, 10, C, H, 1});
    g.register_planar_matrix(w.shared_up.view, {type, 10, C, H, 1});
    g.register_planar_matrix(w.shared_down.view, {type, 10, H, C, 1});
    const auto scratch = allocate_moe_mm_many_scratch(g, shape, capacity);
    const uint64_t in_stride = uint64_t(C) * 4 + 32, out_stride = uint64_t(C) * 4 + 16;
    const auto input = g.zeros(in_stride * rows, "rows in"), output = g.zeros(out_stride * rows, "rows out");
    const auto allocations = g.allocations();

    // activations that binary16 holds exactly, as on the prefill path (multiples of 1/64 below 16)
    std::vector<float> x(size_t(rows) * C);
    uint32_t rng = seed * 77u + 5u;
    for (auto& v : x) { rng = rng * 1664525u + 1013904223u; v = float(int(rng % 1025) - 512) / 64.f; }
    std::vector<uint8_t> staged(in_stride * rows, 0);
    for (uint32_t r = 0; r < rows; ++r) std::memcpy(staged.data() + r * in_stride, x.data() + size_t(r) * C, size_t(C) * 4);
    g.write(input, bytes(staged));
    tso_layer L{C, H, E, K, type, type, gate.data(), up.data(), down.data(), sgate.data(), sup.data(), sdown.data(), srouter.data(), router.data(), 0, 1, 0};
    std::vector<double> expected(size_t(rows) * C);
    require(tso_moe_layer(&L, x.data(), nullptr, rows, expected.data(), nullptr, 4) == TSO_OK, "oracle layer");
    prepare_moe_mm_many(g, w, shape);
    MoeMmLayouts raw;
    raw.down = PrefillWeightLayout::gguf;
    refuses([&] { prepare_moe_mm_many(g, w, shape, raw); }, "a raw GGUF identity was accepted by the tiled path");
    refuses([&] { prepare_moe_mm_many(g, w, {C, H, E, E + 1}); }, "selected > experts accepted by prepare");
    for (int run = 0; run < 2; ++run) {
        g.begin();
        encode_moe_mm_many(g, w, scratch, {input, rows, C, in_stride}, {output, rows, C, out_stride}, shape, RouterMode::softmax, true);
        const auto batch = g.submit();
        require(batch.dispatches == moe_mm_many_dispatches(g, w, shape, rows, capacity) && g.allocations() == allocations, "dispatch / allocation invariant");
        const auto raw = g.read(output);
        double num = 0, den = 0;
        for (uint32_t r = 0; r < rows; ++r)
            for (uint32_t c = 0; c < C; ++c) {
                float v;
                std::memcpy(&v, raw.data() + r * out_stride + size_t(c) * 4, 4);
                const double e = expected[size_t(r) * C + c];
                require(std::isfinite(v), "non-finite row value");
                num += (v - e) * (v - e); den += e * e;
            }
        const double rel = std::sqrt(num / den);
        std::cout << "  encode_moe_mm_many rows " << rows << " capacity " << capacity << ": relative L2 error " << rel << "\n";
        require(rel <= 2e-3, "tiled MoE relative L2 tolerance exceeded");
    }
    {   // the same tensors as raw GGUF super-blocks (the reference's default identity): same staged operands, so the same bits
        const auto planar_rows = g.read(output);
        MoeWeights r = w;
        r.gate = {g.upload(bytes(gate), "gate gguf"), type}; r.up = {g.upload(bytes(up), "up gguf"), type};
        r.down = {g.upload(bytes(down), "down gguf"), type};
        r.shared_gate = {g.upload(bytes(sgate), "sg gguf"), type}; r.shared_up = {g.upload(bytes(sup), "su gguf"), type};
        r.shared_down = {g.upload(bytes(sdown), "sd gguf"), type};
        MoeMmLayouts all_raw;
        all_raw.gate = all_raw.up = all_raw.down = all_raw.shared_gate = all_raw.shared_up = all_raw.shared_down = PrefillWeightLayout::gguf;
        prepare_moe_mm_many(g, r, shape, all_raw);
        refuses([&] { prepare_moe_mm_many(g, r, shape); }, "raw GGUF tensors declared planar were accepted");
        refuses([&] { prepare_moe_mm_many(g, w, shape, all_raw); }, "registered planar tensors declared raw GGUF were accepted");
        const auto before = g.allocations();
        g.begin();
        encode_moe_mm_many(g, r, scratch, {input, rows, C, in_stride}, {output, rows, C, out_stride}, shape, RouterMode::softmax, true, all_raw);
        const auto batch = g.submit();
        require(batch.dispatches == moe_mm_many_dispatches(g, r, shape, rows, capacity, all_raw) && g.allocations() == before, "dispatch / allocation invariant (raw GGUF)");
        require(g.read(output) == planar_rows, "raw GGUF and planar weights gave different rows");
        std::cout << "  encode_moe_mm_many raw GGUF blocks: rows identical to the planar run\n";
        for (const auto& m : {r.gate, r.up, r.down, r.shared_gate, r.shared_up, r.shared_down}) g.release(m.view);
    }
    {   // the reference model's mix: planar Q4_K experts beside a dense shared expert of raw Q8_0 blocks (launches of its own)
        const auto q8g = generated(8, C, H, 1, seed + 14), q8u = generated(8, C, H, 1, seed + 15), q8d = generated(8, H, C, 1, seed + 16);
        MoeWeights m = w;
        m.shared_gate = {g.upload(bytes(q8g), "sg q8"), 8}; m.shared_up = {g.upload(bytes(q8u), "su q8"), 8}; m.shared_down = {g.upload(bytes(q8d), "sd q8"), 8};
        MoeMmLayouts mixed;
        mixed.shared_gate = mixed.shared_up = mixed.shared_down = PrefillWeightLayout::gguf;
        prepare_moe_mm_many(g, m, shape, mixed);
        refuses([&] { prepare_moe_mm_many(g, m, shape); }, "raw Q8_0 shared tensors declared planar were accepted");
        tso_layer LQ{C, H, E, K, type, 8, gate.data(), up.data(), down.data(), q8g.data(), q8u.data(), q8d.data(), srouter.data(), router.data(), 0, 1, 0};
        std::vector<double> want(size_t(rows) * C);
        require(tso_moe_layer(&LQ, x.data(), nullptr, rows, want.data(), nullptr, 4) == TSO_OK, "oracle layer (Q8_0 shared)");
        const auto before = g.allocations();
        g.begin();
        encode_moe_mm_many(g, m, scratch, {input, rows, C, in_stride}, {output, rows, C, out_stride}, shape, RouterMode::softmax, true, mixed);
        const auto batch = g.submit();
        const uint64_t chunks = (uint64_t(rows) + capacity - 1) / capacity;
        require(batch.dispatches == moe_mm_many_dispatches(g, m, shape, rows, capacity, mixed) && batch.dispatches == 12 * chunks && g.allocations() == before,
                "dispatch / allocation invariant (Q8_0 shared)");
        const auto got = g.read(output);
        double num = 0, den = 0;
        for (uint32_t r = 0; r < rows; ++r)
            for (uint32_t c = 0; c < C; ++c) {
                float v;
                std::memcpy(&v, got.data() + r * out_stride + size_t(c) * 4, 4);
                const double e = want[size_t(r) * C + c];
                require(std::isfinite(v), "non-finite row value");
                num += (v - e) * (v - e); den += e * e;
            }
        const double rel = std::sqrt(num / den);
        std::cout << "  encode_moe_mm_many with a dense Q8_0 shared expert: relative L2 error " << rel << "\n";
        require(rel <= 2e-3, "tiled MoE (Q8_0 shared) relative L2 tolerance exceeded");
        for (const auto& t : {m.shared_gate, m.shared_up, m.shared_down}) g.release(t.view);
    }
    g.begin();
    refuses([&] { encode_moe_mm_many(g, w, scratch, {input, rows, C - 1, in_stride}, {output, rows, C, out_stride}, shape, RouterMode::softmax, true); }, "column mismatch accepted");
    refuses([&] { encode_moe_mm_many(g, w, scratch, {input, rows, C, in_stride - 4}, {output, rows, C, out_stride}, shape, RouterMode::softmax, true); }, "unaligned stride accepted");
    refuses([&] { encode_moe_mm_many(g, w, scratch, {input, rows + 1, C, in_stride}, {output, rows + 1, C, out_stride}, shape, RouterMode::softmax, true); }, "rows beyond the views accepted");
    g.abort();
    release_moe_mm_many_scratch(g, scratch);
}
// One layer read from a "tokspur-pack-v3" container (written here with the test-side writer in the reference's layouts: co-located
// planar Q4_K gate / up pairs, planar Q8_0 down, lane-packed dense Q8_0 shared expert, plain F32 routers) and run through
// encode_moe and encode_moe_many against the oracle on the source GGUF bytes.
void pack_layer(uint32_t seed) {
    namespace fs = std::filesystem;
    const uint32_t C = 256, H = 256, E = 8, K = 4;
    pack_v3_test::LayerBytes L{C, H, E, 12, generated(12, C, H, E, seed + 1), generated(12, C, H, E, seed + 2), generated(8, H, C, E, seed + 3),
                               generated(8, C, H, 1, seed + 4), generated(8, C, H, 1, seed + 5), generated(8, H, C, 1, seed + 6),
                               activations(seed + 7, size_t(E) * C, 0.25f), activations(seed + 8, C, 0.125f)};
    const fs::path dir = fs::temp_directory_path() / ("tokspur_b200_pack_layer_" + std::to_string(::getpid()));
    fs::create_directories(dir);
    const fs::path path = dir / "layer.gguf";
    pack_v3_test::write(path, pack_v3_test::layer_entries(L, "blk.3."));
    const PackIndexV3 index = read_pack_v3_index(path);
    CudaGraph g(0, uint64_t(1) << 30);
    MoeShape shape{0, 0, 0, K};
    const MoeWeights w = load_pack_v3_moe_layer(g, path, index, "blk.3.", shape);
    require(shape.channels == C && shape.hidden == H && shape.experts == E && shape.selected == K, "layer shape from the pack directory");
    require(is_planar_moe(g, w, shape) && w.shared_gate.encoding == 8 && !g.planar_matrix_shape(w.shared_gate.view), "registered forms of the pack tensors");
    refuses([&] { MoeShape s2{}; (void)load_pack_v3_moe_layer(g, path, index, "blk.4.", s2); }, "a layer that is not in the pack was loaded");

    tso_layer O{C, H, E, K, 12, 8, L.gate.data(), L.up.data(), L.down.data(), L.sgate.data(), L.sup.data(), L.sdown.data(), L.srouter.data(), L.router.data(), 0, 1, 8};
    const auto scratch = allocate_moe_scratch(g, shape);
    const auto input = g.zeros(C * 4, "input"), output = g.zeros(C * 4, "output");
    for (uint32_t token = 0; token < 3; ++token) {
        const auto x = activations(300 + token + seed, C, 8.f);
        std::vector<double> expected(C);
        require(tso_moe_layer(&O, x.data(), nullptr, 1, expected.data(), nullptr, 1) == TSO_OK, "oracle layer");
        g.write(input, bytes_of(x));
        g.begin();
        encode_moe(g, w, scratch, input, output, shape, RouterMode::softmax, true);
        (void)g.submit();
        close(read<float>(g, output), expected.data(), C);
    }
    const uint32_t rows = 9;
    const auto many = allocate_moe_many_scratch(g, shape, rows);
    const auto xin = activations(400 + seed, size_t(rows) * C, 4.f);
    const auto in = g.zeros(uint64_t(rows) * C * 4, "rows in"), out = g.zeros(uint64_t(rows) * C * 4, "rows out");
    g.write(in, bytes_of(xin));
    std::vector<double> expected(size_t(rows) * C);
    require(tso_moe_layer(&O, xin.data(), nullptr, rows, expected.data(), nullptr, 4) == TSO_OK, "oracle layer rows");
    g.begin();
    encode_moe_many(g, w, many, in, out, shape, RouterMode::softmax, true, rows);
    (void)g.submit();
    close(read<float>(g, out), expected.data(), expected.size());
    release_moe_many_scratch(g, many);
    release_moe_scratch(g, scratch);
    std::cout << "  layer loaded from a pack v3 container: encode_moe and encode_moe_many agree with the oracle\n";
    {   // the same layer for the prefill encoder: the planar Q8_0 down tensor re-laid as raw blocks while loading
        CudaGraph gp(0, uint64_t(1) << 30);
        MoeShape sp{0, 0, 0, K};
        const MoeWeights wp = load_pack_v3_moe_layer(gp, path, index, "blk.3.", sp, {true});
        require(is_planar_gate_up(gp, wp, sp) && !is_planar_moe(gp, wp, sp) && !gp.planar_matrix_shape(wp.down.view), "forms of the tensors loaded for prefill");
        MoeMmLayouts lay;   // gate / up: the registered pairs; down and the shared expert: raw Q8_0 blocks
        lay.down = lay.shared_gate = lay.shared_up = lay.shared_down = PrefillWeightLayout::gguf;
        prepare_moe_mm_many(gp, wp, sp, lay);
        const uint32_t n = 70, capacity = 64;
        const auto ps = allocate_moe_mm_many_scratch(gp, sp, capacity);
        std::vector<float> xr(size_t(n) * C);
        uint32_t rng = seed * 13u + 1u;
        for (auto& v : xr) { rng = rng * 1664525u + 1013904223u; v = float(int(rng % 1025) - 512) / 64.f; }
        const auto pin = gp.zeros(uint64_t(n) * C * 4, "prefill in"), pout = gp.zeros(uint64_t(n) * C * 4, "prefill out");
        gp.write(pin, bytes_of(xr));
        std::vector<double> want(size_t(n) * C);
        require(tso_moe_layer(&O, xr.data(), nullptr, n, want.data(), nullptr, 4) == TSO_OK, "oracle layer (prefill rows)");
        gp.begin();
        encode_moe_mm_many(gp, wp, ps, {pin, n, C, uint64_t(C) * 4}, {pout, n, C, uint64_t(C) * 4}, sp, RouterMode::softmax, true, lay);
        (void)gp.submit();
        const auto got = read<float>(gp, pout);
        double num = 0, den = 0;
        for (size_t i = 0; i < got.size(); ++i) { require(std::isfinite(got[i]), "non-finite row value"); num += (got[i] - want[i]) * (got[i] - want[i]); den += want[i] * want[i]; }
        const double rel = std::sqrt(num / den);
        std::cout << "  pack layer through encode_moe_mm_many (Q4_K pairs, Q8_0 down rows, Q8_0 shared): relative L2 error " << rel << "\n";
        require(rel <= 2e-3, "pack layer prefill tolerance exceeded");
        // one decode row through the same weights (pairs + raw Q8_0 down)
        const auto s1 = allocate_moe_scratch(gp, sp);
        const auto i1 = gp.zeros(C * 4, "in"), o1 = gp.zeros(C * 4, "out");
        gp.write(i1, std::span<const std::byte>(reinterpret_cast<const std::byte*>(xr.data()), size_t(C) * 4));
        gp.begin();
        encode_moe(gp, wp, s1, i1, o1, sp, RouterMode::softmax, true);
        (void)gp.submit();
        close(read<float>(gp, o1), want.data(), C);
    }
    fs::remove_all(dir);
}
// The stand-alone operators of the graph (dense GEMV forms, batched routing with the margin audit, mixture, residual read / write)
// against the oracle's functions.
void operators(CudaGraph& g, uint32_t seed) {
    const uint32_t C = 256, R = 96, T = 5, E = 16, K = 4, B = 4;
    for (uint32_t type : {8u, 12u}) {
        const auto m = generated(type, C, R, 1, seed + type);
        const auto mv = g.upload(bytes(m), "dense matrix");
        const auto x = activations(seed + 3, size_t(C) * T, 4.f);
        const auto in = g.upload(bytes_of(x), "dense in"), out = g.zeros(uint64_t(R) * 4 * T, "dense out");
        g.begin();
        if (type == 8) g.q8_matvec_many(mv, in, out, C, R, T);
        else g.gemv_rows(type, mv, {in, T, C, uint64_t(C) * 4}, {out, T, R, uint64_t(R) * 4});
        (void)g.submit();
        std::vector<double> expected(size_t(R) * T);
        for (uint32_t t = 0; t < T; ++t) require(tso_gemv_f32(type, m.data(), m.size(), C, R, x.data() + size_t(t) * C, expected.data() + size_t(t) * R) == TSO_OK, "oracle gemv");
        close(read<float>(g, out), expected.data(), expected.size());
        if (type == 8) {
            g.begin();
            g.verify_nax_dense_q8(mv, {in, T, C, uint64_t(C) * 4}, {out, T, R, uint64_t(R) * 4});
            g.gemv(type, mv, g.slice(in, 0, uint64_t(C) * 4), g.slice(out, 0, uint64_t(R) * 4), C, R);
            (void)g.submit();
            close(read<float>(g, out), expected.data(), expected.size());
            g.begin();
            refuses([&] { g.q8_matvec_many(mv, in, out, C, R, T + 1); }, "width beyond the views accepted");
            refuses([&] { g.verify_nax_dense_q8(mv, {in, 17, C, uint64_t(C) * 4}, {out, 17, R, uint64_t(R) * 4}); }, "17-row verify batch accepted");
            refuses([&] { g.gemv(5, mv, in, out, C, R); }, "unknown encoding accepted");
            g.abort();
        }
    }
    {   // dense Q8_0 row batch on the tensor cores: 300 strided rows, twice (the second call reuses the staged input rows)
        const uint32_t DC = 512, DR = 256, DT = 300;
        const auto m = generated(8, DC, DR, 1, seed + 21);
        const auto mv = g.upload(bytes(m), "dense q8 matrix");
        std::vector<float> x(size_t(DT) * DC);
        uint32_t rng = seed * 31u + 9u;
        for (auto& v : x) { rng = rng * 1664525u + 1013904223u; v = float(int(rng % 1025) - 512) / 64.f; }   // exact in binary16
        const uint64_t in_stride = uint64_t(DC) * 4 + 16, out_stride = uint64_t(DR) * 4 + 32;
        std::vector<uint8_t> staged(in_stride * DT, 0);
        for (uint32_t r = 0; r < DT; ++r) std::memcpy(staged.data() + r * in_stride, x.data() + size_t(r) * DC, size_t(DC) * 4);
        const auto in = g.upload(bytes(staged), "dense q8 in"), out = g.zeros(out_stride * DT, "dense q8 out");
        refuses([&] { g.begin(); try { g.dense_mm_q8(PrefillWeightLayout::gguf, mv, {in, DT, DC, in_stride}, {out, DT, DR, out_stride}); } catch (...) { g.abort(); throw; } },
                "dense Q8_0 GEMM ran without prepared staging");
        g.prepare_dense_mm_q8(PrefillWeightLayout::gguf, DT, DC);
        std::vector<double> expected(size_t(DR) * DT);
        for (uint32_t t = 0; t < DT; ++t) require(tso_gemv_f32(8, m.data(), m.size(), DC, DR, x.data() + size_t(t) * DC, expected.data() + size_t(t) * DR) == TSO_OK, "oracle gemv");
        for (int run = 0; run < 2; ++run) {
            g.begin();
            g.dense_mm_q8(PrefillWeightLayout::gguf, mv, {in, DT, DC, in_stride}, {out, DT, DR, out_stride}, run == 1);
            const auto batch = g.submit();
            require(batch.dispatches == CudaGraph::dense_mm_q8_dispatches(run == 1), "dense Q8_0 GEMM dispatch count");
            const auto raw = g.read(out);
            double num = 0, den = 0;
            for (uint32_t t = 0; t < DT; ++t)
                for (uint32_t r = 0; r < DR; ++r) {
                    float v;
                    std::memcpy(&v, raw.data() + t * out_stride + size_t(r) * 4, 4);
                    const double e = expected[size_t(t) * DR + r];
                    num += (v - e) * (v - e); den += e * e;
                }
            const double rel = std::sqrt(num / den);
            std::cout << "  dense_mm_q8 " << DT << " rows: relative L2 error " << rel << "\n";
            require(rel <= 2e-3, "dense Q8_0 GEMM relative L2 tolerance exceeded");
        }
        g.begin();
        refuses([&] { g.dense_mm_q8(PrefillWeightLayout::planar, mv, {in, DT, DC, in_stride}, {out, DT, DR, out_stride}); }, "planar identity accepted by the dense Q8_0 GEMM");
        refuses([&] { g.dense_mm_q8(PrefillWeightLayout::gguf, mv, {in, DT, DC, in_stride}, {out, DT, DR - 128, out_stride}); }, "matrix extent mismatch accepted");
        refuses([&] { g.dense_mm_q8(PrefillWeightLayout::gguf, mv, {in, DT + 1, DC, in_stride}, {out, DT + 1, DR, out_stride}); }, "rows beyond the views accepted");
        g.abort();
        g.release(mv); g.release(in); g.release(out);
    }
    // router projection -> audited routing -> mixture
    const auto router = activations(seed + 7, size_t(E) * C, 0.25f), srouter = activations(seed + 8, C, 0.125f);
    const auto x = activations(seed + 9, size_t(C) * T, 1.f);
    const auto rv = g.upload(bytes_of(router), "router"), sv = g.upload(bytes_of(srouter), "shared router"), xv = g.upload(bytes_of(x), "x");
    const auto logits = g.zeros(uint64_t(T) * E * 4, "logits"), slog = g.zeros(T * 4, "shared logits");
    const auto ids = g.zeros(T * K * 4, "ids"), wts = g.zeros(T * K * 4, "weights");
    const auto ex = activations(seed + 10, size_t(T) * K * C, 2.f), sh = activations(seed + 11, size_t(T) * C, 2.f);
    const auto exv = g.upload(bytes_of(ex), "expert rows"), shv = g.upload(bytes_of(sh), "shared rows"), mix = g.zeros(uint64_t(T) * C * 4, "mixture");
    g.configure_router_margin_audit(true);
    g.configure_router_margin_epsilon(1e-4f);
    g.prepare_router_margin_scratch();
    const auto allocations = g.allocations();
    g.begin();
    g.moe_router_rows(rv, sv, {xv, T, C, uint64_t(C) * 4}, logits, slog, E);
    g.moe_route_rows(logits, ids, wts, E, K, T, RouterMode::softmax, true);
    g.prefill_mixture_batch(exv, wts, shv, slog, {mix, T, C, uint64_t(C) * 4}, K);
    (void)g.submit();
    require(g.allocations() == allocations, "operators allocated while encoding");
    const auto gl = read<float>(g, logits), gs = read<float>(g, slog), gw = read<float>(g, wts);
    const auto gi = read<uint32_t>(g, ids);
    std::vector<double> el(size_t(T) * E), es(T), emix(size_t(T) * C);
    for (uint32_t t = 0; t < T; ++t) {
        require(tso_gemv_f32(0, reinterpret_cast<const uint8_t*>(router.data()), router.size() * 4, C, E, x.data() + size_t(t) * C, el.data() + size_t(t) * E) == TSO_OK, "oracle router");
        require(tso_gemv_f32(0, reinterpret_cast<const uint8_t*>(srouter.data()), srouter.size() * 4, C, 1, x.data() + size_t(t) * C, &es[t]) == TSO_OK, "oracle shared router");
    }
    close(gl, el.data(), el.size());
    close(gs, es.data(), T);
    double min_margin = 1e30;
    for (uint32_t t = 0; t < T; ++t) {
        // routing is checked on the logits the device produced, so a near-tie cannot flip an id between the two
        std::vector<double> row(gl.begin() + size_t(t) * E, gl.begin() + size_t(t + 1) * E), ew(K), dex(size_t(K) * C), dsh(C);
        std::vector<uint32_t> ei(K);
        require(tso_route(row.data(), E, K, 0, 1, ei.data(), ew.data()) == TSO_OK, "oracle route");
        require(std::equal(ei.begin(), ei.end(), gi.begin() + size_t(t) * K), "audited route ids differ");
        close(std::vector<float>(gw.begin() + size_t(t) * K, gw.begin() + size_t(t + 1) * K), ew.data(), K);
        std::vector<double> sorted(row);
        std::sort(sorted.begin(), sorted.end(), std::greater<>());
        min_margin = std::min(min_margin, sorted[K - 1] - sorted[K]);
        for (size_t i = 0; i < dex.size(); ++i) dex[i] = ex[size_t(t) * K * C + i];
        for (uint32_t c = 0; c < C; ++c) dsh[c] = sh[size_t(t) * C + c];
        std::vector<double> w64(gw.begin() + size_t(t) * K, gw.begin() + size_t(t + 1) * K);
        require(tso_mixture(dex.data(), w64.data(), K, dsh.data(), C, gs[t], emix.data() + size_t(t) * C) == TSO_OK, "oracle mixture");
    }
    close(read<float>(g, mix), emix.data(), emix.size());
    const bool fallback = g.evaluate_router_margin(T);
    const auto tel = g.router_margin_telemetry();
    require(tel.total_layers == 1 && tel.total_tokens == T && std::abs(tel.min_margin - min_margin) <= 1e-6 * std::max(1.0, std::abs(min_margin)), "margin telemetry");
    require(fallback == (min_margin <= 2e-4) && tel.fallback_layers == (fallback ? 1u : 0u), "margin fallback decision");
    g.begin();
    g.mixture(g.slice(exv, 0, uint64_t(K) * C * 4), g.slice(wts, 0, K * 4), g.slice(shv, 0, uint64_t(C) * 4), g.slice(slog, 0, 4), g.slice(mix, 0, uint64_t(C) * 4));
    (void)g.submit();
    close(read<float>(g, g.slice(mix, 0, uint64_t(C) * 4)), emix.data(), C);
    g.begin();
    refuses([&] { g.prefill_mixture_batch(exv, wts, shv, slog, {mix, T + 1, C, uint64_t(C) * 4}, K); }, "mixture rows beyond the views accepted");
    refuses([&] { g.moe_route_rows(logits, ids, wts, E, K, 4096, RouterMode::softmax, true); }, "audited batch beyond 2048 rows accepted");
    g.abort();
    refuses([&] { g.configure_router_margin_epsilon(0.f); }, "zero margin epsilon accepted");

    // top-64 rows of the logits just produced, against the oracle's row, bit for bit
    {
        const auto scratch = g.zeros(CudaGraph::logit_topk_scratch_bytes(T, E), "topk scratch"), rows = g.zeros(CudaGraph::logit_topk_output_bytes(T), "topk rows");
        g.begin();
        g.logit_topk({logits, T, E, uint64_t(E) * 4}, scratch, rows);
        (void)g.submit();
        const auto raw = g.read(rows);
        for (uint32_t t = 0; t < T; ++t) {
            tso_topk_row want;
            require(tso_logit_topk_row(gl.data() + size_t(t) * E, E, &want) == TSO_OK, "oracle top-k");
            require(std::memcmp(raw.data() + size_t(t) * sizeof want, &want, sizeof want) == 0, "logit top-k row differs from the oracle");
        }
        g.begin();
        refuses([&] { g.logit_topk({logits, T, E, uint64_t(E) * 4}, g.slice(scratch, 0, 528), rows); }, "short top-k scratch accepted");
        g.abort();
    }
    // residual read / write on one token
    std::vector<double> dn(size_t(B) * C), dsc(size_t(B) * C), dinj(B), dstreams(size_t(B) * C), dout(C);
    const auto fn = activations(seed + 20, size_t(B) * C, 1.5f), fsc = activations(seed + 21, size_t(B) * C, 3.f), finj = activations(seed + 22, B, 2.f);
    const auto fst = activations(seed + 23, size_t(B) * C, 5.f), fo = activations(seed + 24, C, 5.f);
    const auto nv = g.upload(bytes_of(fn), "normalized"), scv = g.upload(bytes_of(fsc), "scores"), iv = g.upload(bytes_of(finj), "inject");
    const auto stv = g.upload(bytes_of(fst), "streams"), ov = g.upload(bytes_of(fo), "ffn out");
    const auto rin = g.zeros(C * 4, "ffn in"), scl = g.zeros(B * 4, "write scales"), dst = g.zeros(uint64_t(B) * C * 4, "streams out");
    g.begin();
    g.residual_read(nv, scv, iv, rin, scl, B, C);
    g.residual_write(stv, ov, scl, dst);
    (void)g.submit();
    std::vector<double> ein(C, 0.0), esc(B), edst(size_t(B) * C);
    for (uint32_t b = 0; b < B; ++b) {
        esc[b] = 2.0 * tso_sigmoid(double(finj[b]) / B);
        for (uint32_t c = 0; c < C; ++c) ein[c] += double(fn[size_t(b) * C + c]) * tso_sigmoid(fsc[size_t(b) * C + c]);
    }
    for (auto& v : ein) v /= B;
    const auto gsc = read<float>(g, scl);
    for (uint32_t b = 0; b < B; ++b) for (uint32_t c = 0; c < C; ++c) edst[size_t(b) * C + c] = double(fst[size_t(b) * C + c]) + double(gsc[b]) * fo[c];
    close(read<float>(g, rin), ein.data(), C);
    close(gsc, esc.data(), B);
    close(read<float>(g, dst), edst.data(), edst.size());
    g.begin();
    refuses([&] { g.residual_read(nv, scv, iv, rin, scl, B + 1, C); }, "residual branch mismatch accepted");
    refuses([&] { g.residual_write(stv, ov, scl, g.slice(dst, 0, uint64_t(C) * 4)); }, "short residual destination accepted");
    g.abort();
}
}  // namespace

int main() {
    try {
        CudaGraph g(0, uint64_t(2) << 30);
        refuses([&] { (void)g.zeros(uint64_t(3) << 30, "too large"); }, "allocation beyond the budget accepted");
        layer(g, 12, true, {256, 256, 8, 4}, 1);
        std::cout << "MoE checks passed so far: " << checks << " (worst scaled error " << worst << ")\n";
    } catch (const std::exception& e) {
        std::cerr << "MoE check failed after " << checks << " checks: " << e.what() << '\n';
        return 1;
    }
    // planar registration is frozen after the first batch of a graph, so every weight form gets its own graph
    // the last case is the reference model's pairing: Q5_K gate / up, Q5_1 down, Q8_0 shared expert (raw GGUF rows)
    const struct { uint32_t type; bool planar; MoeShape shape; uint32_t down = 0, shared = 0; } cases[] = {
        {12, false, {256, 256, 8, 4}}, {8, true, {256, 64, 8, 4}}, {8, false, {64, 64, 6, 3}}, {12, true, {512, 256, 16, 10}},
        {13, false, {512, 256, 8, 4}, 7, 8}};
    uint32_t seed = 50;
    for (const auto& c : cases) {
        try {
            CudaGraph g(0, uint64_t(2) << 30);
            layer(g, c.type, c.planar, c.shape, seed += 10, c.down, c.shared);
        } catch (const std::exception& e) {
            std::cerr << "MoE check failed (type " << c.type << ", planar " << c.planar << ") after " << checks << " checks: " << e.what() << '\n';
            return 1;
        }
    }
    try {
        CudaGraph gv(0, uint64_t(2) << 30);
        verify_rows(gv, 12, {256, 256, 8, 4}, 5, 200);
        verify_rows(gv, 8, {256, 64, 8, 4}, 8, 210);
        CudaGraph g(0, uint64_t(2) << 30);
        many(g, {512, 256, 16, 4}, 40, 24, 300);   // two chunks: 24 + 16 rows
        CudaGraph g2(0, uint64_t(2) << 30);
        many(g2, {512, 256, 8, 2}, 200, 256, 400); // one chunk, tiles of more than 32 routes
        CudaGraph g3(0, uint64_t(1) << 30);
        operators(g3, 500);
        pack_layer(600);
    } catch (const std::exception& e) {
        std::cerr << "tiled MoE check failed after " << checks << " checks: " << e.what() << '\n';
        return 1;
    }
    std::cout << "MoE encode checks passed: " << checks << " (worst scaled error " << worst << ")\n";
    return 0;
}
