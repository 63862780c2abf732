// Decode-size routed / dense projections over the five-bit encodings of the reference's model: Q5_K (176-byte super-blocks of
// 256 weights; gate and up tensors) and Q5_1 (24-byte blocks of 32 weights; down tensors), plain GGUF rows.
//
// One warp owns one weight row (gate-up: the gate row and the up row of one hidden unit) for all token rows of a tile. A lane
// takes one 32-weight group at a time: it decodes the group to the exactly rounded FP32 weights (numeric.cpp:38-50:
// d * sc * q and dmin * mn are exact in FP32, so one FMA gives the reference's rounded value), multiplies them with the tile's
// FP32 activation rows and keeps one FP32 partial sum per token; the warp adds the lanes' sums at the end. Weight bytes are read
// once per (tile, row); no shared memory, no pipeline: a coverage path for the encodings the benchmark configurations do not
// use, not a tuned one.
#include "tsp_common.cuh"

namespace tsp {

constexpr uint32_t kK5Warps = 8;       // weight rows (gate-up: hidden units) per block
constexpr uint32_t kK5MaxTokens = 16;  // token rows of a tile (8 per routed tile, 16 for dense row batches)

struct K5Params {
    const uint8_t* a_base; const uint8_t* a_base_hi; const uint8_t* b_base; const uint8_t* b_base_hi;
    uint64_t expert_stride; uint32_t split, experts;
    uint32_t rows, cols, row_bytes;
    const float* x; uint64_t x_stride_bytes; uint32_t in_div;
    const uint32_t* token_map; const uint32_t* counts; const uint32_t* tasks;
    uint32_t tokens, tile_tokens;
    float* out; uint64_t out_stride_bytes;
    uint32_t* error;
};

// the twelve packed 6-bit factors of a K-quant super-block (numeric.cpp:25-31)
__device__ __forceinline__ void k_factors(const uint8_t* block, uint32_t group, uint32_t& sc, uint32_t& mn) {
    const uint32_t lane = group & 3u;
    if (group < 4) { sc = block[4 + lane] & 63u; mn = block[8 + lane] & 63u; return; }
    const uint32_t packed = block[12 + lane];
    sc = (packed & 15u) | ((block[4 + lane] >> 6) << 4);
    mn = (packed >> 4) | ((block[8 + lane] >> 6) << 4);
}

// The 32 weights of group `grp` of a row, four at a time: f(i4, w[4]) for i4 = 0..7 (weights 4 i4 .. 4 i4 + 3 of the group).
template <uint32_t TYPE, typename F>
__device__ __forceinline__ bool decode_group(const uint8_t* row, uint32_t grp, F&& f) {
    if (TYPE == 13u) {   // Q5_K
        const uint8_t* block = row + (grp >> 3) * 176u;
        const uint32_t g = grp & 7u;
        const uint32_t dm = *reinterpret_cast<const uint32_t*>(block);
        const float d = half_bits_to_float(dm & 0xffffu), dmin = half_bits_to_float(dm >> 16);
        uint32_t sc, mn;
        k_factors(block, g, sc, mn);
        const float s = d * static_cast<float>(sc), m = -(dmin * static_cast<float>(mn));   // both exact
        const uint32_t* qs = reinterpret_cast<const uint32_t*>(block + 48 + (g >> 1) * 32);
        const uint32_t* qh = reinterpret_cast<const uint32_t*>(block + 16);
        const uint32_t shift = 4u * (g & 1u);
#pragma unroll
        for (uint32_t i4 = 0; i4 < 8; ++i4) {
            const uint32_t lo = (qs[i4] >> shift) & 0x0f0f0f0fu, hi = ((qh[i4] >> g) & 0x01010101u) << 4;
            const uint32_t q = lo | hi;
            const float w[4] = {fmaf(s, static_cast<float>(q & 255u), m), fmaf(s, static_cast<float>((q >> 8) & 255u), m),
                                fmaf(s, static_cast<float>((q >> 16) & 255u), m), fmaf(s, static_cast<float>(q >> 24), m)};
            f(i4, w);
        }
        return finite_f32(d) && finite_f32(dmin);
    } else {             // Q5_1
        const uint8_t* block = row + grp * 24u;
        const uint32_t dm = *reinterpret_cast<const uint32_t*>(block);
        const float d = half_bits_to_float(dm & 0xffffu), m = half_bits_to_float(dm >> 16);
        const uint32_t qh = *reinterpret_cast<const uint32_t*>(block + 4);
        const uint32_t* qs = reinterpret_cast<const uint32_t*>(block + 8);
#pragma unroll
        for (uint32_t i4 = 0; i4 < 8; ++i4) {
            // weight i: nibble (i / 16) of byte i % 16, fifth bit = bit i of qh
            const uint32_t word = qs[i4 & 3u] >> (4u * (i4 >> 2));
            const uint32_t hb = (qh >> (4u * i4)) & 15u;
            const uint32_t q0 = (word & 15u) | ((hb & 1u) << 4), q1 = ((word >> 8) & 15u) | ((hb & 2u) << 3);
            const uint32_t q2 = ((word >> 16) & 15u) | ((hb & 4u) << 2), q3 = ((word >> 24) & 15u) | ((hb & 8u) << 1);
            const float w[4] = {fmaf(d, static_cast<float>(q0), m), fmaf(d, static_cast<float>(q1), m),
                                fmaf(d, static_cast<float>(q2), m), fmaf(d, static_cast<float>(q3), m)};
            f(i4, w);
        }
        return finite_f32(d) && finite_f32(m);
    }
}

template <uint32_t TYPE, bool GATEUP>
__global__ void __launch_bounds__(kK5Warps * 32) gemv_k5_kernel(const K5Params p) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ uint32_t s_rid[kK5MaxTokens];
    __shared__ uint32_t s_tile[3];
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t n_tiles = p.token_map ? p.tasks[0] : (p.tokens + p.tile_tokens - 1) / p.tile_tokens;
    const uint32_t r = blockIdx.x * kK5Warps + warp;
    const uint32_t groups = p.cols / 32u;
    for (uint32_t tile = blockIdx.y; tile < n_tiles; tile += gridDim.y) {   // uniform over the block
        __syncthreads();   // the previous tile's route ids are no longer read
        if (threadIdx.x == 0) {
            uint32_t expert = 0, start = tile * p.tile_tokens, count = 0;
            if (p.token_map) {
                expert = p.tasks[2 + 2 * tile];
                start = p.tasks[3 + 2 * tile];
                if (expert < p.experts) { const uint32_t c = p.counts[expert]; count = c > start ? min(c - start, p.tile_tokens) : 0u; }
                else expert = 0;
            } else if (start < p.tokens) count = min(p.tokens - start, p.tile_tokens);
            s_tile[0] = expert; s_tile[1] = start; s_tile[2] = count;
        }
        __syncthreads();
        const uint32_t expert = s_tile[0], start = s_tile[1], count = s_tile[2];
        if (threadIdx.x < count)
            s_rid[threadIdx.x] = p.token_map ? p.token_map[static_cast<uint64_t>(expert) * p.tokens + start + threadIdx.x] : start + threadIdx.x;
        __syncthreads();
        if (count == 0 || r >= p.rows) continue;
        const bool hi = expert >= p.split;
        const uint64_t eoff = static_cast<uint64_t>(hi ? expert - p.split : expert) * p.expert_stride + static_cast<uint64_t>(r) * p.row_bytes;
        const uint8_t* rowA = (hi ? p.a_base_hi : p.a_base) + eoff;
        const uint8_t* rowB = GATEUP ? (hi ? p.b_base_hi : p.b_base) + eoff : nullptr;

        float accA[kK5MaxTokens], accB[GATEUP ? kK5MaxTokens : 1];
#pragma unroll
        for (uint32_t j = 0; j < kK5MaxTokens; ++j) { accA[j] = 0.f; if (GATEUP) accB[j] = 0.f; }
        bool ok = true, xbad = false;
        for (uint32_t grp = lane; grp < groups; grp += 32) {
            float wa[32], wb[GATEUP ? 32 : 1];
            ok &= decode_group<TYPE>(rowA, grp, [&](uint32_t i4, const float (&w)[4]) { wa[4 * i4] = w[0]; wa[4 * i4 + 1] = w[1]; wa[4 * i4 + 2] = w[2]; wa[4 * i4 + 3] = w[3]; });
            if (GATEUP)
                ok &= decode_group<TYPE>(rowB, grp, [&](uint32_t i4, const float (&w)[4]) { wb[4 * i4] = w[0]; wb[4 * i4 + 1] = w[1]; wb[4 * i4 + 2] = w[2]; wb[4 * i4 + 3] = w[3]; });
#pragma unroll
            for (uint32_t j = 0; j < kK5MaxTokens; ++j) {
                if (j >= count) break;
                const float4* xr = reinterpret_cast<const float4*>(reinterpret_cast<const char*>(p.x) + static_cast<uint64_t>(s_rid[j] / p.in_div) * p.x_stride_bytes) + grp * 8u;
                float sa = 0.f, sb = 0.f;
#pragma unroll
                for (uint32_t i4 = 0; i4 < 8; ++i4) {
                    const float4 v = xr[i4];
                    xbad |= !finite_f32(v.x) | !finite_f32(v.y) | !finite_f32(v.z) | !finite_f32(v.w);
                    sa = fmaf(wa[4 * i4], v.x, sa); sa = fmaf(wa[4 * i4 + 1], v.y, sa); sa = fmaf(wa[4 * i4 + 2], v.z, sa); sa = fmaf(wa[4 * i4 + 3], v.w, sa);
                    if (GATEUP) { sb = fmaf(wb[4 * i4], v.x, sb); sb = fmaf(wb[4 * i4 + 1], v.y, sb); sb = fmaf(wb[4 * i4 + 2], v.z, sb); sb = fmaf(wb[4 * i4 + 3], v.w, sb); }
                }
                accA[j] += sa;
                if (GATEUP) accB[j] += sb;
            }
        }
        if (!ok || xbad) raise_error(p.error, TSP_ERR_NONFINITE);
#pragma unroll
        for (uint32_t j = 0; j < kK5MaxTokens; ++j) {
            if (j >= count) break;
            float a = accA[j], b = GATEUP ? accB[j] : 0.f;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) { a += __shfl_xor_sync(0xffffffffu, a, o); if (GATEUP) b += __shfl_xor_sync(0xffffffffu, b, o); }
            if (lane == 0) {
                // silu with the branch-stable sigmoid (operators.cpp:28-36)
                const float v = GATEUP ? (a >= 0.f ? a / (1.f + expf(-a)) : a * expf(a) / (1.f + expf(a))) * b : a;
                if (!finite_f32(v)) raise_error(p.error, TSP_ERR_NONFINITE);
                reinterpret_cast<float*>(reinterpret_cast<char*>(p.out) + static_cast<uint64_t>(s_rid[j]) * p.out_stride_bytes)[r] = v;
            }
        }
    }
}

// Exactly rounded FP32 weights of one matrix (test hook)
template <uint32_t TYPE>
__global__ void __launch_bounds__(256) dequant_k5_kernel(const uint8_t* __restrict__ m, uint64_t groups, float* __restrict__ out, uint32_t* error) {
    const uint64_t grp = static_cast<uint64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (grp >= groups) return;
    // a "row" of one super-block / block: decode_group indexes blocks from the pointer it is given
    const uint8_t* base = TYPE == 13u ? m + (grp >> 3) * 176u : m + grp * 24u;
    float* dst = out + grp * 32;
    const bool ok = decode_group<TYPE>(base, TYPE == 13u ? static_cast<uint32_t>(grp & 7u) : 0u,
                                       [&](uint32_t i4, const float (&w)[4]) { reinterpret_cast<float4*>(dst)[i4] = make_float4(w[0], w[1], w[2], w[3]); });
    if (!ok) raise_error(error, TSP_ERR_NONFINITE);
}

int launch_dequant_k5(uint32_t type, const uint8_t* m, uint64_t elements, float* out, uint32_t* error, cudaStream_t st) {
    const uint64_t groups = elements / 32;
    const unsigned grid = static_cast<unsigned>((groups + 255) / 256);
    if (type == TSP_TYPE_Q5_K) dequant_k5_kernel<13u><<<grid, 256, 0, st>>>(m, groups, out, error);
    else dequant_k5_kernel<7u><<<grid, 256, 0, st>>>(m, groups, out, error);
    TSP_CUDA(cudaGetLastError());
    return TSP_OK;
}

int launch_gemv_k5(const tsp_matrix_set* a, const tsp_matrix_set* b, bool gateup, const float* x, uint64_t x_stride_bytes, uint32_t in_div,
                   uint32_t tokens, const uint32_t* token_map, const uint32_t* counts, const uint32_t* tasks, float* out,
                   uint64_t out_stride_bytes, int nc, uint32_t* error, cudaStream_t st) {
    if (a->layout != TSP_LAYOUT_GGUF) return fail(TSP_E_TYPE, "five-bit encodings are read as plain GGUF rows only");
    K5Params p{};
    p.a_base = static_cast<const uint8_t*>(a->base);
    p.a_base_hi = static_cast<const uint8_t*>(a->base_hi ? a->base_hi : a->base);
    if (gateup) {
        p.b_base = static_cast<const uint8_t*>(b->base);
        p.b_base_hi = static_cast<const uint8_t*>(b->base_hi ? b->base_hi : b->base);
    }
    p.expert_stride = a->expert_stride;
    p.split = a->split < a->experts ? a->split : a->experts;
    p.experts = a->experts;
    p.rows = a->rows; p.cols = a->cols;
    p.row_bytes = a->type == TSP_TYPE_Q5_K ? a->cols / 256 * 176 : a->cols / 32 * 24;
    p.x = x; p.x_stride_bytes = x_stride_bytes; p.in_div = in_div ? in_div : 1;
    p.token_map = token_map; p.counts = counts; p.tasks = tasks;
    p.tokens = tokens; p.tile_tokens = 8u * static_cast<uint32_t>(nc);
    p.out = out; p.out_stride_bytes = out_stride_bytes; p.error = error;
    // routed launches learn their tile count on the device: a fixed number of block rows walks the tiles
    const uint32_t dense_tiles = (tokens + p.tile_tokens - 1) / p.tile_tokens;
    const int sms = sm_count();
    if (sms <= 0) return fail(TSP_E_CUDA, "no usable CUDA device");
    const dim3 grid((a->rows + kK5Warps - 1) / kK5Warps, token_map ? static_cast<unsigned>(sms) : (dense_tiles < 1024u ? dense_tiles : 1024u)), block(kK5Warps * 32);
    if (a->type == TSP_TYPE_Q5_K) {
        if (gateup) TSP_CUDA(launch_pdl(gemv_k5_kernel<13u, true>, grid, block, 0, st, p));
        else TSP_CUDA(launch_pdl(gemv_k5_kernel<13u, false>, grid, block, 0, st, p));
    } else {
        if (gateup) TSP_CUDA(launch_pdl(gemv_k5_kernel<7u, true>, grid, block, 0, st, p));
        else TSP_CUDA(launch_pdl(gemv_k5_kernel<7u, false>, grid, block, 0, st, p));
    }
    return TSP_OK;
}

}  // namespace tsp
