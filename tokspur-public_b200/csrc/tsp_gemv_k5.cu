// Decode-size routed / dense projections over the five-bit encodings of the reference's model: Q5_K (176-byte super-blocks of
// 256 weights; gate and up tensors) and Q5_1 (24-byte blocks of 32 weights; down tensors), plain GGUF rows.
//
// One thread owns one weight row (gate-up: the gate row and the up row of one hidden unit) for all token rows of a tile and walks
// its K extent: it decodes 32-weight groups to the exactly rounded FP32 weights (numeric.cpp:38-50: d * sc * q and dmin * mn
// are exact in FP32, so one FMA gives the reference's rounded value), multiplies them with the tile's FP32 activation rows (the
// lanes of a warp read the same activation values: broadcast loads) and keeps one FP32 sum per token. Weight bytes are read once
// per (tile, row); no shared-memory staging, no copy pipeline: a plain path for the encodings the benchmark configurations do
// not use.
#include "tsp_common.cuh"

namespace tsp {

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

// byte k of `q` as a float: 0x4B0000bb is 2^23 + bb, the subtraction is exact (no integer-to-float conversion instruction)
template <uint32_t K>
__device__ __forceinline__ float byte_f32(uint32_t q) { return __uint_as_float(__byte_perm(q, 0x4b000000u, 0x7440u + K)) - 8388608.f; }

// One 32-weight group of a row, opened once (scale, offset, code pointers) and then read four weights at a time:
// get(i4, w) gives weights 4 i4 .. 4 i4 + 3 of the group as the exactly rounded FP32 values.
template <uint32_t TYPE> struct Group5;
template <> struct Group5<13u> {   // Q5_K
    float s, m; const uint32_t* qs; const uint32_t* qh; uint32_t shift, g; bool finite;
    __device__ __forceinline__ Group5(const uint8_t* row, uint32_t grp) {
        const uint8_t* block = row + (grp >> 3) * 176u;
        g = grp & 7u;
        const uint32_t dm = *reinterpret_cast<const uint32_t*>(block);
        const float d = half_bits_to_float(dm & 0xffffu), dmin = half_bits_to_float(dm >> 16);
        uint32_t sc, mn;
        k_factors(block, g, sc, mn);
        s = d * static_cast<float>(sc); m = -(dmin * static_cast<float>(mn));   // both exact
        qs = reinterpret_cast<const uint32_t*>(block + 48 + (g >> 1) * 32);
        qh = reinterpret_cast<const uint32_t*>(block + 16);
        shift = 4u * (g & 1u);
        finite = finite_f32(d) && finite_f32(dmin);
    }
    __device__ __forceinline__ void get(uint32_t i4, float (&w)[4]) const {
        const uint32_t q = ((qs[i4] >> shift) & 0x0f0f0f0fu) | (((qh[i4] >> g) & 0x01010101u) << 4);
        w[0] = fmaf(s, byte_f32<0>(q), m); w[1] = fmaf(s, byte_f32<1>(q), m); w[2] = fmaf(s, byte_f32<2>(q), m); w[3] = fmaf(s, byte_f32<3>(q), m);
    }
};
template <> struct Group5<7u> {    // Q5_1
    float d, m; uint32_t qh; uint32_t qs[4]; bool finite;
    __device__ __forceinline__ Group5(const uint8_t* row, uint32_t grp) {
        const uint2* block = reinterpret_cast<const uint2*>(row + grp * 24u);   // 24-byte blocks of 8-byte aligned rows: three 8-byte loads
        const uint2 h = block[0], q01 = block[1], q23 = block[2];
        d = half_bits_to_float(h.x & 0xffffu); m = half_bits_to_float(h.x >> 16);
        qh = h.y;
        qs[0] = q01.x; qs[1] = q01.y; qs[2] = q23.x; qs[3] = q23.y;
        finite = finite_f32(d) && finite_f32(m);
    }
    __device__ __forceinline__ void get(uint32_t i4, float (&w)[4]) const {
        // weight i: nibble (i / 16) of byte i % 16, fifth bit = bit i of qh
        const uint32_t hb = (qh >> (4u * i4)) & 15u;
        // the four fifth bits spread to bit 4 of each byte: bit k of hb -> bit 8 k + 4
        const uint32_t q = ((qs[i4 & 3u] >> (4u * (i4 >> 2))) & 0x0f0f0f0fu) | (((hb * 0x00204081u) & 0x01010101u) << 4);
        w[0] = fmaf(d, byte_f32<0>(q), m); w[1] = fmaf(d, byte_f32<1>(q), m); w[2] = fmaf(d, byte_f32<2>(q), m); w[3] = fmaf(d, byte_f32<3>(q), m);
    }
};

// Four lanes own one weight row (gate-up: the gate row and the up row of one hidden unit) of a tile: lane q of the four takes the
// units of 128 weights q, q + 4, ... of the row and the four add their sums with two shuffles. A warp covers eight rows, and its
// lanes read four distinct activation addresses per load. MT: token rows of a tile at most (8 routed, 16 dense batches).
constexpr uint32_t kK5Threads = 128, kK5Lanes = 4, kK5Rows = kK5Threads / kK5Lanes;

// A non-finite activation makes the sums it enters non-finite (0 * inf is NaN), so the finished sums are checked, not the inputs.
template <bool GATEUP, uint32_t MT>
struct K5Acc {
    float a[MT], b[GATEUP ? MT : 1];
    uint32_t xo[MT];   // the tile's input rows as float4 offsets from the first row buffer
    // four weights of matrix A (and B) against the tile's activation values at float4 index `at`
    __device__ __forceinline__ void add(const float (&wa)[4], const float (&wb)[4], const float4* x0, uint32_t at, uint32_t count) {
#pragma unroll
        for (uint32_t j = 0; j < MT; ++j) {
            if (j >= count) break;
            const float4 v = x0[xo[j] + at];
            a[j] = fmaf(wa[0], v.x, a[j]); a[j] = fmaf(wa[1], v.y, a[j]); a[j] = fmaf(wa[2], v.z, a[j]); a[j] = fmaf(wa[3], v.w, a[j]);
            if (GATEUP) { b[j] = fmaf(wb[0], v.x, b[j]); b[j] = fmaf(wb[1], v.y, b[j]); b[j] = fmaf(wb[2], v.z, b[j]); b[j] = fmaf(wb[3], v.w, b[j]); }
        }
    }
};

// factors of group g from the header words (y, z, w = the twelve packed bytes), numeric.cpp:25-31
__device__ __forceinline__ void k_factors_w(const uint4& h, uint32_t g, uint32_t& sc, uint32_t& mn) {
    const uint32_t sh = 8u * (g & 3u);
    const uint32_t by = (h.y >> sh) & 255u, bz = (h.z >> sh) & 255u, bw = (h.w >> sh) & 255u;
    if (g < 4) { sc = by & 63u; mn = bz & 63u; }
    else { sc = (bw & 15u) | ((by >> 6) << 4); mn = (bw >> 4) | ((bz >> 6) << 4); }
}

// group g (a run-time value: one copy of this code serves the eight groups, the unrolled token loops are large)
template <bool GATEUP, uint32_t MT>
__device__ __forceinline__ void q5k_group(uint32_t g, const uint8_t* blkA, const uint8_t* blkB, const uint4& hA, const uint4& hB, const uint4 (&qhA)[2],
                                          const uint4 (&qhB)[2], K5Acc<GATEUP, MT>& acc, const float4* x0, uint32_t at0, uint32_t count) {
    uint32_t sc, mn;
    k_factors_w(hA, g, sc, mn);
    const float sA = half_bits_to_float(hA.x & 0xffffu) * static_cast<float>(sc), mA = -(half_bits_to_float(hA.x >> 16) * static_cast<float>(mn));
    float sB = 0.f, mB = 0.f;
    if (GATEUP) {
        k_factors_w(hB, g, sc, mn);
        sB = half_bits_to_float(hB.x & 0xffffu) * static_cast<float>(sc); mB = -(half_bits_to_float(hB.x >> 16) * static_cast<float>(mn));
    }
    const uint4* qsA = reinterpret_cast<const uint4*>(blkA + 48 + (g >> 1) * 32);
    const uint4* qsB = reinterpret_cast<const uint4*>(blkB + 48 + (g >> 1) * 32);
    const uint32_t nib = 4u * (g & 1u);
#pragma unroll
    for (uint32_t h = 0; h < 2; ++h) {
        const uint4 ca = qsA[h], cb = GATEUP ? qsB[h] : make_uint4(0, 0, 0, 0);
        const uint32_t wa_[4] = {ca.x, ca.y, ca.z, ca.w}, wb_[4] = {cb.x, cb.y, cb.z, cb.w};
        const uint32_t ha_[4] = {qhA[h].x, qhA[h].y, qhA[h].z, qhA[h].w}, hb_[4] = {qhB[h].x, qhB[h].y, qhB[h].z, qhB[h].w};
#pragma unroll
        for (uint32_t k = 0; k < 4; ++k) {
            const uint32_t qa = ((wa_[k] >> nib) & 0x0f0f0f0fu) | (((ha_[k] >> g) & 0x01010101u) << 4);
            const uint32_t qb = ((wb_[k] >> nib) & 0x0f0f0f0fu) | (((hb_[k] >> g) & 0x01010101u) << 4);
            const float wa[4] = {fmaf(sA, byte_f32<0>(qa), mA), fmaf(sA, byte_f32<1>(qa), mA), fmaf(sA, byte_f32<2>(qa), mA), fmaf(sA, byte_f32<3>(qa), mA)};
            const float wb[4] = {fmaf(sB, byte_f32<0>(qb), mB), fmaf(sB, byte_f32<1>(qb), mB), fmaf(sB, byte_f32<2>(qb), mB), fmaf(sB, byte_f32<3>(qb), mB)};
            acc.add(wa, wb, x0, at0 + g * 8u + h * 4u + k, count);
        }
    }
}

template <uint32_t TYPE, bool GATEUP, uint32_t MT>
__global__ void __launch_bounds__(kK5Threads) gemv_k5_kernel(const K5Params p) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ uint32_t s_x[kK5MaxTokens];        // the tile's input rows as float4 offsets from p.x
    __shared__ float* s_out[kK5MaxTokens];        // and its output rows
    __shared__ uint32_t s_tile[3];
    const uint32_t n_tiles = p.token_map ? p.tasks[0] : (p.tokens + p.tile_tokens - 1) / p.tile_tokens;
    const uint32_t q = threadIdx.x & (kK5Lanes - 1u), r = blockIdx.x * kK5Rows + threadIdx.x / kK5Lanes;
    for (uint32_t tile = blockIdx.y; tile < n_tiles; tile += gridDim.y) {   // uniform over the block
        __syncthreads();   // the previous tile's rows are no longer read
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
        const uint32_t expert = s_tile[0], start = s_tile[1], count = min(s_tile[2], MT);
        if (threadIdx.x < count) {
            const uint32_t rid = p.token_map ? p.token_map[static_cast<uint64_t>(expert) * p.tokens + start + threadIdx.x] : start + threadIdx.x;
            s_x[threadIdx.x] = static_cast<uint32_t>(static_cast<uint64_t>(rid / p.in_div) * p.x_stride_bytes / 16u);
            s_out[threadIdx.x] = reinterpret_cast<float*>(reinterpret_cast<char*>(p.out) + static_cast<uint64_t>(rid) * p.out_stride_bytes);
        }
        __syncthreads();
        if (count == 0 || r >= p.rows) continue;   // uniform over a warp: its eight rows start at a multiple of eight, and so does rows
        const bool hi = expert >= p.split;
        const uint64_t eoff = static_cast<uint64_t>(hi ? expert - p.split : expert) * p.expert_stride + static_cast<uint64_t>(r) * p.row_bytes;
        const uint8_t* rowA = (hi ? p.a_base_hi : p.a_base) + eoff;
        const uint8_t* rowB = GATEUP ? (hi ? p.b_base_hi : p.b_base) + eoff : rowA;

        K5Acc<GATEUP, MT> acc;
#pragma unroll
        for (uint32_t j = 0; j < MT; ++j) { acc.a[j] = 0.f; if (GATEUP) acc.b[j] = 0.f; acc.xo[j] = j < count ? s_x[j] : 0u; }
        const float4* x0 = reinterpret_cast<const float4*>(p.x);
        bool ok = true;
        if constexpr (TYPE == 13u) {
            for (uint32_t unit = q; unit < p.cols / 128u; unit += kK5Lanes) {   // half a super-block: groups 0..3 or 4..7
                const uint32_t blk = unit >> 1;
                const uint8_t* bA = rowA + blk * 176u;
                const uint8_t* bB = rowB + blk * 176u;
                const uint4 hA = *reinterpret_cast<const uint4*>(bA), hB = *reinterpret_cast<const uint4*>(bB);
                const uint4 qhA[2] = {reinterpret_cast<const uint4*>(bA + 16)[0], reinterpret_cast<const uint4*>(bA + 16)[1]};
                const uint4 qhB[2] = {reinterpret_cast<const uint4*>(bB + 16)[0], reinterpret_cast<const uint4*>(bB + 16)[1]};
                ok &= (hA.x & 0x7c00u) != 0x7c00u && (hA.x & 0x7c000000u) != 0x7c000000u && (hB.x & 0x7c00u) != 0x7c00u && (hB.x & 0x7c000000u) != 0x7c000000u;
                const uint32_t at0 = blk * 64u;
                const uint32_t g0 = (unit & 1u) * 4u;
#pragma unroll 1
                for (uint32_t g = g0; g < g0 + 4u; ++g) q5k_group<GATEUP, MT>(g, bA, bB, hA, hB, qhA, qhB, acc, x0, at0, count);
            }
        } else {
            for (uint32_t unit = q; unit < (p.cols + 127u) / 128u; unit += kK5Lanes)
                for (uint32_t grp = unit * 4u; grp < unit * 4u + 4u && grp < p.cols / 32u; ++grp) {
                    const Group5<7u> ga(rowA, grp), gb(rowB, grp);
                    ok &= ga.finite & gb.finite;
#pragma unroll
                    for (uint32_t i4 = 0; i4 < 8; ++i4) {
                        float wa[4], wb[4] = {0.f, 0.f, 0.f, 0.f};
                        ga.get(i4, wa);
                        if (GATEUP) gb.get(i4, wb);
                        acc.add(wa, wb, x0, grp * 8u + i4, count);
                    }
                }
        }
        if (!ok) raise_error(p.error, TSP_ERR_NONFINITE);
#pragma unroll
        for (uint32_t j = 0; j < MT; ++j) {
            if (j >= count) break;
            float a = acc.a[j], b = GATEUP ? acc.b[j] : 0.f;
            a += __shfl_xor_sync(0xffffffffu, a, 1); a += __shfl_xor_sync(0xffffffffu, a, 2);
            if (GATEUP) { b += __shfl_xor_sync(0xffffffffu, b, 1); b += __shfl_xor_sync(0xffffffffu, b, 2); }
            if (q == 0) {
                // silu with the branch-stable sigmoid (operators.cpp:28-36)
                const float v = GATEUP ? (a >= 0.f ? a / (1.f + expf(-a)) : a * expf(a) / (1.f + expf(a))) * b : a;
                if (!finite_f32(v)) raise_error(p.error, TSP_ERR_NONFINITE);
                s_out[j][r] = v;
            }
        }
    }
}

// Exactly rounded FP32 weights of one matrix (test hook)
template <uint32_t TYPE>
__global__ void __launch_bounds__(256) dequant_k5_kernel(const uint8_t* __restrict__ m, uint64_t groups, float* __restrict__ out, uint32_t* error) {
    const uint64_t grp = static_cast<uint64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (grp >= groups) return;
    // Group5 indexes blocks from the pointer it is given: hand it this group's own block
    const Group5<TYPE> g(TYPE == 13u ? m + (grp >> 3) * 176u : m + grp * 24u, TYPE == 13u ? static_cast<uint32_t>(grp & 7u) : 0u);
    float4* dst = reinterpret_cast<float4*>(out + grp * 32);
#pragma unroll
    for (uint32_t i4 = 0; i4 < 8; ++i4) { float w[4]; g.get(i4, w); dst[i4] = make_float4(w[0], w[1], w[2], w[3]); }
    if (!g.finite) raise_error(error, TSP_ERR_NONFINITE);
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
    if (nc != 1 && nc != 2) return fail(TSP_E_ARG, "five-bit projection: tiles hold 8 or 16 token rows");
    // routed launches learn their tile count on the device: a fixed number of block rows walks the tiles
    const uint32_t dense_tiles = (tokens + p.tile_tokens - 1) / p.tile_tokens;
    const int sms = sm_count();
    if (sms <= 0) return fail(TSP_E_CUDA, "no usable CUDA device");
    // a routed launch has at most 64 routes per token row (selected <= 64), one tile each at worst
    const uint64_t routed_cap = static_cast<uint64_t>(tokens) * 64u;
    const uint32_t walkers = static_cast<uint32_t>(routed_cap < 4u * static_cast<uint32_t>(sms) ? routed_cap : 4u * static_cast<uint32_t>(sms));
    const dim3 grid((a->rows + kK5Rows - 1) / kK5Rows, token_map ? walkers : (dense_tiles < 1024u ? dense_tiles : 1024u)), block(kK5Threads);
#define TSP_K5(T, G) (nc == 1 ? launch_pdl(gemv_k5_kernel<T, G, 8u>, grid, block, 0, st, p) : launch_pdl(gemv_k5_kernel<T, G, 16u>, grid, block, 0, st, p))
    if (a->type == TSP_TYPE_Q5_K) TSP_CUDA(gateup ? TSP_K5(13u, true) : TSP_K5(13u, false));
    else TSP_CUDA(gateup ? TSP_K5(7u, true) : TSP_K5(7u, false));
#undef TSP_K5
    return TSP_OK;
}

}  // namespace tsp
