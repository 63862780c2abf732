// Decode-size routed / dense projections over the five-bit encodings of the reference's model: Q5_K (176-byte super-blocks of
// 256 weights; gate and up tensors) and Q5_1 (24-byte blocks of 32 weights; down tensors), plain GGUF rows.
//
// A block takes one token tile and a run of weight rows. It first stages the tile's FP32 activation rows in shared memory
// (32-value groups padded to 36 values, so that 32 lanes reading 16 bytes each at a group stride touch every bank equally). Then
// the lanes of a warp spread over the K extent of one weight row (gate-up: the gate row and the up row of one hidden unit): a
// lane takes one 32-weight group at a time with 16-byte loads that are contiguous across the warp, decodes it to the exactly
// rounded FP32 weights (numeric.cpp:38-50: d * sc * q and dmin * mn are exact in FP32, so one FMA gives the reference's rounded
// value), multiplies with the staged activations and keeps one FP32 sum per token; the lanes' sums are added with shuffles.
// Weight bytes are read once per (tile, row). FP32 FMAs, no tensor cores, no copy pipeline: a plain path for the encodings the
// benchmark configurations do not use.
#include "tsp_common.cuh"

namespace tsp {

constexpr uint32_t kK5MaxTokens = 16;   // token rows of a tile (8 per routed tile, 16 for dense row batches)
constexpr uint32_t kK5Threads = 256;    // eight warps
constexpr uint32_t kK5BlockRows = 64;   // weight rows (hidden units) per block and tile

struct K5Params {
    const uint8_t* a_base; const uint8_t* a_base_hi; const uint8_t* b_base; const uint8_t* b_base_hi;
    uint64_t expert_stride; uint32_t split, experts;
    uint32_t rows, cols, row_bytes;
    const float* x; uint64_t x_stride_bytes; uint32_t in_div;
    const uint32_t* token_map; const uint32_t* counts; const uint32_t* tasks;
    uint32_t tokens, tile_tokens;
    uint32_t lanes_per_row;   // lanes that share one weight row: the largest power of two <= min(32, groups)
    float* out; uint64_t out_stride_bytes;
    uint32_t* error;
};

// byte k of `q` as a float: 0x4B0000bb is 2^23 + bb, the subtraction is exact (no integer-to-float conversion instruction)
template <uint32_t K>
__device__ __forceinline__ float byte_f32(uint32_t q) { return __uint_as_float(__byte_perm(q, 0x4b000000u, 0x7440u + K)) - 8388608.f; }

// One 32-weight group of a row, fetched with wide loads and then read four weights at a time: get(i4, w) gives weights
// 4 i4 .. 4 i4 + 3 of the group as the exactly rounded FP32 values.
template <uint32_t TYPE> struct Group5;
template <> struct Group5<13u> {   // Q5_K: header (d, dmin, twelve factor bytes), 32 bytes of fifth bits, 128 bytes of nibbles
    float s, m; uint32_t qs[8], qh[8]; uint32_t shift, g; bool finite;
    __device__ __forceinline__ Group5(const uint8_t* row, uint32_t grp) {
        const uint8_t* block = row + (grp >> 3) * 176u;
        g = grp & 7u;
        const uint4 h = *reinterpret_cast<const uint4*>(block);
        const uint4 h0 = reinterpret_cast<const uint4*>(block + 16)[0], h1 = reinterpret_cast<const uint4*>(block + 16)[1];
        const uint4 q0 = reinterpret_cast<const uint4*>(block + 48 + (g >> 1) * 32)[0], q1 = reinterpret_cast<const uint4*>(block + 48 + (g >> 1) * 32)[1];
        qh[0] = h0.x; qh[1] = h0.y; qh[2] = h0.z; qh[3] = h0.w; qh[4] = h1.x; qh[5] = h1.y; qh[6] = h1.z; qh[7] = h1.w;
        qs[0] = q0.x; qs[1] = q0.y; qs[2] = q0.z; qs[3] = q0.w; qs[4] = q1.x; qs[5] = q1.y; qs[6] = q1.z; qs[7] = q1.w;
        // factors of group g from the header words (y, z, w = the twelve packed bytes), numeric.cpp:25-31
        const uint32_t sh = 8u * (g & 3u);
        const uint32_t by = (h.y >> sh) & 255u, bz = (h.z >> sh) & 255u, bw = (h.w >> sh) & 255u;
        const uint32_t sc = g < 4 ? (by & 63u) : ((bw & 15u) | ((by >> 6) << 4));
        const uint32_t mn = g < 4 ? (bz & 63u) : ((bw >> 4) | ((bz >> 6) << 4));
        const float d = half_bits_to_float(h.x & 0xffffu), dmin = half_bits_to_float(h.x >> 16);
        s = d * static_cast<float>(sc); m = -(dmin * static_cast<float>(mn));   // both exact
        shift = 4u * (g & 1u);
        finite = finite_f32(d) && finite_f32(dmin);
    }
    __device__ __forceinline__ void get(uint32_t i4, float (&w)[4]) const {
        const uint32_t q = ((qs[i4] >> shift) & 0x0f0f0f0fu) | (((qh[i4] >> g) & 0x01010101u) << 4);
        w[0] = fmaf(s, byte_f32<0>(q), m); w[1] = fmaf(s, byte_f32<1>(q), m); w[2] = fmaf(s, byte_f32<2>(q), m); w[3] = fmaf(s, byte_f32<3>(q), m);
    }
};
template <> struct Group5<7u> {    // Q5_1: d, m, 32 fifth bits, 16 bytes of nibbles
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

// MT: token rows of a tile at most (8 for routed tiles, 16 for dense row batches of more than 8 rows).
// Shared memory: the tile's rows as [token][group][9 float4] (eight of data, one of padding).
template <uint32_t TYPE, bool GATEUP, uint32_t MT>
__global__ void __launch_bounds__(kK5Threads) gemv_k5_kernel(const K5Params p) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float4 k5_xs[];
    __shared__ const float4* s_x[kK5MaxTokens];   // the tile's input rows
    __shared__ float* s_out[kK5MaxTokens];        // and its output rows
    __shared__ uint32_t s_tile[3];
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t n_tiles = p.token_map ? p.tasks[0] : (p.tokens + p.tile_tokens - 1) / p.tile_tokens;
    const uint32_t groups = p.cols / 32u;
    const uint32_t lpr = p.lanes_per_row, rpw = 32u / lpr;    // lanes per row, rows per warp
    const uint32_t sub = lane / lpr, lig = lane & (lpr - 1u); // this lane's row of the warp's rows, its first group
    const uint32_t row0 = blockIdx.x * kK5BlockRows;
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
        if (count == 0) continue;   // uniform
        if (threadIdx.x < count) {
            const uint32_t rid = p.token_map ? p.token_map[static_cast<uint64_t>(expert) * p.tokens + start + threadIdx.x] : start + threadIdx.x;
            s_x[threadIdx.x] = reinterpret_cast<const float4*>(reinterpret_cast<const char*>(p.x) + static_cast<uint64_t>(rid / p.in_div) * p.x_stride_bytes);
            s_out[threadIdx.x] = reinterpret_cast<float*>(reinterpret_cast<char*>(p.out) + static_cast<uint64_t>(rid) * p.out_stride_bytes);
        }
        __syncthreads();
        // stage the activation rows: consecutive threads read consecutive 16-byte pieces of a row
        for (uint32_t i = threadIdx.x; i < count * groups * 8u; i += kK5Threads) {
            const uint32_t j = i / (groups * 8u), rem = i - j * groups * 8u;
            k5_xs[(j * groups + (rem >> 3)) * 9u + (rem & 7u)] = s_x[j][rem];
        }
        __syncthreads();
        const bool hi = expert >= p.split;
        const uint64_t eoff = static_cast<uint64_t>(hi ? expert - p.split : expert) * p.expert_stride;
        const uint8_t* baseA = (hi ? p.a_base_hi : p.a_base) + eoff;
        const uint8_t* baseB = GATEUP ? (hi ? p.b_base_hi : p.b_base) + eoff : baseA;
        bool ok = true;
        // the warps take the block's rows in turn, `rpw` rows at a time (uniform trip count over the warp: shuffles inside)
        for (uint32_t rb = row0 + warp * rpw; rb < row0 + kK5BlockRows && rb < p.rows; rb += (kK5Threads / 32u) * rpw) {
            const uint32_t r = rb + sub;
            const bool live = r < p.rows && r < row0 + kK5BlockRows;
            const uint8_t* rowA = baseA + static_cast<uint64_t>(live ? r : rb) * p.row_bytes;
            const uint8_t* rowB = baseB + static_cast<uint64_t>(live ? r : rb) * p.row_bytes;
            float accA[MT], accB[GATEUP ? MT : 1];
#pragma unroll
            for (uint32_t j = 0; j < MT; ++j) { accA[j] = 0.f; if (GATEUP) accB[j] = 0.f; }
            for (uint32_t grp = lig; grp < groups; grp += lpr) {
                const Group5<TYPE> ga(rowA, grp), gb(rowB, grp);
                ok &= ga.finite & gb.finite;
#pragma unroll
                for (uint32_t i4 = 0; i4 < 8; ++i4) {
                    float wa[4], wb[4] = {0.f, 0.f, 0.f, 0.f};
                    ga.get(i4, wa);
                    if (GATEUP) gb.get(i4, wb);
#pragma unroll
                    for (uint32_t j = 0; j < MT; ++j) {
                        if (j >= count) break;
                        const float4 v = k5_xs[(j * groups + grp) * 9u + i4];
                        accA[j] = fmaf(wa[0], v.x, accA[j]); accA[j] = fmaf(wa[1], v.y, accA[j]); accA[j] = fmaf(wa[2], v.z, accA[j]); accA[j] = fmaf(wa[3], v.w, accA[j]);
                        if (GATEUP) { accB[j] = fmaf(wb[0], v.x, accB[j]); accB[j] = fmaf(wb[1], v.y, accB[j]); accB[j] = fmaf(wb[2], v.z, accB[j]); accB[j] = fmaf(wb[3], v.w, accB[j]); }
                    }
                }
            }
            // A non-finite activation makes the sums it enters non-finite (0 * inf is NaN): the finished sums are checked
#pragma unroll
            for (uint32_t j = 0; j < MT; ++j) {
                if (j >= count) break;
                float a = accA[j], b = GATEUP ? accB[j] : 0.f;
                for (uint32_t o = lpr >> 1; o > 0; o >>= 1) { a += __shfl_xor_sync(0xffffffffu, a, o); if (GATEUP) b += __shfl_xor_sync(0xffffffffu, b, o); }
                if (lig == 0 && live) {
                    // silu with the branch-stable sigmoid (operators.cpp:28-36)
                    const float v = GATEUP ? (a >= 0.f ? a / (1.f + expf(-a)) : a * expf(a) / (1.f + expf(a))) * b : a;
                    if (!finite_f32(v)) raise_error(p.error, TSP_ERR_NONFINITE);
                    s_out[j][r] = v;
                }
            }
        }
        if (!ok) raise_error(p.error, TSP_ERR_NONFINITE);
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
    if (nc != 1 && nc != 2) return fail(TSP_E_ARG, "five-bit projection: tiles hold 8 or 16 token rows");
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
    const uint32_t groups = a->cols / 32;
    p.lanes_per_row = 1;
    while (p.lanes_per_row * 2 <= groups && p.lanes_per_row < 32) p.lanes_per_row *= 2;
    const size_t smem = static_cast<size_t>(p.tile_tokens) * groups * 9 * sizeof(float4);
    if (smem > 200 * 1024) return fail(TSP_E_ARG, "five-bit projection: %u columns x %u token rows do not fit the activation staging", a->cols, p.tile_tokens);
    // routed launches learn their tile count on the device: a fixed number of block rows walks the tiles (a routed launch has at
    // most 64 routes per token row, one tile each at worst)
    const uint32_t dense_tiles = (tokens + p.tile_tokens - 1) / p.tile_tokens;
    const int sms = sm_count();
    if (sms <= 0) return fail(TSP_E_CUDA, "no usable CUDA device");
    const uint64_t routed_cap = static_cast<uint64_t>(tokens) * 64u;
    const uint32_t walkers = static_cast<uint32_t>(routed_cap < 4u * static_cast<uint32_t>(sms) ? routed_cap : 4u * static_cast<uint32_t>(sms));
    const dim3 grid((a->rows + kK5BlockRows - 1) / kK5BlockRows, token_map ? walkers : (dense_tiles < 1024u ? dense_tiles : 1024u)), block(kK5Threads);
    auto go = [&](auto kernel) -> int {
        static thread_local SmemAttrCache configured;   // per kernel instantiation (one lambda instantiation each), keyed by device
        TSP_CUDA(ensure_dynamic_smem(kernel, configured, smem));
        TSP_CUDA(launch_pdl(kernel, grid, block, smem, st, p));
        return TSP_OK;
    };
    if (a->type == TSP_TYPE_Q5_K) {
        if (gateup) return nc == 1 ? go(gemv_k5_kernel<13u, true, 8u>) : go(gemv_k5_kernel<13u, true, 16u>);
        return nc == 1 ? go(gemv_k5_kernel<13u, false, 8u>) : go(gemv_k5_kernel<13u, false, 16u>);
    }
    if (gateup) return nc == 1 ? go(gemv_k5_kernel<7u, true, 8u>) : go(gemv_k5_kernel<7u, true, 16u>);
    return nc == 1 ? go(gemv_k5_kernel<7u, false, 8u>) : go(gemv_k5_kernel<7u, false, 16u>);
}

}  // namespace tsp
