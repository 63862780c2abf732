// Decode-size routed / dense projections over block-quantised weights (Q4_K, Q8_0; GGUF rows or
// Pack v3 planar planes) for sm_100a.
//
// Shape of the kernel
//   * persistent CTAs, one per SM, each owning a contiguous range of work items; an item is one
//     tile of <= 8*NC routes of one expert x one slab of weight rows over the full K extent;
//   * one producer warp streams the slab's bytes global -> shared with bulk asynchronous copies
//     (TMA, untiled form) into a ring of stages guarded by full/empty mbarriers, so the bytes in
//     flight per SM do not depend on registers or occupancy;
//   * eight (K parts: sixteen) consumer warps dequantise in registers and feed warp-level tensor-core MMAs
//     (m16n8k16, f16 x f16 -> f32): weight codes enter as *exact* small integers (binary16
//     subnormals q*2^-24), activations as binary16 high (+ optional low) halves, and the per-group
//     scales/mins are applied to the FP32 partial sums, so the result carries FP32-level error only;
//   * GGUF Q8_0 matrices whose rows hold a multiple of 8 blocks are walked in K parts instead: a stage is 8 blocks
//     (272 bytes) of 128 rows brought by one tensor copy per matrix, sixteen consumer warps work on it (two per
//     16-row tile, each half of the part's blocks) and reduce their partial sums once per item;
//   * every wait is bounded; a timeout sets TSP_ERR_TIMEOUT in the sticky error word.
//
// The reduction index inside one 8-wide run of K is permuted identically for weights and
// activations (order 0,2,1,3,4,6,5,7): a 32-bit word of codes then splits into MMA register
// pairs with two masks and one shift, with no cross-lane movement.
#include <cuda.h>

#include "tsp_common.cuh"

namespace tsp {

int get_tensor_map_elems(const void* base, uint32_t elem_bytes, uint32_t rank, const uint64_t* dims, const uint64_t* strides, const uint32_t* box,
                         bool swizzle128, CUtensorMap* out);

constexpr int kConsumerWarps = 8;     // consumer warps of most shapes; the K-part mode of a dense matrix runs 16
constexpr uint32_t kMaxStages = 6;

// Tensor maps of the K-part mode: [part bytes as 32-bit elements][rows][experts] of matrix set A (low ids, high ids) and B (same)
struct alignas(64) GemvPartMaps { CUtensorMap m[4]; };

struct GemvParams {
    // weights
    const uint8_t* a_base; const uint8_t* a_base_hi;   // matrix set A (gate, or the only matrix)
    const uint8_t* b_base; const uint8_t* b_base_hi;   // matrix set B (up); unused for plain projections
    uint64_t expert_stride;
    uint32_t split;        // experts >= split live under *_base_hi
    uint32_t experts;
    uint32_t rows;         // rows of ONE matrix (gate-up: hidden units)
    uint32_t cols;         // K
    uint32_t nunit;        // K units per row: Q4_K super-blocks of 256, Q8_0 blocks of 32
    uint64_t sm_off, dm_off;  // planar plane offsets inside one expert
    // item geometry
    uint32_t rows_per_item;   // rows of ONE matrix covered by an item (gate-up: hidden units)
    uint32_t items_per_matrix;
    uint32_t nrt;             // MMA row tiles per item
    uint32_t row_bytes;       // bytes copied per row into the quant area (0: one contiguous copy per matrix)
    uint32_t src_row_pitch;   // bytes between consecutive rows in global memory
    uint32_t kparts;          // K parts per item (1: a stage holds the rows' whole K extent); > 1 only with one row tile per warp
    uint32_t units_per_part;  // K units of a row in one stage
    uint32_t row_stride;      // shared-memory stride between rows of the quant area
    uint32_t quant_bytes;     // quant area bytes per stage
    uint32_t sm_bytes_item;   // planar Q4_K: bytes of the sm plane per matrix per full item
    uint32_t dm_bytes_item;   // planar: bytes of the dm plane per matrix per full item
    uint32_t stage_bytes, n_stages;
    // shared memory carve-up (byte offsets from the dynamic base)
    uint32_t off_xhi, off_xlo, off_sx, off_red, off_stage;
    uint32_t x_stride, sx_stride;
    // activations / routes
    const float* x; uint64_t x_stride_bytes; uint32_t in_div;
    const uint32_t* token_map; const uint32_t* counts; const uint32_t* tasks;
    uint32_t tokens;          // token rows (token_map row length); dense: number of rows
    float* out; uint64_t out_stride_bytes;
    int split_lo;
    int balance;              // K-part mode of a dense plain projection: CTAs split the (item, K part) sequence evenly; an item shared by
                              // two CTAs is summed with atomic adds into output rows the launcher zeroed
    uint32_t* error;
};

__device__ __forceinline__ uint64_t lds64(const uint8_t* p) { return *reinterpret_cast<const uint64_t*>(p); }
__device__ __forceinline__ uint32_t lds32(const uint8_t* p) { return *reinterpret_cast<const uint32_t*>(p); }
__device__ __forceinline__ uint4 lds128(const uint8_t* p) { return *reinterpret_cast<const uint4*>(p); }

__device__ __forceinline__ const uint8_t* expert_ptr(const uint8_t* base, const uint8_t* base_hi, uint32_t e,
                                                     uint32_t split, uint64_t stride) {
    return e < split ? base + static_cast<uint64_t>(e) * stride : base_hi + static_cast<uint64_t>(e - split) * stride;
}

// Shared-memory loads by 32-bit shared-space address (the compiler keeps the constant part of an address as the instruction's offset)
__device__ __forceinline__ uint32_t lds32a(uint32_t a) { uint32_t v; asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(a)); return v; }
__device__ __forceinline__ uint32_t lds16a(uint32_t a) { uint16_t v; asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a)); return v; }
__device__ __forceinline__ float2 lds64fa(uint32_t a) { float2 v; asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(a)); return v; }
__device__ __forceinline__ uint4 lds128a(uint32_t a) {
    uint4 v; asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a)); return v;
}

// (d0, d1) += f * (a0, a1) as one packed FP32 instruction (each half rounds like fmaf)
__device__ __forceinline__ void fma2(float& d0, float& d1, float f, float a0, float a1) {
    asm("{\n\t.reg .b64 dd, ff, aa;\n\t"
        "mov.b64 dd, {%0, %1};\n\tmov.b64 ff, {%2, %2};\n\tmov.b64 aa, {%3, %4};\n\t"
        "fma.rn.f32x2 dd, ff, aa, dd;\n\t"
        "mov.b64 {%0, %1}, dd;\n\t}"
        : "+f"(d0), "+f"(d1) : "f"(f), "f"(a0), "f"(a1));
}

// Eight Q8_0 codes of one row of a 34-byte block as four MMA register pairs of exact binary16 subnormals (code + 128) * 2^-24.
// Lane t of a row takes the aligned words t and t + 4 of the block (the 32 lanes of a warp then read 32 different banks: rows are
// 68 words apart), `a` = block address + 4t. In an odd block the codes start on a word boundary: the words hold codes 4t .. 4t+3
// and 16+4t .. 16+4t+3. In an even block they start 2 bytes off one: the words hold codes 4t-2 .. 4t+1 and 4t+14 .. 4t+17, and
// lane 0, whose first word begins with the block's scale, takes codes 0, 1 from it and 30, 31 from word 8 at `blk` + 32 (`sel` =
// 0x5432 for lane 0, 0x3210 otherwise). Pairs are (byte 0, byte 2) and (byte 1, byte 3) of each word; the activation runs are staged in the
// same order.
template <bool ALIGNED>
__device__ __forceinline__ void q8_pairs(uint32_t blk, uint32_t a, uint32_t sel, uint32_t (&out)[4]) {
    uint32_t w0, w1;
    if (ALIGNED) {
        w0 = lds32a(a + 2); w1 = lds32a(a + 18);
    } else {
        w0 = __byte_perm(lds32a(a), lds32a(blk + 32), sel); w1 = lds32a(a + 16);
    }
    w0 ^= 0x80808080u; w1 ^= 0x80808080u;
    out[0] = __byte_perm(w0, 0u, 0x4240); out[1] = __byte_perm(w0, 0u, 0x4341);
    out[2] = __byte_perm(w1, 0u, 0x4240); out[3] = __byte_perm(w1, 0u, 0x4341);
}

// One block of a warp's four blocks of a K-part stage (GGUF Q8_0, rows 272 bytes apart). aA / aB: shared addresses of the first of
// the four blocks in this lane's two weight rows; xa[c]: this lane's 16 bytes of the first block in the activation rows of token
// group c (+ x_lo_off: the low halves); sa[c]: the pair of pre-scaled block sums of tokens 2t, 2t+1 of the first block, blocks
// `s_step` bytes apart. Everything else is a compile-time offset.
template <int NC, bool LO, int J>
__device__ __forceinline__ void q8_block(uint32_t aA, uint32_t aB, uint32_t t4, const uint32_t (&xa)[NC], uint32_t x_lo_off, const uint32_t (&sa)[NC],
                                         uint32_t s_step, float (&total)[NC][4]) {
    uint32_t A[4], B[4];
    const uint32_t sel = t4 ? 0x3210u : 0x5432u;
    q8_pairs<(J & 1) != 0>(aA + J * 34, aA + J * 34 + t4, sel, A);
    q8_pairs<(J & 1) != 0>(aB + J * 34, aB + J * 34 + t4, sel, B);
    const float fA = half_bits_to_float(lds16a(aA + J * 34));   // the 2^24 of the subnormal codes is applied once per item
    const float fB = half_bits_to_float(lds16a(aB + J * 34));
#pragma unroll
    for (int c = 0; c < NC; ++c) {
        const uint4 xv = lds128a(xa[c] + J * 64);
        const float2 sv = lds64fa(sa[c] + J * s_step);
        float acc[4] = {sv.x, sv.y, sv.x, sv.y};
        mma_f16_16816(acc, A[0], B[0], A[1], B[1], xv.x, xv.y);
        mma_f16_16816(acc, A[2], B[2], A[3], B[3], xv.z, xv.w);
        if (LO) {
            const uint4 yv = lds128a(xa[c] + x_lo_off + J * 64);
            mma_f16_16816(acc, A[0], B[0], A[1], B[1], yv.x, yv.y);
            mma_f16_16816(acc, A[2], B[2], A[3], B[3], yv.z, yv.w);
        }
        fma2(total[c][0], total[c][1], fA, acc[0], acc[1]);
        fma2(total[c][2], total[c][3], fB, acc[2], acc[3]);
    }
}
template <int NC, bool LO>
__device__ __forceinline__ void q8_part(uint32_t aA, uint32_t aB, uint32_t t4, const uint32_t (&xa)[NC], uint32_t x_lo_off, const uint32_t (&sa)[NC],
                                        uint32_t s_step, float (&total)[NC][4]) {
    q8_block<NC, LO, 0>(aA, aB, t4, xa, x_lo_off, sa, s_step, total);
    q8_block<NC, LO, 1>(aA, aB, t4, xa, x_lo_off, sa, s_step, total);
    q8_block<NC, LO, 2>(aA, aB, t4, xa, x_lo_off, sa, s_step, total);
    q8_block<NC, LO, 3>(aA, aB, t4, xa, x_lo_off, sa, s_step, total);
}

// Work item -> (expert, first route of the tile, routes in the tile)
struct TileInfo { uint32_t expert, start, count; };

template <int NC>
__device__ __forceinline__ TileInfo tile_info(const GemvParams& p, uint32_t tile) {
    TileInfo t;
    if (p.token_map) {
        t.expert = p.tasks[2 + 2 * tile];
        t.start = p.tasks[3 + 2 * tile];
        const uint32_t c = t.expert < p.experts ? p.counts[t.expert] : 0u;
        t.count = c > t.start ? min(c - t.start, 8u * NC) : 0u;
        if (t.expert >= p.experts) { t.expert = 0; t.count = 0; }
    } else {
        t.expert = 0;
        t.start = tile * 8u * NC;
        t.count = min(p.tokens - t.start, 8u * NC);
    }
    return t;
}

template <uint32_t TYPE, uint32_t LAYOUT, bool GATEUP, int NC, int CW>
__global__ void __launch_bounds__((CW + 1) * 32, 1) gemv_kernel(const GemvParams p, const __grid_constant__ GemvPartMaps part_maps) {
    pdl_launch_dependents();
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + kMaxStages;
    uint32_t* rids = reinterpret_cast<uint32_t*>(smem + 128);  // route ids of the staged tile, 8*NC entries
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t NS = p.n_stages;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < NS; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], CW); }
        mbar_fence_init();
    }
    __syncthreads();
    pdl_wait();   // everything above touched shared memory only

    const uint32_t n_tiles = p.token_map ? p.tasks[0] : (p.tokens + 8u * NC - 1) / (8u * NC);
    const uint64_t n_items = static_cast<uint64_t>(n_tiles) * p.items_per_matrix;
    // work units of this CTA: whole items, or with p.balance any run of (item, K part) pairs
    const uint64_t n_units = p.balance ? n_items * p.kparts : n_items;
    const uint64_t unit0 = n_units * blockIdx.x / gridDim.x, unit1 = n_units * (blockIdx.x + 1) / gridDim.x;
    const uint32_t upi = p.balance ? p.kparts : 1u;   // units per item
    const uint32_t item0 = static_cast<uint32_t>(unit0 / upi), item1 = static_cast<uint32_t>((unit1 + upi - 1) / upi);
    const uint32_t k_first = p.balance ? static_cast<uint32_t>(unit0 % upi) : 0u;                        // first K part of item0
    const uint32_t k_last = p.balance && unit1 % upi ? static_cast<uint32_t>(unit1 % upi) : p.kparts;   // end K part of item1 - 1
    constexpr uint32_t NMAT = GATEUP ? 2 : 1;
    // K-part mode of GGUF Q8_0 (sixteen consumer warps): stages of eight blocks of 128 rows, rows 272 bytes apart
    constexpr bool KPART = TYPE == TSP_TYPE_Q8_0 && LAYOUT == TSP_LAYOUT_GGUF && CW == 16;

    if (warp == CW) {
        // ------------------------------ producer warp ------------------------------
        uint32_t stage = 0, phase = 0;
        bool ok = true;
        for (uint32_t item = item0; item < item1 && ok; ++item) {
            const uint32_t tile = item / p.items_per_matrix, ri = item % p.items_per_matrix;
            const TileInfo ti = tile_info<NC>(p, tile);
            const uint32_t r0 = ri * p.rows_per_item;
            const uint32_t nr = min(p.rows_per_item, p.rows - r0);
            const uint32_t kbeg = item == item0 ? k_first : 0u, kend = item + 1 == item1 ? k_last : p.kparts;
            for (uint32_t kh = kbeg; kh < kend && ok; ++kh) {
            if (lane == 0) ok = mbar_wait(&empty[stage], phase ^ 1u);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) { if (lane == 0) raise_error(p.error, TSP_ERR_TIMEOUT); break; }
            uint8_t* sbase = smem + p.off_stage + stage * p.stage_bytes;
            if (p.kparts > 1) {
                // K-part stages of GGUF Q8_0 rows: ONE tensor copy per matrix brings this part of all the item's rows ([part bytes]
                // [rows][expert] box; rows past the matrix end are filled with zeros and still count as delivered bytes)
                if (lane == 0) {
                    mbar_arrive_expect_tx(&full[stage], NMAT * p.rows_per_item * p.row_bytes);
                    const bool hi = ti.expert >= p.split;
                    const int el = static_cast<int>(hi ? ti.expert - p.split : ti.expert);
#pragma unroll
                    for (uint32_t m = 0; m < NMAT; ++m)
                        asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                                     ::"r"(smem_u32(sbase + m * p.rows_per_item * p.row_stride)),
                                       "l"(reinterpret_cast<uint64_t>(&part_maps.m[2 * m + (hi ? 1 : 0)])), "r"(smem_u32(&full[stage])),
                                       "r"(static_cast<int>(kh * p.row_bytes / 4)), "r"(static_cast<int>(r0)), "r"(el) : "memory");
                }
                if (++stage == NS) { stage = 0; phase ^= 1u; }
                continue;
            }
            // bytes this fill will deliver
            uint32_t total = 0;
            if (p.row_bytes) total += NMAT * nr * p.row_bytes; else total += NMAT * nr * p.nunit * 34u;
            if (LAYOUT == TSP_LAYOUT_PLANAR) {
                if (TYPE == TSP_TYPE_Q4_K) total += NMAT * nr * p.nunit * 20u; else total += NMAT * nr * p.nunit * 2u;
            }
            if (lane == 0) mbar_arrive_expect_tx(&full[stage], total);
            __syncwarp();
#pragma unroll
            for (uint32_t m = 0; m < NMAT; ++m) {
                const uint8_t* eb = m == 0 ? expert_ptr(p.a_base, p.a_base_hi, ti.expert, p.split, p.expert_stride)
                                           : expert_ptr(p.b_base, p.b_base_hi, ti.expert, p.split, p.expert_stride);
                uint8_t* qdst = sbase + m * p.rows_per_item * p.row_stride;
                if (p.row_bytes) {
                    const uint8_t* src = eb + static_cast<uint64_t>(r0) * p.src_row_pitch + kh * p.row_bytes;
                    for (uint32_t r = lane; r < nr; r += 32)
                        bulk_g2s(qdst + r * p.row_stride, src + static_cast<uint64_t>(r) * p.src_row_pitch, p.row_bytes, &full[stage]);
                } else if (lane == 0) {
                    bulk_g2s(qdst, eb + static_cast<uint64_t>(r0) * p.nunit * 34u, nr * p.nunit * 34u, &full[stage]);
                }
                if (LAYOUT == TSP_LAYOUT_PLANAR && lane == 1) {
                    if (TYPE == TSP_TYPE_Q4_K) {
                        bulk_g2s(sbase + p.quant_bytes + m * p.sm_bytes_item, eb + p.sm_off + static_cast<uint64_t>(r0) * p.nunit * 16u,
                                 nr * p.nunit * 16u, &full[stage]);
                        bulk_g2s(sbase + p.quant_bytes + NMAT * p.sm_bytes_item + m * p.dm_bytes_item,
                                 eb + p.dm_off + static_cast<uint64_t>(r0) * p.nunit * 4u, nr * p.nunit * 4u, &full[stage]);
                    } else {
                        bulk_g2s(sbase + p.quant_bytes + m * p.dm_bytes_item, eb + p.dm_off + static_cast<uint64_t>(r0) * p.nunit * 2u,
                                 nr * p.nunit * 2u, &full[stage]);
                    }
                }
            }
            if (++stage == NS) { stage = 0; phase ^= 1u; }
            }
        }
        return;
    }

    // -------------------------------- consumer warps --------------------------------
    const uint32_t g = lane >> 2, t = lane & 3;
    const uint32_t ctid = threadIdx.x;  // 0 .. 32 CW - 1
    constexpr uint32_t CTHREADS = CW * 32;
    const uint32_t nrt = p.nrt;
    const uint32_t kp_count = nrt >= CW ? 1u : CW / nrt;
    const uint32_t my_kp = nrt >= CW ? 0u : warp / nrt;
    const uint32_t red_slots = nrt >= CW ? 0u : CW - nrt;   // warps that hand partial sums to the first nrt warps
    uint8_t* xhi = smem + p.off_xhi;
    uint8_t* xlo = smem + p.off_xlo;
    uint8_t* sxb = smem + p.off_sx;
    float* red = reinterpret_cast<float*>(smem + p.off_red);
    uint32_t stage = 0, phase = 0, cur_tile = 0xffffffffu, parity = 0;
    bool ok = true;
    TileInfo ti{0, 0, 0};
    for (uint32_t item = item0; item < item1; ++item) {
        const uint32_t tile = item / p.items_per_matrix, ri = item % p.items_per_matrix;
        if (tile != cur_tile) {
            // ---- stage the tile's activation rows: binary16 hi/lo in permuted order + group sums ----
            named_bar_sync(1, CTHREADS);
            ti = tile_info<NC>(p, tile);
            if (ctid < 8u * NC) {
                uint32_t rid = 0;
                if (ctid < ti.count) rid = p.token_map ? p.token_map[static_cast<uint64_t>(ti.expert) * p.tokens + ti.start + ctid] : ti.start + ctid;
                rids[ctid] = rid;
            }
            named_bar_sync(1, CTHREADS);
            const uint32_t per_row = p.cols / 8;
            const uint32_t units = ti.count * per_row;
            bool bad = false;
            for (uint32_t base = 0; base < units; base += CTHREADS) {
                const uint32_t u = base + ctid;
                const bool active = u < units;
                float s = 0.f;
                uint32_t j = 0, k8 = 0;
                if (active) {
                    j = u / per_row; k8 = u % per_row;
                    const uint32_t in_row = rids[j] / p.in_div;
                    float v[8];
                    if (KPART) {
                        // destination run (block b, lane t): the eight activations this MMA lane multiplies with its code pairs (q8_pairs)
                        const uint32_t b = k8 >> 2, tq = k8 & 3u;
                        const float* xr = reinterpret_cast<const float*>(reinterpret_cast<const char*>(p.x) + in_row * p.x_stride_bytes) + b * 32;
                        const uint32_t second = 4 * tq + ((b & 1u) ? 16u : 14u);   // first code of the lane's second word
                        if (!(b & 1u) && tq == 0) { v[0] = xr[0]; v[1] = xr[30]; v[2] = xr[1]; v[3] = xr[31]; }
                        else { const uint32_t first = second - 16; v[0] = xr[first]; v[1] = xr[first + 2]; v[2] = xr[first + 1]; v[3] = xr[first + 3]; }
                        v[4] = xr[second]; v[5] = xr[second + 2]; v[6] = xr[second + 1]; v[7] = xr[second + 3];
                    } else {
                        const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const char*>(p.x) + in_row * p.x_stride_bytes) + k8 * 2;
                        const float4 v0 = src[0], v1 = src[1];
                        v[0] = v0.x; v[1] = v0.y; v[2] = v0.z; v[3] = v0.w; v[4] = v1.x; v[5] = v1.y; v[6] = v1.z; v[7] = v1.w;
                    }
                    __half h[8], l[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        h[i] = __float2half_rn(v[i]);
                        const float hf = __half2float(h[i]);
                        bad |= !finite_f32(hf);
                        l[i] = __float2half_rn(v[i] - hf);
                        s += v[i];
                    }
                    // permuted order inside the run of 8: positions hold elements 0,2,1,3,4,6,5,7 (the K-part mode gathered its runs
                    // in pair order already)
                    const int o1 = KPART ? 1 : 2, o2 = KPART ? 2 : 1, o3 = 3, o4 = 4, o5 = KPART ? 5 : 6, o6 = KPART ? 6 : 5;
                    uint4 ph, pl;
                    ph.x = __half_as_ushort(h[0]) | (uint32_t(__half_as_ushort(h[o1])) << 16);
                    ph.y = __half_as_ushort(h[o2]) | (uint32_t(__half_as_ushort(h[o3])) << 16);
                    ph.z = __half_as_ushort(h[o4]) | (uint32_t(__half_as_ushort(h[o5])) << 16);
                    ph.w = __half_as_ushort(h[o6]) | (uint32_t(__half_as_ushort(h[7])) << 16);
                    *reinterpret_cast<uint4*>(xhi + j * p.x_stride + k8 * 16) = ph;
                    if (p.split_lo) {
                        pl.x = __half_as_ushort(l[0]) | (uint32_t(__half_as_ushort(l[o1])) << 16);
                        pl.y = __half_as_ushort(l[o2]) | (uint32_t(__half_as_ushort(l[o3])) << 16);
                        pl.z = __half_as_ushort(l[o4]) | (uint32_t(__half_as_ushort(l[o5])) << 16);
                        pl.w = __half_as_ushort(l[o6]) | (uint32_t(__half_as_ushort(l[7])) << 16);
                        *reinterpret_cast<uint4*>(xlo + j * p.x_stride + k8 * 16) = pl;
                    }
                }
                s += __shfl_xor_sync(0xffffffffu, s, 1);
                s += __shfl_xor_sync(0xffffffffu, s, 2);
                if (active && (k8 & 3u) == 0) {
                    const uint32_t grp = k8 >> 2;
                    if (TYPE == TSP_TYPE_Q4_K) {
                        const __half sh = __float2half_rn(s);
                        const __half sl = __float2half_rn(s - __half2float(sh));
                        bad |= !finite_f32(__half2float(sh));
                        *reinterpret_cast<__half*>(sxb + j * p.sx_stride + grp * 2) = sh;
                        *reinterpret_cast<__half*>(sxb + (8u * NC + j) * p.sx_stride + grp * 2) = sl;
                    } else {
                        bad |= !finite_f32(s);
                        // K-part mode: the accumulators start at -128 * 2^-24 * (sum of the block's activations), which takes the
                        // +128 of the unsigned codes out again inside the MMA
                        if (KPART) *reinterpret_cast<float*>(sxb + (grp * (8u * NC) + j) * 4) = s * -7.62939453125e-6f;   // [block][token]
                        else *reinterpret_cast<float*>(sxb + j * p.sx_stride + grp * 4) = s;
                    }
                }
            }
            if (bad) raise_error(p.error, TSP_ERR_NONFINITE);
            named_bar_sync(1, CTHREADS);
            cur_tile = tile;
        }

        const uint32_t r0 = ri * p.rows_per_item;
        // every consumer warp has exactly one row tile of the item (nrt <= CW): rt = warp, or warp % nrt when several warps
        // share a tile and split K among them
        const uint32_t rt = nrt >= CW ? warp : warp % nrt;
        {
            float total[NC][4];
#pragma unroll
            for (int c = 0; c < NC; ++c) { total[c][0] = total[c][1] = total[c][2] = total[c][3] = 0.f; }
            // shared-memory rows of this lane's two MMA row slots
            const uint32_t rowA = GATEUP ? rt * 8 + g : rt * 16 + g;
            const uint32_t rowB = GATEUP ? p.rows_per_item + rt * 8 + g : rt * 16 + 8 + g;
            const uint32_t kbeg = item == item0 ? k_first : 0u, kend = item + 1 == item1 ? k_last : p.kparts;
            const bool partial = kend - kbeg != p.kparts;   // the rest of the item's K extent belongs to a neighbouring CTA
            for (uint32_t kh = kbeg; kh < kend; ++kh) {
            // ---- wait for the slab (one K part of the item's rows) ----
            if (ok) {
                ok = mbar_wait(&full[stage], phase);
                if (!ok && lane == 0) raise_error(p.error, TSP_ERR_TIMEOUT);
            }
            const uint8_t* sbase = smem + p.off_stage + stage * p.stage_bytes;
            const uint8_t* qA = sbase + rowA * p.row_stride;
            const uint8_t* qB = sbase + rowB * p.row_stride;
            const uint32_t kb0 = kh * p.units_per_part;   // first K unit of this part (activation offsets use the global unit index)
            if (KPART && ok) {
                // This warp's four blocks of the part: 4 my_kp .. 4 my_kp + 3 (the even ones 2 bytes off a word boundary, the odd ones
                // on one: resolved at compile time)
                const uint32_t sb32 = smem_u32(sbase);
                const uint32_t x_lo_off = smem_u32(xlo) - smem_u32(xhi);
                const uint32_t aA = sb32 + rowA * 272u + my_kp * 136u, aB = sb32 + rowB * 272u + my_kp * 136u;
                const uint32_t kb = kb0 + my_kp * 4u;
                uint32_t xa[NC], sa[NC];
#pragma unroll
                for (int c = 0; c < NC; ++c) {
                    xa[c] = smem_u32(xhi) + (c * 8 + g) * p.x_stride + (kb * 32 + t * 8) * 2;
                    sa[c] = smem_u32(sxb) + (kb * (8u * NC) + c * 8 + 2 * t) * 4;
                }
                if (p.split_lo) q8_part<NC, true>(aA, aB, t * 4u, xa, x_lo_off, sa, 8u * NC * 4u, total);
                else q8_part<NC, false>(aA, aB, t * 4u, xa, x_lo_off, sa, 8u * NC * 4u, total);
            } else if (ok) {
                for (uint32_t b = my_kp; b < p.units_per_part; b += kp_count) {
                    if (TYPE == TSP_TYPE_Q4_K) {
                        // ---- header of the super-block for both rows: d, dmin, sc[8], mn[8] ----
                        uint32_t dmA, dmB, scA[2], scB[2], mnA[2], mnB[2];
                        const uint8_t *qsA, *qsB;
                        if (LAYOUT == TSP_LAYOUT_PLANAR) {
                            const uint8_t* smp = sbase + p.quant_bytes;
                            const uint8_t* dmp = smp + NMAT * p.sm_bytes_item;
                            const uint4 sa = lds128(smp + (rowA * p.nunit + b) * 16);
                            const uint4 sb = lds128(smp + (rowB * p.nunit + b) * 16);
                            scA[0] = sa.x; scA[1] = sa.y; mnA[0] = sa.z; mnA[1] = sa.w;
                            scB[0] = sb.x; scB[1] = sb.y; mnB[0] = sb.z; mnB[1] = sb.w;
                            dmA = lds32(dmp + (rowA * p.nunit + b) * 4);
                            dmB = lds32(dmp + (rowB * p.nunit + b) * 4);
                            qsA = qA + b * 128; qsB = qB + b * 128;
                        } else {
                            const uint4 ha = lds128(qA + b * 144), hb = lds128(qB + b * 144);
                            dmA = ha.x; dmB = hb.x;
                            scA[0] = ha.y & 0x3f3f3f3fu; mnA[0] = ha.z & 0x3f3f3f3fu;
                            scA[1] = (ha.w & 0x0f0f0f0fu) | ((ha.y >> 2) & 0x30303030u);
                            mnA[1] = ((ha.w >> 4) & 0x0f0f0f0fu) | ((ha.z >> 2) & 0x30303030u);
                            scB[0] = hb.y & 0x3f3f3f3fu; mnB[0] = hb.z & 0x3f3f3f3fu;
                            scB[1] = (hb.w & 0x0f0f0f0fu) | ((hb.y >> 2) & 0x30303030u);
                            mnB[1] = ((hb.w >> 4) & 0x0f0f0f0fu) | ((hb.z >> 2) & 0x30303030u);
                            qsA = qA + b * 144 + 16; qsB = qB + b * 144 + 16;
                        }
                        const float dA = half_bits_to_float(dmA & 0xffffu), mA = half_bits_to_float(dmA >> 16);
                        const float dB = half_bits_to_float(dmB & 0xffffu), mB = half_bits_to_float(dmB >> 16);
                        // ---- min term: sum_g mn_g * Sx_g on the tensor cores (codes as subnormals, Sx as hi+lo) ----
                        const uint32_t mnpA = __byte_perm((((t & 2u) ? mnA[1] : mnA[0]) >> (16 * (t & 1))) & 0xffffu, 0u, 0x4140);
                        const uint32_t mnpB = __byte_perm((((t & 2u) ? mnB[1] : mnB[0]) >> (16 * (t & 1))) & 0xffffu, 0u, 0x4140);
                        float amin[NC][4];
#pragma unroll
                        for (int c = 0; c < NC; ++c) {
                            amin[c][0] = amin[c][1] = amin[c][2] = amin[c][3] = 0.f;
                            const uint32_t sh = lds32(sxb + (c * 8 + g) * p.sx_stride + (b * 8 + 2 * t) * 2);
                            const uint32_t sl = lds32(sxb + (8u * NC + c * 8 + g) * p.sx_stride + (b * 8 + 2 * t) * 2);
                            mma_f16_16816(amin[c], mnpA, mnpB, mnpA, mnpB, sh, sl);
                        }
                        const float dA24 = dA * 16777216.f, dB24 = dB * 16777216.f;
                        const float dA20 = dA * 1048576.f, dB20 = dB * 1048576.f;
#pragma unroll
                        for (uint32_t j = 0; j < 4; ++j) {
                            const uint64_t wa = lds64(qsA + j * 32 + t * 8), wb = lds64(qsB + j * 32 + t * 8);
                            const uint32_t a0 = static_cast<uint32_t>(wa), a1 = static_cast<uint32_t>(wa >> 32);
                            const uint32_t b0 = static_cast<uint32_t>(wb), b1 = static_cast<uint32_t>(wb >> 32);
                            const uint32_t a0s = a0 >> 8, a1s = a1 >> 8, b0s = b0 >> 8, b1s = b1 >> 8;
                            const uint32_t sw_a = scA[j >> 1] >> (16 * (j & 1)), sw_b = scB[j >> 1] >> (16 * (j & 1));
                            const float fAl = dA24 * static_cast<float>(sw_a & 0xffu), fAh = dA20 * static_cast<float>((sw_a >> 8) & 0xffu);
                            const float fBl = dB24 * static_cast<float>(sw_b & 0xffu), fBh = dB20 * static_cast<float>((sw_b >> 8) & 0xffu);
#pragma unroll
                            for (int c = 0; c < NC; ++c) {
                                const uint8_t* xr = xhi + (c * 8 + g) * p.x_stride + (b * 256 + j * 64 + t * 8) * 2;
                                const uint4 xl = lds128(xr), xh = lds128(xr + 64);
                                float al[4] = {0.f, 0.f, 0.f, 0.f}, ah[4] = {0.f, 0.f, 0.f, 0.f};
                                mma_f16_16816(al, a0 & 0x000f000fu, b0 & 0x000f000fu, a0s & 0x000f000fu, b0s & 0x000f000fu, xl.x, xl.y);
                                mma_f16_16816(al, a1 & 0x000f000fu, b1 & 0x000f000fu, a1s & 0x000f000fu, b1s & 0x000f000fu, xl.z, xl.w);
                                mma_f16_16816(ah, a0 & 0x00f000f0u, b0 & 0x00f000f0u, a0s & 0x00f000f0u, b0s & 0x00f000f0u, xh.x, xh.y);
                                mma_f16_16816(ah, a1 & 0x00f000f0u, b1 & 0x00f000f0u, a1s & 0x00f000f0u, b1s & 0x00f000f0u, xh.z, xh.w);
                                if (p.split_lo) {
                                    const uint8_t* xq = xlo + (c * 8 + g) * p.x_stride + (b * 256 + j * 64 + t * 8) * 2;
                                    const uint4 yl = lds128(xq), yh = lds128(xq + 64);
                                    mma_f16_16816(al, a0 & 0x000f000fu, b0 & 0x000f000fu, a0s & 0x000f000fu, b0s & 0x000f000fu, yl.x, yl.y);
                                    mma_f16_16816(al, a1 & 0x000f000fu, b1 & 0x000f000fu, a1s & 0x000f000fu, b1s & 0x000f000fu, yl.z, yl.w);
                                    mma_f16_16816(ah, a0 & 0x00f000f0u, b0 & 0x00f000f0u, a0s & 0x00f000f0u, b0s & 0x00f000f0u, yh.x, yh.y);
                                    mma_f16_16816(ah, a1 & 0x00f000f0u, b1 & 0x00f000f0u, a1s & 0x00f000f0u, b1s & 0x00f000f0u, yh.z, yh.w);
                                }
                                total[c][0] = fmaf(fAl, al[0], total[c][0]); total[c][1] = fmaf(fAl, al[1], total[c][1]);
                                total[c][2] = fmaf(fBl, al[2], total[c][2]); total[c][3] = fmaf(fBl, al[3], total[c][3]);
                                total[c][0] = fmaf(fAh, ah[0], total[c][0]); total[c][1] = fmaf(fAh, ah[1], total[c][1]);
                                total[c][2] = fmaf(fBh, ah[2], total[c][2]); total[c][3] = fmaf(fBh, ah[3], total[c][3]);
                            }
                        }
                        const float mA24 = -mA * 16777216.f, mB24 = -mB * 16777216.f;
#pragma unroll
                        for (int c = 0; c < NC; ++c) {
                            total[c][0] = fmaf(mA24, amin[c][0], total[c][0]); total[c][1] = fmaf(mA24, amin[c][1], total[c][1]);
                            total[c][2] = fmaf(mB24, amin[c][2], total[c][2]); total[c][3] = fmaf(mB24, amin[c][3], total[c][3]);
                        }
                    } else {
                        // ---- Q8_0 block of 32 ----
                        uint32_t a0, a1, b0, b1, dbA, dbB;
                        if (LAYOUT == TSP_LAYOUT_PLANAR) {
                            const uint8_t* dmp = sbase + p.quant_bytes;
                            const uint64_t wa = lds64(qA + b * 32 + t * 8), wb = lds64(qB + b * 32 + t * 8);
                            a0 = static_cast<uint32_t>(wa); a1 = static_cast<uint32_t>(wa >> 32);
                            b0 = static_cast<uint32_t>(wb); b1 = static_cast<uint32_t>(wb >> 32);
                            dbA = *reinterpret_cast<const uint16_t*>(dmp + (rowA * p.nunit + b) * 2);
                            dbB = *reinterpret_cast<const uint16_t*>(dmp + (rowB * p.nunit + b) * 2);
                        } else {
                            // 34-byte blocks leave the codes only 2-byte aligned: three aligned words + funnel shift
                            const uint8_t* pa = qA + b * 34 + 2 + t * 8;
                            const uint8_t* pb = qB + b * 34 + 2 + t * 8;
                            const uint32_t sa = (static_cast<uint32_t>(reinterpret_cast<uintptr_t>(pa)) & 3u) * 8u;
                            const uint32_t sb = (static_cast<uint32_t>(reinterpret_cast<uintptr_t>(pb)) & 3u) * 8u;
                            const uint8_t* pa4 = pa - (sa >> 3);
                            const uint8_t* pb4 = pb - (sb >> 3);
                            const uint32_t w0 = lds32(pa4), w1 = lds32(pa4 + 4), w2 = lds32(pa4 + 8);
                            const uint32_t v0 = lds32(pb4), v1 = lds32(pb4 + 4), v2 = lds32(pb4 + 8);
                            a0 = __funnelshift_r(w0, w1, sa); a1 = __funnelshift_r(w1, w2, sa);
                            b0 = __funnelshift_r(v0, v1, sb); b1 = __funnelshift_r(v1, v2, sb);
                            dbA = *reinterpret_cast<const uint16_t*>(qA + b * 34);
                            dbB = *reinterpret_cast<const uint16_t*>(qB + b * 34);
                        }
                        a0 ^= 0x80808080u; a1 ^= 0x80808080u; b0 ^= 0x80808080u; b1 ^= 0x80808080u;  // code + 128 in [0,255]
                        const float dA = half_bits_to_float(dbA), dB = half_bits_to_float(dbB);
                        const float fA = dA * 16777216.f, fB = dB * 16777216.f;
                        const float oA = -128.f * dA, oB = -128.f * dB;
                        const uint32_t pa0 = __byte_perm(a0, 0u, 0x4240), pa1 = __byte_perm(a0, 0u, 0x4341);
                        const uint32_t pa2 = __byte_perm(a1, 0u, 0x4240), pa3 = __byte_perm(a1, 0u, 0x4341);
                        const uint32_t pb0 = __byte_perm(b0, 0u, 0x4240), pb1 = __byte_perm(b0, 0u, 0x4341);
                        const uint32_t pb2 = __byte_perm(b1, 0u, 0x4240), pb3 = __byte_perm(b1, 0u, 0x4341);
#pragma unroll
                        for (int c = 0; c < NC; ++c) {
                            const uint4 xv = lds128(xhi + (c * 8 + g) * p.x_stride + ((kb0 + b) * 32 + t * 8) * 2);
                            float acc[4] = {0.f, 0.f, 0.f, 0.f};
                            mma_f16_16816(acc, pa0, pb0, pa1, pb1, xv.x, xv.y);
                            mma_f16_16816(acc, pa2, pb2, pa3, pb3, xv.z, xv.w);
                            if (p.split_lo) {
                                const uint4 yv = lds128(xlo + (c * 8 + g) * p.x_stride + ((kb0 + b) * 32 + t * 8) * 2);
                                mma_f16_16816(acc, pa0, pb0, pa1, pb1, yv.x, yv.y);
                                mma_f16_16816(acc, pa2, pb2, pa3, pb3, yv.z, yv.w);
                            }
                            const float s0 = *reinterpret_cast<const float*>(sxb + (c * 8 + 2 * t) * p.sx_stride + (kb0 + b) * 4);
                            const float s1 = *reinterpret_cast<const float*>(sxb + (c * 8 + 2 * t + 1) * p.sx_stride + (kb0 + b) * 4);
                            total[c][0] = fmaf(fA, acc[0], fmaf(oA, s0, total[c][0]));
                            total[c][1] = fmaf(fA, acc[1], fmaf(oA, s1, total[c][1]));
                            total[c][2] = fmaf(fB, acc[2], fmaf(oB, s0, total[c][2]));
                            total[c][3] = fmaf(fB, acc[3], fmaf(oB, s1, total[c][3]));
                        }
                    }
                }
            }
            if (kh + 1 < kend) {   // more parts of this item follow: hand the stage back and move on
                __syncwarp();
                if (lane == 0 && ok) mbar_arrive(&empty[stage]);
                if (++stage == NS) { stage = 0; phase ^= 1u; }
            }
            }
            if (KPART) {
#pragma unroll
                for (int c = 0; c < NC; ++c) { total[c][0] *= 16777216.f; total[c][1] *= 16777216.f; total[c][2] *= 16777216.f; total[c][3] *= 16777216.f; }
            }
            // ---- cross-warp reduction over the K parts (only when one row tile is shared by several warps) ----
            if (kp_count > 1) {
                float* slot = red + ((parity * red_slots + (my_kp != 0 ? warp - nrt : 0u)) * 32 + lane) * (4 * NC);
                if (my_kp != 0) {
#pragma unroll
                    for (int c = 0; c < NC; ++c) *reinterpret_cast<float4*>(slot + 4 * c) = make_float4(total[c][0], total[c][1], total[c][2], total[c][3]);
                }
                __syncwarp();
                if (lane == 0 && ok) mbar_arrive(&empty[stage]);
                named_bar_sync(1, CTHREADS);
                if (my_kp == 0) {
                    for (uint32_t kp = 1; kp < kp_count; ++kp) {
                        const float* other = red + ((parity * red_slots + (kp - 1) * nrt + rt) * 32 + lane) * (4 * NC);
#pragma unroll
                        for (int c = 0; c < NC; ++c) {
                            const float4 v = *reinterpret_cast<const float4*>(other + 4 * c);
                            total[c][0] += v.x; total[c][1] += v.y; total[c][2] += v.z; total[c][3] += v.w;
                        }
                    }
                }
            }
            // ---- epilogue ----
            if (my_kp == 0 && ok) {
                bool bad = false;
#pragma unroll
                for (int c = 0; c < NC; ++c) {
#pragma unroll
                    for (int q = 0; q < 2; ++q) {
                        const uint32_t j = c * 8 + 2 * t + q;
                        if (j >= ti.count) continue;
                        float* orow = reinterpret_cast<float*>(reinterpret_cast<char*>(p.out) + rids[j] * p.out_stride_bytes);
                        if (GATEUP) {
                            const uint32_t hu = r0 + rt * 8 + g;
                            if (hu < p.rows) {
                                const float v = stable_silu(total[c][q]) * total[c][2 + q];
                                bad |= !finite_f32(v);
                                orow[hu] = v;
                            }
                        } else {
                            const uint32_t r = r0 + rt * 16 + g;
                            if (partial) {   // two CTAs share the item: each adds its part onto the zeroed rows (two addends: order-free)
                                if (r < p.rows) { bad |= !finite_f32(total[c][q]); atomicAdd(orow + r, total[c][q]); }
                                if (r + 8 < p.rows) { bad |= !finite_f32(total[c][2 + q]); atomicAdd(orow + r + 8, total[c][2 + q]); }
                                continue;
                            }
                            if (r < p.rows) { bad |= !finite_f32(total[c][q]); orow[r] = total[c][q]; }
                            if (r + 8 < p.rows) { bad |= !finite_f32(total[c][2 + q]); orow[r + 8] = total[c][2 + q]; }
                        }
                    }
                }
                if (bad) raise_error(p.error, TSP_ERR_NONFINITE);
            }
        }
        if (kp_count == 1) {
            __syncwarp();
            if (lane == 0 && ok) mbar_arrive(&empty[stage]);
        }
        parity ^= 1u;
        if (++stage == NS) { stage = 0; phase ^= 1u; }
    }
}

int launch_gemv_k5(const tsp_matrix_set*, const tsp_matrix_set*, bool, const float*, uint64_t, uint32_t, uint32_t, const uint32_t*, const uint32_t*,
                   const uint32_t*, float*, uint64_t, int, uint32_t*, cudaStream_t);
int launch_gemv_q4k_tma(const tsp_matrix_set*, const tsp_matrix_set*, bool, const float*, uint64_t, uint32_t, uint32_t, const uint32_t*,
                        const uint32_t*, const uint32_t*, float*, uint64_t, int, int, uint32_t*, cudaStream_t, const GemvShared*);

// ---------------------------------------------------------------------------------------------
// host side: geometry, shared-memory plan, launch
// ---------------------------------------------------------------------------------------------
static uint32_t pad_row(uint32_t row_bytes) {
    // smallest multiple-of-16 pad that puts consecutive rows 32 or 96 bytes apart modulo 128, so the four
    // row groups of a half-warp's 64-bit loads fall on disjoint banks
    for (uint32_t pad = 0; pad < 128; pad += 16) {
        const uint32_t m = (row_bytes + pad) % 128;
        if (m == 32 || m == 96) return row_bytes + pad;
    }
    return row_bytes + 32;
}

template <uint32_t TYPE, uint32_t LAYOUT, bool GATEUP, int NC, int CW = kConsumerWarps>
static int launch_one(const GemvParams& p, const GemvPartMaps& map, size_t smem, int grid, cudaStream_t st) {
    auto kernel = gemv_kernel<TYPE, LAYOUT, GATEUP, NC, CW>;
    static thread_local SmemAttrCache configured;   // per kernel instantiation, keyed by device
    TSP_CUDA(ensure_dynamic_smem(kernel, configured, smem));
    TSP_CUDA(launch_pdl(kernel, dim3(grid), dim3((CW + 1) * 32), smem, st, p, map));
    return TSP_OK;
}

int launch_gemv(const tsp_matrix_set* a, const tsp_matrix_set* b, bool gateup, const float* x, uint64_t x_stride_bytes,
                uint32_t in_div, uint32_t tokens, const uint32_t* token_map, const uint32_t* counts, const uint32_t* tasks,
                float* out, uint64_t out_stride_bytes, int f16_exact, int nc, uint32_t* error, cudaStream_t st, const GemvShared* shared) {
    // `shared` (an extra dense expert in the same launch) is served by the second-generation pipeline only: return 1 = not done
    if (shared && a->type != TSP_TYPE_Q4_K) return 1;
    if (a->type == TSP_TYPE_Q5_K || a->type == TSP_TYPE_Q5_1)   // the reference model's five-bit encodings: their own plain kernel
        return launch_gemv_k5(a, b, gateup, x, x_stride_bytes, in_div, tokens, token_map, counts, tasks, out, out_stride_bytes, nc, error, st);
    if (a->type == TSP_TYPE_Q4_K) {   // the second-generation pipeline covers Q4_K; shapes it declines (return 1) fall through
        const int rc = launch_gemv_q4k_tma(a, b, gateup, x, x_stride_bytes, in_div, tokens, token_map, counts, tasks, out,
                                           out_stride_bytes, f16_exact, nc, error, st, shared);
        if (rc <= 0 || shared) return rc;
    }
    GemvParams p{};
    const uint32_t type = a->type, layout = a->layout;
    p.a_base = static_cast<const uint8_t*>(a->base);
    p.a_base_hi = static_cast<const uint8_t*>(a->base_hi ? a->base_hi : a->base);
    if (gateup) {
        p.b_base = static_cast<const uint8_t*>(b->base);
        p.b_base_hi = static_cast<const uint8_t*>(b->base_hi ? b->base_hi : b->base);
    }
    p.expert_stride = a->expert_stride;
    p.split = a->split < a->experts ? a->split : a->experts;
    p.experts = a->experts;
    p.rows = a->rows;
    p.cols = a->cols;
    const bool q4 = type == TSP_TYPE_Q4_K;
    p.nunit = q4 ? a->cols / 256 : a->cols / 32;
    const uint64_t total_units = static_cast<uint64_t>(a->rows) * p.nunit;
    if (layout == TSP_LAYOUT_PLANAR) {
        p.sm_off = q4 ? total_units * 128 : 0;
        p.dm_off = q4 ? total_units * 144 : total_units * 32;
    }
    // bytes of one row in the quant area
    uint32_t row_bytes;
    if (layout == TSP_LAYOUT_PLANAR) row_bytes = q4 ? p.nunit * 128 : p.nunit * 32;
    else row_bytes = q4 ? p.nunit * 144 : p.nunit * 34;
    const bool contiguous = (row_bytes % 16) != 0;  // GGUF Q8_0 rows that are not 16-byte multiples
    p.src_row_pitch = row_bytes;
    p.kparts = 1;
    p.units_per_part = p.nunit;
    // GGUF Q8_0 matrices (the vocabulary head, the experts of the MTP block) are walked in K parts of 8 blocks (272 bytes per
    // row): a stage then holds 128 rows (gate-up: 64 + 64) and the partial sums of a row tile are reduced once per item (with
    // whole rows per stage only 16 or 32 rows fit, and the warps reduce through shared memory after every stage).
    if (!q4 && layout == TSP_LAYOUT_GGUF && !contiguous && p.nunit % 8 == 0 && p.nunit > 8 && a->rows >= 128) {
        p.units_per_part = 8;   // parts of 16 blocks leave room for two stages only and measured slower (0.108 against 0.094 ms)
        p.kparts = p.nunit / p.units_per_part;
        row_bytes = p.units_per_part * 34;
    }
    p.row_bytes = contiguous ? 0 : row_bytes;
    // a tensor copy lays the rows of a K part down densely; per-row copies pad the rows against bank conflicts
    p.row_stride = contiguous || p.kparts > 1 ? row_bytes : pad_row(row_bytes);
    // rows per stage: as many as fit ~40 KB, in MMA tiles of 16 rows
    const uint32_t per_row_total = p.row_stride + (layout == TSP_LAYOUT_PLANAR ? (q4 ? p.nunit * 20 : p.nunit * 2) : 0);
    uint32_t stage_rows = 128;
    // a dense matrix (vocabulary head) takes larger stages: with one 16-row MMA tile per stage the eight warps split K and
    // pay a cross-warp reduction per 16 rows (measured 0.180 ms against 0.144 ms for the [151936 x 2048] Q8_0 head)
    const uint32_t stage_cap = (a->experts == 1 ? 72u : 44u) * 1024u;
    while (stage_rows > 16 && stage_rows * per_row_total > stage_cap) stage_rows >>= 1;
    const uint32_t matrix_rows_cap = gateup ? a->rows * 2 : a->rows;
    while (stage_rows > 16 && stage_rows / 2 >= matrix_rows_cap) stage_rows >>= 1;
    if (stage_rows * per_row_total > 150 * 1024) return fail(TSP_E_ARG, "matrix rows of %u bytes do not fit a shared-memory stage", row_bytes);
    p.nrt = stage_rows / 16;
    p.rows_per_item = gateup ? stage_rows / 2 : stage_rows;
    p.items_per_matrix = (a->rows + p.rows_per_item - 1) / p.rows_per_item;
    p.quant_bytes = stage_rows * p.row_stride + 16;  // +16: the unaligned-code path may read one word past the last row
    p.quant_bytes = (p.quant_bytes + 15u) & ~15u;
    p.sm_bytes_item = (layout == TSP_LAYOUT_PLANAR && q4) ? p.rows_per_item * p.nunit * 16 : 0;
    p.dm_bytes_item = layout == TSP_LAYOUT_PLANAR ? p.rows_per_item * p.nunit * (q4 ? 4 : 2) : 0;
    const uint32_t nmat = gateup ? 2 : 1;
    p.stage_bytes = p.quant_bytes + nmat * (p.sm_bytes_item + p.dm_bytes_item);
    p.stage_bytes = (p.stage_bytes + 127u) & ~127u;
    // activations
    const uint32_t tok = 8u * static_cast<uint32_t>(nc);
    p.split_lo = f16_exact ? 0 : 1;
    p.x_stride = a->cols * 2 + 64;
    const uint32_t ngroups = a->cols / 32;
    p.sx_stride = q4 ? ngroups * 2 + 16 : ngroups * 4 + 16;
    uint32_t off = 256;
    p.off_xhi = off; off += tok * p.x_stride;
    p.off_xlo = off; if (p.split_lo) off += tok * p.x_stride;
    p.off_sx = off; off += (q4 ? 2 : 1) * tok * p.sx_stride;
    off = (off + 15u) & ~15u;
    // consumer warps: 16 in the K-part mode (two warps per 16-row tile, each half of a part's blocks, one reduction per item: with
    // eight the warps were bound by their own dependent-instruction latency at half the issue rate), 8 otherwise
    const uint32_t cw = p.kparts > 1 ? 16u : static_cast<uint32_t>(kConsumerWarps);
    p.off_red = off; off += 2 * (cw > p.nrt ? cw - p.nrt : 0u) * 32 * 4 * nc * 4;
    off = (off + 127u) & ~127u;
    p.off_stage = off;
    const uint32_t budget = 227 * 1024;
    if (off + p.stage_bytes > budget) return fail(TSP_E_ARG, "K extent of %u columns needs more shared memory than one SM has", a->cols);
    p.n_stages = (budget - off) / p.stage_bytes;
    if (p.n_stages > kMaxStages) p.n_stages = kMaxStages;
    const size_t smem = off + static_cast<size_t>(p.n_stages) * p.stage_bytes;
    p.x = x; p.x_stride_bytes = x_stride_bytes; p.in_div = in_div ? in_div : 1;
    p.token_map = token_map; p.counts = counts; p.tasks = tasks; p.tokens = tokens;
    p.out = out; p.out_stride_bytes = out_stride_bytes; p.error = error;
    const int grid = sm_count();
    if (grid <= 0) return fail(TSP_E_CUDA, "no usable CUDA device");
    // A dense plain projection in K parts (the vocabulary head): 1187 items of 128 rows over 148 CTAs leave three CTAs a ninth item
    // while the rest idle. Splitting the (item, K part) sequence evenly instead costs one pass of zeros over the output rows.
    p.balance = (p.kparts > 1 && !gateup && !token_map && a->experts == 1 && p.items_per_matrix >= static_cast<uint32_t>(grid)) ? 1 : 0;
    if (p.balance) TSP_CUDA(cudaMemset2DAsync(out, out_stride_bytes, 0, static_cast<size_t>(a->rows) * 4, tokens, st));
    GemvPartMaps map{};
    if (p.kparts > 1) {   // [row bytes][rows][experts] as 32-bit elements: a box of one K part (272 or 544 bytes) of the item's rows
        if (p.expert_stride % 16 != 0 && a->experts > 1) return fail(TSP_E_ARG, "project: expert stride must be a multiple of 16 bytes");
        const uint32_t box[3] = {p.row_bytes / 4, p.rows_per_item, 1};
        const uint64_t n_lo = p.split ? p.split : 1, n_hi = p.experts > p.split ? p.experts - p.split : 1;
        const uint64_t strides[2] = {p.src_row_pitch, p.expert_stride ? p.expert_stride : static_cast<uint64_t>(a->rows) * p.src_row_pitch};
        for (uint32_t m = 0; m < nmat; ++m) {
            const uint64_t d_lo[3] = {p.src_row_pitch / 4, a->rows, n_lo}, d_hi[3] = {p.src_row_pitch / 4, a->rows, n_hi};
            if (int rc = get_tensor_map_elems(m ? p.b_base : p.a_base, 4, 3, d_lo, strides, box, false, &map.m[2 * m])) return rc;
            if (int rc = get_tensor_map_elems(m ? p.b_base_hi : p.a_base_hi, 4, 3, d_hi, strides, box, false, &map.m[2 * m + 1])) return rc;
        }
    }

#define TSP_DISPATCH(T, L)                                                                           \
    if (type == T && layout == L) {                                                                   \
        if (gateup) return nc == 1 ? launch_one<T, L, true, 1>(p, map, smem, grid, st) : launch_one<T, L, true, 2>(p, map, smem, grid, st); \
        return nc == 1 ? launch_one<T, L, false, 1>(p, map, smem, grid, st) : launch_one<T, L, false, 2>(p, map, smem, grid, st);           \
    }
    if (p.kparts > 1) {   // GGUF Q8_0 in K parts
        if (gateup) return nc == 1 ? launch_one<TSP_TYPE_Q8_0, TSP_LAYOUT_GGUF, true, 1, 16>(p, map, smem, grid, st)
                                   : launch_one<TSP_TYPE_Q8_0, TSP_LAYOUT_GGUF, true, 2, 16>(p, map, smem, grid, st);
        return nc == 1 ? launch_one<TSP_TYPE_Q8_0, TSP_LAYOUT_GGUF, false, 1, 16>(p, map, smem, grid, st)
                       : launch_one<TSP_TYPE_Q8_0, TSP_LAYOUT_GGUF, false, 2, 16>(p, map, smem, grid, st);
    }
    TSP_DISPATCH(TSP_TYPE_Q4_K, TSP_LAYOUT_PLANAR)
    TSP_DISPATCH(TSP_TYPE_Q4_K, TSP_LAYOUT_GGUF)
    TSP_DISPATCH(TSP_TYPE_Q8_0, TSP_LAYOUT_PLANAR)
    TSP_DISPATCH(TSP_TYPE_Q8_0, TSP_LAYOUT_GGUF)
#undef TSP_DISPATCH
    return fail(TSP_E_TYPE, "no kernel for encoding %u in layout %u", type, layout);
}

}  // namespace tsp
