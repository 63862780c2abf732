// Decode-size routed / dense projections over Q4_K weights, second-generation pipeline for sm_100a:
// tiled TMA (cp.async.bulk.tensor) with the 128-byte shared-memory swizzle, and one private
// software pipeline per consumer warp.
//
//   * A work unit is one group of weight rows (gate-up: 8 hidden units = 8 gate + 8 up rows; plain:
//     16 or 32 rows) of one expert over one part of K (up to 4 super-blocks of 256 columns).
//   * The producer warp brings a unit's 4-bit codes with ONE tensor copy per matrix: the tensor map
//     views the code plane as [128 B of a super-block][row][super-block][expert], so a box of
//     rows x super-blocks lands in shared memory as 128-byte lines whose 16-byte chunks are XOR-ed
//     with (row & 7). The eight row groups of a warp-wide 64-bit load then fall on disjoint banks
//     without any padding, and the copy stays one large request. Scales/mins (planar `sm`, `dm`
//     planes) come as two small contiguous bulk copies covering the unit's rows over the full K.
//   * Units are dealt round-robin to the consumer warps; unit u lives in stage u % stages with its
//     own full/empty mbarrier pair (one arrival each), so warps never synchronise with each other
//     except where the token tile changes. Each warp therefore always has its next unit in flight
//     while it computes the current one.
//   * Arithmetic as in the first-generation kernel: codes enter warp-level MMAs (m16n8k16,
//     f16 x f16 -> f32) as exact binary16 subnormals, scales are applied to FP32 partial sums.
//   * Every wait is bounded (TSP_ERR_TIMEOUT).
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "tsp_common.cuh"

namespace tsp {

constexpr int kW2 = 8;                       // pipelines per CTA (one warp each, or a pair of warps each)
constexpr uint32_t kMaxStages2 = 6;    // per warp
constexpr uint32_t kTableTiles = 32;   // token tiles whose routing data a CTA caches in shared memory

struct Gemv2Params {
    const uint8_t* base[4];   // planar 1D planes: A_lo, A_hi, B_lo, B_hi expert-0 addresses
    uint64_t expert_stride;
    uint32_t split, experts;
    uint32_t rows, cols, nblk;
    uint64_t sm_off, dm_off;
    uint32_t rows_per_unit;   // rows of ONE matrix in a unit (gate-up: 8*nt hidden units; plain: 16*nt rows)
    uint32_t nt;              // MMA row tiles per unit
    uint32_t kb, kparts;      // super-blocks per unit, units per row group
    uint32_t groups;          // row groups per expert
    uint32_t qs_bytes, sm_bytes, dm_bytes;  // per matrix per stage (qs_bytes: region size, a multiple of 1024)
    uint32_t box_bytes;       // bytes one tensor copy delivers
    uint32_t stage_bytes, n_stages;   // n_stages: per warp
    uint32_t off_xhi, off_xlo, off_sx, off_red, off_stage;
    uint32_t x_stride, sx_stride;
    const float* x; uint64_t x_stride_bytes; uint32_t in_div;
    const uint32_t* token_map; const uint32_t* counts; const uint32_t* tasks;
    uint32_t tokens;
    float* out; uint64_t out_stride_bytes;
    int split_lo;
    uint32_t* error;
    // optional dense "shared" expert processed by the same launch after the routed tiles (sh_tiles == 0: none):
    // same shape/encoding/layout as the routed experts, every token row as input, its own output rows
    const uint8_t* sh_base[2];
    const float* sh_x; uint64_t sh_x_stride_bytes;
    float* sh_out; uint64_t sh_out_stride_bytes;
    uint32_t sh_tiles;
};

__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

struct Tile2 { uint32_t expert, start, count; };

// A tile of the shared expert carries the expert id p.experts (one past the routed ids) and identity route ids.
template <int NC>
__device__ __forceinline__ Tile2 tile2(const Gemv2Params& p, uint32_t tile, uint32_t routed_tiles) {
    Tile2 t;
    if (tile >= routed_tiles && p.sh_tiles) {
        t.expert = p.experts;
        t.start = (tile - routed_tiles) * 8u * NC;
        t.count = min(p.tokens - t.start, 8u * NC);
        return t;
    }
    if (p.token_map) {
        t.expert = p.tasks[2 + 2 * tile];
        t.start = p.tasks[3 + 2 * tile];
        if (t.expert >= p.experts) { t.expert = 0; t.start = 0; t.count = 0; return t; }
        const uint32_t c = p.counts[t.expert];
        t.count = c > t.start ? min(c - t.start, 8u * NC) : 0u;
    } else {
        t.expert = 0;
        t.start = tile * 8u * NC;
        t.count = min(p.tokens - t.start, 8u * NC);
    }
    return t;
}

// LAYOUT: TSP_LAYOUT_PLANAR (swizzled code boxes + sm/dm planes) or TSP_LAYOUT_GGUF (whole 144-byte blocks, unswizzled)
//
// Every warp runs its own pipeline: it owns `stages_per_warp` stages, its lane 0 issues the copies of the
// unit that will reuse a stage right after the warp has finished reading that stage, and it waits only on
// the full-barriers of its own stages. Program order inside the warp orders the reads of a stage before the
// copy that overwrites it, so no empty-barrier is needed and no warp ever waits for another one.
//
// PAIR: two warps share each pipeline and split its super-blocks between them (16 warps per SM instead of 8, for
// latency hiding); they meet at a 64-thread named barrier once per unit, where the second warp also hands its
// partial sums to the first at the end of a row group.
// KBT: super-blocks per unit fixed at compile time (the loop over them is then fully unrolled), or 0 for the run-time value.
// SPLIT: also run the low-half pass of the activations (needed unless every activation is exactly a binary16 value).
template <uint32_t LAYOUT, bool GATEUP, int NC, int NT, bool PAIR, int KBT, bool SPLIT>
__global__ void __launch_bounds__(kW2 * 32 * (PAIR ? 2 : 1), 1)
gemv2_kernel(const __grid_constant__ CUtensorMap map_a_lo, const __grid_constant__ CUtensorMap map_a_hi,
             const __grid_constant__ CUtensorMap map_b_lo, const __grid_constant__ CUtensorMap map_b_hi,
             const __grid_constant__ CUtensorMap map_s_a, const __grid_constant__ CUtensorMap map_s_b, const Gemv2Params p) {
    extern __shared__ uint8_t smem2_raw[];
    // the 128-byte swizzle is a function of the shared-memory address: stage bases must sit on 1024-byte boundaries
    uint8_t* smem2 = smem2_raw + ((1024u - (smem_u32(smem2_raw) & 1023u)) & 1023u);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem2);
    uint32_t* rids = reinterpret_cast<uint32_t*>(smem2 + 512);
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t warp = PAIR ? threadIdx.x >> 6 : threadIdx.x >> 5;   // pipeline index
    const uint32_t half = PAIR ? (threadIdx.x >> 5) & 1u : 0u;          // which warp of the pair
    constexpr uint32_t NH = PAIR ? 2 : 1;
    const uint32_t S = p.n_stages;   // stages per pipeline
    constexpr uint32_t NMAT = GATEUP ? 2 : 1;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < S * kW2; ++s) mbar_init(&full[s], 1);
        mbar_fence_init();
    }
    __syncthreads();

    const uint32_t routed_tiles = p.token_map ? p.tasks[0] : (p.tokens + 8u * NC - 1) / (8u * NC);
    const uint32_t n_tiles = routed_tiles + p.sh_tiles;
    const uint64_t n_items = static_cast<uint64_t>(n_tiles) * p.groups;   // item = (tile, row group)
    const uint32_t item0 = static_cast<uint32_t>(n_items * blockIdx.x / gridDim.x);
    const uint32_t item1 = static_cast<uint32_t>(n_items * (blockIdx.x + 1) / gridDim.x);
    const uint32_t KP = p.kparts;
    // Tile table: the (expert, first route, route count) and route ids of the first kTableTiles token tiles this CTA touches,
    // fetched once and in parallel, so that the dependent global loads behind them are not paid again at every tile change.
    uint32_t* tt = reinterpret_cast<uint32_t*>(smem2 + 1024);          // [kTableTiles][4]
    uint32_t* trid = reinterpret_cast<uint32_t*>(smem2 + 1024 + 512);  // [kTableTiles][16]
    const uint32_t t0 = item0 / p.groups;
    for (uint32_t i = threadIdx.x; i < kTableTiles * 16; i += blockDim.x) {
        const uint32_t tl = i >> 4, slot = i & 15u, tile = t0 + tl;
        if (tile < n_tiles && item0 < item1) {
            const Tile2 ti = tile2<NC>(p, tile, routed_tiles);
            if (slot == 0) { tt[tl * 4] = ti.expert; tt[tl * 4 + 1] = ti.start; tt[tl * 4 + 2] = ti.count; }
            uint32_t rid = 0;
            if (slot < ti.count) rid = (p.token_map && ti.expert < p.experts) ? p.token_map[static_cast<uint64_t>(ti.expert) * p.tokens + ti.start + slot] : ti.start + slot;
            trid[i] = rid;
        }
    }
    __syncthreads();
    auto get_tile = [&](uint32_t tile) {
        const uint32_t tl = tile - t0;
        if (tl < kTableTiles) return Tile2{tt[tl * 4], tt[tl * 4 + 1], tt[tl * 4 + 2]};
        return tile2<NC>(p, tile, routed_tiles);
    };
    // this warp's items are item0 + warp + 8n; its unit k is part (k % KP) of item item0 + warp + 8*(k / KP)
    const uint32_t my_items = item0 + warp < item1 ? (item1 - item0 - warp + kW2 - 1) / kW2 : 0u;
    const uint32_t my_units = my_items * KP;
    uint8_t* my_stage0 = smem2 + p.off_stage + warp * S * p.stage_bytes;
    uint64_t* my_full = full + warp * S;

    // lane 0: issue the copies of this pipeline's next unit (units are issued strictly in order, so the stage, K part,
    // row group and tile advance incrementally; nothing here divides)
    uint32_t iss_tile = (item0 + warp) / p.groups, iss_grp = (item0 + warp) % p.groups, iss_kh = 0, iss_s = 0, issued = 0;
    uint32_t iss_ti_tile = 0xffffffffu;
    Tile2 issue_ti{0, 0, 0};
    auto issue_next = [&]() {
        if (iss_tile != iss_ti_tile) { issue_ti = get_tile(iss_tile); iss_ti_tile = iss_tile; }
        const uint32_t kh = iss_kh, s = iss_s;
        const uint32_t r0 = iss_grp * p.rows_per_unit;
        const uint32_t nr = min(p.rows_per_unit, p.rows - r0);
        const bool shared = issue_ti.expert >= p.experts;
        const bool hi = !shared && issue_ti.expert >= p.split;
        const uint32_t el = shared ? 0u : (hi ? issue_ti.expert - p.split : issue_ti.expert);
        ++issued;
        if (++iss_s == S) iss_s = 0;
        if (++iss_kh == KP) {
            iss_kh = 0;
            iss_grp += kW2;
            while (iss_grp >= p.groups) { iss_grp -= p.groups; ++iss_tile; }
        }
        uint8_t* sb = my_stage0 + s * p.stage_bytes;
        uint32_t bytes = NMAT * p.box_bytes;
        if (LAYOUT == TSP_LAYOUT_PLANAR) bytes += NMAT * nr * p.nblk * 20u;
        mbar_arrive_expect_tx(&my_full[s], bytes);
#pragma unroll
        for (uint32_t m = 0; m < NMAT; ++m) {
            const CUtensorMap* map = shared ? (m == 0 ? &map_s_a : &map_s_b) : m == 0 ? (hi ? &map_a_hi : &map_a_lo) : (hi ? &map_b_hi : &map_b_lo);
            if (LAYOUT == TSP_LAYOUT_PLANAR) {
                tma_load_4d(sb + m * p.qs_bytes, map, 0, static_cast<int>(r0), static_cast<int>(kh * p.kb), static_cast<int>(el), &my_full[s]);
                const uint8_t* eb = shared ? p.sh_base[m] : p.base[m * 2 + (hi ? 1 : 0)] + static_cast<uint64_t>(el) * p.expert_stride;
                bulk_g2s(sb + NMAT * p.qs_bytes + m * p.sm_bytes, eb + p.sm_off + static_cast<uint64_t>(r0) * p.nblk * 16u, nr * p.nblk * 16u, &my_full[s]);
                bulk_g2s(sb + NMAT * (p.qs_bytes + p.sm_bytes) + m * p.dm_bytes, eb + p.dm_off + static_cast<uint64_t>(r0) * p.nblk * 4u,
                         nr * p.nblk * 4u, &my_full[s]);
            } else {
                tma_load_4d(sb + m * p.qs_bytes, map, 0, static_cast<int>(kh * p.kb), static_cast<int>(r0), static_cast<int>(el), &my_full[s]);
            }
        }
    };
    if (lane == 0 && half == 0) while (issued < min(S, my_units)) issue_next();

    const uint32_t g = lane >> 2, t = lane & 3;
    const uint32_t ctid = threadIdx.x;
    constexpr uint32_t CT = kW2 * 32 * NH;
    float* red = reinterpret_cast<float*>(smem2 + p.off_red);
    uint32_t red_parity = 0;
    uint8_t* xhi = smem2 + p.off_xhi;
    uint8_t* xlo = smem2 + p.off_xlo;
    uint8_t* sxb = smem2 + p.off_sx;
    bool ok = true;
    // lane constants: byte offset of this lane's 8 code bytes of pair j inside a (swizzled) 128-byte line
    uint32_t qoff[4];
#pragma unroll
    for (uint32_t j = 0; j < 4; ++j) qoff[j] = (((2 * j + (t >> 1)) ^ (LAYOUT == TSP_LAYOUT_PLANAR ? g : 0u)) << 4) + (t & 1u) * 8u;
    const uint32_t xlane = g * p.x_stride + t * 16;     // this lane's B-fragment offset inside a token-row block
    const uint32_t sxlane = g * p.sx_stride + t * 4;
    const uint32_t mn_shift = 16 * (t & 1);

    uint32_t my_it = item0 + warp;                  // this pipeline's next item
    uint32_t my_grp = (item0 + warp) % p.groups;    // its row group
    uint32_t cs = 0, cph = 0;                       // stage and phase of this pipeline's next unit
    uint32_t item = item0;
    while (item < item1) {
        // ---- one token tile: the segment of this CTA's items that share it ----
        const uint32_t tile = item / p.groups;
        const uint32_t seg_end = min(item1, (tile + 1) * p.groups);
        __syncthreads();   // every warp is done with the previous tile's activations
        const Tile2 ti = get_tile(tile);
        const uint32_t* cur_rids = trid + (tile - t0) * 16;
        if (tile - t0 >= kTableTiles) {   // beyond the cached window: fetch this tile's route ids now
            if (ctid < 8u * NC) {
                uint32_t rid = 0;
                if (ctid < ti.count) rid = (p.token_map && ti.expert < p.experts) ? p.token_map[static_cast<uint64_t>(ti.expert) * p.tokens + ti.start + ctid] : ti.start + ctid;
                rids[ctid] = rid;
            }
            cur_rids = rids;
            __syncthreads();
        }
        {
            const uint32_t per_row = p.cols / 8;
            const uint32_t units = ti.count * per_row;
            bool bad = false;
            for (uint32_t base = 0; base < units; base += CT) {
                const uint32_t u = base + ctid;
                const bool active = u < units;
                float s = 0.f;
                uint32_t j = 0, k8 = 0;
                if (active) {
                    j = u / per_row; k8 = u % per_row;
                    const bool sh_tile = ti.expert >= p.experts;
                    const uint32_t in_row = sh_tile ? cur_rids[j] : cur_rids[j] / p.in_div;
                    const float4* src = reinterpret_cast<const float4*>(sh_tile ? reinterpret_cast<const char*>(p.sh_x) + in_row * p.sh_x_stride_bytes
                                                                                : reinterpret_cast<const char*>(p.x) + in_row * p.x_stride_bytes) + k8 * 2;
                    const float4 v0 = src[0], v1 = src[1];
                    const float v[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
                    uint32_t hb[8], lb[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const __half h = __float2half_rn(v[i]);
                        const float hf = __half2float(h);
                        bad |= !finite_f32(hf);
                        hb[i] = __half_as_ushort(h);
                        lb[i] = __half_as_ushort(__float2half_rn(v[i] - hf));
                        s += v[i];
                    }
                    // permuted order inside the run of 8: positions hold elements 0,2,1,3,4,6,5,7
                    *reinterpret_cast<uint4*>(xhi + j * p.x_stride + k8 * 16) =
                        make_uint4(hb[0] | (hb[2] << 16), hb[1] | (hb[3] << 16), hb[4] | (hb[6] << 16), hb[5] | (hb[7] << 16));
                    if (SPLIT)
                        *reinterpret_cast<uint4*>(xlo + j * p.x_stride + k8 * 16) =
                            make_uint4(lb[0] | (lb[2] << 16), lb[1] | (lb[3] << 16), lb[4] | (lb[6] << 16), lb[5] | (lb[7] << 16));
                }
                s += __shfl_xor_sync(0xffffffffu, s, 1);
                s += __shfl_xor_sync(0xffffffffu, s, 2);
                if (active && (k8 & 3u) == 0) {
                    const uint32_t grp = k8 >> 2;
                    const __half sh = __float2half_rn(s);
                    const __half sl = __float2half_rn(s - __half2float(sh));
                    bad |= !finite_f32(__half2float(sh));
                    *reinterpret_cast<__half*>(sxb + j * p.sx_stride + grp * 2) = sh;
                    *reinterpret_cast<__half*>(sxb + (8u * NC + j) * p.sx_stride + grp * 2) = sl;
                }
            }
            if (bad) raise_error(p.error, TSP_ERR_NONFINITE);
        }
        __syncthreads();

        // ---- this warp's row groups of the segment ----
        for (; my_it < seg_end; my_it += kW2) {
            const uint32_t r0 = my_grp * p.rows_per_unit;
            my_grp += kW2;
            while (my_grp >= p.groups) my_grp -= p.groups;
            float total[NT][NC][4];
#pragma unroll
            for (int n = 0; n < NT; ++n)
#pragma unroll
                for (int c = 0; c < NC; ++c) total[n][c][0] = total[n][c][1] = total[n][c][2] = total[n][c][3] = 0.f;

            for (uint32_t kh = 0; kh < KP; ++kh) {
                const uint32_t s = cs, ph = cph;
                if (++cs == S) { cs = 0; cph ^= 1u; }
                if (ok) {
                    ok = mbar_wait(&my_full[s], ph);
                    if (!ok && lane == 0) raise_error(p.error, TSP_ERR_TIMEOUT);
                }
                const uint8_t* sb = my_stage0 + s * p.stage_bytes;
                const uint32_t R = p.rows_per_unit;
                const uint32_t KB = KBT ? KBT : p.kb;
                const uint32_t kb_here = !ok ? 0u : (KBT ? KBT : min(p.kb, p.nblk - kh * p.kb));
                if (kb_here)
#pragma unroll
                for (uint32_t bl = half; bl < (KBT ? KBT : kb_here); bl += NH) {
                    const uint32_t b = kh * KB + bl;   // super-block index along K
                    const uint8_t* xb = xhi + xlane + b * 512;
                    const uint8_t* xq = xlo + xlane + b * 512;
                    const uint8_t* sxp = sxb + sxlane + b * 16;
#pragma unroll
                    for (int n = 0; n < NT; ++n) {
                        const uint32_t rowA = GATEUP ? n * 8 + g : n * 16 + g;        // row inside matrix A's box
                        const uint32_t rowB = GATEUP ? n * 8 + g : n * 16 + 8 + g;    // gate-up: same row of matrix B's box
                        const uint8_t* boxB = GATEUP ? sb + p.qs_bytes : sb;
                        uint32_t dmA, dmB, scA[2], scB[2], mnA[2], mnB[2];
                        const uint8_t *lineA, *lineB;
                        if (LAYOUT == TSP_LAYOUT_PLANAR) {
                            const uint8_t* smp = sb + NMAT * p.qs_bytes;
                            const uint8_t* dmp = smp + NMAT * p.sm_bytes;
                            const uint8_t* smA = smp + (rowA * p.nblk + b) * 16;
                            const uint8_t* smB = smp + (GATEUP ? p.sm_bytes : 0) + (rowB * p.nblk + b) * 16;
                            const uint4 sa = *reinterpret_cast<const uint4*>(smA), sv = *reinterpret_cast<const uint4*>(smB);
                            scA[0] = sa.x; scA[1] = sa.y; mnA[0] = sa.z; mnA[1] = sa.w;
                            scB[0] = sv.x; scB[1] = sv.y; mnB[0] = sv.z; mnB[1] = sv.w;
                            dmA = *reinterpret_cast<const uint32_t*>(dmp + (rowA * p.nblk + b) * 4);
                            dmB = *reinterpret_cast<const uint32_t*>(dmp + (GATEUP ? p.dm_bytes : 0) + (rowB * p.nblk + b) * 4);
                            lineA = sb + (bl * R + rowA) * 128;   // box order: byte, row, super-block
                            lineB = boxB + (bl * R + rowB) * 128;
                        } else {
                            const uint8_t* blkA = sb + (rowA * KB + bl) * 144;   // box order: byte, super-block, row
                            const uint8_t* blkB = boxB + (rowB * KB + bl) * 144;
                            const uint4 ha = *reinterpret_cast<const uint4*>(blkA), hb = *reinterpret_cast<const uint4*>(blkB);
                            dmA = ha.x; dmB = hb.x;
                            scA[0] = ha.y & 0x3f3f3f3fu; mnA[0] = ha.z & 0x3f3f3f3fu;
                            scA[1] = (ha.w & 0x0f0f0f0fu) | ((ha.y >> 2) & 0x30303030u);
                            mnA[1] = ((ha.w >> 4) & 0x0f0f0f0fu) | ((ha.z >> 2) & 0x30303030u);
                            scB[0] = hb.y & 0x3f3f3f3fu; mnB[0] = hb.z & 0x3f3f3f3fu;
                            scB[1] = (hb.w & 0x0f0f0f0fu) | ((hb.y >> 2) & 0x30303030u);
                            mnB[1] = ((hb.w >> 4) & 0x0f0f0f0fu) | ((hb.z >> 2) & 0x30303030u);
                            lineA = blkA + 16; lineB = blkB + 16;
                        }
                        const float dA = half_bits_to_float(dmA & 0xffffu), mA = half_bits_to_float(dmA >> 16);
                        const float dB = half_bits_to_float(dmB & 0xffffu), mB = half_bits_to_float(dmB >> 16);
                        // ---- min term on the tensor cores: codes as subnormals, group sums as hi + lo ----
                        const uint32_t mnpA = __byte_perm((((t & 2u) ? mnA[1] : mnA[0]) >> mn_shift) & 0xffffu, 0u, 0x4140);
                        const uint32_t mnpB = __byte_perm((((t & 2u) ? mnB[1] : mnB[0]) >> mn_shift) & 0xffffu, 0u, 0x4140);
                        float amin[NC][4];
#pragma unroll
                        for (int c = 0; c < NC; ++c) {
                            const uint32_t sh = *reinterpret_cast<const uint32_t*>(sxp + c * 8 * p.sx_stride);
                            const uint32_t sl = *reinterpret_cast<const uint32_t*>(sxp + (8u * NC + c * 8) * p.sx_stride);
                            mma_f16_16816_zero(amin[c], mnpA, mnpB, mnpA, mnpB, sh, sl);
                        }
                        // scale factors: float(sc) through the 2^23 magic number, folded into one FMA each
                        const float dA24 = dA * 16777216.f, dB24 = dB * 16777216.f;
                        const float dA20 = dA * 1048576.f, dB20 = dB * 1048576.f;
                        const float nA24 = -dA24 * 8388608.f, nB24 = -dB24 * 8388608.f, nA20 = -dA20 * 8388608.f, nB20 = -dB20 * 8388608.f;
#pragma unroll
                        for (uint32_t j = 0; j < 4; ++j) {
                            const uint64_t wa = *reinterpret_cast<const uint64_t*>(lineA + qoff[j]);
                            const uint64_t wb = *reinterpret_cast<const uint64_t*>(lineB + qoff[j]);
                            const uint32_t a0 = static_cast<uint32_t>(wa), a1 = static_cast<uint32_t>(wa >> 32);
                            const uint32_t b0 = static_cast<uint32_t>(wb), b1 = static_cast<uint32_t>(wb >> 32);
                            const uint32_t a0s = a0 >> 8, a1s = a1 >> 8, b0s = b0 >> 8, b1s = b1 >> 8;
                            const uint32_t swa = scA[j >> 1], swb = scB[j >> 1];
                            const uint32_t selL = (j & 1) ? 0x7442 : 0x7440, selH = (j & 1) ? 0x7443 : 0x7441;   // 0x4B0000ss = 2^23 + ss
                            const float fAl = fmaf(dA24, __uint_as_float(__byte_perm(swa, 0x4b000000u, selL)), nA24);
                            const float fAh = fmaf(dA20, __uint_as_float(__byte_perm(swa, 0x4b000000u, selH)), nA20);
                            const float fBl = fmaf(dB24, __uint_as_float(__byte_perm(swb, 0x4b000000u, selL)), nB24);
                            const float fBh = fmaf(dB20, __uint_as_float(__byte_perm(swb, 0x4b000000u, selH)), nB20);
#pragma unroll
                            for (int c = 0; c < NC; ++c) {
                                const uint8_t* xr = xb + c * 8 * p.x_stride + j * 128;
                                const uint4 xl = *reinterpret_cast<const uint4*>(xr), xh = *reinterpret_cast<const uint4*>(xr + 64);
                                float al[4], ah[4];
                                mma_f16_16816_zero(al, a0 & 0x000f000fu, b0 & 0x000f000fu, a0s & 0x000f000fu, b0s & 0x000f000fu, xl.x, xl.y);
                                mma_f16_16816(al, a1 & 0x000f000fu, b1 & 0x000f000fu, a1s & 0x000f000fu, b1s & 0x000f000fu, xl.z, xl.w);
                                mma_f16_16816_zero(ah, a0 & 0x00f000f0u, b0 & 0x00f000f0u, a0s & 0x00f000f0u, b0s & 0x00f000f0u, xh.x, xh.y);
                                mma_f16_16816(ah, a1 & 0x00f000f0u, b1 & 0x00f000f0u, a1s & 0x00f000f0u, b1s & 0x00f000f0u, xh.z, xh.w);
                                if (SPLIT) {
                                    const uint8_t* xs = xq + c * 8 * p.x_stride + j * 128;
                                    const uint4 yl = *reinterpret_cast<const uint4*>(xs), yh = *reinterpret_cast<const uint4*>(xs + 64);
                                    mma_f16_16816(al, a0 & 0x000f000fu, b0 & 0x000f000fu, a0s & 0x000f000fu, b0s & 0x000f000fu, yl.x, yl.y);
                                    mma_f16_16816(al, a1 & 0x000f000fu, b1 & 0x000f000fu, a1s & 0x000f000fu, b1s & 0x000f000fu, yl.z, yl.w);
                                    mma_f16_16816(ah, a0 & 0x00f000f0u, b0 & 0x00f000f0u, a0s & 0x00f000f0u, b0s & 0x00f000f0u, yh.x, yh.y);
                                    mma_f16_16816(ah, a1 & 0x00f000f0u, b1 & 0x00f000f0u, a1s & 0x00f000f0u, b1s & 0x00f000f0u, yh.z, yh.w);
                                }
                                total[n][c][0] = fmaf(fAl, al[0], total[n][c][0]); total[n][c][1] = fmaf(fAl, al[1], total[n][c][1]);
                                total[n][c][2] = fmaf(fBl, al[2], total[n][c][2]); total[n][c][3] = fmaf(fBl, al[3], total[n][c][3]);
                                total[n][c][0] = fmaf(fAh, ah[0], total[n][c][0]); total[n][c][1] = fmaf(fAh, ah[1], total[n][c][1]);
                                total[n][c][2] = fmaf(fBh, ah[2], total[n][c][2]); total[n][c][3] = fmaf(fBh, ah[3], total[n][c][3]);
                            }
                        }
                        const float mA24 = -mA * 16777216.f, mB24 = -mB * 16777216.f;
#pragma unroll
                        for (int c = 0; c < NC; ++c) {
                            total[n][c][0] = fmaf(mA24, amin[c][0], total[n][c][0]); total[n][c][1] = fmaf(mA24, amin[c][1], total[n][c][1]);
                            total[n][c][2] = fmaf(mB24, amin[c][2], total[n][c][2]); total[n][c][3] = fmaf(mB24, amin[c][3], total[n][c][3]);
                        }
                    }
                }
                // the stage is free again: bring in the unit that will use it next
                if (PAIR) {
                    if (half == 1 && kh + 1 == KP) {   // hand the partial sums of this row group to the first warp
                        float* slot = red + ((red_parity * kW2 + warp) * 32 + lane) * (NT * NC * 4);
#pragma unroll
                        for (int n = 0; n < NT; ++n)
#pragma unroll
                            for (int c = 0; c < NC; ++c)
                                *reinterpret_cast<float4*>(slot + (n * NC + c) * 4) = make_float4(total[n][c][0], total[n][c][1], total[n][c][2], total[n][c][3]);
                    }
                    named_bar_sync(1 + warp, 64);
                } else {
                    __syncwarp();
                }
                if (lane == 0 && half == 0 && issued < my_units) issue_next();
            }
            if (PAIR) {
                if (half == 0) {
                    const float* slot = red + ((red_parity * kW2 + warp) * 32 + lane) * (NT * NC * 4);
#pragma unroll
                    for (int n = 0; n < NT; ++n)
#pragma unroll
                        for (int c = 0; c < NC; ++c) {
                            const float4 v = *reinterpret_cast<const float4*>(slot + (n * NC + c) * 4);
                            total[n][c][0] += v.x; total[n][c][1] += v.y; total[n][c][2] += v.z; total[n][c][3] += v.w;
                        }
                }
                red_parity ^= 1u;
            }
            // ---- epilogue: this warp owns its rows' complete sums ----
            if (ok && half == 0) {
                bool bad = false;
#pragma unroll
                for (int n = 0; n < NT; ++n)
#pragma unroll
                    for (int c = 0; c < NC; ++c)
#pragma unroll
                        for (int q = 0; q < 2; ++q) {
                            const uint32_t j = c * 8 + 2 * t + q;
                            if (j >= ti.count) continue;
                            float* orow = reinterpret_cast<float*>(ti.expert >= p.experts ? reinterpret_cast<char*>(p.sh_out) + cur_rids[j] * p.sh_out_stride_bytes
                                                                                          : reinterpret_cast<char*>(p.out) + cur_rids[j] * p.out_stride_bytes);
                            if (GATEUP) {
                                const uint32_t hu = r0 + n * 8 + g;
                                if (hu < p.rows) {
                                    const float v = stable_silu(total[n][c][q]) * total[n][c][2 + q];
                                    bad |= !finite_f32(v);
                                    orow[hu] = v;
                                }
                            } else {
                                const uint32_t r = r0 + n * 16 + g;
                                if (r < p.rows) { bad |= !finite_f32(total[n][c][q]); orow[r] = total[n][c][q]; }
                                if (r + 8 < p.rows) { bad |= !finite_f32(total[n][c][2 + q]); orow[r + 8] = total[n][c][2 + q]; }
                            }
                        }
                if (bad) raise_error(p.error, TSP_ERR_NONFINITE);
            }
        }
        item = seg_end;
    }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    });
    return fn;
}

struct MapKey {
    const void* base; uint64_t stride; uint32_t layout, rows, nblk, experts, box_rows, box_kb;
    bool operator==(const MapKey& o) const {
        return base == o.base && stride == o.stride && layout == o.layout && rows == o.rows && nblk == o.nblk && experts == o.experts &&
               box_rows == o.box_rows && box_kb == o.box_kb;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = reinterpret_cast<size_t>(k.base) * 1000003u ^ k.stride;
        for (uint32_t v : {k.layout, k.rows, k.nblk, k.experts, k.box_rows, k.box_kb}) h = h * 1000003u ^ v;
        return h;
    }
};

// Tensor maps depend only on (address, shape, box); weights are immutable imports, so they are encoded once and kept.
static int get_map(const MapKey& k, CUtensorMap* out) {
    static std::mutex mu;
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(k);
    if (it != cache.end()) { *out = it->second; return TSP_OK; }
    EncodeTiledFn enc = encode_fn();
    if (!enc) return fail(TSP_E_CUDA, "the CUDA driver does not export cuTensorMapEncodeTiled");
    CUtensorMap m;
    cuuint64_t dims[4], strides[3];
    cuuint32_t box[4], estr[4] = {1, 1, 1, 1};
    CUtensorMapSwizzle swz;
    if (k.layout == TSP_LAYOUT_PLANAR) {   // [128 B][row][super-block][expert]
        dims[0] = 128; dims[1] = k.rows; dims[2] = k.nblk; dims[3] = k.experts;
        strides[0] = static_cast<cuuint64_t>(k.nblk) * 128; strides[1] = 128; strides[2] = k.stride;
        box[0] = 128; box[1] = k.box_rows; box[2] = k.box_kb; box[3] = 1;
        swz = CU_TENSOR_MAP_SWIZZLE_128B;
    } else {                               // [144 B][super-block][row][expert]
        dims[0] = 144; dims[1] = k.nblk; dims[2] = k.rows; dims[3] = k.experts;
        strides[0] = 144; strides[1] = static_cast<cuuint64_t>(k.nblk) * 144; strides[2] = k.stride;
        box[0] = 144; box[1] = k.box_kb; box[2] = k.box_rows; box[3] = 1;
        swz = CU_TENSOR_MAP_SWIZZLE_NONE;
    }
    const CUresult r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(k.base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(TSP_E_CUDA, "cuTensorMapEncodeTiled failed with %d", static_cast<int>(r));
    if (cache.size() > 4096) cache.clear();
    cache.emplace(k, m);
    *out = m;
    return TSP_OK;
}

// Generic cached tensor map over bytes (rank <= 4), shared with the grouped tensor-core kernels.
struct GenKey {
    const void* base; uint32_t rank; uint64_t dims[4]; uint64_t strides[3]; uint32_t box[4]; uint32_t swizzle;
    bool operator==(const GenKey& o) const {
        if (base != o.base || rank != o.rank || swizzle != o.swizzle) return false;
        for (int i = 0; i < 4; ++i) if (dims[i] != o.dims[i] || box[i] != o.box[i]) return false;
        for (int i = 0; i < 3; ++i) if (strides[i] != o.strides[i]) return false;
        return true;
    }
};
struct GenKeyHash {
    size_t operator()(const GenKey& k) const {
        size_t h = reinterpret_cast<size_t>(k.base) * 1000003u ^ k.rank ^ (k.swizzle << 8);
        for (int i = 0; i < 4; ++i) h = (h * 1000003u ^ k.dims[i]) * 31u ^ k.box[i];
        for (int i = 0; i < 3; ++i) h = h * 1000003u ^ k.strides[i];
        return h;
    }
};

// dims/box in bytes for dimension 0 (element type is UINT8); strides are the byte strides of dimensions 1..rank-1.
int get_tensor_map_bytes(const void* base, uint32_t rank, const uint64_t* dims, const uint64_t* strides, const uint32_t* box,
                         bool swizzle128, CUtensorMap* out) {
    static std::mutex mu;
    static std::unordered_map<GenKey, CUtensorMap, GenKeyHash> cache;
    GenKey k{};
    k.base = base; k.rank = rank; k.swizzle = swizzle128 ? 1u : 0u;
    for (uint32_t i = 0; i < 4; ++i) { k.dims[i] = i < rank ? dims[i] : 1; k.box[i] = i < rank ? box[i] : 1; }
    for (uint32_t i = 0; i < 3; ++i) k.strides[i] = i + 1 < rank ? strides[i] : 0;
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(k);
    if (it != cache.end()) { *out = it->second; return TSP_OK; }
    EncodeTiledFn enc = encode_fn();
    if (!enc) return fail(TSP_E_CUDA, "the CUDA driver does not export cuTensorMapEncodeTiled");
    cuuint64_t d[4], st[3];
    cuuint32_t b[4], es[4] = {1, 1, 1, 1};
    for (uint32_t i = 0; i < rank; ++i) { d[i] = dims[i]; b[i] = box[i]; }
    for (uint32_t i = 0; i + 1 < rank; ++i) st[i] = strides[i];
    CUtensorMap m;
    const CUresult r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_UINT8, rank, const_cast<void*>(base), d, st, b, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(TSP_E_CUDA, "cuTensorMapEncodeTiled failed with %d", static_cast<int>(r));
    if (cache.size() > 4096) cache.clear();
    cache.emplace(k, m);
    *out = m;
    return TSP_OK;
}

template <uint32_t LAYOUT, bool GATEUP, int NC, int NT, bool PAIR, int KBT, bool SPLIT>
static int launch2(const CUtensorMap* maps, const Gemv2Params& p, size_t smem, int grid, cudaStream_t st) {
    auto kernel = gemv2_kernel<LAYOUT, GATEUP, NC, NT, PAIR, KBT, SPLIT>;
    static thread_local size_t configured = 0;
    if (smem > configured) {
        TSP_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        configured = smem;
    }
    kernel<<<grid, kW2 * 32 * (PAIR ? 2 : 1), smem, st>>>(maps[0], maps[1], maps[2], maps[3], maps[4], maps[5], p);
    TSP_CUDA(cudaGetLastError());
    return TSP_OK;
}

// Returns TSP_OK after launching, or 1 when this pipeline does not cover the shape (the caller then uses the
// first-generation kernel), or a negative error.
int launch_gemv_q4k_tma(const tsp_matrix_set* a, const tsp_matrix_set* b, bool gateup, const float* x, uint64_t x_stride_bytes,
                        uint32_t in_div, uint32_t tokens, const uint32_t* token_map, const uint32_t* counts, const uint32_t* tasks,
                        float* out, uint64_t out_stride_bytes, int f16_exact, int nc, uint32_t* error, cudaStream_t st,
                        const GemvShared* shared) {
    if (a->type != TSP_TYPE_Q4_K) return 1;
    if (shared) {   // the extra dense expert must look exactly like a routed one, and the launch must be a routed one
        const tsp_matrix_set* sa = shared->a;
        if (!token_map || nc != 1 || !sa || sa->experts != 1 || sa->type != a->type || sa->layout != a->layout || sa->rows != a->rows ||
            sa->cols != a->cols || (gateup && (!shared->b || shared->b->rows != a->rows || shared->b->cols != a->cols ||
                                               shared->b->type != a->type || shared->b->layout != a->layout))) return 1;
    }
    const uint32_t nblk = a->cols / 256;
    if (a->rows % (gateup ? 8 : 16)) return 1;
    Gemv2Params p{};
    const bool planar = a->layout == TSP_LAYOUT_PLANAR;
    p.split = a->split < a->experts ? a->split : a->experts;
    p.experts = a->experts;
    p.expert_stride = a->expert_stride;
    p.rows = a->rows; p.cols = a->cols; p.nblk = nblk;
    const uint64_t total_units = static_cast<uint64_t>(a->rows) * nblk;
    p.sm_off = total_units * 128; p.dm_off = total_units * 144;
    p.base[0] = static_cast<const uint8_t*>(a->base);
    p.base[1] = static_cast<const uint8_t*>(a->base_hi ? a->base_hi : a->base);
    if (gateup) {
        p.base[2] = static_cast<const uint8_t*>(b->base);
        p.base[3] = static_cast<const uint8_t*>(b->base_hi ? b->base_hi : b->base);
    }
    // unit geometry: K in parts of at most 4 super-blocks; plain projections with a short K take two row tiles per unit
    p.kb = nblk <= 4 ? nblk : 4;
    p.kparts = (nblk + p.kb - 1) / p.kb;
    p.nt = (!gateup && p.kparts == 1 && nblk <= 2 && a->rows % 32 == 0) ? 2 : 1;
    p.rows_per_unit = (gateup ? 8 : 16) * p.nt;
    p.groups = a->rows / p.rows_per_unit;
    const uint32_t nmat = gateup ? 2 : 1;
    p.box_bytes = p.rows_per_unit * p.kb * (planar ? 128 : 144);
    p.qs_bytes = (p.box_bytes + 1023u) & ~1023u;
    p.sm_bytes = planar ? p.rows_per_unit * nblk * 16 : 0;
    p.dm_bytes = planar ? p.rows_per_unit * nblk * 4 : 0;
    p.stage_bytes = (nmat * (p.qs_bytes + p.sm_bytes + p.dm_bytes) + 1023u) & ~1023u;
    const uint32_t tok = 8u * static_cast<uint32_t>(nc);
    p.split_lo = f16_exact ? 0 : 1;
    p.x_stride = a->cols * 2 + 64;
    p.sx_stride = (a->cols / 32) * 2 + 16;
    uint32_t off = 4096;   // barriers, fallback route ids, tile table
    p.off_xhi = off; off += tok * p.x_stride;
    p.off_xlo = off; if (p.split_lo) off += tok * p.x_stride;
    p.off_sx = off; off += 2 * tok * p.sx_stride;
    off = (off + 15u) & ~15u;
    const bool pair = false;   // paired warps (two per pipeline) measured no faster than one warp per pipeline; kept in the kernel, not dispatched
    p.off_red = off; if (pair) off += 2 * kW2 * 32 * p.nt * nc * 16;
    off = (off + 1023u) & ~1023u;
    p.off_stage = off;
    const uint32_t budget = 226 * 1024;   // 1 KB of the 227 KB is kept for aligning the dynamic base
    if (off + 2 * kW2 * p.stage_bytes > budget) return 1;   // too little room for a double-buffered pipeline per warp
    p.n_stages = (budget - off) / (kW2 * p.stage_bytes);     // stages per warp
    if (p.n_stages > kMaxStages2) p.n_stages = kMaxStages2;
    const size_t smem = off + static_cast<size_t>(p.n_stages) * kW2 * p.stage_bytes + 1024;
    p.x = x; p.x_stride_bytes = x_stride_bytes; p.in_div = in_div ? in_div : 1;
    p.token_map = token_map; p.counts = counts; p.tasks = tasks; p.tokens = tokens;
    p.out = out; p.out_stride_bytes = out_stride_bytes; p.error = error;

    CUtensorMap maps[6];
    const uint32_t n_lo = p.split, n_hi = a->experts - p.split;
    for (int m = 0; m < 4; ++m) {
        if (!gateup && m >= 2) { maps[m] = maps[0]; continue; }
        const bool hi = m & 1;
        if (hi && n_hi == 0) { maps[m] = maps[m - 1]; continue; }
        MapKey k{p.base[m], a->experts > 1 ? a->expert_stride : tsp_expert_bytes(a->type, a->layout, a->rows, a->cols), a->layout, a->rows, nblk,
                 hi ? n_hi : n_lo, p.rows_per_unit, p.kb};
        if (k.stride % 16) return 1;
        if (int rc = get_map(k, &maps[m])) return rc;
    }
    maps[4] = maps[0]; maps[5] = maps[0];
    if (shared) {
        p.sh_tiles = (tokens + 7) / 8;
        p.sh_x = shared->x; p.sh_x_stride_bytes = shared->x_stride_bytes;
        p.sh_out = shared->out; p.sh_out_stride_bytes = shared->out_stride_bytes;
        for (int m = 0; m < (gateup ? 2 : 1); ++m) {
            const tsp_matrix_set* sm = m == 0 ? shared->a : shared->b;
            p.sh_base[m] = static_cast<const uint8_t*>(sm->base);
            MapKey k{sm->base, tsp_expert_bytes(a->type, a->layout, a->rows, a->cols), a->layout, a->rows, nblk, 1, p.rows_per_unit, p.kb};
            if (int rc = get_map(k, &maps[4 + m])) return rc;
        }
    }
    const int grid = sm_count();
    if (grid <= 0) return fail(TSP_E_CUDA, "no usable CUDA device");
    // compile-time super-block count for the common shapes of the planar layout (K a multiple of 1024, or K = 512)
    const int kbt = (planar && nblk % p.kb == 0 && (p.kb == 4 || (p.kb == 2 && p.nt == 2))) ? static_cast<int>(p.kb) : 0;
#define TSP_D3(L, G, NCV, NTV, K)                                                        \
    return p.split_lo ? launch2<L, G, NCV, NTV, false, K, true>(maps, p, smem, grid, st) \
                      : launch2<L, G, NCV, NTV, false, K, false>(maps, p, smem, grid, st)
#define TSP_D2(L, SPEC)                                                                 \
    if (a->layout == L) {                                                                \
        if (gateup) {                                                                    \
            if (SPEC && kbt == 4) { if (nc == 1) TSP_D3(L, true, 1, 1, 4); TSP_D3(L, true, 2, 1, 4); } \
            if (nc == 1) TSP_D3(L, true, 1, 1, 0);                                       \
            TSP_D3(L, true, 2, 1, 0);                                                    \
        }                                                                                \
        if (p.nt == 2) {                                                                 \
            if (SPEC && kbt == 2) { if (nc == 1) TSP_D3(L, false, 1, 2, 2); TSP_D3(L, false, 2, 2, 2); } \
            if (nc == 1) TSP_D3(L, false, 1, 2, 0);                                      \
            TSP_D3(L, false, 2, 2, 0);                                                   \
        }                                                                                \
        if (SPEC && kbt == 4) { if (nc == 1) TSP_D3(L, false, 1, 1, 4); TSP_D3(L, false, 2, 1, 4); } \
        if (nc == 1) TSP_D3(L, false, 1, 1, 0);                                          \
        TSP_D3(L, false, 2, 1, 0);                                                       \
    }
    TSP_D2(TSP_LAYOUT_PLANAR, true)
    TSP_D2(TSP_LAYOUT_GGUF, false)
#undef TSP_D2
#undef TSP_D3
    return 1;
}

}  // namespace tsp
