// Decode-size routed / dense projections over Q4_K weights, second-generation pipeline for sm_100a:
// tiled TMA (cp.async.bulk.tensor) with the 128-byte shared-memory swizzle, one private software
// pipeline per consumer warp, and producer warps that do nothing but issue the copies.
//
//   * A work item is one group of weight rows (gate-up: 8 hidden units = 8 gate + 8 up rows; plain:
//     16 or 32 rows) of one expert over the whole K; it is consumed in units of KB super-blocks of
//     256 columns. Items are dealt round-robin to the 8 consumer warps of a CTA.
//   * A unit's 4-bit codes arrive with ONE tensor copy: the tensor map views the code plane as
//     [128 B of a super-block][row][super-block][matrix][expert], so a box of rows x super-blocks of the
//     gate AND the up matrix (co-located at a constant distance) lands in shared memory as 128-byte
//     lines whose 16-byte chunks are XOR-ed with (line & 7). The eight row groups of a warp-wide
//     64-bit load then fall on disjoint banks without padding. (Matrices at no constant distance
//     take one copy each.)
//   * The planar layout's scale bytes and (d, dmin) pairs of an item's rows cover the whole K; they
//     come once per item, as two more tensor copies, into a header buffer of the warp's own (the
//     scale bytes swizzled like the codes).
//   * Issuing one bulk or tensor copy costs the issuing lane 130-260 cycles, and a unit is computed in
//     about 1200: the copies are therefore issued by four producer warps (one lane per pipeline,
//     two lanes per warp running one instruction stream) while the eight consumer warps only
//     wait, compute and arrive. setmaxnreg moves the producers' registers to the consumers.
//     16-byte cp.async copies issued by the consumers themselves were measured slower: they stall
//     in the load/store queue long before enough bytes are in flight.
//   * Consumer warps never synchronise with each other except where the token tile changes.
//   * Arithmetic as in the first-generation kernel: codes enter warp-level MMAs (m16n8k16,
//     f16 x f16 -> f32) as exact binary16 subnormals, scales are applied to FP32 partial sums.
//   * Every wait is bounded (TSP_ERR_TIMEOUT).
#include <cuda.h>

#include "tsp_common.cuh"

namespace tsp {

int get_tensor_map_bytes(const void* base, uint32_t rank, const uint64_t* dims, const uint64_t* strides, const uint32_t* box,
                         bool swizzle128, CUtensorMap* out);

constexpr int kW3 = 8;                  // consumer warps per CTA, one private pipeline each (plain short-K projections run 16)
constexpr int kProd3 = 4;               // producer warps per CTA (one warpgroup); each feeds kW3 / kProd3 pipelines
constexpr int kThreads3 = (kW3 + kProd3) * 32;
constexpr int kConsRegs = 232, kProdRegs = 40;   // (kW3 * kConsRegs + kProd3 * kProdRegs) * 32 <= 65536
// Registers a consumer thread asks for with setmaxnreg.inc. The request is served from what the producer warps of the same
// CTA give back and blocks until it is: W * (consumer - launch) <= kProd3 * (launch - kProdRegs) must hold for the
// register count the kernel is launched with (168 for 12 warps, 96 for 20), or the consumers would wait for ever.
// launch3() checks this against the compiled kernel before the first launch.
__host__ __device__ constexpr int cons_regs(int w) { return w == kW3 ? kConsRegs : 104; }
constexpr uint32_t kMaxStages3 = 8;     // per pipeline
constexpr uint32_t kMaxHeaders3 = 4;    // per pipeline
constexpr uint32_t kTableTiles = 32;    // token tiles whose routing data a CTA caches in shared memory

// Tensor maps of one launch: index = plane * 6 + which, plane 0 codes, 1 scale bytes, 2 (d, dmin) pairs;
// which: 0 A low ids, 1 A high ids, 2 B low ids, 3 B high ids, 4 shared A, 5 shared B.
struct alignas(64) Gemv3Maps { CUtensorMap m[18]; };

struct Gemv3Params {
    uint32_t split, experts;
    uint32_t rows, cols, nblk;
    uint32_t groups;          // row groups (items) per expert
    uint32_t upi;             // units per item = nblk / KB
    uint32_t merged, sh_merged;            // both matrices of an expert in one copy (routed experts; shared expert)
    uint32_t code_mat_bytes;               // code bytes of one matrix in a unit
    uint32_t sm_mat_bytes, dm_mat_bytes;   // header bytes of one matrix: scale bytes, (d, dmin) pairs
    uint32_t sm_lines, dm_inner;           // header box geometry: 128-byte lines of scale bytes per item; inner extent of the pair map
    uint32_t hdr_bytes, n_hdr;             // one header buffer; buffers per pipeline
    uint32_t stage_bytes, n_stages;        // one unit; stages per pipeline
    uint32_t warp_bytes;                   // n_hdr * hdr_bytes + n_stages * stage_bytes
    uint32_t off_xhi, off_xlo, off_sx, off_warp;
    uint32_t x_stride, sx_stride;
    const float* x; uint64_t x_stride_bytes; uint32_t in_div;
    const uint8_t* x16; uint64_t x16_stride_bytes;   // optional binary16 copy of the token rows (routed and shared tiles read it instead)
    const uint32_t* token_map; const uint32_t* counts; const uint32_t* tasks;
    uint32_t tokens;
    float* out; uint64_t out_stride_bytes;
    uint32_t* error;
    // optional dense "shared" expert processed by the same launch after the routed tiles (sh_tiles == 0: none):
    // same shape/encoding/layout as the routed experts, every token row as input, its own output rows
    const float* sh_x; uint64_t sh_x_stride_bytes;
    float* sh_out; uint64_t sh_out_stride_bytes;
    uint32_t sh_tiles, sh_tokens;
};

__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
__device__ __forceinline__ void tma_load_5d(void* smem_dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, int c4, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
        : "memory");
}

struct Tile3 { uint32_t expert, start, count; };

// SiLU with the hardware exponential and reciprocal (relative error of a few 2^-22: far inside the layer tolerance).
// exp(-v) overflows to +inf for v < -88, which the division turns into -0, the limit of the exact function.
__device__ __forceinline__ float fast_silu(float v) { return __fdividef(v, 1.f + __expf(-v)); }

// A tile of the shared expert carries the expert id p.experts (one past the routed ids) and identity route ids.
template <int NC>
__device__ __forceinline__ Tile3 tile3(const Gemv3Params& p, uint32_t tile, uint32_t routed_tiles) {
    Tile3 t;
    if (tile >= routed_tiles && p.sh_tiles) {
        t.expert = p.experts;
        t.start = (tile - routed_tiles) * 8u * NC;
        t.count = min(p.sh_tokens - t.start, 8u * NC);
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

// LAYOUT: TSP_LAYOUT_PLANAR (code lines + scale / (d, dmin) planes) or TSP_LAYOUT_GGUF (whole 144-byte blocks, unswizzled)
// KB: super-blocks per unit. SPLIT: also run the low-half pass of the activations (needed unless every
// activation is exactly a binary16 value).
// W: consumer warps (pipelines) per CTA. Every launch uses eight (232 registers each); the parameter exists for experiments.
template <uint32_t LAYOUT, bool GATEUP, int NC, int NT, int KB, bool SPLIT, int W = kW3>
__global__ void __launch_bounds__((W + kProd3) * 32, 1) gemv3_kernel(const __grid_constant__ Gemv3Maps maps, const Gemv3Params p) {
    pdl_launch_dependents();
    extern __shared__ uint8_t smem3_raw[];
    // the 128-byte swizzle is a function of the shared-memory address: box bases must sit on 1024-byte boundaries
    uint8_t* smem3 = smem3_raw + ((1024u - (smem_u32(smem3_raw) & 1023u)) & 1023u);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem3);             // [W][S]
    uint64_t* empty = reinterpret_cast<uint64_t*>(smem3 + 512);      // [W][S]
    uint32_t* tt = reinterpret_cast<uint32_t*>(smem3 + 1024);        // [kTableTiles][4] expert, first route, count
    uint32_t* trid = reinterpret_cast<uint32_t*>(smem3 + 1536);      // [kTableTiles][16] route ids (output rows)
    uint32_t* tin = trid + kTableTiles * 16;                         // [kTableTiles][16] input rows
    uint32_t* rids = reinterpret_cast<uint32_t*>(smem3 + 5632);      // the same two for a tile beyond the cached window
    uint32_t* rins = rids + 16;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t warp = threadIdx.x >> 5;   // consumers: pipeline index; producers: W + producer index
    const uint32_t S = p.n_stages, HB = p.n_hdr, UPI = p.upi;
    constexpr uint32_t NMAT = GATEUP ? 2 : 1;
    constexpr uint32_t R = (GATEUP ? 8 : 16) * NT;       // rows of one matrix in an item
    constexpr bool PLANAR = LAYOUT == TSP_LAYOUT_PLANAR;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < S * W; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        mbar_fence_init();
    }
    pdl_wait();   // everything above touched shared memory only

    const uint32_t routed_tiles = p.token_map ? p.tasks[0] : (p.tokens + 8u * NC - 1) / (8u * NC);
    const uint32_t n_tiles = routed_tiles + p.sh_tiles;
    const uint64_t n_items = static_cast<uint64_t>(n_tiles) * p.groups;   // item = (tile, row group)
    // Static split by cost, not by item count: besides its items a token tile costs the staging of its activation rows, about
    // 0.8 items per row of 2048 columns. Routed tiles carry routes / tiles rows on average, the dense expert's tiles eight: with
    // an even split the CTAs that get the dense expert's tiles (the last ones) finished 9-14 us after the rest of a 100 us launch.
    // Cost per item in 1/256 item units: 256 + rows of the tile * row cost / groups, piecewise constant over the two kinds of tile.
    const uint64_t row_cost = 200ull * p.cols / 2048u;
    const uint64_t routes = p.token_map ? p.tasks[1] : p.tokens;
    const uint64_t ci_r = 256ull + (routed_tiles ? routes * row_cost / (static_cast<uint64_t>(routed_tiles) * p.groups) : 0ull);
    const uint64_t ci_s = 256ull + static_cast<uint64_t>(p.sh_tiles ? (p.sh_tokens + p.sh_tiles - 1) / p.sh_tiles : 0u) * row_cost / p.groups;
    const uint64_t n_r = static_cast<uint64_t>(routed_tiles) * p.groups, cost_r = n_r * ci_r, cost_all = cost_r + (n_items - n_r) * ci_s;
    auto boundary = [&](uint32_t b) -> uint32_t {
        if (b >= gridDim.x) return static_cast<uint32_t>(n_items);
        const uint64_t c = cost_all * b / gridDim.x;
        return static_cast<uint32_t>(c < cost_r ? c / ci_r : n_r + (c - cost_r) / ci_s);
    };
    const uint32_t item0 = boundary(blockIdx.x), item1 = boundary(blockIdx.x + 1);
    // Tile table: the (expert, first route, route count), route ids and input rows of the first kTableTiles token tiles this
    // CTA touches, fetched once and in parallel, so that the dependent global loads behind them are not paid at every tile.
    const uint32_t t0 = item0 / p.groups;
    for (uint32_t i = threadIdx.x; i < kTableTiles * 16; i += blockDim.x) {
        const uint32_t tl = i >> 4, slot = i & 15u, tile = t0 + tl;
        if (tile < n_tiles && item0 < item1) {
            const Tile3 ti = tile3<NC>(p, tile, routed_tiles);
            if (slot == 0) { tt[tl * 4] = ti.expert; tt[tl * 4 + 1] = ti.start; tt[tl * 4 + 2] = ti.count; }
            uint32_t rid = 0;
            if (slot < ti.count) rid = (p.token_map && ti.expert < p.experts) ? p.token_map[static_cast<uint64_t>(ti.expert) * p.tokens + ti.start + slot] : ti.start + slot;
            trid[i] = rid;
            tin[i] = ti.expert < p.experts ? rid / p.in_div : rid;
        }
    }
    __syncthreads();
    auto get_tile = [&](uint32_t tile) {
        const uint32_t tl = tile - t0;
        if (tl < kTableTiles) return Tile3{tt[tl * 4], tt[tl * 4 + 1], tt[tl * 4 + 2]};
        return tile3<NC>(p, tile, routed_tiles);
    };
    // pipeline w's items are item0 + w + 8n, each of UPI units
    auto units_of = [&](uint32_t w) { return item0 + w < item1 ? (item1 - item0 - w + W - 1) / W * UPI : 0u; };

    if (warp >= W) {
        // ---------------- producer warps: lane i < PER of producer q feeds the pipeline of consumer warp PER q + i ----------------
        // The lanes run one instruction stream: a pass issues the next unit of every pipeline whose stage is free, so a
        // pipeline waits at most one pass (a few hundred cycles) for its copy, whatever the other pipelines do.
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kProdRegs));
        constexpr uint32_t PER = W / kProd3;
        if (lane >= PER) return;
        constexpr uint32_t mask = (1u << PER) - 1u;
        const uint32_t w = (warp - W) * PER + lane;
        // Units of a pipeline are issued strictly in order, so its stage, unit, header buffer, row group and tile advance
        // incrementally; nothing here divides.
        uint32_t f_tile = (item0 + w) / p.groups, f_grp = (item0 + w) % p.groups, f_u = 0, f_s = 0, f_h = 0, f_issued = 0, f_wrap = 0;
        const uint32_t f_units = units_of(w);
        uint64_t* w_full = full + w * S;
        uint64_t* w_empty = empty + w * S;
        uint8_t* wb = smem3 + p.off_warp + w * p.warp_bytes;
        // per item: expert-local id, map index of matrix A (matrix B's is two further; the shared expert's one further), copies per plane
        int el = 0; uint32_t which = 0, ncopy = 1;
        uint32_t idle = 0;
        while (__any_sync(mask, f_issued < f_units)) {
            bool ready = f_issued < f_units;
            // the stage's previous unit must have been consumed
            if (ready && f_issued >= S) ready = mbar_try_wait(&w_empty[f_s], (f_wrap & 1u) ^ 1u);
            if (!__any_sync(mask, ready)) {
                if (++idle > (1u << 22)) { if (lane == 0) raise_error(p.error, TSP_ERR_TIMEOUT); return; }
                if (idle > 16) __nanosleep(32);
                continue;
            }
            idle = 0;
            if (ready) {
                const bool first = f_u == 0;
                if (first) {
                    const Tile3 ti = get_tile(f_tile);
                    const bool shared = ti.expert >= p.experts;
                    const bool hi = !shared && ti.expert >= p.split;
                    el = shared ? 0 : static_cast<int>(hi ? ti.expert - p.split : ti.expert);
                    which = shared ? 4u : (hi ? 1u : 0u);
                    ncopy = (NMAT == 1 || (shared ? p.sh_merged : p.merged)) ? 1u : NMAT;
                }
                const int r0 = static_cast<int>(f_grp * R);
                uint8_t* sb = wb + HB * p.hdr_bytes + f_s * p.stage_bytes;
                uint32_t bytes = NMAT * p.code_mat_bytes;
                if (PLANAR && first) bytes += NMAT * (p.sm_mat_bytes + p.dm_mat_bytes);
                mbar_arrive_expect_tx(&w_full[f_s], bytes);
                for (uint32_t m = 0; m < ncopy; ++m) {
                    const uint32_t wm = which + (which == 4 ? m : 2 * m);
                    tma_load_5d(sb + m * p.code_mat_bytes, &maps.m[wm], 0, r0, static_cast<int>(f_u * KB), 0, el, &w_full[f_s]);
                }
                if (PLANAR && first) {
                    uint8_t* hd = wb + f_h * p.hdr_bytes;
                    for (uint32_t m = 0; m < ncopy; ++m) {
                        const uint32_t wm = which + (which == 4 ? m : 2 * m);
                        tma_load_4d(hd + m * p.sm_mat_bytes, &maps.m[6 + wm], 0, static_cast<int>(f_grp * p.sm_lines), 0, el, &w_full[f_s]);
                        tma_load_4d(hd + NMAT * p.sm_mat_bytes + m * p.dm_mat_bytes, &maps.m[12 + wm], 0,
                                    static_cast<int>(f_grp * (R * p.nblk * 4 / p.dm_inner)), 0, el, &w_full[f_s]);
                    }
                }
                ++f_issued;
                if (++f_s == S) { f_s = 0; ++f_wrap; }
                if (++f_u == UPI) {
                    f_u = 0;
                    if (++f_h == HB) f_h = 0;
                    f_grp += W;
                    while (f_grp >= p.groups) { f_grp -= p.groups; ++f_tile; }
                }
            }
        }
        return;
    }

    // ---------------- consumer warps ----------------
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(cons_regs(W)));
    const uint32_t my_units = units_of(warp);
    (void)my_units;
    const uint8_t* my_hdr0 = smem3 + p.off_warp + warp * p.warp_bytes;
    const uint8_t* my_stage0 = my_hdr0 + HB * p.hdr_bytes;
    uint64_t* my_full = full + warp * S;
    uint64_t* my_empty = empty + warp * S;

    const uint32_t g = lane >> 2, t = lane & 3;
    const uint32_t ctid = threadIdx.x;
    constexpr uint32_t CT = W * 32;   // consumer threads: they alone meet at the tile-change barriers (named barrier 1)
    uint8_t* xhi = smem3 + p.off_xhi;
    uint8_t* xlo = smem3 + p.off_xlo;
    uint8_t* sxb = smem3 + p.off_sx;
    bool ok = true;
    // lane constants: byte offset of this lane's 8 code bytes of pair j inside a (swizzled) 128-byte line
    uint32_t qoff[4];
#pragma unroll
    for (uint32_t j = 0; j < 4; ++j) qoff[j] = (((2 * j + (t >> 1)) ^ (PLANAR ? g : 0u)) << 4) + (t & 1u) * 8u;
    const uint32_t xlane = g * p.x_stride + t * 16;     // this lane's B-fragment offset inside a token-row block
    const uint32_t sxlane = g * p.sx_stride + t * 4;
    const uint32_t mn_shift = 16 * (t & 1);

    // Activation chunks of the CTA's NEXT token tile, loaded into registers while the current tile is computed, so that
    // the tile change pays no global-load latency (PF chunks per thread: enough for 2 token rows of 2048 columns).
    // Only the binary16 source is fetched ahead (16 bytes per chunk).
    constexpr int PF = 2;
    uint4 pf[PF];
    uint32_t pf_tile = 0xffffffffu;
#pragma unroll
    for (int i = 0; i < PF; ++i) pf[i] = make_uint4(0, 0, 0, 0);

    uint32_t my_it = item0 + warp;                  // this ring's next item
    uint32_t my_grp = (item0 + warp) % p.groups;    // its row group
    uint32_t cs = 0, cph = 0, ch = 0;               // stage, phase and header buffer of this ring's next unit / item
    uint32_t item = item0;
    while (item < item1) {
        // ---- one token tile: the segment of this CTA's items that share it ----
        const uint32_t tile = item / p.groups;
        const uint32_t seg_end = min(item1, (tile + 1) * p.groups);
        named_bar_sync(1, CT);   // every consumer warp is done with the previous tile's activations
        const Tile3 ti = get_tile(tile);
        const uint32_t* cur_rids = trid + (tile - t0) * 16;
        const uint32_t* cur_rins = tin + (tile - t0) * 16;
        if (tile - t0 >= kTableTiles) {   // beyond the cached window: fetch this tile's route ids now
            if (ctid < 8u * NC) {
                uint32_t rid = 0;
                if (ctid < ti.count) rid = (p.token_map && ti.expert < p.experts) ? p.token_map[static_cast<uint64_t>(ti.expert) * p.tokens + ti.start + ctid] : ti.start + ctid;
                rids[ctid] = rid;
                rins[ctid] = ti.expert < p.experts ? rid / p.in_div : rid;
            }
            cur_rids = rids;
            cur_rins = rins;
            named_bar_sync(1, CT);
        }
        {
            // Stage the tile's activation rows: 8-column chunks, four per thread in flight so that their global loads overlap.
            const uint32_t per_row = p.cols / 8;
            const uint32_t units = ti.count * per_row;
            const bool sh_tile = ti.expert >= p.experts;
            bool bad = false;
            if (p.x16) {
                // binary16 rows: no conversion, only the reordering inside each run of 8 and the group sums; the first PF
                // chunks of a thread were fetched ahead while the previous tile was computed
                const bool fetched = pf_tile == tile;
                for (uint32_t base = 0; base < units; base += 4 * CT) {
                    uint4 vv[4];
                    uint32_t jj[4], kk[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t u = base + i * CT + ctid;
                        jj[i] = 0xffffffffu; kk[i] = 0;
                        vv[i] = make_uint4(0, 0, 0, 0);
                        if (u < units) {
                            jj[i] = u / per_row; kk[i] = u - jj[i] * per_row;
                            if (i < PF && base == 0 && fetched) vv[i] = pf[i < PF ? i : 0];
                            else vv[i] = *(reinterpret_cast<const uint4*>(p.x16 + cur_rins[jj[i]] * p.x16_stride_bytes) + kk[i]);
                        }
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        if (base + i * CT >= units) break;   // uniform: no thread has work in this slot
                        const bool active = jj[i] != 0xffffffffu;
                        const uint32_t j = jj[i], k8 = kk[i];
                        const uint32_t w[4] = {vv[i].x, vv[i].y, vv[i].z, vv[i].w};
                        float s = 0.f;
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[e]));
                            s += f.x + f.y;
                            bad |= (w[e] & 0x7c00u) == 0x7c00u || (w[e] & 0x7c000000u) == 0x7c000000u;
                        }
                        if (active) {
                            // permuted order inside the run of 8: positions hold elements 0,2,1,3,4,6,5,7
                            *reinterpret_cast<uint4*>(xhi + j * p.x_stride + k8 * 16) =
                                make_uint4(__byte_perm(w[0], w[1], 0x5410), __byte_perm(w[0], w[1], 0x7632), __byte_perm(w[2], w[3], 0x5410), __byte_perm(w[2], w[3], 0x7632));
                            if (SPLIT) *reinterpret_cast<uint4*>(xlo + j * p.x_stride + k8 * 16) = make_uint4(0, 0, 0, 0);
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
                }
                // fetch ahead for the next tile of this CTA (its routing data must be in the cached window)
                pf_tile = 0xffffffffu;
                if (seg_end < item1 && tile + 1 - t0 < kTableTiles) {
                    const Tile3 tn = get_tile(tile + 1);
                    const uint32_t* nrins = tin + (tile + 1 - t0) * 16;
#pragma unroll
                    for (int i = 0; i < PF; ++i) {
                        const uint32_t u = i * CT + ctid;
                        if (u < tn.count * per_row) {
                            const uint32_t jn = u / per_row, kn = u - jn * per_row;
                            pf[i] = *(reinterpret_cast<const uint4*>(p.x16 + nrins[jn] * p.x16_stride_bytes) + kn);
                        }
                    }
                    pf_tile = tile + 1;
                }
            } else {
                const char* xsrc = sh_tile ? reinterpret_cast<const char*>(p.sh_x) : reinterpret_cast<const char*>(p.x);
                const uint64_t xsrc_stride = sh_tile ? p.sh_x_stride_bytes : p.x_stride_bytes;
                for (uint32_t base = 0; base < units; base += 4 * CT) {
                    float4 va[4], vb[4];
                    uint32_t jj[4], kk[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t u = base + i * CT + ctid;
                        jj[i] = 0xffffffffu; kk[i] = 0;
                        va[i] = vb[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (u < units) {
                            jj[i] = u / per_row; kk[i] = u - jj[i] * per_row;
                            const float4* src = reinterpret_cast<const float4*>(xsrc + cur_rins[jj[i]] * xsrc_stride) + kk[i] * 2;
                            va[i] = src[0]; vb[i] = src[1];
                        }
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        if (base + i * CT >= units) break;   // uniform: no thread has work in this slot
                        const bool active = jj[i] != 0xffffffffu;
                        const uint32_t j = jj[i], k8 = kk[i];
                        const float v[8] = {va[i].x, va[i].y, va[i].z, va[i].w, vb[i].x, vb[i].y, vb[i].z, vb[i].w};
                        float s = 0.f;
                        uint32_t hb[8], lb[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            const __half h = __float2half_rn(v[e]);
                            const float hf = __half2float(h);
                            bad |= !finite_f32(hf);
                            hb[e] = __half_as_ushort(h);
                            lb[e] = __half_as_ushort(__float2half_rn(v[e] - hf));
                            s += v[e];
                        }
                        if (active) {
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
                }
            }
            if (bad) raise_error(p.error, TSP_ERR_NONFINITE);
        }
        named_bar_sync(1, CT);
        // this lane's output rows (tokens 2t, 2t+1 of each column block) for the whole tile
        float* orow[NC][2];
#pragma unroll
        for (int c = 0; c < NC; ++c)
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                const uint32_t j = c * 8 + 2 * t + q;
                orow[c][q] = j >= ti.count ? nullptr
                             : reinterpret_cast<float*>(ti.expert >= p.experts ? reinterpret_cast<char*>(p.sh_out) + cur_rids[j] * p.sh_out_stride_bytes
                                                                               : reinterpret_cast<char*>(p.out) + cur_rids[j] * p.out_stride_bytes);
            }

        // ---- this warp's row groups of the segment ----
        for (; my_it < seg_end; my_it += W) {
            const uint32_t r0 = my_grp * R;
            my_grp += W;
            while (my_grp >= p.groups) my_grp -= p.groups;
            float total[NT][NC][4];
#pragma unroll
            for (int n = 0; n < NT; ++n)
#pragma unroll
                for (int c = 0; c < NC; ++c) total[n][c][0] = total[n][c][1] = total[n][c][2] = total[n][c][3] = 0.f;
            const uint8_t* smp = my_hdr0 + ch * p.hdr_bytes;        // scale bytes: [matrix][row][super-block][16]
            const uint8_t* dmp = smp + NMAT * p.sm_mat_bytes;       // (d, dmin): [matrix][row][super-block][4]
            if (++ch == HB) ch = 0;

            for (uint32_t u = 0; u < UPI; ++u) {
                const uint32_t s = cs, ph = cph;
                if (++cs == S) { cs = 0; cph ^= 1u; }
                if (ok) {
                    ok = mbar_wait(&my_full[s], ph);
                    if (!ok && lane == 0) raise_error(p.error, TSP_ERR_TIMEOUT);
                }
                const uint8_t* sb = my_stage0 + s * p.stage_bytes;
                if (ok)
#pragma unroll
                for (uint32_t bl = 0; bl < KB; ++bl) {
                    const uint32_t b = u * KB + bl;   // super-block index along K
                    const uint8_t* xb = xhi + xlane + b * 512;
                    const uint8_t* xq = xlo + xlane + b * 512;
                    const uint8_t* sxp = sxb + sxlane + b * 16;
#pragma unroll
                    for (int n = 0; n < NT; ++n) {
                        const uint32_t rowA = GATEUP ? n * 8 + g : n * 16 + g;        // row inside matrix A's rows of the item
                        const uint32_t rowB = GATEUP ? n * 8 + g : n * 16 + 8 + g;    // gate-up: same row of matrix B
                        constexpr uint32_t boxB = GATEUP ? KB : 0;                    // matrix B's lines follow matrix A's
                        uint32_t dmA, dmB, scA[2], scB[2], mnA[2], mnB[2];
                        const uint8_t *lineA, *lineB;
                        if (PLANAR) {
                            // scale bytes sit in 128-byte lines swizzled like the codes: chunk ^= line & 7
                            const uint32_t oA = (rowA * p.nblk + b) * 16, oB = (GATEUP ? p.sm_mat_bytes : 0) + (rowB * p.nblk + b) * 16;
                            const uint8_t* smA = smp + (oA ^ (((oA >> 7) & 7u) << 4));
                            const uint8_t* smB = smp + (oB ^ (((oB >> 7) & 7u) << 4));
                            const uint4 sa = *reinterpret_cast<const uint4*>(smA), sv = *reinterpret_cast<const uint4*>(smB);
                            scA[0] = sa.x; scA[1] = sa.y; mnA[0] = sa.z; mnA[1] = sa.w;
                            scB[0] = sv.x; scB[1] = sv.y; mnB[0] = sv.z; mnB[1] = sv.w;
                            dmA = *reinterpret_cast<const uint32_t*>(dmp + (rowA * p.nblk + b) * 4);
                            dmB = *reinterpret_cast<const uint32_t*>(dmp + (GATEUP ? p.dm_mat_bytes : 0) + (rowB * p.nblk + b) * 4);
                            lineA = sb + (bl * R + rowA) * 128;   // line order: matrix, super-block, row
                            lineB = sb + ((boxB + bl) * R + rowB) * 128;
                        } else {
                            const uint8_t* blkA = sb + (bl * R + rowA) * 144;   // block order: matrix, super-block, row
                            const uint8_t* blkB = sb + ((boxB + bl) * R + rowB) * 144;
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
                // the stage is free again: tell the producer
                __syncwarp();
                if (lane == 0) mbar_arrive(&my_empty[s]);
            }
            // ---- epilogue: this warp owns its rows' complete sums ----
            if (ok) {
                bool bad = false;
#pragma unroll
                for (int n = 0; n < NT; ++n)
#pragma unroll
                    for (int c = 0; c < NC; ++c)
#pragma unroll
                        for (int q = 0; q < 2; ++q) {
                            float* o = orow[c][q];
                            if (GATEUP) {
                                const float v = fast_silu(total[n][c][q]) * total[n][c][2 + q];
                                if (o) { bad |= !finite_f32(v); o[r0 + n * 8 + g] = v; }
                            } else if (o) {
                                const uint32_t r = r0 + n * 16 + g;
                                bad |= !finite_f32(total[n][c][q]) | !finite_f32(total[n][c][2 + q]);
                                o[r] = total[n][c][q];
                                o[r + 8] = total[n][c][2 + q];
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
template <uint32_t LAYOUT, bool GATEUP, int NC, int NT, int KB, bool SPLIT, int W = kW3>
static int launch3(const Gemv3Maps& maps, const Gemv3Params& p, size_t smem, int grid, cudaStream_t st) {
    auto kernel = gemv3_kernel<LAYOUT, GATEUP, NC, NT, KB, SPLIT, W>;
    static thread_local int regs_ok = -1;   // the register hand-over between producer and consumer warps adds up for this build
    if (regs_ok < 0) {
        cudaFuncAttributes fa{};
        TSP_CUDA(cudaFuncGetAttributes(&fa, kernel));
        regs_ok = (fa.numRegs >= kProdRegs && W * (cons_regs(W) - fa.numRegs) <= kProd3 * (fa.numRegs - kProdRegs)) ? 1 : 0;
    }
    if (!regs_ok) return fail(TSP_E_CUDA, "decode projection kernel: the compiled register count does not allow the producer/consumer register hand-over");
    static thread_local SmemAttrCache configured;   // per kernel instantiation, keyed by device
    TSP_CUDA(ensure_dynamic_smem(kernel, configured, smem));
    TSP_CUDA(launch_pdl(kernel, dim3(grid), dim3((W + kProd3) * 32), smem, st, maps, p));
    return TSP_OK;
}

// The three tensor maps (codes, scale bytes, (d, dmin) pairs) of one set of expert images starting at `base`.
// `mats` = 2: the second matrix of every expert sits `delta` bytes after the first and one copy brings both.
static int make_maps(Gemv3Maps& out, uint32_t which, const uint8_t* base, uint32_t experts, uint64_t expert_stride, uint32_t mats,
                     uint64_t delta, bool planar, uint32_t rows, uint32_t nblk, uint32_t R, uint32_t kb, uint32_t dm_inner) {
    const uint64_t es = experts > 1 ? expert_stride : 16, ds = mats > 1 ? delta : 16;
    if (planar) {
        {   // codes: [128 B][row][super-block][matrix][expert]
            const uint64_t dims[5] = {128, rows, nblk, mats, experts}, strides[4] = {static_cast<uint64_t>(nblk) * 128, 128, ds, es};
            const uint32_t box[5] = {128, R, kb, mats, 1};
            if (int rc = get_tensor_map_bytes(base, 5, dims, strides, box, true, &out.m[which])) return rc;
        }
        const uint64_t units = static_cast<uint64_t>(rows) * nblk;
        {   // scale bytes: [128 B][line][matrix][expert]
            const uint64_t dims[4] = {128, units / 8, mats, experts}, strides[3] = {128, ds, es};
            const uint32_t box[4] = {128, R * nblk / 8, mats, 1};
            if (int rc = get_tensor_map_bytes(base + units * 128, 4, dims, strides, box, true, &out.m[6 + which])) return rc;
        }
        {   // (d, dmin) pairs: [dm_inner B][line][matrix][expert]
            const uint64_t dims[4] = {dm_inner, units * 4 / dm_inner, mats, experts}, strides[3] = {dm_inner, ds, es};
            const uint32_t box[4] = {dm_inner, R * nblk * 4 / dm_inner, mats, 1};
            if (int rc = get_tensor_map_bytes(base + units * 144, 4, dims, strides, box, false, &out.m[12 + which])) return rc;
        }
    } else {   // whole blocks: [144 B][row][super-block][matrix][expert]
        const uint64_t dims[5] = {144, rows, nblk, mats, experts}, strides[4] = {static_cast<uint64_t>(nblk) * 144, 144, ds, es};
        const uint32_t box[5] = {144, R, kb, mats, 1};
        if (int rc = get_tensor_map_bytes(base, 5, dims, strides, box, false, &out.m[which])) return rc;
        out.m[6 + which] = out.m[which];
        out.m[12 + which] = out.m[which];
    }
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
    const bool planar = a->layout == TSP_LAYOUT_PLANAR;
    Gemv3Params p{};
    p.split = a->split < a->experts ? a->split : a->experts;
    p.experts = a->experts;
    p.rows = a->rows; p.cols = a->cols; p.nblk = nblk;
    // item geometry: plain projections with a short K take two row tiles per item
    const uint32_t nt = (!gateup && nblk <= 2 && a->rows % 32 == 0) ? 2 : 1;
    const uint32_t R = (gateup ? 8 : 16) * nt;
    const uint32_t nmat = gateup ? 2 : 1;
    // Eight pipelines. Sixteen (104 registers per consumer thread, stages of one super-block) were measured on the short-K
    // plain projection of the decode layer: 0.077 ms against 0.067 ms with eight, so no launch selects them.
    uint32_t warps = static_cast<uint32_t>(kW3);
    const uint32_t tok = 8u * static_cast<uint32_t>(nc);
    const bool split_lo = !f16_exact;
    uint32_t kb = 1, off = 0, best_s = 0, best_h = 0;
    for (;;) {
        kb = warps == 16 ? 1 : (nblk % 4 == 0 && nblk >= 8) ? 4 : (nblk % 2 == 0 && (nblk >= 4 || nt == 2)) ? 2 : 1;
        if (R * nblk > 2048) return 1;   // header boxes are limited to 256 lines
        p.upi = nblk / kb;
        p.groups = a->rows / R;
        p.code_mat_bytes = R * kb * (planar ? 128 : 144);
        p.stage_bytes = (nmat * p.code_mat_bytes + 1023u) & ~1023u;
        p.sm_mat_bytes = planar ? R * nblk * 16 : 0;
        p.dm_mat_bytes = planar ? R * nblk * 4 : 0;
        if (nmat == 2 && p.dm_mat_bytes % 128) return 1;   // the second matrix's pairs must start on a 128-byte boundary
        p.sm_lines = R * nblk / 8;
        for (p.dm_inner = 256; p.dm_inner > 16 && (R * nblk * 4) % p.dm_inner; p.dm_inner >>= 1) {}
        p.hdr_bytes = (nmat * (p.sm_mat_bytes + p.dm_mat_bytes) + 1023u) & ~1023u;
        p.x_stride = a->cols * 2 + 64;
        p.sx_stride = (a->cols / 32) * 2 + 16;
        off = 6144;   // barriers, tile tables, fallback route ids
        p.off_xhi = off; off += tok * p.x_stride;
        p.off_xlo = off; if (split_lo) off += tok * p.x_stride;
        p.off_sx = off; off += 2 * tok * p.sx_stride;
        off = (off + 1023u) & ~1023u;
        p.off_warp = off;
        const uint32_t budget = 226 * 1024;   // 1 KB of the 227 KB is kept for aligning the dynamic base
        if (off >= budget) return 1;
        const uint32_t per_warp = ((budget - off) / warps) & ~1023u;
        const uint32_t max_stages = warps == 16 ? 4u : kMaxStages3;   // the barrier arrays hold 64 entries
        // pipeline depth and header buffers: a header buffer is reused after n_hdr items, so the producer may run at most
        // (n_hdr - 1) items + 1 unit ahead of the consumer
        best_s = 0; best_h = 0;
        for (uint32_t h = planar ? 2 : 0; h <= (planar ? kMaxHeaders3 : 0); ++h) {
            if (h * p.hdr_bytes + 2 * p.stage_bytes > per_warp) break;
            uint32_t s = (per_warp - h * p.hdr_bytes) / p.stage_bytes;
            if (s > max_stages) s = max_stages;
            if (planar && s > (h - 1) * p.upi + 1) s = (h - 1) * p.upi + 1;
            if (s > best_s) { best_s = s; best_h = h; }
        }
        if (best_s >= 2 || warps == static_cast<uint32_t>(kW3)) break;
        warps = kW3;
    }
    if (best_s < 2) return 1;   // too little room for a double-buffered pipeline per warp
    p.n_stages = best_s; p.n_hdr = best_h;
    p.warp_bytes = p.n_hdr * p.hdr_bytes + p.n_stages * p.stage_bytes;
    const size_t smem = off + static_cast<size_t>(warps) * p.warp_bytes + 1024;
    p.x = x; p.x_stride_bytes = x_stride_bytes; p.in_div = in_div ? in_div : 1;
    p.token_map = token_map; p.counts = counts; p.tasks = tasks; p.tokens = tokens;
    p.out = out; p.out_stride_bytes = out_stride_bytes; p.error = error;

    // ---- tensor maps ----
    const uint8_t* base[4] = {static_cast<const uint8_t*>(a->base), static_cast<const uint8_t*>(a->base_hi ? a->base_hi : a->base), nullptr, nullptr};
    if (gateup) {
        base[2] = static_cast<const uint8_t*>(b->base);
        base[3] = static_cast<const uint8_t*>(b->base_hi ? b->base_hi : b->base);
    }
    const uint64_t stride = a->experts > 1 ? a->expert_stride : 16;
    if (stride % 16) return 1;
    for (int m = 0; m < (gateup ? 4 : 2); ++m)
        if (reinterpret_cast<uintptr_t>(base[m]) % 16) return 1;
    auto mergeable = [](const uint8_t* first, const uint8_t* second, uint64_t* delta) {
        if (second <= first) return false;
        *delta = static_cast<uint64_t>(second - first);
        return *delta % 16 == 0 && *delta < (1ull << 40);
    };
    uint64_t delta = 0, delta_hi = 0;
    p.merged = gateup && mergeable(base[0], base[2], &delta) && mergeable(base[1], base[3], &delta_hi) && delta == delta_hi;
    const uint32_t n_lo = p.split, n_hi = a->experts - p.split;
    Gemv3Maps maps;
    for (uint32_t m = 0; m < (gateup && !p.merged ? 2u : 1u); ++m) {
        if (int rc = make_maps(maps, 2 * m, base[2 * m], n_lo ? n_lo : 1, stride, p.merged ? 2 : 1, delta, planar, a->rows, nblk, R, kb, p.dm_inner)) return rc;
        if (n_hi) {
            if (int rc = make_maps(maps, 2 * m + 1, base[2 * m + 1], n_hi, stride, p.merged ? 2 : 1, delta, planar, a->rows, nblk, R, kb, p.dm_inner)) return rc;
        } else {
            for (int pl = 0; pl < 3; ++pl) maps.m[pl * 6 + 2 * m + 1] = maps.m[pl * 6 + 2 * m];
        }
    }
    if (!gateup || p.merged)
        for (int pl = 0; pl < 3; ++pl) { maps.m[pl * 6 + 2] = maps.m[pl * 6]; maps.m[pl * 6 + 3] = maps.m[pl * 6 + 1]; }
    for (int pl = 0; pl < 3; ++pl) { maps.m[pl * 6 + 4] = maps.m[pl * 6]; maps.m[pl * 6 + 5] = maps.m[pl * 6]; }
    if (shared) {
        p.sh_tokens = shared->tokens ? shared->tokens : tokens;
        p.sh_tiles = (p.sh_tokens + 7) / 8;
        p.sh_x = shared->x; p.sh_x_stride_bytes = shared->x_stride_bytes;
        p.sh_out = shared->out; p.sh_out_stride_bytes = shared->out_stride_bytes;
        if (shared->x16 && f16_exact && reinterpret_cast<uintptr_t>(shared->x16) % 16 == 0 && shared->x16_stride_bytes % 16 == 0) {
            p.x16 = static_cast<const uint8_t*>(shared->x16); p.x16_stride_bytes = shared->x16_stride_bytes;
        }
        const uint8_t* sa = static_cast<const uint8_t*>(shared->a->base);
        const uint8_t* sb = gateup ? static_cast<const uint8_t*>(shared->b->base) : nullptr;
        if (reinterpret_cast<uintptr_t>(sa) % 16 || reinterpret_cast<uintptr_t>(sb) % 16) return 1;
        uint64_t sdelta = 0;
        p.sh_merged = gateup && mergeable(sa, sb, &sdelta);
        if (int rc = make_maps(maps, 4, sa, 1, 16, p.sh_merged ? 2 : 1, sdelta, planar, a->rows, nblk, R, kb, p.dm_inner)) return rc;
        if (gateup && !p.sh_merged) {
            if (int rc = make_maps(maps, 5, sb, 1, 16, 1, 0, planar, a->rows, nblk, R, kb, p.dm_inner)) return rc;
        }
    }
    const int grid = sm_count();
    if (grid <= 0) return fail(TSP_E_CUDA, "no usable CUDA device");
#define TSP_D4(L, G, NCV, NTV, K)                                                  \
    return split_lo ? launch3<L, G, NCV, NTV, K, true>(maps, p, smem, grid, st)    \
                    : launch3<L, G, NCV, NTV, K, false>(maps, p, smem, grid, st)
#define TSP_D3(L, G, NCV, NTV)                                                     \
    do { if (kb == 4) { TSP_D4(L, G, NCV, NTV, 4); } else if (kb == 2) { TSP_D4(L, G, NCV, NTV, 2); } else { TSP_D4(L, G, NCV, NTV, 1); } } while (0)
#define TSP_D2(L)                                                                  \
    if (a->layout == L) {                                                          \
        if (gateup) { if (nc == 1) TSP_D3(L, true, 1, 1); TSP_D3(L, true, 2, 1); } \
        if (nt == 2) { if (kb == 2) { if (nc == 1) TSP_D4(L, false, 1, 2, 2); TSP_D4(L, false, 2, 2, 2); } if (nc == 1) TSP_D4(L, false, 1, 2, 1); TSP_D4(L, false, 2, 2, 1); } \
        if (nc == 1) TSP_D3(L, false, 1, 1);                                       \
        TSP_D3(L, false, 2, 1);                                                    \
    }
    TSP_D2(TSP_LAYOUT_PLANAR)
    TSP_D2(TSP_LAYOUT_GGUF)
#undef TSP_D2
#undef TSP_D3
#undef TSP_D4
    return 1;
}

}  // namespace tsp
