// Prefill-size grouped expert GEMMs on the 5th-generation tensor cores (tcgen05) for sm_100a.
//
// One launch computes, for every tile of <= 128 routes of one expert, either
//   gate-up:  H[pos][h]  = silu(W_gate[h] . x[pos]) * (W_up[h] . x[pos])     (two accumulators sharing the activation tile)
//   down:     Y[route][c] = W_down[c] . H[pos]
// with the weights as the M operand (128 weight rows per CTA tile fill the MMA's M extent whatever the number of
// tokens), the tokens as the N operand (32, 64 or 128 columns) and K walked in chunks of 64.
//
// Roles inside a CTA (one persistent CTA per SM):
//   warp 0      TMA producer of the quantised planes: Pack v3 planar code boxes + 6-bit factor boxes of one super-block
//               (256 columns of K) per quant stage, gate and up in one copy each; the (d, dmin) pairs once per item.
//   warp 1      allocates tensor memory, issues tcgen05.mma (one elected lane), commits to mbarriers.
//   warps 2..9  dequantise (two warps per SM sub-partition, a thread per half row of a K chunk): read 4-bit codes +
//               6-bit factors from the quant stage, write binary16 weights in the K-major 128-byte-swizzled operand layout.
//   warp 10     TMA producer of the activation tiles (tokens x 64 binary16, 128-byte swizzled) of every K chunk.
//   warps 11..18 epilogue (two per tensor-memory lane quarter): tcgen05.ld of their 32 accumulator lanes, SwiGLU / store. The accumulators are double-buffered
//               in tensor memory (2 x 256 columns), so the epilogue of an item runs under the MMAs of the next one.
// Accumulation is FP32 in tensor memory. Operands are binary16 (kind::f16, f16 inputs): the activations of this path are
// binary16-exact, and Q4_K values keep 11 significant bits instead of bf16's 8, which keeps the two chained GEMMs well
// inside the 2e-3 relative-L2 bar that bf16 operands would only just meet.
// Every mbarrier wait is bounded; a timeout sets TSP_ERR_TIMEOUT, and every path still frees the tensor memory.
#include <cuda.h>

#include "tsp_common.cuh"

namespace tsp {

int get_tensor_map_bytes(const void* base, uint32_t rank, const uint64_t* dims, const uint64_t* strides, const uint32_t* box,
                         bool swizzle128, CUtensorMap* out);

// ---------------------------------------------------------------------------------------------
// tcgen05 / TMEM wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// D[tmem] (+)= A[smem desc] * B[smem desc], kind::f16, one CTA
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// arrive on an mbarrier when all MMAs issued so far by this thread have completed
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// 32 lanes x 16 consecutive columns of 32-bit accumulators -> 16 registers per thread
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
}
// 32 lanes x 32 consecutive columns -> 32 registers per thread
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_load_4d_g(void* smem_dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
                 ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                 : "memory");
}

// Shared-memory matrix descriptor of a K-major operand tile whose rows are 128 bytes (64 binary16) in the 128-byte swizzle:
// start address >> 4, leading byte offset (unused for this layout) 1, stride byte offset 1024 (eight rows), descriptor
// version 1 (sm_100), layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t umma_desc_k128(const void* smem_tile) {
    const uint64_t addr = smem_u32(smem_tile);
    return ((addr & 0x3FFFFull) >> 4) | (1ull << 16) | (uint64_t(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor for kind::f16: D = FP32, A = B = binary16, both K-major, M x N tile.
__host__ __device__ constexpr uint32_t umma_idesc_f16(uint32_t m, uint32_t n) {
    return (1u << 4) | (0u << 7) | (0u << 10) | (0u << 15) | (0u << 16) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

constexpr uint32_t kDqWarps = 8;           // dequantise warps: two per SM sub-partition, each thread half a row of a K chunk
// epilogue warps: two per tensor-memory lane quarter, taking the 32-column batches in turn (with one per quarter the down
// GEMM, whose items are only 8 K chunks long, was bound by its epilogue: 0.39 ms against 0.26 ms)
__host__ __device__ constexpr uint32_t ep_warps(bool) { return 8u; }
__host__ __device__ constexpr uint32_t g_warps(bool gateup) { return 3 + kDqWarps + ep_warps(gateup); }   // weight producer, MMA, dequant warps, activation producer, epilogue warps
constexpr uint32_t kMaxBStages = 8;
constexpr uint32_t kTileRoutes = 128;      // routes per tile (N extent at most)
constexpr uint32_t kRowsM = 128;           // weight rows per CTA tile (M)
constexpr uint32_t kChunkK = 64;           // K per pipeline step: 64 binary16 = one 128-byte swizzled row

// Tensor maps of one launch: codes (low ids, high ids; second matrix low, high), factors (same four), (d, dmin) pairs (same four),
// activation tiles of 32 / 64 / 128 token rows.
// Indices 4, 5 of q / f / d and 3..5 of x belong to the optional dense shared expert of the layer (sh_tiles != 0).
struct alignas(64) GroupedMaps { CUtensorMap q[6], f[6], d[6], x[6]; };

struct GroupedParams {
    uint32_t split, experts;
    uint32_t rows, cols, nblk;     // rows of ONE matrix, K, super-blocks per row
    uint32_t row_blocks;           // rows / 128
    uint32_t merged;               // both matrices of an expert arrive with one copy per plane
    // optional dense shared expert processed by the same launch after the routed tiles: every one of sh_tokens rows, in
    // row order (position = token = route id), its own activation rows and output rows
    uint32_t sh_tiles, sh_tokens, sh_merged;
    void* sh_out; uint64_t sh_out_stride_bytes;
    // routes
    const uint32_t* tasks;         // {tiles, routes, (expert, start)...} with tiles of kTileRoutes
    const uint32_t* counts;
    const uint32_t* offsets;       // first permuted position of each expert
    const uint32_t* pos_route;     // route id (token*selected + slot) of each permuted position
    // output
    void* out; uint64_t out_stride_bytes;
    uint32_t* error;
    // shared-memory plan
    uint32_t off_q, q_stage_bytes, off_d, d_stage_bytes, dm_mat_bytes, off_a, off_b, nb_stages;
};

// bounded wait with a short limit: a stalled pipeline ends in tens of milliseconds, never hangs
__device__ __forceinline__ bool gwait(uint64_t* bar, uint32_t parity) { return mbar_wait(bar, parity, 1u << 21); }

struct GTile { uint32_t expert, start, count, row0, ncols; };

// A tile of the shared expert carries the expert id p.experts (one past the routed ids).
__device__ __forceinline__ GTile gtile(const GroupedParams& p, uint32_t tile) {
    GTile t;
    const uint32_t routed = p.tasks[0];
    if (tile >= routed) {
        t.expert = p.experts;
        t.start = (tile - routed) * kTileRoutes;
        t.count = t.start < p.sh_tokens ? min(p.sh_tokens - t.start, kTileRoutes) : 0u;
        t.row0 = t.start;
        t.ncols = t.count <= 32 ? 32u : (t.count <= 64 ? 64u : 128u);
        return t;
    }
    t.expert = p.tasks[2 + 2 * tile];
    t.start = p.tasks[3 + 2 * tile];
    if (t.expert >= p.experts) { t.expert = 0; t.start = 0; t.count = 0; t.row0 = 0; t.ncols = 32; return t; }
    const uint32_t c = p.counts[t.expert];
    t.count = c > t.start ? min(c - t.start, kTileRoutes) : 0u;
    t.row0 = p.offsets[t.expert] + t.start;
    t.ncols = t.count <= 32 ? 32u : (t.count <= 64 ? 64u : 128u);
    return t;
}

__device__ __forceinline__ void tma_load_5d_g(void* smem_dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, int c4, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
                 ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
                 : "memory");
}

// GATEUP: two weight matrices (gate, up) and the SwiGLU epilogue writing binary16 hidden rows in permuted position order;
// otherwise one matrix and FP32 rows scattered to their route ids.
template <bool GATEUP>
__global__ void __launch_bounds__(g_warps(GATEUP) * 32, 1) grouped_mma_kernel(const __grid_constant__ GroupedMaps maps, const GroupedParams p) {
    pdl_launch_dependents();
    extern __shared__ uint8_t gsm_raw[];
    uint8_t* gsm = gsm_raw + ((1024u - (smem_u32(gsm_raw) & 1023u)) & 1023u);
    uint64_t* bars = reinterpret_cast<uint64_t*>(gsm);
    // rings: quantised super-blocks (2 stages, TMA), the (d, dmin) pairs of an item (2 stages, TMA), dequantised weight tiles
    // (2 stages, filled by the dequant warps) and activation tiles (nb_stages, TMA); the activation ring is deep because its
    // loads see full memory latency while a weight tile is produced on chip
    uint64_t *qfull = bars, *qempty = bars + 2, *afull = bars + 4, *aempty = bars + 6, *dfull = bars + 8, *dempty = bars + 10,
             *bfull = bars + 12, *bempty = bars + 12 + kMaxBStages, *acc_full = bars + 12 + 2 * kMaxBStages, *acc_empty = acc_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gsm + 512);
    const uint32_t NB = p.nb_stages;
    constexpr uint32_t NMAT = GATEUP ? 2 : 1;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < 2; ++s) {
            mbar_init(&qfull[s], 1); mbar_init(&qempty[s], kDqWarps);
            mbar_init(&afull[s], kDqWarps); mbar_init(&aempty[s], 1);
            mbar_init(&dfull[s], 1); mbar_init(&dempty[s], kDqWarps);
        }
        for (uint32_t s = 0; s < NB; ++s) { mbar_init(&bfull[s], 1); mbar_init(&bempty[s], 1); }
        for (int s = 0; s < 2; ++s) { mbar_init(&acc_full[s], 1); mbar_init(&acc_empty[s], ep_warps(GATEUP)); }
        mbar_fence_init();
    }
    if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }   // two accumulator sets of 256 columns: the epilogue of an item overlaps the MMAs of the next
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();   // everything above touched shared and tensor memory only

    const uint32_t n_tiles = p.tasks[0] + p.sh_tiles;
    const uint64_t n_items = static_cast<uint64_t>(n_tiles) * p.row_blocks;
    const uint32_t item0 = static_cast<uint32_t>(n_items * blockIdx.x / gridDim.x);
    const uint32_t item1 = static_cast<uint32_t>(n_items * (blockIdx.x + 1) / gridDim.x);
    const uint32_t chunks_per_item = p.nblk * 4;   // K chunks of 64

    if (warp == 0) {
        // =========================== TMA producer of the quantised planes ===========================
        if (lane == 0) {
            bool ok = true;
            uint32_t qs = 0, qph = 0, ds = 0, dph = 0, cur_tile = 0xffffffffu;
            GTile t{};
            for (uint32_t item = item0; item < item1 && ok; ++item) {
                if (item / p.row_blocks != cur_tile) { cur_tile = item / p.row_blocks; t = gtile(p, cur_tile); }   // consecutive items share the tile
                const int r0 = static_cast<int>((item % p.row_blocks) * kRowsM);
                const bool shared = t.expert >= p.experts;
                const bool hi = !shared && t.expert >= p.split;
                const int el = shared ? 0 : static_cast<int>(hi ? t.expert - p.split : t.expert);
                const uint32_t mi = shared ? 4u : (hi ? 1u : 0u);                 // map of matrix A; matrix B's is `ms` further
                const uint32_t ms = shared ? 1u : 2u;
                const uint32_t ncopy = (NMAT == 1 || (shared ? p.sh_merged : p.merged)) ? 1u : NMAT;
                // the (d, dmin) pairs of the item's rows over the whole K
                ok = gwait(&dempty[ds], dph ^ 1u);
                if (!ok) break;
                mbar_arrive_expect_tx(&dfull[ds], NMAT * p.dm_mat_bytes);
                for (uint32_t m = 0; m < ncopy; ++m)
                    tma_load_4d_g(gsm + p.off_d + ds * p.d_stage_bytes + m * p.dm_mat_bytes, &maps.d[mi + ms * m], 0,
                                  static_cast<int>((item % p.row_blocks) * 2 * p.nblk), 0, el, &dfull[ds]);
                if (++ds == 2) { ds = 0; dph ^= 1u; }
                for (uint32_t sb = 0; sb < p.nblk && ok; ++sb) {
                    // quant stage: code boxes and factor boxes of this super-block
                    ok = gwait(&qempty[qs], qph ^ 1u);
                    if (!ok) break;
                    uint8_t* q = gsm + p.off_q + qs * p.q_stage_bytes;
                    mbar_arrive_expect_tx(&qfull[qs], NMAT * (kRowsM * 128u + kRowsM * 16u));
                    for (uint32_t m = 0; m < ncopy; ++m) {
                        tma_load_5d_g(q + m * 16384u, &maps.q[mi + ms * m], 0, r0, static_cast<int>(sb), 0, el, &qfull[qs]);
                        tma_load_4d_g(q + NMAT * 16384u + m * 2048u, &maps.f[mi + ms * m], static_cast<int>(sb * 16), r0, 0, el, &qfull[qs]);
                    }
                    if (++qs == 2) { qs = 0; qph ^= 1u; }
                }
            }
            if (!ok) raise_error(p.error, TSP_ERR_TIMEOUT);
        }
    } else if (warp == 2 + kDqWarps) {
        // =========================== activation-tile producer ===========================
        if (lane == 0) {
            bool ok = true;
            uint32_t bs = 0, bph = 0, cur_tile = 0xffffffffu;
            GTile t{};
            for (uint32_t item = item0; item < item1 && ok; ++item) {
                if (item / p.row_blocks != cur_tile) { cur_tile = item / p.row_blocks; t = gtile(p, cur_tile); }   // consecutive items share the tile
                const CUtensorMap* xmap = &maps.x[(t.expert >= p.experts ? 3 : 0) + (t.ncols == 32 ? 0 : (t.ncols == 64 ? 1 : 2))];
                for (uint32_t c = 0; c < chunks_per_item && ok; ++c) {
                    ok = gwait(&bempty[bs], bph ^ 1u);
                    if (!ok) break;
                    mbar_arrive_expect_tx(&bfull[bs], t.ncols * 128u);
                    // byte coordinate: the map's element is a byte
                    tma_load_2d(gsm + p.off_b + bs * 16384u, xmap, static_cast<int>(c * 128), static_cast<int>(t.row0), &bfull[bs]);
                    if (++bs == NB) { bs = 0; bph ^= 1u; }
                }
            }
            if (!ok) raise_error(p.error, TSP_ERR_TIMEOUT);
        }
    } else if (warp == 1) {
        // =========================== MMA issuer ===========================
        if (lane == 0) {
            bool ok = true;
            uint32_t ms = 0, mph = 0, bs = 0, bph = 0, ab = 0, accph = 0, cur_tile = 0xffffffffu;
            GTile t{};
            for (uint32_t item = item0; item < item1 && ok; ++item) {
                if (item / p.row_blocks != cur_tile) { cur_tile = item / p.row_blocks; t = gtile(p, cur_tile); }   // consecutive items share the tile
                const uint32_t idesc = umma_idesc_f16(kRowsM, t.ncols);
                ok = gwait(&acc_empty[ab], accph ^ 1u);   // the epilogue has drained this accumulator set (used two items ago)
                if (!ok) break;
                tc_fence_after();
                for (uint32_t c = 0; c < chunks_per_item && ok; ++c) {
                    ok = gwait(&afull[ms], mph) && gwait(&bfull[bs], bph);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t bdesc = umma_desc_k128(gsm + p.off_b + bs * 16384u);
#pragma unroll
                    for (uint32_t m = 0; m < NMAT; ++m) {
                        const uint64_t adesc = umma_desc_k128(gsm + p.off_a + ms * NMAT * 16384u + m * 16384u);
#pragma unroll
                        for (uint32_t kk = 0; kk < 4; ++kk)
                            umma_f16(tmem_base + ab * 256u + m * 128u, adesc + kk * 2, bdesc + kk * 2, idesc, (c | kk) != 0 ? 1u : 0u);
                    }
                    umma_commit(&aempty[ms]);   // both rings' stages are free once the MMAs above have read them
                    umma_commit(&bempty[bs]);
                    if (++ms == 2) { ms = 0; mph ^= 1u; }
                    if (++bs == NB) { bs = 0; bph ^= 1u; }
                }
                if (ok) umma_commit(&acc_full[ab]);
                if (++ab == 2) { ab = 0; accph ^= 1u; }
            }
            if (!ok) raise_error(p.error, TSP_ERR_TIMEOUT);
        }
    } else if (warp < 2 + kDqWarps) {
        // =========================== dequantise (warps 2 .. 2 + kDqWarps - 1) ===========================
        const uint32_t dw = warp - 2;                         // 0..7
        const uint32_t row = (dw & 3u) * 32 + lane;           // weight row of the tile this thread dequantises ...
        const uint32_t kh = dw >> 2;                          // ... and which half of every 64-wide K chunk (code bytes 16 kh .. 16 kh + 15)
        const uint32_t sw = row & 7u;
        bool ok = true;
        uint32_t qs = 0, qph = 0, ms = 0, mph = 0, ds = 0, dph = 0;
        for (uint32_t item = item0; item < item1; ++item) {
            if (ok) ok = gwait(&dfull[ds], dph);
            const uint8_t* dmp = gsm + p.off_d + ds * p.d_stage_bytes;
            for (uint32_t sb = 0; sb < p.nblk; ++sb) {
                if (ok) ok = gwait(&qfull[qs], qph);
                const uint8_t* q = gsm + p.off_q + qs * p.q_stage_bytes;
                // per matrix: d, dmin and the sixteen 6-bit factors of this row's super-block
                float dd[NMAT], dmn[NMAT];
                uint4 fac[NMAT];
#pragma unroll
                for (uint32_t m = 0; m < NMAT; ++m) {
                    fac[m] = *reinterpret_cast<const uint4*>(q + NMAT * 16384u + m * 2048u + row * 16u);
                    const uint32_t dmw = *reinterpret_cast<const uint32_t*>(dmp + m * p.dm_mat_bytes + (row * p.nblk + sb) * 4u);
                    dd[m] = half_bits_to_float(dmw & 0xffffu);
                    dmn[m] = half_bits_to_float(dmw >> 16);
                    if (ok && (!finite_f32(dd[m]) || !finite_f32(dmn[m]))) raise_error(p.error, TSP_ERR_NONFINITE);
                }
                for (uint32_t c = 0; c < 4; ++c) {
                    if (ok) ok = gwait(&aempty[ms], mph ^ 1u);   // the MMAs that read this A tile two chunks ago are done
                    if (ok) {
#pragma unroll
                        for (uint32_t m = 0; m < NMAT; ++m) {
                            const uint8_t* line = q + m * 16384u + row * 128u;
                            const uint4 w0 = *reinterpret_cast<const uint4*>(line + (((2 * c + kh) ^ sw) << 4));
                            const uint32_t scw = c < 2 ? fac[m].x : fac[m].y, mnw = c < 2 ? fac[m].z : fac[m].w;
                            // factor byte -> float through the 2^23 magic number (0x4B0000bb = 2^23 + bb), folded into one FMA each
                            const uint32_t selL = 0x7440u + 2u * (c & 1u), selH = selL + 1u;
                            const float s_lo = fmaf(dd[m], __uint_as_float(__byte_perm(scw, 0x4b000000u, selL)), dd[m] * -8388608.f);
                            const float s_hi = fmaf(dd[m], __uint_as_float(__byte_perm(scw, 0x4b000000u, selH)), dd[m] * -8388608.f);
                            const float m_lo = fmaf(dmn[m], __uint_as_float(__byte_perm(mnw, 0x4b000000u, selL)), dmn[m] * -8388608.f);
                            const float m_hi = fmaf(dmn[m], __uint_as_float(__byte_perm(mnw, 0x4b000000u, selH)), dmn[m] * -8388608.f);
                            const __half2 sL = __float2half2_rn(s_lo), sH = __float2half2_rn(s_hi);
                            const __half2 nL = __float2half2_rn(-m_lo), nH = __float2half2_rn(-m_hi);
                            const __half2 k1024 = __float2half2_rn(1024.f), k16th = __float2half2_rn(0.0625f), kn64 = __float2half2_rn(-64.f);
                            uint8_t* arow = gsm + p.off_a + ms * NMAT * 16384u + m * 16384u + row * 128u;
                            const uint32_t words[4] = {w0.x, w0.y, w0.z, w0.w};
                            // output chunk qq (8 binary16 = K positions 8qq..8qq+7 of this 64-wide slice, in the shared 0,2,1,3,4,6,5,7 order):
                            // qq < 4 from the low nibbles of code bytes 8qq..8qq+7, qq >= 4 from the high nibbles of bytes 8(qq-4)..; this
                            // thread has bytes 16 kh .. 16 kh + 15, i.e. qq = 2 kh, 2 kh + 1 and their high-nibble partners
#pragma unroll
                            for (uint32_t q2 = 0; q2 < 2; ++q2) {
                                const uint32_t qq = 2 * kh + q2;
                                const uint32_t a = words[2 * q2], b = words[2 * q2 + 1];
                                uint32_t lo[4], hi4[4];
                                const uint32_t src[4] = {a, a >> 8, b, b >> 8};
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    const uint32_t l = (src[i] & 0x000f000fu) | 0x64006400u;     // 1024 + q
                                    const uint32_t h = (src[i] & 0x00f000f0u) | 0x64006400u;     // 1024 + 16 q
                                    const __half2 ql = __hsub2(*reinterpret_cast<const __half2*>(&l), k1024);
                                    const __half2 qh = __hfma2(*reinterpret_cast<const __half2*>(&h), k16th, kn64);
                                    const __half2 wl = __hfma2(ql, sL, nL), wh = __hfma2(qh, sH, nH);
                                    lo[i] = *reinterpret_cast<const uint32_t*>(&wl);
                                    hi4[i] = *reinterpret_cast<const uint32_t*>(&wh);
                                }
                                *reinterpret_cast<uint4*>(arow + ((qq ^ sw) << 4)) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                                *reinterpret_cast<uint4*>(arow + (((qq + 4) ^ sw) << 4)) = make_uint4(hi4[0], hi4[1], hi4[2], hi4[3]);
                            }
                        }
                        fence_async_smem();   // make the generic-proxy writes visible to the tensor-core (async) proxy
                    }
                    __syncwarp();
                    if (lane == 0 && ok) mbar_arrive(&afull[ms]);
                    if (++ms == 2) { ms = 0; mph ^= 1u; }
                }
                __syncwarp();
                if (lane == 0 && ok) mbar_arrive(&qempty[qs]);
                if (++qs == 2) { qs = 0; qph ^= 1u; }
            }
            __syncwarp();
            if (lane == 0 && ok) mbar_arrive(&dempty[ds]);
            if (++ds == 2) { ds = 0; dph ^= 1u; }
        }
        if (!ok && lane == 0) raise_error(p.error, TSP_ERR_TIMEOUT);
    } else {
        // =========================== epilogue (the last ep_warps warps) ===========================
        const uint32_t quarter = warp & 3u;                   // tensor-memory lane quarter this warp may read
        constexpr uint32_t EH = ep_warps(GATEUP) / 4;         // warps per quarter: they take the 32-column batches in turn
        const uint32_t ehalf = (warp - (3 + kDqWarps)) >> 2;
        bool ok = true;
        uint32_t ab = 0, accph = 0, cur_tile = 0xffffffffu;
        GTile t{};
        for (uint32_t item = item0; item < item1; ++item) {
            if (item / p.row_blocks != cur_tile) { cur_tile = item / p.row_blocks; t = gtile(p, cur_tile); }   // consecutive items share the tile
            const uint32_t rb = item % p.row_blocks;
            // this warp's 32 accumulator lanes = weight rows rb*128 + quarter*32 + lane, all token columns
            // route ids of the tile's positions, fetched before the wait so their latency hides behind the MMAs:
            // lane l keeps positions l, 32 + l, 64 + l, 96 + l
            uint32_t rt[4] = {0, 0, 0, 0};
            if (!GATEUP) {
#pragma unroll
                for (uint32_t qd = 0; qd < 4; ++qd)
                    if (qd * 32 + lane < t.count) rt[qd] = t.expert >= p.experts ? t.row0 + qd * 32 + lane : p.pos_route[t.row0 + qd * 32 + lane];
            }
            if (ok) ok = gwait(&acc_full[ab], accph);
            if (ok) {
                tc_fence_after();
                const uint32_t wrow = rb * kRowsM + quarter * 32 + lane;
                const uint32_t taddr = tmem_base + ((quarter * 32u) << 16) + ab * 256u;
                // hidden rows feed the down GEMM as its K operand: same order inside each run of 8 as the weight tiles use
                const uint32_t hcol = (wrow & ~7u) | ((wrow & 4u) | ((wrow & 1u) << 1) | ((wrow & 2u) >> 1));
                char* const obase = reinterpret_cast<char*>(t.expert >= p.experts ? p.sh_out : p.out);
                const uint64_t ostride = t.expert >= p.experts ? p.sh_out_stride_bytes : p.out_stride_bytes;
                char* hrow = obase + static_cast<uint64_t>(t.row0) * ostride + (GATEUP ? hcol * 2 : 0);
                bool bad = false;
                for (uint32_t j0 = ehalf * 32; j0 < t.ncols && j0 < t.count; j0 += 32 * EH) {
                    uint32_t g[32], u[GATEUP ? 32 : 1];
                    const uint32_t rq = j0 < 32 ? rt[0] : (j0 < 64 ? rt[1] : (j0 < 96 ? rt[2] : rt[3]));   // this lane's route id in the 32-wide group of j0
                    tmem_ld32(taddr + j0, g);
                    if constexpr (GATEUP) tmem_ld32(taddr + 128u + j0, u);
                    tmem_ld_wait();
#pragma unroll
                    for (uint32_t i = 0; i < 32; ++i) {
                        const uint32_t j = j0 + i;
                        if (GATEUP) {
                            if (j < t.count) {
                                const float gv = __uint_as_float(g[i]);
                                const float v = __fdividef(gv, 1.f + __expf(-gv)) * __uint_as_float(u[GATEUP ? i : 0]);   // silu(g) * u
                                const __half hv = __float2half_rn(v);
                                bad |= !finite_f32(__half2float(hv));
                                *reinterpret_cast<__half*>(hrow + static_cast<uint64_t>(j) * ostride) = hv;
                            }
                        } else {
                            const uint32_t route = __shfl_sync(0xffffffffu, rq, j & 31u);
                            if (j < t.count) {
                                const float v = __uint_as_float(g[i]);
                                bad |= !finite_f32(v);
                                reinterpret_cast<float*>(obase + static_cast<uint64_t>(route) * ostride)[wrow] = v;
                            }
                        }
                    }
                }
                if (bad) raise_error(p.error, TSP_ERR_NONFINITE);
                tc_fence_before();
            }
            __syncwarp();
            if (lane == 0 && ok) mbar_arrive(&acc_empty[ab]);
            if (++ab == 2) { ab = 0; accph ^= 1u; }
        }
        if (!ok && lane == 0) raise_error(p.error, TSP_ERR_TIMEOUT);
    }
    // every path ends here: free the tensor memory
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 512);
}


// ---------------------------------------------------------------------------------------------
// helpers: route offsets, gather of the routed rows into permuted order
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) route_offsets_kernel(const uint32_t* __restrict__ counts, uint32_t experts, uint32_t* __restrict__ offsets) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ uint32_t warp_sum[8];
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint32_t carry = 0;
    for (uint32_t base = 0; base < experts; base += 256) {
        const uint32_t e = base + tid;
        const uint32_t c = e < experts ? counts[e] : 0u;
        uint32_t incl = c;
        for (int o = 1; o < 32; o <<= 1) { const uint32_t v = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= static_cast<uint32_t>(o)) incl += v; }
        if (lane == 31) warp_sum[warp] = incl;
        __syncthreads();
        uint32_t before = 0, total = 0;
        for (uint32_t i = 0; i < 8; ++i) { if (i < warp) before += warp_sum[i]; total += warp_sum[i]; }
        if (e < experts) offsets[e] = carry + before + incl - c;
        carry += total;
        __syncthreads();
    }
    if (tid == 0) offsets[experts] = carry;
}

// position p of the permuted order belongs to the expert e with offsets[e] <= p < offsets[e+1]; its route id is
// token_map[e*tokens + p - offsets[e]]. Rows are written as binary16 with the K order 0,2,1,3,4,6,5,7 inside each run of 8.
__global__ void __launch_bounds__(256)
gather_rows_kernel(const float* __restrict__ x, uint64_t x_stride, uint32_t in_div, const uint32_t* __restrict__ token_map,
                   const uint32_t* __restrict__ offsets, uint32_t experts, uint32_t tokens, uint32_t cols, __half* __restrict__ xp,
                   uint64_t xp_stride, uint32_t* __restrict__ pos_route, uint32_t* error) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t pos = blockIdx.x * 4 + (threadIdx.x >> 6);
    uint32_t rid = pos;   // no tables: every row in its own position (a dense expert)
    if (token_map) {
        if (pos >= offsets[experts]) return;
        uint32_t lo = 0, hi = experts;   // largest e with offsets[e] <= pos
        while (hi - lo > 1) { const uint32_t mid = (lo + hi) >> 1; if (offsets[mid] <= pos) lo = mid; else hi = mid; }
        rid = token_map[static_cast<uint64_t>(lo) * tokens + (pos - offsets[lo])];
    } else if (pos >= tokens) {
        return;
    }
    const uint32_t t64 = threadIdx.x & 63;
    if (t64 == 0 && pos_route) pos_route[pos] = rid;
    const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const char*>(x) + static_cast<uint64_t>(rid / in_div) * x_stride);
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<char*>(xp) + static_cast<uint64_t>(pos) * xp_stride);
    bool bad = false;
    for (uint32_t k8 = t64; k8 < cols / 8; k8 += 64) {
        const float4 a = src[2 * k8], b = src[2 * k8 + 1];
        const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        uint32_t h[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) { const __half hv = __float2half_rn(v[i]); bad |= !finite_f32(__half2float(hv)); h[i] = __half_as_ushort(hv); }
        dst[k8] = make_uint4(h[0] | (h[2] << 16), h[1] | (h[3] << 16), h[4] | (h[6] << 16), h[5] | (h[7] << 16));
    }
    if (bad) raise_error(error, TSP_ERR_NONFINITE);
}

int launch_route_offsets(const uint32_t* counts, uint32_t experts, uint32_t* offsets, cudaStream_t st) {
    TSP_CUDA(launch_pdl(route_offsets_kernel, dim3(1), dim3(256), 0, st, counts, experts, offsets));
    return TSP_OK;
}

int launch_gather_rows(const float* x, uint64_t x_stride, uint32_t in_div, const uint32_t* token_map, const uint32_t* offsets, uint32_t experts,
                       uint32_t tokens, uint32_t max_routes, uint32_t cols, void* xp, uint64_t xp_stride, uint32_t* pos_route, uint32_t* error,
                       cudaStream_t st) {
    TSP_CUDA(launch_pdl(gather_rows_kernel, dim3((max_routes + 3) / 4), dim3(256), 0, st, x, x_stride, in_div, token_map, offsets, experts, tokens, cols, static_cast<__half*>(xp), xp_stride, pos_route, error));
    TSP_CUDA(cudaGetLastError());
    return TSP_OK;
}

// ---------------------------------------------------------------------------------------------
// host launcher of the grouped tensor-core GEMMs
// ---------------------------------------------------------------------------------------------
template <bool GATEUP>
static int launch_grouped_t(const GroupedMaps& m, const GroupedParams& p, size_t smem, int grid, cudaStream_t st) {
    auto kernel = grouped_mma_kernel<GATEUP>;
    static thread_local size_t configured = 0;
    if (smem > configured) {
        TSP_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        configured = smem;
    }
    TSP_CUDA(launch_pdl(kernel, dim3(grid), dim3(g_warps(GATEUP) * 32), smem, st, m, p));
    return TSP_OK;
}

// a/b: Q4_K Pack v3 planar matrix sets [rows x cols]; act: binary16 rows in permuted position order ([max_positions] rows of
// `cols` values, 16-byte aligned stride); out: gate-up -> binary16 rows [positions x rows] in permuted order, down -> FP32 rows by route id.
int launch_grouped(const tsp_matrix_set* a, const tsp_matrix_set* b, bool gateup, const void* act, uint64_t act_stride, uint32_t max_positions,
                   const uint32_t* tasks, const uint32_t* counts, const uint32_t* offsets, const uint32_t* pos_route, void* out,
                   uint64_t out_stride, uint32_t* error, cudaStream_t st, const GroupedShared* sh) {
    if (a->type != TSP_TYPE_Q4_K || a->layout != TSP_LAYOUT_PLANAR) return fail(TSP_E_TYPE, "grouped GEMM: only Q4_K Pack v3 planar weights have a tensor-core kernel");
    TSP_REQUIRE(a->rows % kRowsM == 0 && a->cols % 256 == 0, "grouped GEMM: rows must be a multiple of 128 and columns of 256");
    GroupedParams p{};
    const uint32_t nblk = a->cols / 256;
    TSP_REQUIRE(nblk <= 32, "grouped GEMM: K extent too large");
    p.split = a->split < a->experts ? a->split : a->experts;
    p.experts = a->experts;
    p.rows = a->rows; p.cols = a->cols; p.nblk = nblk; p.row_blocks = a->rows / kRowsM;
    const uint64_t total_units = static_cast<uint64_t>(a->rows) * nblk;
    const uint64_t sm_off = total_units * 128, dm_off = total_units * 144;
    const uint8_t* base[4] = {static_cast<const uint8_t*>(a->base), static_cast<const uint8_t*>(a->base_hi ? a->base_hi : a->base), nullptr, nullptr};
    if (gateup) {
        base[2] = static_cast<const uint8_t*>(b->base);
        base[3] = static_cast<const uint8_t*>(b->base_hi ? b->base_hi : b->base);
    }
    for (int i = 0; i < (gateup ? 4 : 2); ++i) TSP_REQUIRE(reinterpret_cast<uintptr_t>(base[i]) % 16 == 0, "grouped GEMM: expert images must be 16-byte aligned");
    p.tasks = tasks; p.counts = counts; p.offsets = offsets; p.pos_route = pos_route;
    p.out = out; p.out_stride_bytes = out_stride; p.error = error;
    const uint32_t nmat = gateup ? 2 : 1;
    p.dm_mat_bytes = kRowsM * nblk * 4u;
    p.off_q = 1024;
    p.q_stage_bytes = nmat * (16384u + 2048u);
    p.off_d = p.off_q + 2 * p.q_stage_bytes;
    p.d_stage_bytes = (nmat * p.dm_mat_bytes + 1023u) & ~1023u;
    p.off_a = p.off_d + 2 * p.d_stage_bytes;
    p.off_b = p.off_a + 2 * nmat * 16384u;
    TSP_REQUIRE(p.off_b + 2 * 16384u + 1024 <= 227 * 1024, "grouped GEMM: K extent needs more shared memory than one SM has");
    p.nb_stages = (227 * 1024 - 1024 - p.off_b) / 16384u;
    if (p.nb_stages > kMaxBStages) p.nb_stages = kMaxBStages;
    const size_t smem = p.off_b + p.nb_stages * 16384u + 1024;

    // gate and up of an expert at one constant distance: one copy per plane brings both
    auto mergeable = [](const uint8_t* first, const uint8_t* second, uint64_t* delta) {
        if (second <= first) return false;
        *delta = static_cast<uint64_t>(second - first);
        return *delta % 16 == 0 && *delta < (1ull << 40);
    };
    uint64_t delta = 0, delta_hi = 0;
    p.merged = gateup && mergeable(base[0], base[2], &delta) && mergeable(base[1], base[3], &delta_hi) && delta == delta_hi;
    const uint32_t mats = p.merged ? 2 : 1;
    const uint64_t ds = p.merged ? delta : 16;
    GroupedMaps maps;
    const uint64_t stride = a->experts > 1 ? a->expert_stride : 16;
    TSP_REQUIRE(stride % 16 == 0, "grouped GEMM: expert stride must be a multiple of 16");
    const uint32_t n_lo = p.split, n_hi = a->experts - p.split;
    for (uint32_t i = 0; i < 4; ++i) {
        const uint32_t m = i >> 1;
        const bool hi = i & 1;
        if (m == 1 && (!gateup || p.merged)) { maps.q[i] = maps.q[i - 2]; maps.f[i] = maps.f[i - 2]; maps.d[i] = maps.d[i - 2]; continue; }
        if (hi && n_hi == 0) { maps.q[i] = maps.q[i - 1]; maps.f[i] = maps.f[i - 1]; maps.d[i] = maps.d[i - 1]; continue; }
        const uint32_t n = hi ? n_hi : (n_lo ? n_lo : 1);
        const uint8_t* bp = base[i];
        {   // codes: [128 B of a super-block][row][super-block][matrix][expert], 128-byte swizzle
            const uint64_t dims[5] = {128, a->rows, nblk, mats, n}, strides[4] = {uint64_t(nblk) * 128, 128, ds, stride};
            const uint32_t box[5] = {128, kRowsM, 1, mats, 1};
            if (int rc = get_tensor_map_bytes(bp, 5, dims, strides, box, true, &maps.q[i])) return rc;
        }
        {   // factors: [16 B x super-blocks][row][matrix][expert]
            const uint64_t dims[4] = {uint64_t(nblk) * 16, a->rows, mats, n}, strides[3] = {uint64_t(nblk) * 16, ds, stride};
            const uint32_t box[4] = {16, kRowsM, mats, 1};
            if (int rc = get_tensor_map_bytes(bp + sm_off, 4, dims, strides, box, false, &maps.f[i])) return rc;
        }
        {   // (d, dmin) pairs: the plane in lines of 256 bytes, [256 B][line][matrix][expert]; a row block of 128 rows is 2 * nblk lines
            const uint64_t dims[4] = {256, total_units * 4 / 256, mats, n}, strides[3] = {256, ds, stride};
            const uint32_t box[4] = {256, 2 * nblk, mats, 1};
            if (int rc = get_tensor_map_bytes(bp + dm_off, 4, dims, strides, box, false, &maps.d[i])) return rc;
        }
    }
    const uint32_t ns[3] = {32, 64, 128};
    for (int i = 0; i < 3; ++i) {
        const uint64_t dims[2] = {uint64_t(a->cols) * 2, max_positions}, strides[1] = {act_stride};
        const uint32_t box[2] = {128, ns[i]};
        if (int rc = get_tensor_map_bytes(act, 2, dims, strides, box, true, &maps.x[i])) return rc;
        maps.x[3 + i] = maps.x[i];
    }
    for (int i = 4; i < 6; ++i) { maps.q[i] = maps.q[0]; maps.f[i] = maps.f[0]; maps.d[i] = maps.d[0]; }
    if (sh) {   // the layer's dense shared expert: same shape, one expert, its own rows
        const uint8_t* sa = static_cast<const uint8_t*>(sh->a->base);
        const uint8_t* sb = gateup ? static_cast<const uint8_t*>(sh->b->base) : nullptr;
        TSP_REQUIRE(reinterpret_cast<uintptr_t>(sa) % 16 == 0 && reinterpret_cast<uintptr_t>(sb) % 16 == 0, "grouped GEMM: expert images must be 16-byte aligned");
        uint64_t sdelta = 0;
        p.sh_merged = gateup && mergeable(sa, sb, &sdelta);
        p.sh_tokens = sh->tokens;
        p.sh_tiles = (sh->tokens + kTileRoutes - 1) / kTileRoutes;
        p.sh_out = sh->out; p.sh_out_stride_bytes = sh->out_stride;
        const uint32_t smats = p.sh_merged ? 2 : 1;
        const uint64_t sds = p.sh_merged ? sdelta : 16;
        for (uint32_t m = 0; m < (gateup && !p.sh_merged ? 2u : 1u); ++m) {
            const uint8_t* bp = m == 0 ? sa : sb;
            const uint64_t dq[5] = {128, a->rows, nblk, smats, 1}, sq[4] = {uint64_t(nblk) * 128, 128, sds, 16};
            const uint32_t bq[5] = {128, kRowsM, 1, smats, 1};
            if (int rc = get_tensor_map_bytes(bp, 5, dq, sq, bq, true, &maps.q[4 + m])) return rc;
            const uint64_t df[4] = {uint64_t(nblk) * 16, a->rows, smats, 1}, sf[3] = {uint64_t(nblk) * 16, sds, 16};
            const uint32_t bf[4] = {16, kRowsM, smats, 1};
            if (int rc = get_tensor_map_bytes(bp + sm_off, 4, df, sf, bf, false, &maps.f[4 + m])) return rc;
            const uint64_t dd[4] = {256, total_units * 4 / 256, smats, 1}, sd[3] = {256, sds, 16};
            const uint32_t bd[4] = {256, 2 * nblk, smats, 1};
            if (int rc = get_tensor_map_bytes(bp + dm_off, 4, dd, sd, bd, false, &maps.d[4 + m])) return rc;
        }
        for (int i = 0; i < 3; ++i) {
            const uint64_t dims[2] = {uint64_t(a->cols) * 2, sh->tokens}, strides[1] = {sh->act_stride};
            const uint32_t box[2] = {128, ns[i]};
            if (int rc = get_tensor_map_bytes(sh->act, 2, dims, strides, box, true, &maps.x[3 + i])) return rc;
        }
    }
    const int grid = sm_count();
    if (grid <= 0) return fail(TSP_E_CUDA, "no usable CUDA device");
    return gateup ? launch_grouped_t<true>(maps, p, smem, grid, st) : launch_grouped_t<false>(maps, p, smem, grid, st);
}

}  // namespace tsp
